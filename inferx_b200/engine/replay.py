"""Trace replay: feed given token ids through the model step by step, keep logits.

Nothing is sampled.  A ``ReplaySession`` owns a ``Runtime`` (the same model
loader, cache manager, step function and kernels that generation uses) and plays
the part of the scheduler by hand: it opens a request at its first appearance,
reserves pages for the tokens a step brings, runs the step, advances the request
and gives its pages back when the trace says the request has ended.  The
reference has no such tool; its tests and benches hand-build batches and call
``Step`` the same way (tests/kernel/deepseek_v2_model_test.cc:565-590, 657-680,
734-759).

A step is a mapping ``{"step": n, "entries": [{"id", "tokens", "want"}], "end":
[ids]}``; the result of a step is the fp32 logits ``[wanted, vocab]`` in the order
of the entries and of ``want`` (None when nothing is wanted).
"""
from __future__ import annotations

import json
import os
import sys
from typing import Any, Iterable, Mapping, Optional

import torch

from .executor import StepEntry
from .runtime import Runtime, load_model


class ReplayError(RuntimeError):
    pass


def pages_for(max_tokens: int, page_size: int, max_live: int = 1) -> int:
    """Pages for live requests that hold ``max_tokens`` tokens in all, each request's
    count rounded up to a multiple of 64.  A request of k * 64 tokens needs at most
    k * ceil(64 / page_size) pages, whatever the page size; pages larger than 64 tokens
    can cost every live request one page more than its share."""
    units = -(-int(max_tokens) // 64)
    if page_size <= 64:
        return max(1, units * -(-64 // page_size))
    return max(1, -(-units * 64 // page_size) + max_live)


class ReplaySession:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, *, page_size: int = 16,
                 max_live: int = 8, device: str = "cuda", ops=None, use_graphs: bool = False):
        _, model = load_model(model_dir, dtype=dtype, device=device, ops=ops)
        self.runtime = Runtime(model, page_size=page_size,
                               num_pages=pages_for(max_tokens, page_size, max_live),
                               max_slots=max_live,
                               use_graphs=use_graphs)
        self.manager = self.runtime.manager
        self.executor = self.runtime.executor

    def run_step(self, step: Mapping[str, Any]) -> Optional[torch.Tensor]:
        entries = []
        mgr = self.manager
        for e in step.get("entries", []):
            rid, tokens = e["id"], list(e["tokens"])
            if not tokens:
                continue                  # an entry that brings nothing runs nothing
            if not mgr.has(rid):
                if mgr.open(rid) is None:
                    raise ReplayError(f"step {step.get('step')}: no free state slot for "
                                      f"request {rid!r} ({mgr.max_slots} live at most)")
            if not mgr.reserve(rid, mgr.length(rid) + len(tokens)):
                raise ReplayError(
                    f"step {step.get('step')}: the cache pool has no page left for request "
                    f"{rid!r} ({mgr.length(rid)} + {len(tokens)} tokens); --max-tokens is too small")
            entries.append(StepEntry(rid, tokens, list(e.get("want", []))))
        logits = self.executor.step(entries) if entries else None
        for e in entries:
            mgr.advance(e.request, len(e.tokens))
        for rid in step.get("end", []):
            if mgr.has(rid):
                mgr.close(rid)
        return logits


def wanted_rows(session: ReplaySession, step: Mapping[str, Any]):
    """[(request id, position)] of the rows a step's logits file will hold, in order: what
    the reference's logits files carry beside the values (scripts/gen_reference_logits.py:
    15-23).  Call before the step runs."""
    out = []
    for e in step.get("entries", []):
        if not e.get("tokens"):
            continue
        base = session.manager.length(e["id"]) if session.manager.has(e["id"]) else 0
        out += [(e["id"], base + int(w)) for w in e.get("want", [])]
    return out


def run_stream(session: ReplaySession, lines: Iterable[str], out_dir: str, report=None,
               index: bool = False) -> int:
    """Replay JSON lines; write ``<out_dir>/<step>.f32`` for steps that want logits
    and call ``report(step)`` after every step.  With ``index``, a step that wants
    logits also gets ``<step>.rows.json``: the request id and position of every row."""
    os.makedirs(out_dir, exist_ok=True)
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        tags = wanted_rows(session, step) if index else None
        logits = session.run_step(step)
        if logits is not None:
            arr = logits.detach().to("cpu", torch.float32).contiguous().numpy()
            arr.astype("<f4").tofile(os.path.join(out_dir, f"{step['step']}.f32"))
            if index:
                with open(os.path.join(out_dir, f"{step['step']}.rows.json"), "w") as f:
                    json.dump({"vocab": int(arr.shape[1]),
                               "rows": [{"id": r, "position": p} for r, p in tags]}, f)
        elif session.executor.device.type == "cuda":
            torch.cuda.synchronize()
        session.executor.poll_errors()
        if report is not None:
            report(step["step"])
        n += 1
    return n


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(
        prog="trace_run",
        description="Feed token ids through a model step by step and write logits "
                    "(reads one JSON step per line from standard input).")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-live", type=int, default=8, help="requests alive at once")
    ap.add_argument("--index", action="store_true",
                    help="also write <step>.rows.json: request id and position of each row")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 3
    session = ReplaySession(args.model, args.dtype, args.max_tokens, page_size=args.block_size,
                            max_live=args.max_live)

    def report(step):
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()

    # one line at a time: the sender may wait for "done <step>" before it writes the next
    run_stream(session, iter(sys.stdin.readline, ""), args.out, report, index=args.index)
    return 0
