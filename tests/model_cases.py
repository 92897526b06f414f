"""Shared pieces of the model tests: tiny model folders, requests, comparisons."""
import random

import torch

import plain_qwen2_moe as plain
import traces
from inferx_b200.weights.random_model import write_random_model


def sharpen(name, t):
    """Random N(0, 0.02) weights give near-uniform attention and routing, which would
    hide a wrong key or a wrong expert; make both decisive."""
    if name.endswith(("q_proj.weight", "k_proj.weight")):
        return t * 6.0
    if name.endswith("mlp.gate.weight"):
        return t * 12.0
    if name.endswith("embed_tokens.weight"):
        return t * 3.0
    return t


def sharpen_wide(name, t):
    """The same idea at hidden size 2048, where the tiny models' factors would make
    attention an argmax that bfloat16 rounding flips: scores and router logits with a
    spread of two or three."""
    if name.endswith(("q_proj.weight", "k_proj.weight")):
        return t * 1.75
    if name.endswith("mlp.gate.weight"):
        return t * 2.0
    return t


def make_model_dir(cfg, path, seed, dtype="float32"):
    adjust = sharpen_wide if cfg["hidden_size"] >= 1024 else sharpen
    write_random_model(cfg, str(path), seed=seed, dtype=dtype, adjust=adjust)
    return str(path)


def make_requests(cfg, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)]
            for i, n in enumerate(lengths)}


def reference_rows(model_dir, requests):
    """{(rid, position): logits row} from the plain implementation."""
    cfg, w = plain.read_model_folder(model_dir)
    rows = {}
    for rid, toks in requests.items():
        lg = plain.forward(cfg, w, toks)
        for p in range(len(toks)):
            rows[(rid, p)] = lg[p]
    return rows


def bf16_bound(model_dir, requests, factor=3.0, floor=5e-3):
    """Error bound for a bfloat16 engine on this model and these requests, relative to
    the largest logit: ``factor`` times what rounding every stored activation to
    bfloat16 costs the plain model itself (fp32 run vs the same run with rounding).
    Derived, not chosen: a model whose routing or attention is close to a tie has a
    larger budget, a smooth one a small one."""
    cfg, w = plain.read_model_folder(model_dir)
    worst = 0.0
    for toks in requests.values():
        a = plain.forward(cfg, w, toks)
        b = plain.forward(cfg, w, toks, plain.round_bf16)
        worst = max(worst, float((a - b).abs().max()) / float(a.abs().max()))
    return max(floor, factor * worst)


def bound_for(dtype, model_dir, requests):
    return 2e-5 if dtype == "float32" else bf16_bound(model_dir, requests)


def run_trace(session, steps):
    outs = []
    for st in steps:
        lg = session.run_step(st)
        outs.append(None if lg is None else lg.detach().float().cpu())
    session.manager.check_invariants()
    assert not session.manager.live_requests(), "a finished request still holds cache"
    return traces.collect(steps, outs)


def compare(rows, ref, rel, what):
    """Every produced row against the plain implementation; the error bound is
    ``rel`` times the largest reference logit magnitude of that request."""
    assert rows, "nothing was compared"
    worst = (0.0, None)
    scale = {}
    for (rid, p), v in ref.items():
        scale[rid] = max(scale.get(rid, 0.0), float(v.abs().max()))
    for key, row in rows.items():
        err = float((row - ref[key]).abs().max()) / scale[key[0]]
        if err > worst[0]:
            worst = (err, key)
    assert worst[0] <= rel, (f"{what}: first/worst mismatch at request {worst[1][0]} position "
                             f"{worst[1][1]}: relative error {worst[0]:.3e} > {rel:.1e}")
    return worst[0]


TRACE_KINDS = {
    "whole": lambda reqs: traces.whole(reqs),
    "tail": lambda reqs: traces.tail_decode(reqs, 32),
    "portions": lambda reqs: traces.portions(reqs),
    "mixed": lambda reqs: traces.mixed(reqs, max_live=4, seed=3),
}
