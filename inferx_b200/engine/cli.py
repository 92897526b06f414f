"""``inferx-generate``: token ids in, token ids out, on one GPU.

Option names and meanings follow the reference's ``inferx-serve``
(src/support/options.cc:47-174): the model folder as the positional ``MODEL`` or
``--model``, ``--max-num-seqs``, ``--max-model-len``, ``--max-num-batched-tokens``
(default max(2048, max-model-len), options.cc:332-336), ``--block-size``,
``--num-gpu-blocks-override``, ``--gpu-memory-utilization``,
``--kv-cache-memory-bytes``, ``--dtype``, ``--enforce-eager``, ``--log-level``, ``--v``,
``--log-json``, ``--log-file``, with the older spellings the reference still takes
(``--max-running``, ``--max-seq-len``, ``--kv-blocks``, ``--no-cuda-graphs``).  Options of
the reference for what this engine does not have are taken only at the value that means
"off" and refused otherwise, with the reason (``--enable-prefix-caching``,
``--tensor-parallel-size``, ``--quantization``, ``--kv-cache-dtype``, ``--device``);
``--no-enable-chunked-prefill`` is refused as it is there (options.cc:306-308).
There is no tokenizer here, so prompts are lists of token ids.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def _parse_ids(text: str) -> List[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="inferx-generate", description=__doc__.split("\n\n")[0])
    ap.add_argument("model_pos", nargs="?", metavar="MODEL", help="model folder")
    ap.add_argument("--model", help="model folder (config.json + safetensors)")
    ap.add_argument("--dtype", default="auto",
                    choices=["auto", "bfloat16", "bf16", "float", "float32", "fp32", "half",
                             "float16"],
                    help="auto is bfloat16; float32 is the true 32-bit path; there is no fp16")
    ap.add_argument("--max-num-seqs", "--max-running", dest="max_num_seqs", type=int, default=8)
    ap.add_argument("--max-model-len", "--max-seq-len", dest="max_model_len", type=int,
                    default=2048)
    ap.add_argument("--max-num-batched-tokens", type=int, default=0)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--num-gpu-blocks-override", "--kv-blocks", dest="num_gpu_blocks_override",
                    type=int, default=0)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.92)
    ap.add_argument("--kv-cache-memory-bytes", type=int, default=0)
    ap.add_argument("--enforce-eager", "--no-cuda-graphs", dest="enforce_eager",
                    action="store_true")
    ap.add_argument("--no-enforce-eager", dest="enforce_eager", action="store_false")
    ap.add_argument("--enable-chunked-prefill", dest="chunked_prefill", action="store_true",
                    default=True, help="always on")
    ap.add_argument("--no-enable-chunked-prefill", dest="chunked_prefill", action="store_false")
    ap.add_argument("--enable-prefix-caching", dest="prefix_caching", action="store_true")
    ap.add_argument("--no-enable-prefix-caching", dest="prefix_caching", action="store_false")
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--quantization", "-q", default=None)
    ap.add_argument("--kv-cache-dtype", default="auto")
    ap.add_argument("--log-level", default="info", choices=["debug", "info", "warning", "error"])
    ap.add_argument("--v", type=int, default=0, help="more detail in debug messages")
    ap.add_argument("--log-json", action="store_true", help="log lines as JSON objects")
    ap.add_argument("--log-file", help="append the log lines to this file as well")
    ap.add_argument("--prefill-chunk", type=int, default=0,
                    help="most prompt tokens one request runs per step (0: the batch budget)")
    ap.add_argument("--random-weights", metavar="CONFIG_JSON",
                    help="draw weights from --seed for this config.json instead of loading a folder")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help='a prompt as token ids, "1,2,3"; may be given several times')
    ap.add_argument("--prompt-file", help="file with one prompt per line (token ids)")
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--min-tokens", type=int, default=0,
                    help="stop tokens cannot be chosen before this many were generated")
    ap.add_argument("--logprobs", type=int, default=None, metavar="K",
                    help="report each token's log-probability and K alternatives (0 to 20)")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--stop-token-ids", default="", help="token ids that end a request")
    return ap


_LEVELS = {"debug": 0, "info": 1, "warning": 2, "error": 3}


class _Log:
    """Log lines to stderr (and a file), plain or one JSON object a line."""

    def __init__(self, level: str, as_json: bool, path):
        self.level, self.as_json = _LEVELS[level], as_json
        self.file = open(path, "a") if path else None

    def __call__(self, level: str, message: str, **fields) -> None:
        if _LEVELS[level] < self.level:
            return
        if self.as_json:
            line = json.dumps({"ts": round(time.time(), 3), "level": level, "msg": message,
                               **fields})
        else:
            extra = "".join(f" {k}={v}" for k, v in fields.items())
            line = f"[inferx-generate] {message}{extra}"
        for out in (sys.stderr, self.file):
            if out is not None:
                print(line, file=out, flush=True)


def _refusals(args) -> List[str]:
    """What was asked for that this engine does not have."""
    why = []
    if args.dtype in ("half", "float16"):
        why.append(f"--dtype {args.dtype}: this engine runs bfloat16 or float32")
    if not args.chunked_prefill:
        why.append("chunked prefill cannot be disabled")
    if args.prefix_caching:
        why.append("--enable-prefix-caching: there is no prefix cache in this engine")
    if args.tensor_parallel_size != 1:
        why.append("--tensor-parallel-size: this engine runs on one GPU")
    if args.device != "cuda":
        why.append(f"--device {args.device}: this engine runs on CUDA only")
    if args.quantization not in (None, "none"):
        why.append("--quantization: weights are bfloat16 or float32 here")
    if args.kv_cache_dtype not in ("auto", "bfloat16"):
        why.append("--kv-cache-dtype: the cache has the model's element type here")
    return why


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    refused = _refusals(args)
    if refused:
        for r in refused:
            print(f"inferx-generate: {r}", file=sys.stderr)
        return 2
    if args.dtype in ("auto", "bf16"):
        args.dtype = "bfloat16"
    elif args.dtype in ("float", "fp32"):
        args.dtype = "float32"
    log = _Log(args.log_level, args.log_json, args.log_file)
    model = args.model or args.model_pos
    if not model and not args.random_weights:
        print("inferx-generate: give a MODEL folder or --random-weights CONFIG_JSON",
              file=sys.stderr)
        return 2
    prompts = [_parse_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_parse_ids(ln) for ln in f if ln.strip()]
    if not prompts:
        print("inferx-generate: no prompts (--prompt-ids or --prompt-file)", file=sys.stderr)
        return 2

    import torch
    from ..sampling.params import SamplingParams
    from .engine import Engine, EngineConfig, Request
    if not torch.cuda.is_available():
        print("inferx-generate: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 3
    cfg_json = None
    if args.random_weights:
        with open(args.random_weights) as f:
            cfg_json = json.load(f)
    t0 = time.time()
    engine = Engine.create(EngineConfig(
        model=None if cfg_json is not None else model, dtype=args.dtype,
        max_num_seqs=args.max_num_seqs, max_model_len=args.max_model_len,
        max_num_batched_tokens=args.max_num_batched_tokens, block_size=args.block_size,
        num_gpu_blocks_override=args.num_gpu_blocks_override,
        kv_cache_memory_bytes=args.kv_cache_memory_bytes,
        gpu_memory_utilization=args.gpu_memory_utilization, prefill_chunk=args.prefill_chunk,
        enforce_eager=args.enforce_eager, config_json=cfg_json, seed=args.seed))
    log("info", f"model ready in {time.time() - t0:.1f}s",
        cache_pages=engine.stats()["pages_total"], page_tokens=args.block_size)
    if args.v > 0:
        log("debug", "engine", config=json.dumps(engine.model_config.to_json(), sort_keys=True)
            if hasattr(engine.model_config, "to_json") else str(engine.model_config))
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature,
                            top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                            ignore_eos=args.ignore_eos, seed=args.seed,
                            stop_tokens=tuple(_parse_ids(args.stop_token_ids)),
                            presence_penalty=args.presence_penalty,
                            frequency_penalty=args.frequency_penalty,
                            repetition_penalty=args.repetition_penalty,
                            min_tokens=args.min_tokens,
                            want_logprobs=args.logprobs is not None,
                            top_logprobs=args.logprobs or 0)
    t0 = time.time()
    done = engine.generate([Request(p, params) for p in prompts])
    dt = time.time() - t0
    for i, c in enumerate(done):
        rec = {"index": i, "output_ids": c.output_tokens, "finish_reason": c.reason}
        if c.logprobs is not None:
            rec["logprobs"] = [{"token": lp.token, "logprob": round(lp.logprob, 6),
                                "top": [[t, round(p, 6)] for t, p in lp.top]}
                               for lp in c.logprobs]
        print(json.dumps(rec))
    st = engine.stats()
    log("info", f"{st['tokens_generated']} tokens in {dt:.2f}s", steps=st["steps"],
        preemptions=st["preemptions"], graph_replays=st["graph_replays"])
    return 0
