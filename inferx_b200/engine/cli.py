"""``inferx-generate``: token ids in, token ids out, on one GPU.

Option names and meanings follow the reference's ``inferx-serve``
(src/support/options.cc:47-174): the model folder as the positional ``MODEL`` or
``--model``, ``--max-num-seqs``, ``--max-model-len``, ``--max-num-batched-tokens``
(default max(2048, max-model-len), options.cc:332-336), ``--block-size``,
``--num-gpu-blocks-override``, ``--gpu-memory-utilization``,
``--kv-cache-memory-bytes``, ``--dtype``, ``--enforce-eager``, ``--log-level``.
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
    ap.add_argument("--dtype", default="bfloat16",
                    choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--max-num-seqs", type=int, default=8)
    ap.add_argument("--max-model-len", type=int, default=2048)
    ap.add_argument("--max-num-batched-tokens", type=int, default=0)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--num-gpu-blocks-override", type=int, default=0)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.92)
    ap.add_argument("--kv-cache-memory-bytes", type=int, default=0)
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--log-level", default="info", choices=["debug", "info", "warning", "error"])
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


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
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
    quiet = args.log_level in ("warning", "error")
    if not quiet:
        print(f"[inferx-generate] model ready in {time.time() - t0:.1f}s; cache "
              f"{engine.stats()['pages_total']} pages of {args.block_size}", file=sys.stderr)
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
    if not quiet:
        st = engine.stats()
        print(f"[inferx-generate] {st['tokens_generated']} tokens in {dt:.2f}s, {st['steps']} steps, "
              f"{st['preemptions']} preemptions", file=sys.stderr)
    return 0
