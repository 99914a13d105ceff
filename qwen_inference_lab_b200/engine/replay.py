"""Trace replay: feed given token ids through the model step by step, write logits.

Nothing is sampled.  Each line of standard input is one step,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

and runs through the same model, step function, cache manager and kernels that
generation uses.  For a step that wants logits, ``<out>/<step>.f32`` receives them
as little-endian float32 ``[wanted, vocab]`` in the order of the entries and of
``want``.  After every step a line ``done <step>`` is printed and flushed.

The reference has no such program; its nearest relatives are the teacher-forced
loops of its tests (tests/qil/test_model.py:19-33).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def build_parser():
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, type=Path, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", required=True, type=int,
                        help="most tokens live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (divides 64)")
    parser.add_argument("--max-live", type=int, default=8, help="most requests alive at once")
    return parser


def main(argv=None, stdin=None, stdout=None) -> int:
    args = build_parser().parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    if args.max_tokens < 1:
        raise SystemExit("--max-tokens must be positive")
    if args.page_size < 1 or 64 % args.page_size:
        raise SystemExit("--page-size must divide 64")
    import torch

    from ..cache import CacheManager
    from ..loading import load_model, resolve_dtype
    from .step import StepEntry, StepRunner

    dtype = resolve_dtype(args.dtype)
    model = load_model(args.model, device="cuda", dtype=dtype)
    pool_tokens = (args.max_tokens + 63) // 64 * 64
    cache = CacheManager(model.cache_specs(), num_pages=pool_tokens // args.page_size, page_size=args.page_size,
                         max_requests=args.max_live, max_context=model.max_positions, dtype=dtype,
                         device=model.device)
    runner = StepRunner(model, cache, max_step_tokens=min(pool_tokens, 8192))
    args.out.mkdir(parents=True, exist_ok=True)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = []
        for item in step.get("entries", []):
            if item["id"] not in cache.rows:
                if not cache.admit(item["id"]):
                    raise SystemExit(f"step {step['step']}: more than {args.max_live} live requests")
            entries.append(StepEntry(item["id"], [int(t) for t in item["tokens"]],
                                     [int(w) for w in item.get("want", [])]))
        if entries:
            logits = runner.run(entries)
            if logits is not None:
                data = logits.detach().to(torch.float32).cpu().contiguous().numpy()
                runner.check()
                data.astype("<f4", copy=False).tofile(args.out / f"{step['step']}.f32")
        for request_id in step.get("end", []):
            if request_id in cache.rows:
                cache.release(request_id)
        print(f"done {step['step']}", file=stdout, flush=True)
    torch.cuda.synchronize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
