"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step: every live request gets one token.  The default run
has the layer sizes of Qwen3-8B (36 layers, hidden 4096, 32/8 heads of 128,
intermediate 12288, vocabulary 151936, untied head) with random bfloat16 weights,
8 requests at a context of 8192 tokens, pages of 16.  One JSON line is printed:
``value`` is decoded tokens per second timed on the device over K graph-replayed
steps; ``e2e`` is the same through ``Engine.step`` with host token ids in and
sampled ids out; ``prefill`` times one 2048-token prompt; ``roofline`` relates the
bytes a decode step must read (every weight once, the cache of the live requests)
to the measured copy bandwidth; ``points`` holds decode at batch 1 and 64 at the same
context and at batch 16, 32 and 64 at a context of 1024 (tokens per second), and
``points_detail`` their milliseconds, bytes and fraction of the copy bandwidth.
Peaks come from MEASURED_PEAKS.json beside this file when present.
``--shape 32b|0.6b`` prints the same line for the other layer sizes; ``--impl reference``
the same line for the unmodified reference engine.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

QWEN3_8B = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                rms_norm_eps=1e-6, rope_theta=1000000.0, attention_bias=False, tie_word_embeddings=False,
                eos_token_id=None)
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64)
QWEN3_06B = dict(QWEN3_8B, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 tie_word_embeddings=True)
# name -> (sizes, label, context of the decode measurements)
SHAPES = {"8b": (QWEN3_8B, "Qwen3-8B shape", 8192), "32b": (QWEN3_32B, "Qwen3-32B shape", 8192),
          "0.6b": (QWEN3_06B, "Qwen3-0.6B shape", 4096)}
CONTEXT = 8192
PAGE_SIZE = 16
PREFILL_TOKENS = 2048


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            flat = {}
            def walk(node):
                if isinstance(node, dict):
                    for key, value in node.items():
                        if isinstance(value, (int, float)) and key not in flat:
                            flat[key] = float(value)
                        else:
                            walk(value)
                elif isinstance(node, list):
                    for item in node:
                        walk(item)
            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return {"hbm_gbs": flat["hbm_gbs"], "bf16_tflops": flat["bf16_tflops"],
                        "bf16_tflops_sustained": flat.get("bf16_tflops_sustained"), "source": "measured"}
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.proc, self.thread = [], None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0],
                                          f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        mhz, max_mhz, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6 or not parts[0].isdigit():
                continue
            mhz.append(int(parts[0])); max_mhz.append(int(parts[1]))
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": int(statistics.median(mhz)), "sm_max_mhz": max(max_mhz), "reasons": sorted(reasons)}


def gemm_params(cfg):
    """Matrix elements every token passes through: the four projections of each layer and the head."""
    h, d = cfg["hidden_size"], cfg["head_dim"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * d * h
    o = cfg["num_attention_heads"] * d * h
    mlp = 3 * cfg["intermediate_size"] * h
    return cfg["num_hidden_layers"] * (qkv + o + mlp), cfg["vocab_size"] * h


def decode_bytes(cfg, batch, context, dtype_bytes=2):
    layer_params, head_params = gemm_params(cfg)
    norms = cfg["num_hidden_layers"] * (2 * cfg["hidden_size"] + 2 * cfg["head_dim"]) + cfg["hidden_size"]
    kv_per_token = cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * cfg["head_dim"]
    return dtype_bytes * (layer_params + head_params + norms + batch * context * kv_per_token)


def prefill_flops(cfg, tokens, logit_rows=1):
    layer_params, head_params = gemm_params(cfg)
    gemm = 2.0 * tokens * layer_params + 2.0 * logit_rows * head_params
    attention = cfg["num_hidden_layers"] * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * (tokens + 1) / 2
    return gemm + attention


def config_record(cfg, label, batch, context, full_layers, of):
    """The ``config`` of a bench line: every size by name, flat; the same keys for both arms."""
    return {"model": label, "layers": cfg["num_hidden_layers"], "layers_of_config": full_layers,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "tied": cfg["tie_word_embeddings"],
            "global_batch": batch, "seq_len": context, "page_size": PAGE_SIZE, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (decode reads >16 GB per step); prefill flushes a 256 MB buffer",
            "peaks": of}


# --------------------------------------------------------------------------- our engine
class OursBench:
    def __init__(self, cfg, layers=None, dtype="bfloat16"):
        import torch
        from qwen_inference_lab_b200.config import Qwen3Config
        from qwen_inference_lab_b200.loading import random_model
        self.torch = torch
        self.cfg = dict(cfg)
        self.full_layers = cfg["num_hidden_layers"]
        if layers:
            self.cfg["num_hidden_layers"] = layers
        self.dtype = getattr(torch, dtype)
        self.model = random_model(Qwen3Config.from_dict(dict(self.cfg, model_type="qwen3")), seed=0,
                                  device="cuda", dtype=self.dtype)
        torch.cuda.synchronize()

    def largest_context(self, batch, wanted, reserve=6 << 30):
        """The longest context (a multiple of 1024, at most ``wanted``) whose cache for ``batch`` requests fits."""
        free, _ = self.torch.cuda.mem_get_info()
        per_token = (self.cfg["num_hidden_layers"] * 2 * self.cfg["num_key_value_heads"] * self.cfg["head_dim"]
                     * self.dtype.itemsize)
        fits = int((free - reserve) // (batch * per_token)) // 1024 * 1024
        return max(1024, min(wanted, fits))

    def _fill_cache(self, cache, ids, context):
        for g in cache.kv_groups:
            g.storage.normal_(0.0, 0.5)
        for rid in ids:
            assert cache.admit(rid)
            cache.ensure(rid, context)
            cache.advance(rid, context)

    def decode(self, batch, context, steps, warmup, sample_clocks=False):
        """Device-timed decode: K steps of ``batch`` single tokens at ``context`` cached tokens each."""
        torch = self.torch
        from qwen_inference_lab_b200.cache import CacheManager
        from qwen_inference_lab_b200.engine import StepEntry, StepRunner
        from qwen_inference_lab_b200.kernels import ops
        total = context + steps + warmup + 2
        pages_per_request = (total + PAGE_SIZE - 1) // PAGE_SIZE
        cache = CacheManager(self.model.cache_specs(), num_pages=batch * pages_per_request, page_size=PAGE_SIZE,
                             max_requests=batch, max_context=pages_per_request * PAGE_SIZE, dtype=self.dtype,
                             device=self.model.device)
        runner = StepRunner(self.model, cache, max_step_tokens=max(batch, 64))
        ids = list(range(batch))
        self._fill_cache(cache, ids, context)
        generator = torch.Generator().manual_seed(1)
        tokens = torch.randint(0, self.cfg["vocab_size"], (steps + warmup + 1, batch), generator=generator).tolist()
        def one(i):
            return runner.run([StepEntry(rid, [tokens[i][rid]], [0]) for rid in ids])
        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        launches_before = ops.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.__enter__()
        torch.cuda.synchronize()
        start.record()
        for i in range(warmup, warmup + steps):
            logits = one(i)
        stop.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.__exit__()
        ms = start.elapsed_time(stop) / steps
        assert torch.isfinite(logits).all()
        per_step = getattr(runner, "launches_per_graph", {}).get(batch)
        result = dict(ms_per_step=ms, tokens_per_s=batch / ms * 1e3,
                      bytes=decode_bytes(self.cfg, batch, context + warmup + steps // 2, self.dtype.itemsize),
                      launches=per_step * steps if per_step else ops.launch_count() - launches_before,
                      clocks=sampler.summary() if sampler else None)
        del runner, cache
        torch.cuda.empty_cache()
        return result

    def prefill(self, tokens_n, reps=9, warmup=4):
        torch = self.torch
        from qwen_inference_lab_b200.cache import CacheManager
        from qwen_inference_lab_b200.engine import StepEntry, StepRunner
        pages = (tokens_n + PAGE_SIZE - 1) // PAGE_SIZE + 1
        cache = CacheManager(self.model.cache_specs(), num_pages=pages, page_size=PAGE_SIZE, max_requests=2,
                             max_context=pages * PAGE_SIZE, dtype=self.dtype, device=self.model.device)
        runner = StepRunner(self.model, cache, max_step_tokens=tokens_n)
        generator = torch.Generator().manual_seed(2)
        prompt = torch.randint(0, self.cfg["vocab_size"], (tokens_n,), generator=generator).tolist()
        times = []
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        sampler = ClockSampler()
        sampler.__enter__()
        for i in range(warmup + reps):
            cache.admit("p")
            flush.zero_()   # a buffer larger than L2 between timed iterations
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            logits = runner.run([StepEntry("p", prompt, [tokens_n - 1])])
            stop.record()
            torch.cuda.synchronize()
            cache.release("p")
            if i >= warmup:
                times.append(start.elapsed_time(stop))
        sampler.__exit__()
        self.last_prefill_clocks = sampler.summary()
        assert torch.isfinite(logits).all()
        ms = statistics.median(times)
        self.last_prefill_times = sorted(round(t, 3) for t in times)
        del runner, cache, flush
        torch.cuda.empty_cache()
        return ms

    def e2e(self, batch, context, steps, warmup):
        """Decode through Engine.step: host token ids in (pinned staging), sampled ids out, every step."""
        torch = self.torch
        from qwen_inference_lab_b200 import Engine
        new_tokens = steps + warmup + 4
        prompt_len = context - 1
        pages = batch * ((prompt_len + new_tokens + PAGE_SIZE - 1) // PAGE_SIZE + 1)
        engine = Engine(self.model, num_pages=pages, page_size=PAGE_SIZE, token_budget=2048, prefill_chunk=2048,
                        max_active=batch, overlap=True)       # a step ahead of the host, as generate() runs
        generator = torch.Generator().manual_seed(3)
        for _ in range(batch):
            prompt = torch.randint(0, self.cfg["vocab_size"], (prompt_len,), generator=generator).tolist()
            engine.submit(prompt, max_new_tokens=new_tokens, ignore_eos=True)
        while engine.scheduler.prefilling:
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        begin = time.perf_counter()
        emitted = 0
        for _ in range(steps):
            emitted += len(engine.step())
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - begin
        h2d = engine.runner.last_upload_bytes
        engine.close()
        del engine
        torch.cuda.empty_cache()
        return dict(value=emitted / elapsed, unit="tokens/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=2 * 4 * batch,
                    ms_per_step=elapsed / steps * 1e3)


def mixed_workload(bench, requests=64, new_tokens=128, longest=2048, seed=4):
    """Requests with prompts of 16 to ``longest`` tokens (uniform, seeded), ``new_tokens`` each, all
    submitted at once to ``Engine.generate``: output tokens per second of the whole run, wall clock."""
    import torch
    from qwen_inference_lab_b200 import Engine
    generator = torch.Generator().manual_seed(seed)
    lengths = torch.randint(16, longest + 1, (requests,), generator=generator).tolist()
    prompts = [torch.randint(0, bench.cfg["vocab_size"], (n,), generator=generator).tolist() for n in lengths]
    pages = sum((n + new_tokens + PAGE_SIZE - 1) // PAGE_SIZE + 1 for n in lengths)
    engine = Engine(bench.model, num_pages=pages, page_size=PAGE_SIZE, token_budget=4096, prefill_chunk=2048,
                    max_active=requests)
    # set-up outside the timed run, as the reference's harness keeps load and warm-up out of its samples
    # (docs/batched-gpu-validation-2026-09-20.md:19-24): the same workload once, which also records the decode
    # steps' graphs for the batch sizes and context ranges it passes through
    engine.generate(prompts, max_new_tokens=new_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    steps_before = engine.runner.steps_run
    begin = time.perf_counter()
    rows = engine.generate(prompts, max_new_tokens=new_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - begin
    produced = sum(len(row["token_ids"]) for row in rows)
    steps = engine.runner.steps_run - steps_before
    engine.close()
    return {"value": round(produced / elapsed, 1), "unit": "output tokens/s", "requests": requests,
            "prompt_tokens": sum(lengths), "new_tokens": produced, "steps": steps, "seconds": round(elapsed, 3)}


def run_ours(args):
    import torch
    pk = peaks()
    sizes, label, context = SHAPES[args.shape]
    bench = OursBench(sizes, layers=args.layers, dtype=args.dtype)
    cfg = bench.cfg
    batch = args.batch
    if args.only == "mixed":
        print(json.dumps({"workload": "mixed", "model": label, "dtype": args.dtype, **mixed_workload(bench)}))
        return
    if args.only == "decode":
        part = bench.decode(batch, args.context, args.steps, args.warmup)
        print(f"decode batch {batch} context {args.context} layers {cfg['num_hidden_layers']}: {part['ms_per_step']:.3f} ms/step")
        return
    if args.only == "prefill":
        ms = bench.prefill(args.prefill_tokens, reps=args.steps if args.steps != 32 else 2, warmup=3)
        frac = prefill_flops(cfg, args.prefill_tokens) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12)
        print(f"prefill {args.prefill_tokens} tokens layers {cfg['num_hidden_layers']}: {ms:.3f} ms "
              f"({args.prefill_tokens / ms * 1e3:.0f} tokens/s, {frac:.3f} of the bf16 peak; all: {bench.last_prefill_times})")
        return
    main = bench.decode(batch, context, args.steps, args.warmup, sample_clocks=True)
    points, points_detail = {}, {}
    short = min(1024, context)
    for b, wanted in ((1, context), (64, context), (16, short), (32, short), (64, short)):
        if args.quick:
            break
        fits = bench.largest_context(b, wanted)      # the 32B shape holds 64 requests only at a shorter context
        key = f"decode_b{b}" if fits == context else f"decode_b{b}_context{fits}"
        part = bench.decode(b, fits, max(8, args.steps // 2), args.warmup)
        points[key] = round(part["tokens_per_s"], 1)
        gbs = part["bytes"] / (part["ms_per_step"] * 1e-3) / 1e9
        points_detail[key] = {"ms": round(part["ms_per_step"], 4), "gbytes": round(part["bytes"] / 1e9, 3),
                              "gbs": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 4)}
    prefill_ms = bench.prefill(PREFILL_TOKENS)
    e2e = bench.e2e(batch, context, args.steps, args.warmup)
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    achieved = main["bytes"] / (main["ms_per_step"] * 1e-3) / 1e9
    of = "of measured" if pk["source"] == "measured" else "of fallback"
    line = {
        "metric": f"decode tokens/s ({label}, batch {batch}, context {context})",
        "value": round(main["tokens_per_s"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic: random weights, random token ids, random cache contents",
        "impl": "ours",
        "config": config_record(cfg, label, batch, context, bench.full_layers, of),
        "clocks": main["clocks"],
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(main["launches"]),
        "prefill": {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    # the peak is the bfloat16 tensor-core one: no fraction for the float32 check path
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4) if args.dtype == "bfloat16" else None,
                    "ms_min": bench.last_prefill_times[0], "ms_max": bench.last_prefill_times[-1],
                    "sm_mhz": bench.last_prefill_clocks["sm_mhz"], "reasons": bench.last_prefill_clocks["reasons"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "points_detail": points_detail,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- the reference
def run_reference(args):
    ref = ROOT / "baseline" / "_ref"
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0
    if not (ref / "qil" / "engine.py").is_file():
        return unavailable("the reference is not installed under baseline/_ref")
    sys.path.insert(0, str(ref))
    try:
        import torch
        from qil.config import ModelConfig
        from qil.engine import Engine
        from qil.model import Qwen3
    except Exception as error:  # noqa: BLE001
        return unavailable(f"import failed: {type(error).__name__}: {error}")
    batch = args.batch
    fields = ModelConfig.__dataclass_fields__
    config = ModelConfig(**{k: v for k, v in QWEN3_8B.items() if k in fields})
    try:
        torch.manual_seed(0)
        with torch.device("cuda"):
            model = Qwen3(config).to(dtype=torch.bfloat16).eval()
        with torch.no_grad():
            for parameter in model.parameters():
                if parameter.ndim == 2:
                    parameter.normal_(0.0, 0.02)
        new_tokens = args.steps + args.warmup + 4
        prompt_len = CONTEXT - 1
        pages = batch * ((prompt_len + new_tokens + PAGE_SIZE - 1) // PAGE_SIZE + 1)
        engine = Engine(model, num_pages=pages, page_size=PAGE_SIZE, token_budget=2048, prefill_chunk=2048,
                        max_active=batch, decode_attention="paged")
        generator = torch.Generator().manual_seed(3)
        for _ in range(batch):
            prompt = torch.randint(0, config.vocab_size, (prompt_len,), generator=generator).tolist()
            engine.submit(prompt, max_new_tokens=new_tokens, ignore_eos=True)
        while any(r.computed < len(r.prompt) for r in engine.scheduler.requests.values()):
            engine.step()
        for _ in range(args.warmup):
            engine.step()
        torch.cuda.synchronize()
        with ClockSampler() as sampler:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin = time.perf_counter()
            start.record()
            emitted = 0
            for _ in range(args.steps):
                emitted += len(engine.step())
            stop.record()
            torch.cuda.synchronize()
            elapsed = time.perf_counter() - begin
        ms = start.elapsed_time(stop) / args.steps
    except Exception as error:  # noqa: BLE001
        return unavailable(f"the reference failed on this configuration: {type(error).__name__}: {str(error)[:200]}")
    pk = peaks()
    achieved = decode_bytes(QWEN3_8B, batch, CONTEXT) / (ms * 1e-3) / 1e9
    of = "of measured" if pk["source"] == "measured" else "of fallback"
    # What the reference copies per decode step (qil/model.py:143-152, qil/cache.py:103-131, qil/engine.py:96-100):
    # it builds int64 tensors from Python lists for the token ids, the positions (lengths derive from them on the
    # device), the write slots and the padded page table, and reads back one flag and the chosen ids.
    table_width = (CONTEXT + args.warmup + args.steps + PAGE_SIZE - 1) // PAGE_SIZE
    h2d = 8 * (batch + batch + batch + batch * table_width)
    d2h = 1 + 8 * batch
    print(json.dumps({
        "metric": "decode tokens/s (Qwen3-8B shape, batch 8, context 8192)", "impl": "reference",
        "value": round(batch / ms * 1e3, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights, random token ids",
        "config": config_record(QWEN3_8B, "Qwen3-8B shape", batch, CONTEXT, QWEN3_8B["num_hidden_layers"], of),
        "clocks": sampler.summary(),
        "e2e": {"value": round(emitted / elapsed, 2), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(elapsed / args.steps * 1e3, 2)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }), flush=True)
    return 0


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    parser.add_argument("--quick", action="store_true", help="skip the batch 1 and 64 points")
    parser.add_argument("--only", choices=["decode", "prefill", "mixed"], default=None,
                        help="run just this part and print its result instead of the JSON line; mixed = 64 requests "
                             "with prompts of 16 to 2048 tokens and 128 new tokens each through Engine.generate")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="8b", help="layer sizes (default: Qwen3-8B)")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--context", type=int, default=CONTEXT, help="cached tokens per request (profiling aid)")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                        help="prompt length of --only prefill (the JSON line always uses 2048)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    run_ours(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
