"""Shared helpers of the GPU tests: tiny model folders, replay schedules, comparisons."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from qwen_inference_lab_b200.weights import write_safetensors
from tests.plain import qwen3_plain as plain
from tests.tiny_configs import tiny_weights

TOLERANCE = {torch.float32: dict(atol=1e-5, rtol=1e-5), torch.bfloat16: dict(atol=4e-3, rtol=2e-2)}


def write_folder(cfg, seed, folder, storage=torch.bfloat16) -> dict:
    """Write config.json + model.safetensors for a tiny configuration; returns the float32 weights."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    weights = tiny_weights(cfg, seed, torch.float32)
    stored = {k: v.to(storage) for k, v in weights.items()}
    if cfg.get("tie_word_embeddings", True):
        stored.pop("lm_head.weight", None)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", stored)
    return weights


def random_tokens(cfg, count, seed):
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab_size"], (count,), generator=generator).tolist()


def build_engine_parts(folder, dtype, *, num_pages, page_size, max_requests=4, use_graphs=True):
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.engine import StepRunner
    from qwen_inference_lab_b200.loading import load_model
    model = load_model(folder, device="cuda", dtype=dtype)
    cache = CacheManager(model.cache_specs(), num_pages=num_pages, page_size=page_size,
                         max_requests=max_requests, max_context=model.max_positions, dtype=dtype,
                         device=model.device)
    cache.poison()
    runner = StepRunner(model, cache, max_step_tokens=1024, use_graphs=use_graphs)
    return model, cache, runner


class PageLedger:
    """Who held each page last: counts pages that pass from one request to another, and poisons the
    pages of a request that has ended so that whoever reads a predecessor's data gets NaN."""

    def __init__(self, cache):
        self.cache = cache
        self.last_owner = [dict() for _ in cache.kv_groups]
        self.handovers = 0
        self.peak_held = 0

    def after_step(self, live_ids):
        for group, owners in zip(self.cache.kv_groups, self.last_owner):
            for rid in live_ids:
                for page in group.tables.get(rid, ()):
                    if page < 0:
                        continue
                    before = owners.get(page)
                    if before is not None and before != rid:
                        self.handovers += 1
                    owners[page] = rid
        self.peak_held = max(self.peak_held, max((g.capacity - len(g.free) for g in self.cache.kv_groups), default=0))

    def release(self, request_id, poison=True):
        pages = [[p for p in g.tables[request_id] if p >= 0] for g in self.cache.kv_groups]
        self.cache.release(request_id)
        if poison:
            for group, mine in zip(self.cache.kv_groups, pages):
                if mine:
                    group.storage[:, torch.tensor(mine, device=group.storage.device)] = float("nan")


def run_schedule(runner, cache, schedule, ledger=None):
    """schedule: list of steps; a step is (entries, ended) with entries = [(id, tokens, want)].

    Returns {(id, absolute position): float32 logits row on the CPU}.  With a ``PageLedger`` the pages
    of ended requests are filled with NaN and hand-overs between requests are counted.
    """
    from qwen_inference_lab_b200.engine import StepEntry
    rows = {}
    for entries, ended in schedule:
        batch = []
        for request_id, tokens, want in entries:
            if request_id not in cache.rows:
                assert cache.admit(request_id)
            batch.append(StepEntry(request_id, list(tokens), list(want)))
        starts = {e.request_id: cache.written(e.request_id) for e in batch}
        logits = runner.run(batch) if batch else None
        if ledger is not None:
            ledger.after_step([e.request_id for e in batch])
        if logits is not None:
            logits = logits.float().cpu()
            index = 0
            for e in batch:
                for w in e.want:
                    rows[(e.request_id, starts[e.request_id] + w)] = logits[index]
                    index += 1
            assert index == logits.shape[0]
        for request_id in ended:
            if ledger is not None:
                ledger.release(request_id)
            else:
                cache.release(request_id)
        cache.check_invariants()
    runner.check()
    return rows


def peak_pages(schedule, page_size, round_to=1):
    """The most pages that live requests hold at any step of ``schedule`` (each request's tokens rounded
    up to ``round_to`` first): the smallest pool the schedule runs in."""
    held, peak = {}, 0
    for entries, ended in schedule:
        for rid, tokens, _ in entries:
            held[rid] = held.get(rid, 0) + len(tokens)
        now = sum(-(-(-(-n // round_to) * round_to) // page_size) for n in held.values())
        peak = max(peak, now)
        for rid in ended:
            held.pop(rid, None)
    return peak


def simulate_pages(schedule, num_pages, page_size, max_requests=8):
    """Walk ``schedule`` through a cache manager on the CPU (no model): (hand-overs of pages between
    requests, most pages held).  The replay program takes and frees pages in the same order."""
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.parts import KVCacheSpec
    cache = CacheManager([KVCacheSpec(1, 1)], num_pages=num_pages, page_size=page_size, max_requests=max_requests,
                         max_context=1 << 20, dtype=torch.float32, device="cpu")
    ledger = PageLedger(cache)
    for entries, ended in schedule:
        for rid, tokens, _ in entries:
            if rid not in cache.rows:
                assert cache.admit(rid)
            end = cache.written(rid) + len(tokens)
            cache.ensure(rid, end)
            cache.advance(rid, end)
        ledger.after_step([rid for rid, _, _ in entries])
        for rid in ended:
            ledger.release(rid, poison=False)
    return ledger.handovers, ledger.peak_held


def cut(tokens, sizes):
    """Cut ``tokens`` into portions of the given sizes, repeating the pattern as needed."""
    portions, i, k = [], 0, 0
    while i < len(tokens):
        size = sizes[k % len(sizes)]
        portions.append(tokens[i:i + size])
        i += size
        k += 1
    return portions


def whole_schedule(requests):
    """Each request alone and whole, all positions wanted."""
    return [([(rid, tokens, list(range(len(tokens))))], [rid]) for rid, tokens in requests.items()]


def tail_decode_schedule(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    schedule = []
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        schedule.append(([(rid, tokens[:head], list(range(head)))], []))
        for i in range(head, len(tokens)):
            schedule.append(([(rid, tokens[i:i + 1], [0])], [rid] if i == len(tokens) - 1 else []))
        if head == len(tokens):
            schedule[-1] = (schedule[-1][0], [rid])
    return schedule


def chunk_schedule(requests, sizes=(16, 7, 2, 5, 2, 33, 3)):
    schedule = []
    for rid, tokens in requests.items():
        portions = cut(tokens, sizes)
        for i, portion in enumerate(portions):
            schedule.append(([(rid, portion, list(range(len(portion))))], [rid] if i == len(portions) - 1 else []))
    return schedule


def mixed_schedule(requests, max_live=4, sizes=(9, 2, 17, 4, 30)):
    """Up to ``max_live`` requests at once: portions of prompts beside single tokens of others.

    Every request first walks through the first 60% of its tokens in portions, then the
    rest one token a step; a request is left out of a step now and then; a new one starts
    when one ends, so pages are given back and used again.
    """
    pending = list(requests.items())
    live, schedule, tick = {}, [], 0
    while pending or live:
        while pending and len(live) < max_live:
            rid, tokens = pending.pop(0)
            live[rid] = dict(tokens=tokens, done=0, split=max(2, int(len(tokens) * 0.6)), k=len(live))
        entries, ended = [], []
        for rid, state in list(live.items()):
            tick += 1
            if tick % 5 == 0 and len(live) > 1:
                continue        # sits this step out
            remaining = len(state["tokens"]) - state["done"]
            if state["done"] < state["split"]:
                size = min(sizes[(state["k"] + tick) % len(sizes)], state["split"] - state["done"])
            else:
                size = 1
            size = min(size, remaining)
            portion = state["tokens"][state["done"]:state["done"] + size]
            entries.append((rid, portion, list(range(len(portion)))))
            state["done"] += size
            if state["done"] == len(state["tokens"]):
                ended.append(rid)
                del live[rid]
        if entries:
            schedule.append((entries, ended))
    return schedule


def plain_rows(requests, weights, cfg, dtype=torch.float32):
    rows = {}
    for rid, tokens in requests.items():
        logits = plain.logits(tokens, weights, cfg, dtype)
        for position in range(len(tokens)):
            rows[(rid, position)] = logits[position]
    return rows


def assert_rows_close(actual, expected, dtype, what="", yardstick=None):
    """Compare logits rows with the plain implementation's float32 rows.

    float32: elementwise ``atol``/``rtol``.  bfloat16: rounding noise is as large as some
    logits, so the bar is what bfloat16 costs the plain implementation itself: ``yardstick``
    holds the plain implementation's rows computed in bfloat16 at the reference's rounding
    points, and the engine may be at most 1.5 times as far from the float32 rows as that
    (root-mean-square error of every row against the mean row error of the yardstick or, where
    larger, the yardstick's error in that row; the largest error against the yardstick's largest).
    Tokens are judged beside the numbers (a tie can flip a token inside any tolerance,
    docs/OPTIMIZATION_DEBUG_LOG.md:102-115 of the reference): wherever the float32 row's best logit
    leads the runner-up by more than four times the plain bfloat16 implementation's largest error in
    that row, the engine's best token must be the float32 row's.
    """
    assert set(actual) == set(expected), f"{what}: different (request, position) sets"
    keys = sorted(expected, key=lambda k: (str(k[0]), k[1]))
    for key in keys:
        assert torch.isfinite(actual[key]).all(), f"{what}: non-finite logits at {key}"
    if dtype == torch.float32:
        tolerance = TOLERANCE[dtype]
        bad = [k for k in keys if ((actual[k] - expected[k]).abs() - tolerance["atol"]
                                   - tolerance["rtol"] * expected[k].abs()).max() > 0]
        if bad:
            worst = max(bad, key=lambda k: (actual[k] - expected[k]).abs().max().item())
            raise AssertionError(
                f"{what}: logits differ; first wrong (request, position) = {bad[0]}, worst = {worst} "
                f"max abs difference {(actual[worst] - expected[worst]).abs().max().item():.3e}")
        return
    assert yardstick is not None, "bfloat16 comparisons need the plain bfloat16 rows as a yardstick"
    rms = lambda rows, k: (rows[k] - expected[k]).pow(2).mean().sqrt().item()
    peak = lambda rows, k: (rows[k] - expected[k]).abs().max().item()
    bar_rms = 1.5 * sum(rms(yardstick, k) for k in keys) / len(keys)
    bar_peak = 1.5 * max(peak(yardstick, k) for k in keys)
    # a row is judged against the plain bfloat16 error of that same row where that is the larger bar: some
    # rows are hard for bfloat16 itself (seen: a row at 2.8 times the mean error in the plain bfloat16
    # implementation and 2.7 times in the engine)
    bad = [k for k in keys if rms(actual, k) > max(bar_rms * 1.5, 1.5 * rms(yardstick, k))
           or peak(actual, k) > bar_peak]
    judged = flipped = 0
    for k in keys:
        best = expected[k].topk(2).values
        if (best[0] - best[1]).item() > 4 * peak(yardstick, k):
            judged += 1
            if actual[k].argmax().item() != expected[k].argmax().item():
                flipped += 1
                bad.append(k)
    assert judged > len(keys) // 4, f"{what}: only {judged} of {len(keys)} rows have a clear best token; use other weights"
    mean_rms = sum(rms(actual, k) for k in keys) / len(keys)
    if bad or mean_rms > bar_rms:
        worst = max(keys, key=lambda k: peak(actual, k))
        raise AssertionError(
            f"{what}: bfloat16 logits are further from the float32 rows than 1.5x the plain bfloat16 "
            f"arithmetic: first wrong (request, position) = {bad[0] if bad else None}, worst = {worst}, "
            f"mean rms {mean_rms:.3e} (bar {bar_rms:.3e}), peak {peak(actual, worst):.3e} (bar {bar_peak:.3e}), "
            f"{flipped} of {judged} clear best tokens differ")


def check_greedy(prompt, tokens, weights, cfg, dtype):
    """The engine's tokens are the plain implementation's best token at every step.  In bfloat16 a token may
    differ only where the plain float32 logits of the two lie closer than four times what bfloat16 costs the
    plain implementation itself on that row (a tie within rounding); the engine's own token is then followed."""
    sequence = list(prompt)
    for token in tokens:
        logits = plain.logits(sequence, weights, cfg)[-1]
        best = int(logits.argmax())
        if token != best:
            assert dtype == torch.bfloat16, f"token {token} instead of {best} after {len(sequence)} tokens"
            noise = (plain.logits(sequence, weights, cfg, torch.bfloat16)[-1] - logits).abs().max().item()
            assert float(logits[best] - logits[token]) < 4 * noise, \
                f"token {token} instead of {best} after {len(sequence)} tokens: its logit is " \
                f"{float(logits[best] - logits[token]):.4f} lower, bfloat16 costs {noise:.4f} on this row"
        sequence.append(token)


# ----------------------------------------------------------------------------- parts alone
class OnePartModel:
    """Just enough of a model for the step function to run a single part over a batch.

    ``body(ctx, x, view)`` is called with the rows of ``inputs`` that belong to the step's
    tokens (request order, then position) and must return a tensor; outputs are collected.
    """

    def __init__(self, part, hidden, dtype, body, vocab_size=1 << 20, max_positions=4096):
        from qwen_inference_lab_b200.parts import LayerCall
        self.part, self.body, self.hidden = part, body, hidden
        self.device, self.dtype = torch.device("cuda"), dtype
        self.vocab_size, self.max_positions = vocab_size, max_positions
        self.order = [LayerCall(0)]
        self.inputs = None           # [n_inputs, hidden]: token id t of a step selects row t
        self.outputs = []

    def cache_specs(self):
        spec = getattr(self.part, "cache_spec", lambda: None)()
        return [spec]

    def is_graph_safe(self):
        return False

    def step_planners(self):
        return self.part.step_planners() if hasattr(self.part, "step_planners") else {}

    def forward(self, ctx, views, logit_rows):
        x = self.inputs[ctx.token_ids.long()].contiguous()
        self.outputs.append(self.body(ctx, x, views[0]).float().cpu())
        return None


def run_part(part, hidden, dtype, body, inputs_by_request, cuts, page_size=4, num_pages=64):
    """Run ``part`` over whole sequences of input rows cut into portions; returns {request: [T, out]}.

    ``inputs_by_request``: {id: tensor [T, hidden]}; ``cuts``: {id: list of portion sizes}.
    All requests advance together, one portion each per step (a mixed batch).
    """
    from qwen_inference_lab_b200.cache import CacheManager
    from qwen_inference_lab_b200.engine import StepEntry, StepRunner
    model = OnePartModel(part, hidden, dtype, body)
    cache = CacheManager(model.cache_specs(), num_pages=num_pages, page_size=page_size, max_requests=4,
                         max_context=4096, dtype=dtype, device="cuda")
    cache.poison()
    runner = StepRunner(model, cache, use_graphs=False)
    offsets, rows = {}, []
    for rid, x in inputs_by_request.items():
        offsets[rid] = sum(r.shape[0] for r in rows)
        rows.append(x)
        cache.admit(rid)
    model.inputs = torch.cat(rows).to(dtype).cuda()
    done = {rid: 0 for rid in inputs_by_request}
    portions = {rid: list(sizes) for rid, sizes in cuts.items()}
    collected = {rid: [] for rid in inputs_by_request}
    while any(portions.values()):
        entries, owners = [], []
        for rid in inputs_by_request:
            if portions[rid]:
                size = portions[rid].pop(0)
                ids = list(range(offsets[rid] + done[rid], offsets[rid] + done[rid] + size))
                entries.append(StepEntry(rid, ids, []))
                owners.append((rid, size))
                done[rid] += size
        runner.run(entries)
        out = model.outputs.pop()
        start = 0
        for rid, size in owners:
            collected[rid].append(out[start:start + size])
            start += size
    return {rid: torch.cat(parts) for rid, parts in collected.items()}
