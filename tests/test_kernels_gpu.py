"""Each kernel alone against a plain PyTorch float32 reference, at sizes other than the engine's."""
import math

import pytest
import torch

from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
IDS = ["float32", "bfloat16"]


def ops():
    from qwen_inference_lab_b200.kernels import ops as module
    return module


def close(actual, expected, dtype, scale=1.0):
    if dtype == torch.float32:
        torch.testing.assert_close(actual.float().cpu(), expected.float().cpu(), atol=2e-6 * scale, rtol=2e-5)
    else:  # one bfloat16 rounding of the result (2^-8 relative) plus the same on a few inputs
        torch.testing.assert_close(actual.float().cpu(), expected.float().cpu(), atol=8e-3 * scale, rtol=8e-3)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("table_dtype", DTYPES, ids=IDS)
def test_embed_gather(dtype, table_dtype):
    torch.manual_seed(0)
    table = torch.randn(333, 72).to(table_dtype).cuda()
    ids = torch.tensor([0, 332, 17, 17, 5], dtype=torch.int32).cuda()
    out = torch.empty(5, 72, dtype=dtype).cuda()
    ops().embed_gather(table, ids, out)
    assert torch.equal(out.cpu(), table.cpu()[ids.cpu().long()].to(dtype))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("weight_dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("width,eps", [(96, 1e-5), (1000, 1e-6), (4104, 1e-3)])
def test_rmsnorm(dtype, weight_dtype, width, eps):
    torch.manual_seed(1)
    x = (torch.randn(7, width) * 3).to(dtype)
    w = (1 + 0.1 * torch.randn(width)).to(weight_dtype)
    expected = plain.rms_norm(x.float(), w.float(), eps) if dtype == torch.float32 else \
        (plain.rms_norm(x, torch.ones(width), eps).float() * w.float()).to(dtype)
    out = ops().rmsnorm(x.cuda(), w.cuda(), eps)
    close(out, expected, dtype, scale=3)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32).cuda()
    picked = ops().rmsnorm(x.cuda(), w.cuda(), eps, rows=rows)
    assert torch.equal(picked.cpu(), out.cpu()[[6, 0, 3]])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("width", [200, 37, 1024])
def test_silu_mul(dtype, width):
    torch.manual_seed(2)
    gate_up = (torch.randn(9, 2 * width) * 2).to(dtype)
    expected = torch.nn.functional.silu(gate_up[:, :width]) * gate_up[:, width:]
    out = ops().silu_mul(gate_up.cuda())
    close(out, expected, dtype, scale=4)


@pytest.mark.parametrize("act,wt", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                    (torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (3, 200, 96), (65, 129, 130), (130, 64, 33)])
def test_gemm_f32(act, wt, m, n, k):
    torch.manual_seed(3)
    a = torch.randn(m, k).to(act)
    w = (torch.randn(n, k) * 0.1).to(wt)
    bias = (torch.randn(n) * 0.1).to(wt)
    residual = torch.randn(m, n).to(act)
    expected = a.double() @ w.double().t() + bias.double() + residual.double()
    out = ops().gemm_f32(a.cuda(), w.cuda(), bias=bias.cuda(), residual=residual.cuda())
    close(out, expected.float(), act, scale=4)
    plain_out = ops().gemm_f32(a.cuda(), w.cuda())
    close(plain_out, (a.double() @ w.double().t()).float(), act, scale=4)
    # a row's result does not depend on which other rows share the launch
    alone = ops().gemm_f32(a[-1:].cuda().contiguous(), w.cuda())
    assert torch.equal(alone.cpu()[0], plain_out.cpu()[-1])


def paged(keys, values, page_size, num_pages, dtype, seed=0, rows=1, row=0, poison=True):
    """Scatter dense keys/values [T, Hkv, D] into a poisoned pool through a shuffled page list."""
    T, n_kv, d = keys.shape
    generator = torch.Generator().manual_seed(seed)
    order = torch.randperm(num_pages, generator=generator).tolist()
    needed = (T + page_size - 1) // page_size
    pool = torch.full((num_pages, 2, n_kv, page_size, d), float("nan") if poison else 0.0, dtype=dtype)
    table = torch.full((rows, needed + 2), -1, dtype=torch.int32)
    for i in range(needed):
        page = order[i]
        table[row, i] = page
        chunk = slice(i * page_size, min(T, (i + 1) * page_size))
        count = chunk.stop - chunk.start
        pool[page, 0, :, :count] = keys[chunk].transpose(0, 1).to(dtype)
        pool[page, 1, :, :count] = values[chunk].transpose(0, 1).to(dtype)
    return pool, table


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("n_q,n_kv,d,rot,page", [(4, 2, 16, 16, 4), (6, 2, 48, 32, 3), (8, 8, 128, 128, 16), (3, 1, 72, 0, 5)])
def test_qk_norm_rope_store(dtype, n_q, n_kv, d, rot, page):
    from qwen_inference_lab_b200.parts import rotary_table
    torch.manual_seed(4)
    T, theta, eps = 11, 10000.0, 1e-5
    qkv = torch.randn(T, (n_q + 2 * n_kv) * d).to(dtype)
    qw, kw = (1 + 0.1 * torch.randn(d)).to(dtype), (1 + 0.1 * torch.randn(d)).to(dtype)
    start = 6
    positions = torch.arange(start, start + T, dtype=torch.int32)
    q, k, v = qkv.split([n_q * d, n_kv * d, n_kv * d], dim=1)
    q, k, v = q.reshape(T, n_q, d), k.reshape(T, n_kv, d), v.reshape(T, n_kv, d)
    qn, kn = plain.rms_norm(q, qw, eps), plain.rms_norm(k, kw, eps)
    if rot:
        angles = plain.rotary_angles(positions, rot, theta)
        qn = torch.cat((plain.rotate(qn[..., :rot], angles), qn[..., rot:]), dim=-1)
        kn = torch.cat((plain.rotate(kn[..., :rot], angles), kn[..., rot:]), dim=-1)
    num_pages = 12
    pool, table = paged(torch.zeros(start + T, n_kv, d), torch.zeros(start + T, n_kv, d), page, num_pages, dtype,
                        rows=3, row=1)
    pool_before = pool.clone()
    rope = rotary_table(rot, theta, 64, dtype).cuda() if rot else None
    q_out = torch.empty(T, n_q * d, dtype=dtype).cuda()
    pool_gpu = pool.cuda()
    ops().qk_norm_rope_store(qkv.cuda(), q_out, pool_gpu, qw.cuda(), kw.cuda(), eps, rope, rot, positions.cuda(),
                             torch.full((T,), 1, dtype=torch.int32).cuda(), table.cuda(), n_q, n_kv, d, page)
    close(q_out.reshape(T, n_q, d), qn, dtype, scale=4)
    got = pool_gpu.cpu()
    for i, pos in enumerate(range(start, start + T)):
        page_id, slot = int(table[1, pos // page]), pos % page
        close(got[page_id, 0, :, slot], kn[i], dtype, scale=4)
        assert torch.equal(got[page_id, 1, :, slot], v[i])
        pool_before[page_id, :, :, slot] = got[page_id, :, :, slot]
    # nothing else in the pool was touched
    assert torch.equal(torch.nan_to_num(got.float(), nan=-7.0), torch.nan_to_num(pool_before.float(), nan=-7.0))


def attention_case(n_q, n_kv, d, lengths, chunk_starts, dtype, page, seed, window=0, spike=None):
    """Requests with histories in a poisoned paged pool and query chunks over their last tokens.

    Returns the flat queries, the metadata and the expected outputs of every query token.
    ``spike`` = (request, key position): that key and the request's queries are scaled so that
    one far score stands out, and its value is made large: a kernel that drops it shows.
    """
    generator = torch.Generator().manual_seed(seed)
    num_pages = sum((n + page - 1) // page for n in lengths) + 3
    pool = torch.full((num_pages, 2, n_kv, page, d), float("nan"), dtype=dtype)
    free = torch.randperm(num_pages, generator=generator).tolist()
    width = max((n + page - 1) // page for n in lengths) + 1
    table = torch.full((len(lengths) + 1, width), -1, dtype=torch.int32)
    q_rows, expected, seg_start, seg_len, seg_pos0, seg_row = [], [], [], [], [], []
    for r, (length, start) in enumerate(zip(lengths, chunk_starts)):
        keys = torch.randn(length, n_kv, d, generator=generator)
        values = torch.randn(length, n_kv, d, generator=generator)
        queries = torch.randn(length, n_q, d, generator=generator)
        if spike is not None and spike[0] == r:
            keys[spike[1]] *= 6.0
            queries[start:] = keys[spike[1]].repeat_interleave(n_q // n_kv, dim=0)[None] * 0.8 \
                + 0.2 * queries[start:]
            values[spike[1]] += 25.0
        keys, values, queries = keys.to(dtype), values.to(dtype), queries.to(dtype)
        row = r + 1
        for i in range((length + page - 1) // page):
            pg = free.pop()
            table[row, i] = pg
            chunk = slice(i * page, min(length, (i + 1) * page))
            pool[pg, 0, :, :chunk.stop - chunk.start] = keys[chunk].transpose(0, 1)
            pool[pg, 1, :, :chunk.stop - chunk.start] = values[chunk].transpose(0, 1)
        full = plain.causal_attention(queries.float(), keys.float(), values.float(), d ** -0.5, window=window)
        seg_start.append(sum(seg_len))
        seg_len.append(length - start)
        seg_pos0.append(start)
        seg_row.append(row)
        q_rows.append(queries[start:].reshape(length - start, n_q * d))
        expected.append(full[start:].reshape(length - start, n_q * d))
    meta = dict(seg_start=seg_start, seg_len=seg_len, seg_pos0=seg_pos0, seg_row=seg_row)
    return torch.cat(q_rows), pool, table, meta, torch.cat(expected)


def flat_meta(meta):
    positions, token_row = [], []
    for start, length, pos0, row in zip(meta["seg_start"], meta["seg_len"], meta["seg_pos0"], meta["seg_row"]):
        positions += list(range(pos0, pos0 + length))
        token_row += [row] * length
    as_int = lambda values: torch.tensor(values, dtype=torch.int32).cuda()
    return as_int(positions), as_int(token_row)


ATTENTION_CASES = [
    # n_q, n_kv, d, lengths, chunk starts, page, window
    (4, 2, 16, [1, 15, 16, 17], [0, 14, 0, 16], 4, 0),
    (6, 2, 40, [65, 3, 511, 257], [64, 0, 300, 256], 3, 0),
    (8, 2, 128, [1025, 1, 256, 513], [1024, 0, 200, 512], 16, 0),
    (4, 4, 64, [31, 512], [30, 0], 8, 0),
    (16, 1, 256, [3, 257], [2, 190], 7, 0),
    (4, 2, 32, [300, 129, 700], [250, 128, 699], 16, 100),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("case", ATTENTION_CASES, ids=[f"case{i}" for i in range(len(ATTENTION_CASES))])
def test_attention_generic(dtype, case):
    n_q, n_kv, d, lengths, starts, page, window = case
    q, pool, table, meta, expected = attention_case(n_q, n_kv, d, lengths, starts, dtype, page, seed=5, window=window)
    positions, token_row = flat_meta(meta)
    out = torch.empty_like(q).cuda()
    ops().attention_generic(q.cuda(), pool.cuda(), out, positions, token_row, table.cuda(), n_q, n_kv, d, page,
                            window, d ** -0.5)
    close(out, expected, dtype, scale=2)


def run_mma(q, pool, table, meta, n_q, n_kv, d, page, window, span_len=256, tickets=False):
    from qwen_inference_lab_b200.kernels import attention_mma
    as_int = lambda values: torch.tensor(values, dtype=torch.int32).cuda()
    tile_info, decode_info = [], []
    for start, length, pos0, row in zip(meta["seg_start"], meta["seg_len"], meta["seg_pos0"], meta["seg_row"]):
        if length == 1:
            decode_info += [start, pos0, row, 0]
        else:
            for off in range(0, length, 64):
                tile_info += [start + off, pos0 + off, min(64, length - off), row]
    out = torch.full(q.shape, float("nan"), dtype=q.dtype).cuda()
    qg, pg = q.cuda(), pool.cuda()
    if tile_info:
        attention_mma.prefill(qg, pg, out, as_int(tile_info), len(tile_info) // 4, table.cuda(),
                              n_q, n_kv, d, page, window, d ** -0.5)
    if decode_info:
        n_decode = len(decode_info) // 4
        longest = max(p0 + n for p0, n in zip(meta["seg_pos0"], meta["seg_len"]))
        if span_len == 0:       # the kernels cut the longest context, which every entry carries, into the grid's spans
            decode_info[3::4] = [longest] * n_decode
            n_spans, span_len = attention_mma.plan_spans(n_decode, n_q, n_kv, longest + 300, d, longest // 2)   # as under a recorded graph's bounds
            span_len = -span_len
        else:
            n_spans = (longest + span_len - 1) // span_len + 1   # one spare span
        part_o = torch.full((n_decode * n_q * n_spans * d,), float("nan"), dtype=torch.float32).cuda()
        part_ml = torch.full((n_decode * n_q * n_spans * 2,), float("nan"), dtype=torch.float32).cuda()
        counters = torch.zeros(n_decode * n_q, dtype=torch.int32).cuda() if tickets else None
        attention_mma.decode(qg, pg, out, as_int(decode_info), n_decode, part_o, part_ml, n_spans, span_len,
                             table.cuda(), n_q, n_kv, d, page, window, d ** -0.5, tickets=counters)
        if tickets:
            assert int(counters.sum()) == 0            # the last block of every token's spans put its counter back
    return out


MMA_CASES = [c for c in ATTENTION_CASES if c[2] % 16 == 0] + [
    (32, 8, 128, [2100, 64, 640], [2099, 0, 600], 16, 0),
    (20, 1, 48, [700, 400], [699, 330], 5, 0),          # a group of 20 heads: two head chunks per kv head
    (6, 3, 80, [520, 130], [519, 1], 16, 64),
    (3, 3, 96, [200, 70], [199, 6], 16, 0),             # head sizes between the usual ones: every multiple of 16 is taken
    (4, 2, 144, [330, 65], [300, 64], 8, 0),
]


@pytest.mark.parametrize("case", MMA_CASES, ids=[f"case{i}" for i in range(len(MMA_CASES))])
def test_attention_tensor_core(case):
    n_q, n_kv, d, lengths, starts, page, window = case
    q, pool, table, meta, expected = attention_case(n_q, n_kv, d, lengths, starts, torch.bfloat16, page, seed=6,
                                                    window=window)
    out = run_mma(q, pool, table, meta, n_q, n_kv, d, page, window)
    close(out, expected, torch.bfloat16, scale=2)
    # all-decode form of the same requests: the last token of each
    last_q = torch.stack([q[s + n - 1] for s, n in zip(meta["seg_start"], meta["seg_len"])])
    last_meta = dict(seg_start=list(range(len(lengths))), seg_len=[1] * len(lengths),
                     seg_pos0=[n - 1 for n in lengths], seg_row=meta["seg_row"])
    last_expected = torch.stack([expected[s + n - 1] for s, n in zip(meta["seg_start"], meta["seg_len"])])
    for span_len in (64, 256, 2048, 0):
        out = run_mma(last_q, pool, table, last_meta, n_q, n_kv, d, page, window, span_len=span_len)
        close(out, last_expected, torch.bfloat16, scale=2)
        # the spans merged by the span kernel's own last blocks (ticket counters) instead of a second kernel:
        # the same sums in the same order, so the same bits
        merged_in_kernel = run_mma(last_q, pool, table, last_meta, n_q, n_kv, d, page, window, span_len=span_len,
                                   tickets=True)
        assert torch.equal(out, merged_in_kernel)


@pytest.mark.parametrize("n_q,n_kv,d,lengths,page,window,rotary,norms,own", [
    (32, 8, 128, [2100, 64, 641], 16, 0, 128, True, True),
    (6, 3, 80, [520, 130, 1], 16, 64, 40, True, True),        # half of the head rotated, a window, a first token
    (4, 1, 48, [300, 77], 8, 0, 0, False, True),              # no rotation, no norms
    (16, 2, 64, [257, 70], 4, 0, 64, True, False),            # a layer that reads another layer's cache
])
def test_attention_single_tokens_from_the_projection(n_q, n_kv, d, lengths, page, window, rotary, norms, own):
    """The single-token kernel fed with the raw q/k/v projection (it norms, rotates and stores what it needs)
    against the two kernels it replaces: the same outputs and the same pages, bit for bit."""
    from types import SimpleNamespace
    from qwen_inference_lab_b200.kernels import attention_mma
    from qwen_inference_lab_b200.parts.rotary import rotary_table
    _, pool, table, meta, _ = attention_case(n_q, n_kv, d, lengths, [n - 1 for n in lengths], torch.bfloat16, page,
                                             seed=16, window=window)
    torch.manual_seed(17)
    n, own_kv, eps = len(lengths), (n_kv if own else 0), 1e-5
    qkv = torch.randn(n, (n_q + 2 * own_kv) * d).to(torch.bfloat16).cuda()
    q_norm = (1 + 0.3 * torch.randn(d)).to(torch.bfloat16).cuda() if norms else None
    k_norm = (1 + 0.3 * torch.randn(d)).to(torch.bfloat16).cuda() if norms else None
    rope = rotary_table(rotary, 10000.0, 4096, torch.bfloat16).cuda() if rotary else None
    as_int = lambda values: torch.tensor(values, dtype=torch.int32).cuda()
    positions, token_row = as_int([m - 1 for m in lengths]), as_int(meta["seg_row"])
    longest = max(lengths)
    decode_info = as_int([v for i in range(n) for v in (i, lengths[i] - 1, meta["seg_row"][i], longest)])
    for span_len, bound in ((64, longest), (256, longest), (2048, longest), (0, longest), (0, 2 * longest + 100)):
        # span_len 0: the kernels choose the span; ``bound`` stands for a recorded graph's upper bound
        if span_len == 0:
            n_spans, span_len = attention_mma.plan_spans(n, n_q, n_kv, bound, d, longest)
            span_len = -span_len
            planned = True
        else:
            n_spans, planned = (longest + span_len - 1) // span_len, False
        scratch = lambda: (torch.full((n * n_q * n_spans * d,), float("nan")).cuda(),
                           torch.full((n * n_q * n_spans * 2,), float("nan")).cuda())
        # the two kernels
        pages_a = pool.cuda().clone()
        q = torch.empty(n, n_q * d, dtype=torch.bfloat16).cuda()
        ops().qk_norm_rope_store(qkv, q, pages_a, q_norm, k_norm, eps, rope, rotary, positions, token_row, table.cuda(),
                                 n_q, own_kv, d, page)
        out_a = torch.full((n, n_q * d), float("nan"), dtype=torch.bfloat16).cuda()
        attention_mma.decode(q, pages_a, out_a, decode_info, n, *scratch(), n_spans, span_len, table.cuda(), n_q, n_kv,
                             d, page, window, d ** -0.5)
        # the one kernel
        pages_b = pool.cuda().clone()
        out_b = torch.full((n, n_q * d), float("nan"), dtype=torch.bfloat16).cuda()
        part_o, part_ml = scratch()
        plan = SimpleNamespace(array=dict(decode_info=decode_info),
                               count=dict(decode_info=4 * n, tile_info=0, big_tile_info=0, rest_tile_info=0))
        ctx = SimpleNamespace(n_tokens=n, max_context=bound, min_context=longest,
                              plans={attention_mma.PLAN_KEY: plan},
                              extras={"attn_decode_scratch": (part_o, part_ml, torch.zeros(n * n_q, dtype=torch.int32).cuda())},
                              device=qkv.device)
        cache = SimpleNamespace(pages=pages_b, block_table=table.cuda(), page_size=page)
        assert attention_mma.projection_tail_usable(ctx, qkv, cache, n_q, n_kv, d, rotary, (q_norm, k_norm))
        attention_mma.attend_projection(ctx, qkv, cache, out_b, n_q, n_kv, own_kv, d, window, d ** -0.5, q_norm,
                                        k_norm, eps, rope, rotary)
        torch.cuda.synchronize()
        assert not torch.isnan(out_b).any()
        if planned:
            assert torch.equal(out_a, out_b)        # the same spans in both: the same bits
        else:
            close(out_b, out_a, torch.bfloat16, scale=2)
        same = (pages_a == pages_b) | (torch.isnan(pages_a) & torch.isnan(pages_b))
        assert bool(same.all())


@pytest.mark.parametrize("form", ["portion", "single"])
def test_attention_far_key_stands_out(form):
    """One key hundreds of positions back dominates the softmax: dropping it would change everything."""
    n_q, n_kv, d, page = 8, 2, 64, 16
    lengths, starts = [900, 40], ([700, 0] if form == "portion" else [899, 39])
    q, pool, table, meta, expected = attention_case(n_q, n_kv, d, lengths, starts, torch.bfloat16, page, seed=7,
                                                    spike=(0, 129))
    assert expected[:lengths[0] - starts[0]].abs().mean() > 10     # the spiked value really dominates
    out = run_mma(q, pool, table, meta, n_q, n_kv, d, page, 0)
    close(out, expected, torch.bfloat16, scale=25)
    generic = torch.empty_like(q).cuda()
    positions, token_row = flat_meta(meta)
    ops().attention_generic(q.cuda(), pool.cuda(), generic, positions, token_row, table.cuda(), n_q, n_kv, d, page,
                            0, d ** -0.5)
    close(generic, expected, torch.bfloat16, scale=25)


def test_sample_rows_greedy_ties_and_nonfinite():
    logits = torch.zeros(4, 1000)
    logits[0, 17] = 3.0; logits[0, 900] = 3.0          # tie: lowest index wins
    logits[1, 999] = 1.0
    logits[2, 5] = float("nan")
    logits[3, 7] = float("inf")
    tokens, bad = ops().sample_rows(logits.cuda())
    assert tokens.cpu().tolist()[:2] == [17, 999]
    assert bad.cpu().tolist() == [0, 0, 1, 1]
    # a vocabulary that is cut into many slices: equal maxima in the first and the last slice, a lone
    # maximum in the very last entry, a non-finite value in a middle slice; twice, since the slices'
    # tickets must be back at zero after a call; and more rows than one launch takes
    wide = torch.randn(4, 100003)
    wide[0, 123] = 50.0; wide[0, 99990] = 50.0
    wide[1, 100002] = 60.0
    wide[2, 51234] = float("-inf")
    for _ in range(2):
        tokens, bad = ops().sample_rows(wide.cuda())
        assert tokens.cpu().tolist()[:2] == [123, 100002] and tokens.cpu().tolist()[3] == int(wide[3].argmax())
        assert bad.cpu().tolist() == [0, 0, 1, 0]
    many = torch.randn(5000, 7)
    tokens, bad = ops().sample_rows(many.cuda())
    assert torch.equal(tokens.cpu().long(), many.argmax(dim=1)) and int(bad.sum()) == 0


def test_feed_tokens_and_the_sampler_tickets():
    """Tokens that stay on the device between two steps: the kernel that puts them into the next step's
    token list (out-of-range places and sources are left alone), and the sampler's begin/finish pair."""
    from qwen_inference_lab_b200.sampling import NonFiniteLogits, Sampler
    token_ids = torch.tensor([5, -1, 7, -1, -1, 9], dtype=torch.int32).cuda()
    pairs = torch.tensor([1, 2, 3, 0, 4, 99, 77, 1], dtype=torch.int32).cuda()      # (place, source) pairs
    source = torch.tensor([40, 41, 42], dtype=torch.int32).cuda()
    ops().feed_tokens(token_ids, pairs, 4, source)
    assert token_ids.cpu().tolist() == [5, 42, 7, 40, -1, 9]
    sampler = Sampler("cuda", max_rows=2)
    logits = torch.randn(3, 1000)
    first = sampler.begin(logits.cuda())
    second = sampler.begin((-logits).cuda())              # two tickets may be open at a time
    assert sampler.finish(first) == logits.argmax(dim=1).tolist()
    assert first.tokens.cpu().tolist() == logits.argmax(dim=1).tolist()
    assert sampler.finish(second) == logits.argmin(dim=1).tolist()
    bad = logits.clone(); bad[1, 3] = float("nan")
    with pytest.raises(NonFiniteLogits):
        sampler.finish(sampler.begin(bad.cuda()))
    assert sampler.choose(logits.cuda()) == logits.argmax(dim=1).tolist()


def test_sample_rows_temperature_matches_plain_and_is_batch_independent():
    torch.manual_seed(8)
    vocab = 1517
    logits = torch.randn(5, vocab) * 2
    temperature = torch.tensor([0.8, 0.0, 1.3, 0.8, 0.5])
    seed = torch.tensor([11, 12, 13, 11, 99], dtype=torch.int64)
    counter = torch.tensor([0, 1, 2, 0, 7], dtype=torch.int64)
    tokens, bad = ops().sample_rows(logits.cuda(), temperature.cuda(), seed.cuda(), counter.cuda())
    tokens = tokens.cpu().tolist()
    assert bad.cpu().sum() == 0
    for r in range(5):
        assert tokens[r] == plain.sample(logits[r], float(temperature[r]), int(seed[r]), int(counter[r]))
    alone, _ = ops().sample_rows(logits[2:3].cuda().contiguous(), temperature[2:3].cuda(), seed[2:3].cuda(),
                                 counter[2:3].cuda())
    assert alone.cpu().tolist() == [tokens[2]]
    # the draws follow softmax(logits / T): chi-square-free sanity check on a small vocabulary
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).repeat(4000, 1)
    t = torch.full((4000,), 0.7)
    drawn, _ = ops().sample_rows(small.cuda(), t.cuda(), torch.arange(4000, dtype=torch.int64).cuda(),
                                 torch.zeros(4000, dtype=torch.int64).cuda())
    freq = torch.bincount(drawn.cpu().long(), minlength=4).float() / 4000
    want = torch.softmax(small[0] / 0.7, dim=0)
    assert (freq - want).abs().max() < 0.03


def test_sample_rows_with_settings_in_state_slots():
    """Temperature, seed and the number of draws kept per request on the device: the same tokens as with the
    three uploaded arrays, and the kernel counts the draws itself."""
    from qwen_inference_lab_b200.sampling import Sampler
    torch.manual_seed(18)
    vocab = 70001                           # several slices a row: every block must read the count before it moves
    logits = torch.randn(3, vocab) * 2
    state = torch.zeros(6, 4, dtype=torch.int64).cuda()
    sampler = Sampler("cuda", max_rows=4)
    sampler.configure(state, 4, 0.8, 11)
    sampler.configure(state, 1, 1.3, 2**63 + 5)            # seeds are taken modulo 2^63
    owner = torch.tensor([4, 2, 1], dtype=torch.int32).cuda()      # slot 2 was never configured: greedy
    for draw in range(3):
        tokens = sampler.finish(sampler.begin(logits.cuda() + draw, state=state, owner=owner))
        assert tokens[0] == plain.sample(logits[0] + draw, 0.8, 11, draw)
        assert tokens[1] == int((logits[1] + draw).argmax())
        assert tokens[2] == plain.sample(logits[2] + draw, 1.3, 5, draw)
    assert state[:, 2].cpu().tolist() == [0, 3, 3, 0, 3, 0]
    with pytest.raises(Exception, match="owners"):
        ops().sample_rows(logits.cuda(), state=state)


@pytest.mark.parametrize("m,n,k", [(1, 16, 8), (3, 200, 96), (8, 129, 136), (9, 64, 4096), (16, 1000, 520)])
def test_gemm_small_m(m, n, k):
    torch.manual_seed(9)
    a = torch.randn(m, k).to(torch.bfloat16)
    w = (torch.randn(n, k) * 0.1).to(torch.bfloat16)
    bias = (torch.randn(n) * 0.1).to(torch.bfloat16)
    residual = torch.randn(m, n).to(torch.bfloat16)
    product = a.double() @ w.double().t()
    close(ops().gemm_small_m(a.cuda(), w.cuda()), product.float(), torch.bfloat16, scale=4)
    close(ops().gemm_small_m(a.cuda(), w.cuda(), bias=bias.cuda(), residual=residual.cuda()),
          (product + bias.double() + residual.double()).float(), torch.bfloat16, scale=4)
    exact = ops().gemm_small_m(a.cuda(), w.cuda(), out_float32=True)
    assert exact.dtype == torch.float32
    torch.testing.assert_close(exact.cpu(), product.float(), atol=1e-4, rtol=1e-4)
    # in place on the residual, and a row's result does not depend on the other rows
    buffer = residual.cuda().clone()
    ops().gemm_small_m(a.cuda(), w.cuda(), residual=buffer, out=buffer)
    close(buffer, (product + residual.double()).float(), torch.bfloat16, scale=4)
    alone = ops().gemm_small_m(a[-1:].cuda().contiguous(), w.cuda(), out_float32=True)
    assert torch.equal(alone.cpu()[0], exact.cpu()[-1])


@pytest.mark.parametrize("m,n,k,eps", [(1, 16, 8, 1e-6), (3, 200, 96, 1e-5), (8, 136, 520, 1e-6), (9, 64, 4096, 3e-6),
                                       (16, 1000, 1032, 1e-6)])
def test_gemm_small_m_with_the_norm_inside(m, n, k, eps):
    """RMSNorm fused into the product: rows of very different size (the norm must bring each to its
    own scale), a norm weight far from one, and the same epilogues."""
    torch.manual_seed(14)
    a = (torch.randn(m, k) * torch.logspace(-2, 2, m).unsqueeze(1)).to(torch.bfloat16)
    norm_w = (1 + torch.randn(k) * 0.3).to(torch.bfloat16)
    w = (torch.randn(n, k) * 0.1).to(torch.bfloat16)
    bias = (torch.randn(n) * 0.1).to(torch.bfloat16)
    residual = torch.randn(m, n).to(torch.bfloat16)
    normed = a.double() * torch.rsqrt(a.double().pow(2).mean(-1, keepdim=True) + eps) * norm_w.double()
    product = normed @ w.double().t()
    run = lambda **kw: ops().gemm_small_m(a.cuda(), w.cuda(), norm_weight=norm_w.cuda(), norm_eps=eps, **kw)
    close(run(), product.float(), torch.bfloat16, scale=4)
    close(run(bias=bias.cuda(), residual=residual.cuda()), (product + bias.double() + residual.double()).float(),
          torch.bfloat16, scale=4)
    exact = run(out_float32=True)
    # one bfloat16 rounding of x * w_norm is all that separates this from the float64 product
    torch.testing.assert_close(exact.cpu(), product.float(), atol=0.03 * float(product.abs().max()) / 4, rtol=0.02)
    # against the two-kernel form (norm kernel, then the product): the same up to the norm's two roundings
    separate = ops().gemm_small_m(ops().rmsnorm(a.cuda(), norm_w.cuda(), eps), w.cuda(), out_float32=True)
    assert (exact - separate).abs().max() <= 0.03 * float(product.abs().max())
    assert (exact.cpu() - product.float()).abs().mean() <= 1.2 * (separate.cpu() - product.float()).abs().mean()
    alone = ops().gemm_small_m(a[-1:].cuda().contiguous(), w.cuda(), norm_weight=norm_w.cuda(), norm_eps=eps,
                               out_float32=True)
    assert torch.equal(alone.cpu()[0], exact.cpu()[-1])
    if n % 16 == 0:     # the gate/up epilogue scales both halves before the activation
        gate_up = run(silu_pairs=True)
        half = product.float().view(m, n // 16, 2, 8)
        expected = torch.nn.functional.silu(half[:, :, 0]) * half[:, :, 1]
        close(gate_up, expected.reshape(m, n // 2), torch.bfloat16, scale=max(2.0, float(expected.abs().max()) / 2))


@pytest.mark.parametrize("m,inner,k", [(1, 8, 16), (5, 200, 96), (16, 1024, 256)])
def test_gemm_small_m_with_gate_epilogue_and_paired_silu(m, inner, k):
    torch.manual_seed(10)
    a = torch.randn(m, k).to(torch.bfloat16)
    gate_w = (torch.randn(inner, k) * 0.2).to(torch.bfloat16)
    up_w = (torch.randn(inner, k) * 0.2).to(torch.bfloat16)
    gate = (a.float() @ gate_w.float().t()).to(torch.bfloat16)
    up = (a.float() @ up_w.float().t()).to(torch.bfloat16)
    expected = torch.nn.functional.silu(gate) * up
    paired = torch.cat([gate_w, up_w]).view(2, inner // 8, 8, k).transpose(0, 1).reshape(2 * inner, k).contiguous()
    fused = ops().gemm_small_m(a.cuda(), paired.cuda(), silu_pairs=True)
    assert fused.shape == (m, inner)
    close(fused, expected, torch.bfloat16, scale=2)
    # the stand-alone activation kernel reads the same paired layout (prompt portions use it after the library GEMM)
    paired_columns = torch.cat([gate, up], dim=1).view(m, 2, inner // 8, 8).transpose(1, 2).reshape(m, 2 * inner)
    separate = ops().silu_mul(paired_columns.contiguous().cuda(), pairs8=True)
    assert torch.equal(separate.cpu(), expected)
    close(ops().silu_mul(paired_columns.float().contiguous().cuda(), pairs8=True),
          torch.nn.functional.silu(gate.float()) * up.float(), torch.float32, scale=2)


@pytest.mark.parametrize("m,n,k,eps", [(1, 32, 8, 1e-6), (5, 320, 1000, 1e-5), (8, 4768, 264, 1e-6), (12, 96, 520, 3e-6),
                                       (16, 64, 4096, 1e-6)])
def test_gemm_small_m_with_32_features_a_block(m, n, k, eps):
    """The form with two weight tiles a block (what wide matrices get; forced here at small ones too): every
    epilogue against float64, and against the 16-feature form, whose sums differ only in their order."""
    from qwen_inference_lab_b200.kernels import tuning
    torch.manual_seed(15)
    a = (torch.randn(m, k) * torch.logspace(-1, 1, m).unsqueeze(1)).to(torch.bfloat16)
    norm_w = (1 + torch.randn(k) * 0.3).to(torch.bfloat16)
    w = (torch.randn(n, k) * 0.1).to(torch.bfloat16)
    bias = (torch.randn(n) * 0.1).to(torch.bfloat16)
    residual = torch.randn(m, n).to(torch.bfloat16)
    product = a.double() @ w.double().t()
    normed = a.double() * torch.rsqrt(a.double().pow(2).mean(-1, keepdim=True) + eps) * norm_w.double()
    normed_product = normed @ w.double().t()
    wide = lambda **kw: ops().gemm_small_m(a.cuda(), w.cuda(), rows_per_block=32, **kw)
    narrow = lambda **kw: ops().gemm_small_m(a.cuda(), w.cuda(), rows_per_block=16, **kw)
    scale = max(4.0, float(product.abs().max()) / 4)
    close(wide(bias=bias.cuda(), residual=residual.cuda()), (product + bias.double() + residual.double()).float(),
          torch.bfloat16, scale=scale)
    exact = wide(out_float32=True)
    torch.testing.assert_close(exact.cpu(), product.float(), atol=1e-4 * scale, rtol=1e-4)
    torch.testing.assert_close(exact, narrow(out_float32=True), atol=1e-4 * scale, rtol=1e-4)
    with_norm = wide(norm_weight=norm_w.cuda(), norm_eps=eps, out_float32=True)
    torch.testing.assert_close(with_norm.cpu(), normed_product.float(), atol=0.03 * float(normed_product.abs().max()) / 4,
                               rtol=0.02)
    torch.testing.assert_close(with_norm, narrow(norm_weight=norm_w.cuda(), norm_eps=eps, out_float32=True),
                               atol=1e-3 * float(normed_product.abs().max()), rtol=1e-3)
    half = normed_product.float().view(m, n // 16, 2, 8)
    expected = torch.nn.functional.silu(half[:, :, 0]) * half[:, :, 1]
    close(wide(norm_weight=norm_w.cuda(), norm_eps=eps, silu_pairs=True), expected.reshape(m, n // 2), torch.bfloat16,
          scale=max(2.0, float(expected.abs().max()) / 2))
    buffer = residual.cuda().clone()
    ops().gemm_small_m(a.cuda(), w.cuda(), residual=buffer, out=buffer, rows_per_block=32)
    close(buffer, (product + residual.double()).float(), torch.bfloat16, scale=scale)
    alone = ops().gemm_small_m(a[-1:].cuda().contiguous(), w.cuda(), out_float32=True, rows_per_block=32)
    assert torch.equal(alone.cpu()[0], exact.cpu()[-1])
    # left to itself the face takes this form from 148 blocks of 32 features on
    chosen = ops().gemm_small_m(a.cuda(), w.cuda(), out_float32=True)
    assert torch.equal(chosen, exact if n // 32 >= tuning.SMALL_M_WIDE_MIN_BLOCKS else narrow(out_float32=True))
    with pytest.raises(Exception, match="32"):
        ops().gemm_small_m(a.cuda(), w[:n - 16].contiguous().cuda(), rows_per_block=32)


@pytest.mark.parametrize("m,n,k", [(17, 8, 8), (128, 256, 64), (100, 264, 200), (300, 520, 1000), (2048, 1024, 4096)])
def test_gemm_tensor_memory(m, n, k):
    """The tcgen05/TMA kernel: plain, with bias and residual, in place, at sizes that are no multiple of a tile."""
    from qwen_inference_lab_b200.kernels import gemm_tc
    torch.manual_seed(11)
    a = torch.randn(m, k).to(torch.bfloat16)
    w = (torch.randn(n, k) * 0.1).to(torch.bfloat16)
    bias = (torch.randn(n) * 0.1).to(torch.bfloat16)
    residual = torch.randn(m, n).to(torch.bfloat16)
    product = a.double() @ w.double().t()
    scale = float(product.abs().max()) / 2
    close(gemm_tc.gemm_tc(a.cuda(), w.cuda()), product.float(), torch.bfloat16, scale=scale)
    close(gemm_tc.gemm_tc(a.cuda(), w.cuda(), bias=bias.cuda(), residual=residual.cuda()),
          (product + bias.double() + residual.double()).float(), torch.bfloat16, scale=scale)
    buffer = residual.cuda().clone()
    gemm_tc.gemm_tc(a.cuda(), w.cuda(), residual=buffer, out=buffer)
    close(buffer, (product + residual.double()).float(), torch.bfloat16, scale=scale)
    torch.cuda.synchronize()
    gemm_tc.check()


@pytest.mark.parametrize("m,inner,k", [(17, 8, 16), (130, 200, 96), (512, 1024, 512)])
def test_gemm_tensor_memory_with_gate_epilogue(m, inner, k):
    from qwen_inference_lab_b200.kernels import gemm_tc
    torch.manual_seed(12)
    a = torch.randn(m, k).to(torch.bfloat16)
    gate_w = (torch.randn(inner, k) * 0.2).to(torch.bfloat16)
    up_w = (torch.randn(inner, k) * 0.2).to(torch.bfloat16)
    gate = (a.float() @ gate_w.float().t()).to(torch.bfloat16)
    up = (a.float() @ up_w.float().t()).to(torch.bfloat16)
    expected = torch.nn.functional.silu(gate) * up
    paired = torch.cat([gate_w, up_w]).view(2, inner // 8, 8, k).transpose(0, 1).reshape(2 * inner, k).contiguous()
    fused = gemm_tc.gemm_tc(a.cuda(), paired.cuda(), silu_pairs=True)
    assert fused.shape == (m, inner)
    # gate, silu(gate) and the product each round to bfloat16: an element may sit two roundings from the
    # reference's, so the absolute term scales with the largest value
    close(fused, expected, torch.bfloat16, scale=max(2.0, float(expected.abs().max()) / 2))
    # the same rows through the decode kernel's epilogue give the same activations
    if m <= 16:
        assert torch.equal(ops().gemm_small_m(a.cuda(), paired.cuda(), silu_pairs=True), fused)
    torch.cuda.synchronize()
    gemm_tc.check()


@pytest.mark.parametrize("m,k,n_q,n_kv,page,bias,norms,rope", [
    (100, 136, 3, 1, 8, True, True, True),       # the one-block kernel, an odd number of heads
    (300, 256, 4, 2, 16, False, True, True),     # pairs of SMs; the last tile of tokens is partly empty
    (700, 520, 6, 2, 64, True, False, True),
    (260, 64, 2, 0, 16, False, True, False),     # a layer without keys and values of its own, no rotation
])
def test_gemm_tensor_memory_with_the_qkv_tail(m, k, n_q, n_kv, page, bias, norms, rope):
    """Projection, per-head norm, rotation and the write into shuffled pages in one kernel, against the same
    steps as separate kernels (product, then the norm/rotation/store kernel) and against plain float32."""
    from qwen_inference_lab_b200.kernels import gemm_tc
    from qwen_inference_lab_b200.parts.rotary import rotary_table
    torch.manual_seed(15)
    d, eps = 128, 1e-5
    heads = n_q + 2 * n_kv
    a = torch.randn(m, k).to(torch.bfloat16).cuda()
    w = (torch.randn(heads * d, k) * 0.1).to(torch.bfloat16).cuda()
    b = (torch.randn(heads * d) * 0.5).to(torch.bfloat16).cuda() if bias else None
    q_norm = (1 + 0.3 * torch.randn(d)).to(torch.bfloat16).cuda() if norms else None
    k_norm = (1 + 0.3 * torch.randn(d)).to(torch.bfloat16).cuda() if norms else None
    table = rotary_table(d, 10000.0, 2048, torch.bfloat16).cuda() if rope else None
    # two requests: the first fills positions 37.. of block-table row 1, the second 0.. of row 0
    first = m * 2 // 3
    positions = torch.cat([torch.arange(37, 37 + first), torch.arange(0, m - first)]).to(torch.int32).cuda()
    token_row = torch.cat([torch.full((first,), 1), torch.full((m - first,), 0)]).to(torch.int32).cuda()
    pages_per_request = (37 + first + page - 1) // page + 1
    num_pages = 2 * pages_per_request + 3
    block_table = torch.randperm(num_pages)[:2 * pages_per_request].view(2, pages_per_request).to(torch.int32).cuda()
    def run(fused):
        q = torch.full((m, n_q * d), float("nan"), dtype=torch.bfloat16).cuda()
        pages = torch.full((num_pages, 2, max(n_kv, 1), page, d), float("nan"), dtype=torch.bfloat16).cuda()
        if fused:
            gemm_tc.gemm_tc_qkv(a, w, b, q, pages if n_kv else None, table, q_norm, k_norm, eps, positions, token_row,
                                block_table, n_q, n_kv, page)
        else:
            qkv = gemm_tc.gemm_tc(a, w, bias=b)
            ops().qk_norm_rope_store(qkv, q, pages, q_norm, k_norm, eps, table, d if rope else 0, positions, token_row,
                                     block_table, n_q, n_kv, d, page)
        torch.cuda.synchronize()
        gemm_tc.check()
        return q, pages
    q_fused, pages_fused = run(True)
    q_split, pages_split = run(False)
    assert not torch.isnan(q_fused).any()
    # the same slots written, nothing else touched
    assert torch.equal(torch.isnan(pages_fused), torch.isnan(pages_split))
    # the two differ only where a normalising factor differs in its last bit and a value sits on a rounding edge
    scale = 4.0
    close(q_fused, q_split, torch.bfloat16, scale=scale)
    close(torch.nan_to_num(pages_fused), torch.nan_to_num(pages_split), torch.bfloat16, scale=scale)
    assert (q_fused != q_split).float().mean() < 0.02
    # and against plain float32 arithmetic on the bfloat16-rounded product
    qkv = (a.float() @ w.float().t() + (b.float() if bias else 0)).to(torch.bfloat16).float().view(m, heads, d).cpu()
    def norm_rotate(x, weight):
        if weight is not None:
            x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.float().cpu()
        if rope:
            cs = table.cpu()[positions.cpu().long()]
            c, s_ = cs[:, None, :d // 2], cs[:, None, d // 2:]
            lo, hi = x[..., :d // 2], x[..., d // 2:]
            x = torch.cat([lo * c - hi * s_, lo * s_ + hi * c], dim=-1)
        return x
    close(q_fused.view(m, n_q, d), norm_rotate(qkv[:, :n_q], q_norm), torch.bfloat16, scale=scale)
    if n_kv:
        keys = norm_rotate(qkv[:, n_q:n_q + n_kv], k_norm)
        for token in (0, first - 1, first, m - 1):
            pos, row = int(positions[token]), int(token_row[token])
            page_id = int(block_table[row, pos // page])
            close(pages_fused[page_id, 0, :, pos % page], keys[token], torch.bfloat16, scale=scale)
            close(pages_fused[page_id, 1, :, pos % page], qkv[token, n_q + n_kv:], torch.bfloat16, scale=scale)


TENSOR_MEMORY_ATTENTION_CASES = [
    # n_q, n_kv, lengths, chunk starts (chunk lengths are multiples of 128), page
    (1, 1, [128], [0], 16),
    (4, 2, [384, 200], [128, 72], 16),
    (8, 2, [1024, 133], [0, 5], 8),
    (4, 4, [700], [60], 64),
    (6, 1, [2100, 300], [1972, 44], 32),
    (32, 8, [2048], [0], 16),
]


@pytest.mark.parametrize("case", TENSOR_MEMORY_ATTENTION_CASES,
                         ids=[f"case{i}" for i in range(len(TENSOR_MEMORY_ATTENTION_CASES))])
def test_attention_tensor_memory(case):
    """The tcgen05 kernel on whole 128-token tiles over poisoned, shuffled pages, at positions that are no
    multiple of anything, against the plain float32 attention."""
    from qwen_inference_lab_b200.kernels import attention_tc
    n_q, n_kv, lengths, starts, page = case
    d = 128
    q, pool, table, meta, expected = attention_case(n_q, n_kv, d, lengths, starts, torch.bfloat16, page, seed=13)
    info = []
    for start, length, pos0, row in zip(meta["seg_start"], meta["seg_len"], meta["seg_pos0"], meta["seg_row"]):
        assert length % 128 == 0
        for off in range(0, length, 128):
            info += [start + off, pos0 + off, 128, row]
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16).cuda()
    attention_tc.prefill(q.cuda(), pool.cuda(), out, torch.tensor(info, dtype=torch.int32).cuda(), len(info) // 4,
                         table.cuda(), n_q, n_kv, page, d ** -0.5)
    torch.cuda.synchronize()
    attention_tc.check()
    close(out, expected, torch.bfloat16, scale=2)


def test_attention_tensor_memory_far_key_and_big_scores():
    """One key far back dominates (its value is large), and scores are large enough that the running maximum
    must move by more than 2^8 between tiles: the lazy rescale of the accumulator has to happen and be right."""
    from qwen_inference_lab_b200.kernels import attention_tc
    n_q, n_kv, d, page = 4, 2, 128, 16
    q, pool, table, meta, expected = attention_case(n_q, n_kv, d, [1300, 256], [1044, 0], torch.bfloat16, page, seed=14,
                                                    spike=(0, 700))
    assert expected[:256].abs().mean() > 10
    info = []
    for start, length, pos0, row in zip(meta["seg_start"], meta["seg_len"], meta["seg_pos0"], meta["seg_row"]):
        for off in range(0, length, 128):
            info += [start + off, pos0 + off, 128, row]
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16).cuda()
    attention_tc.prefill(q.cuda(), pool.cuda(), out, torch.tensor(info, dtype=torch.int32).cuda(), len(info) // 4,
                         table.cuda(), n_q, n_kv, page, d ** -0.5)
    torch.cuda.synchronize()
    attention_tc.check()
    close(out, expected, torch.bfloat16, scale=25)
