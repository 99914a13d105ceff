"""The attention entry point that allocates nothing, called through its exported C symbol.

Some users of the library may not allocate device memory once they are running (a host
program whose own pool owns all of it, or a loop that must not risk the device-wide stall
an allocation can cause).  ``qil_attn_decode_noalloc`` serves them from a fixed scratch
array inside the library.  Here it is called twice in a row, on different inputs, and each
result is compared with the regular entry point's, which takes scratch from the caller.
Collected last, so a run that stops at the first failure has already run everything else.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

HEAD_DIM = 64


def load_library():
    from qwen_inference_lab_b200.kernels import build
    lib = build.load(f"qil_attn_noalloc_d{HEAD_DIM}", ["attention_decode_noalloc.cu"], {"QIL_HEAD_DIM": HEAD_DIM},
                     depends=["attention_mma.cu", "attention_decode_noalloc.h"])
    lib.qil_attn_decode_noalloc.restype = c_int
    lib.qil_attn_decode_noalloc_max_floats.restype = ctypes.c_longlong
    return lib


def decode_case(lengths, n_q, n_kv, page, seed, span_len=256):
    """The last token of each request attends over its paged history (built as in the kernel tests)."""
    from tests.test_kernels_gpu import attention_case
    starts = [n - 1 for n in lengths]
    q, pool, table, meta, expected = attention_case(n_q, n_kv, HEAD_DIM, lengths, starts, torch.bfloat16, page, seed)
    info = [v for token, (pos, row) in enumerate(zip(meta["seg_pos0"], meta["seg_row"])) for v in (token, pos, row, 0)]
    return dict(q=q.cuda(), pool=pool.cuda(), table=table.cuda(), expected=expected, n_q=n_q, n_kv=n_kv, page=page,
                decode_info=torch.tensor(info, dtype=torch.int32).cuda(), span_len=span_len,
                n_spans=(max(lengths) + span_len - 1) // span_len)


def regular(case):
    from qwen_inference_lab_b200.kernels import attention_mma
    n = case["q"].shape[0]
    out = torch.full_like(case["q"], float("nan"))
    slots = n * case["n_q"] * case["n_spans"]
    part_o = torch.empty(slots * HEAD_DIM, dtype=torch.float32, device="cuda")
    part_ml = torch.empty(slots * 2, dtype=torch.float32, device="cuda")
    attention_mma.decode(case["q"], case["pool"], out, case["decode_info"], n, part_o, part_ml, case["n_spans"],
                         case["span_len"], case["table"], case["n_q"], case["n_kv"], HEAD_DIM, case["page"], 0,
                         HEAD_DIM ** -0.5)
    return out


def no_alloc(lib, case, n_spans=None):
    n = case["q"].shape[0]
    out = torch.full_like(case["q"], float("nan"))
    ptr = lambda t: c_void_p(t.data_ptr())
    code = lib.qil_attn_decode_noalloc(
        ptr(case["q"]), ptr(case["pool"]), ptr(out), ptr(case["decode_info"]), c_int(n),
        c_int(n_spans or case["n_spans"]), c_int(case["span_len"]), ptr(case["table"]),
        c_int(case["table"].shape[1]), c_int(case["n_q"]), c_int(case["n_kv"]), c_int(case["page"]),
        c_int(case["pool"].shape[0]), c_int(0), c_float(HEAD_DIM ** -0.5),
        c_void_p(torch.cuda.current_stream().cuda_stream))
    return code, out


def test_no_alloc_entry_point_matches_the_regular_one_twice_in_a_row():
    lib = load_library()
    assert lib.qil_attn_decode_noalloc_max_floats() == 4 * 1024 * 1024
    first = decode_case([700, 33, 257, 1], n_q=8, n_kv=2, page=16, seed=40)
    second = decode_case([90, 1300], n_q=4, n_kv=4, page=8, seed=41, span_len=512)   # other sizes: stale scratch must not matter
    allocated_before = torch.cuda.memory_allocated()
    for case in (first, second):
        want = regular(case)
        torch.cuda.synchronize()
        code, got = no_alloc(lib, case)
        torch.cuda.synchronize()
        assert code == 0, lib.qil_last_error().decode()
        # the tolerance of the kernel tests for one bfloat16 result (the two share their kernels, so they agree exactly)
        torch.testing.assert_close(got.float().cpu(), want.float().cpu(), atol=8e-3 * 2, rtol=8e-3)
        torch.testing.assert_close(got.float().cpu(), case["expected"].float(), atol=8e-3 * 2, rtol=8e-3)
    del want, got
    assert torch.cuda.memory_allocated() <= allocated_before + 4 * first["q"].numel() * 2 + 4096


def test_no_alloc_entry_point_refuses_what_its_array_cannot_hold():
    lib = load_library()
    case = decode_case([40, 50], n_q=8, n_kv=2, page=16, seed=42)
    code, out = no_alloc(lib, case, n_spans=200000)          # 2 * 8 * 200000 * 66 floats: far beyond 16 MiB
    torch.cuda.synchronize()
    assert code == -1
    message = lib.qil_last_error().decode()
    assert "floats of scratch" in message and "4194304" in message
    assert torch.isnan(out.float()).all()                    # nothing was launched


def test_the_two_entry_points_of_one_library_share_the_kernels_shared_memory_limit():
    """The regular entry point of the same library with a short span, then the no-allocation one with the longest
    span: the first must not have lowered the kernel's shared-memory limit under what the second needs."""
    lib = load_library()
    lib.qil_attn_decode.restype = c_int
    short = decode_case([100, 64], n_q=8, n_kv=2, page=16, seed=43, span_len=64)
    n = short["q"].shape[0]
    slots = n * short["n_q"] * short["n_spans"]
    part_o = torch.empty(slots * HEAD_DIM, dtype=torch.float32, device="cuda")
    part_ml = torch.empty(slots * 2, dtype=torch.float32, device="cuda")
    tickets = torch.zeros(n * short["n_q"], dtype=torch.int32, device="cuda")
    out = torch.full_like(short["q"], float("nan"))
    ptr = lambda t: c_void_p(t.data_ptr())
    code = lib.qil_attn_decode(
        ptr(short["q"]), ptr(short["pool"]), ptr(out), ptr(short["decode_info"]), c_int(n), ptr(part_o), ptr(part_ml),
        ptr(tickets), c_int(short["n_spans"]), c_int(short["span_len"]), ptr(short["table"]), c_int(short["table"].shape[1]),
        c_int(short["n_q"]), c_int(short["n_kv"]), c_int(short["page"]), c_int(short["pool"].shape[0]), c_int(0),
        c_float(HEAD_DIM ** -0.5), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert code == 0, lib.qil_last_error().decode()
    torch.testing.assert_close(out.float().cpu(), short["expected"].float(), atol=8e-3 * 2, rtol=8e-3)
    assert int(tickets.sum()) == 0               # the kernel leaves its counters at zero
    long = decode_case([2000, 5], n_q=8, n_kv=2, page=4, seed=44, span_len=2048)     # many more page ids per span
    code, got = no_alloc(lib, long)
    torch.cuda.synchronize()
    assert code == 0, lib.qil_last_error().decode()
    torch.testing.assert_close(got.float().cpu(), long["expected"].float(), atol=8e-3 * 2, rtol=8e-3)


def test_spans_that_do_not_reach_a_token_give_nan_not_a_shortened_softmax():
    lib = load_library()
    case = decode_case([300, 40], n_q=8, n_kv=2, page=16, seed=45, span_len=64)      # needs 5 spans
    code, out = no_alloc(lib, case, n_spans=3)                                        # 192 positions: the first token is beyond
    torch.cuda.synchronize()
    assert code == 0
    assert torch.isnan(out[0].float()).all()
    torch.testing.assert_close(out[1].float().cpu(), case["expected"][1].float(), atol=8e-3 * 2, rtol=8e-3)
