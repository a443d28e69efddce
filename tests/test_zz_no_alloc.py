"""The decode-attention entry point that allocates nothing, called through its exported
C symbol the way a foreign caller would, against the ordinary entry point.

Such callers hold device pointers but may not allocate (a stream capture in progress,
a fixed-memory real-time loop, buffers owned by another runtime's allocator); the entry
point keeps its scratch in an array inside the library.  This file sorts last so that a
run which stops at the first failure has already run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_FLOATS = 2 * 1024 * 1024


def _lib():
    from skyla_kernel_b200.kernels import build
    lib = build.load("attention_mma")
    f = lib.skyla_attention_decode_no_alloc
    f.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                  c_int, c_int, c_void_p, c_float, c_int, c_int, c_void_p]
    f.restype = c_int
    return lib, f


def _problem(B, nq, nkv, hd, lens, seed):
    g = torch.Generator().manual_seed(seed)
    width = max(-(-l // 64) for l in lens)
    n_pages = B * width + 2
    k_pool = torch.randn(n_pages, nkv, 64, hd, generator=g).to(torch.bfloat16).to(DEV)
    v_pool = torch.randn(n_pages, nkv, 64, hd, generator=g).to(torch.bfloat16).to(DEV)
    pages = torch.randperm(n_pages, generator=g)[: B * width].to(torch.int32).view(B, width).contiguous().to(DEV)
    q = torch.randn(B, nq * hd, generator=g).to(torch.bfloat16).to(DEV)
    tok_pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    return q, k_pool, v_pool, pages, tok_pos, width


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from skyla_kernel_b200.kernels import ops
    lib, f = _lib()
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different problems in a row: the second must not be disturbed by what the first left in the array
    # (the third looks back over a window only; the fourth has more (sequence, head) pairs than the entry
    # point has counters, so the pieces that different blocks read are merged by the second kernel)
    for call, (B, nq, nkv, hd, lens, n_blocks, window) in enumerate([
            (5, 8, 2, 128, [1, 64, 65, 300, 777], 9, 0),
            (3, 6, 1, 32, [500, 17, 129], 7, 0),
            (4, 4, 2, 64, [700, 90, 257, 64], 24, 130),
            (700, 8, 8, 16, [1 + (37 * i) % 190 for i in range(700)], 1000, 0)]):
        q, k_pool, v_pool, pages, tok_pos, width = _problem(B, nq, nkv, hd, lens, 90 + call)
        scale = 1.0 / math.sqrt(hd)
        want = torch.empty(B, nq * hd, dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(ops.attention_decode_scratch(B, nq, nkv, hd, n_blocks), dtype=torch.float32, device=DEV)
        ops.attention_decode(q, want, scratch, nq, nkv, hd, k_pool, v_pool, pages, 64, tok_pos, scale, window, n_blocks)
        got = torch.full_like(want, float("nan"))
        args = (q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), B, nq, nkv, hd, k_pool.data_ptr(),
                v_pool.data_ptr(), pages.data_ptr(), width, 64, tok_pos.data_ptr(), scale, window, n_blocks, stream)
        # one warm call: the first call on a device looks up the array's address, and the driver loads a
        # kernel's code when it is first launched; memory is compared around the call after it
        assert f(*args) == 0, lib.skyla_error_message().decode()
        got.fill_(float("nan"))
        torch.cuda.synchronize()
        # the driver's own count of free memory sees every allocation on the device, whoever makes it
        before, before_torch = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        rc = f(*args)
        assert rc == 0, lib.skyla_error_message().decode()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == before and torch.cuda.memory_allocated() == before_torch
        # the same kernels on the same inputs: the same bits; the suite's bf16 tolerance is the stated bound
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        if B * nkv <= 4096:  # merged inside the kernel on both sides: the same arithmetic
            assert torch.equal(got, want)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib, f = _lib()
    B, nq, nkv, hd = 256, 64, 8, 128
    n_blocks = 8
    assert (n_blocks + B * nkv) * (nq // nkv) * (hd + 2) > SCRATCH_FLOATS  # a partial result per (slot, head)
    rc = f(None, 0, None, 0, B, nq, nkv, hd, None, None, None, 0, 64, None, 1.0, 0, n_blocks, None)
    assert rc != 0
    msg = lib.skyla_error_message().decode()
    assert "built-in array holds" in msg and str(SCRATCH_FLOATS) in msg
    rc = f(None, 0, None, 0, 2, 8, 2, 64, None, None, None, 0, 64, None, 1.0, 0, 1025, None)  # more blocks than plan rows
    assert rc != 0 and "built-in plan holds" in lib.skyla_error_message().decode()
