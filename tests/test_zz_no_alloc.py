"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some programs that embed the kernels may not allocate device memory at all: they gave the whole
GPU to a pool of their own, or they run inside someone else's CUDA context with only a stream to
launch on.  For them ``erb_attention_decode_static`` keeps the split-KV partial results in an
array built into the library.  This test calls it twice in a row with different inputs (the
array is shared and keeps the previous call's contents, so a second call is the interesting
one) and checks both results against the ordinary entry point that takes caller-provided
scratch.  It also checks that a call too large for the built-in array is refused with a message
instead of being launched.  The file name sorts last on purpose: if this test fails, a run that
stops at the first failure has already seen every other test.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_ARGS = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
               c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]


def _case(seed, n_seqs, nq, nkv, d, ps, ctx_lens, dtype):
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-c // ps) for c in ctx_lens]
    n_pages = sum(pages_per) + 2
    kp = torch.randn((n_pages, nkv, ps, d), generator=g).to(dtype).cuda()
    vp = torch.randn((n_pages, nkv, ps, d), generator=g).to(dtype).cuda()
    perm = torch.randperm(n_pages, generator=g).tolist()
    tables = torch.zeros((n_seqs, max(pages_per)), dtype=torch.int32)
    for s, n in enumerate(pages_per):
        tables[s, :n] = torch.tensor([perm.pop() for _ in range(n)], dtype=torch.int32)
    q = torch.randn((n_seqs, nq * d), generator=g).to(dtype).cuda()
    pos = torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32).cuda()
    return q, kp, vp, tables.cuda(), pos


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_entry_point_matches_the_ordinary_one(dtype):
    from edgerag_b200.ops import kernels, native

    lib = native.load("attention", "bfloat16" if dtype == torch.bfloat16 else "float32")
    fn = lib.erb_attention_decode_static
    fn.argtypes, fn.restype = STATIC_ARGS, c_int
    lib.erb_attention_decode_static_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.erb_attention_decode_static_floats.restype = c_longlong
    limit = 1 << 20
    stream = torch.cuda.current_stream().cuda_stream

    nq, nkv, d, ps, split = 8, 2, 64, 16, 128
    # two calls in a row; the second has fewer sequences and other lengths, so it reads scratch
    # entries that the first call left non-zero unless it writes them itself
    for seed, ctx_lens in ((1, [700, 129, 1, 333, 64]), (2, [90, 515, 256])):
        n = len(ctx_lens)
        q, kp, vp, tables, pos = _case(seed, n, nq, nkv, d, ps, ctx_lens, dtype)
        tok = torch.arange(n, dtype=torch.int32).cuda()
        max_splits = max((c - 1) // split + 1 for c in ctx_lens)
        assert lib.erb_attention_decode_static_floats(n, nq, d, max_splits) <= limit
        out_static = torch.full((n, nq * d), float("nan"), dtype=dtype, device="cuda")
        rc = fn(q.data_ptr(), q.stride(0), kp.data_ptr(), vp.data_ptr(), tables.data_ptr(), tables.shape[1],
                tok.data_ptr(), pos.data_ptr(), out_static.data_ptr(), out_static.stride(0), max_splits, n, nq, nkv,
                d, ps, 0, split, d ** -0.5, stream)
        assert rc == 0, lib.erb_last_error().decode()
        acc_n, ml_n = kernels.decode_scratch_floats(n, nq, d, max_splits)
        out_ref = torch.full_like(out_static, float("nan"))
        kernels.attention_decode(q, kp, vp, tables, tok, pos, out_ref, nq, d ** -0.5,
                                 torch.empty(acc_n, device="cuda"), torch.empty(ml_n, device="cuda"), max_splits,
                                 split_keys=split)
        torch.cuda.synchronize()
        assert torch.isfinite(out_static.float()).all()
        tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(out_static.float(), out_ref.float(), **tol)
        assert torch.equal(out_static, out_ref)        # same kernels, same split boundaries

    # a call that needs more than the built-in array is refused before anything is launched
    n_big, splits_big = 64, 64
    assert lib.erb_attention_decode_static_floats(n_big, 32, 64, splits_big) > limit
    rc = fn(q.data_ptr(), q.stride(0), kp.data_ptr(), vp.data_ptr(), tables.data_ptr(), tables.shape[1],
            tok.data_ptr(), pos.data_ptr(), out_static.data_ptr(), out_static.stride(0), splits_big, n_big, 32, 32,
            64, ps, 0, split, 0.125, stream)
    assert rc != 0 and "built-in array holds" in lib.erb_last_error().decode()
    torch.cuda.synchronize()
