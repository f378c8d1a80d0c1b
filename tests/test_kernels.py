"""Each CUDA kernel alone against a plain float32 PyTorch computation of the same operation,
at sizes other than the tiny models' (odd widths, head sizes 48/80, shuffled pages, windows)."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.fixture(scope="module")
def k():
    from edgerag_b200.ops import kernels

    return kernels


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(shape, generator=g)).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_rows(k, dtype):
    table, embeds = rand((301, 72), dtype, 0), rand((4, 72), dtype, 1)
    ids = torch.tensor([5, 300, 0, 17, 9, 2], dtype=torch.int32).cuda()
    erow = torch.tensor([-1, -1, 2, -1, 0, 3], dtype=torch.int32).cuda()
    hidden = torch.full((6, 72), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.embed_rows(hidden, table, ids, status, embeds=embeds, embed_row=erow)
    want = table[ids.long()].float()
    want[2], want[4], want[5] = embeds[2].float(), embeds[0].float(), embeds[3].float()
    assert torch.equal(hidden, want) and int(status) == 0
    bad = torch.tensor([5, 301, 1, 1, 1, 1], dtype=torch.int32).cuda()
    k.embed_rows(hidden, table, bad, status)
    assert int(status) == 2 and torch.equal(hidden[1], torch.zeros(72, device="cuda"))   # flagged, nothing read


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 200, 2050])
def test_add_rmsnorm(k, dtype, width):
    hidden = rand((9, width), torch.float32, 2, 3.0)
    delta = rand((9, width), dtype, 3)
    weight = rand((width,), torch.float32, 4).add_(1.0)
    if dtype == torch.bfloat16:
        weight = weight.bfloat16().float()
    eps = 3e-4
    summed = hidden + delta.float()
    want = plain.rms_norm(summed.to(dtype), weight.to(dtype), eps)  # the reference casts before the weight
    if dtype == torch.bfloat16:   # the engine's residual stays float32: compare with statistics of the float32 sum
        x = summed * torch.rsqrt(summed.pow(2).mean(-1, keepdim=True) + eps)
        want = (weight * x.to(dtype).float()).to(dtype)
    out = torch.empty((9, width), dtype=dtype, device="cuda")
    h = hidden.clone()
    k.add_rmsnorm(h, weight, out, eps, delta=delta)
    torch.testing.assert_close(h, summed, atol=0, rtol=0)            # the residual sum is exact float32
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))
    # rows selected, nothing written back
    rows = torch.tensor([7, 0, 3], dtype=torch.int32).cuda()
    out2 = torch.empty((3, width), dtype=dtype, device="cuda")
    h2 = hidden.clone()
    k.add_rmsnorm(h2, weight, out2, eps, delta=delta, rows=rows, write_back=False)
    assert torch.equal(h2, hidden) and torch.equal(out2, out[rows.long()])
    # no delta
    k.add_rmsnorm(h2, weight, out, eps)
    ref = plain.rms_norm(hidden, weight, eps)
    torch.testing.assert_close(out.float(), ref, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,rows", [(72, 9), (1001, 5), (2048, 70), (2052, 33), (4096, 130)])
def test_add_rmsnorm_of_partial_sums(k, dtype, width, rows):
    """The update given as float32 partial sums [parts, rows, width] (widths for the one-pass, the two-pass and
    the scalar kernel): the same bits as the norm fed their sum, added in order and rounded to the element
    type once; rows selected; the plain residual add likewise."""
    parts = rand((5, rows, width), torch.float32, 31, 0.7)
    hidden = rand((rows, width), torch.float32, 32, 2.0)
    weight = rand((width,), torch.float32, 33).add_(1.0)
    total = parts[0].clone()
    for s in range(1, 5):
        total += parts[s]
    delta = total.to(dtype)
    want, h_want = torch.empty((rows, width), dtype=dtype, device="cuda"), hidden.clone()
    k.add_rmsnorm(h_want, weight, want, 2e-5, delta=delta)
    got, h_got = torch.full((rows, width), float("nan"), dtype=dtype, device="cuda"), hidden.clone()
    k.add_rmsnorm(h_got, weight, got, 2e-5, delta=parts)
    assert torch.equal(h_got, h_want) and torch.equal(got, want)
    picks = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32).cuda()
    some, h_same = torch.empty((3, width), dtype=dtype, device="cuda"), hidden.clone()
    k.add_rmsnorm(h_same, weight, some, 2e-5, delta=parts[:, :, :], rows=picks, write_back=False)
    assert torch.equal(h_same, hidden) and torch.equal(some, want[picks.long()])
    k.residual_add(h_same, parts, dtype)
    assert torch.equal(h_same, h_want)
    # a view of the parts with a stride between them (a scratch buffer made for more rows)
    roomy = torch.zeros((5, rows + 3, width), dtype=torch.float32, device="cuda")
    roomy[:, :rows] = parts
    with pytest.raises(k.KernelError):
        k.add_rmsnorm(hidden.clone(), weight, got, 2e-5, delta=roomy[:, :rows])       # parts must be contiguous


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [2048, 4096, 2052])
def test_add_rmsnorm_gives_a_row_the_same_bits_in_any_batch(k, dtype, width):
    """Wide rows are normed by more threads when the batch has few rows and by fewer, busier threads
    when it has many; a row's result is the same bits either way."""
    many = rand((200, width), torch.float32, 5, 2.0)
    delta = rand((200, width), dtype, 6)
    weight = rand((width,), torch.float32, 7).add_(1.0)
    out_many = torch.empty((200, width), dtype=dtype, device="cuda")
    h = many.clone()
    k.add_rmsnorm(h, weight, out_many, 1e-5, delta=delta)
    few, out_few = many[120:125].clone(), torch.empty((5, width), dtype=dtype, device="cuda")
    k.add_rmsnorm(few, weight, out_few, 1e-5, delta=delta[120:125].clone())
    assert torch.equal(out_few, out_many[120:125]) and torch.equal(few, h[120:125])


def test_product_in_parts_and_the_norm_that_adds_them(k):
    """17 to 64 bfloat16 rows against a weight of few rows: the slices of k as float32 partial results
    (against float64, N and K no multiples of a tile), a row's parts the same bits whatever the number
    of rows, and the residual add + norm that takes the parts against the same norm fed their sum."""
    for m, n, kk in ((17, 2048, 2048), (64, 2048, 8192), (40, 960, 2560), (33, 204, 1032), (64, 576, 1536), (24, 100, 136)):
        a, w = rand((m, kk), torch.bfloat16, 180 + m, 0.5), rand((n, kk), torch.bfloat16, 181 + m, 0.5)
        count = k.linear_parts_slices(w)
        # the dispatcher takes a product in parts from 17 rows on, and only against weights large enough to pay
        assert k.linear_parts_count(a, w) == (count if n * kk >= k.PARTS_MIN_WEIGHT_ELEMENTS else 0)
        assert count >= 1 and k.linear_parts_count(a[:16], w) == 0
        parts = torch.full((count, m, n), float("nan"), dtype=torch.float32, device="cuda")
        k.linear_parts(a, w, parts)
        total = parts[0].clone()
        for s in range(1, count):
            total += parts[s]
        torch.testing.assert_close(total.double(), a.double() @ w.double().T, atol=2e-3 * (kk ** 0.5) / 8, rtol=1e-4)
        if count > 1:       # the slices cover k once: each differs from the whole
            assert float((parts[0].double() - total.double()).abs().max()) > 1e-3
        fewer = torch.empty((count, 17, n), dtype=torch.float32, device="cuda")
        k.linear_parts(a[:17], w, fewer)
        assert torch.equal(fewer, parts[:, :17])
        # the norm: hidden += sum of the parts, in their order
        weight = rand((n,), torch.float32, 7).add_(1.0)
        hidden = rand((m, n), torch.float32, 8, 2.0)
        h_parts, h_sum = hidden.clone(), hidden.clone()
        out_parts = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        k.add_rmsnorm(h_parts, weight, out_parts, 1e-5, delta=parts)
        summed = hidden + total.bfloat16().float()      # the parts' sum is rounded once, like a stored product
        assert torch.equal(h_parts, summed)
        x = summed * torch.rsqrt(summed.pow(2).mean(-1, keepdim=True) + 1e-5)
        torch.testing.assert_close(out_parts.float(), (weight * x.bfloat16().float()).bfloat16().float(), **tol(torch.bfloat16))
        rows = torch.tensor([m - 1, 0, 5], dtype=torch.int32).cuda()
        picked = torch.empty((3, n), dtype=torch.bfloat16, device="cuda")
        k.add_rmsnorm(h_sum, weight, picked, 1e-5, delta=parts, rows=rows, write_back=False)
        assert torch.equal(h_sum, hidden) and torch.equal(picked, out_parts[rows.long()])
        k.residual_add(h_sum, parts, torch.bfloat16)
        assert torch.equal(h_sum, summed)
    # weights with many rows are not taken in parts (whole tiles of them fill the SMs)
    assert k.linear_parts_count(rand((40, 256), torch.bfloat16, 1), rand((49155, 256), torch.bfloat16, 2)) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rot", [48, 32])
def test_rope_cache_write(k, dtype, rot):
    nq, nkv, d, ps, n_pages = 6, 3, 48, 8, 7
    n = 11
    qkv = rand((n, (nq + 2 * nkv) * d), dtype, 5)
    positions = torch.tensor([0, 1, 2, 7000, 7001, 35, 36, 37, 38, 39, 8191], dtype=torch.int32).cuda()
    slots = torch.tensor([3, 4, 5, 55, 8, -1, 17, 16, 30, 31, 0], dtype=torch.int32).cuda()
    theta = 50000.0
    inv_freq = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.int64).float() / rot))).cuda()
    kp = torch.full((n_pages, nkv, ps, d), float("nan"), dtype=dtype, device="cuda")
    vp = torch.full_like(kp, float("nan"))
    before = qkv.clone()
    k.rope_cache_write(qkv, positions, inv_freq, nq, nkv, d, rot, slots=slots, k_pages=kp, v_pages=vp, page_size=ps)

    x = before.float().view(n, nq + 2 * nkv, d)
    cos, sin = plain.rope_tables(positions.cpu(), rot, theta)
    cos, sin = cos.cuda()[:, None], sin.cuda()[:, None]
    rotated = x[:, : nq + nkv].clone()
    part = rotated[..., :rot]
    rotated[..., :rot] = part * cos + plain.rotate_half(part) * sin
    got = qkv.float().view(n, nq + 2 * nkv, d)
    torch.testing.assert_close(got[:, :nq], rotated[:, :nq].to(dtype).float(), **tol(dtype))
    assert torch.equal(got[:, nq + nkv:], x[:, nq + nkv:])                       # v untouched
    written = torch.zeros(n_pages * ps, dtype=torch.bool)
    for t in range(n):
        s = int(slots[t])
        if s < 0:
            continue
        page, off = divmod(s, ps)
        written[s] = True
        torch.testing.assert_close(kp[page, :, off].float(), rotated[t, nq:].to(dtype).float(), **tol(dtype))
        assert torch.equal(vp[page, :, off].float(), x[t, nq + nkv:])
    untouched = kp.float().permute(0, 2, 1, 3).reshape(n_pages * ps, -1)[~written]
    assert torch.isnan(untouched).all()                                          # no stray write


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_and_residual_and_gather(k, dtype):
    for inter in (304, 300, 150):          # widths that take the 16-byte path, and ones that do not
        gu = rand((5, 2 * inter), dtype, 6, 2.0)
        out = torch.full((5, inter), float("nan"), dtype=dtype, device="cuda")
        k.swiglu(gu, out)
        want = torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()
        torch.testing.assert_close(out.float(), want, **tol(dtype))
    gu = rand((5, 2 * 300), dtype, 6, 2.0)
    out = torch.empty((5, 300), dtype=dtype, device="cuda")
    k.swiglu(gu, out)
    h = rand((5, 300), torch.float32, 7)
    h0 = h.clone()
    k.residual_add(h, out)
    assert torch.equal(h, h0 + out.float())
    rows = torch.tensor([4, 1], dtype=torch.int32).cuda()
    dst = torch.empty((2, 300), dtype=dtype, device="cuda")
    k.gather_cast(h, dst, rows)
    assert torch.equal(dst, h[rows.long()].to(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [1, 7, 16, 33, 64, 130])
def test_linear(k, dtype, m):
    n, kk = 133, 72
    a, w = rand((m, kk), dtype, 8), rand((n, kk), dtype, 9)
    want = a.double() @ w.double().T
    out32 = torch.empty((m, n), dtype=torch.float32, device="cuda")
    k.linear(a, w, out32)
    torch.testing.assert_close(out32.double(), want, atol=1e-4 if dtype == torch.float32 else 2e-3, rtol=1e-5)
    if dtype == torch.float32:
        # true 32-bit products: a TF32 product would be off by ~1e-3 relative here
        assert float((out32.double() - want).abs().max()) < 5e-5
    out = torch.empty((m, n), dtype=dtype, device="cuda")
    k.linear(a, w, out)
    torch.testing.assert_close(out.float(), want.float(), **(dict(atol=1e-4, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.15, rtol=2e-2)))
    # strided views (a slice of a wider buffer in, a slice out) and accumulation
    wide_in = torch.zeros((m, kk + 24), dtype=dtype, device="cuda")
    wide_in[:, 8: 8 + kk] = a
    wide_out = torch.zeros((m, n + 8), dtype=torch.float32, device="cuda")
    k.linear(wide_in[:, 8: 8 + kk], w, wide_out[:, :n])
    torch.testing.assert_close(wide_out[:, :n], out32, atol=1e-5, rtol=1e-5)
    assert float(wide_out[:, n:].abs().max()) == 0
    k.linear(a, w, out32, accumulate=True)
    torch.testing.assert_close(out32.double(), 2 * want, atol=2e-4 if dtype == torch.float32 else 4e-3, rtol=1e-5)


def test_linear_for_few_rows_streams_weights(k):
    """Few bfloat16 rows go through this package's own kernel (16 rows of w per block, any N, K a
    multiple of 8 but not of a pass); more rows, or float32, through the library."""
    for m, n, kk in ((8, 49155 // 7, 2048), (3, 50, 8), (16, 257, 1032), (5, 2048, 8192), (64, 100, 72), (29, 31, 264)):
        a, w = rand((m, kk), torch.bfloat16, 40 + m, 0.5), rand((n, kk), torch.bfloat16, 41 + m, 0.5)
        want = a.double() @ w.double().T
        out = torch.empty((m, n + 3), dtype=torch.float32, device="cuda")[:, :n]
        k.linear_few_rows(a, w, out)
        torch.testing.assert_close(out.double(), want, atol=2e-3 * (kk ** 0.5) / 8, rtol=1e-4)
        out16 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        k.linear_few_rows(a, w, out16)
        assert torch.equal(out16, out.bfloat16())          # same sums, rounded once
        before = dict(k.launch_counts)
        k.linear(a, w, out16)                                # the dispatcher picks by the number of rows
        own = m <= k.SKINNY_MAX_ROWS
        assert k.launch_counts["own"] == before["own"] + int(own)
        assert k.launch_counts["library"] == before["library"] + int(not own)


def test_gated_product_equals_product_then_gate(k):
    """The decode step's gate/up product with the gate in its epilogue gives, bit for bit, what the
    plain product into a [M, 2N] buffer followed by the gate kernel gives, and both follow the
    formula silu(x Wg^T) * (x Wu^T); N no multiple of the 8 gate rows a block takes, K no multiple of a pass."""
    for m, n, kk in ((1, 96, 64), (8, 8192 // 4, 2048), (5, 203, 1032), (16, 77, 264), (11, 1024, 4096), (17, 203, 1032),
                     (40, 2048, 2048), (64, 77, 264), (33, 1024, 4096)):
        a = rand((m, kk), torch.bfloat16, 70 + m, 0.5)
        w = rand((2 * n, kk), torch.bfloat16, 71 + m, 0.3)
        assert k.linear_glu_supported(a, w, 64) and k.linear_glu_supported(a, w) == (m <= 16)
        both = torch.empty((m, 2 * n), dtype=torch.bfloat16, device="cuda")
        k.linear_few_rows(a, w, both)
        two_steps = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        k.swiglu(both, two_steps)
        fused = torch.full((m, n + 5), float("nan"), dtype=torch.bfloat16, device="cuda")[:, :n]
        k.linear_glu(a, w, fused)
        assert torch.equal(fused, two_steps)
        g, u = (a.double() @ w.double().T).split(n, dim=1)
        want = torch.nn.functional.silu(g) * u
        torch.testing.assert_close(fused.double(), want, atol=0.02 * (kk ** 0.5) / 8, rtol=0.02)
    assert not k.linear_glu_supported(rand((65, 64), torch.bfloat16, 1), rand((32, 64), torch.bfloat16, 2))
    assert not k.linear_glu_supported(rand((4, 64), torch.float32, 1), rand((32, 64), torch.float32, 2))


def test_projection_with_rotation_and_cache_write_equals_the_three_steps(k):
    """The decode step's q/k/v product with the rotary encoding and the cache write in its epilogue
    leaves, bit for bit, the q columns and the cache pages that the product, then the rotation
    kernel leave; a token with a negative slot writes no key or value."""
    for m, nq, nkv, d, kk, ps in ((1, 4, 2, 16, 64, 4), (8, 32, 32, 64, 2048, 16), (5, 9, 3, 48, 264, 8), (16, 6, 1, 128, 1032, 16),
                                  (17, 9, 3, 48, 264, 8), (64, 32, 32, 64, 2048, 16), (37, 15, 5, 64, 960, 16)):
        width = (nq + 2 * nkv) * d
        a = rand((m, kk), torch.bfloat16, 80 + m, 0.5)
        w = rand((width, kk), torch.bfloat16, 81 + m, 0.3)
        inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))).cuda()
        positions = torch.tensor([3 + 977 * i for i in range(m)], dtype=torch.int32).cuda()
        n_pages = m + 2
        slots = torch.tensor([((i * 5 + 1) % n_pages) * ps + (i * 3) % ps for i in range(m)], dtype=torch.int32)
        if m > 2:
            slots[2] = -1
        slots = slots.cuda()
        assert k.linear_rope_store_supported(a, w, d, d, 64) and k.linear_rope_store_supported(a, w, d, d) == (m <= 16)
        results = []
        for fused in (False, True):
            kp = torch.full((n_pages, nkv, ps, d), 7.0, dtype=torch.bfloat16, device="cuda")
            vp = torch.full_like(kp, 7.0)
            qkv = torch.zeros((m, width), dtype=torch.bfloat16, device="cuda")
            if fused:
                k.linear_rope_store(a, w, qkv, positions, inv_freq, nq, nkv, d, slots, kp, vp, ps)
            else:
                k.linear_few_rows(a, w, qkv)
                k.rope_cache_write(qkv, positions, inv_freq, nq, nkv, d, d, slots=slots, k_pages=kp, v_pages=vp, page_size=ps)
            results.append((qkv[:, : nq * d].clone(), kp, vp))
        for two, one in zip(*results):
            assert torch.equal(two, one)
        assert float(results[1][1].float().sub(7.0).abs().sum()) > 0      # something was written
    assert not k.linear_rope_store_supported(rand((4, 64), torch.bfloat16, 1), rand((96, 64), torch.bfloat16, 2), 16, 8)


def test_tensor_core_products_for_few_rows(k):
    """The TMA + tcgen05 weight-streaming kernel for up to 64 rows: plain products against float64 (N and K
    no multiples of a tile, float and bfloat16 out), the gated and the rotating epilogues bit-equal to
    product-then-kernel, products split over k by a cluster, and a row's bits the same whatever the
    number of rows."""
    for m, n, kk in ((8, 6144, 2048), (1, 96, 64), (16, 257, 1032), (5, 2048, 8192), (64, 100, 72), (29, 311, 264),
                     (64, 2048, 2048), (33, 49155 // 7, 2048), (48, 16384, 2048)):
        a, w = rand((m, kk), torch.bfloat16, 140 + m, 0.5), rand((n, kk), torch.bfloat16, 141 + m, 0.5)
        want = a.double() @ w.double().T
        out = torch.full((m, n + 3), float("nan"), dtype=torch.float32, device="cuda")[:, :n]
        k.linear_tc(a, w, out)
        torch.testing.assert_close(out.double(), want, atol=2e-3 * (kk ** 0.5) / 8, rtol=1e-4)
        out16 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        k.linear_tc(a, w, out16)
        assert torch.equal(out16, out.bfloat16())          # same sums, rounded once
    for m, n, kk in ((1, 96, 64), (8, 2048, 2048), (5, 203, 1032), (17, 203, 1032), (64, 8192, 2048), (33, 1024, 4096)):
        a, w = rand((m, kk), torch.bfloat16, 150 + m, 0.5), rand((2 * n, kk), torch.bfloat16, 151 + m, 0.3)
        both = torch.empty((m, 2 * n), dtype=torch.bfloat16, device="cuda")
        k.linear_tc(a, w, both)
        two_steps = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        k.swiglu(both, two_steps)
        fused = torch.full((m, n + 5), float("nan"), dtype=torch.bfloat16, device="cuda")[:, :n]
        k.linear_tc_glu(a, w, fused)
        assert torch.equal(fused, two_steps)
    for m, nq, nkv, d, kk, ps in ((1, 4, 2, 32, 64, 4), (8, 32, 32, 64, 2048, 16), (5, 9, 3, 64, 264, 8), (16, 6, 1, 128, 1032, 16),
                                  (64, 32, 32, 64, 2048, 16), (37, 15, 5, 64, 960, 16)):
        width = (nq + 2 * nkv) * d
        a, w = rand((m, kk), torch.bfloat16, 160 + m, 0.5), rand((width, kk), torch.bfloat16, 161 + m, 0.3)
        inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))).cuda()
        positions = torch.tensor([3 + 977 * i for i in range(m)], dtype=torch.int32).cuda()
        n_pages = m + 2
        slots = torch.tensor([((i * 5 + 1) % n_pages) * ps + (i * 3) % ps for i in range(m)], dtype=torch.int32)
        if m > 2:
            slots[2] = -1
        slots = slots.cuda()
        results = []
        for fused in (False, True):
            kp = torch.full((n_pages, nkv, ps, d), 7.0, dtype=torch.bfloat16, device="cuda")
            vp = torch.full_like(kp, 7.0)
            qkv = torch.zeros((m, width), dtype=torch.bfloat16, device="cuda")
            if fused:
                k.linear_tc_rope_store(a, w, qkv, positions, inv_freq, nq, nkv, d, slots, kp, vp, ps)
            else:
                k.linear_tc(a, w, qkv)
                k.rope_cache_write(qkv, positions, inv_freq, nq, nkv, d, d, slots=slots, k_pages=kp, v_pages=vp, page_size=ps)
            results.append((qkv[:, : nq * d].clone(), kp, vp))
        for two, one in zip(*results):
            assert torch.equal(two, one)
    for n, kk in ((6144, 2048), (2048, 8192), (49155, 2048)):
        a, w = rand((64, kk), torch.bfloat16, 170, 0.5), rand((n, kk), torch.bfloat16, 171, 0.5)
        full = torch.empty((64, n), dtype=torch.float32, device="cuda")
        k.linear_tc(a, w, full)
        for m in (1, 8, 17, 40):
            part = torch.empty((m, n), dtype=torch.float32, device="cuda")
            k.linear_tc(a[:m], w, part)
            assert torch.equal(part, full[:m]), (n, kk, m)
    # the dispatcher: 17 to 64 rows of a product with many rows of w (an output head) take this kernel
    a, w = rand((40, 256), torch.bfloat16, 172, 0.5), rand((49155, 256), torch.bfloat16, 173, 0.5)
    out = torch.empty((40, 49155), dtype=torch.float32, device="cuda")
    before = dict(k.launch_counts)
    k.linear(a, w, out)
    assert k.launch_counts["own"] == before["own"] + 1 and k.launch_counts["library"] == before["library"]
    torch.testing.assert_close(out.double(), a.double() @ w.double().T, atol=2e-3, rtol=1e-4)


def test_few_rows_give_a_row_the_same_bits_in_any_batch(k):
    """The register-fed kernels (up to 16 rows): a row's sums do not depend on how many rows there are,
    whichever variant (8, 16 or twice 16 warps per tile of w) the sizes of w select."""
    for n, kk in ((6144, 2048), (2048, 2048), (2048, 8192), (49155 // 3, 2048), (960, 2560)):
        a, w = rand((16, kk), torch.bfloat16, 180, 0.5), rand((n, kk), torch.bfloat16, 181, 0.5)
        full = torch.empty((16, n), dtype=torch.float32, device="cuda")
        k.linear_few_rows(a, w, full)
        torch.testing.assert_close(full.double(), a.double() @ w.double().T, atol=2e-3 * (kk ** 0.5) / 8, rtol=1e-4)
        for m in (1, 5, 8, 9):
            part = torch.empty((m, n), dtype=torch.float32, device="cuda")
            k.linear_few_rows(a[:m], w, part)
            assert torch.equal(part, full[:m]), (n, kk, m)


# --- attention -------------------------------------------------------------------------------

def paged_case(dtype, seed, nq, nkv, d, ps, ctx_lens, q_lens, poison=True):
    """Random keys/values for several sequences scattered over shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    n_seqs = len(ctx_lens)
    pages_per = [-(-c // ps) for c in ctx_lens]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    kp = torch.full((n_pages, nkv, ps, d), float("nan") if poison else 0.0, dtype=dtype)
    vp = torch.full_like(kp, float("nan") if poison else 0.0)
    max_pages = max(pages_per)
    tables = torch.zeros((n_seqs, max_pages), dtype=torch.int32)
    ks, vs = [], []
    for s, c in enumerate(ctx_lens):
        mine = [perm.pop() for _ in range(pages_per[s])]
        tables[s, : len(mine)] = torch.tensor(mine, dtype=torch.int32)
        kk = torch.randn((c, nkv, d), generator=g).to(dtype)
        vv = torch.randn((c, nkv, d), generator=g).to(dtype)
        ks.append(kk)
        vs.append(vv)
        for p in range(c):
            kp[mine[p // ps], :, p % ps] = kk[p]
            vp[mine[p // ps], :, p % ps] = vv[p]
    n_tok = sum(q_lens)
    q = torch.randn((n_tok, nq * d), generator=g).to(dtype)
    seq_of, pos = [], []
    for s, (c, ql) in enumerate(zip(ctx_lens, q_lens)):
        seq_of += [s] * ql
        pos += list(range(c - ql, c))
    return dict(q=q, kp=kp, vp=vp, tables=tables, ks=ks, vs=vs,
                seq_of=torch.tensor(seq_of, dtype=torch.int32), pos=torch.tensor(pos, dtype=torch.int32))


def attention_reference(case, nq, nkv, d, scale, window=0):
    out = []
    r = nq // nkv
    for t in range(case["q"].shape[0]):
        s, p = int(case["seq_of"][t]), int(case["pos"][t])
        lo = max(0, p - window + 1) if window else 0
        kk = case["ks"][s][lo: p + 1].double().repeat_interleave(r, dim=1)     # (keys, nq, d)
        vv = case["vs"][s][lo: p + 1].double().repeat_interleave(r, dim=1)
        qq = case["q"][t].double().view(nq, d)
        scores = torch.einsum("hd,khd->hk", qq, kk) * scale
        probs = torch.softmax(scores, dim=-1)
        out.append(torch.einsum("hk,khd->hd", probs, vv).reshape(-1))
    return torch.stack(out).float()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,ps,window", [(6, 2, 80, 8, 0), (4, 4, 48, 16, 0), (3, 1, 16, 4, 21), (8, 2, 128, 32, 0)])
def test_attention_rows(k, dtype, nq, nkv, d, ps, window):
    ctx_lens, q_lens = [37, 150, 9, 64], [37, 21, 2, 1]
    case = paged_case(dtype, 10 + d, nq, nkv, d, ps, ctx_lens, q_lens)
    scale = d ** -0.5
    dev = {n: case[n].cuda() for n in ("q", "kp", "vp", "tables", "seq_of", "pos")}
    out = torch.full((dev["q"].shape[0], nq * d), float("nan"), dtype=dtype, device="cuda")
    k.attention_rows(dev["q"], dev["kp"], dev["vp"], dev["tables"], dev["seq_of"], dev["pos"], out, nq, scale, window=window)
    want = attention_reference(case, nq, nkv, d, scale, window)
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,ps,window,split", [(6, 2, 80, 8, 0, 64), (4, 4, 64, 16, 0, 512), (3, 1, 16, 4, 100, 32), (2, 1, 256, 16, 0, 128)])
def test_attention_decode(k, dtype, nq, nkv, d, ps, window, split):
    ctx_lens = [1, 63, 64, 65, 700, 129]
    q_lens = [1] * len(ctx_lens)
    case = paged_case(dtype, 20 + d, nq, nkv, d, ps, ctx_lens, q_lens)
    scale = d ** -0.5
    dev = {n: case[n].cuda() for n in ("q", "kp", "vp", "tables", "seq_of", "pos")}
    n = len(ctx_lens)
    max_splits = max((c - 1) // split - (max(0, c - window) if window else 0) // split + 1 for c in ctx_lens)
    acc_n, ml_n = k.decode_scratch_floats(n, nq, d, max_splits)
    part_acc = torch.full((acc_n,), float("nan"), device="cuda")
    part_ml = torch.full((ml_n,), float("nan"), device="cuda")
    out = torch.full((n, nq * d), float("nan"), dtype=dtype, device="cuda")
    token_of_seq = torch.arange(n, dtype=torch.int32).cuda()
    k.attention_decode(dev["q"], dev["kp"], dev["vp"], dev["tables"], token_of_seq, dev["pos"], out, nq, scale,
                       part_acc, part_ml, max_splits, window=window, split_keys=split)
    want = attention_reference(case, nq, nkv, d, scale, window)
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))
    # the row kernel gives the same answer for the same tokens
    out2 = torch.empty_like(out)
    k.attention_rows(dev["q"], dev["kp"], dev["vp"], dev["tables"], dev["seq_of"], dev["pos"], out2, nq, scale, window=window)
    torch.testing.assert_close(out2.float(), out.float(), **tol(dtype))


@pytest.mark.parametrize("nq,nkv,d,ps,split", [(4, 4, 64, 16, 512), (6, 2, 64, 4, 128), (8, 1, 128, 16, 512),
                                               (2, 2, 32, 64, 256), (5, 5, 64, 24, 512), (8, 8, 64, 16, 512),
                                               (16, 8, 64, 8, 512), (4, 4, 128, 16, 256), (15, 5, 64, 16, 512),
                                               (9, 3, 64, 16, 1024), (10, 10, 64, 16, 512), (6, 6, 64, 16, 256),
                                               (7, 7, 32, 16, 512), (3, 3, 128, 16, 2048), (4, 4, 64, 16, 2048)])
def test_attention_decode_bulk_copies(k, nq, nkv, d, ps, split):
    """The decode kernel that streams pages with bulk asynchronous copies: lengths around stage and
    split edges, grouped heads, head counts that the heads per block do not divide (a last group
    with fewer heads, or one block for 5 or 6 heads), page sizes that do and do not divide a stage,
    a single split (the kernel then writes the result itself), NaN in unwritten slots."""
    dtype = torch.bfloat16
    ctx_lens = [1, 63, 64, 65, 1300, 512, 513, 129]
    case = paged_case(dtype, 90 + d + ps, nq, nkv, d, ps, ctx_lens, [1] * len(ctx_lens))
    scale = d ** -0.5
    dev = {n: case[n].cuda() for n in ("q", "kp", "vp", "tables", "seq_of", "pos")}
    n = len(ctx_lens)
    max_splits = max((c - 1) // split + 1 for c in ctx_lens)
    acc_n, ml_n = k.decode_scratch_floats(n, nq, d, max_splits)
    part_acc = torch.full((acc_n,), float("nan"), device="cuda")
    part_ml = torch.full((ml_n,), float("nan"), device="cuda")
    out = torch.full((n, nq * d), float("nan"), dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tok = torch.arange(n, dtype=torch.int32).cuda()
    k.attention_decode_bulk(dev["q"], dev["kp"], dev["vp"], dev["tables"], tok, dev["pos"], out, nq, scale,
                            part_acc, part_ml, max_splits, status, split_keys=split)
    torch.cuda.synchronize()
    assert int(status) == 0
    want = attention_reference(case, nq, nkv, d, scale)
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("nq,nkv,d,ps,split,heads", [(8, 8, 64, 16, 64, 1), (8, 8, 64, 16, 64, 2), (8, 8, 64, 16, 128, 4),
                                                     (32, 32, 64, 16, 256, 2), (12, 6, 64, 8, 128, 4), (7, 7, 32, 16, 64, 2),
                                                     (5, 5, 128, 16, 256, 2), (32, 32, 64, 16, 512, 8), (3, 3, 64, 32, 64, 4)])
def test_attention_decode_bulk_heads_per_block(k, nq, nkv, d, ps, split, heads):
    """The bulk decode kernel with a given number of kv heads per block (fewer heads: more and shorter
    blocks for small batches), many short splits merged by the block that finishes last, head counts
    that the group does not divide; the counters are back at zero afterwards, and a second call on
    the same counters gives the same bits.  A group that the sizes do not allow is refused."""
    dtype = torch.bfloat16
    lib = k.native.load("attention_tc", None)
    if lib.erb_attention_decode_bulk_head_group(nkv, d, ps, split, heads) != heads:
        pytest.skip("these sizes do not allow this group")
    ctx_lens = [1, 63, 64, 65, 640, 513, 129, 1000]
    case = paged_case(dtype, 290 + d + ps + heads, nq, nkv, d, ps, ctx_lens, [1] * len(ctx_lens))
    scale = d ** -0.5
    dev = {n: case[n].cuda() for n in ("q", "kp", "vp", "tables", "seq_of", "pos")}
    n = len(ctx_lens)
    max_splits = max((c - 1) // split + 1 for c in ctx_lens)
    acc_n, ml_n = k.decode_scratch_floats(n, nq, d, max_splits)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tok = torch.arange(n, dtype=torch.int32).cuda()
    outs = []
    for _ in range(2):
        part_acc = torch.full((acc_n,), float("nan"), device="cuda")
        part_ml = torch.full((ml_n,), float("nan"), device="cuda")
        out = torch.full((n, nq * d), float("nan"), dtype=dtype, device="cuda")
        k.attention_decode_bulk(dev["q"], dev["kp"], dev["vp"], dev["tables"], tok, dev["pos"], out, nq, scale,
                                part_acc, part_ml, max_splits, status, split_keys=split, head_group=heads)
        torch.cuda.synchronize()
        assert int(status) == 0
        assert int(k.split_counters(out.device, 1).abs().sum()) == 0, "a counter was left standing"
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    want = attention_reference(case, nq, nkv, d, scale)
    torch.testing.assert_close(outs[0].float().cpu(), want, **tol(dtype))
    with pytest.raises(k.KernelError):
        k.attention_decode_bulk(dev["q"], dev["kp"], dev["vp"], dev["tables"], tok, dev["pos"], out, nq, scale,
                                part_acc, part_ml, max_splits, status, split_keys=split, head_group=3)


def test_decode_plan_is_a_function_of_the_batch_and_a_bound_on_the_context(k):
    """The plan (keys per split, heads per block) that a decode step takes: allowed by the kernel, at
    most 64 splits for the bound, more blocks for a small batch than the default grouping gives, the
    default for batches that fill the GPU anyway, nothing for the kernel that groups by itself."""
    lib = k.native.load("attention_tc", None)
    for n_seqs in (1, 2, 3, 8, 16, 64):
        for bound in (128, 1024, 8192):
            split, heads = k.choose_decode_plan(n_seqs, 32, bound, 16, 64)
            assert split % 16 == 0 and -(-bound // split) <= 64
            assert heads == 0 or lib.erb_attention_decode_bulk_head_group(32, 64, 16, split, heads) == heads
    split, heads = k.choose_decode_plan(1, 32, 1024, 16, 64)
    assert heads == 2 and 1 * 16 * -(-1024 // split) >= 128
    assert k.choose_decode_plan(64, 32, 8192, 16, 64)[1] == 0
    assert k.choose_decode_plan(8, 5, 8192, 16, 64, grouped=True) == (k.choose_decode_split(8, 5, 8192, 16, 64), 0)


@pytest.mark.parametrize("nq,nkv,ps,split", [(15, 5, 16, 512), (9, 3, 16, 1024), (6, 2, 8, 128), (8, 1, 16, 256),
                                             (16, 8, 32, 512), (20, 10, 16, 2048), (24, 3, 64, 512), (4, 2, 128, 256)])
def test_attention_decode_for_grouped_heads_on_tensor_cores(k, nq, nkv, ps, split):
    """Several query heads per kv head as the rows of one tensor-core tile, pages brought in by TMA
    tensor copies: lengths around stage, page and split edges, head groups with a smaller last
    group, NaN in unwritten slots (masked keys must not reach the product)."""
    dtype, d = torch.bfloat16, 64
    assert k.decode_gqa_supported(dtype, d, 0, nq, nkv, ps, split)
    ctx_lens = [1, 15, 16, 17, 63, 64, 65, 1300, 512, 513, 129, 2048]
    case = paged_case(dtype, 190 + nq + ps, nq, nkv, d, ps, ctx_lens, [1] * len(ctx_lens))
    scale = d ** -0.5
    dev = {n: case[n].cuda() for n in ("q", "kp", "vp", "tables", "seq_of", "pos")}
    n = len(ctx_lens)
    max_splits = max((c - 1) // split + 1 for c in ctx_lens)
    acc_n, ml_n = k.decode_scratch_floats(n, nq, d, max_splits)
    part_acc = torch.full((acc_n,), float("nan"), device="cuda")
    part_ml = torch.full((ml_n,), float("nan"), device="cuda")
    out = torch.full((n, nq * d), float("nan"), dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tok = torch.arange(n, dtype=torch.int32).cuda()
    k.attention_decode_gqa(dev["q"], dev["kp"], dev["vp"], dev["tables"], tok, dev["pos"], out, nq, scale,
                           part_acc, part_ml, max_splits, status, split_keys=split)
    torch.cuda.synchronize()
    assert int(status) == 0
    want = attention_reference(case, nq, nkv, d, scale)
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))
    assert not k.decode_gqa_supported(dtype, d, 0, 4, 4, ps, split)          # one query head per kv head: the other kernel
    assert not k.decode_gqa_supported(dtype, 128, 0, nq, nkv, ps, split)


@pytest.mark.parametrize("which", ["general", "bulk"])
def test_attention_decode_merges_no_more_splits_than_it_was_sized_for(k, which):
    """A caller that understates ``max_splits`` gets a wrong answer (only the first splits are merged),
    but the merge must not walk past the scratch of its own (sequence, head): the floats behind it are
    NaN here and would show in the result."""
    dtype, nq, nkv, d, ps, split = torch.bfloat16, 4, 4, 64, 16, 128
    ctx_lens = [700, 300]                       # 6 and 3 splits
    case = paged_case(dtype, 55, nq, nkv, d, ps, ctx_lens, [1, 1])
    dev = {n: case[n].cuda() for n in ("q", "kp", "vp", "tables", "seq_of", "pos")}
    understated = 2
    acc_n, ml_n = k.decode_scratch_floats(2, nq, d, understated)
    part_acc = torch.full((acc_n + 4096,), float("nan"), device="cuda")
    part_ml = torch.full((ml_n + 4096,), float("nan"), device="cuda")
    out = torch.full((2, nq * d), float("nan"), dtype=dtype, device="cuda")
    tok = torch.arange(2, dtype=torch.int32).cuda()
    if which == "general":
        k.attention_decode(dev["q"], dev["kp"], dev["vp"], dev["tables"], tok, dev["pos"], out, nq, d ** -0.5,
                           part_acc, part_ml, understated, split_keys=split)
    else:
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        k.attention_decode_bulk(dev["q"], dev["kp"], dev["vp"], dev["tables"], tok, dev["pos"], out, nq, d ** -0.5,
                                part_acc, part_ml, understated, status, split_keys=split)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert torch.isnan(part_acc[acc_n:]).all() and torch.isnan(part_ml[ml_n:]).all()
    # what it merged is attention over the first two splits of each sequence
    short = dict(case, pos=torch.tensor([2 * split - 1, 2 * split - 1], dtype=torch.int32))
    want = attention_reference(short, nq, nkv, d, d ** -0.5)
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(k, dtype):
    """One key far back, in the first page, gets a score that stands out: the output must be its value.
    A kernel that drops a page, mis-walks the block table or masks too much cannot pass."""
    nq, nkv, d, ps = 4, 2, 64, 16
    ctx = 900
    case = paged_case(dtype, 77, nq, nkv, d, ps, [ctx, ctx], [1, 5])
    far = {0: 3, 1: 17}
    for s in (0, 1):
        page, off = int(case["tables"][s, far[s] // ps]), far[s] % ps
        for h in range(nkv):
            key = torch.zeros(d)
            key[5 + h] = 12.0
            case["ks"][s][far[s], h] = key.to(dtype)
            case["kp"][page, h, off] = key.to(dtype)
    q = torch.zeros((6, nq, d))
    for h in range(nq):
        q[:, h, 5 + h // 2] = 12.0          # q.k_far * scale = 144 / 8 = 18; every other score is ~N(0, 1.5^2)
    case["q"] = q.view(6, -1).to(dtype)
    scale = d ** -0.5
    dev = {n: case[n].cuda() for n in ("q", "kp", "vp", "tables", "seq_of", "pos")}
    out = torch.empty((6, nq * d), dtype=dtype, device="cuda")
    k.attention_rows(dev["q"], dev["kp"], dev["vp"], dev["tables"], dev["seq_of"], dev["pos"], out, nq, scale)
    want = attention_reference(case, nq, nkv, d, scale)
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))
    for t in range(6):
        s = int(case["seq_of"][t])
        v_far = case["vs"][s][far[s]].float().repeat_interleave(2, dim=0).reshape(-1)
        assert float((out[t].float().cpu() - v_far).abs().max()) < 0.02 + (0.02 if dtype == torch.bfloat16 else 0)
    acc_n, ml_n = k.decode_scratch_floats(1, nq, d, 8)
    out_d = torch.empty((1, nq * d), dtype=dtype, device="cuda")
    k.attention_decode(dev["q"][:1], dev["kp"], dev["vp"], dev["tables"], torch.zeros(1, dtype=torch.int32).cuda(),
                       dev["pos"], out_d, nq, scale, torch.empty(acc_n, device="cuda"), torch.empty(ml_n, device="cuda"),
                       8, split_keys=128)
    torch.testing.assert_close(out_d.float().cpu(), want[:1], **tol(dtype))


def prefill_ranges(k, n_rows, nq, ranges):
    """Keyword arguments of ``attention_prefill_tc`` for ``ranges`` key ranges (scratch poisoned with NaN)."""
    if ranges == 1:
        return {}
    need_o, need_ml = k.prefill_tc_scratch_floats(n_rows, nq, ranges)
    return dict(key_splits=ranges, part_o=torch.full((need_o,), float("nan"), device="cuda"),
                part_ml=torch.full((need_ml,), float("nan"), device="cuda"))


@pytest.mark.parametrize("nq,nkv,ps,ranges", [(4, 2, 16, 1), (2, 2, 8, 1), (3, 1, 64, 1), (4, 2, 16, 3), (3, 1, 64, 2), (2, 2, 8, 7)])
def test_attention_prefill_tensor_cores(k, nq, nkv, ps, ranges):
    """The tcgen05 kernel for prompt portions: whole prompts, a portion that continues from the cache
    across a tile edge, lengths around 128 and 256, shuffled pages with NaN in every unwritten slot;
    with every block's keys cut into ranges (more ranges than some blocks have key tiles: empty ranges)."""
    d = 64
    ctx_lens = [37, 500, 128, 129, 256, 700]
    q_lens = [37, 300, 128, 129, 2, 257]
    case = paged_case(torch.bfloat16, 50 + ps, nq, nkv, d, ps, ctx_lens, q_lens)
    scale = d ** -0.5
    dev = {n: case[n].cuda() for n in ("q", "kp", "vp", "tables", "seq_of", "pos")}
    n_tok = dev["q"].shape[0]
    # q as the leading columns of a wider qkv-like buffer
    qkv = torch.zeros((n_tok, (nq + 2 * nkv) * d), dtype=torch.bfloat16, device="cuda")
    qkv[:, : nq * d] = dev["q"]
    starts = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32).cuda()
    out = torch.full((n_tok, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    n_tiles = k.prefill_tc_blocks(q_lens)
    k.attention_prefill_tc(qkv, dev["kp"], dev["vp"], dev["tables"], starts, dev["pos"], out, n_tiles, nq, scale, status,
                           **prefill_ranges(k, n_tok, nq, ranges))
    torch.cuda.synchronize()
    assert int(status) == 0, f"the kernel gave up waiting on the tensor cores (status {int(status)})"
    want = attention_reference(case, nq, nkv, d, scale)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2)
    # and it agrees with the general row kernel on the same inputs
    out2 = torch.empty_like(out)
    k.attention_rows(dev["q"], dev["kp"], dev["vp"], dev["tables"], dev["seq_of"], dev["pos"], out2, nq, scale)
    torch.testing.assert_close(out.float(), out2.float(), atol=2e-2, rtol=2e-2)


def plant_strong_keys(case, seq, nkv, d, ps, places, dtype, axis=5):
    """Key ``p`` of sequence ``seq`` becomes ``b * e_axis`` for every ``(p, b)`` of ``places`` (in the
    pages and in the plain copy).  A query row with ``q[axis] = 8`` then scores ``b`` on it at head size
    64 (scale 1/8), far above the N(0, 1) scores of the random keys."""
    for p, b in places:
        page, off = int(case["tables"][seq, p // ps]), p % ps
        key = torch.zeros(d)
        key[axis] = b
        for h in range(nkv):
            case["ks"][seq][p, h] = key.to(dtype)
            case["kp"][page, h, off] = key.to(dtype)


@pytest.mark.parametrize("nq,nkv,ps,ranges", [(4, 2, 16, 1), (2, 2, 8, 1), (4, 2, 16, 2), (2, 2, 8, 5)])
def test_attention_prefill_tensor_cores_when_row_maxima_jump(k, nq, nkv, ps, ranges):
    """Random scores never move a row's maximum much after the first tile, so the path that rescales the
    output accumulator when a maximum jumps would go untested.  Here keys with scores of 10, 25 and 40
    (natural-log units: each more than 2^8 above everything before it) sit in later tiles of the keys, for
    every third query row only, so that a warp holds rows that jump beside rows that do not; one sequence
    continues from the cache with a strong key in the cached part and one in the new part."""
    d, dtype = 64, torch.bfloat16
    ctx_lens, q_lens = [1300, 700, 200], [1300, 257, 200]
    case = paged_case(dtype, 333 + ps, nq, nkv, d, ps, ctx_lens, q_lens)
    plant_strong_keys(case, 0, nkv, d, ps, [(300, 10.0), (600, 25.0), (1290, 40.0)], dtype)
    plant_strong_keys(case, 1, nkv, d, ps, [(140, 10.0), (300, 25.0), (600, 40.0)], dtype)
    plant_strong_keys(case, 2, nkv, d, ps, [(3, 40.0), (150, 10.0)], dtype)      # the strongest first: no jump later
    q = case["q"].float().view(-1, nq, d)
    q[::3, :, 5] = 8.0
    case["q"] = q.view(-1, nq * d).to(dtype)
    scale = d ** -0.5
    dev = {n: case[n].cuda() for n in ("q", "kp", "vp", "tables", "seq_of", "pos")}
    n_tok = dev["q"].shape[0]
    qkv = torch.zeros((n_tok, (nq + 2 * nkv) * d), dtype=dtype, device="cuda")
    qkv[:, : nq * d] = dev["q"]
    starts = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32).cuda()
    out = torch.full((n_tok, nq * d), float("nan"), dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.attention_prefill_tc(qkv, dev["kp"], dev["vp"], dev["tables"], starts, dev["pos"], out,
                           k.prefill_tc_blocks(q_lens), nq, scale, status, **prefill_ranges(k, n_tok, nq, ranges))
    torch.cuda.synchronize()
    assert int(status) == 0
    want = attention_reference(case, nq, nkv, d, scale)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2)
    # the planted keys decide the rows that look for them: row 1299 of sequence 0 is the value of key 1290
    v_far = case["vs"][0][1290].float().repeat_interleave(nq // nkv, dim=0).reshape(-1)
    assert float((got[1299] - v_far).abs().max()) < 0.03 and 1299 % 3 == 0
    out2 = torch.empty_like(out)
    k.attention_rows(dev["q"], dev["kp"], dev["vp"], dev["tables"], dev["seq_of"], dev["pos"], out2, nq, scale)
    torch.testing.assert_close(out.float(), out2.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("which,nq,nkv,ps,split", [("bulk", 4, 4, 16, 512), ("bulk", 4, 4, 16, 2048), ("gqa", 6, 2, 16, 512),
                                                   ("gqa", 15, 5, 16, 1024)])
def test_decode_attention_finds_far_keys_and_follows_rising_maxima(k, which, nq, nkv, ps, split):
    """The bulk-copy and the tensor-core decode kernels: one key in the first page decides a row; in
    another row, keys of rising strength sit in later stages and later splits, so the running maximum
    jumps inside a warp's stream, between the warps of a block and between splits."""
    d, dtype = 64, torch.bfloat16
    ctx_lens = [900, 1500, 1500, 77]
    case = paged_case(dtype, 444 + nq, nq, nkv, d, ps, ctx_lens, [1] * 4)
    plant_strong_keys(case, 0, nkv, d, ps, [(3, 18.0)], dtype)
    plant_strong_keys(case, 1, nkv, d, ps, [(40, 10.0), (200, 25.0), (700, 40.0), (1400, 55.0)], dtype)
    plant_strong_keys(case, 2, nkv, d, ps, [(1400, 10.0), (700, 25.0), (200, 40.0), (40, 55.0)], dtype)   # falling instead
    q = case["q"].float().view(-1, nq, d)
    q[:3, :, 5] = 8.0
    case["q"] = q.view(-1, nq * d).to(dtype)
    scale = d ** -0.5
    dev = {n: case[n].cuda() for n in ("q", "kp", "vp", "tables", "seq_of", "pos")}
    n = len(ctx_lens)
    max_splits = max((c - 1) // split + 1 for c in ctx_lens)
    acc_n, ml_n = k.decode_scratch_floats(n, nq, d, max_splits)
    part_acc, part_ml = torch.full((acc_n,), float("nan"), device="cuda"), torch.full((ml_n,), float("nan"), device="cuda")
    out = torch.full((n, nq * d), float("nan"), dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tok = torch.arange(n, dtype=torch.int32).cuda()
    fn = k.attention_decode_bulk if which == "bulk" else k.attention_decode_gqa
    fn(dev["q"], dev["kp"], dev["vp"], dev["tables"], tok, dev["pos"], out, nq, scale, part_acc, part_ml, max_splits,
       status, split_keys=split)
    torch.cuda.synchronize()
    assert int(status) == 0
    want = attention_reference(case, nq, nkv, d, scale)
    got = out.float().cpu()
    torch.testing.assert_close(got, want, **tol(dtype))
    for s, far in ((0, 3), (1, 1400), (2, 40)):
        v_far = case["vs"][s][far].float().repeat_interleave(nq // nkv, dim=0).reshape(-1)
        assert float((got[s] - v_far).abs().max()) < 0.04, (s, far)


def test_attention_refuses_bad_head_sizes(k):
    from edgerag_b200.ops.kernels import KernelError

    q = torch.zeros((1, 2 * 24), device="cuda")
    kp = torch.zeros((1, 2, 4, 24), device="cuda")
    t = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(KernelError, match="head_dim 24"):
        k.attention_rows(q, kp, kp, t, z, z, torch.empty_like(q), 2, 1.0)


# --- sampling --------------------------------------------------------------------------------

@pytest.mark.parametrize("vocab", [1000, 49155])
def test_greedy_takes_the_first_maximum(k, vocab):
    logits = rand((5, vocab + 5), torch.float32, 30)[:, :vocab]        # a row-strided view, as the engine's
    logits[1, 77] = logits[1, 900] = 50.0                               # a tie: the first index wins
    logits[2, vocab - 1] = 60.0
    logits[3, 0] = 60.0
    tokens = torch.full((5,), -1, dtype=torch.int32, device="cuda")
    k.sample_rows(logits, tokens)
    want = [int(logits[i].argmax()) for i in range(5)]
    want[1] = 77
    assert tokens.tolist() == want


def test_temperature_sampling_follows_the_distribution(k):
    vocab, rows, temp = 1000, 4096, 0.7
    base = rand((1, vocab), torch.float32, 31, 2.0)
    logits = base.expand(rows, vocab).contiguous()
    states = torch.arange(rows, dtype=torch.int64).mul_(0x9E3779B97F4A7C15 % (1 << 62)).cuda()
    temps = torch.full((rows,), temp, device="cuda")
    temps[:3] = 0.0                                                     # greedy rows in the same launch
    tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
    k.sample_rows(logits, tokens, temps, states)
    probs = plain.temperature_probs(base[0].cpu(), temp)
    cdf = torch.cumsum(probs, 0).numpy()
    got = tokens.cpu().numpy()
    assert (got[:3] == int(base.argmax())).all()
    # every draw sits where the inverse CDF of its own uniform puts it (up to float32 rounding of the sums)
    for r in range(3, rows, 7):
        u = k.uniform_from_state(int(states[r]))
        t = int(got[r])
        lo = cdf[t - 1] if t else 0.0
        assert lo - 1e-5 <= u < cdf[t] + 1e-5, (r, u, t, lo, cdf[t])
    # and the draws as a whole follow the distribution
    counts = np.bincount(got[3:], minlength=vocab)
    top = np.argsort(-probs.numpy())[:20]
    n = rows - 3
    for t in top:
        p = float(probs[t])
        assert abs(counts[t] / n - p) < 5 * math.sqrt(p * (1 - p) / n) + 1e-3
    # same state, same token; a different state changes some tokens
    again = torch.empty_like(tokens)
    k.sample_rows(logits, again, temps, states)
    assert torch.equal(again, tokens)
