"""Parity of the memory-bound DIOPI ops (CUDA, through the C-ABI) against torch CPU arithmetic - the arithmetic of
DIPU's forced CPU fallback. Shapes and tolerances of the small cases come from the reference's own unit tests
(dipu/tests/python/unittests/test_*.py, cited per test); the bf16 [T, 4096] cases are the op-sweep configuration with
the stated tolerance: max-abs <= 2e-2 and rel-L2 <= 5e-3 against the fp32 CPU result; index / copy work is bit-exact.
The sweeps run at every T of the op-sweep configuration, the benchmarked 16384 and 65536 included.
"""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def rnd(shape, dtype=torch.float32, seed=0, scale=1.0):
    rng = np.random.default_rng(seed)
    return (torch.from_numpy(rng.standard_normal(size=shape, dtype=np.float32)) * scale).to(dtype)


def check_bf16(got, ref_fp32, max_abs=2e-2, rel_l2=5e-3):
    got = got.float().cpu()
    err = (got - ref_fp32).abs().max().item()
    rel = ((got - ref_fp32).norm() / ref_fp32.norm().clamp_min(1e-30)).item()
    assert err <= max_abs and rel <= rel_l2, "max_abs=%g rel_l2=%g" % (err, rel)


def check_close(got, ref, rtol=1e-5, atol=1e-5):
    np.testing.assert_allclose(got.float().cpu().numpy(), ref.float().numpy(), rtol=rtol, atol=atol)


# ---- copy / cast -------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("t", [1, 64, 1024, 4097, 16384, 65536])
def test_cast_bf16_fp32_roundtrip_bit_exact(diopi, ctx, t):
    x = rnd((t, 4096), torch.bfloat16, seed=t)
    xd = x.to(DEV)
    up = torch.empty((t, 4096), dtype=torch.float32, device=DEV)
    diopi.diopiCopyInp(ctx, xd, up)
    assert torch.equal(up.cpu(), x.float())  # widening is exact
    f = rnd((t, 4096), torch.float32, seed=t + 1)
    down = torch.empty((t, 4096), dtype=torch.bfloat16, device=DEV)
    diopi.diopiCopyInp(ctx, f.to(DEV), down)
    assert torch.equal(down.cpu().view(torch.int16), f.to(torch.bfloat16).view(torch.int16))  # round-to-nearest-even like torch CPU


def test_cast_int64_to_others(diopi, ctx):
    # dipu/tests/python/unittests/test_cast.py:8-14
    x = torch.arange(200, dtype=torch.int64)
    for dt in (torch.float64, torch.int32, torch.int64, torch.float32, torch.float16):
        out = torch.empty(200, dtype=dt, device=DEV)
        diopi.diopiCopyInp(ctx, x.to(DEV), out)
        assert torch.equal(out.cpu(), x.to(dt))


def test_copy_transpose_materialisation_bit_exact(diopi, ctx):
    # [B, S, H, D] -> [B, H, S, D], the layout change around attention
    x = rnd((2, 33, 4, 128), torch.bfloat16, seed=3)
    xd = x.to(DEV)
    out = torch.empty((2, 4, 33, 128), dtype=torch.bfloat16, device=DEV)
    diopi.diopiCopyInp(ctx, xd.transpose(1, 2), out)
    assert torch.equal(out.cpu(), x.transpose(1, 2).contiguous())
    # shapes that reach the tiled kernel (>= 8 heads, >= 16 positions), ragged against its 8 x 16 tiles, both directions,
    # 64- and 128-element rows, and a leading batch dimension
    for shape in ((3, 50, 12, 128), (1, 17, 9, 64), (2, 256, 32, 128), (1, 16, 8, 256)):
        x = rnd(shape, torch.bfloat16, seed=sum(shape))
        xd = x.to(DEV)
        out = torch.empty((shape[0], shape[2], shape[1], shape[3]), dtype=torch.bfloat16, device=DEV)
        diopi.diopiCopyInp(ctx, xd.transpose(1, 2), out)
        assert torch.equal(out.cpu(), x.transpose(1, 2).contiguous())
        back = torch.empty(shape, dtype=torch.bfloat16, device=DEV)
        diopi.diopiCopyInp(ctx, out.transpose(1, 2), back)
        assert torch.equal(back.cpu(), x)
    # odd inner extent: falls back to narrower words
    y = rnd((5, 7, 3), torch.float32, seed=4)
    o2 = torch.empty((3, 7, 5), dtype=torch.float32, device=DEV)
    diopi.diopiCopyInp(ctx, y.to(DEV).permute(2, 1, 0), o2)
    assert torch.equal(o2.cpu(), y.permute(2, 1, 0).contiguous())


def test_copy_expand_and_hollow_destination(diopi, ctx):
    # dipu/tests/python/unittests/test_copy.py:40-85: broadcast source, strided ("hollow") destination
    src = rnd((1, 6), torch.float32, seed=5)
    dst = torch.zeros((4, 6), dtype=torch.float16, device=DEV)
    diopi.diopiCopyInp(ctx, src.to(DEV), dst)
    assert torch.equal(dst.cpu(), src.expand(4, 6).to(torch.float16))
    big = torch.zeros((8, 10), dtype=torch.float32, device=DEV)
    view = big[::2, 1:9:2]
    s2 = rnd((4, 4), torch.float32, seed=6)
    diopi.diopiCopyInp(ctx, s2.to(DEV), view)
    ref = torch.zeros((8, 10))
    ref[::2, 1:9:2] = s2
    assert torch.equal(big.cpu(), ref)


def test_copy_kv_append_slice(diopi, ctx):
    cache = torch.zeros((2, 3, 16, 8), dtype=torch.bfloat16, device=DEV)
    new = rnd((2, 3, 8), torch.bfloat16, seed=7)
    diopi.diopiCopyInp(ctx, new.to(DEV), cache[:, :, 5, :])
    ref = torch.zeros((2, 3, 16, 8), dtype=torch.bfloat16)
    ref[:, :, 5, :] = new
    assert torch.equal(cache.cpu(), ref)


def test_copy_empty(diopi, ctx):
    a = torch.empty((0, 4), device=DEV)
    b = torch.empty((0, 4), device=DEV)
    diopi.diopiCopyInp(ctx, a, b)


# ---- gather ----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("t", [1, 64, 1024, 16384, 65536])
def test_embedding_gather_bit_exact(diopi, ctx, t):
    rng = np.random.default_rng(t)
    table = rnd((32000, 4096), torch.bfloat16, seed=11, scale=0.02)
    ids = torch.from_numpy(rng.integers(0, 32000, size=t, dtype=np.int64))
    td = table.to(DEV)
    out = torch.empty((t, 4096), dtype=torch.bfloat16, device=DEV)
    diopi.diopiIndexSelect(ctx, out, td, 0, ids.to(DEV))
    assert torch.equal(out.cpu(), table[ids])
    out2 = torch.empty((t, 4096), dtype=torch.bfloat16, device=DEV)
    diopi.diopiEmbedding(ctx, out2, td, ids.to(DEV), -1, False, False)
    assert torch.equal(out2.cpu(), table[ids])


def test_index_select_dims(diopi, ctx):
    # dipu/tests/python/unittests/test_index.py:65-76
    x = rnd((3, 4), seed=1)
    idx = torch.tensor([0, 2])
    for dim, shape in ((0, (2, 4)), (1, (3, 2))):
        out = torch.empty(shape, device=DEV)
        diopi.diopiIndexSelect(ctx, out, x.to(DEV), dim, idx.to(DEV))
        assert torch.equal(out.cpu(), torch.index_select(x, dim, idx))
    # int32 indices, empty index
    out = torch.empty((2, 4), device=DEV)
    diopi.diopiIndexSelect(ctx, out, x.to(DEV), 0, idx.to(torch.int32).to(DEV))
    assert torch.equal(out.cpu(), x[idx])
    out = torch.empty((0, 4), device=DEV)
    diopi.diopiIndexSelect(ctx, out, x.to(DEV), 0, torch.empty(0, dtype=torch.int64, device=DEV))


# ---- element-wise --------------------------------------------------------------------------------------------------------
def test_add_mul_reference_cases(diopi, ctx):
    # dipu/tests/python/unittests/test_add.py:8-32, test_mul.py:8-23
    a, b = rnd((3, 4), seed=1), rnd((3, 4), seed=2)
    out = torch.empty((3, 4), device=DEV)
    diopi.diopiAdd(ctx, out, a.to(DEV), b.to(DEV), 1)
    assert torch.equal(out.cpu(), a + b)
    diopi.diopiAdd(ctx, out, a.to(DEV), b.to(DEV), 0.3)
    check_close(out, torch.add(a, b, alpha=0.3), 1e-6, 1e-6)
    ad = a.to(DEV).clone()
    diopi.diopiAddInpScalar(ctx, ad, 3, 1)
    assert torch.equal(ad.cpu(), a + 3)
    # scalar self: add(2, x, alpha=0.3) reaches the library as a 0-dim host tensor
    diopi.diopiAdd(ctx, out, torch.tensor(2.0), b.to(DEV), 0.3)
    check_close(out, torch.add(torch.tensor(2.0), b, alpha=0.3), 1e-6, 1e-6)
    # broadcast [4,1] * [1,4]
    c, d = rnd((4, 1), seed=3), rnd((1, 4), seed=4)
    o2 = torch.empty((4, 4), device=DEV)
    diopi.diopiMul(ctx, o2, c.to(DEV), d.to(DEV))
    assert torch.equal(o2.cpu(), c * d)
    diopi.diopiMul(ctx, out, a.to(DEV), torch.tensor(2.5))  # host 0-dim scalar tensor
    assert torch.equal(out.cpu(), a * 2.5)
    diopi.diopiMulScalar(ctx, out, a.to(DEV), 3)
    assert torch.equal(out.cpu(), a * 3)
    diopi.diopiSub(ctx, out, a.to(DEV), b.to(DEV), 2)
    check_close(out, a - 2 * b, 1e-6, 1e-6)
    diopi.diopiDivScalar(ctx, out, a.to(DEV), 8.0, diopi.RoundModeNone)
    assert torch.equal(out.cpu(), a / 8.0)
    diopi.diopiDiv(ctx, out, a.to(DEV), b.to(DEV), diopi.RoundModeFloor)
    check_close(out, torch.div(a, b, rounding_mode="floor"), 0, 0)


def test_integer_and_mixed_dtype_arithmetic(diopi, ctx):
    a = torch.arange(-6, 6, dtype=torch.int64).view(3, 4)
    b = torch.full((3, 4), 4, dtype=torch.int32)
    out = torch.empty((3, 4), dtype=torch.int64, device=DEV)
    diopi.diopiAdd(ctx, out, a.to(DEV), b.to(DEV), 2)
    assert torch.equal(out.cpu(), a + 2 * b)
    diopi.diopiDiv(ctx, out, a.to(DEV), b.to(DEV), diopi.RoundModeFloor)
    assert torch.equal(out.cpu(), torch.div(a, b, rounding_mode="floor"))
    # bf16 * fp32 -> fp32 (type promotion done by the host, mixed inputs handled by the library)
    x, w = rnd((5, 16), torch.bfloat16, seed=1), rnd((16,), torch.float32, seed=2)
    o = torch.empty((5, 16), dtype=torch.float32, device=DEV)
    diopi.diopiMul(ctx, o, x.to(DEV), w.to(DEV))
    assert torch.equal(o.cpu(), x.float() * w)


@pytest.mark.parametrize("t", [1, 64, 1024, 4096, 16384, 65536])
def test_sweep_silu_mul_add_bf16(diopi, ctx, t):
    a, b = rnd((t, 4096), torch.bfloat16, seed=t), rnd((t, 4096), torch.bfloat16, seed=t + 1)
    ad, bd = a.to(DEV), b.to(DEV)
    out = torch.empty_like(ad)
    diopi.diopiSilu(ctx, out, ad)
    check_bf16(out, torch.nn.functional.silu(a.float()))
    diopi.diopiMul(ctx, out, ad, bd)
    assert torch.equal(out.cpu(), (a.float() * b.float()).to(torch.bfloat16))
    diopi.diopiAdd(ctx, out, ad, bd, 1)
    assert torch.equal(out.cpu(), (a.float() + b.float()).to(torch.bfloat16))
    g = ad.clone()
    diopi.diopiSiluInp(ctx, g)
    diopi.diopiMulInp(ctx, g, bd)
    # two chained bf16 ops: equal to the CPU computing the same two ops on bf16 tensors up to one rounding step of the
    # intermediate, and within the relative bound of the fp32 result (values reach |16|, where a bf16 ulp is 0.06)
    step = (torch.nn.functional.silu(a.float()).to(torch.bfloat16).float() * b.float()).to(torch.bfloat16).float()
    check_bf16(g, step, max_abs=0.13, rel_l2=2e-3)
    check_bf16(g, torch.nn.functional.silu(a.float()) * b.float(), max_abs=0.13, rel_l2=5e-3)


def test_broadcast_fast_path_and_ragged_tail(diopi, ctx):
    # [B*H, S, S] + [S, S] (mask add) and [T, H] * [H]; sizes that leave a tail for the vector kernel
    s = rnd((6, 40, 40), torch.bfloat16, seed=1)
    m = torch.triu(torch.full((40, 40), float("-inf")), diagonal=1).to(torch.bfloat16)
    sd = s.to(DEV)
    diopi.diopiAddInp(ctx, sd, m.to(DEV), 1)
    assert torch.equal(sd.cpu(), (s.float() + m.float()).to(torch.bfloat16))
    x, w = rnd((37, 24), torch.bfloat16, seed=2), rnd((24,), torch.bfloat16, seed=3)
    out = torch.empty((37, 24), dtype=torch.bfloat16, device=DEV)
    diopi.diopiMul(ctx, out, x.to(DEV), w.to(DEV))
    assert torch.equal(out.cpu(), (x.float() * w.float()).to(torch.bfloat16))
    y = rnd((1003,), torch.float32, seed=4)
    o = torch.empty(1003, device=DEV)
    diopi.diopiNeg(ctx, o, y.to(DEV))
    assert torch.equal(o.cpu(), -y)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_elementwise_on_views_with_dense_rows(diopi, ctx, dtype):
    """The op-by-op rotary embedding of a plain torch model: q as a transposed view, tables broadcast over batch and heads,
    halves of the head dimension as slices, outputs that keep the view's permutation. bf16 add / mul of two bf16 values
    round an exact fp32 result once: bit-exact against torch CPU."""
    b, s, h, d = 2, 37, 3, 64
    q = rnd((b, s, h, d), dtype, seed=1)
    cos = rnd((1, 1, s, d), dtype, seed=2)
    qd, cd = q.to(DEV), cos.to(DEV)
    qt, qtd = q.transpose(1, 2), qd.transpose(1, 2)                  # [b, h, s, d] view, pitches (s*h*d, d, h*d, 1)
    out = torch.empty_strided(qt.shape, qt.stride(), dtype=dtype, device=DEV)   # the permuted layout torch gives the result
    diopi.diopiMul(ctx, out, qtd, cd)
    assert torch.equal(out.cpu(), qt * cos)
    dense = torch.empty(qt.shape, dtype=dtype, device=DEV)
    diopi.diopiAdd(ctx, dense, qtd, cd, 1)
    assert torch.equal(dense.cpu(), qt + cos)
    # halves of the last dimension (32 elements = 64 or 128 bytes, 16-byte aligned starts)
    neg = torch.empty((b, h, s, d // 2), dtype=dtype, device=DEV)
    diopi.diopiNeg(ctx, neg, qtd[..., d // 2:])
    assert torch.equal(neg.cpu(), -qt[..., d // 2:])
    half = torch.empty((b, h, s, d // 2), dtype=dtype, device=DEV)
    diopi.diopiMul(ctx, half, qtd[..., : d // 2], qtd[..., d // 2:])
    assert torch.equal(half.cpu(), qt[..., : d // 2] * qt[..., d // 2:])
    # an input that is constant along the row ([.., 1] against [.., d]) and one that repeats over the leading dimensions
    col = rnd((b, h, s, 1), dtype, seed=3)
    diopi.diopiMul(ctx, dense, qtd, col.to(DEV))
    assert torch.equal(dense.cpu(), qt * col)
    row = rnd((d,), dtype, seed=4)
    diopi.diopiAddInp(ctx, out, row.to(DEV), 1)
    assert torch.equal(out.cpu(), qt * cos + row)
    # in place on a view
    diopi.diopiSiluInp(ctx, qtd)
    if dtype == torch.float32:
        check_close(qtd, torch.nn.functional.silu(qt), 1e-5, 1e-6)
    else:
        check_bf16(qtd, torch.nn.functional.silu(qt.float()))


def test_unary_reference_cases(diopi, ctx):
    # test_rsqrt.py:7-19, test_silu.py:8-34, test_neg.py
    x = torch.rand(10, generator=torch.Generator().manual_seed(1)) * 0.98 + 0.01
    out = torch.empty(10, device=DEV)
    diopi.diopiRsqrt(ctx, out, x.to(DEV))
    check_close(out, torch.rsqrt(x), 1e-5, 1e-5)
    xd = x.to(DEV).clone()
    diopi.diopiRsqrtInp(ctx, xd)
    check_close(xd, torch.rsqrt(x), 1e-5, 1e-5)
    y = torch.tensor([-2.0, 3.0])
    o2 = torch.empty(2, device=DEV)
    diopi.diopiSilu(ctx, o2, y.to(DEV))
    check_close(o2, torch.nn.functional.silu(y), 1e-5, 1e-5)
    h = torch.empty(2, dtype=torch.float16, device=DEV)
    diopi.diopiSilu(ctx, h, y.to(torch.float16).to(DEV))
    check_close(h, torch.nn.functional.silu(y), 1e-2, 1e-2)
    for name, fn in (("diopiNeg", torch.neg), ("diopiExp", torch.exp), ("diopiSin", torch.sin), ("diopiCos", torch.cos),
                     ("diopiSqrt", torch.sqrt), ("diopiReciprocal", torch.reciprocal), ("diopiSigmoid", torch.sigmoid),
                     ("diopiTanh", torch.tanh), ("diopiRelu", torch.relu)):
        getattr(diopi, name)(ctx, out, x.to(DEV))
        check_close(out, fn(x), 1e-5, 1e-6)
    d = x.double()
    od = torch.empty(10, dtype=torch.float64, device=DEV)
    diopi.diopiExp(ctx, od, d.to(DEV))
    np.testing.assert_allclose(od.cpu().numpy(), torch.exp(d).numpy(), rtol=1e-12)


def test_pow_fill_masks(diopi, ctx):
    x = rnd((4, 6), seed=1)
    out = torch.empty((4, 6), device=DEV)
    diopi.diopiPow(ctx, out, x.to(DEV), 2)
    assert torch.equal(out.cpu(), x.pow(2))
    diopi.diopiPow(ctx, out, x.abs().to(DEV), 1.7)
    check_close(out, x.abs().pow(1.7), 1e-5, 1e-6)
    diopi.diopiPowScalar(ctx, out, 10000.0, (x * 0.1).to(DEV))
    check_close(out, torch.pow(10000.0, x * 0.1), 1e-5, 1e-6)
    diopi.diopiFill(ctx, out, float("-inf"))
    assert torch.isinf(out).all().item()
    sq = torch.empty((6, 6), dtype=torch.bfloat16, device=DEV)
    diopi.diopiFill(ctx, sq, float("-inf"))
    diopi.diopiTriuInp(ctx, sq, 1)
    assert torch.equal(sq.cpu().float(), torch.triu(torch.full((6, 6), float("-inf")), diagonal=1))
    m = torch.rand(4, 6, generator=torch.Generator().manual_seed(2)) > 0.5
    diopi.diopiMaskedFillScalar(ctx, out, x.to(DEV), m.to(DEV), -1.5)
    assert torch.equal(out.cpu(), x.masked_fill(m, -1.5))
    y = rnd((4, 6), seed=3)
    diopi.diopiWhere(ctx, out, m.to(DEV), x.to(DEV), y.to(DEV))
    assert torch.equal(out.cpu(), torch.where(m, x, y))
    ar = torch.empty(17, dtype=torch.int64, device=DEV)
    diopi.diopiArange(ctx, ar, 3, 37, 2)
    assert torch.equal(ar.cpu(), torch.arange(3, 37, 2))
    af = torch.empty(128, dtype=torch.float32, device=DEV)
    diopi.diopiArange(ctx, af, 0, 128, 1)
    assert torch.equal(af.cpu(), torch.arange(128).float())
    z = torch.ones((3, 5), device=DEV)
    diopi.diopiZeroInp(ctx, z)
    assert (z == 0).all().item()
    diopi.diopiOnes(ctx, z, [3, 5])
    assert (z == 1).all().item()


def test_cat(diopi, ctx):
    # dipu/tests/python/unittests/test_cat.py:7-32
    xs = [rnd((2, 3), seed=i) for i in range(3)]
    for dim, shape in ((0, (6, 3)), (1, (2, 9))):
        out = torch.empty(shape, device=DEV)
        diopi.diopiCat(ctx, out, [x.to(DEV) for x in xs], dim)
        assert torch.equal(out.cpu(), torch.cat(xs, dim))
    big = rnd((8, 8732), torch.float32, seed=9).double()
    bd = big.to(DEV)
    out = torch.empty((8, 8000), dtype=torch.float64, device=DEV)
    diopi.diopiCat(ctx, out, [bd[:, :4000], bd[:, 4732:]], 1)
    assert torch.equal(out.cpu(), torch.cat([big[:, :4000], big[:, 4732:]], 1))


# ---- reductions / normalisation -------------------------------------------------------------------------------------------------
def test_mean_sum(diopi, ctx):
    # dipu/tests/python/unittests/test_mean_std.py:12-36
    x = rnd((4, 4, 6, 7), seed=1)
    for dims, keep in (([1], False), ([1, 3], False), ([1, 3], True), ([3], False), ([2, 3], False), ([], False)):
        ref = x.mean(dims, keepdim=keep) if dims else x.mean()
        out = torch.empty(ref.shape, device=DEV)
        diopi.diopiMean(ctx, out, x.to(DEV), dims)
        check_close(out, ref, 1e-5, 1e-6)
    out = torch.empty((4, 4, 6), device=DEV)
    diopi.diopiSum(ctx, out, x.to(DEV), [3])
    check_close(out, x.sum(3), 1e-5, 1e-5)
    # the RMSNorm decomposition's mean over [T, H] bf16 -> fp32 rows
    y = rnd((64, 4096), torch.float32, seed=2)
    o2 = torch.empty((64, 1), device=DEV)
    diopi.diopiMean(ctx, o2, y.to(DEV), [-1])
    check_close(o2, y.mean(-1, keepdim=True), 1e-4, 1e-6)


@pytest.mark.parametrize("t", [1, 64, 1024, 4096, 16384, 65536])
def test_sweep_rmsnorm_bf16(diopi, ctx, t):
    x = rnd((t, 4096), torch.bfloat16, seed=t)
    w = (1.0 + 0.1 * rnd((4096,), torch.float32, seed=1)).to(torch.bfloat16)
    out = torch.empty((t, 4096), dtype=torch.bfloat16, device=DEV)
    inv = torch.empty((t, 1), dtype=torch.float32, device=DEV)
    diopi.diopiRMSNorm(ctx, out, inv, x.to(DEV), [4096], w.to(DEV), None, 1e-6)
    xf = x.float()
    ref_inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)
    check_bf16(out, xf * ref_inv * w.float())
    check_close(inv, ref_inv, 1e-5, 1e-6)


def test_rmsnorm_fp32_matches_golden(diopi, ctx):
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rmsnorm.npz"))
    out = torch.empty((64, 512), device=DEV)
    diopi.diopiRMSNorm(ctx, out, None, torch.from_numpy(g["x"]).to(DEV), [512], torch.from_numpy(g["weight"]).to(DEV), None, 1e-6)
    np.testing.assert_allclose(out.cpu().numpy(), g["y"], rtol=1e-5, atol=1e-6)


def test_rmsnorm_decomposed_equals_fused(diopi, ctx):
    # the op stream DIPU dispatches for the reference's RMSNorm module: pow, mean, add scalar, rsqrt, mul, mul
    x = rnd((16, 512), torch.float32, seed=3)
    w = rnd((512,), torch.float32, seed=4)
    xd, wd = x.to(DEV), w.to(DEV)
    sq = torch.empty_like(xd)
    diopi.diopiPow(ctx, sq, xd, 2)
    ms = torch.empty((16, 1), device=DEV)
    diopi.diopiMean(ctx, ms, sq, [-1])
    diopi.diopiAddInpScalar(ctx, ms, 1e-6, 1)
    diopi.diopiRsqrtInp(ctx, ms)
    y = torch.empty_like(xd)
    diopi.diopiMul(ctx, y, xd, ms)
    diopi.diopiMulInp(ctx, y, wd)
    fused = torch.empty_like(xd)
    diopi.diopiRMSNorm(ctx, fused, None, xd, [512], wd, None, 1e-6)
    check_close(y, fused.cpu(), 1e-5, 1e-6)


@pytest.mark.parametrize("t", [1, 64, 1024, 16384, 65536])
def test_sweep_layernorm_bf16(diopi, ctx, t):
    x = rnd((t, 4096), torch.bfloat16, seed=t)
    w = (1.0 + 0.1 * rnd((4096,), seed=1)).to(torch.bfloat16)
    b = (0.1 * rnd((4096,), seed=2)).to(torch.bfloat16)
    out = torch.empty((t, 4096), dtype=torch.bfloat16, device=DEV)
    mean = torch.empty((t, 1), dtype=torch.bfloat16, device=DEV)
    rstd = torch.empty((t, 1), dtype=torch.bfloat16, device=DEV)
    diopi.diopiLayerNorm(ctx, out, mean, rstd, x.to(DEV), w.to(DEV), b.to(DEV), [4096], 1e-5)
    ref, rm, rr = torch.native_layer_norm(x.float(), [4096], w.float(), b.float(), 1e-5)
    check_bf16(out, ref, max_abs=4e-2)
    check_bf16(mean, rm, max_abs=1e-2, rel_l2=1e-2)
    check_bf16(rstd, rr, max_abs=1e-2, rel_l2=1e-2)


def test_layernorm_reference_cases(diopi, ctx):
    # dipu/tests/python/unittests/test_layer_norm.py:57-92: normalise the trailing dims, affine on/off, non-contiguous input
    x = rnd((4, 3, 4, 5, 6, 8), seed=1)
    for ndims in (2, 3):
        shape = list(x.shape[-ndims:])
        w, b = rnd(shape, seed=2), rnd(shape, seed=3)
        rows = x.numel() // int(np.prod(shape))
        stat_shape = list(x.shape[:-ndims]) + [1] * ndims
        for affine in (True, False):
            out = torch.empty(x.shape, device=DEV)
            mean = torch.empty(stat_shape, device=DEV)
            rstd = torch.empty(stat_shape, device=DEV)
            diopi.diopiLayerNorm(ctx, out, mean, rstd, x.to(DEV), w.to(DEV) if affine else None, b.to(DEV) if affine else None, shape, 1e-5)
            ref, rm, rr = torch.native_layer_norm(x, shape, w if affine else None, b if affine else None, 1e-5)
            check_close(out, ref, 1e-4, 1e-3)
            check_close(mean.view(rows), rm.reshape(rows), 1e-4, 1e-5)
            check_close(rstd.view(rows), rr.reshape(rows), 1e-4, 1e-5)
    xt = rnd((6, 5, 8), seed=4)
    out = torch.empty((5, 6, 8), device=DEV)
    diopi.diopiLayerNorm(ctx, out, None, None, xt.to(DEV).transpose(0, 1), None, None, [8], 1e-5)
    check_close(out, torch.layer_norm(xt.transpose(0, 1), [8]), 1e-4, 1e-3)
    assert out.is_contiguous()


@pytest.mark.parametrize("t", [1, 64, 1024, 4096, 16384, 65536])
def test_sweep_softmax_bf16(diopi, ctx, t):
    x = rnd((t, 4096), torch.bfloat16, seed=t, scale=3.0)
    out = torch.empty((t, 4096), dtype=torch.bfloat16, device=DEV)
    diopi.diopiSoftmax(ctx, out, x.to(DEV), -1)
    check_bf16(out, torch.softmax(x.float(), -1))


@pytest.mark.parametrize("rows,cols,dtype", [(4096, 2048, torch.bfloat16), (2000, 264, torch.bfloat16), (1500, 1000, torch.float32),
                                            (1025, 8, torch.float16), (3000, 1024, torch.float32), (1027, 1544, torch.float16)])
def test_softmax_many_short_rows(diopi, ctx, rows, cols, dtype):
    """Score-tensor-like inputs (many rows of at most 256 vectors) take the warp-per-row kernel, 2-byte rows of more than 128 vectors
    the two-warps-per-row one (also with a row count that does not fill the last CTA and a ragged vector count); causal -inf entries,
    in place."""
    x = rnd((rows, cols), dtype, seed=rows, scale=3.0)
    k = min(rows, cols)
    x[:k, :k] = (x[:k, :k].float() + torch.triu(torch.full((k, k), float("-inf")), diagonal=1)).to(dtype)
    xd = x.to(DEV)
    diopi.diopiSoftmax(ctx, xd, xd, -1)
    ref = torch.softmax(x.float(), -1)
    if dtype == torch.float32:
        check_close(xd, ref, 1e-4, 1e-6)
    else:
        check_bf16(xd, ref)
    assert torch.isfinite(xd.float()).all()


def test_softmax_reference_cases(diopi, ctx):
    # dipu/tests/python/unittests/test_softmax.py:24-70: fp32, U(0,10), dim = 0 and last
    g = torch.Generator().manual_seed(1)
    for shape in ((256, 1000), (32, 48, 1024), (8, 6, 18, 1000)):
        x = torch.rand(shape, generator=g) * 10
        for dim in (0, -1, 1):
            out = torch.empty(shape, device=DEV)
            diopi.diopiSoftmax(ctx, out, x.to(DEV), dim)
            check_close(out, torch.softmax(x, dim), 1e-4, 1e-4)
    # causal rows: -inf entries, and in-place use (out aliases the input)
    s = rnd((3, 64, 64), torch.bfloat16, seed=2)
    s = (s.float() + torch.triu(torch.full((64, 64), float("-inf")), diagonal=1)).to(torch.bfloat16)
    sd = s.to(DEV)
    diopi.diopiSoftmax(ctx, sd, sd, -1)
    check_bf16(sd, torch.softmax(s.float(), -1))
    # bf16 in, fp32 out (half_to_float)
    o32 = torch.empty((3, 64, 64), dtype=torch.float32, device=DEV)
    diopi.diopiSoftmax(ctx, o32, s.to(DEV), -1)
    check_close(o32, torch.softmax(s.float(), -1), 1e-5, 1e-6)


# ---- rotary embedding ----------------------------------------------------------------------------------------------------------------------
def _tables(d, n):
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
    ang = torch.outer(torch.arange(n).float(), inv)
    return torch.cos(ang), torch.sin(ang)


def _rope_half_ref(x, cos, sin):
    t, h, d = x.shape
    reps = t // cos.shape[0]
    c, s = cos.repeat(reps, 1).view(t, 1, -1), sin.repeat(reps, 1).view(t, 1, -1)
    x0, x1 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat((x0 * c - x1 * s, x0 * s + x1 * c), -1)


@pytest.mark.parametrize("t", [1, 64, 1024, 16384, 65536])
def test_sweep_rope_bf16(diopi, ctx, t):
    x = rnd((t, 32, 128), torch.bfloat16, seed=t)
    cos, sin = _tables(128, t)
    out = torch.empty((t, 32, 128), dtype=torch.bfloat16, device=DEV)
    diopi.diopiRotaryEmbedding(ctx, out, x.to(DEV), cos.to(DEV), sin.to(DEV), False, False)
    check_bf16(out, _rope_half_ref(x.float(), cos, sin))
    # tables broadcast over the batch: [B*S] tokens, [S] rows; bf16 tables; conj rotates back
    if t >= 64:
        cb, sb = cos[: t // 2], sin[: t // 2]
        diopi.diopiRotaryEmbedding(ctx, out, x.to(DEV), cb.to(torch.bfloat16).to(DEV), sb.to(torch.bfloat16).to(DEV), False, False)
        check_bf16(out, _rope_half_ref(x.float(), cb.to(torch.bfloat16).float(), sb.to(torch.bfloat16).float()))
    back = torch.empty_like(out)
    diopi.diopiRotaryEmbedding(ctx, out, x.to(DEV), cos.to(DEV), sin.to(DEV), False, False)
    diopi.diopiRotaryEmbedding(ctx, back, out, cos.to(DEV), sin.to(DEV), True, False)
    check_bf16(back, x.float(), max_abs=6e-2, rel_l2=1e-2)  # two bf16 roundings


def test_rope_matches_golden_both_layouts(diopi, ctx):
    import os
    gold = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    g = np.load(os.path.join(gold, "ext_ops.npz"))
    x = torch.from_numpy(g["x"])
    out = torch.empty(x.shape, device=DEV)
    diopi.diopiRotaryEmbedding(ctx, out, x.to(DEV), torch.from_numpy(g["cos"]).to(DEV), torch.from_numpy(g["sin"]).to(DEV), False, False)
    np.testing.assert_allclose(out.cpu().numpy(), g["rotary_out"], rtol=1e-5, atol=1e-6)
    r = np.load(os.path.join(gold, "rotary.npz"))
    cos, sin = _tables(64, 16)
    q = torch.from_numpy(r["q"])  # [2, 16, 8, 64]
    o = torch.empty(q.shape, device=DEV)
    diopi.diopiRotaryEmbedding(ctx, o, q.to(DEV), cos.to(DEV), sin.to(DEV), False, True)
    np.testing.assert_allclose(o.cpu().numpy(), r["q_out"], rtol=1e-5, atol=1e-6)


# ---- fused steps of a decode iteration (include/diopi/functions_b200.h) -----------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(1, 4096), (64, 4096), (7, 512), (33, 8192)])
def test_add_rmsnorm_equals_the_two_calls(diopi, ctx, rows, cols):
    """diopiB200AddRMSNorm against diopiAdd followed by diopiRMSNorm: the same bits (it rounds where they round)."""
    x, r = rnd((rows, cols), torch.bfloat16, seed=rows), rnd((rows, cols), torch.bfloat16, seed=rows + 1)
    w = (1.0 + 0.1 * rnd((cols,), seed=2)).to(torch.bfloat16)
    xd, rd, wd = x.to(DEV), r.to(DEV), w.to(DEV)
    s1, n1 = torch.empty_like(xd), torch.empty_like(xd)
    diopi.diopiAdd(ctx, s1, xd, rd, 1)
    diopi.diopiRMSNorm(ctx, n1, None, s1, [cols], wd, None, 1e-6)
    s2, n2 = torch.empty_like(xd), torch.empty_like(xd)
    diopi.diopiB200AddRMSNorm(ctx, s2, n2, xd, rd, wd, 1e-6)
    assert torch.equal(s2, s1)
    assert torch.equal(s2.cpu(), (x.float() + r.float()).to(torch.bfloat16))
    sf = s1.float().cpu()
    check_bf16(n2, sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float())
    assert (n2.float() - n1.float()).abs().max().item() <= 2 ** -6 * n1.float().abs().max().item()   # at most one bf16 step apart
    # inputs that are row slices of wider tensors, no weight
    wide = rnd((rows, cols + 64), torch.bfloat16, seed=9).to(DEV)
    diopi.diopiB200AddRMSNorm(ctx, s2, n2, wide[:, :cols], rd, None, 1e-6)
    sf = (wide[:, :cols].float() + rd.float()).to(torch.bfloat16).float().cpu()
    assert torch.equal(s2.float().cpu(), sf)
    check_bf16(n2, sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-6))


@pytest.mark.parametrize("b,hq,hk,table_rows", [(4, 8, 8, 1), (64, 32, 32, 1), (6, 8, 2, 6), (3, 4, 1, 1)])
def test_rope_append_kv_equals_the_separate_calls(diopi, ctx, b, hq, hk, table_rows):
    """diopiB200RopeAppendKV against diopiRotaryEmbedding on q and k plus the two cache copies: the same bits, and nothing but
    slot `position` of the caches changes."""
    d, cap, pos = 128, 40, 17
    qkv = rnd((b, (hq + 2 * hk) * d), torch.bfloat16, seed=b)
    cos, sin = _tables(d, 64)
    cos, sin = cos[5:5 + table_rows].contiguous(), sin[5:5 + table_rows].contiguous()
    kc, vc = rnd((b, hk, cap, d), torch.bfloat16, seed=3), rnd((b, hk, cap, d), torch.bfloat16, seed=4)
    qd, kd, vd = qkv.to(DEV), kc.to(DEV), vc.to(DEV)
    q_out = torch.empty((b, hq, d), dtype=torch.bfloat16, device=DEV)
    diopi.diopiB200RopeAppendKV(ctx, q_out, qd, cos.to(DEV), sin.to(DEV), kd, vd, pos)
    q_in = qd[:, : hq * d].reshape(b, hq, d).contiguous()
    k_in = qd[:, hq * d:(hq + hk) * d].reshape(b, hk, d).contiguous()
    v_in = qkv[:, (hq + hk) * d:].reshape(b, hk, d)
    q_ref, k_ref = torch.empty_like(q_in), torch.empty_like(k_in)
    diopi.diopiRotaryEmbedding(ctx, q_ref, q_in, cos.to(DEV), sin.to(DEV), False, False)
    diopi.diopiRotaryEmbedding(ctx, k_ref, k_in, cos.to(DEV), sin.to(DEV), False, False)
    assert torch.equal(q_out, q_ref)
    assert torch.equal(kd[:, :, pos], k_ref)
    assert torch.equal(vd[:, :, pos].cpu(), v_in)
    keep = torch.ones(cap, dtype=torch.bool)
    keep[pos] = False
    assert torch.equal(kd.cpu()[:, :, keep], kc[:, :, keep]) and torch.equal(vd.cpu()[:, :, keep], vc[:, :, keep])
    # against the CPU arithmetic
    reps = b // table_rows
    c_, s_ = cos.repeat(reps, 1).view(b, 1, d // 2), sin.repeat(reps, 1).view(b, 1, d // 2)
    qf = q_in.float().cpu()
    x0, x1 = qf[..., : d // 2], qf[..., d // 2:]
    check_bf16(q_out, torch.cat((x0 * c_ - x1 * s_, x0 * s_ + x1 * c_), -1))
    with pytest.raises(diopi.DiopiError):
        diopi.diopiB200RopeAppendKV(ctx, q_out, qd, cos.to(DEV), sin.to(DEV), kd, vd, cap)   # no such slot


@pytest.mark.parametrize("m,k,f", [(64, 4096, 11008), (1, 512, 1376), (128, 1024, 344), (5, 264, 72)])
def test_mm_swiglu_against_the_separate_calls(diopi, ctx, m, k, f):
    """diopiB200MmSwiGLU over the interleaved gate / up weight against fp32 CPU (stated tolerance) and against the op-by-op
    device sequence mm, mm, silu, mul (which rounds four times where the fused form rounds once)."""
    x = rnd((m, k), torch.bfloat16, seed=m)
    w1, w3 = rnd((f, k), torch.bfloat16, seed=1, scale=k ** -0.5), rnd((f, k), torch.bfloat16, seed=2, scale=k ** -0.5)
    w13 = torch.stack([w1, w3], dim=1).reshape(2 * f, k).contiguous()
    xd = x.to(DEV)
    out = torch.empty((m, f), dtype=torch.bfloat16, device=DEV)
    diopi.diopiB200MmSwiGLU(ctx, out, xd, w13.to(DEV).t())
    g, u = x.float() @ w1.float().t(), x.float() @ w3.float().t()
    want = torch.nn.functional.silu(g) * u
    check_bf16(out, want, max_abs=2e-2 * max(1.0, want.abs().max().item()))   # outputs reach |10|: the bound follows the magnitude
    gd, ud = torch.empty((m, f), dtype=torch.bfloat16, device=DEV), torch.empty((m, f), dtype=torch.bfloat16, device=DEV)
    diopi.diopiMm(ctx, gd, xd, w1.to(DEV).t())
    diopi.diopiMm(ctx, ud, xd, w3.to(DEV).t())
    diopi.diopiSiluInp(ctx, gd)
    diopi.diopiMulInp(ctx, gd, ud)
    step = gd.float().cpu()
    check_bf16(out, step, max_abs=3 * 2.0 ** -8 * max(1.0, step.abs().max().item()), rel_l2=5e-3)   # a few bf16 steps at the largest magnitude
    assert diopi.gemm_status() == 0
    with pytest.raises(diopi.DiopiError):
        diopi.diopiB200MmSwiGLU(ctx, torch.empty((200, f), dtype=torch.bfloat16, device=DEV), rnd((200, k), torch.bfloat16).to(DEV), w13.to(DEV).t())


def test_error_reporting(diopi, ctx):
    a = torch.empty((3, 4), device=DEV)
    b = torch.empty((5, 4), device=DEV)
    with pytest.raises(diopi.DiopiError) as e:
        diopi.diopiAdd(ctx, a, a, b, 1)
    assert "broadcast" in str(e.value)
    with pytest.raises(diopi.DiopiError):
        diopi.diopiSoftmax(ctx, a, a, 5)
    with pytest.raises(diopi.DiopiError):
        diopi.diopiIndexSelect(ctx, a, a, 0, torch.zeros(3, device=DEV))  # float index
    assert math.isfinite(0.0)
