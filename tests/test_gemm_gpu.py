"""Dense contractions through the DIOPI C-ABI against torch CPU.

Small fp32 cases are the reference's own unit-test shapes (dipu/tests/python/unittests/test_mm.py:8-15,
test_bmm.py:8-15, test_addmm.py:55-69, test_matmul.py:15-71, test_linear.py:33-70) at their tolerances; bf16 cases
cover the tcgen05 kernel (both B layouts, ragged edges, batches, every tile width) and the skinny decode kernels with
the stated bf16 tolerance (max-abs <= 2e-2 scaled to the output magnitude, rel-L2 <= 5e-3 vs fp32 CPU).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(shape, dtype=torch.float32, seed=0, scale=1.0):
    rng = np.random.default_rng(seed)
    return (torch.from_numpy(rng.standard_normal(size=shape, dtype=np.float32)) * scale).to(dtype)


def check_lowp(got, ref, rel_l2=5e-3, max_rel=2e-2):
    got = got.float().cpu()
    scale = ref.abs().max().clamp_min(1e-6).item()
    err = (got - ref).abs().max().item() / scale
    rel = ((got - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    assert err <= max_rel and rel <= rel_l2, "max_err/scale=%g rel_l2=%g" % (err, rel)


def test_mm_bmm_fp32_reference_shapes(diopi, ctx):
    a, b = rnd((2, 3), seed=1), rnd((3, 4), seed=2)
    out = torch.empty((2, 4), device=DEV)
    diopi.diopiMm(ctx, out, a.to(DEV), b.to(DEV))
    np.testing.assert_allclose(out.cpu().numpy(), (a @ b).numpy(), rtol=1e-5, atol=1e-5)
    x, y = rnd((3, 3, 2), seed=3), rnd((3, 2, 4), seed=4)
    o = torch.empty((3, 3, 4), device=DEV)
    diopi.diopiBmm(ctx, o, x.to(DEV), y.to(DEV))
    np.testing.assert_allclose(o.cpu().numpy(), torch.bmm(x, y).numpy(), rtol=1e-5, atol=1e-5)
    # fp32 at layer sizes of the CPU configuration (T=128, 512 -> 1376), transposed-view weight
    h, w = rnd((128, 512), seed=5), rnd((1376, 512), seed=6, scale=0.02)
    o2 = torch.empty((128, 1376), device=DEV)
    diopi.diopiMm(ctx, o2, h.to(DEV), w.to(DEV).t())
    np.testing.assert_allclose(o2.cpu().numpy(), (h @ w.t()).numpy(), rtol=1e-4, atol=1e-5)
    d = rnd((5, 7), seed=7).double()
    e = rnd((7, 3), seed=8).double()
    o3 = torch.empty((5, 3), dtype=torch.float64, device=DEV)
    diopi.diopiMm(ctx, o3, d.to(DEV), e.to(DEV))
    np.testing.assert_allclose(o3.cpu().numpy(), (d @ e).numpy(), rtol=1e-12)


def test_addmm_baddbmm_reference_shapes(diopi, ctx):
    bias, m1, m2 = rnd((3, 3), seed=1), rnd((3, 5), seed=2), rnd((5, 3), seed=3)
    out = torch.empty((3, 3), device=DEV)
    diopi.diopiAddmm(ctx, out, bias.to(DEV), m1.to(DEV), m2.to(DEV), 0.7, 1.3)
    np.testing.assert_allclose(out.cpu().numpy(), torch.addmm(bias, m1, m2, beta=0.7, alpha=1.3).numpy(), rtol=1e-4, atol=1e-5)
    # mat2 given as a transposed view, bias broadcast from [3]
    m3 = rnd((3, 5), seed=4)
    b1 = rnd((3,), seed=5)
    diopi.diopiAddmm(ctx, out, b1.to(DEV), m1.to(DEV), m3.to(DEV).t(), 1, 1)
    np.testing.assert_allclose(out.cpu().numpy(), torch.addmm(b1, m1, m3.t()).numpy(), rtol=1e-4, atol=1e-5)
    x, y, z = rnd((4, 3, 6), seed=6), rnd((4, 3, 5), seed=7), rnd((4, 5, 6), seed=8)
    o = torch.empty((4, 3, 6), device=DEV)
    diopi.diopiBaddbmm(ctx, o, x.to(DEV), y.to(DEV), z.to(DEV), 0.5, 2.0)
    np.testing.assert_allclose(o.cpu().numpy(), torch.baddbmm(x, y, z, beta=0.5, alpha=2.0).numpy(), rtol=1e-4, atol=1e-5)


def test_matmul_folding_and_linear(diopi, ctx):
    cases = [((4,), (4,)), ((3, 4), (4,)), ((10, 3, 4), (4,)), ((10, 3, 4), (10, 4, 5)), ((10, 3, 4), (4, 5)), ((20, 10, 3, 4), (4, 5)),
             ((20, 10, 3, 4), (10, 4, 5)), ((4,), (4, 10)), ((3, 4), (4, 5))]
    for i, (sa, sb) in enumerate(cases):
        a, b = rnd(sa, seed=i), rnd(sb, seed=100 + i)
        ref = torch.matmul(a, b)
        out = torch.empty(ref.shape, device=DEV)
        diopi.diopiMatmul(ctx, out, a.to(DEV), b.to(DEV))
        np.testing.assert_allclose(out.cpu().numpy(), ref.numpy(), rtol=1e-3, atol=1e-4, err_msg=str((sa, sb)))
    for shape in ((3,), (2, 3), (2, 2, 3), (2, 1, 2, 3)):
        x, w, b = rnd(shape, seed=1), torch.ones(2, 3), rnd((2,), seed=2)
        ref = torch.nn.functional.linear(x, w, b)
        out = torch.empty(ref.shape, device=DEV)
        diopi.diopiLinear(ctx, out, x.to(DEV), w.to(DEV), b.to(DEV))
        np.testing.assert_allclose(out.cpu().numpy(), ref.numpy(), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (300, 264, 136), (1024, 4096, 512), (64, 4096, 4096), (64, 64, 4096),
                                   (130, 40, 72), (2048, 11008, 512)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_tc_mm_kmajor_weight(diopi, ctx, m, n, k, dtype):
    """mm(x, W.t()): B arrives as the transposed view of an [N, K] weight (K contiguous)."""
    if dtype == torch.float16 and m > 300:
        pytest.skip("fp16 covered by the small shapes")
    x, w = rnd((m, k), dtype, seed=m + n), rnd((n, k), dtype, seed=k, scale=0.05)
    out = torch.empty((m, n), dtype=dtype, device=DEV)
    diopi.diopiMm(ctx, out, x.to(DEV), w.to(DEV).t())
    check_lowp(out, x.float() @ w.float().t())
    assert diopi.gemm_status() == 0


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 320, 200), (512, 4096, 1024), (77, 72, 40)])
def test_tc_mm_nmajor(diopi, ctx, m, n, k):
    """mm(a, b) with a plain row-major [K, N] B (N contiguous)."""
    a, b = rnd((m, k), torch.bfloat16, seed=1), rnd((k, n), torch.bfloat16, seed=2, scale=0.05)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    diopi.diopiMm(ctx, out, a.to(DEV), b.to(DEV))
    check_lowp(out, a.float() @ b.float())
    # fp32 output from bf16 operands
    o32 = torch.empty((m, n), dtype=torch.float32, device=DEV)
    diopi.diopiMm(ctx, o32, a.to(DEV), b.to(DEV))
    check_lowp(o32, a.float() @ b.float(), rel_l2=1e-4, max_rel=1e-4)
    assert diopi.gemm_status() == 0


@pytest.mark.parametrize("m,n,k,nk", [(64, 4096, 4096, True), (64, 11008, 4096, True), (64, 4096, 11008, True), (16, 512, 4096, True),
                                      (100, 1376, 512, True), (128, 264, 72, True), (64, 4096, 1024, False), (33, 136, 200, False),
                                      (64, 64, 4096, True), (8, 4096, 328, False)])
def test_tc_split_k_single_row_block(diopi, ctx, m, n, k, nk):
    """M <= 128 (decode): a cluster of CTAs splits K and sums the partial tiles through distributed shared memory."""
    a = rnd((m, k), torch.bfloat16, seed=m + k)
    b = rnd((n, k) if nk else (k, n), torch.bfloat16, seed=n, scale=0.05)
    ref = a.float() @ (b.float().t() if nk else b.float())
    bd = b.to(DEV)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    diopi.diopiMm(ctx, out, a.to(DEV), bd.t() if nk else bd)
    check_lowp(out, ref)
    # deterministic: a second run gives the same bits
    out2 = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    diopi.diopiMm(ctx, out2, a.to(DEV), bd.t() if nk else bd)
    assert torch.equal(out, out2)
    # bias / scale epilogue and fp32 output
    bias = rnd((n,), torch.float32, seed=5)
    o32 = torch.empty((m, n), dtype=torch.float32, device=DEV)
    diopi.diopiAddmm(ctx, o32, bias.to(DEV), a.to(DEV), bd.t() if nk else bd, 0.5, 2.0)
    check_lowp(o32, 0.5 * bias + 2.0 * ref, rel_l2=1e-4, max_rel=1e-4)
    assert diopi.gemm_status() == 0


@pytest.mark.parametrize("m,n,k,nk,batch", [(2048, 4096, 512, True, 1), (3000, 2600, 264, True, 1), (2048, 4096, 320, False, 1),
                                            (1000, 4136, 256, False, 1), (512, 512, 256, True, 40), (512, 640, 256, False, 24),
                                            (2048, 4096, 1024, True, 1), (2304, 2816, 584, False, 1)])
def test_tc_cta_pair_tiles(diopi, ctx, m, n, k, nk, batch):
    """Products large enough for the CTA-pair kernel (256 x 256 tiles over two SMs): ragged edges, both B layouts, batches,
    scaled / biased epilogue, fp32 output. K up to 512 takes the instantiation with eight epilogue warps per CTA (short K
    loops), the longer ones the one with four."""
    shape_a = (batch, m, k) if batch > 1 else (m, k)
    shape_b = ((batch, n, k) if nk else (batch, k, n)) if batch > 1 else ((n, k) if nk else (k, n))
    a = rnd(shape_a, torch.bfloat16, seed=m + k)
    b = rnd(shape_b, torch.bfloat16, seed=n, scale=0.05)
    bt = b.float().transpose(-1, -2) if nk else b.float()
    ref = torch.matmul(a.float(), bt)
    ad, bd = a.to(DEV), b.to(DEV)
    bv = bd.transpose(-1, -2) if nk else bd
    out = torch.empty(ref.shape, dtype=torch.bfloat16, device=DEV)
    if batch > 1:
        diopi.diopiBmm(ctx, out, ad, bv)
    else:
        diopi.diopiMm(ctx, out, ad, bv)
    check_lowp(out, ref)
    if batch == 1:
        bias = rnd((m, n), torch.float32, seed=7)
        o32 = torch.empty((m, n), dtype=torch.float32, device=DEV)
        diopi.diopiAddmm(ctx, o32, bias.to(DEV), ad, bv, 0.5, 2.0)
        check_lowp(o32, 0.5 * bias + 2.0 * ref, rel_l2=1e-4, max_rel=1e-4)
    else:
        mask = rnd((m, n), torch.bfloat16, seed=8)
        ob = torch.empty(ref.shape, dtype=torch.bfloat16, device=DEV)
        diopi.diopiBaddbmm(ctx, ob, mask.to(DEV), ad, bv, 1.0, 0.25)
        check_lowp(ob, mask.float() + 0.25 * ref)
    assert diopi.gemm_status() == 0


def test_tc_linearity_and_identity(diopi, ctx):
    """Size-independent properties at a large shape: A*I == A bit for bit, and (A1 + A2)*B == A1*B + A2*B within rounding."""
    m, n = 4096, 4096
    a = rnd((m, n), torch.bfloat16, seed=3).to(DEV)
    eye = torch.eye(n, dtype=torch.bfloat16, device=DEV)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    diopi.diopiMm(ctx, out, a, eye)
    assert torch.equal(out, a)
    diopi.diopiMm(ctx, out, a, eye.t())
    assert torch.equal(out, a)
    assert diopi.gemm_status() == 0


def test_tc_bmm_attention_shapes(diopi, ctx):
    """Q*K^T (B given as a transposed view: K-major) and P*V (N-major) with prefill-like batches."""
    bh, s, d = 24, 256, 128
    q, k, v = rnd((bh, s, d), torch.bfloat16, seed=1), rnd((bh, s, d), torch.bfloat16, seed=2), rnd((bh, s, d), torch.bfloat16, seed=3)
    scores = torch.empty((bh, s, s), dtype=torch.bfloat16, device=DEV)
    diopi.diopiBmm(ctx, scores, q.to(DEV), k.to(DEV).transpose(1, 2))
    check_lowp(scores, torch.bmm(q.float(), k.float().transpose(1, 2)))
    p = torch.softmax(rnd((bh, s, s), torch.float32, seed=4), -1).to(torch.bfloat16)
    av = torch.empty((bh, s, d), dtype=torch.bfloat16, device=DEV)
    diopi.diopiBmm(ctx, av, p.to(DEV), v.to(DEV))
    check_lowp(av, torch.bmm(p.float(), v.float()))
    # ragged sequence length and head dim 64
    q2, k2 = rnd((5, 100, 64), torch.bfloat16, seed=5), rnd((5, 136, 64), torch.bfloat16, seed=6)
    s2 = torch.empty((5, 100, 136), dtype=torch.bfloat16, device=DEV)
    diopi.diopiBmm(ctx, s2, q2.to(DEV), k2.to(DEV).transpose(1, 2))
    check_lowp(s2, torch.bmm(q2.float(), k2.float().transpose(1, 2)))
    assert diopi.gemm_status() == 0


def test_tc_addmm_epilogue(diopi, ctx):
    m, n, k = 256, 384, 128
    a, w = rnd((m, k), torch.bfloat16, seed=1), rnd((n, k), torch.bfloat16, seed=2, scale=0.1)
    bias = rnd((n,), torch.bfloat16, seed=3)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    diopi.diopiAddmm(ctx, out, bias.to(DEV), a.to(DEV), w.to(DEV).t(), 1, 1)
    check_lowp(out, bias.float() + a.float() @ w.float().t())
    full = rnd((m, n), torch.bfloat16, seed=4)
    diopi.diopiAddmm(ctx, out, full.to(DEV), a.to(DEV), w.to(DEV).t(), 0.5, 2.0)
    check_lowp(out, 0.5 * full.float() + 2.0 * (a.float() @ w.float().t()))
    assert diopi.gemm_status() == 0


@pytest.mark.parametrize("m", [1, 2, 4, 8])
@pytest.mark.parametrize("length", [513, 512])
def test_decode_attention_few_rows(diopi, ctx, m, length):
    """q*K^T and p*V over a KV cache, [B*h, m, D] x [B*h, D, L] and [B*h, m, L] x [B*h, L, D], cache slices with a capacity stride.
    Length 512 meets the TMA rules (tensor-core kernel); 513 makes the probability rows unaligned (skinny / general kernels)."""
    bh, cap, d = 48, 640, 128
    kc, vc = rnd((bh, cap, d), torch.bfloat16, seed=1), rnd((bh, cap, d), torch.bfloat16, seed=2)
    q = rnd((bh, m, d), torch.bfloat16, seed=3)
    kd, vd = kc.to(DEV), vc.to(DEV)
    scores = torch.empty((bh, m, length), dtype=torch.bfloat16, device=DEV)
    diopi.diopiBmm(ctx, scores, q.to(DEV), kd[:, :length].transpose(1, 2))
    check_lowp(scores, torch.bmm(q.float(), kc[:, :length].float().transpose(1, 2)))
    p = torch.softmax(rnd((bh, m, length), torch.float32, seed=4), -1).to(torch.bfloat16)
    out = torch.empty((bh, m, d), dtype=torch.bfloat16, device=DEV)
    diopi.diopiBmm(ctx, out, p.to(DEV), vd[:, :length])
    check_lowp(out, torch.bmm(p.float(), vc[:, :length].float()))


def test_gemm_errors(diopi, ctx):
    a = torch.empty((3, 4), device=DEV)
    b = torch.empty((5, 6), device=DEV)
    out = torch.empty((3, 6), device=DEV)
    with pytest.raises(diopi.DiopiError) as e:
        diopi.diopiMm(ctx, out, a, b)
    assert "inner" in str(e.value)
    with pytest.raises(diopi.DiopiError):
        diopi.diopiMm(ctx, out, a, torch.empty((4, 6), dtype=torch.bfloat16, device=DEV))
    empty = torch.empty((0, 6), device=DEV)
    diopi.diopiMm(ctx, empty, torch.empty((0, 4), device=DEV), torch.empty((4, 6), device=DEV))
