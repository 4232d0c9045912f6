"""Fused attention (diopiMultiHeadAttention) on the GPU against the CPU restatement of the reference's fused operator."""
import math

import numpy as np
import pytest
import torch

from oracle import llama_cpu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(b, sq, skv, h, hk, d, seed, dtype):
    rng = np.random.default_rng(seed)
    q = torch.from_numpy(rng.standard_normal((b, sq, h, d), dtype=np.float32)).to(dtype)
    k = torch.from_numpy(rng.standard_normal((b, skv, hk, d), dtype=np.float32)).to(dtype)
    v = torch.from_numpy(rng.standard_normal((b, skv, hk, d), dtype=np.float32)).to(dtype)
    return q, k, v


def _check(pkg, ctx, q, k, v, causal, qd, kd, vd, lse=True, scale=None):
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    ref, ref_lse = llama_cpu.fused_attention(q, k, v, causal, scale)
    out = torch.full(q.shape, float("nan"), dtype=q.dtype, device=DEV)
    lse_d = torch.empty(q.shape[0], q.shape[2], q.shape[1], dtype=torch.float32, device=DEV) if lse else None
    pkg.diopi.diopiMultiHeadAttention(ctx, qd, kd, vd, 0.0, causal, False, scale, out, lse_d, None, None)
    torch.cuda.synchronize()
    assert pkg.diopi.gemm_status() == 0
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    # probabilities are rounded to the operand type before the second product, like the op-by-op path: bf16 tolerance of
    # the layer (max-abs 2e-2, relative L2 5e-3) against the fp32 CPU result computed from the same rounded inputs
    max_abs = (got - ref).abs().max().item()
    rel = ((got - ref).norm() / ref.norm()).item()
    assert max_abs <= 2e-2 and rel <= 5e-3, (max_abs, rel)
    if lse:
        torch.testing.assert_close(lse_d.cpu(), ref_lse, rtol=1e-4, atol=2e-3)
    return out


@pytest.mark.parametrize("b,s,h,hk", [(2, 512, 4, 4), (1, 1024, 8, 2), (3, 256, 2, 1)])
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_attention(pkg, ctx, b, s, h, hk, causal):
    q, k, v = _inputs(b, s, s, h, hk, 128, seed=5 + s, dtype=torch.bfloat16)
    _check(pkg, ctx, q, k, v, causal, q.to(DEV), k.to(DEV), v.to(DEV))


@pytest.mark.parametrize("sq,skv", [(300, 300), (77, 77), (1, 129), (128, 384), (200, 457), (257, 640)])
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_attention_ragged(pkg, ctx, sq, skv, causal):
    """Lengths that are no multiple of the 128-row tiles; more keys than queries (causal mask aligned to the last key)."""
    q, k, v = _inputs(2, sq, skv, 4, 2, 128, seed=sq * 7 + skv, dtype=torch.bfloat16)
    _check(pkg, ctx, q, k, v, causal, q.to(DEV), k.to(DEV), v.to(DEV))


def test_prefill_attention_strided_views_fp16(pkg, ctx):
    """q, k, v as views of one fused [B, S, (H + 2 Hk) * D] projection output and out as a view of a wider buffer: taken as
    they are, without copies."""
    b, s, h, hk, d = 2, 384, 4, 2, 128
    q, k, v = _inputs(b, s, s, h, hk, d, seed=11, dtype=torch.float16)
    fused = torch.cat([q.reshape(b, s, h * d), k.reshape(b, s, hk * d), v.reshape(b, s, hk * d)], dim=-1).to(DEV)
    qd = fused[:, :, :h * d].view(b, s, h, d)
    kd = fused[:, :, h * d:(h + hk) * d].view(b, s, hk, d)
    vd = fused[:, :, (h + hk) * d:].view(b, s, hk, d)
    assert not qd.is_contiguous()
    _check(pkg, ctx, q, k, v, True, qd, kd, vd, lse=False)


def test_prefill_attention_twice_same_result(pkg, ctx):
    q, k, v = _inputs(2, 640, 640, 4, 4, 128, seed=3, dtype=torch.bfloat16)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    a = _check(pkg, ctx, q, k, v, True, qd, kd, vd)
    b = _check(pkg, ctx, q, k, v, True, qd, kd, vd)
    assert torch.equal(a, b)


def test_prefill_attention_large_scores(pkg, ctx):
    """Scores that grow along the key axis force the running maximum to move (the accumulator rescale path)."""
    b, s, h, d = 1, 512, 2, 128
    q, k, v = _inputs(b, s, s, h, h, d, seed=9, dtype=torch.bfloat16)
    ramp = torch.linspace(0.2, 6.0, s).view(1, s, 1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    _check(pkg, ctx, q, k, v, False, q.to(DEV), k.to(DEV), v.to(DEV), scale=0.5)


def test_attention_rejects_what_it_cannot_run(pkg, ctx):
    q = torch.zeros(1, 16, 2, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(pkg.diopi.DiopiError, match="head dim 128"):
        pkg.diopi.diopiMultiHeadAttention(ctx, q, q, q, 0.0, True, False, 0.125, torch.empty_like(q), None, None, None)
    q = torch.zeros(1, 16, 3, 128, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(1, 16, 2, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(pkg.diopi.DiopiError, match="cannot share"):
        pkg.diopi.diopiMultiHeadAttention(ctx, q, k, k, 0.0, True, False, 0.1, torch.empty_like(q), None, None, None)
    with pytest.raises(pkg.diopi.DiopiError, match="dropout"):
        pkg.diopi.diopiMultiHeadAttention(ctx, k, k, k, 0.1, True, False, 0.1, torch.empty_like(k), None, None, None)
