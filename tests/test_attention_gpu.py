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


@pytest.mark.parametrize("b,length,h,hk", [(4, 300, 8, 8), (3, 1000, 8, 2), (2, 129, 8, 4), (1, 5000, 2, 2), (2, 1, 4, 4), (5, 33, 6, 2),
                                           (1, 20000, 8, 1)])
def test_decode_attention(pkg, ctx, b, length, h, hk):
    """One query per sequence against a cache kept as [B, kv heads, capacity, D]: the kernel takes the [B, L, kv heads, D]
    view of the filled part by its pitches. Few sequences exercise the split over keys and the merge kernel."""
    cap = length + 17
    q, k, v = _inputs(b, 1, cap, h, hk, 128, seed=length + h, dtype=torch.bfloat16)
    kc = k.transpose(1, 2).contiguous().to(DEV)   # [B, hk, cap, D]
    vc = v.transpose(1, 2).contiguous().to(DEV)
    kd = kc[:, :, :length, :].transpose(1, 2)
    vd = vc[:, :, :length, :].transpose(1, 2)
    _check(pkg, ctx, q, k[:, :length], v[:, :length], False, q.to(DEV), kd, vd)


def test_decode_attention_fp16_causal_flag(pkg, ctx):
    """With one query the causal flag changes nothing: every cached key is visible."""
    q, k, v = _inputs(3, 1, 700, 4, 4, 128, seed=2, dtype=torch.float16)
    _check(pkg, ctx, q, k, v, True, q.to(DEV), k.to(DEV), v.to(DEV))


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


def test_attention_against_reference_golden(pkg, ctx):
    """Inputs and outputs recorded from the reference's own fused operators (ext_ops.py:66-86,100-126): the inputs are
    exactly representable in bf16, so only the kernel's arithmetic differs."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ext_attention.npz"))
    seq, heads, dim = 160, 4, 128
    bf = torch.bfloat16
    q, k, v = (torch.from_numpy(g[n]).view(1, seq, heads, dim).to(bf).to(DEV) for n in ("prompt_q", "prompt_k", "prompt_v"))
    out = torch.empty_like(q)
    pkg.diopi.diopiMultiHeadAttention(ctx, q, k, v, 0.0, True, False, dim ** -0.5, out, None, None, None)
    ref = torch.from_numpy(g["prompt_out"])
    got = out[0].float().cpu()
    assert (got - ref).abs().max().item() <= 2e-2 and ((got - ref).norm() / ref.norm()).item() <= 5e-3
    fq, fk, fv = (torch.from_numpy(g[n]).to(bf).to(DEV) for n in ("flash_q", "flash_k", "flash_v"))
    for i, length in enumerate(g["flash_lens"]):
        length = int(length)
        o = torch.empty(1, 1, heads, dim, dtype=bf, device=DEV)
        pkg.diopi.diopiMultiHeadAttention(ctx, fq[i].view(1, 1, heads, dim), fk[:length].view(1, length, heads, dim),
                                          fv[:length].view(1, length, heads, dim), 0.0, False, False, dim ** -0.5, o, None, None, None)
        ref = torch.from_numpy(g["flash_out"][i])
        got = o.view(heads, dim).float().cpu()
        assert (got - ref).abs().max().item() <= 2e-2 and ((got - ref).norm() / ref.norm()).item() <= 5e-3
    torch.cuda.synchronize()
    assert pkg.diopi.gemm_status() == 0


def test_prefill_attention_two_threads_per_row_variant(pkg):
    """The non-default kernel variant (two threads per query row, selected by B200_ATTN_ROW_SPLIT=2 when the library first
    launches the kernel) in a child process: same parity bar."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import sys, math, numpy as np, torch\n"
        "sys.path.insert(0, %r)\n"
        "import __graft_entry__ as e\n"
        "from oracle import llama_cpu\n"
        "pkg = e.load_package(); ctx = pkg.diopi.Context()\n"
        "rng = np.random.default_rng(1)\n"
        "for (b, sq, skv, h, hk, causal) in [(2, 640, 640, 4, 2, True), (1, 200, 457, 2, 2, False), (1, 300, 300, 2, 1, True)]:\n"
        "    q, k, v = (torch.from_numpy(rng.standard_normal(s, dtype=np.float32)).to(torch.bfloat16) for s in ((b, sq, h, 128), (b, skv, hk, 128), (b, skv, hk, 128)))\n"
        "    ref, lse_ref = llama_cpu.fused_attention(q, k, v, causal)\n"
        "    out = torch.empty(q.shape, dtype=q.dtype, device='cuda:0'); lse = torch.empty(b, h, sq, device='cuda:0')\n"
        "    pkg.diopi.diopiMultiHeadAttention(ctx, q.cuda(), k.cuda(), v.cuda(), 0.0, causal, False, 128 ** -0.5, out, lse, None, None)\n"
        "    torch.cuda.synchronize()\n"
        "    got = out.float().cpu()\n"
        "    assert (got - ref).abs().max().item() <= 2e-2 and ((got - ref).norm() / ref.norm()).item() <= 5e-3\n"
        "    torch.testing.assert_close(lse.cpu(), lse_ref, rtol=1e-4, atol=2e-3)\n"
        "assert pkg.diopi.gemm_status() == 0\n"
        "print('variant ok')\n" % root)
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, B200_ATTN_ROW_SPLIT="2"), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "variant ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
