"""CPU oracle for the decoder-layer hot path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may import this module; the product
(deeplink.framework_b200/) never does.

What it restates: DIPU's forced CPU fallback executes every op with torch's CPU aten kernels
(dipu/torch_dipu/csrc_dipu/aten/CPUFallback.cpp:130 redispatches the boxed op to DispatchKey::CPU), so the oracle is
torch CPU arithmetic, written as the op sequence of the reference's own Llama block:

    RMSNorm        dicp/test/model/llama/model.py:28-39   (x.float() -> x * rsqrt(mean(x^2) + eps) -> * weight)
    rotary (pairs) dicp/test/model/llama/model.py:58-69   (complex multiply on interleaved pairs)
    rotary (halves) dicp/dicp/vendor/AscendGraph/ext_ops.py:24-33 (x0 * cos - x1 * sin | x0 * sin + x1 * cos)
    attention      dicp/test/model/llama/model.py:146-155 (matmul / sqrt(d) + mask -> softmax(float) -> matmul)
    SwiGLU         dicp/test/model/llama/model.py:174-175 (w2(silu(w1 x) * w3 x))
    block          dicp/test/model/llama/model.py:193-201 (two residual adds)

Pinning: tests/golden/ holds outputs of the reference's own TransformerBlock / RMSNorm / apply_rotary_emb, produced by
importing dicp/test/model/llama/model.py unmodified (tests/golden/make_golden.py); tests/test_oracle.py checks this
module against them. The reference stores no golden vectors of its own for this path.

All tensors are float32 unless a function says otherwise. Parameters come from numpy's PCG64 generator so that the
same seed gives the same values wherever the tests run.
"""
import dataclasses
import math

import numpy as np
import torch


@dataclasses.dataclass
class LayerConfig:
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 32
    head_dim: int = 128
    ffn: int = 11008
    eps: float = 1e-6
    rope_base: float = 10000.0
    rope_layout: str = "half"  # "half": pairs (i, i + d/2);  "interleaved": pairs (2i, 2i+1)


def _normal(rng, shape, std):
    return torch.from_numpy((rng.standard_normal(size=shape, dtype=np.float32) * np.float32(std)))


def make_weights(cfg, seed=1234):
    """N(0, 0.02) projection weights in nn.Linear layout [out_features, in_features]; norm weights are ones."""
    rng = np.random.default_rng(seed)
    h, d = cfg.hidden, cfg.head_dim
    return {
        "wq": _normal(rng, (cfg.heads * d, h), 0.02),
        "wk": _normal(rng, (cfg.kv_heads * d, h), 0.02),
        "wv": _normal(rng, (cfg.kv_heads * d, h), 0.02),
        "wo": _normal(rng, (h, cfg.heads * d), 0.02),
        "w1": _normal(rng, (cfg.ffn, h), 0.02),  # gate
        "w3": _normal(rng, (cfg.ffn, h), 0.02),  # up
        "w2": _normal(rng, (h, cfg.ffn), 0.02),  # down
        "attention_norm": torch.ones(h),
        "ffn_norm": torch.ones(h),
    }


def make_embedding(vocab, hidden, seed=1234):
    rng = np.random.default_rng(seed + 1)
    return _normal(rng, (vocab, hidden), 0.02)


def make_token_ids(batch, seq, seed=1234, vocab=32000):
    rng = np.random.default_rng(seed + 2)
    return torch.from_numpy(rng.integers(0, vocab, size=(batch, seq), dtype=np.int64))


def make_kv_cache(cfg, batch, length, seed=1234):
    """N(0,1) cache in [batch, kv_heads, length, head_dim] layout."""
    rng = np.random.default_rng(seed + 3)
    shape = (batch, cfg.kv_heads, length, cfg.head_dim)
    return _normal(rng, shape, 1.0), _normal(rng, shape, 1.0)


def round_tensor(t, dtype):
    """The value a tensor has after being stored in `dtype`, as float32."""
    return t.to(dtype).to(torch.float32)


def round_weights(weights, dtype):
    return {k: round_tensor(v, dtype) for k, v in weights.items()}


# ---- single ops -----------------------------------------------------------------------------------------------
def rms_norm(x, weight, eps):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def rope_tables(head_dim, positions, base=10000.0):
    """cos, sin of shape [len(positions), head_dim/2] (float32), angle[p, i] = p * base^(-2i/d)."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    ang = torch.outer(positions.float(), inv).float()
    return torch.cos(ang), torch.sin(ang)


def rotary_half(x, cos, sin):
    """x [tokens, heads, d]; cos/sin [tokens or seq, d/2]; rows repeat over the leading (batch) part of tokens."""
    t, h, d = x.shape
    reps = t // cos.shape[0]
    c = cos.repeat(reps, 1).view(t, 1, d // 2)
    s = sin.repeat(reps, 1).view(t, 1, d // 2)
    x0, x1 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat((x0 * c - x1 * s, x0 * s + x1 * c), dim=-1)


def rotary_interleaved(x, cos, sin):
    t, h, d = x.shape
    reps = t // cos.shape[0]
    f = torch.polar(torch.ones_like(cos), torch.atan2(sin, cos)).repeat(reps, 1).view(t, 1, d // 2)
    xc = torch.view_as_complex(x.float().reshape(t, h, d // 2, 2))
    return torch.view_as_real(xc * f).flatten(2)


def rotary(cfg, x, cos, sin):
    return rotary_half(x, cos, sin) if cfg.rope_layout == "half" else rotary_interleaved(x, cos, sin)


def causal_mask(seq):
    m = torch.full((seq, seq), float("-inf"))
    return torch.triu(m, diagonal=1)


def _expand_kv(cfg, t):
    """[B, kv_heads, S, D] -> [B, heads, S, D] (grouped-query attention: each KV head serves heads/kv_heads query heads)."""
    g = cfg.heads // cfg.kv_heads
    return t if g == 1 else t.repeat_interleave(g, dim=1)


def fused_attention(q, k, v, causal, scale=None):
    """The fused attention operator restated on CPU in fp32: q [B, Sq, H, D], k / v [B, Skv, Hkv, D] -> [B, Sq, H, D].
    Follows dicp/dicp/vendor/AscendGraph/ext_ops.py:52-86 (prompt_attention_inference: scores / sqrt(d), additive
    causal mask, softmax, times V, heads of a group sharing K / V) and dicp/test/model/llama/model.py:146-150.
    With Sq != Skv the causal mask is aligned to the last key: key j is visible to query i iff j <= i + Skv - Sq
    (ext_ops.py:89-126, flash_attention_inference, is the Sq = 1 case: every cached key is visible).
    Returns (out, lse) with lse [B, H, Sq] the natural log of the softmax denominator."""
    b, sq, h, d = q.shape
    skv, hk = k.shape[1], k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(h // hk, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(h // hk, dim=1)
    scores = torch.matmul(qf, kf.transpose(2, 3)) * scale
    if causal:
        i = torch.arange(sq).view(sq, 1)
        j = torch.arange(skv).view(1, skv)
        scores = scores.masked_fill(j > i + (skv - sq), float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    out = torch.matmul(torch.softmax(scores, dim=-1), vf).transpose(1, 2).contiguous()
    return out, lse


# ---- the layer --------------------------------------------------------------------------------------------------------
# `step` is applied wherever the eager op stream materialises a tensor. The identity gives the fp32 oracle. Rounding to
# bf16 there (step=stepwise(torch.bfloat16)) gives what the reference's literal CPU fallback produces on bf16 tensors:
# its custom fallbacks up-cast fp16 only, so every op reads and writes bf16
# (dipu/torch_dipu/csrc_dipu/aten/ops/CustomFallbackFunctions.hpp:23-30) while computing in fp32 internally.
def _identity(t):
    return t


def stepwise(dtype):
    return lambda t: t.to(dtype).to(torch.float32)


def row_parallel(x, weight, step=_identity, tp=1, residual=None):
    """x @ weight.t() the way `tp` tensor-parallel ranks compute a row-parallel linear (wo, w2): the contraction is cut into tp
    contiguous slices, every rank materialises its partial product (`step`), and the all-reduce sums the partials and materialises
    the sum (DIPU's caller: ProcessGroupDICL::allreduce on the bf16 partial sums,
    dipu/torch_dipu/csrc_dipu/runtime/distributed/ProcessGroupDICL.cpp:539-567). tp = 1 is the plain product. `residual`: rank 0
    adds it to its partial before materialising it (the addmm form), so that the sum is the block's output."""
    if tp == 1:
        return step(x @ weight.t()) if residual is None else step(residual + x @ weight.t())
    k = x.shape[-1]
    assert k % tp == 0
    ks = k // tp
    total = None
    for r in range(tp):
        part = x[..., r * ks:(r + 1) * ks] @ weight[:, r * ks:(r + 1) * ks].t()
        if r == 0 and residual is not None:
            part = residual + part
        part = step(part)
        total = part if total is None else total + part
    return step(total)


def attention_prefill(cfg, w, x, batch, seq, step=_identity, scores_by_baddbmm=False, fused=False, tp=1):
    t = batch * seq
    d = cfg.head_dim
    q = step(x @ w["wq"].t()).view(t, cfg.heads, d)
    k = step(x @ w["wk"].t()).view(t, cfg.kv_heads, d)
    v = step(x @ w["wv"].t()).view(batch, seq, cfg.kv_heads, d)
    cos, sin = rope_tables(d, torch.arange(seq), cfg.rope_base)
    if fused:
        # the attention core as ONE materialising op (the fused operator): rounding only where it writes its output
        qb = step(rotary(cfg, q, cos, sin)).view(batch, seq, cfg.heads, d)
        kb = step(rotary(cfg, k, cos, sin)).view(batch, seq, cfg.kv_heads, d)
        out = step(fused_attention(qb, kb, v, True)[0]).view(t, cfg.heads * d)
        return row_parallel(out, w["wo"], step, tp)
    q = step(rotary(cfg, q, cos, sin)).view(batch, seq, cfg.heads, d).transpose(1, 2)
    k = step(rotary(cfg, k, cos, sin)).view(batch, seq, cfg.kv_heads, d).transpose(1, 2)
    v = v.transpose(1, 2)
    k, v = _expand_kv(cfg, k), _expand_kv(cfg, v)
    if scores_by_baddbmm:
        # torch.baddbmm(mask, q, k^T, beta=1, alpha=1/sqrt(d)): one rounding after scale and mask
        scores = step(causal_mask(seq) + torch.matmul(q, k.transpose(2, 3)) * (1.0 / math.sqrt(d)))
    else:
        scores = step(step(torch.matmul(q, k.transpose(2, 3))) / math.sqrt(d))
        scores = step(scores + causal_mask(seq))
    probs = step(torch.softmax(scores.float(), dim=-1))
    out = step(torch.matmul(probs, v)).transpose(1, 2).contiguous().view(t, cfg.heads * d)
    return row_parallel(out, w["wo"], step, tp)


def feed_forward(w, x, step=_identity, fused_gate_up=False, residual=None, tp=1):
    """residual (with fused_gate_up only): the block's residual is added to the unrounded down projection, one materialising op
    (an addmm) instead of a product and an add. Returns the block's output then, else the feed-forward result."""
    if fused_gate_up:
        # SiLU(gate) * up as ONE materialising op over the two products (the fused gate / up projection): one rounding
        inner = step(torch.nn.functional.silu(x @ w["w1"].t()) * (x @ w["w3"].t()))
        return row_parallel(inner, w["w2"], step, tp, residual)
    gate = step(torch.nn.functional.silu(step(x @ w["w1"].t())))
    return row_parallel(step(gate * step(x @ w["w3"].t())), w["w2"], step, tp)


def decoder_layer_prefill_from_hidden(cfg, w, x, batch, seq, step=_identity, scores_by_baddbmm=False, fused=False, tp=1):
    """tp: the row-parallel linears as `tp` tensor-parallel ranks compute them (row_parallel); everything else is unsharded."""
    h = step(x + attention_prefill(cfg, w, step(rms_norm(x, w["attention_norm"], cfg.eps)), batch, seq, step, scores_by_baddbmm, fused, tp))
    return step(h + feed_forward(w, step(rms_norm(h, w["ffn_norm"], cfg.eps)), step, tp=tp))


def decoder_layer_prefill(cfg, w, embedding, ids, step=_identity, scores_by_baddbmm=False, fused=False):
    """ids [B, S] int64 -> layer output [B*S, hidden] float32."""
    batch, seq = ids.shape
    return decoder_layer_prefill_from_hidden(cfg, w, embedding[ids.reshape(-1)], batch, seq, step, scores_by_baddbmm, fused)


def decoder_layer_decode(cfg, w, x, k_cache, v_cache, position, step=_identity, fused=False, fused_gate_up=False, tp=1):
    """One new token per sequence. x [B, hidden]; caches [B, kv_heads, L, D] whose slot `position` is overwritten by the
    new token's key / value; attention covers slots 0..position. Returns (out [B, hidden], k_cache, v_cache).
    fused: the attention core as one materialising op; fused_gate_up: SiLU(gate) * up as one materialising op."""
    b = x.shape[0]
    d = cfg.head_dim
    hn = step(rms_norm(x, w["attention_norm"], cfg.eps))
    q = step(hn @ w["wq"].t()).view(b, cfg.heads, d)
    k = step(hn @ w["wk"].t()).view(b, cfg.kv_heads, d)
    v = step(hn @ w["wv"].t()).view(b, cfg.kv_heads, d)
    cos, sin = rope_tables(d, torch.tensor([position]), cfg.rope_base)
    q = step(rotary(cfg, q, cos, sin))
    k = step(rotary(cfg, k, cos, sin))
    k_cache = k_cache.clone()
    v_cache = v_cache.clone()
    k_cache[:, :, position, :] = k
    v_cache[:, :, position, :] = v
    if fused:
        kb = k_cache[:, :, : position + 1, :].transpose(1, 2)
        vb = v_cache[:, :, : position + 1, :].transpose(1, 2)
        ctx = step(fused_attention(q.unsqueeze(1), kb, vb, False)[0]).reshape(b, cfg.heads * d)
        h = step(x + row_parallel(ctx, w["wo"], step, tp))
        if fused_gate_up:
            out = feed_forward(w, step(rms_norm(h, w["ffn_norm"], cfg.eps)), step, True, residual=h, tp=tp)
        else:
            out = step(h + feed_forward(w, step(rms_norm(h, w["ffn_norm"], cfg.eps)), step, tp=tp))
        return out, k_cache, v_cache
    keys = _expand_kv(cfg, k_cache[:, :, : position + 1, :])
    vals = _expand_kv(cfg, v_cache[:, :, : position + 1, :])
    scores = step(step(torch.matmul(q.unsqueeze(2), keys.transpose(2, 3))) / math.sqrt(d))  # [B, heads, 1, L]
    probs = step(torch.softmax(scores.float(), dim=-1))
    ctx = step(torch.matmul(probs, vals)).reshape(b, cfg.heads * d)
    h = step(x + row_parallel(ctx, w["wo"], step, tp))
    out = step(h + feed_forward(w, step(rms_norm(h, w["ffn_norm"], cfg.eps)), step, tp=tp))
    return out, k_cache, v_cache


# ---- tensor-parallel sharding (Megatron style) -------------------------------------------------------------------------
def shard_weights(cfg, w, rank, size):
    """Column-parallel wq/wk/wv/w1/w3 (output features split), row-parallel wo/w2 (input features split)."""
    assert cfg.heads % size == 0 and cfg.kv_heads % size == 0 and cfg.ffn % size == 0
    d = cfg.head_dim
    hq, hk, f = cfg.heads // size, cfg.kv_heads // size, cfg.ffn // size
    return {
        "wq": w["wq"][rank * hq * d:(rank + 1) * hq * d].contiguous(),
        "wk": w["wk"][rank * hk * d:(rank + 1) * hk * d].contiguous(),
        "wv": w["wv"][rank * hk * d:(rank + 1) * hk * d].contiguous(),
        "wo": w["wo"][:, rank * hq * d:(rank + 1) * hq * d].contiguous(),
        "w1": w["w1"][rank * f:(rank + 1) * f].contiguous(),
        "w3": w["w3"][rank * f:(rank + 1) * f].contiguous(),
        "w2": w["w2"][:, rank * f:(rank + 1) * f].contiguous(),
        "attention_norm": w["attention_norm"],
        "ffn_norm": w["ffn_norm"],
    }


def local_config(cfg, size):
    return dataclasses.replace(cfg, heads=cfg.heads // size, kv_heads=cfg.kv_heads // size, ffn=cfg.ffn // size)
