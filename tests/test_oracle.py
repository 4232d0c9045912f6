"""The CPU oracle against the golden fixtures produced by the reference's own Python code (tests/golden/make_golden.py)."""
import hashlib
import os

import numpy as np
import torch

from oracle import llama_cpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return {k: v for k, v in np.load(os.path.join(GOLD, name)).items()}


def _c1():
    cfg = llama_cpu.LayerConfig(hidden=512, heads=8, kv_heads=8, head_dim=64, ffn=1376, eps=1e-6, rope_layout="interleaved")
    return cfg, llama_cpu.make_weights(cfg, seed=1234)


def test_weights_are_reproducible():
    g = _load("c1_block.npz")
    _, w = _c1()
    h = hashlib.sha256()
    for k in sorted(w):
        h.update(w[k].numpy().tobytes())
    assert h.hexdigest() == bytes(g["weights_sha256"]).decode()


def test_inputs_are_reproducible():
    g = _load("c1_block.npz")
    ids = llama_cpu.make_token_ids(1, 128, seed=1234)
    emb = llama_cpu.make_embedding(32000, 512, seed=1234)
    assert np.array_equal(ids.numpy(), g["ids"])
    assert np.array_equal(emb[ids.reshape(-1)].numpy().reshape(1, 128, 512), g["x"])  # embedding gather is bit-exact


def test_block_matches_reference_transformer_block():
    g = _load("c1_block.npz")
    cfg, w = _c1()
    torch.set_num_threads(1)
    x = torch.from_numpy(g["x"]).view(128, 512)
    attn = llama_cpu.attention_prefill(cfg, w, llama_cpu.rms_norm(x, w["attention_norm"], cfg.eps), 1, 128)
    y = llama_cpu.decoder_layer_prefill_from_hidden(cfg, w, x, 1, 128)
    np.testing.assert_allclose(attn.numpy().reshape(1, 128, 512), g["attn"], rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(y.numpy().reshape(1, 128, 512), g["y"], rtol=1e-4, atol=1e-6)


def test_half_layout_equals_interleaved_on_permuted_features():
    # the two rotary layouts are the same rotation on a fixed permutation of the head features
    rng = np.random.default_rng(3)
    x = torch.from_numpy(rng.standard_normal((6, 2, 16), dtype=np.float32))
    cos, sin = llama_cpu.rope_tables(16, torch.arange(6))
    perm = torch.cat((torch.arange(0, 16, 2), torch.arange(1, 16, 2)))  # interleaved index of each half-layout slot
    a = llama_cpu.rotary_interleaved(x, cos, sin)[..., perm]
    b = llama_cpu.rotary_half(x[..., perm], cos, sin)
    np.testing.assert_allclose(a.numpy(), b.numpy(), rtol=1e-5, atol=1e-6)


def test_rms_norm_matches_reference_module():
    g = _load("rmsnorm.npz")
    y = llama_cpu.rms_norm(torch.from_numpy(g["x"]), torch.from_numpy(g["weight"]), 1e-6)
    np.testing.assert_allclose(y.numpy(), g["y"], rtol=1e-6, atol=1e-7)


def test_rotary_interleaved_matches_reference_apply_rotary_emb():
    g = _load("rotary.npz")
    cos, sin = llama_cpu.rope_tables(64, torch.arange(16))
    for name in ("q", "k"):
        x = torch.from_numpy(g[name]).reshape(32, 8, 64)
        out = llama_cpu.rotary_interleaved(x, cos, sin).reshape(2, 16, 8, 64)
        np.testing.assert_allclose(out.numpy(), g[name + "_out"], rtol=1e-5, atol=1e-6)


def test_ext_ops_restatements():
    g = _load("ext_ops.npz")
    out = llama_cpu.rotary_half(torch.from_numpy(g["x"]), torch.from_numpy(g["cos"]), torch.from_numpy(g["sin"]))
    np.testing.assert_allclose(out.numpy(), g["rotary_out"], rtol=1e-6, atol=1e-7)
    y = llama_cpu.rms_norm(torch.from_numpy(g["rms_x"]), torch.from_numpy(g["rms_w"]), 1e-6)
    np.testing.assert_allclose(y.numpy(), g["rms_out"], rtol=1e-6, atol=1e-7)


def test_decode_step_equals_last_row_of_prefill():
    # size-independent property: decoding token S-1 over a cache of the first S-1 keys/values reproduces prefill's last row
    cfg = llama_cpu.LayerConfig(hidden=64, heads=4, kv_heads=2, head_dim=16, ffn=96, eps=1e-6)
    w = llama_cpu.make_weights(cfg, seed=5)
    rng = np.random.default_rng(9)
    b, s = 2, 9
    x = torch.from_numpy(rng.standard_normal((b * s, 64), dtype=np.float32))
    full = llama_cpu.decoder_layer_prefill_from_hidden(cfg, w, x, b, s).view(b, s, 64)
    # build the cache from the prefill's own keys / values
    hn = llama_cpu.rms_norm(x, w["attention_norm"], cfg.eps)
    cos, sin = llama_cpu.rope_tables(16, torch.arange(s))
    k = llama_cpu.rotary(cfg, (hn @ w["wk"].t()).view(b * s, 2, 16), cos, sin).view(b, s, 2, 16).transpose(1, 2).contiguous()
    v = (hn @ w["wv"].t()).view(b, s, 2, 16).transpose(1, 2).contiguous()
    k[:, :, s - 1] = 0
    v[:, :, s - 1] = 0
    out, _, _ = llama_cpu.decoder_layer_decode(cfg, w, x.view(b, s, 64)[:, s - 1], k, v, s - 1)
    np.testing.assert_allclose(out.numpy(), full[:, s - 1].numpy(), rtol=1e-4, atol=1e-5)


def test_tensor_parallel_shards_sum_to_full_layer():
    cfg = llama_cpu.LayerConfig(hidden=64, heads=4, kv_heads=4, head_dim=16, ffn=96, eps=1e-6)
    w = llama_cpu.make_weights(cfg, seed=11)
    rng = np.random.default_rng(12)
    x = torch.from_numpy(rng.standard_normal((10, 64), dtype=np.float32))
    hn = llama_cpu.rms_norm(x, w["attention_norm"], cfg.eps)
    full = llama_cpu.attention_prefill(cfg, w, hn, 2, 5)
    parts = [llama_cpu.attention_prefill(llama_cpu.local_config(cfg, 2), llama_cpu.shard_weights(cfg, w, r, 2), hn, 2, 5) for r in range(2)]
    np.testing.assert_allclose((parts[0] + parts[1]).numpy(), full.numpy(), rtol=1e-4, atol=1e-6)
    ff = llama_cpu.feed_forward(w, hn)
    fparts = [llama_cpu.feed_forward(llama_cpu.shard_weights(cfg, w, r, 2), hn) for r in range(2)]
    np.testing.assert_allclose((fparts[0] + fparts[1]).numpy(), ff.numpy(), rtol=1e-4, atol=1e-6)


def test_fused_attention_matches_reference_ext_ops():
    """The restated fused attention against the reference's own prompt_attention_inference / flash_attention_inference
    (dicp/dicp/vendor/AscendGraph/ext_ops.py:66-86,100-126), recorded in ext_attention.npz."""
    g = np.load(os.path.join(GOLD, "ext_attention.npz"))
    seq, heads, dim = 160, 4, 128
    q, k, v = (torch.from_numpy(g[n]).view(1, seq, heads, dim) for n in ("prompt_q", "prompt_k", "prompt_v"))
    out, lse = llama_cpu.fused_attention(q, k, v, True)
    np.testing.assert_allclose(out[0].numpy(), g["prompt_out"], rtol=1e-5, atol=2e-6)
    assert lse.shape == (1, heads, seq)
    fq, fk, fv = (torch.from_numpy(g[n]) for n in ("flash_q", "flash_k", "flash_v"))
    for i, length in enumerate(g["flash_lens"]):
        length = int(length)
        out, _ = llama_cpu.fused_attention(fq[i].view(1, 1, heads, dim), fk[:length].view(1, length, heads, dim),
                                           fv[:length].view(1, length, heads, dim), False)
        np.testing.assert_allclose(out.view(heads, dim).numpy(), g["flash_out"][i], rtol=1e-5, atol=2e-6)


def test_fused_attention_equals_op_by_op_attention():
    """The fused restatement and the bmm / softmax sequence of the layer agree in fp32 (grouped heads included)."""
    cfg = llama_cpu.LayerConfig(hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=512, eps=1e-6)
    w = llama_cpu.make_weights(cfg, seed=3)
    x = torch.from_numpy(np.random.default_rng(4).standard_normal((2 * 40, 256), dtype=np.float32))
    a = llama_cpu.attention_prefill(cfg, w, x, 2, 40)
    b = llama_cpu.attention_prefill(cfg, w, x, 2, 40, fused=True)
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


def test_row_parallel_forms():
    """The tensor-parallel evaluation of the row-parallel linears: in fp32 it is the plain product (to rounding of the fp32 sums);
    with bf16 materialisation every rank's partial is rounded before the sum; the addmm form adds the residual on rank 0."""
    g = torch.Generator().manual_seed(5)
    x, wgt, res = torch.randn((7, 64), generator=g), torch.randn((24, 64), generator=g), torch.randn((7, 24), generator=g)
    plain = x @ wgt.t()
    for tp in (1, 2, 4, 8):
        assert torch.allclose(llama_cpu.row_parallel(x, wgt, tp=tp), plain, atol=1e-5)
        assert torch.allclose(llama_cpu.row_parallel(x, wgt, tp=tp, residual=res), res + plain, atol=1e-5)
    bf = llama_cpu.stepwise(torch.bfloat16)
    want = bf(bf(x[:, :32] @ wgt[:, :32].t()) + bf(x[:, 32:] @ wgt[:, 32:].t()))
    assert torch.equal(llama_cpu.row_parallel(x, wgt, bf, tp=2), want)
    want_res = bf(bf(res + x[:, :32] @ wgt[:, :32].t()) + bf(x[:, 32:] @ wgt[:, 32:].t()))
    assert torch.equal(llama_cpu.row_parallel(x, wgt, bf, tp=2, residual=res), want_res)
    cfg = llama_cpu.LayerConfig(hidden=64, heads=4, kv_heads=4, head_dim=16, ffn=96, eps=1e-6)
    w = llama_cpu.make_weights(cfg, seed=9)
    h = torch.randn((2 * 8, 64), generator=g)
    a = llama_cpu.decoder_layer_prefill_from_hidden(cfg, w, h, 2, 8)
    b = llama_cpu.decoder_layer_prefill_from_hidden(cfg, w, h, 2, 8, tp=4)
    assert torch.allclose(a, b, atol=1e-5)
