"""Generates the golden fixtures in this directory by running the REFERENCE's own Python code on CPU.

Run once where a checkout of the reference project is available; REFERENCE_ROOT names its top directory:

    REFERENCE_ROOT=<reference checkout> python tests/golden/make_golden.py

It imports dicp/test/model/llama/model.py unmodified (only the relative import of a device helper is satisfied with a
stub that answers "cpu") and records, for seeded inputs:

    c1_block.npz     TransformerBlock forward, fp32, batch 1, seq 128, dim 512, 8 heads, FFN 1376, eps 1e-6
                     (the CPU configuration of the benchmark description): input x, output y, attention output
    rmsnorm.npz      RMSNorm module forward on [64, 512]
    rotary.npz       apply_rotary_emb (interleaved pairs) on [2, 16, 8, 64] q and k
    ext_ops.npz      the half-split rotary and the fused rms_norm exactly as written in
                     dicp/dicp/vendor/AscendGraph/ext_ops.py:24-33,47-49 (that file cannot be imported without
                     torch_dipu, so the two three-line function bodies are exec'd from its source text)
    ext_attention.npz  the fused attention operators of the same file (prompt_attention_inference :66-86,
                     flash_attention_inference :100-126), exec'd the same way, on bf16-representable inputs
                     (`python tests/golden/make_golden.py attention` regenerates only this file)

Weights are NOT stored (12 MB): they are regenerated from the numpy seed by oracle.llama_cpu.make_weights, and a
checksum of them is stored instead. The tests never read the reference checkout; only this script does.
"""
import hashlib
import importlib.util
import os
import re
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set REFERENCE_ROOT to the top directory of the reference checkout")
sys.path.insert(0, ROOT)
from oracle import llama_cpu  # noqa: E402


def load_reference_model():
    # model.py does `from ...common.utils import get_device`; give it a parent package chain with that one function
    for name in ("refpkg", "refpkg.common", "refpkg.common.utils", "refpkg.model", "refpkg.model.llama"):
        sys.modules[name] = types.ModuleType(name)
        sys.modules[name].__path__ = []
    sys.modules["refpkg.common.utils"].get_device = lambda: "cpu"
    path = os.path.join(REF, "dicp", "test", "model", "llama", "model.py")
    spec = importlib.util.spec_from_file_location("refpkg.model.llama.model", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["refpkg.model.llama.model"] = mod
    spec.loader.exec_module(mod)
    return mod


def load_ext_ops_bodies():
    src = open(os.path.join(REF, "dicp", "dicp", "vendor", "AscendGraph", "ext_ops.py")).read()
    ns = {"torch": torch}
    for fn in ("lightllm_rotary_emb_impl", "lightllm_rms_norm_impl"):
        m = re.search(r"^def %s\(.*?(?=^\S)" % fn, src, re.S | re.M)
        exec(m.group(0), ns)
    return ns["lightllm_rotary_emb_impl"], ns["lightllm_rms_norm_impl"]


def load_ext_attention_bodies():
    import math
    import torch.nn.functional as F
    src = open(os.path.join(REF, "dicp", "dicp", "vendor", "AscendGraph", "ext_ops.py")).read()
    ns = {"torch": torch, "math": math, "F": F}
    for fn in ("lightllm_prompt_attention_inference_impl", "lightllm_flash_attention_inference_impl"):
        m = re.search(r"^def %s\(.*?(?=^\S)" % fn, src, re.S | re.M)
        exec(m.group(0), ns)
    return ns["lightllm_prompt_attention_inference_impl"], ns["lightllm_flash_attention_inference_impl"]


def make_attention_golden():
    """ext_attention.npz: the reference's fused attention operators (ext_ops.py:66-86 prompt_attention_inference,
    ext_ops.py:100-126 flash_attention_inference) on inputs that are exactly representable in bf16."""
    torch.set_num_threads(1)
    prompt, flash = load_ext_attention_bodies()
    rng = np.random.default_rng(17)

    def rn(*shape):
        return torch.from_numpy(rng.standard_normal(shape, dtype=np.float32)).to(torch.bfloat16).float()

    seq, heads, dim = 160, 4, 128
    pq, pk, pv = rn(1, seq, heads * dim), rn(1, seq, heads * dim), rn(1, seq, heads * dim)
    pout = prompt(pq, pk, pv, torch.tensor(seq), heads, dim, heads)          # [seq, heads, dim]
    batch, cap = 3, 200
    lens = [200, 77, 150]
    fq, fk, fv = rn(batch, heads, dim), rn(cap, heads, dim), rn(cap, heads, dim)
    fout = flash(fq, fk, fv, lens, cap, heads, heads, dim)                   # [batch, heads, dim]
    np.savez_compressed(os.path.join(HERE, "ext_attention.npz"), prompt_q=pq.numpy(), prompt_k=pk.numpy(), prompt_v=pv.numpy(),
                        prompt_out=pout.numpy(), flash_q=fq.numpy(), flash_k=fk.numpy(), flash_v=fv.numpy(),
                        flash_lens=np.array(lens, dtype=np.int64), flash_out=fout.numpy())


def weights_checksum(w):
    h = hashlib.sha256()
    for k in sorted(w):
        h.update(w[k].numpy().tobytes())
    return h.hexdigest()


def main():
    torch.set_num_threads(1)  # fixed reduction order
    ref = load_reference_model()
    cfg = llama_cpu.LayerConfig(hidden=512, heads=8, kv_heads=8, head_dim=64, ffn=1376, eps=1e-6, rope_layout="interleaved")
    w = llama_cpu.make_weights(cfg, seed=1234)
    seq = 128
    args = ref.ModelArgs(dim=512, n_layers=1, n_heads=8, vocab_size=32000, multiple_of=32, norm_eps=1e-6, max_batch_size=1,
                         max_seq_len=seq, max_prompt_size=seq)
    block = ref.TransformerBlock(0, args)
    assert block.feed_forward.w1.weight.shape == (1376, 512)
    with torch.no_grad():
        block.attention.wq.weight.copy_(w["wq"]); block.attention.wk.weight.copy_(w["wk"])
        block.attention.wv.weight.copy_(w["wv"]); block.attention.wo.weight.copy_(w["wo"])
        block.feed_forward.w1.weight.copy_(w["w1"]); block.feed_forward.w2.weight.copy_(w["w2"])
        block.feed_forward.w3.weight.copy_(w["w3"])
        block.attention_norm.weight.copy_(w["attention_norm"]); block.ffn_norm.weight.copy_(w["ffn_norm"])
    emb = llama_cpu.make_embedding(32000, 512, seed=1234)
    ids = llama_cpu.make_token_ids(1, seq, seed=1234)
    x = emb[ids.reshape(-1)].view(1, seq, 512)
    freqs = torch.view_as_real(ref.precompute_freqs_cis(64, seq))
    mask = torch.triu(torch.full((1, 1, seq, seq), float("-inf")), diagonal=1)
    with torch.no_grad():
        attn = block.attention.forward(block.attention_norm(x), freqs, mask, seq)
        y = block.forward(x, freqs, mask, seq)
    np.savez_compressed(os.path.join(HERE, "c1_block.npz"), ids=ids.numpy(), x=x.numpy(), attn=attn.numpy(), y=y.numpy(),
                        weights_sha256=np.frombuffer(weights_checksum(w).encode(), dtype=np.uint8))

    rng = np.random.default_rng(7)
    xr = torch.from_numpy(rng.standard_normal((64, 512), dtype=np.float32))
    wr = torch.from_numpy(rng.standard_normal(512, dtype=np.float32))
    norm = ref.RMSNorm(512, eps=1e-6)
    with torch.no_grad():
        norm.weight.copy_(wr)
        yr = norm(xr)
    np.savez_compressed(os.path.join(HERE, "rmsnorm.npz"), x=xr.numpy(), weight=wr.numpy(), y=yr.numpy())

    q = torch.from_numpy(rng.standard_normal((2, 16, 8, 64), dtype=np.float32))
    k = torch.from_numpy(rng.standard_normal((2, 16, 8, 64), dtype=np.float32))
    fr = torch.view_as_real(ref.precompute_freqs_cis(64, 16))
    qo, ko = ref.apply_rotary_emb(q, k, fr)
    np.savez_compressed(os.path.join(HERE, "rotary.npz"), q=q.numpy(), k=k.numpy(), q_out=qo.numpy(), k_out=ko.numpy())

    rotary_half, rms = load_ext_ops_bodies()
    xe = torch.from_numpy(rng.standard_normal((16, 8, 64), dtype=np.float32))
    cos, sin = llama_cpu.rope_tables(64, torch.arange(16))
    np.savez_compressed(os.path.join(HERE, "ext_ops.npz"), x=xe.numpy(), cos=cos.numpy(), sin=sin.numpy(),
                        rotary_out=rotary_half(xe, cos, sin).numpy(), rms_x=xr.numpy(), rms_w=wr.numpy(),
                        rms_out=rms(xr, wr, 1e-6).numpy())
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "attention":
        make_attention_golden()   # only ext_attention.npz
    else:
        main()
        make_attention_golden()
