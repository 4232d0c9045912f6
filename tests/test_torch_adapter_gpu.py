"""The eager adapter: a plain nn.Module run on torch.device("dipu"), every op dispatched to a wrapper that calls the DIOPI
C-ABI (the shape of the reference's generated wrappers, dipu/scripts/autogen_diopi_wrapper/diopi_wrapper_template.py:100-142),
compared with the same module on CPU. Shapes and tolerances follow the reference's unit tests
(dipu/tests/python/unittests/test_mm.py, test_softmax.py, test_layer_norm.py, test_cat.py, test_index.py, test_copy.py)."""
import importlib
import math

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def adapter(pkg):
    return importlib.import_module(pkg.__name__ + ".torch_adapter")


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x) * self.weight


def rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


class Block(nn.Module):
    """A Llama-style decoder block in plain torch: nothing in it knows about the device."""

    def __init__(self, dim, heads, kv_heads, ffn):
        super().__init__()
        self.heads, self.kv_heads, self.head_dim = heads, kv_heads, dim // heads
        self.wq = nn.Linear(dim, heads * self.head_dim, bias=False)
        self.wk = nn.Linear(dim, kv_heads * self.head_dim, bias=False)
        self.wv = nn.Linear(dim, kv_heads * self.head_dim, bias=False)
        self.wo = nn.Linear(heads * self.head_dim, dim, bias=False)
        self.w1 = nn.Linear(dim, ffn, bias=False)
        self.w2 = nn.Linear(ffn, dim, bias=False)
        self.w3 = nn.Linear(dim, ffn, bias=False)
        self.attention_norm, self.ffn_norm = RMSNorm(dim), RMSNorm(dim)

    def forward(self, x, cos, sin, mask):
        b, s, _ = x.shape
        h = self.attention_norm(x)
        q = self.wq(h).view(b, s, self.heads, self.head_dim).transpose(1, 2)
        k = self.wk(h).view(b, s, self.kv_heads, self.head_dim).transpose(1, 2)
        v = self.wv(h).view(b, s, self.kv_heads, self.head_dim).transpose(1, 2)
        q = q * cos + rotate_half(q) * sin
        k = k * cos + rotate_half(k) * sin
        if self.kv_heads != self.heads:
            g = self.heads // self.kv_heads
            k = k[:, :, None].expand(b, self.kv_heads, g, s, self.head_dim).reshape(b, self.heads, s, self.head_dim)
            v = v[:, :, None].expand(b, self.kv_heads, g, s, self.head_dim).reshape(b, self.heads, s, self.head_dim)
        scores = torch.matmul(q, k.transpose(2, 3)) / math.sqrt(self.head_dim)
        scores = F.softmax((scores + mask).float(), dim=-1).type_as(q)
        a = torch.matmul(scores, v).transpose(1, 2).contiguous().view(b, s, -1)
        x = x + self.wo(a)
        h = self.ffn_norm(x)
        return x + self.w2(F.silu(self.w1(h)) * self.w3(h))


def _tables(seq, head_dim):
    inv = 1.0 / (10000.0 ** (torch.arange(0, head_dim, 2).float() / head_dim))
    ang = torch.outer(torch.arange(seq).float(), inv)
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos()[None, None], emb.sin()[None, None]


@pytest.mark.parametrize("dtype,kv_heads", [(torch.float32, 4), (torch.bfloat16, 4), (torch.bfloat16, 2)])
def test_unmodified_module_runs_on_dipu(adapter, dtype, kv_heads):
    torch.manual_seed(0)
    dim, heads, ffn, b, s = 512, 4, 1376, 2, 96
    block = Block(dim, heads, kv_heads, ffn)
    for p in block.parameters():
        if p.dim() == 2:
            nn.init.normal_(p, std=0.02)
    x = torch.randn(b, s, dim) * 0.5
    cos, sin = _tables(s, dim // heads)
    mask = torch.triu(torch.full((1, 1, s, s), float("-inf")), diagonal=1)
    if dtype != torch.float32:   # the CPU side computes in fp32 from the rounded parameters and inputs
        block = block.to(dtype).float()
        x, cos, sin = x.to(dtype).float(), cos.to(dtype).float(), sin.to(dtype).float()
    with torch.no_grad():
        ref = block(x, cos, sin, mask)
        before = adapter.stats()["diopi_calls"]
        dev = torch.device("dipu:0")
        dblock = Block(dim, heads, kv_heads, ffn)
        dblock.load_state_dict(block.state_dict())
        dblock = dblock.to(dtype).to(dev)
        assert next(dblock.parameters()).device.type == "dipu"
        y = dblock(x.to(dtype).to(dev), cos.to(dtype).to(dev), sin.to(dtype).to(dev), mask.to(dev))
        assert y.device.type == "dipu" and y.dtype == dtype
        got = y.float().cpu()
    assert adapter.stats()["diopi_calls"] - before > 40   # every op of the block went through a DIOPI call
    err = (got - ref).abs().max().item()
    rel = ((got - ref).norm() / ref.norm()).item()
    if dtype == torch.float32:
        assert err <= 2e-4 and rel <= 1e-5, (err, rel)
    else:
        assert err <= 2e-2 and rel <= 1e-2, (err, rel)   # whole bf16 layer against fp32: the layer tests' bound


def test_single_ops_against_cpu(adapter):
    dev = torch.device("dipu:0")
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        # embedding lowers to index_select: bit-exact
        table = torch.randn(1000, 64, generator=g)
        ids = torch.randint(0, 1000, (3, 17), generator=g)
        assert torch.equal(F.embedding(ids.to(dev), table.to(dev)).cpu(), F.embedding(ids, table))
        # copies: cast, transpose materialisation, expand, slices, host round trip
        a = torch.randn(5, 7, 9, generator=g)
        ad = a.to(dev)
        assert torch.equal(ad.cpu(), a)
        assert torch.equal(ad.transpose(0, 2).contiguous().cpu(), a.transpose(0, 2).contiguous())
        assert torch.equal(ad.to(torch.bfloat16).cpu(), a.to(torch.bfloat16))
        assert torch.equal(ad[1:4, ::2].cpu(), a[1:4, ::2])
        assert torch.equal(ad[:, :1].expand(5, 7, 9).contiguous().cpu(), a[:, :1].expand(5, 7, 9).contiguous())
        assert abs(ad[2, 3, 4].item() - a[2, 3, 4].item()) == 0.0
        # layer norm with statistics (reference unittests/test_layer_norm.py shapes)
        x = torch.randn(4, 6, 32, generator=g)
        w, b = torch.randn(32, generator=g), torch.randn(32, generator=g)
        torch.testing.assert_close(F.layer_norm(x.to(dev), [32], w.to(dev), b.to(dev), 1e-5).cpu(), F.layer_norm(x, [32], w, b, 1e-5), rtol=1e-4,
                                   atol=1e-5)
        # mm / addmm / bmm / baddbmm
        m1, m2, bias = torch.randn(33, 20, generator=g), torch.randn(20, 45, generator=g), torch.randn(45, generator=g)
        torch.testing.assert_close(torch.mm(m1.to(dev), m2.to(dev)).cpu(), torch.mm(m1, m2), rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(torch.addmm(bias.to(dev), m1.to(dev), m2.to(dev), beta=0.5, alpha=2.0).cpu(),
                                   torch.addmm(bias, m1, m2, beta=0.5, alpha=2.0), rtol=1e-4, atol=1e-4)
        b1, b2 = torch.randn(3, 8, 5, generator=g), torch.randn(3, 5, 6, generator=g)
        torch.testing.assert_close(torch.bmm(b1.to(dev), b2.to(dev)).cpu(), torch.bmm(b1, b2), rtol=1e-4, atol=1e-4)
        # scalars on either side, in-place forms, mixed dtypes
        torch.testing.assert_close((2.0 * x.to(dev) + 1.5).cpu(), 2.0 * x + 1.5)
        torch.testing.assert_close((x.to(dev) / 3.0 - x.to(dev) * x.to(dev)).cpu(), x / 3.0 - x * x)
        y = x.to(dev).clone()
        y.mul_(0.5).add_(x.to(dev), alpha=2.0)
        torch.testing.assert_close(y.cpu(), x * 0.5 + 2.0 * x)
        torch.testing.assert_close((x.to(dev).to(torch.bfloat16) + x.to(dev)).cpu(), x.to(torch.bfloat16) + x)
        # masks and selection
        cond = x > 0
        torch.testing.assert_close(torch.where(cond.to(dev), x.to(dev), -x.to(dev)).cpu(), torch.where(cond, x, -x))
        z = x.to(dev).clone()
        z.masked_fill_(cond.to(dev), -1.0)
        torch.testing.assert_close(z.cpu(), x.masked_fill(cond, -1.0))
        torch.testing.assert_close(torch.triu(torch.ones(6, 6, device=dev), diagonal=1).cpu(), torch.triu(torch.ones(6, 6), diagonal=1))
        torch.testing.assert_close(torch.cat([x.to(dev), x.to(dev)[:, :2]], dim=1).cpu(), torch.cat([x, x[:, :2]], dim=1))
        torch.testing.assert_close(torch.softmax(x.to(dev), dim=1).cpu(), torch.softmax(x, dim=1), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(torch.zeros(3, 4, device=dev).cpu(), torch.zeros(3, 4))
        # the fused norm entry of recent torch
        out, rstd = torch.ops.aten._fused_rms_norm(x.to(dev), [32], w.to(dev), 1e-6)
        want = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
        torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("kv_heads,causal", [(4, True), (4, False), (1, True)])
def test_scaled_dot_product_attention_reaches_the_fused_kernel(adapter, kv_heads, causal):
    """F.scaled_dot_product_attention on the dipu device dispatches to the library's fused attention (one DIOPI call, views
    taken as they are); anything it cannot run (here: an explicit mask) takes torch's op-by-op composite instead."""
    dev = torch.device("dipu:0")
    g = torch.Generator().manual_seed(9)
    b, s, h, d = 2, 300, 4, 128
    q = torch.randn(b, s, h, d, generator=g).to(torch.bfloat16)
    k = torch.randn(b, s, kv_heads, d, generator=g).to(torch.bfloat16)
    v = torch.randn(b, s, kv_heads, d, generator=g).to(torch.bfloat16)
    rep = h // kv_heads
    ref = F.scaled_dot_product_attention(q.float().transpose(1, 2), k.float().transpose(1, 2).repeat_interleave(rep, 1),
                                         v.float().transpose(1, 2).repeat_interleave(rep, 1), is_causal=causal)
    with torch.no_grad():
        before = adapter.stats()["diopi_calls"]
        out = F.scaled_dot_product_attention(q.to(dev).transpose(1, 2), k.to(dev).transpose(1, 2), v.to(dev).transpose(1, 2), is_causal=causal,
                                             enable_gqa=kv_heads != h)
        calls = adapter.stats()["diopi_calls"] - before
        got = out.float().cpu()
    assert calls == 1, calls
    assert out.shape == (b, h, s, d)
    err, rel = (got - ref).abs().max().item(), ((got - ref).norm() / ref.norm()).item()
    assert err <= 2e-2 and rel <= 5e-3, (err, rel)


@pytest.mark.parametrize("sq,skv", [(1, 200), (72, 300), (300, 72), (260, 130)])
def test_scaled_dot_product_attention_causal_with_unequal_lengths(adapter, sq, skv):
    """is_causal with L != S: torch aligns the mask to the first key (query i sees keys 0..i, the lower triangle of ones(L, S)),
    the library's operator to the last one. The adapter has to give torch's answer: L = 1 sees key 0 only, and with more
    queries than keys the late queries see every key."""
    dev = torch.device("dipu:0")
    g = torch.Generator().manual_seed(sq * 1000 + skv)
    b, h, d = 2, 4, 128
    q = torch.randn(b, sq, h, d, generator=g).to(torch.bfloat16)
    k = torch.randn(b, skv, h, d, generator=g).to(torch.bfloat16)
    v = torch.randn(b, skv, h, d, generator=g).to(torch.bfloat16)
    ref = F.scaled_dot_product_attention(q.float().transpose(1, 2), k.float().transpose(1, 2), v.float().transpose(1, 2), is_causal=True)
    with torch.no_grad():
        out = F.scaled_dot_product_attention(q.to(dev).transpose(1, 2), k.to(dev).transpose(1, 2), v.to(dev).transpose(1, 2), is_causal=True)
        got = out.float().cpu()
    assert out.shape == (b, h, sq, d)
    err, rel = (got - ref).abs().max().item(), ((got - ref).norm() / ref.norm()).item()
    assert err <= 2e-2 and rel <= 5e-3, (err, rel)


def test_sampling_ops_through_the_adapter(adapter):
    dev = torch.device("dipu:0")
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(4, 5000, generator=g)
    ld = logits.to(dev)
    with torch.no_grad():
        assert torch.equal(torch.argmax(ld, dim=-1).cpu(), torch.argmax(logits, dim=-1))
        v, i = torch.topk(ld, 20, dim=-1)
        rv, ri = torch.topk(logits, 20, dim=-1)
        assert torch.equal(v.cpu(), rv) and torch.equal(i.cpu(), ri)
        sv, si = torch.sort(torch.softmax(ld, -1), dim=-1, descending=True, stable=True)
        rsv, rsi = torch.sort(torch.softmax(logits, -1), dim=-1, descending=True, stable=True)
        torch.testing.assert_close(sv.cpu(), rsv, rtol=1e-5, atol=1e-8)
        torch.testing.assert_close(torch.cumsum(sv, -1).cpu(), torch.cumsum(rsv, -1), rtol=1e-4, atol=1e-5)
        pos = torch.multinomial(sv, 1)
        assert pos.shape == (4, 1) and pos.dtype == torch.int64
        tok = torch.gather(si, 1, pos)
        assert torch.equal(tok.cpu(), si.cpu().gather(1, pos.cpu()))


def test_missing_wrapper_raises_instead_of_falling_back(adapter):
    x = torch.ones(8, device="dipu:0")
    with pytest.raises(NotImplementedError):
        torch.flip(x, [0])


# ---- copies: the cases of dipu/tests/python/unittests/test_copy.py:88-150 -------------------------------------------------
def test_h2d_copies_from_freed_pageable_buffers_stay_correct(adapter):
    """500 non-blocking host-to-device copies whose pageable source tensors are freed right after the call
    (test_copy.py:126-143): every device tensor must hold its value."""
    dev = torch.device("dipu:0")

    def copy_tensor(device_tensor, val):
        cpu_tensor = torch.empty(device_tensor.shape, dtype=torch.float32, pin_memory=False).fill_(val)
        device_tensor.copy_(cpu_tensor, non_blocking=True)
        del cpu_tensor

    tensors = []
    for i in range(500):
        t = torch.empty(100, 100, dtype=torch.float32, device=dev)
        copy_tensor(t, float(i))
        tensors.append(t)
    for i in range(500):
        assert torch.equal(tensors[i].cpu(), torch.full((100, 100), float(i)))


def test_h2d_copy_blocking_is_really_blocking(adapter):
    # test_copy.py:145-150: the source may change as soon as copy_ returns
    a = torch.ones(1000000, pin_memory=True)
    b = torch.zeros(1000000, device="dipu:0")
    b.copy_(a, non_blocking=False)
    a[-1].fill_(-1)
    assert torch.equal(b.cpu(), torch.ones(1000000))


def test_copy_into_a_hollow_strided_destination(adapter):
    # test_copy.py:78-85
    g = torch.Generator().manual_seed(3)
    t1 = torch.rand((6, 4), generator=g)
    d1 = t1.to("dipu:0")
    dst = d1.as_strided((2, 2), (4, 1))
    src = torch.rand((2, 2), generator=g)
    dst.copy_(src.to("dipu:0"))
    assert torch.equal(dst.cpu(), src)
    want = t1.clone()
    want.as_strided((2, 2), (4, 1)).copy_(src)
    assert torch.equal(d1.cpu(), want)   # nothing outside the view was touched


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_copies_between_two_devices(adapter):
    """test_copy.py:88-117: copy_ between tensors of two devices in both directions, and a non-contiguous source (relayed
    through a dense tensor on its own device)."""
    g = torch.Generator().manual_seed(4)
    for a, b in ((0, 1), (1, 0)):
        src_h, dst_h = torch.rand((640, 400), generator=g), torch.rand((640, 400), generator=g)
        src, dst = src_h.to("dipu:%d" % a), dst_h.to("dipu:%d" % b)
        dst.copy_(src)
        assert torch.equal(dst.cpu(), src_h) and dst.device.index == b and src.device.index == a
    big = torch.rand((640, 990), generator=g)
    src = big.to("dipu:1")[::2, ::3]
    dst = src.to("dipu:0")
    assert torch.equal(dst.cpu(), big[::2, ::3]) and dst.device.index == 0
    # other dtype and a strided destination on the receiving side
    dst2 = torch.zeros((320, 660), dtype=torch.bfloat16, device="dipu:0")[:, ::2]
    dst2.copy_(src)
    assert torch.equal(dst2.cpu(), big[::2, ::3].to(torch.bfloat16))
