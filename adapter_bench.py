"""Timing of the eager adapter: a plain-torch Llama-style block on torch.device("dipu") at the 7B prefill shape, and the
host cost of one wrapper call.

    python adapter_bench.py [--batch 8 --seq 2048 --steps 10]

Prints one JSON line: ms per layer step and tokens/s through torch dispatch + wrapper + DIOPI (the path DIPU's generated
wrappers take, reference dipu/scripts/autogen_diopi_wrapper/diopi_wrapper_template.py:100-142), the number of DIOPI
calls per step, and the per-call host time of a 1-element add through the adapter and through the ctypes binding.
Device time is measured with the vendor runtime's events on the stream the wrappers launch on."""
import argparse
import importlib
import json
import math
import os
import sys
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


class Block(nn.Module):
    def __init__(self, dim, heads, ffn, sdpa=False):
        super().__init__()
        self.heads, self.head_dim, self.sdpa = heads, dim // heads, sdpa
        self.wq, self.wk, self.wv, self.wo = (nn.Linear(dim, dim, bias=False) for _ in range(4))
        self.w1, self.w3 = nn.Linear(dim, ffn, bias=False), nn.Linear(dim, ffn, bias=False)
        self.w2 = nn.Linear(ffn, dim, bias=False)
        self.attention_norm, self.ffn_norm = RMSNorm(dim), RMSNorm(dim)

    def forward(self, x, cos, sin, mask):
        b, s, _ = x.shape
        h = self.attention_norm(x)
        q = self.wq(h).view(b, s, self.heads, self.head_dim).transpose(1, 2)
        k = self.wk(h).view(b, s, self.heads, self.head_dim).transpose(1, 2)
        v = self.wv(h).view(b, s, self.heads, self.head_dim).transpose(1, 2)
        q = q * cos + rotate_half(q) * sin
        k = k * cos + rotate_half(k) * sin
        if self.sdpa:
            # torch's own fused-attention entry: on the dipu device it reaches diopiMultiHeadAttention
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, s, -1)
        else:
            scores = torch.matmul(q, k.transpose(2, 3)) / math.sqrt(self.head_dim)
            scores = F.softmax(scores + mask, dim=-1)
            a = torch.matmul(scores, v).transpose(1, 2).contiguous().view(b, s, -1)
        x = x + self.wo(a)
        h = self.ffn_norm(x)
        return x + self.w2(F.silu(self.w1(h)) * self.w3(h))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--sdpa", action="store_true", help="attention through F.scaled_dot_product_attention instead of matmul / softmax / matmul")
    args = ap.parse_args()
    import __graft_entry__ as entry
    pkg = entry.load_package()
    adapter = importlib.import_module(pkg.__name__ + ".torch_adapter")
    devapis, diopi = pkg.devapis, pkg.diopi
    dev = torch.device("dipu:0")
    dim, heads, ffn, bf = 4096, 32, 11008, torch.bfloat16
    torch.manual_seed(1234)
    with torch.no_grad():
        block = Block(dim, heads, ffn, sdpa=args.sdpa)
        for p in block.parameters():
            if p.dim() == 2:
                nn.init.normal_(p, std=0.02)
        block = block.to(bf).to(dev)
        x = (torch.randn(args.batch, args.seq, dim) * 0.5).to(bf).to(dev)
        inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2).float() / 128))
        ang = torch.outer(torch.arange(args.seq).float(), inv)
        emb = torch.cat((ang, ang), dim=-1)
        cos, sin = emb.cos()[None, None].to(bf).to(dev), emb.sin()[None, None].to(bf).to(dev)
        mask = torch.triu(torch.full((1, 1, args.seq, args.seq), float("-inf")), diagonal=1).to(bf).to(dev)
        stream = devapis.getDefaultStream(0)
        for _ in range(3):
            block(x, cos, sin, mask)
        devapis.syncStream(stream)
        c0 = adapter.stats()["diopi_calls"]
        e0, e1 = devapis.createEvent(), devapis.createEvent()
        t0 = time.perf_counter()
        devapis.recordEvent(e0, stream)
        for _ in range(args.steps):
            block(x, cos, sin, mask)
        devapis.recordEvent(e1, stream)
        host_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        devapis.waitEvent(e1)
        ms = devapis.eventElapsedTime(e0, e1) / args.steps
        calls = (adapter.stats()["diopi_calls"] - c0) // args.steps
        # host cost of one wrapper call: 1-element add, queue kept short by syncing in batches
        a, b = torch.ones(1, device=dev, dtype=bf), torch.ones(1, device=dev, dtype=bf)
        out = torch.empty_like(a)
        n = 2000
        torch.add(a, b, out=out)
        devapis.syncStream(stream)
        t0 = time.perf_counter()
        for _ in range(n):
            torch.add(a, b, out=out)
        adapter_us = (time.perf_counter() - t0) * 1e6 / n
        devapis.syncStream(stream)
    ca, cb, cout = (torch.ones(1, device="cuda:0", dtype=bf) for _ in range(3))
    ctx = diopi.Context(stream=stream, device=0)
    diopi.diopiAdd(ctx, cout, ca, cb, 1)
    devapis.syncStream(stream)
    t0 = time.perf_counter()
    for _ in range(n):
        diopi.diopiAdd(ctx, cout, ca, cb, 1)
    ctypes_us = (time.perf_counter() - t0) * 1e6 / n
    devapis.syncStream(stream)
    tokens = args.batch * args.seq
    print(json.dumps({"workload": "plain-torch Llama-style block on torch.device('dipu'), bf16, batch %d x seq %d, attention by %s"
                                  % (args.batch, args.seq, "F.scaled_dot_product_attention" if args.sdpa else "matmul / softmax / matmul"),
                      "ms_per_step": round(ms, 3), "tokens_per_s": round(tokens / (ms * 1e-3)), "host_ms_per_step": round(host_ms, 3),
                      "diopi_calls_per_step": int(calls), "add_1_element_host_us": {"torch dispatch + wrapper": round(adapter_us, 2),
                                                                                     "ctypes binding": round(ctypes_us, 2)}}))


if __name__ == "__main__":
    main()
