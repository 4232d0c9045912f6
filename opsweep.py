"""Per-op sweep on one GPU: achieved HBM GB/s of the memory-bound DIOPI ops and TFLOP/s of the dense contractions.

    python opsweep.py                       # the whole sweep, one JSON line per case
    python opsweep.py --ops rmsnorm --tokens 16384 --iters 5    # one case (e.g. under a profiler)

Memory-bound ops run on bf16 [T, 4096] tensors, T in {1, 64, 1024, 16384, 65536}, values N(0,1); the embedding gathers
int64 ids uniform in [0, 32000) from a [32000, 4096] bf16 table. Each case cycles through enough distinct buffer sets that
the working set exceeds the 126 MB L2, and is timed with CUDA events on the launching stream after warm-up. GB/s uses
the algorithmic bytes of the op (stated per case in the output), the fraction is against the measured copy bandwidth in
MEASURED_PEAKS.json when that file is present. GEMM cases are the layer's shapes (prefill and decode).
"""
import argparse
import json
import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = HERE
sys.path.insert(0, ROOT)

H = 4096
L2_BYTES = 126 << 20


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def time_cases(fn_list, iters, stream):
    """fn_list: one closure per buffer set; returns mean milliseconds per call."""
    n = len(fn_list)
    for i in range(max(3, min(n, 8))):
        fn_list[i % n]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(iters):
        fn_list[i % n]()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def nsets(bytes_per_set):
    return int(max(2, min(64, math.ceil(2.0 * L2_BYTES / max(bytes_per_set, 1)))))


def mem_case(name, t, diopi, ctx, dev):
    bf = torch.bfloat16
    g = torch.Generator(device=dev)
    g.manual_seed(t)

    def rn(*shape, dtype=bf):
        return torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(dtype)

    n = t * H
    es = 2
    if name == "rmsnorm":
        alg = 2 * es * n + es * H
        k = nsets(alg)
        w = rn(H)
        xs, ys = [rn(t, H) for _ in range(k)], [torch.empty((t, H), dtype=bf, device=dev) for _ in range(k)]
        fns = [lambda i=i: diopi.diopiRMSNorm(ctx, ys[i], None, xs[i], [H], w, None, 1e-6) for i in range(k)]
    elif name == "layernorm":
        alg = 2 * es * n + 2 * es * H + 2 * es * t
        k = nsets(alg)
        w, b = rn(H), rn(H)
        xs, ys = [rn(t, H) for _ in range(k)], [torch.empty((t, H), dtype=bf, device=dev) for _ in range(k)]
        ms, rs = torch.empty((t, 1), dtype=bf, device=dev), torch.empty((t, 1), dtype=bf, device=dev)
        fns = [lambda i=i: diopi.diopiLayerNorm(ctx, ys[i], ms, rs, xs[i], w, b, [H], 1e-5) for i in range(k)]
    elif name == "softmax":
        alg = 2 * es * n
        k = nsets(alg)
        xs, ys = [rn(t, H) for _ in range(k)], [torch.empty((t, H), dtype=bf, device=dev) for _ in range(k)]
        fns = [lambda i=i: diopi.diopiSoftmax(ctx, ys[i], xs[i], -1) for i in range(k)]
    elif name == "rope":
        alg = 2 * es * n + 2 * 4 * t * 64
        k = nsets(alg)
        inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2, device=dev).float() / 128))
        ang = torch.outer(torch.arange(t, device=dev).float(), inv)
        cos, sin = torch.cos(ang), torch.sin(ang)
        xs, ys = [rn(t, 32, 128) for _ in range(k)], [torch.empty((t, 32, 128), dtype=bf, device=dev) for _ in range(k)]
        fns = [lambda i=i: diopi.diopiRotaryEmbedding(ctx, ys[i], xs[i], cos, sin, False, False) for i in range(k)]
    elif name == "silu_mul":
        # as dispatched: silu (read + write) then mul (2 reads + write) = 5 * es * numel
        alg = 5 * es * n
        k = nsets(alg)
        gs, us, ys = [rn(t, H) for _ in range(k)], [rn(t, H) for _ in range(k)], [torch.empty((t, H), dtype=bf, device=dev) for _ in range(k)]

        def f(i):
            diopi.diopiSilu(ctx, ys[i], gs[i])
            diopi.diopiMul(ctx, ys[i], ys[i], us[i])
        fns = [lambda i=i: f(i) for i in range(k)]
    elif name == "add":
        alg = 3 * es * n
        k = nsets(alg)
        a, b, ys = [rn(t, H) for _ in range(k)], [rn(t, H) for _ in range(k)], [torch.empty((t, H), dtype=bf, device=dev) for _ in range(k)]
        fns = [lambda i=i: diopi.diopiAdd(ctx, ys[i], a[i], b[i], 1) for i in range(k)]
    elif name == "div_scalar":
        alg = 2 * es * n
        k = nsets(alg)
        a = [rn(t, H) for _ in range(k)]
        fns = [lambda i=i: diopi.diopiDivInpScalar(ctx, a[i], 11.313708498984761, 0) for i in range(k)]
    elif name == "mask_add":
        # [T/2048, 2048, 2048]-style broadcast add of a [2048, 2048] block needs T*H % 2048^2 == 0; use a [H] row broadcast otherwise
        alg = 2 * es * n
        k = nsets(alg)
        if t >= 1024 and t % 1024 == 0:
            a = [rn(t // 1024, 1024, H) for _ in range(k)]  # like [batch*heads, S, S] scores + an [S, S] mask
            blk = rn(1024, H)
        else:
            a = [rn(t, H) for _ in range(k)]
            blk = rn(H)
        fns = [lambda i=i: diopi.diopiAddInp(ctx, a[i], blk, 1) for i in range(k)]
    elif name == "cast_up":
        alg = 6 * n
        k = nsets(alg)
        xs, ys = [rn(t, H) for _ in range(k)], [torch.empty((t, H), dtype=torch.float32, device=dev) for _ in range(k)]
        fns = [lambda i=i: diopi.diopiCopyInp(ctx, xs[i], ys[i]) for i in range(k)]
    elif name == "cast_down":
        alg = 6 * n
        k = nsets(alg)
        xs, ys = [rn(t, H, dtype=torch.float32) for _ in range(k)], [torch.empty((t, H), dtype=bf, device=dev) for _ in range(k)]
        fns = [lambda i=i: diopi.diopiCopyInp(ctx, xs[i], ys[i]) for i in range(k)]
    elif name == "transpose_copy":
        # [B, S, 32, 128] -> [B, 32, S, 128] with B*S = T
        alg = 2 * es * n
        k = nsets(alg)
        s = min(t, 2048)
        b = max(t // s, 1)
        xs, ys = [rn(b, s, 32, 128) for _ in range(k)], [torch.empty((b, 32, s, 128), dtype=bf, device=dev) for _ in range(k)]
        fns = [lambda i=i: diopi.diopiCopyInp(ctx, xs[i].transpose(1, 2), ys[i]) for i in range(k)]
    elif name == "embedding":
        alg = 2 * es * n + 8 * t
        k = nsets(alg)
        table = rn(32000, H)
        ids = [torch.randint(0, 32000, (t,), generator=g, device=dev, dtype=torch.int64) for _ in range(k)]
        ys = [torch.empty((t, H), dtype=bf, device=dev) for _ in range(k)]
        fns = [lambda i=i: diopi.diopiIndexSelect(ctx, ys[i], table, 0, ids[i]) for i in range(k)]
    else:
        raise SystemExit("unknown op " + name)
    return fns, alg


MEM_OPS = ["rmsnorm", "layernorm", "softmax", "rope", "silu_mul", "cast_up", "cast_down", "embedding", "add", "div_scalar", "mask_add",
           "transpose_copy"]

# (label, batch, M, N, K, B layout): the 7B-shaped layer's contractions
GEMM_CASES = [
    ("prefill q/k/v/o proj", 1, 16384, 4096, 4096, "nk"),
    ("prefill gate/up proj", 1, 16384, 11008, 4096, "nk"),
    ("prefill down proj", 1, 16384, 4096, 11008, "nk"),
    ("prefill QK^T", 256, 2048, 2048, 128, "nk"),
    ("prefill PV", 256, 2048, 128, 2048, "kn"),
    ("decode q/k/v/o proj", 1, 64, 4096, 4096, "nk"),
    ("decode gate/up proj", 1, 64, 11008, 4096, "nk"),
    ("decode down proj", 1, 64, 4096, 11008, "nk"),
    ("decode QK^T", 2048, 1, 4096, 128, "nk"),
    ("decode PV", 2048, 1, 128, 4096, "kn"),
]


def gemm_case(case, diopi, ctx, dev):
    label, batch, m, n, k, layout = case
    bf = torch.bfloat16
    g = torch.Generator(device=dev)
    g.manual_seed(m + n + k)
    per_set = 2 * (batch * (m * k + n * k + m * n))
    sets = int(max(1, min(8, math.ceil(2.0 * L2_BYTES / per_set))))
    fns = []
    for _ in range(sets):
        if batch == 1:
            a = torch.randn((m, k), generator=g, device=dev, dtype=torch.float32).to(bf)
            b = (torch.randn((n, k) if layout == "nk" else (k, n), generator=g, device=dev, dtype=torch.float32) * 0.05).to(bf)
            out = torch.empty((m, n), dtype=bf, device=dev)
            bv = b.t() if layout == "nk" else b
            fns.append(lambda out=out, a=a, bv=bv: diopi.diopiMm(ctx, out, a, bv))
        else:
            a = torch.randn((batch, m, k), generator=g, device=dev, dtype=torch.float32).to(bf)
            b = (torch.randn((batch, n, k) if layout == "nk" else (batch, k, n), generator=g, device=dev, dtype=torch.float32) * 0.05).to(bf)
            out = torch.empty((batch, m, n), dtype=bf, device=dev)
            bv = b.transpose(1, 2) if layout == "nk" else b
            fns.append(lambda out=out, a=a, bv=bv: diopi.diopiBmm(ctx, out, a, bv))
    flops = 2.0 * batch * m * n * k
    return fns, flops, per_set


# (label, batch, seq_q, seq_kv, heads, kv_heads, causal): fused attention, head dim 128
ATTENTION_CASES = [
    ("prefill 7B causal", 8, 2048, 2048, 32, 32, True),
    ("prefill 7B full", 8, 2048, 2048, 32, 32, False),
    ("prefill 70B-shaped TP8 shard causal", 4, 4096, 4096, 8, 1, True),
    ("prefill long causal", 1, 16384, 16384, 32, 32, True),
    ("decode 7B, KV 4096", 64, 1, 4096, 32, 32, False),
    ("decode 70B-shaped TP8 shard, KV 4096", 64, 1, 4096, 8, 1, False),
    ("decode 7B, 4 sequences, KV 16384", 4, 1, 16384, 32, 32, False),
]


def attention_case(case, diopi, ctx, dev):
    label, b, sq, skv, h, hk, causal = case
    bf = torch.bfloat16
    g = torch.Generator(device=dev)
    g.manual_seed(b * skv + h)
    per_set = 2 * b * 128 * (2 * sq * h + 2 * skv * hk)   # q + out, k + v
    sets = int(max(1, min(8, math.ceil(2.0 * L2_BYTES / per_set))))
    fns = []
    for _ in range(sets):
        q = torch.randn((b, sq, h, 128), generator=g, device=dev, dtype=torch.float32).to(bf)
        # keys / values in the cache layout [B, kv heads, L, D], handed over as the [B, L, kv heads, D] view
        k = torch.randn((b, hk, skv, 128), generator=g, device=dev, dtype=torch.float32).to(bf).transpose(1, 2)
        v = torch.randn((b, hk, skv, 128), generator=g, device=dev, dtype=torch.float32).to(bf).transpose(1, 2)
        out = torch.empty_like(q)
        fns.append(lambda q=q, k=k, v=v, out=out: diopi.diopiMultiHeadAttention(ctx, q, k, v, 0.0, causal, False, 128 ** -0.5, out, None, None, None))
    # products actually needed: 4*d flop per visible (query, key) pair
    pairs = b * h * (sq * (sq + 1) // 2 + sq * (skv - sq) if causal else sq * skv)
    return fns, 4.0 * 128 * pairs, per_set


# (emulated ranks, rows, columns, K per rank): the 7B layer's o_proj / down_proj at TP 2 and 8, the 70B down_proj at TP 8
FUSED_LINEAR_CASES = [(2, 16384, 4096, 2048), (2, 16384, 4096, 5504), (8, 16384, 4096, 512), (8, 16384, 4096, 1376), (8, 16384, 8192, 3584)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="all", help="comma list of: %s, gemm, attention, sampling, fused_linear (not part of 'all')" % ", ".join(MEM_OPS))
    ap.add_argument("--tokens", default="1,64,1024,16384,65536")
    ap.add_argument("--gemm", default="all", help="comma list of indices into the GEMM case table, or 'all'")
    ap.add_argument("--attention", default="all", help="comma list of indices into the attention case table, or 'all'")
    ap.add_argument("--fused-linear", default="all", help="comma list of indices into the fused-linear case table, or 'all'")
    ap.add_argument("--iters", type=int, default=50)
    args = ap.parse_args()

    import __graft_entry__ as entry
    pkg = entry.load_package()
    assert torch.cuda.is_available(), "the sweep needs a CUDA device"
    pkg.install_caching_allocator()
    dev = "cuda:0"
    torch.cuda.set_device(0)
    diopi = pkg.diopi
    stream = torch.cuda.current_stream()
    ctx = diopi.Context(stream=stream.cuda_stream, device=0)
    hbm, tflops, src = peaks()
    ops = MEM_OPS + ["gemm", "attention", "sampling"] if args.ops == "all" else args.ops.split(",")
    tokens = [int(x) for x in args.tokens.split(",")]
    for op in ops:
        if op == "fused_linear":
            # Row-parallel linear with the all-reduce fused in, ranks emulated on this one device (all "peer" memory is local,
            # so the figures show the kernels' own cost without NVLink): the storing product, the pushing product, and the
            # reduce-gather kernel of rank 0 once every rank's pieces are there.
            bf = torch.bfloat16
            which = range(len(FUSED_LINEAR_CASES)) if args.fused_linear == "all" else [int(v) for v in args.fused_linear.split(",")]
            for n, m, cols, k in [FUSED_LINEAR_CASES[i] for i in which]:
                x = torch.randn((m, k), device=dev, dtype=bf)
                w = torch.randn((cols, k), device=dev, dtype=bf) * 0.02
                res = torch.randn((m, cols), device=dev, dtype=bf)
                out = torch.empty((m, cols), device=dev, dtype=bf)
                spaces = pkg.devapis.PeerSpace.emulated(n, m * cols * 2, 1)
                sp = spaces[0]
                flops = 2.0 * m * cols * k

                def push():
                    ep, _ = sp.begin(0)
                    diopi.diopiB200MmPush(ctx, x, w.t(), sp, 0, ep, 0)
                ms_mm = time_cases([lambda: diopi.diopiMm(ctx, out, x, w.t())], args.iters, stream)
                ms_push = time_cases([push], args.iters, stream)
                ep = 1 << 20
                for s_ in spaces:
                    diopi.diopiB200MmPush(ctx, x, w.t(), s_, 0, ep, 0)
                ms_red = time_cases([lambda: sp.reduce_gather(0, ep, res.data_ptr(), m, cols, diopi.DTYPE[bf], stream.cuda_stream)], args.iters, stream)
                shard = m * cols * 2 // n
                alg = (n + 1) * shard + n * shard  # n partial shards + residual shard read, the finished shard written to n ranks
                torch.cuda.synchronize()
                print(json.dumps({"op": "fused_linear", "ranks_emulated": n, "m": m, "n": cols, "k": k, "mm_store_ms": round(ms_mm, 4),
                                  "mm_store_tflops": round(flops / (ms_mm * 1e-3) / 1e12, 1), "mm_push_ms": round(ms_push, 4),
                                  "mm_push_tflops": round(flops / (ms_push * 1e-3) / 1e12, 1), "reduce_gather_ms": round(ms_red, 4),
                                  "reduce_gather_gbs": round(alg / (ms_red * 1e-3) / 1e9, 1),
                                  "frac_of_%s_hbm" % src: round(alg / (ms_red * 1e-3) / 1e9 / hbm, 4),
                                  "status": [diopi.gemm_status(), sp.status()]}), flush=True)
                for s_ in spaces:
                    s_.close()
                del x, w, res, out
                ctx.release_workspace()
            continue
        if op == "sampling":
            # one sampling step over a [64, 32000] fp32 logits matrix, each operator timed on its own
            b, v = 64, 32000
            g = torch.Generator(device=dev)
            g.manual_seed(7)
            logits = torch.randn((b, v), generator=g, device=dev, dtype=torch.float32)
            probs = torch.softmax(logits, -1)
            vals, idx = torch.empty_like(logits), torch.empty((b, v), dtype=torch.int64, device=dev)
            tv, ti = torch.empty((b, 50), device=dev), torch.empty((b, 50), dtype=torch.int64, device=dev)
            am, pick = torch.empty((b,), dtype=torch.int64, device=dev), torch.empty((b, 1), dtype=torch.int64, device=dev)
            cum = torch.empty_like(logits)
            cases = [("argmax", lambda: diopi.diopiArgmax(ctx, am, logits, 1, False), 4 * b * v),
                     ("topk k=50", lambda: diopi.diopiTopk(ctx, tv, ti, logits, 50, 1, True, True), 4 * b * v),
                     ("sort descending", lambda: diopi.diopiSort(ctx, vals, idx, probs, 1, True, True), 16 * b * v),
                     ("cumsum", lambda: diopi.diopiCumsum(ctx, cum, probs, 1), 8 * b * v),
                     ("multinomial 1 sample", lambda: diopi.diopiMultinomial(ctx, pick, probs, 1, True, None), 4 * b * v),
                     ("gather", lambda: diopi.diopiGather(ctx, pick, idx, 1, pick), 16 * b)]
            for label, fn, alg in cases:
                ms = time_cases([fn], args.iters, stream)
                print(json.dumps({"op": "sampling", "case": label, "rows": b, "vocabulary": v, "us": round(ms * 1e3, 2), "algorithmic_bytes": alg,
                                  "gbs": round(alg / (ms * 1e-3) / 1e9, 1)}), flush=True)
                ctx.release_workspace()
            continue
        if op == "attention":
            which = range(len(ATTENTION_CASES)) if args.attention == "all" else [int(x) for x in args.attention.split(",")]
            for case in [ATTENTION_CASES[i] for i in which]:
                fns, flops, per_set = attention_case(case, diopi, ctx, dev)
                ms = time_cases(fns, max(2, args.iters // 2), stream)
                rec = {"op": "attention", "case": case[0], "batch": case[1], "seq_q": case[2], "seq_kv": case[3], "heads": case[4], "kv_heads": case[5],
                       "causal": case[6], "ms": round(ms, 4), "tflops_visible_pairs": round(flops / (ms * 1e-3) / 1e12, 2),
                       "frac_of_%s_bf16_burst" % src: round(flops / (ms * 1e-3) / 1e12 / tflops, 4), "algorithmic_bytes": per_set,
                       "gbs": round(per_set / (ms * 1e-3) / 1e9, 1), "frac_of_%s_hbm" % src: round(per_set / (ms * 1e-3) / 1e9 / hbm, 4)}
                print(json.dumps(rec), flush=True)
                del fns
                ctx.release_workspace()
            continue
        if op == "gemm":
            idx = range(len(GEMM_CASES)) if args.gemm == "all" else [int(x) for x in args.gemm.split(",")]
            for i in idx:
                fns, flops, per_set = gemm_case(GEMM_CASES[i], diopi, ctx, dev)
                ms = time_cases(fns, max(5, args.iters // 2) if flops > 1e11 else args.iters, stream)
                label, batch, m, n, k, layout = GEMM_CASES[i]
                rec = {"op": "gemm", "case": label, "batch": batch, "m": m, "n": n, "k": k, "b_layout": layout, "ms": round(ms, 4),
                       "tflops": round(flops / (ms * 1e-3) / 1e12, 2), "frac_of_%s_bf16_burst" % src: round(flops / (ms * 1e-3) / 1e12 / tflops, 4),
                       "gbs": round(per_set / (ms * 1e-3) / 1e9, 1), "frac_of_%s_hbm" % src: round(per_set / (ms * 1e-3) / 1e9 / hbm, 4)}
                print(json.dumps(rec), flush=True)
                ctx.release_workspace()
            continue
        for t in tokens:
            fns, alg = mem_case(op, t, diopi, ctx, dev)
            ms = time_cases(fns, args.iters, stream)
            gbs = alg / (ms * 1e-3) / 1e9
            print(json.dumps({"op": op, "tokens": t, "hidden": H, "algorithmic_bytes": alg, "us": round(ms * 1e3, 2), "gbs": round(gbs, 1),
                              "frac_of_%s_hbm" % src: round(gbs / hbm, 4)}), flush=True)
            del fns
            ctx.release_workspace()
    assert diopi.gemm_status() == 0


if __name__ == "__main__":
    main()
