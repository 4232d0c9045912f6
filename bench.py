"""Benchmark of the hot path: decoder-layer tokens/s through the DIOPI C-ABI on the B200 vendor backend.

    python bench.py --gpus N --steps K --warmup W            # this repository's arm
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path (torch CPU aten), host cores

Workload (config.workload): the Llama-2-7B-shaped decoder layer in prefill, bf16, batch 8 x seq 2048 (16384 tokens),
hidden 4096, 32 heads x 128, SwiGLU 11008, causal attention through bmm + softmax, weights N(0, 0.02), activations from
seeded token ids through the embedding table [32000, 4096]. Everything is synthetic and seeded. With N > 1 GPUs the layer
is tensor-parallel (column-parallel q/k/v/gate/up, row-parallel o/down, diclAllReduce after o_proj and down_proj): total
work is fixed, so scaling is "strong".

A step is one layer forward over the 16384 tokens. `value` times steps whose input hidden states are resident in HBM;
`e2e` times the call a user makes with host buffers: token ids copied from pinned host memory, embedding lookup, layer,
and the layer output copied back to pinned host memory, every step. One JSON line is printed by rank 0.

Beside the timings the run checks what it timed, outside every timed region: the last output of each variant against the
CPU oracle on the rows of sequence 0 (`parity`), the decode outputs on four of the 64 sequences, with N > 1 every
collective of the communicator against closed-form values (`checks`), and at N = 1 the per-op sweep of the memory-bound
operators (`op_sweep`). A failed parity or collective check makes the process exit non-zero after the line is printed.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import bench_checks  # noqa: E402  (untimed checks: collectives against closed forms, parity figures against the CPU oracle)

SEED = 1234
VOCAB = 32000


class Cfg:
    def __init__(self, hidden=4096, heads=32, kv_heads=32, head_dim=128, ffn=11008, eps=1e-6, rope_base=10000.0, rope_layout="half"):
        self.hidden, self.heads, self.kv_heads, self.head_dim, self.ffn = hidden, heads, kv_heads, head_dim, ffn
        self.eps, self.rope_base, self.rope_layout = eps, rope_base, rope_layout


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops_burst": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks, power and throttle reasons through NVML (read-only queries) while the timed region runs."""

    def __init__(self, gpu_index, period_s=0.02):
        self.gpu_index, self.period_s = gpu_index, period_s
        self.samples, self.power, self.reasons = [], [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self.thread = None
        self.nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nvml = None
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        n = self.nvml
        names = {"hw_slowdown": getattr(n, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(n, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(n, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(n, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                self.power.append(n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
                mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(self.period_s)

    def stop(self):
        if self.nvml is None or self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self._stop.set()
        self.thread.join(timeout=2)
        sm = sorted(self.samples)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(sm), "power_w_max": max(self.power) if self.power else None}


def make_device_weights(cfg, device, dtype, seed=SEED):
    """Full (unsharded) N(0, 0.02) weights, identical on every rank (same seed), generated on the device."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def n(*shape):
        return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)

    d = cfg.head_dim
    return {
        "wq": n(cfg.heads * d, cfg.hidden), "wk": n(cfg.kv_heads * d, cfg.hidden), "wv": n(cfg.kv_heads * d, cfg.hidden),
        "wo": n(cfg.hidden, cfg.heads * d), "w1": n(cfg.ffn, cfg.hidden), "w3": n(cfg.ffn, cfg.hidden), "w2": n(cfg.hidden, cfg.ffn),
        "attention_norm": torch.ones(cfg.hidden, device=device, dtype=dtype), "ffn_norm": torch.ones(cfg.hidden, device=device, dtype=dtype),
    }


def workload_config(workload, cfg, batch, seq, n_layers, world):
    """The `config` object: the same for this repository's arm and for the reference arm of the same run."""
    tokens = batch * seq
    name = ("llama2-7b-shaped decoder layer, prefill, batch %d x seq %d, bmm+softmax attention" % (batch, seq)) if workload == "7b" \
        else ("stack of 4 llama2-70b-shaped decoder layers (GQA 64/8), prefill, batch %d x seq %d, bmm+softmax attention" % (batch, seq))
    weight_mb = (2 * (2 * cfg.hidden * cfg.heads * cfg.head_dim + 2 * cfg.hidden * cfg.kv_heads * cfg.head_dim + 3 * cfg.hidden * cfg.ffn)) >> 20
    return {"workload": name, "layers": n_layers, "kv_heads": cfg.kv_heads, "hidden": cfg.hidden, "heads": cfg.heads, "head_dim": cfg.head_dim,
            "ffn": cfg.ffn, "tokens_per_step": tokens, "parallelism": "tp%d" % world,
            "l2": "inputs larger than L2: weights %d MB per layer + %d MB per activation tensor, no flush" % (weight_mb, (tokens * cfg.hidden * 2) >> 20)}


def workload_shape(args):
    if args.workload == "70b":
        return Cfg(hidden=8192, heads=64, kv_heads=8, head_dim=128, ffn=28672), 4, 4096, 4
    return Cfg(), args.batch, args.seq, 1


def layer_flops(cfg, batch, seq, tp):
    t = batch * seq
    d = cfg.head_dim
    lin = 2 * t * (cfg.hidden * (cfg.heads * d) * 2 + cfg.hidden * (cfg.kv_heads * d) * 2 + 3 * cfg.hidden * cfg.ffn) / tp
    attn = 4 * batch * cfg.heads * seq * seq * d / tp
    return lin, attn


# ---------------------------------------------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """The reference's own CPU implementation of the path: DIPU's forced CPU fallback executes torch CPU aten kernels
    (CPUFallback.cpp:130). Timed on the host cores with all threads; a step is one forward pass over the whole batch of the
    workload (the same tokens per step as this repository's arm), fp32."""
    if rank != 0:
        return
    from oracle import llama_cpu
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg, batch, seq, n_layers = workload_shape(args)
    ws = [llama_cpu.make_weights(cfg, seed=SEED + 100 * li) for li in range(n_layers)]
    emb = llama_cpu.make_embedding(VOCAB, cfg.hidden, seed=SEED)
    ids = llama_cpu.make_token_ids(batch, seq, seed=SEED)

    def step():
        # the sequences of a batch are independent under the causal mask; they run one after the other so that the score
        # tensor of one sequence (heads x seq x seq fp32) is what is resident, as a host with bounded memory would run it
        for b in range(batch):
            x = emb[ids[b]]
            for w in ws:
                x = llama_cpu.decoder_layer_prefill_from_hidden(cfg, w, x, 1, seq)
        return x

    with torch.no_grad():
        for _ in range(max(min(args.warmup, 2), 1)):
            step()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step()
        dt = time.perf_counter() - t0
    tokens = batch * seq
    value = tokens * args.steps / dt
    sample = "the whole batch per step (%d sequences x %d tokens, one sequence at a time), fp32, torch CPU aten, %d threads" % (batch, seq, cores)
    line = {
        "impl": "reference", "metric": "decoder-layer tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, cfg, batch, seq, n_layers, args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_leg():
    """Bounded CPU sample for the cpu_baseline object of this repository's arm (rank 0, N = 1 only)."""
    from oracle import llama_cpu
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = llama_cpu.LayerConfig(hidden=4096, heads=32, kv_heads=32, head_dim=128, ffn=11008)
    w = llama_cpu.make_weights(cfg, seed=SEED)
    emb = llama_cpu.make_embedding(VOCAB, cfg.hidden, seed=SEED)
    ids = llama_cpu.make_token_ids(8, 2048, seed=SEED)[:1]
    with torch.no_grad():
        llama_cpu.decoder_layer_prefill(cfg, w, emb, ids)
        t0 = time.perf_counter()
        reps = 0
        while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 50):
            llama_cpu.decoder_layer_prefill(cfg, w, emb, ids)
            reps += 1
        dt = time.perf_counter() - t0
    return {"value": 2048 * reps / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": "%d forward passes over 1 of the 8 sequences (2048 tokens), fp32, torch CPU aten, %d threads" % (reps, cores)}


# ---------------------------------------------------------------------------------------------------------------------------
PREFILL_FORMS = {
    # name -> keyword arguments of the oracle's layer: all-fp32, and the op-by-op bf16 CPU path (every materialised tensor
    # rounded to bf16, what the reference's CPU fallback computes on bf16 tensors) in the three op orders that are timed
    "fp32": {},
    "bf16_stepwise": {"stepwise": True},
    "bf16_stepwise_baddbmm": {"stepwise": True, "scores_by_baddbmm": True},
    "bf16_stepwise_fused": {"stepwise": True, "fused": True},
}


def prefill_oracle_refs(cfg, host_weights, x0, seq, rank, dist, forms, world=1):
    """CPU oracle outputs for ONE sequence (rows [0, seq) of the batch: sequences are independent under the causal mask),
    computed on rank 0 from the same bf16-rounded weights and embedding rows the device holds, then handed to every rank.
    x0: [seq, hidden] float32 on the host (rank 0). world: the row-parallel linears are evaluated as `world` tensor-parallel
    ranks evaluate them (every rank's partial product rounded, then their sum), which is what the reference's path computes."""
    out = {}
    if rank == 0:
        from oracle import llama_cpu
        torch.set_num_threads(os.cpu_count() or 1)
        with torch.no_grad():
            for name in forms:
                kw = dict(PREFILL_FORMS[name])
                step = llama_cpu.stepwise(torch.bfloat16) if kw.pop("stepwise", False) else (lambda t: t)
                h = x0
                for w in host_weights:
                    h = llama_cpu.decoder_layer_prefill_from_hidden(cfg, w, h, 1, seq, step, tp=world, **kw)
                out[name] = h.contiguous()
    if dist is not None:
        for name in forms:
            t = out[name] if rank == 0 else torch.empty((seq, cfg.hidden), dtype=torch.float32)
            dist.broadcast(t, src=0)
            out[name] = t
    return out


def decode_oracle_refs(cfg, w, x4, kc4, vc4, position, world, rank, dist):
    """CPU oracle outputs of the decode step for the first sequences of the batch. kc4 / vc4: this rank's cache shard
    [n, local kv heads, L, D]; every rank fills its shard from the same seed, so the unsharded cache is the shard repeated
    over the ranks along the head dimension."""
    names = ("fp32", "bf16_stepwise", "bf16_stepwise_fused", "bf16_stepwise_fused_step")
    out = {}
    if rank == 0:
        from oracle import llama_cpu
        kc, vc = kc4.float().cpu().repeat(1, world, 1, 1), vc4.float().cpu().repeat(1, world, 1, 1)
        xf = x4.float().cpu()
        bf = llama_cpu.stepwise(torch.bfloat16)
        with torch.no_grad():
            out["fp32"] = llama_cpu.decoder_layer_decode(cfg, w, xf, kc, vc, position)[0]
            out["bf16_stepwise"] = llama_cpu.decoder_layer_decode(cfg, w, xf, kc, vc, position, step=bf, tp=world)[0]
            out["bf16_stepwise_fused"] = llama_cpu.decoder_layer_decode(cfg, w, xf, kc, vc, position, step=bf, fused=True, tp=world)[0]
            out["bf16_stepwise_fused_step"] = llama_cpu.decoder_layer_decode(cfg, w, xf, kc, vc, position, step=bf, fused=True, fused_gate_up=True,
                                                                             tp=world)[0]
    if dist is not None:
        for name in names:
            t = out[name].contiguous() if rank == 0 else torch.empty((x4.shape[0], cfg.hidden), dtype=torch.float32)
            dist.broadcast(t, src=0)
            out[name] = t
    return out


def all_ranks(flag, dist):
    """True when `flag` is true on every rank."""
    if dist is None:
        return bool(flag)
    t = torch.tensor([1 if flag else 0], dtype=torch.int64)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the secondary decode measurement")
    ap.add_argument("--decode-steps", type=int, default=200, help="graph replays timed per decode variant (a quarter of it for the eager one)")
    ap.add_argument("--no-parity", action="store_true", help="skip the (untimed) comparison of every variant's output with the CPU oracle")
    ap.add_argument("--no-checks", action="store_true", help="N > 1: skip the (untimed) closed-form checks of the collectives")
    ap.add_argument("--no-op-sweep", action="store_true", help="N = 1: skip the per-op sweep of the memory-bound operators")
    ap.add_argument("--no-caching-allocator", action="store_true", help="let torch use its own allocator for tensors")
    ap.add_argument("--workload", default="7b", choices=["7b", "70b"],
                    help="7b: one Llama-2-7B-shaped layer, batch 8 x seq 2048 (default). 70b: a stack of four Llama-2-70B-shaped "
                         "layers (GQA 64/8), batch 4 x seq 4096, meant for --gpus 2/4/8")
    ap.add_argument("--fused-collective-parts", default="1", choices=["1", "2", "both"],
                    help="N > 1: time the fused-collective variants with the batch in one piece (measured fastest at 2, 4 and 8 GPUs), "
                         "in two interleaved halves, or both")
    ap.add_argument("--overlap", default="auto", choices=["auto", "on", "off"],
                    help="tensor-parallel prefill: interleave two half-batches so the all-reduces overlap compute")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import __graft_entry__ as entry
    pkg = entry.load_package()  # raises when the CUDA libraries are missing: there is no fallback path
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the product has no CPU path")
    if not args.no_caching_allocator:
        pkg.install_caching_allocator()
    torch.cuda.set_device(local_rank)
    device = "cuda:%d" % local_rank
    from dipu_b200 import devapis, diopi
    from dipu_b200 import layer as L

    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo", rank=rank, world_size=world)  # control plane only: barriers and timing exchange
    tp_group = None
    if world > 1:
        uid = [devapis.diclGetUniqueId() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)  # the unique id travels through the store as bytes, as in ProcessGroupDICL
        tp_group = L.TpGroup(rank, world, uid[0], local_rank)

    dtype = torch.bfloat16
    cfg, batch, seq, n_layers = workload_shape(args)
    if args.workload == "70b":
        args.no_decode = True
        args.no_cpu_baseline = True
        args.no_op_sweep = True
    tokens = batch * seq
    layers = []
    host_weights = []  # rank 0: the full (unsharded) bf16 weights as float32 on the host, for the oracle of the parity checks
    for li in range(n_layers):
        weights = make_device_weights(cfg, device, dtype, seed=SEED + 100 * li)
        layers.append(L.DecoderLayer(cfg, weights, dtype=dtype, device=device, tp_rank=rank, tp_size=world, tp_group=tp_group))
        if rank == 0 and not args.no_parity:
            host_weights.append({k: v.float().cpu() for k, v in weights.items()})
        del weights
    for l_ in layers:
        l_.overlap_comm = (world >= 4) if args.overlap == "auto" else (args.overlap == "on")
    lay = layers[0]
    g = torch.Generator(device=device)
    g.manual_seed(SEED + 1)
    table = (torch.randn((VOCAB, cfg.hidden), generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)
    gi = torch.Generator()
    gi.manual_seed(SEED + 2)
    ids_host = torch.randint(0, VOCAB, (batch, seq), generator=gi, dtype=torch.int64).pin_memory()
    ids_dev = torch.empty((batch, seq), dtype=torch.int64, device=device)
    # the layer output is replicated after the last all-reduce: every rank returns its own 1/N of the token rows to its host
    # process, so the N PCIe links share the transfer (N = 1: the whole tensor)
    rows_per_rank = (tokens + world - 1) // world
    row_lo = min(rank * rows_per_rank, tokens)
    row_hi = min(row_lo + rows_per_rank, tokens)
    out_host = [torch.empty((max(row_hi - row_lo, 1), cfg.hidden), dtype=dtype).pin_memory() for _ in range(2)]  # double-buffered results
    copy_stream = devapis.getStreamFromPool(local_rank)   # D2H of step i overlaps the compute of step i+1
    copy_events = [devapis.getEventFromPool(), devapis.getEventFromPool()]
    done_events = [devapis.getEventFromPool(), devapis.getEventFromPool()]

    # Work runs on the runtime's default stream for the device: a created, non-blocking stream as in DIPU (the legacy NULL
    # stream cannot be captured into a graph and serialises against every other stream).
    torch.cuda.synchronize()
    stream = torch.cuda.ExternalStream(devapis.getDefaultStream(local_rank), device=device)
    torch.cuda.set_stream(stream)
    ctx = diopi.Context(stream=stream.cuda_stream, device=local_rank)
    x = L.embed(table, ids_host.to(device), ctx)  # resident input of the device-timed region

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def run_layers(h):
        for l_ in layers:
            h = l_.prefill(h, batch, seq, ctx)
        return h

    def step_resident():
        return run_layers(x)

    e2e_state = {"i": 0}

    def step_e2e():
        """Host buffers in, host buffers out. The result goes back on a pool stream, handed over with events the way DIPU's
        non-blocking copies do; the allocator is told that the copy stream still reads the block (record_stream)."""
        i = e2e_state["i"] & 1
        e2e_state["i"] += 1
        devapis.memCopyH2DAsync(stream.cuda_stream, ids_host.numel() * 8, ids_dev.data_ptr(), ids_host.data_ptr())  # this step's input
        h = L.embed(table, ids_dev, ctx)
        y = run_layers(h)
        if row_hi <= row_lo:
            return y
        devapis.recordEvent(copy_events[i], stream.cuda_stream)
        devapis.streamWaitEvent(copy_stream, copy_events[i])
        if e2e_state["i"] > 2:
            devapis.waitEvent(done_events[i])  # the host buffer's previous copy (two steps back) has landed
        row_bytes = cfg.hidden * y.element_size()
        devapis.memCopyD2HAsync(copy_stream, (row_hi - row_lo) * row_bytes, out_host[i].data_ptr(), y.data_ptr() + row_lo * row_bytes)  # this step's result
        devapis.recordEvent(done_events[i], copy_stream)
        if not args.no_caching_allocator:
            devapis.CachingAllocator.recordStream(y.data_ptr(), copy_stream)
        else:
            y.record_stream(torch.cuda.ExternalStream(copy_stream))
        return y

    # ---- device-resident timing ----
    if tp_group is not None:
        # communicator set-up, not part of any step: NCCL picks its channels and registers buffers during its first calls
        # on a message size, which would otherwise fall into the first timed steps
        scratch = torch.empty((tokens, cfg.hidden), dtype=dtype, device=device)
        for _ in range(10):
            tp_group.all_reduce_(scratch, stream.cuda_stream)
        torch.cuda.synchronize()
        del scratch
    for _ in range(args.warmup):
        step_resident()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for l_ in layers:
        l_.launches = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step_resident()
    e1.record(stream)
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    launches = sum(l_.launches for l_ in layers)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end-to-end timing (host buffers in, host buffers out) ----
    # warm-up of this leg: the two result buffers' copies keep two output blocks alive beside the step's own, so the caching
    # allocator reaches its steady pool only after a few steps (a cudaMalloc inside the timed region costs milliseconds)
    for _ in range(max(4, args.warmup)):
        step_e2e()
    barrier()
    devapis.syncStream(copy_stream)
    e0.record(stream)
    for _ in range(args.steps):
        step_e2e()
    # the timed region ends when the last result has landed in host memory
    devapis.recordEvent(copy_events[0], copy_stream)
    devapis.streamWaitEvent(stream.cuda_stream, copy_events[0])
    e1.record(stream)
    barrier()
    devapis.syncStream(copy_stream)
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))

    # ---- parity of what was timed (outside every timed region) ----
    parity = {}
    refs = None
    # Whole prefill layer at the benchmarked shapes: 1e-2 against the op-by-op bf16 CPU path, and against fp32 no further than
    # 1.25 x that CPU path's own distance from fp32 (bench_checks.py states why); "fp32" below stands for that bound.
    SW = LOOSE = bench_checks.layer_rel_bound(world)
    if not args.no_parity:
        forms = ["fp32", "bf16_stepwise", "bf16_stepwise_fused"] + (["bf16_stepwise_baddbmm"] if args.workload == "7b" else [])
        x0 = x[:seq].float().cpu() if rank == 0 else None
        refs = prefill_oracle_refs(cfg, host_weights, x0, seq, rank, dist, forms, world)

    def layerwise_parity(form, bound):
        """Every layer of the stack (with the variant flags as they are now) against the op-by-op oracle of THAT layer on the
        input the device layer had: rows of sequence 0, rank 0 computes, every rank compares its own copy."""
        kw = dict(PREFILL_FORMS[form])
        kw.pop("stepwise", None)
        res = []
        h = x
        for i, l_ in enumerate(layers):
            h_in = h[:seq].float().cpu() if rank == 0 else None
            h = l_.prefill(h, batch, seq, ctx)
            torch.cuda.synchronize()
            want = torch.empty((seq, cfg.hidden), dtype=torch.float32)
            if rank == 0:
                from oracle import llama_cpu
                with torch.no_grad():
                    want = llama_cpu.decoder_layer_prefill_from_hidden(cfg, host_weights[i], h_in, 1, seq, llama_cpu.stepwise(torch.bfloat16),
                                                                       tp=world, **kw).contiguous()
            if dist is not None:
                dist.broadcast(want, src=0)
            e = bench_checks.parity_entry(h[:seq], {form: (want, bound)})
            res.append({"layer": i, "max_abs": e[form]["max_abs"], "max_abs_bound": e[form]["max_abs_bound"], "rel_l2": e[form]["rel_l2"],
                        "rel_l2_bound": e[form]["rel_l2_bound"], "ok": e["ok"]})
        return res

    def record_parity(name, y, against):
        """Rows of sequence 0 of a variant's last output against the oracle forms in `against` ({form: relative-L2 bound});
        every rank checks its own (replicated) copy."""
        if refs is None:
            return
        bf16_form = [f for f in against if f != "fp32"][0]
        bounds = {f: (b if f != "fp32" else bench_checks.fp32_bound(refs[bf16_form], refs["fp32"])) for f, b in against.items()}
        if len(layers) > 1:
            # A stack: two bf16 evaluations drift apart from layer to layer (at 4 layers of the 70B shape the CPU bf16 path is
            # itself 5.5e-2 from fp32), so the single-layer bound against the op-by-op path is applied LAYER BY LAYER, every
            # layer's oracle fed with the input the device layer had; the whole stack is held to the fp32 bound (1.25 x the CPU
            # bf16 path's own distance) and its distance from the op-by-op path is reported beside it.
            entry = bench_checks.parity_entry(y[:seq], {"fp32": (refs["fp32"], bounds["fp32"])})
            mx, rl = bench_checks.errors(y[:seq], refs[bf16_form])
            entry[bf16_form + "_whole_stack"] = {"max_abs": round(mx, 6), "rel_l2": round(rl, 6)}
            per_layer = layerwise_parity("bf16_stepwise_baddbmm" if "baddbmm" in name else bf16_form, against[bf16_form])
            entry["layer_by_layer"] = per_layer
            entry["ok"] = bool(entry["ok"] and all(e["ok"] for e in per_layer))
        else:
            entry = bench_checks.parity_entry(y[:seq], {f: (refs[f], bounds[f]) for f in against})
        entry["cpu_bf16_path_vs_fp32_rel_l2"] = round(bench_checks.errors(refs[bf16_form], refs["fp32"])[1], 6)
        entry["all_ranks_ok"] = all_ranks(entry["ok"], dist)
        entry["rows_checked"] = "sequence 0 (%d tokens)" % seq
        parity[name] = entry

    y_lit = step_resident()
    torch.cuda.synchronize()
    record_parity("literal", y_lit, {"bf16_stepwise": SW, "fp32": LOOSE})
    if refs is not None and row_hi > row_lo:
        # the end-to-end leg's last host copy holds the rows this rank returns: the same bits as the device-resident result
        last = (e2e_state["i"] - 1) & 1
        got, want = out_host[last][: row_hi - row_lo].float(), y_lit[row_lo:row_hi].float().cpu()
        gap = (got - want).abs().max().item()
        parity["e2e_host_copy"] = {"equals_device_result_bitwise": bool(torch.equal(got, want)), "max_abs_vs_device_result": gap,
                                   "ok": bool(gap <= bench_checks.MAX_ABS), "all_ranks_ok": all_ranks(gap <= bench_checks.MAX_ABS, dist)}
    del y_lit

    # ---- per-op device times: the same step with events around every DIOPI call ----
    per_op = {}

    def make_timed(orig_call):
        def timed_call(fn, c, *a):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            r = orig_call(fn, c, *a)
            e.record(stream)
            per_op.setdefault(fn.__name__, []).append((s, e, a))
            return r
        return timed_call

    originals = [l_._call for l_ in layers]
    for l_ in layers:
        l_._call = make_timed(l_._call)
    reps = 3
    for _ in range(reps):
        step_resident()
    torch.cuda.synchronize()
    for l_, o_ in zip(layers, originals):
        l_._call = o_
    peaks = measured_peaks()
    ops = {}
    mm_flops, mm_ms, bmm_flops, bmm_ms = 0.0, 0.0, 0.0, 0.0
    for name, recs in per_op.items():
        ms = sum(s.elapsed_time(e) for s, e, _ in recs) / reps
        ops[name] = {"ms_per_step": round(ms, 4), "calls_per_step": len(recs) // reps}
        if name in ("diopiMm", "diopiBmm"):
            fl = 0.0
            for _, _, a in recs:
                out, a0, b0 = a[0], a[1], a[2]
                fl += 2.0 * out.numel() * a0.shape[-1]
            fl /= reps
            ops[name]["tflops"] = round(fl / (ms * 1e-3) / 1e12, 1)
            if name == "diopiMm":
                mm_flops, mm_ms = fl, ms
            else:
                bmm_flops, bmm_ms = fl, ms
        else:
            # bytes moved: every tensor argument once per appearance (an output that is also an input, diopiSoftmax(x, x),
            # is read and written), plus the write of the first operand of an in-place function; a gather reads rows, not
            # the table
            by = 0.0
            for _, _, a in recs:
                if name == "diopiIndexSelect":
                    by += 2 * a[0].numel() * a[0].element_size() + a[3].numel() * a[3].element_size()
                    continue
                for t in a:
                    if isinstance(t, torch.Tensor) and t.is_cuda:
                        by += t.numel() * t.element_size()
                if name.endswith("Inp") or name.endswith("InpScalar"):
                    by += a[0].numel() * a[0].element_size()  # read-modify-write of the first operand
            by /= reps
            ops[name]["gbs"] = round(by / (ms * 1e-3) / 1e9, 1)
    mm_calls = ops.get("diopiMm", {}).get("calls_per_step", 1)
    achieved = mm_flops / (mm_ms * 1e-3) / 1e12 if mm_ms > 0 else 0.0
    # DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the projection GEMMs at the single-GPU 7B
    # shapes, from one ncu capture of `opsweep.py --ops gemm --gemm 0,1,2`: q/k/v/o 447.6 MB (x4), gate/up 1216.5 MB (x2),
    # down 2087 MB (x1); algorithmic 302 / 585 / 585 MB. Other shapes (tensor-parallel shards, the 70B stack): not captured.
    traffic = None
    if world == 1 and args.workload == "7b" and (batch, seq) == (8, 2048):
        traffic = (4 * 447.6e6 + 2 * 1216.5e6 + 2087.0e6) / 7
    roofline = {"bound": "tensor", "kernel": "gemm_tc_pair_kernel / gemm_tc_kernel (diopiMm: the 7 projection GEMMs of the layer)",
                "achieved": round(achieved, 1),
                "peak": peaks["tflops_sustained"], "unit": "TFLOP/s", "frac": round(achieved / peaks["tflops_sustained"], 4),
                "peak_source": "%s bf16 cuBLAS, sustained (kernel timed inside a long step)" % peaks["source"],
                "flops_per_launch": mm_flops / max(mm_calls, 1), "ms_per_launch": mm_ms / max(mm_calls, 1), "traffic": traffic,
                "traffic_unit": "bytes per launch (mean over the 7 launches), ncu dram__bytes_read.sum + dram__bytes_write.sum",
                "traffic_source": "one ncu capture of the three projection shapes (profiles/gemm_tc_pair_kernel_prefill_gate_up_16384x11008x4096.md); "
                                  "a constant of that capture, not re-measured in this run",
                "algorithmic_bytes_per_launch": (4 * 302.0e6 + 3 * 585.1e6) / 7 if traffic else None}

    # ---- variant: attention scores through one baddbmm (scale and mask-add in the GEMM epilogue) ----
    # `value` above is the reference block's literal op order (bmm, div, add, softmax, bmm). A model written with
    # torch.baddbmm(mask, q, k^T, alpha=1/sqrt(d)) reaches diopiBaddbmm instead; timed here with the same K steps.
    def time_steps():
        """Three warm-up steps, then K timed steps (device events, max over ranks). Returns (ms, the last step's output)."""
        y = None
        for _ in range(3):
            step_resident()
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            y = step_resident()
        e1.record(stream)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)), y

    for l_ in layers:
        l_.scores_by_baddbmm = True
    ms_badd, y_v = time_steps()
    record_parity("attention_scores_by_baddbmm", y_v, {("bf16_stepwise_baddbmm" if args.workload == "7b" else "bf16_stepwise"): SW, "fp32": LOOSE})
    for l_ in layers:
        l_.scores_by_baddbmm = False
    variants = {"attention_scores_by_baddbmm": {"value": tokens * args.steps / (ms_badd * 1e-3), "unit": "tokens/s",
                                                "ms_per_step": ms_badd / args.steps,
                                                "note": "diopiBaddbmm(mask, q, k^T, beta=1, alpha=1/sqrt(d)) replaces diopiBmm + diopiDivInpScalar + diopiAddInp"}}

    # ---- variant: attention through the fused operator (diopiMultiHeadAttention: no score tensor, no transposes) ----
    for l_ in layers:
        l_.fused_attention = True
    ms_fused, y_v = time_steps()
    # the fused operator rounds its probabilities at another point than any op-by-op evaluation can: whole-layer bound 1e-2
    record_parity("fused_attention", y_v, {"bf16_stepwise_fused": LOOSE, "fp32": LOOSE})
    for l_ in layers:
        l_.fused_attention = False
    variants["fused_attention"] = {"value": tokens * args.steps / (ms_fused * 1e-3), "unit": "tokens/s", "ms_per_step": ms_fused / args.steps,
                                   "note": "diopiMultiHeadAttention (causal) replaces the transposes, diopiBmm, diopiDivInpScalar, diopiAddInp, "
                                           "diopiSoftmax, diopiBmm of the attention core"}
    del y_v

    # ---- variants (N > 1): row-parallel linears with the all-reduce and the residual add fused into the kernels ----
    # diopiB200MmPush pushes each output tile to the rank that owns its rows while the product is still running; one
    # reduce-gather kernel per linear sums the pieces, adds the residual and writes the finished rows to every rank. No
    # library collective and no separate diopiAdd on this path.
    if world > 1 and tokens % (256 * world) == 0 and cfg.hidden % 256 == 0:
        choices = [1, 2] if args.fused_collective_parts == "both" else [int(args.fused_collective_parts)]
        for parts in choices:
            if batch % parts != 0 or (tokens // parts) % (256 * world) != 0:
                continue
            try:
                tp_group.enable_fused_linear(tokens // parts, cfg.hidden, parts, on_comm_stream=(parts > 1))
            except Exception as exc:  # e.g. peer mappings refused on this host: report it, keep the line
                variants["fused_collective"] = {"unavailable": str(exc)[:200]}
                break
            for l_ in layers:
                l_.fused_collective = True
            for fused_attn in (False, True):
                for l_ in layers:
                    l_.fused_attention = fused_attn
                ms_v, y_v = time_steps()
                ok = tp_group.space.status() == 0 and diopi.gemm_status() == 0
                name = ("fused_attention_" if fused_attn else "") + "fused_collective" + ("_interleaved_halves" if parts > 1 else "")
                # one rounding (fp32 sum + residual) where the op-by-op path has two: whole-layer bound 1e-2 against either oracle
                record_parity(name, y_v, {("bf16_stepwise_fused" if fused_attn else "bf16_stepwise"): LOOSE, "fp32": LOOSE})
                del y_v
                variants[name] = {"value": tokens * args.steps / (ms_v * 1e-3), "unit": "tokens/s", "ms_per_step": ms_v / args.steps, "status_ok": ok,
                                  "note": "diopiB200MmPush + peer reduce-gather replace diopiMm + diclAllReduce + diopiAdd after the attention "
                                          "and FFN blocks" + ("; two half-batches interleaved, reductions on the communication stream" if parts > 1 else "")}
            for l_ in layers:
                l_.fused_collective = False
                l_.fused_attention = False
            barrier()
            tp_group.disable_fused_linear()

    # ---- secondary measurement: the same layer in decode (batch 64, KV length 4096) ----
    decode = None
    if not args.no_decode:
        decode = run_decode(lay, cfg, ctx, stream, device, dtype, world, barrier, max_over_ranks, peaks, rank, dist,
                            host_weights[0] if host_weights else None, not args.no_parity, max(1, args.decode_steps))
        if decode.get("parity") is not None:
            parity["decode"] = decode.pop("parity")

    # ---- N > 1: every collective of the communicator against closed-form values, at the world size of this run ----
    checks = None
    if world > 1 and not args.no_checks:
        def exchange(obj, src):
            box = [obj]
            dist.broadcast_object_list(box, src=src)
            return box[0]
        barrier()
        checks = bench_checks.collective_checks(devapis, diopi.DTYPE, tp_group.comm, tp_group.stream, rank, world, device, exchange)
        barrier()
        checks.update(bench_checks.peer_all_reduce_checks(devapis, diopi.DTYPE, tp_group.comm, tp_group.stream, rank, world, device))
        barrier()
        mine = all(v for k, v in checks.items() if isinstance(v, bool))
        checks["all_ranks_ok"] = all_ranks(mine, dist)

    # ---- N = 1: the per-op sweep of the memory-bound operators (bf16 [T, 4096], T in {1, 64, 1024, 16384, 65536}) ----
    op_sweep = None
    if world == 1 and not args.no_op_sweep:
        op_sweep = run_op_sweep(diopi, ctx, device, stream, peaks)

    if rank == 0:
        lin, attn = layer_flops(cfg, batch, seq, world)
        lin, attn = lin * n_layers, attn * n_layers
        value = tokens * args.steps / (ms_total * 1e-3)
        e2e_value = tokens * args.steps / (ms_e2e * 1e-3)
        line = {
            "metric": "decoder-layer tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": workload_config(args.workload, cfg, batch, seq, n_layers, world),
            "setup": {"overlap_allreduce": bool(lay.overlap_comm and world > 1),
                      "allocator": "torch default" if args.no_caching_allocator else "b200 caching allocator (pluggable)"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": ids_host.numel() * 8,
                    "d2h_bytes_per_step": tokens * cfg.hidden * 2,
                    "note": "result copied back on a pool stream, overlapping the next step's compute"
                            + ("" if world == 1 else "; each rank returns its 1/%d of the (replicated) output rows" % world)},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": roofline,
            "layer_tflops": round((lin + attn) * args.steps / (ms_total * 1e-3) / 1e12, 1),
            "ops": ops,
            "variants": variants,
            "decode": decode,
            "parity": parity if not args.no_parity else None,
            "checks": checks,
            "op_sweep": op_sweep,
            "gemm_status": diopi.gemm_status(),
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg()
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    failed = [k for k, v in parity.items() if not (v.get("ok", True) and v.get("all_ranks_ok", True))]
    if checks is not None and not checks.get("all_ranks_ok", True):
        failed.append("checks")
    if tp_group is not None:
        barrier()
        tp_group.close()
    if dist is not None:
        dist.destroy_process_group()
    if failed:
        sys.stderr.write("bench.py: rank %d: checks failed: %s\n" % (rank, ", ".join(failed)))
        sys.exit(1)


def run_op_sweep(diopi, ctx, device, stream, peaks):
    """The op sweep of the workload description: each memory-bound operator on bf16 [T, 4096], T in {1, 64, 1024, 16384,
    65536} (cases, buffers and algorithmic bytes as in opsweep.py: enough distinct buffer sets per case to exceed L2,
    CUDA events on the launching stream). T >= 16384 is reported as GB/s and fraction of the measured copy bandwidth, the
    small T as latency: `us` with one host call per launch (the host's per-call cost bounds it), `us_graph` with the same
    launches replayed from one CUDA graph (the device's own pace), the latter also as GB/s."""
    import opsweep
    from dipu_b200 import devapis
    out = {"unit": "GB/s of algorithmic bytes; frac = of %s HBM copy bandwidth (%.0f GB/s)" % (peaks["source"], peaks["hbm_gbs"]), "ops": {}}

    def graph_time(fns, iters):
        devapis.graphBeginCapture(stream.cuda_stream)
        try:
            for i in range(iters):
                fns[i % len(fns)]()
        finally:
            graph = devapis.graphEndCapture(stream.cuda_stream)
        devapis.graphLaunch(graph, stream.cuda_stream)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        devapis.graphLaunch(graph, stream.cuda_stream)
        e1.record(stream)
        torch.cuda.synchronize()
        devapis.graphDestroy(graph)
        return e0.elapsed_time(e1) / iters

    for op in ("rmsnorm", "layernorm", "softmax", "rope", "silu_mul", "cast_up", "cast_down", "embedding", "add"):
        rec = {}
        for t in (1, 64, 1024, 16384, 65536):
            fns, alg = opsweep.mem_case(op, t, diopi, ctx, device)
            ms = opsweep.time_cases(fns, 30 if t >= 16384 else 100, stream)
            gbs = alg / (ms * 1e-3) / 1e9
            if t >= 16384:
                rec["T=%d" % t] = {"us": round(ms * 1e3, 2), "gbs": round(gbs, 1), "frac": round(gbs / peaks["hbm_gbs"], 4)}
            else:
                ms_g = graph_time(fns, 100)
                rec["T=%d" % t] = {"us": round(ms * 1e3, 2), "us_graph": round(ms_g * 1e3, 2), "gbs_graph": round(alg / (ms_g * 1e-3) / 1e9, 1),
                                   "frac_graph": round(alg / (ms_g * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}
            del fns
            ctx.release_workspace()
        out["ops"][op] = rec
    torch.cuda.synchronize()
    out["cpu"] = cpu_op_sweep(16384)
    return out


def cpu_op_sweep(t):
    """The same operators on the host cores at one size (the arithmetic of the reference's CPU fallback: torch CPU aten on
    bf16-rounded inputs computed in fp32, all threads): a reported baseline beside the device figures, a few seconds of work."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator()
    g.manual_seed(t)
    h = 4096
    x = torch.randn((t, h), generator=g).bfloat16().float()
    y = torch.randn((t, h), generator=g).bfloat16().float()
    w = torch.ones(h)
    ids = torch.randint(0, VOCAB, (t,), generator=g)
    table = torch.randn((VOCAB, h), generator=g).bfloat16()
    inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2).float() / 128))
    ang = torch.outer(torch.arange(t).float(), inv)
    cos, sin = torch.cos(ang).view(t, 1, 64), torch.sin(ang).view(t, 1, 64)

    def rope():
        v = x.view(t, 32, 128)
        a, b = v[..., :64], v[..., 64:]
        return torch.cat((a * cos - b * sin, a * sin + b * cos), -1)

    cases = {
        "rmsnorm": lambda: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w,
        "layernorm": lambda: torch.nn.functional.layer_norm(x, (h,), w, w, 1e-5),
        "softmax": lambda: torch.softmax(x, -1),
        "rope": rope,
        "silu_mul": lambda: torch.nn.functional.silu(x) * y,
        "cast_up": lambda: table[:t].float(),
        "cast_down": lambda: x.bfloat16(),
        "embedding": lambda: table[ids],
        "add": lambda: x + y,
    }
    res = {}
    with torch.no_grad():
        for name, fn in cases.items():
            fn()
            t0 = time.perf_counter()
            reps = 0
            while reps < 3 or (time.perf_counter() - t0 < 0.3 and reps < 20):
                fn()
                reps += 1
            res[name] = {"us": round((time.perf_counter() - t0) / reps * 1e6, 1)}
    return {"tokens": t, "cores": cores, "kind": "port (torch CPU aten, fp32 compute on bf16-rounded inputs)", "ops": res}


def run_decode(lay, cfg, ctx, stream, device, dtype, world, barrier, max_over_ranks, peaks, rank=0, dist=None, host_w=None, check=False, graph_steps=200):
    """7B-shaped layer in decode: batch 64, one new token per sequence, bf16 KV cache of length 4096 per sequence."""
    b, length = 64, 4096
    n_check = 4  # sequences whose output is compared with the CPU oracle
    outs = {}
    g = torch.Generator(device=device)
    g.manual_seed(SEED + 3)
    kc = torch.randn((b, lay.kv_heads, length, cfg.head_dim), generator=g, device=device, dtype=torch.float32).to(dtype)
    vc = torch.randn((b, lay.kv_heads, length, cfg.head_dim), generator=g, device=device, dtype=torch.float32).to(dtype)
    xd = (torch.randn((b, cfg.hidden), generator=g, device=device, dtype=torch.float32) * 0.5).to(dtype)
    for _ in range(5):
        lay.decode(xd, kc, vc, length - 1, ctx)
    barrier()
    steps = max(1, graph_steps // 4)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        lay.decode(xd, kc, vc, length - 1, ctx)
    e1.record(stream)
    barrier()
    ms_eager = max_over_ranks(e0.elapsed_time(e1)) / steps
    outs["eager"] = lay.decode(xd, kc, vc, length - 1, ctx)[:n_check].clone()
    # the same step captured once into a CUDA graph and replayed: one launch per step instead of ~30 host-side calls
    from dipu_b200 import devapis
    replay, out_g = lay.capture_decode(xd, kc, vc, length - 1, ctx)
    for _ in range(5):
        replay()
    barrier()
    steps = graph_steps
    e0.record(stream)
    for _ in range(steps):
        replay()
    e1.record(stream)
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / steps
    outs["graph"] = out_g[:n_check].clone()
    devapis.graphDestroy(replay.graph)
    # variant: the attention core through the fused operator (K and V read once, no score tensor), again graph-replayed
    lay.fused_attention = True
    for _ in range(3):
        lay.decode(xd, kc, vc, length - 1, ctx)
    replay, out_g = lay.capture_decode(xd, kc, vc, length - 1, ctx)
    for _ in range(5):
        replay()
    barrier()
    e0.record(stream)
    for _ in range(steps):
        replay()
    e1.record(stream)
    barrier()
    ms_fused = max_over_ranks(e0.elapsed_time(e1)) / steps
    outs["fused_attention"] = out_g[:n_check].clone()
    devapis.graphDestroy(replay.graph)
    # variant: the whole step through the fused entry points (one q/k/v projection, rotary + cache append, add + RMSNorm,
    # SiLU * up in the epilogue of one gate / up product, the last residual add in the down projection): eight launches instead of nineteen
    lay.fused_decode = True
    for _ in range(3):
        lay.decode(xd, kc, vc, length - 1, ctx)
    replay, out_g = lay.capture_decode(xd, kc, vc, length - 1, ctx)
    for _ in range(5):
        replay()
    barrier()
    e0.record(stream)
    for _ in range(steps):
        replay()
    e1.record(stream)
    barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1)) / steps
    outs["fused_step"] = out_g[:n_check].clone()
    devapis.graphDestroy(replay.graph)
    lay.fused_decode = False
    # tensor parallel: the two 512 KiB partial sums per step reduced by ONE kernel over peer memory on the compute stream
    # (b200_dicl_peer_all_reduce) instead of ncclAllReduce on the communication stream; fused attention stays on
    ms_peer = None
    ms_step_peer = None
    peer_ok = False
    if world > 1 and lay.tp_group is not None:
        try:
            lay.tp_group.enable_peer_reduce(1 << 20)
            peer_ok = True
        except Exception:  # peer mappings refused on this host: the variant is reported as absent
            lay.tp_group.peer = None
    if peer_ok:
        barrier()
        for _ in range(3):
            lay.decode(xd, kc, vc, length - 1, ctx)
        replay, out_g = lay.capture_decode(xd, kc, vc, length - 1, ctx)
        for _ in range(5):
            replay()
        barrier()
        e0.record(stream)
        for _ in range(steps):
            replay()
        e1.record(stream)
        barrier()
        ms_peer = max_over_ranks(e0.elapsed_time(e1)) / steps
        outs["fused_attention_peer_all_reduce"] = out_g[:n_check].clone()
        devapis.graphDestroy(replay.graph)
        lay.fused_decode = True
        for _ in range(3):
            lay.decode(xd, kc, vc, length - 1, ctx)
        replay, out_g = lay.capture_decode(xd, kc, vc, length - 1, ctx)
        for _ in range(5):
            replay()
        barrier()
        e0.record(stream)
        for _ in range(steps):
            replay()
        e1.record(stream)
        barrier()
        ms_step_peer = max_over_ranks(e0.elapsed_time(e1)) / steps
        outs["fused_step_peer_all_reduce"] = out_g[:n_check].clone()
        devapis.graphDestroy(replay.graph)
        lay.fused_decode = False
        assert lay.tp_group.peer.status() == 0, "a peer all-reduce wait timed out"
        lay.tp_group.peer.close()
        lay.tp_group.peer = None
    lay.fused_attention = False
    parity = None
    if check:
        # four of the 64 sequences against the CPU oracle: op-by-op variants within 5e-3 of the op-by-op bf16 CPU path, the
        # fused-attention variants within 5e-3 of the oracle's fused form, everything within 1e-2 of fp32
        torch.cuda.synchronize()
        refs = decode_oracle_refs(cfg, host_w, xd[:n_check], kc[:n_check], vc[:n_check], length - 1, world, rank, dist)
        parity = {}
        for name, got in outs.items():
            form = "bf16_stepwise_fused_step" if name.startswith("fused_step") else ("bf16_stepwise_fused" if name.startswith("fused") else "bf16_stepwise")
            sw = bench_checks.REL_STEPWISE if world == 1 else bench_checks.REL_LOOSE  # TP: partial sums travel rounded to bf16
            entry = bench_checks.parity_entry(got, {form: (refs[form], sw), "fp32": (refs["fp32"], bench_checks.fp32_bound(refs[form], refs["fp32"]))})
            entry["all_ranks_ok"] = all_ranks(entry["ok"], dist)
            parity[name] = entry
        parity["ok"] = all(v["ok"] for v in parity.values())
        parity["all_ranks_ok"] = all(v["all_ranks_ok"] for k, v in parity.items() if isinstance(v, dict))
        parity["rows_checked"] = "%d of the %d sequences" % (n_check, b)
    d = cfg.head_dim
    weight_bytes = 2 * (cfg.hidden * lay.heads * d * 2 + cfg.hidden * lay.kv_heads * d * 2 + 3 * cfg.hidden * lay.ffn)
    kv_bytes = 2 * 2 * b * lay.kv_heads * length * d
    gbs = (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9
    return {"parity": parity,
            "workload": "decode, batch 64, KV length 4096, tp%d, step replayed from a CUDA graph" % world, "tokens_per_s": b / (ms * 1e-3),
            "ms_per_step": ms, "eager_tokens_per_s": b / (ms_eager * 1e-3), "eager_ms_per_step": ms_eager,
            "algorithmic_bytes_per_step_per_gpu": weight_bytes + kv_bytes, "achieved_gbs": round(gbs, 1),
            "hbm_frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": peaks["source"],
            "fused_attention": {"tokens_per_s": b / (ms_fused * 1e-3), "ms_per_step": ms_fused,
                                "hbm_frac": round((weight_bytes + kv_bytes) / (ms_fused * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                                "note": "diopiMultiHeadAttention on views of the cache replaces diopiBmm, diopiDivInpScalar, diopiSoftmax, diopiBmm"},
            "fused_step": {"tokens_per_s": b / (ms_step * 1e-3), "ms_per_step": ms_step,
                           "hbm_frac": round((weight_bytes + kv_bytes) / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                           "note": "as fused_attention, with one q/k/v projection, diopiB200RopeAppendKV, diopiB200AddRMSNorm and "
                                   "diopiB200MmSwiGLU (include/diopi/functions_b200.h), diopiAddmm for down projection + residual: eight launches per step"},
            "fused_step_peer_all_reduce": None if ms_step_peer is None else {
                "tokens_per_s": b / (ms_step_peer * 1e-3), "ms_per_step": ms_step_peer,
                "note": "as fused_step, with both all-reduces done by one kernel each over peer memory"},
            "fused_attention_peer_all_reduce": None if ms_peer is None else {
                "tokens_per_s": b / (ms_peer * 1e-3), "ms_per_step": ms_peer,
                "note": "as fused_attention, with both all-reduces done by one kernel each over peer memory (NVLink loads, bounded flag waits)"}}


if __name__ == "__main__":
    main()
