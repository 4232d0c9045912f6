"""One rank of the DICL communicator test (run as a child process by test_dicl_gpu.py):
    python tests/dicl_worker.py <rank> <world> <rendezvous dir>
Expected values are closed-form, as in the reference's dipu/tests/python/individual_scripts/test_rt_ddp.py:103-476."""
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, rdv = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    import __graft_entry__ as entry
    pkg = entry.load_package()
    dv, DT = pkg.devapis, pkg.diopi.DTYPE
    torch.cuda.set_device(rank)
    dev = "cuda:%d" % rank
    # rank 0 creates the unique id; it travels as plain bytes (here through a file, in DIPU through the c10d store)
    path = os.path.join(rdv, "uid")
    if rank == 0:
        uid = dv.diclGetUniqueId()
        with open(path + ".tmp", "wb") as f:
            f.write(uid)
        os.rename(path + ".tmp", path)
    else:
        t0 = time.time()
        while not os.path.exists(path):
            if time.time() - t0 > 60:
                raise SystemExit("rank %d: no unique id after 60 s" % rank)
            time.sleep(0.05)
        uid = open(path, "rb").read()
    assert len(uid) == dv.DICL_UNIQUE_ID_BYTES_SIZE
    comm = dv.diclCommInitRank(world, uid, rank, rank)
    stream = dv.getStreamFromPool(rank)
    assert dv.diclGetCommAsyncError(comm) == dv.diclResult_t.DICL_SUCCESS
    assert dv.diclGetCommName(comm).startswith("dicl_b200_")

    def sync():
        dv.syncStream(stream)

    # every collective of the interface against closed-form values (the cases bench.py also runs at its world size)
    import bench_checks
    counter = [0]

    def exchange(obj, src):
        """A small object from rank `src` to everybody, through files in the rendezvous directory."""
        counter[0] += 1
        box = os.path.join(rdv, "x%d" % counter[0])
        if rank == src:
            with open(box + ".tmp", "wb") as f:
                f.write(obj)
            os.rename(box + ".tmp", box)
            return obj
        t0 = time.time()
        while not os.path.exists(box):
            if time.time() - t0 > 60:
                raise SystemExit("rank %d: nothing from rank %d after 60 s" % (rank, src))
            time.sleep(0.02)
        return open(box, "rb").read()

    res = bench_checks.collective_checks(dv, DT, comm, stream, rank, world, dev, exchange)
    bad = [k for k, v in res.items() if v is False] + [("%s: %s" % (k, v)) for k, v in res.items() if k.endswith("_error")]
    assert not bad, bad
    expected = {"all_reduce_sum", "all_reduce_max_min_avg", "all_reduce_bool_uint8", "broadcast", "all_gather", "reduce", "reduce_scatter",
                "send_recv_ring", "gather_scatter_by_send_recv", "all_to_all_equal", "all_to_all_unequal", "comm_name_and_error_state"}
    if world >= 4:
        expected.add("sub_group")
    assert expected <= set(res), sorted(expected - set(res))

    # all-reduce in one kernel over peer memory: closed-form sums, bit-identical on every rank, in place and out of place,
    # sizes from one vector to the handle's limit, back-to-back calls (the call counter lives on the device)
    assert dv.diclCommRank(comm) == (rank, world)
    res = bench_checks.peer_all_reduce_checks(dv, DT, comm, stream, rank, world, dev)
    assert res.get("peer_all_reduce") and res.get("peer_all_reduce_back_to_back") and res.get("peer_all_reduce_refuses_oversize"), res

    # tensor-parallel layer: every rank's output equals the unsharded CPU oracle
    from oracle import llama_cpu
    from dipu_b200 import layer as L
    cfg = llama_cpu.LayerConfig(hidden=512, heads=8, kv_heads=8, head_dim=64, ffn=1376, eps=1e-6)
    w = llama_cpu.make_weights(cfg, seed=77)
    emb = llama_cpu.make_embedding(32000, 512, seed=77)
    ids = llama_cpu.make_token_ids(2, 64, seed=77)
    ref = llama_cpu.decoder_layer_prefill(cfg, w, emb, ids)

    class Group:
        def __init__(self):
            self.rank, self.size, self.device, self.comm, self.stream, self.peer, self.space = rank, world, rank, comm, stream, None, None
    grp = L.TpGroup.__new__(L.TpGroup)
    grp.__dict__.update(Group().__dict__)
    lay = L.DecoderLayer(cfg, w, dtype=torch.float32, device=dev, tp_rank=rank, tp_size=world, tp_group=grp)
    for overlap in (True, False):  # all-reduces overlapped with the other half-batch's compute, and the plain order
        lay.overlap_comm = overlap
        y = lay.prefill(L.embed(emb.to(dev), ids.to(dev)), 2, 64)
        torch.cuda.synchronize()
        err = (y.cpu() - ref).abs().max().item()
        assert err <= 2e-4, (overlap, err)

    # the same layer with its partial sums (256 KiB each) reduced by the peer-memory kernel on the compute stream
    grp.enable_peer_reduce(1 << 20)
    lay.overlap_comm = False
    for _ in range(3):
        y = lay.prefill(L.embed(emb.to(dev), ids.to(dev)), 2, 64)
    torch.cuda.synchronize()
    assert grp.peer.status() == 0
    err = (y.cpu() - ref).abs().max().item()
    assert err <= 2e-4, ("peer reduce", err)
    grp.peer.close()   # collective: the ranks meet inside before anything is unmapped
    grp.peer = None

    # row-parallel linears with the all-reduce and the residual add fused into the kernels: tiles pushed to the owners of
    # their rows, one reduce-gather kernel per linear; against the op-by-op bf16 CPU oracle and against the NCCL path
    seq = 128 * world
    # an FFN width whose shard stays a multiple of 8 elements at every world size up to 8 (the tensor-core kernels' pitch rule)
    cfg = llama_cpu.LayerConfig(hidden=512, heads=8, kv_heads=8, head_dim=64, ffn=1408, eps=1e-6)
    w = llama_cpu.make_weights(cfg, seed=79)
    idsb = llama_cpu.make_token_ids(2, seq, seed=78)
    # the op-by-op bf16 oracle with its row-parallel linears evaluated as `world` ranks evaluate them (partials rounded, then summed)
    refb = llama_cpu.decoder_layer_prefill_from_hidden(cfg, llama_cpu.round_weights(w, torch.bfloat16),
                                                       llama_cpu.round_tensor(emb, torch.bfloat16)[idsb.reshape(-1)], 2, seq,
                                                       llama_cpu.stepwise(torch.bfloat16), tp=world)
    ref32 = llama_cpu.decoder_layer_prefill(cfg, w, emb, idsb)
    layb = L.DecoderLayer(cfg, w, dtype=torch.bfloat16, device=dev, tp_rank=rank, tp_size=world, tp_group=grp)
    xb = L.embed(emb.to(torch.bfloat16).to(dev), idsb.to(dev))
    y_nccl = layb.prefill(xb, 2, seq).float().cpu()
    for parts, on_comm in ((2, True), (1, False), (2, False)):
        grp.enable_fused_linear(2 * seq // parts, cfg.hidden, parts, on_comm_stream=on_comm)
        layb.fused_collective = True
        for _ in range(3):
            y = layb.prefill(xb, 2, seq)
        torch.cuda.synchronize()
        assert grp.space.status() == 0 and pkg.diopi.gemm_status() == 0
        got = y.float().cpu()
        # The sum of the partial products and the residual add happen in fp32 with ONE rounding, where the op-by-op path
        # rounds the all-reduced sum and then the add: closer to the fp32 layer, but no longer step-for-step the bf16 oracle.
        # Whole-layer bounds as for the other fused paths: max-abs 2e-2, relative L2 1e-2 against either oracle.
        for name, want in (("bf16 op-by-op oracle", refb), ("fp32 oracle", ref32), ("library all-reduce path", y_nccl)):
            max_abs = (got - want).abs().max().item()
            rel = ((got - want).norm() / want.norm()).item()
            print("rank %d fused collective parts=%d comm_stream=%s vs %s: max_abs %.3e rel %.3e" % (rank, parts, on_comm, name, max_abs, rel), flush=True)
            assert max_abs <= 2e-2 and rel <= 1e-2, ("fused collective", parts, on_comm, name, max_abs, rel)
        layb.fused_collective = False
        grp.disable_fused_linear()

    dv.diclCommDestroy(comm)
    print("rank %d ok" % rank, flush=True)


if __name__ == "__main__":
    main()
