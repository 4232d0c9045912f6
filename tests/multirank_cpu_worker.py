"""One gloo rank of the CPU multi-process test (run by test_multirank_cpu.py through torch.distributed.run):
the host-side logic of the tensor-parallel path - sharding, per-rank configuration, the two SUM all-reduces of a layer,
max-over-ranks timing exchange - with the CPU oracle standing in for the kernels."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import llama_cpu  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    cfg = llama_cpu.LayerConfig(hidden=256, heads=8, kv_heads=4, head_dim=32, ffn=512, eps=1e-6)
    w = llama_cpu.make_weights(cfg, seed=5)     # every rank generates the FULL tensors from the base seed and slices its shard
    emb = llama_cpu.make_embedding(1000, cfg.hidden, seed=5)
    ids = llama_cpu.make_token_ids(2, 24, seed=5, vocab=1000)
    full = llama_cpu.decoder_layer_prefill(cfg, w, emb, ids)
    ws, lc = llama_cpu.shard_weights(cfg, w, rank, world), llama_cpu.local_config(cfg, world)
    assert lc.heads == cfg.heads // world and lc.kv_heads == cfg.kv_heads // world and lc.ffn == cfg.ffn // world
    x = emb[ids.reshape(-1)]
    # attention partial sum -> all-reduce -> residual; FFN partial sum -> all-reduce -> residual (two collectives per layer)
    attn = llama_cpu.attention_prefill(lc, ws, llama_cpu.rms_norm(x, w["attention_norm"], cfg.eps), 2, 24)
    dist.all_reduce(attn, op=dist.ReduceOp.SUM)
    h = x + attn
    ffn = llama_cpu.feed_forward(ws, llama_cpu.rms_norm(h, w["ffn_norm"], cfg.eps))
    ffn_partial = ffn.clone()
    dist.all_reduce(ffn, op=dist.ReduceOp.SUM)
    out = h + ffn
    # The fused row-parallel linear's decomposition of that all-reduce + add: rank r owns rows [r * T / n, (r + 1) * T / n);
    # every rank hands each owner its partial sums of the owner's rows (the pushing product), the owner adds them in rank
    # order to its residual rows (the reduce-gather kernel) and every rank receives every owner's finished rows.
    rows = ffn_partial.shape[0] // world
    mine = [torch.empty(rows, cfg.hidden) for _ in range(world)]
    reqs = []
    for peer in range(world):
        if peer == rank:
            mine[rank] = ffn_partial[rank * rows:(rank + 1) * rows]
        else:
            reqs.append(dist.isend(ffn_partial[peer * rows:(peer + 1) * rows].contiguous(), dst=peer))
            reqs.append(dist.irecv(mine[peer], src=peer))
    for q in reqs:
        q.wait()
    owned = h[rank * rows:(rank + 1) * rows].clone()
    for src in range(world):
        owned += mine[src]
    finished = [torch.empty_like(owned) for _ in range(world)]
    dist.all_gather(finished, owned)
    assert (torch.cat(finished) - out).abs().max().item() <= 1e-5
    err = (out - full).abs().max().item()
    assert err <= 1e-4, err
    # every rank holds the same result (replicated after the all-reduce)
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    assert all(torch.allclose(g, gathered[0], atol=1e-6) for g in gathered)
    # the timing exchange of the bench: the reported time is the maximum over ranks
    t = torch.tensor([10.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == 10.0 + world - 1
    # the unique id of a communicator travels as bytes from rank 0
    obj = [bytes(range(128)) if rank == 0 else None]
    dist.broadcast_object_list(obj, src=0)
    assert obj[0] == bytes(range(128))
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok" % rank, flush=True)


if __name__ == "__main__":
    main()
