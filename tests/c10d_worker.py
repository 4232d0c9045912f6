"""One rank of the c10d-backend test (run as a child process by test_dicl_gpu.py):
    python tests/c10d_worker.py <rank> <world> <port>
torch.distributed with backend "dicl" on tensors of the dipu device: the collectives a tensor-parallel module uses, with
closed-form expectations (values as in the reference's dipu/tests/python/individual_scripts/test_rt_ddp.py:103-476), and a
column- / row-parallel MLP written in plain torch against the unsharded CPU result."""
import importlib
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    import __graft_entry__ as entry
    pkg = entry.load_package()
    adapter = importlib.import_module(pkg.__name__ + ".torch_adapter")
    pkg.devapis.setDevice(rank)
    dev = torch.device("dipu", rank)
    dist.init_process_group("dicl", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    assert dist.get_backend() == "dicl"

    with torch.no_grad():
        x = torch.full((1000,), float(rank + 1), device=dev)
        dist.all_reduce(x)
        assert torch.equal(x.cpu(), torch.full((1000,), float(world * (world + 1) // 2)))
        y = torch.full((257,), float(rank + 1), device=dev, dtype=torch.bfloat16)
        dist.all_reduce(y, op=dist.ReduceOp.MAX)
        assert torch.equal(y.float().cpu(), torch.full((257,), float(world)))
        z = (torch.arange(16) * (rank + 1)).to(dev)
        dist.broadcast(z, src=world - 1)
        assert torch.equal(z.cpu(), torch.arange(16) * world)
        g_in = torch.full((4,), float(rank), device=dev)
        g_out = torch.empty((world * 4,), device=dev)
        dist.all_gather_into_tensor(g_out, g_in)
        assert torch.equal(g_out.cpu(), torch.arange(world).float().repeat_interleave(4))
        parts = [torch.empty((4,), device=dev) for _ in range(world)]
        dist.all_gather(parts, g_in)
        assert all(torch.equal(parts[r].cpu(), torch.full((4,), float(r))) for r in range(world))
        rs_in = torch.arange(world * 4, dtype=torch.float32).to(dev)
        rs_out = torch.empty((4,), device=dev)
        dist.reduce_scatter_tensor(rs_out, rs_in)
        assert torch.equal(rs_out.cpu(), torch.arange(rank * 4, rank * 4 + 4).float() * world)
        a_in = (torch.arange(world * 2, dtype=torch.float32) + 100 * rank).to(dev)
        a_out = torch.empty_like(a_in)
        dist.all_to_all_single(a_out, a_in)
        want = torch.cat([torch.arange(rank * 2, rank * 2 + 2).float() + 100 * r for r in range(world)])
        assert torch.equal(a_out.cpu(), want)
        r_in = torch.full((8,), float(rank + 1), device=dev)
        dist.reduce(r_in, dst=0)
        if rank == 0:
            assert torch.equal(r_in.cpu(), torch.full((8,), float(world * (world + 1) // 2)))
        s_buf, r_buf = torch.full((32,), float(rank), device=dev), torch.empty((32,), device=dev)
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        if rank % 2 == 0:
            dist.send(s_buf, nxt)
            dist.recv(r_buf, prv)
        else:
            dist.recv(r_buf, prv)
            dist.send(s_buf, nxt)
        assert torch.equal(r_buf.cpu(), torch.full((32,), float(prv)))
        # gather to / scatter from the last rank (the reference proxy's construction: point-to-point + one device copy)
        root = world - 1
        mine = torch.full((6,), float(rank) + 0.5, device=dev)
        outs = [torch.empty((6,), device=dev) for _ in range(world)] if rank == root else None
        dist.gather(mine, outs, dst=root)
        if rank == root:
            assert all(torch.equal(outs[r].cpu(), torch.full((6,), r + 0.5)) for r in range(world))
        ins = [torch.arange(r * 6, r * 6 + 6, dtype=torch.float32).to(dev) for r in range(world)] if rank == root else None
        got = torch.empty((6,), device=dev)
        dist.scatter(got, ins, src=root)
        assert torch.equal(got.cpu(), torch.arange(rank * 6, rank * 6 + 6).float())
        # bool tensors stay [True, False, True] under SUM / MAX / MIN (they travel as uint8)
        for op in (dist.ReduceOp.SUM, dist.ReduceOp.MAX, dist.ReduceOp.MIN):
            b = torch.tensor([True, False, True]).to(dev)
            dist.all_reduce(b, op=op)
            assert torch.equal(b.cpu(), torch.tensor([True, False, True])), op
        w = dist.all_reduce(x, async_op=True)     # async form: a Work whose wait() orders the compute stream behind it
        w.wait()
        assert w.is_success()
        dist.barrier()

        # a tensor-parallel MLP in plain torch: column-parallel gate / up, row-parallel down, one all-reduce
        torch.manual_seed(3)
        hidden, ffn, tokens = 256, 512, 40
        w1, w3, w2 = torch.randn(ffn, hidden) * 0.05, torch.randn(ffn, hidden) * 0.05, torch.randn(hidden, ffn) * 0.05
        inp = torch.randn(tokens, hidden)
        ref = F.linear(F.silu(F.linear(inp, w1)) * F.linear(inp, w3), w2)
        f = ffn // world
        sl = slice(rank * f, (rank + 1) * f)
        xd = inp.to(dev)
        part = F.linear(F.silu(F.linear(xd, w1[sl].to(dev))) * F.linear(xd, w3[sl].to(dev)), w2[:, sl].contiguous().to(dev))
        dist.all_reduce(part)
        torch.testing.assert_close(part.cpu(), ref, rtol=1e-4, atol=1e-5)
    assert adapter.stats()["diopi_calls"] > 0
    dist.destroy_process_group()
    print("rank %d ok" % rank, flush=True)


if __name__ == "__main__":
    main()
