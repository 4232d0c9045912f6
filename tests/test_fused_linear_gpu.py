"""Row-parallel linear with the all-reduce fused in (diopiB200MmPush + b200_dicl_peer_reduce_gather), on ONE device: the
ranks of a group are emulated inside this process (all blocks in this GPU's memory), their products are enqueued first and
their reductions afterwards, so that no kernel waits for one that has not run. The result must equal
residual + sum over ranks of x_r @ w_r^T on every rank, bit-identical between the ranks."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _operands(n, rows, k, cols, seed, dtype):
    rng = np.random.default_rng(seed)
    xs = [torch.from_numpy(rng.standard_normal((rows, k), dtype=np.float32)).to(dtype) for _ in range(n)]
    ws = [torch.from_numpy(rng.standard_normal((cols, k), dtype=np.float32) / np.sqrt(k * n)).to(dtype) for _ in range(n)]
    res = torch.from_numpy(rng.standard_normal((rows, cols), dtype=np.float32)).to(dtype)
    return xs, ws, res


def _reference(xs, ws, res):
    """fp32 CPU: every rank's partial product rounded to the operand type (as it travels), summed in fp32 with the residual.
    Also the elementwise error bound: a partial whose fp32 accumulation order differs may round to the neighbouring value
    (one ulp of the partial: 2^-7 of it for bf16, 2^-10 for fp16), and so may the final sum."""
    ulp = 2.0 ** -7 if xs[0].dtype == torch.bfloat16 else 2.0 ** -10
    acc = res.float() if res is not None else torch.zeros(xs[0].shape[0], ws[0].shape[0])
    bound = torch.full_like(acc, 1e-3)
    for x, w in zip(xs, ws):
        part = (x.float() @ w.float().t()).to(x.dtype).float()
        acc = acc + part
        bound = bound + ulp * part.abs()
    return acc, bound + ulp * acc.abs()


def _run(pkg, ctx, spaces, slot, xs, ws, res, dtype):
    n = len(spaces)
    rows, cols = xs[0].shape[0], ws[0].shape[0]
    xd = [x.to(DEV) for x in xs]
    wd = [w.to(DEV) for w in ws]
    rd = res.to(DEV) if res is not None else None
    numbers = [sp.begin(slot) for sp in spaces]
    assert len(set(numbers)) == 1
    epoch, prev = numbers[0]
    for r in range(n):
        pkg.diopi.diopiB200MmPush(ctx, xd[r], wd[r].t(), spaces[r], slot, epoch, prev)
    for r in range(n):
        spaces[r].reduce_gather(slot, epoch, rd.data_ptr() if rd is not None else None, rows, cols, pkg.diopi.DTYPE[dtype], ctx.stream)
    torch.cuda.synchronize()
    assert pkg.diopi.gemm_status() == 0
    outs = []
    for r in range(n):
        assert spaces[r].status() == 0
        outs.append(pkg.devapis.tensorFromDevicePtr(spaces[r].result_ptr(slot), (rows, cols), dtype, DEV).cpu())
    return outs


def _check(outs, ref_and_bound):
    ref, bound = ref_and_bound
    for o in outs[1:]:
        assert torch.equal(o, outs[0]), "ranks hold different results"
    got = outs[0].float()
    assert torch.isfinite(got).all()
    excess = ((got - ref).abs() - bound).max().item()
    rel = ((got - ref).norm() / ref.norm()).item()
    assert excess <= 0 and rel <= 3e-3, (excess, rel)


@pytest.mark.parametrize("n", [1, 2, 4, 8])
def test_fused_row_linear_emulated_ranks(pkg, ctx, n):
    rows, k, cols = 2048, 320, 512
    spaces = pkg.devapis.PeerSpace.emulated(n, rows * cols * 2, 2)
    try:
        xs, ws, res = _operands(n, rows, k, cols, seed=100 + n, dtype=torch.bfloat16)
        _check(_run(pkg, ctx, spaces, 0, xs, ws, res, torch.bfloat16), _reference(xs, ws, res))
        # the same slot again with other data (staging and flags are re-used), then the other slot without a residual
        xs, ws, res = _operands(n, rows, k, cols, seed=200 + n, dtype=torch.bfloat16)
        _check(_run(pkg, ctx, spaces, 0, xs, ws, res, torch.bfloat16), _reference(xs, ws, res))
        _check(_run(pkg, ctx, spaces, 1, xs, ws, None, torch.bfloat16), _reference(xs, ws, None))
    finally:
        for sp in spaces:
            sp.close()


def test_fused_row_linear_fp16_smaller_than_slot(pkg, ctx):
    """A result that fills only part of a slot, float16, K with a ragged last block."""
    n, rows, k, cols = 2, 512, 200, 768
    spaces = pkg.devapis.PeerSpace.emulated(n, 2048 * 1024 * 2, 1)
    try:
        xs, ws, res = _operands(n, rows, k, cols, seed=7, dtype=torch.float16)
        _check(_run(pkg, ctx, spaces, 0, xs, ws, res, torch.float16), _reference(xs, ws, res))
    finally:
        for sp in spaces:
            sp.close()


def test_fused_row_linear_rejects_bad_shapes(pkg, ctx):
    spaces = pkg.devapis.PeerSpace.emulated(2, 512 * 512 * 2, 1)
    try:
        sp = spaces[0]
        x = torch.zeros(384, 256, dtype=torch.bfloat16, device=DEV)   # rows not a multiple of 256
        w = torch.zeros(512, 256, dtype=torch.bfloat16, device=DEV)
        with pytest.raises(pkg.diopi.DiopiError):
            pkg.diopi.diopiB200MmPush(ctx, x, w.t(), sp, 0, 1, 0)
        x = torch.zeros(1024, 256, dtype=torch.bfloat16, device=DEV)  # result larger than the slot
        with pytest.raises(pkg.diopi.DiopiError):
            pkg.diopi.diopiB200MmPush(ctx, x, w.t(), sp, 0, 1, 0)
        x = torch.zeros(512, 256, dtype=torch.bfloat16, device=DEV)
        with pytest.raises(pkg.diopi.DiopiError):
            pkg.diopi.diopiB200MmPush(ctx, x, w.t(), sp, 3, 1, 0)       # no such slot
        with pytest.raises(pkg.devapis.VendorError):
            sp.reduce_gather(0, 1, None, 500, 512, 12, ctx.stream)
    finally:
        for sp in spaces:
            sp.close()


def test_reduce_gather_wait_runs_out_and_is_reported(pkg, ctx):
    """A rank whose product is never enqueued: with the wait limit set to a few milliseconds the other ranks' reductions give
    up, return, and report it - status word, DICL_ERR_UNDEF from check(), a message - instead of waiting for ever or handing
    out stale rows; after a status reset the next call on the same slot works. Nothing faults: the kernels only stop waiting."""
    dv = pkg.devapis
    n, rows, k, cols = 2, 1024, 320, 512
    spaces = dv.PeerSpace.emulated(n, rows * cols * 2, 1)
    try:
        xs, ws, res = _operands(n, rows, k, cols, seed=31, dtype=torch.bfloat16)
        _check(_run(pkg, ctx, spaces, 0, xs, ws, res, torch.bfloat16), _reference(xs, ws, res))   # a healthy call first
        dv.setPeerWaitLimitNs(5_000_000)   # 5 ms
        try:
            numbers = [sp.begin(0) for sp in spaces]
            epoch, prev = numbers[0]
            pkg.diopi.diopiB200MmPush(ctx, xs[0].to(DEV), ws[0].to(DEV).t(), spaces[0], 0, epoch, prev)   # rank 1's product is missing
            rd = res.to(DEV)
            for sp in spaces:
                sp.reduce_gather(0, epoch, rd.data_ptr(), rows, cols, pkg.diopi.DTYPE[torch.bfloat16], ctx.stream)
            torch.cuda.synchronize()
        finally:
            dv.setPeerWaitLimitNs(0)
        assert pkg.diopi.gemm_status() == 0   # the product itself had nothing to wait for
        for sp in spaces:
            assert sp.status() == 1
            assert sp.check() == dv.diclResult_t.DICL_ERR_UNDEF
            assert "ran out" in dv.last_error()
            sp.reset_status()
            assert sp.status() == 0 and sp.check() == dv.diclResult_t.DICL_SUCCESS
        # the slot is usable again
        xs, ws, res = _operands(n, rows, k, cols, seed=32, dtype=torch.bfloat16)
        _check(_run(pkg, ctx, spaces, 0, xs, ws, res, torch.bfloat16), _reference(xs, ws, res))
    finally:
        for sp in spaces:
            sp.close()
