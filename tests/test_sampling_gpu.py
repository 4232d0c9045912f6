"""Operators of a sampling loop on the GPU against torch CPU (shapes follow the reference's unit tests
dipu/tests/python/unittests/test_topk.py, test_sort.py, test_argmax.py, test_cumsum.py, test_gather.py, test_multinomial.py,
test_index.py, test_index_put.py): bit-exact values and indices where the order is determined, distribution checks for
the random draws."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(shape, dtype=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(dtype)


@pytest.mark.parametrize("shape,dim", [((7, 1000), -1), ((4, 33, 5), 1), ((3, 32000), 1), ((65,), 0), ((2, 3, 40000), 2)])
@pytest.mark.parametrize("descending", [False, True])
def test_sort(diopi, ctx, shape, dim, descending):
    x = _rand(shape, seed=sum(shape))
    xd = x.to(DEV)
    vals = torch.empty(shape, device=DEV)
    idx = torch.empty(shape, dtype=torch.int64, device=DEV)
    diopi.diopiSort(ctx, vals, idx, xd, dim, descending, True)
    rv, ri = torch.sort(x, dim=dim, descending=descending, stable=True)
    assert torch.equal(vals.cpu(), rv) and torch.equal(idx.cpu(), ri)
    ctx.release_workspace()


def test_sort_ties_nan_and_other_dtypes(diopi, ctx):
    # equal keys keep their order (stable), NaN sorts above every number, bf16 / int32 / uint8 keys
    x = torch.tensor([[3.0, 1.0, float("nan"), 1.0, -0.0, 0.0, float("inf"), -float("inf"), 1.0]])
    for desc in (False, True):
        vals = torch.empty_like(x, device=DEV)
        idx = torch.empty(x.shape, dtype=torch.int64, device=DEV)
        diopi.diopiSort(ctx, vals, idx, x.to(DEV), 1, desc, None)
        rv, ri = torch.sort(x, dim=1, descending=desc, stable=True)
        assert torch.equal(idx.cpu(), ri), (desc, idx.cpu(), ri)
        assert torch.equal(vals.cpu().isnan(), rv.isnan()) and torch.equal(vals.cpu().nan_to_num(7.0), rv.nan_to_num(7.0))
    for dtype in (torch.bfloat16, torch.float16, torch.int32, torch.uint8):
        y = (torch.randint(0, 50, (5, 300), generator=torch.Generator().manual_seed(3)) - (0 if dtype == torch.uint8 else 25)).to(dtype)
        vals = torch.empty(y.shape, dtype=dtype, device=DEV)
        idx = torch.empty(y.shape, dtype=torch.int64, device=DEV)
        diopi.diopiSort(ctx, vals, idx, y.to(DEV), -1, False, True)
        rv, ri = torch.sort(y, dim=-1, stable=True)
        assert torch.equal(vals.cpu(), rv) and torch.equal(idx.cpu(), ri), dtype


@pytest.mark.parametrize("shape,k,dim,largest", [((64, 32000), 50, -1, True), ((3, 100), 100, 1, False), ((5, 9, 11), 4, 1, True), ((1, 50000), 1, 1, True)])
def test_topk(diopi, ctx, shape, k, dim, largest):
    x = _rand(shape, seed=k)
    out_shape = list(shape)
    out_shape[dim] = k
    vals = torch.empty(out_shape, device=DEV)
    idx = torch.empty(out_shape, dtype=torch.int64, device=DEV)
    diopi.diopiTopk(ctx, vals, idx, x.to(DEV), k, dim, largest, True)
    rv, ri = torch.topk(x, k, dim=dim, largest=largest, sorted=True)
    assert torch.equal(vals.cpu(), rv) and torch.equal(idx.cpu(), ri)   # random floats: no ties, the order is determined
    ctx.release_workspace()


@pytest.mark.parametrize("largest", [True, False])
@pytest.mark.parametrize("dtype,k", [(torch.float32, 2048), (torch.bfloat16, 37), (torch.int32, 500)])
def test_topk_by_selection_with_heavy_ties(diopi, ctx, dtype, k, largest):
    """Long rows with few distinct values: the threshold key has many equals, of which the lowest positions must be taken -
    the result equals the first k entries of a stable sort."""
    g = torch.Generator().manual_seed(k)
    x = torch.randint(-10, 10, (5, 20000), generator=g).to(dtype)
    vals = torch.empty((5, k), dtype=dtype, device=DEV)
    idx = torch.empty((5, k), dtype=torch.int64, device=DEV)
    diopi.diopiTopk(ctx, vals, idx, x.to(DEV), k, 1, largest, True)
    rv, ri = torch.sort(x.float(), dim=1, descending=largest, stable=True)
    assert torch.equal(vals.cpu().float(), rv[:, :k]) and torch.equal(idx.cpu(), ri[:, :k])
    # a middle dimension
    y = torch.randn(3, 9000, 4, generator=g)
    v2 = torch.empty((3, 5, 4), device=DEV)
    i2 = torch.empty((3, 5, 4), dtype=torch.int64, device=DEV)
    diopi.diopiTopk(ctx, v2, i2, y.to(DEV), 5, 1, largest, True)
    tv, ti = torch.topk(y, 5, dim=1, largest=largest)
    assert torch.equal(v2.cpu(), tv) and torch.equal(i2.cpu(), ti)


@pytest.mark.parametrize("shape,dim,keepdim", [((16, 32000), 1, False), ((4, 5, 6), 0, True), ((4, 5, 6), -1, False), ((1000,), None, False),
                                               ((3, 7), None, False)])
def test_argmax(diopi, ctx, shape, dim, keepdim):
    x = _rand(shape, seed=len(shape))
    x.view(-1)[3] = x.max() + 1 if dim is None else x.view(-1)[3]
    ref = torch.argmax(x, dim=dim, keepdim=keepdim)
    out = torch.empty(ref.shape, dtype=torch.int64, device=DEV)
    diopi.diopiArgmax(ctx, out, x.to(DEV), dim, keepdim)
    assert torch.equal(out.cpu(), ref)
    # ties resolve to the lowest index, in bf16 too
    t = torch.tensor([[1.0, 5.0, 5.0, 2.0], [7.0, 7.0, 7.0, 7.0]], dtype=torch.bfloat16)
    o2 = torch.empty(2, dtype=torch.int64, device=DEV)
    diopi.diopiArgmax(ctx, o2, t.to(DEV), 1, False)
    assert o2.cpu().tolist() == [1, 0]


@pytest.mark.parametrize("shape,dim", [((8, 32000), 1), ((5, 300, 7), 1), ((4097,), 0), ((3, 4), 0)])
def test_cumsum(diopi, ctx, shape, dim):
    x = torch.rand(shape, generator=torch.Generator().manual_seed(5))
    out = torch.empty(shape, device=DEV)
    diopi.diopiCumsum(ctx, out, x.to(DEV), dim)
    torch.testing.assert_close(out.cpu(), torch.cumsum(x, dim), rtol=2e-5, atol=2e-4)
    xi = torch.randint(-5, 6, shape, generator=torch.Generator().manual_seed(6))
    oi = torch.empty(shape, dtype=torch.int64, device=DEV)
    diopi.diopiCumsum(ctx, oi, xi.to(DEV), dim)
    assert torch.equal(oi.cpu(), torch.cumsum(xi, dim))   # integers: exact


def test_gather(diopi, ctx):
    x = _rand((6, 50, 9), seed=2)
    g = torch.Generator().manual_seed(8)
    for dim, ishape in ((1, (6, 20, 9)), (0, (3, 50, 4)), (2, (6, 50, 1))):
        index = torch.randint(0, x.shape[dim], ishape, generator=g)
        out = torch.empty(ishape, device=DEV)
        diopi.diopiGather(ctx, out, x.to(DEV), dim, index.to(DEV))
        assert torch.equal(out.cpu(), torch.gather(x, dim, index))
    # the sampling loop's use: token ids back from sorted positions, bf16 payload, strided input
    probs = _rand((4, 1000), torch.bfloat16, seed=9)
    pos = torch.randint(0, 1000, (4, 1), generator=g)
    out = torch.empty((4, 1), dtype=torch.bfloat16, device=DEV)
    diopi.diopiGather(ctx, out, probs.to(DEV), 1, pos.to(DEV))
    assert torch.equal(out.cpu(), torch.gather(probs, 1, pos))


def test_multinomial_with_replacement_matches_distribution(pkg, diopi, ctx):
    w = torch.tensor([[0.0, 1.0, 3.0, 0.0, 4.0, 2.0], [5.0, 0.0, 0.0, 0.0, 0.0, 5.0]])
    n = 200000
    gen = diopi.Generator(seed=1234)
    out = torch.empty((2, n), dtype=torch.int64, device=DEV)
    diopi.diopiMultinomial(ctx, out, w.to(DEV), n, True, gen)
    seed, off = gen.state()
    assert seed == 1234 and off == 2 * n and off % 4 == 0      # the generator advanced by the draws it served
    o = out.cpu()
    for r in range(2):
        freq = torch.bincount(o[r], minlength=6).double() / n
        want = (w[r] / w[r].sum()).double()
        assert (freq[w[r] == 0] == 0).all()                      # zero-weight categories are never drawn
        assert (freq - want).abs().max().item() < 5e-3           # ~5 sigma at n = 200000
    # the same seed and offset reproduce the draw; another offset does not
    gen.set_state(1234, 0)
    again = torch.empty_like(out)
    diopi.diopiMultinomial(ctx, again, w.to(DEV), n, True, gen)
    assert torch.equal(again.cpu(), o)
    other = torch.empty_like(out)
    diopi.diopiMultinomial(ctx, other, w.to(DEV), n, True, gen)
    assert not torch.equal(other.cpu(), o)
    # one sample per row from a vocabulary-sized bf16 distribution: always a category with non-zero weight
    p = torch.softmax(_rand((64, 32000), seed=4) * 4, dim=-1)
    p[:, ::2] = 0
    pick = torch.empty((64, 1), dtype=torch.int64, device=DEV)
    diopi.diopiMultinomial(ctx, pick, p.to(torch.bfloat16).to(DEV), 1, False, None)
    picked = pick.cpu().view(-1)
    assert ((picked % 2) == 1).all() and (picked >= 0).all() and (picked < 32000).all()


def test_multinomial_never_draws_a_masked_token(diopi, ctx):
    """Rows as they look after top-k / top-p masking: a few positive weights spread over a vocabulary of zeros, of very
    different magnitude (so that running sums round), many draws per row: an index of weight zero must never come back."""
    rows, vocab, n = 32, 32000, 50000
    rng = np.random.default_rng(21)
    w = torch.zeros((rows, vocab))
    for r in range(rows):
        keep = torch.from_numpy(rng.choice(vocab, size=5 + r, replace=False))
        w[r, keep] = torch.from_numpy(rng.random(keep.numel()).astype(np.float32) ** 6 + 1e-7)
    out = torch.empty((rows, n), dtype=torch.int64, device=DEV)
    diopi.diopiMultinomial(ctx, out, w.to(DEV), n, True, diopi.Generator(seed=99))
    o = out.cpu()
    assert (o >= 0).all() and (o < vocab).all()
    assert (torch.gather(w, 1, o) > 0).all()
    # and the heaviest token of a row is drawn about as often as its weight says
    top = w.argmax(1)
    freq = (o == top.view(-1, 1)).double().mean(1)
    want = (w.max(1).values / w.sum(1)).double()
    assert (freq - want).abs().max().item() < 2e-2


def test_multinomial_without_replacement(diopi, ctx):
    w = torch.tensor([[1.0, 0.0, 2.0, 3.0, 0.0, 4.0, 5.0, 1.0]])
    gen = diopi.Generator(seed=7)
    counts = torch.zeros(8)
    trials = 4000
    for _ in range(trials // 100):
        out = torch.empty((100, 3), dtype=torch.int64, device=DEV)
        diopi.diopiMultinomial(ctx, out, w.expand(100, 8).contiguous().to(DEV), 3, False, gen)
        o = out.cpu()
        assert all(len(set(row.tolist())) == 3 for row in o)          # no duplicates within a draw
        assert not torch.isin(o, torch.tensor([1, 4])).any()           # zero-weight categories never appear
        counts += torch.bincount(o[:, 0], minlength=8).float()
        ctx.release_workspace()
    first = counts / trials                                             # the first draw follows the weights
    assert (first - w[0] / w.sum()).abs().max().item() < 0.03


def test_index_masks_skipped_dimensions_and_empty_cases(diopi, ctx):
    """The cases of dipu/tests/python/unittests/test_index.py:8-63: index tensors on several leading dimensions, on inner
    dimensions (`x[..., i, ...]`), boolean masks (alone, mixed with index tensors, of several dimensions), non-adjacent
    indexed dimensions (S goes first), empty index tensors and an empty input - each against torch's own indexing."""
    def idx(x, *entries):
        got = diopi.diopiIndex(ctx, x.to(DEV), [None if e is None else e.to(DEV) for e in entries])
        torch.cuda.synchronize()
        ctx.release_workspace()
        return got.cpu()

    x = _rand((3, 4, 5, 6), seed=21)
    i = torch.arange(0, 3)
    assert torch.equal(idx(x, i), x[i])
    assert torch.equal(idx(x, i, i), x[i, i])
    assert torch.equal(idx(x, i, i, i), x[i, i, i])
    assert torch.equal(idx(x, i, i, i, i), x[i, i, i, i])
    assert torch.equal(idx(x, None, i), x[:, i])                       # an inner dimension
    assert torch.equal(idx(x, None, None, torch.tensor([4, 0, 0])), x[:, :, torch.tensor([4, 0, 0])])
    assert torch.equal(idx(x, i, None, i), x[i, :, i])                  # not adjacent: S first
    assert torch.equal(idx(x, torch.tensor([[0], [2]]), None, None, torch.tensor([1, 5, 5])), x[torch.tensor([[0], [2]]), :, :, torch.tensor([1, 5, 5])])
    # test_index_bool
    inp = torch.arange(16).reshape(4, 2, 2)
    i1, i2, m3 = torch.tensor([2]), torch.tensor([1]), torch.tensor([False, True])
    assert torch.equal(idx(inp, i1), inp[i1])
    assert torch.equal(idx(inp, i1, i2), inp[i1, i2])
    assert torch.equal(idx(inp, None, i2), inp[..., i2, :])
    assert torch.equal(idx(inp, i1, i2, m3), inp[i1, i2, m3])
    assert torch.equal(idx(inp, i1, None, m3), inp[i1, ..., m3])
    m = _rand((4, 2, 2), seed=5) > 0
    assert torch.equal(idx(inp, m), inp[m])                             # a mask over all dimensions
    assert torch.equal(idx(inp, m[:, :, 0]), inp[m[:, :, 0]])           # over the two leading ones (a strided mask)
    assert torch.equal(idx(inp, None, m[0]), inp[:, m[0]])              # over the two trailing ones
    assert torch.equal(idx(inp, torch.zeros(4, dtype=torch.bool)), inp[torch.zeros(4, dtype=torch.bool)])   # nothing selected
    big = _rand((3000, 7), seed=6)
    bm = big[:, 0] > 0.3
    assert torch.equal(idx(big, bm), big[bm])                           # several chunks of the compaction
    # test_index_empty_index / test_index_empty_input
    e3, e1 = torch.empty((0, 3), dtype=torch.long), torch.empty((0, 1), dtype=torch.long)
    assert idx(inp, e3).shape == inp[e3].shape == (0, 3, 2, 2)
    assert idx(inp, e3, e1).shape == inp[e3, e1].shape
    empty = torch.tensor([])
    assert idx(empty, torch.tensor([], dtype=torch.bool)).shape == (0,)
    # index_put_ through a mask and through an inner dimension
    y = _rand((5, 6), seed=8)
    mk = y > 0
    yd = y.to(DEV)
    diopi.diopiIndexPutInp(ctx, yd, torch.tensor(0.0).to(DEV), [mk.to(DEV)], False)
    torch.cuda.synchronize()
    want = y.clone()
    want[mk] = 0.0
    assert torch.equal(yd.cpu(), want)
    vals = _rand((5, 2), seed=9)
    diopi.diopiIndexPutInp(ctx, yd, vals.to(DEV), [None, torch.tensor([5, 1]).to(DEV)], False)
    torch.cuda.synchronize()
    want[:, torch.tensor([5, 1])] = vals
    assert torch.equal(yd.cpu(), want)
    with pytest.raises(diopi.DiopiError):
        diopi.diopiIndex(ctx, inp.to(DEV), [torch.ones(3, dtype=torch.bool).to(DEV)])   # mask of the wrong length


def test_index_and_index_put(diopi, ctx):
    x = _rand((10, 6, 4), seed=11)
    i0 = torch.tensor([0, 9, -1, 3, 3])
    got = diopi.diopiIndex(ctx, x.to(DEV), [i0.to(DEV)])
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), x[i0])
    i1 = torch.tensor([[1], [5]])
    got = diopi.diopiIndex(ctx, x.to(DEV), [i0.to(DEV), i1.to(DEV)])     # index tensors broadcast to [2, 5]
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), x[i0, i1])
    ctx.release_workspace()
    # index_put_: overwrite and accumulate (duplicates add up), values broadcast
    y = x.clone()
    yd = x.to(DEV).clone()
    vals = _rand((5, 6, 4), seed=12)
    ii = torch.tensor([0, 2, 4, 6, 8])
    diopi.diopiIndexPutInp(ctx, yd, vals.to(DEV), [ii.to(DEV)], False)
    y[ii] = vals
    assert torch.equal(yd.cpu(), y)
    dup = torch.tensor([1, 1, 1, 7])
    diopi.diopiIndexPutInp(ctx, yd, torch.ones(4, device=DEV), [dup.to(DEV), torch.tensor([2, 2, 2, 0]).to(DEV)], True)
    y.index_put_((dup, torch.tensor([2, 2, 2, 0])), torch.ones(4), accumulate=True)
    torch.testing.assert_close(yd.cpu(), y)
    # the sampling loop's use: logits[row, token] = -inf for a list of (row, token) pairs, bf16
    logits = _rand((4, 100), torch.bfloat16, seed=13)
    ld = logits.to(DEV).clone()
    rows, toks = torch.tensor([0, 0, 3]), torch.tensor([5, 99, 0])
    diopi.diopiIndexPutInp(ctx, ld, torch.tensor(float("-inf"), dtype=torch.bfloat16, device=DEV), [rows.to(DEV), toks.to(DEV)], False)
    logits[rows, toks] = float("-inf")
    assert torch.equal(ld.cpu(), logits)
    with pytest.raises(diopi.DiopiError, match="mask's shape"):
        diopi.diopiIndex(ctx, x.to(DEV), [(i0 > 0).to(DEV)])     # a mask of 5 elements over a dimension of 10
    with pytest.raises(diopi.DiopiError, match="int64 tensors or boolean masks"):
        diopi.diopiIndex(ctx, x.to(DEV), [i0.to(torch.int32).to(DEV)])
    ctx.release_workspace()


def test_top_p_sampling_step(diopi, ctx):
    """The ops together: softmax -> sort -> cumsum -> mask -> multinomial -> gather, against the same steps in torch CPU."""
    logits = _rand((8, 32000), seed=21) * 3
    ld = logits.to(DEV)
    probs = torch.empty_like(ld)
    diopi.diopiSoftmax(ctx, probs, ld, -1)
    sp, si = torch.empty_like(ld), torch.empty(ld.shape, dtype=torch.int64, device=DEV)
    diopi.diopiSort(ctx, sp, si, probs, -1, True, True)
    cum = torch.empty_like(ld)
    diopi.diopiCumsum(ctx, cum, sp, -1)
    rp = torch.softmax(logits, -1)
    rsp, rsi = torch.sort(rp, dim=-1, descending=True, stable=True)
    torch.testing.assert_close(sp.cpu(), rsp, rtol=1e-5, atol=1e-8)
    torch.testing.assert_close(cum.cpu(), torch.cumsum(rsp, -1), rtol=1e-4, atol=1e-5)
    # keep the smallest prefix whose mass exceeds 0.9, draw one position from it, map it back to a token id
    keep = (cum.cpu() - sp.cpu()) < 0.9
    filtered = (sp.cpu() * keep).to(DEV)
    pos = torch.empty((8, 1), dtype=torch.int64, device=DEV)
    diopi.diopiMultinomial(ctx, pos, filtered, 1, True, diopi.Generator(seed=3))
    tok = torch.empty((8, 1), dtype=torch.int64, device=DEV)
    diopi.diopiGather(ctx, tok, si, 1, pos)
    p, t = pos.cpu(), tok.cpu()
    assert keep.gather(1, p).all()                                   # every drawn position lies inside the nucleus
    assert torch.equal(t, si.cpu().gather(1, p))
    ctx.release_workspace()
