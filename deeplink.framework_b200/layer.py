"""A Llama decoder layer expressed as the stream of DIOPI calls DIPU dispatches for it.

This is harness code, not a model library: it stands where the Python op stream of an eager torch module stands in a
DIPU process (reference call stack: torch dispatcher -> generated wrapper -> ::diopiXxx, see
dipu/scripts/autogen_diopi_wrapper/diopi_wrapper_template.py:100-142). Every arithmetic step is one DIOPI call through
the C-ABI; reshapes / transposes are metadata-only views, which DIPU also serves without calling DIOPI
(dipu/torch_dipu/csrc_dipu/aten/RegisterDIPU.cpp:382-406). The op order follows the reference's own Llama block
(dicp/test/model/llama/model.py:104-201).

Tensor parallelism (Megatron style): wq / wk / wv / w1 / w3 are split by output features (heads, FFN columns), wo / w2 by
input features; the partial sums after wo and w2 are all-reduced through devapis.diclAllReduce on a pool stream,
bracketed by events the way ProcessGroupDICL::doComm does it
(dipu/torch_dipu/csrc_dipu/runtime/distributed/ProcessGroupDICL.cpp:438-485).
"""
import math

import torch

from . import devapis, diopi


def _cfg_get(cfg, name, default=None):
    return getattr(cfg, name, default)


def rope_tables(head_dim, positions, base, device):
    """cos / sin [len(positions), head_dim/2] in float32, built on the host (a one-off table, as in the reference model)."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    ang = torch.outer(positions.float(), inv).float()
    return torch.cos(ang).to(device), torch.sin(ang).to(device)


def embed(table, ids, ctx=None):
    """Embedding lookup the way DIPU runs it: aten::embedding lowers to index_select(weight, 0, ids.reshape(-1))."""
    ctx = ctx or diopi.Context()
    flat = ids.reshape(-1)
    out = torch.empty((flat.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    diopi.diopiIndexSelect(ctx, out, table, 0, flat)
    return out


class TpGroup:
    """The communicator side of a tensor-parallel group: one DICL communicator and one pool stream per rank."""

    def __init__(self, rank, size, unique_id, device):
        self.rank, self.size, self.device = rank, size, device
        self.comm = devapis.diclCommInitRank(size, unique_id, rank, device)
        self.stream = devapis.getStreamFromPool(device)
        self.peer = None  # one-kernel all-reduce over peer memory for small messages (enable_peer_reduce)
        self.space = None  # staging / result slots for row-parallel linears with the all-reduce fused in (enable_fused_linear)

    def enable_peer_reduce(self, max_bytes=1 << 20):
        """Collective: from now on dense bf16 / fp16 / fp32 messages of up to max_bytes are summed by one kernel over peer
        memory on the compute stream itself (no stream hop, no library call); larger ones keep going through diclAllReduce."""
        self.peer = devapis.PeerAllReduce(self.comm, max_bytes, self.stream)
        devapis.syncStream(self.stream)

    def enable_fused_linear(self, part_rows, cols, parts, on_comm_stream=True, space=None):
        """Collective: allocates the peer space for row-parallel linears of [part_rows, K] x [K, cols] whose all-reduce and
        residual add are fused into the kernels (fused_row_linear). A layer call handles `parts` row blocks (1, or 2 when
        two half-batches are interleaved), each with an attention and an FFN linear: 2 * parts slots, the slots of one
        linear adjacent so that the parts' results form one [parts * part_rows, cols] tensor."""
        self.space_parts, self.space_rows, self.space_cols = parts, part_rows, cols
        self.fused_on_comm_stream = on_comm_stream
        self.space = space or devapis.PeerSpace(self.comm, part_rows * cols * 2, 2 * parts, self.stream)
        if self.stream is not None:
            devapis.syncStream(self.stream)

    def _torch_device(self):
        return torch.device("cuda", self.device) if isinstance(self.device, int) else torch.device(self.device)

    def disable_fused_linear(self):
        """Collective: frees the peer space. A rank's last kernel writes flags into the peers' memory, so every rank first
        drains its device and then meets the others in a small all-reduce before anything is unmapped."""
        if self.space is None:
            return
        devapis.syncDevice()
        token = torch.zeros(1, dtype=torch.float32, device=self._torch_device())
        devapis.diclAllReduce(token.data_ptr(), token.data_ptr(), 1, diopi.DTYPE[token.dtype], devapis.ReduceOp.SUM, self.comm, self.stream)
        devapis.syncStream(self.stream)
        self.space.close()
        self.space = None

    def fused_result(self, which, dtype):
        """The [parts * part_rows, cols] tensor the `which`-th linear (0: attention output, 1: FFN down) of a layer call fills."""
        ptr = self.space.result_ptr(which * self.space_parts)
        return devapis.tensorFromDevicePtr(ptr, (self.space_parts * self.space_rows, self.space_cols), dtype, self._torch_device())

    def fused_row_linear(self, ctx, x, w_t, residual, which, part):
        """residual + sum over ranks of x @ w_t, for row block `part` of the layer call's `which`-th row-parallel linear:
        the product pushes its tiles to the owners of their rows while it runs (diopiB200MmPush), then one kernel sums the
        pieces this rank owns, adds the residual rows and writes the finished rows into every rank's result slot. Returns
        an event to wait for before reading the result (None when the reduction runs on the compute stream itself)."""
        sp = self.space
        slot = which * self.space_parts + part
        epoch, prev = sp.begin(slot)
        diopi.diopiB200MmPush(ctx, x, w_t, sp, slot, epoch, prev)
        rows, cols = x.shape[0], w_t.shape[1]
        dt = diopi.DTYPE[x.dtype]
        if not self.fused_on_comm_stream:
            sp.reduce_gather(slot, epoch, residual.data_ptr() if residual is not None else None, rows, cols, dt, ctx.stream)
            return None
        pre = devapis.getEventFromPool()
        devapis.recordEvent(pre, ctx.stream)
        devapis.streamWaitEvent(self.stream, pre)
        devapis.restoreEventToPool(pre)
        sp.reduce_gather(slot, epoch, residual.data_ptr() if residual is not None else None, rows, cols, dt, self.stream)
        post = devapis.getEventFromPool()
        devapis.recordEvent(post, self.stream)
        return post

    def all_reduce_(self, tensor, compute_stream):
        """In-place SUM all-reduce of a dense tensor; the compute stream waits for the result without a host block."""
        nbytes = tensor.numel() * tensor.element_size()
        if (self.peer is not None and nbytes <= self.peer.max_bytes and nbytes % 16 == 0 and tensor.data_ptr() % 16 == 0
                and tensor.dtype in (torch.bfloat16, torch.float16, torch.float32)):
            self.peer.all_reduce(tensor.data_ptr(), tensor.data_ptr(), tensor.numel(), diopi.DTYPE[tensor.dtype], compute_stream)
            return
        self.wait(self.all_reduce_async_(tensor, compute_stream), compute_stream)

    def all_reduce_async_(self, tensor, compute_stream):
        """Starts an in-place SUM all-reduce on the communication stream once the compute stream has produced `tensor`;
        returns the event that marks its completion. The compute stream keeps running until wait() is called."""
        pre = devapis.getEventFromPool()
        devapis.recordEvent(pre, compute_stream)
        devapis.streamWaitEvent(self.stream, pre)
        devapis.restoreEventToPool(pre)  # the wait was enqueued against this record; the event may be re-used
        devapis.diclAllReduce(tensor.data_ptr(), tensor.data_ptr(), tensor.numel(), diopi.DTYPE[tensor.dtype], devapis.ReduceOp.SUM, self.comm,
                              self.stream)
        post = devapis.getEventFromPool()
        devapis.recordEvent(post, self.stream)
        return post

    def wait(self, event, compute_stream):
        devapis.streamWaitEvent(compute_stream, event)
        devapis.restoreEventToPool(event)

    def close(self):
        devapis.syncStream(self.stream)
        if self.peer is not None:
            self.peer.close()
            self.peer = None
        self.disable_fused_linear()
        devapis.diclCommDestroy(self.comm)
        self.comm = None


class DecoderLayer:
    def __init__(self, cfg, weights, dtype=torch.bfloat16, device="cuda:0", tp_rank=0, tp_size=1, tp_group=None):
        self.hidden = cfg.hidden
        self.head_dim = cfg.head_dim
        self.heads_total = cfg.heads
        self.kv_heads_total = _cfg_get(cfg, "kv_heads", cfg.heads)
        assert self.heads_total % tp_size == 0 and self.kv_heads_total % tp_size == 0 and cfg.ffn % tp_size == 0
        self.heads = self.heads_total // tp_size
        self.kv_heads = self.kv_heads_total // tp_size
        self.ffn = cfg.ffn // tp_size
        self.eps = cfg.eps
        self.rope_base = _cfg_get(cfg, "rope_base", 10000.0)
        self.interleaved = _cfg_get(cfg, "rope_layout", "half") == "interleaved"
        self.dtype, self.device = dtype, torch.device(device)
        self.tp_rank, self.tp_size, self.tp_group = tp_rank, tp_size, tp_group
        self.overlap_comm = True  # prefill: interleave two half-batches so the all-reduces overlap compute
        self.scores_by_baddbmm = False  # prefill attention scores through one baddbmm instead of bmm, div, add
        self.fused_attention = False  # prefill attention through the fused operator (no score tensor, no transposes)
        self.fused_collective = False  # prefill: row-parallel linears push their tiles to the peers (TpGroup.enable_fused_linear)
        self.fused_decode = False  # decode: merged q/k/v projection, rotary + cache append, add + RMSNorm and SwiGLU-in-the-GEMM kernels
        self._wqkv = None  # [(hq + 2 hk) d, hidden]: wq, wk, wv stacked (built on first use of the fused decode path)
        self._w13 = None   # [2 f, hidden]: rows 2j / 2j+1 are the gate / up weights of feature j
        d, r = self.head_dim, tp_rank
        hq, hk, f = self.heads, self.kv_heads, self.ffn

        def put(t):
            return t.to(dtype).contiguous().to(self.device)

        self.wq = put(weights["wq"][r * hq * d:(r + 1) * hq * d])
        self.wk = put(weights["wk"][r * hk * d:(r + 1) * hk * d])
        self.wv = put(weights["wv"][r * hk * d:(r + 1) * hk * d])
        self.wo = put(weights["wo"][:, r * hq * d:(r + 1) * hq * d])
        self.w1 = put(weights["w1"][r * f:(r + 1) * f])
        self.w3 = put(weights["w3"][r * f:(r + 1) * f])
        self.w2 = put(weights["w2"][:, r * f:(r + 1) * f])
        self.attention_norm = put(weights["attention_norm"])
        self.ffn_norm = put(weights["ffn_norm"])
        self._tables = {}
        self._masks = {}
        self._keep = None  # while capturing a graph: every temporary, so that its memory stays reserved for replays
        self.launches = 0  # DIOPI calls issued (each is at least one kernel launch or device copy)

    # ---- helpers ------------------------------------------------------------------------------------------
    def _empty(self, *shape, dtype=None):
        t = torch.empty(shape, dtype=dtype or self.dtype, device=self.device)
        if self._keep is not None:
            self._keep.append(t)
        return t

    def _like(self, x):
        return self._empty(*x.shape, dtype=x.dtype)

    def _call(self, fn, ctx, *args):
        self.launches += 1
        return fn(ctx, *args)

    def _linear(self, ctx, x, w):
        """F.linear on the CUDA vendor reaches DIOPI as mm(x, W.t()) with a transposed view of the weight."""
        out = self._empty(x.shape[0], w.shape[0])
        self._call(diopi.diopiMm, ctx, out, x, w.t())
        return out

    def _tables_for(self, positions_key, positions):
        if positions_key not in self._tables:
            self._tables[positions_key] = rope_tables(self.head_dim, positions, self.rope_base, self.device)
        return self._tables[positions_key]

    def _mask_for(self, ctx, seq):
        """Additive causal mask [seq, seq]: -inf above the diagonal, built once with fill + triu."""
        if seq not in self._masks:
            m = self._empty(seq, seq)
            self._call(diopi.diopiFill, ctx, m, float("-inf"))
            self._call(diopi.diopiTriuInp, ctx, m, 1)
            self._masks[seq] = m
        return self._masks[seq]

    def _rope(self, ctx, x, cos, sin):
        out = self._like(x)
        self._call(diopi.diopiRotaryEmbedding, ctx, out, x, cos, sin, False, self.interleaved)
        return out

    def _expand_kv(self, ctx, t):
        """[B, kv_heads, S, D] -> [B, heads, S, D] for grouped-query attention: an expand view materialised by copy_."""
        g = self.heads // self.kv_heads
        if g == 1:
            return t
        b, hk, s, d = t.shape
        out = self._empty(b, hk, g, s, d)
        self._call(diopi.diopiCopyInp, ctx, t.unsqueeze(2).expand(b, hk, g, s, d), out)
        return out.view(b, hk * g, s, d)

    def _all_reduce(self, ctx, t):
        if self.tp_size > 1:
            self.tp_group.all_reduce_(t, ctx.stream)

    def _ffn_core(self, ctx, h):
        """RMSNorm -> gate / up -> SiLU * up: the input of the (row-parallel) down projection."""
        hn = self._like(h)
        self._call(diopi.diopiRMSNorm, ctx, hn, None, h, [self.hidden], self.ffn_norm, None, self.eps)
        g = self._linear(ctx, hn, self.w1)
        u = self._linear(ctx, hn, self.w3)
        self._call(diopi.diopiSiluInp, ctx, g)
        self._call(diopi.diopiMulInp, ctx, g, u)
        return g

    def _ffn_partial(self, ctx, h):
        """RMSNorm -> gate / up -> SiLU * up -> down projection: this rank's partial sum (before the all-reduce)."""
        return self._linear(ctx, self._ffn_core(ctx, h), self.w2)

    def _ffn(self, ctx, h, out=None):
        dn = self._ffn_partial(ctx, h)
        self._all_reduce(ctx, dn)
        out = self._like(h) if out is None else out
        self._call(diopi.diopiAdd, ctx, out, h, dn, 1)
        return out

    # ---- prefill ---------------------------------------------------------------------------------------------------
    def _attention_partial(self, ctx, x, batch, seq):
        """RMSNorm -> q/k/v -> rotary -> causal attention through bmm + softmax -> o_proj: this rank's partial sum."""
        return self._linear(ctx, self._attention_core(ctx, x, batch, seq), self.wo)

    def _attention_core(self, ctx, x, batch, seq):
        """Everything of the attention block before the (row-parallel) output projection: [batch*seq, local heads * D]."""
        t, d, hq, hk = batch * seq, self.head_dim, self.heads, self.kv_heads
        hn = self._like(x)
        self._call(diopi.diopiRMSNorm, ctx, hn, None, x, [self.hidden], self.attention_norm, None, self.eps)
        q = self._linear(ctx, hn, self.wq).view(t, hq, d)
        k = self._linear(ctx, hn, self.wk).view(t, hk, d)
        v = self._linear(ctx, hn, self.wv).view(batch, seq, hk, d)
        cos, sin = self._tables_for(("prefill", seq), torch.arange(seq))
        q = self._rope(ctx, q, cos, sin).view(batch, seq, hq, d)
        k = self._rope(ctx, k, cos, sin).view(batch, seq, hk, d)
        if self.fused_attention and d == 128 and self.dtype in (torch.bfloat16, torch.float16):
            # one call on the [B, S, h, D] views: grouped heads share K / V inside the kernel, output lands merged
            merged = self._empty(batch, seq, hq, d)
            self._call(diopi.diopiMultiHeadAttention, ctx, q, k, v, 0.0, True, False, 1.0 / math.sqrt(d), merged, None, None, None)
            return merged.view(t, hq * d)
        # [B, S, h, D] -> [B, h, S, D]: .transpose(1, 2).contiguous() is a copy_ from a strided view
        qt, kt, vt = self._empty(batch, hq, seq, d), self._empty(batch, hk, seq, d), self._empty(batch, hk, seq, d)
        self._call(diopi.diopiCopyInp, ctx, q.transpose(1, 2), qt)
        self._call(diopi.diopiCopyInp, ctx, k.transpose(1, 2), kt)
        self._call(diopi.diopiCopyInp, ctx, v.transpose(1, 2), vt)
        kt, vt = self._expand_kv(ctx, kt), self._expand_kv(ctx, vt)
        scores = self._empty(batch * hq, seq, seq)
        if self.scores_by_baddbmm:
            # torch.baddbmm(mask, q, k^T, beta=1, alpha=1/sqrt(d)): scale and mask-add ride in the GEMM epilogue
            self._call(diopi.diopiBaddbmm, ctx, scores, self._mask_for(ctx, seq), qt.view(batch * hq, seq, d),
                       kt.view(batch * hq, seq, d).transpose(1, 2), 1.0, 1.0 / math.sqrt(d))
        else:
            # the reference block's order: matmul, / sqrt(d), + mask (dicp/test/model/llama/model.py:146-149)
            self._call(diopi.diopiBmm, ctx, scores, qt.view(batch * hq, seq, d), kt.view(batch * hq, seq, d).transpose(1, 2))
            self._call(diopi.diopiDivInpScalar, ctx, scores, math.sqrt(d), diopi.RoundModeNone)
            self._call(diopi.diopiAddInp, ctx, scores, self._mask_for(ctx, seq), 1)
        self._call(diopi.diopiSoftmax, ctx, scores, scores, -1)
        av = self._empty(batch * hq, seq, d)
        self._call(diopi.diopiBmm, ctx, av, scores, vt.view(batch * hq, seq, d))
        merged = self._empty(batch, seq, hq, d)
        self._call(diopi.diopiCopyInp, ctx, av.view(batch, hq, seq, d).transpose(1, 2), merged)
        return merged.view(t, hq * d)

    def prefill(self, x, batch, seq, ctx=None):
        """x [batch*seq, hidden] -> [batch*seq, hidden]; causal attention through bmm + softmax."""
        ctx = ctx or diopi.Context()
        if self.fused_collective and self.tp_group is not None and self.tp_group.space is not None:
            return self._prefill_fused_collective(x, batch, seq, ctx)
        if self.tp_size > 1 and self.overlap_comm and batch % 2 == 0:
            return self._prefill_overlapped(x, batch, seq, ctx)
        attn = self._attention_partial(ctx, x, batch, seq)
        self._all_reduce(ctx, attn)
        h = self._like(x)
        self._call(diopi.diopiAdd, ctx, h, x, attn, 1)
        out = self._ffn(ctx, h)
        ctx.release_workspace()
        return out

    def _prefill_overlapped(self, x, batch, seq, ctx):
        """Tensor-parallel prefill with the four all-reduces hidden behind compute: the batch is cut into two halves
        whose blocks are interleaved, so that while one half's partial sums travel over NVLink on the communication
        stream the other half's attention / FFN runs on the compute stream. Same DIOPI calls, on half the rows each."""
        grp, cs = self.tp_group, ctx.stream
        half = batch // 2
        rows = half * seq
        xs = (x[:rows], x[rows:])
        out = self._like(x)
        outs = (out[:rows], out[rows:])
        attn, ev_attn, h, dn, ev_dn = [None, None], [None, None], [None, None], [None, None], [None, None]
        for i in range(2):
            attn[i] = self._attention_partial(ctx, xs[i], half, seq)
            ev_attn[i] = grp.all_reduce_async_(attn[i], cs)
        for i in range(2):
            grp.wait(ev_attn[i], cs)
            h[i] = self._like(xs[i])
            self._call(diopi.diopiAdd, ctx, h[i], xs[i], attn[i], 1)
            dn[i] = self._ffn_partial(ctx, h[i])
            ev_dn[i] = grp.all_reduce_async_(dn[i], cs)
        for i in range(2):
            grp.wait(ev_dn[i], cs)
            self._call(diopi.diopiAdd, ctx, outs[i], h[i], dn[i], 1)
        ctx.release_workspace()
        return out

    def _prefill_fused_collective(self, x, batch, seq, ctx):
        """Tensor-parallel prefill without library collectives and without separate residual adds: each row-parallel linear
        pushes its output tiles to the ranks that own the rows while it is still multiplying, and one kernel per linear
        sums the arrived pieces, adds the residual and hands the finished rows to every rank (TpGroup.fused_row_linear).
        With two parts the reductions run on the communication stream while the other half-batch computes. The returned
        tensor lives in the group's peer space: it keeps its content until the next call's FFN linear."""
        grp, cs = self.tp_group, ctx.stream
        parts = grp.space_parts
        assert batch % parts == 0 and (batch // parts) * seq == grp.space_rows and self.hidden == grp.space_cols, \
            "the peer space was sized for %d parts of %d rows" % (parts, grp.space_rows)
        pb, rows = batch // parts, grp.space_rows
        xs = [x[i * rows:(i + 1) * rows] for i in range(parts)]
        h_all, out_all = grp.fused_result(0, self.dtype), grp.fused_result(1, self.dtype)
        hs = [h_all[i * rows:(i + 1) * rows] for i in range(parts)]
        ev = [None] * parts
        for i in range(parts):
            merged = self._attention_core(ctx, xs[i], pb, seq)
            self.launches += 2
            ev[i] = grp.fused_row_linear(ctx, merged, self.wo.t(), xs[i], 0, i)
        for i in range(parts):
            if ev[i] is not None:
                grp.wait(ev[i], cs)
            g = self._ffn_core(ctx, hs[i])
            self.launches += 2
            ev[i] = grp.fused_row_linear(ctx, g, self.w2.t(), hs[i], 1, i)
        for i in range(parts):
            if ev[i] is not None:
                grp.wait(ev[i], cs)
        ctx.release_workspace()
        return out_all

    def capture_decode(self, x, k_cache, v_cache, position, ctx):
        """Captures one decode step (every DIOPI call, the KV append and, under tensor parallelism, the all-reduces on the
        communication stream) into a CUDA graph. Returns (replay, out): replay() enqueues the whole step with one launch;
        it reads x / the caches in place and writes `out`. The step must have run at least once before (warm-up: the first
        call of a kernel may set attributes or allocate its status word, which is not allowed while capturing)."""
        self._keep = []
        devapis.graphBeginCapture(ctx.stream)
        try:
            out = self.decode(x, k_cache, v_cache, position, ctx)
        finally:
            graph = devapis.graphEndCapture(ctx.stream)
        keep = self._keep  # the graph holds raw addresses: the temporaries live as long as the replay closure
        self._keep = None

        def replay(_keep=keep):
            devapis.graphLaunch(graph, ctx.stream)
        replay.graph = graph
        return replay, out

    # ---- decode ------------------------------------------------------------------------------------------------------
    def _merged_weights(self):
        """One-time re-layout for the fused decode path, as a loader would do it: q / k / v weights stacked into one matrix,
        gate / up weights interleaved row by row so that a feature's two products are neighbouring output columns."""
        if self._wqkv is None:
            self._wqkv = torch.cat([self.wq, self.wk, self.wv], dim=0).contiguous()
            self._w13 = torch.stack([self.w1, self.w3], dim=1).reshape(2 * self.ffn, self.hidden).contiguous()
        return self._wqkv, self._w13

    def _decode_fused(self, x, k_cache, v_cache, position, ctx):
        """The decode step with the library's fused entry points (include/diopi/functions_b200.h): eight launches (nine when the
        attention splits the keys over CTAs) instead of nineteen. Same arithmetic as the op-by-op step except that SiLU * up is formed in fp32 from the unrounded products."""
        b, d, hq, hk = x.shape[0], self.head_dim, self.heads, self.kv_heads
        length = position + 1
        wqkv, w13 = self._merged_weights()
        hn = self._like(x)
        self._call(diopi.diopiRMSNorm, ctx, hn, None, x, [self.hidden], self.attention_norm, None, self.eps)
        qkv = self._linear(ctx, hn, wqkv)
        cos, sin = self._tables_for(("decode", position), torch.tensor([position]))
        q = self._empty(b, hq, d)
        self._call(diopi.diopiB200RopeAppendKV, ctx, q, qkv, cos, sin, k_cache, v_cache, position)
        keys, vals = k_cache[:, :, :length, :], v_cache[:, :, :length, :]
        av = self._empty(b, 1, hq, d)
        self._call(diopi.diopiMultiHeadAttention, ctx, q.view(b, 1, hq, d), keys.transpose(1, 2), vals.transpose(1, 2), 0.0, False, False,
                   1.0 / math.sqrt(d), av, None, None, None)
        attn = self._linear(ctx, av.view(b, hq * d), self.wo)
        self._all_reduce(ctx, attn)
        h, hn2 = self._like(x), self._like(x)
        self._call(diopi.diopiB200AddRMSNorm, ctx, h, hn2, x, attn, self.ffn_norm, self.eps)
        g = self._empty(b, self.ffn)
        self._call(diopi.diopiB200MmSwiGLU, ctx, g, hn2, w13.t())
        # the block's residual rides in the down projection (diopiAddmm: the sum is formed in fp32 and rounded once); under tensor
        # parallelism rank 0 alone adds it, so that the all-reduce of the partial sums delivers the block's output
        out = self._like(x)
        if self.tp_rank == 0:
            self._call(diopi.diopiAddmm, ctx, out, h, g, self.w2.t(), 1.0, 1.0)
        else:
            self._call(diopi.diopiMm, ctx, out, g, self.w2.t())
        self._all_reduce(ctx, out)
        ctx.release_workspace()
        return out

    def decode(self, x, k_cache, v_cache, position, ctx=None):
        """x [batch, hidden]; caches [batch, local kv heads, L, D], slot `position` receives the new key / value and
        attention covers slots 0..position. Returns [batch, hidden]."""
        ctx = ctx or diopi.Context()
        b, d, hq, hk = x.shape[0], self.head_dim, self.heads, self.kv_heads
        length = position + 1
        if (self.fused_decode and d == 128 and self.dtype in (torch.bfloat16, torch.float16) and not self.interleaved and b <= 128):
            return self._decode_fused(x, k_cache, v_cache, position, ctx)
        hn = self._like(x)
        self._call(diopi.diopiRMSNorm, ctx, hn, None, x, [self.hidden], self.attention_norm, None, self.eps)
        q = self._linear(ctx, hn, self.wq).view(b, hq, d)
        k = self._linear(ctx, hn, self.wk).view(b, hk, d)
        v = self._linear(ctx, hn, self.wv).view(b, hk, d)
        cos, sin = self._tables_for(("decode", position), torch.tensor([position]))
        q = self._rope(ctx, q, cos, sin)
        k = self._rope(ctx, k, cos, sin)
        # KV append: copy_ into a strided slice of the cache
        self._call(diopi.diopiCopyInp, ctx, k, k_cache[:, :, position, :])
        self._call(diopi.diopiCopyInp, ctx, v, v_cache[:, :, position, :])
        keys, vals = k_cache[:, :, :length, :], v_cache[:, :, :length, :]
        if self.fused_attention and d == 128 and self.dtype in (torch.bfloat16, torch.float16):
            # one call on views of the cache ([B, L, kv heads, D] by pitches): K and V are read once, grouped heads share them
            av = self._empty(b, 1, hq, d)
            self._call(diopi.diopiMultiHeadAttention, ctx, q.view(b, 1, hq, d), keys.transpose(1, 2), vals.transpose(1, 2), 0.0, False, False,
                       1.0 / math.sqrt(d), av, None, None, None)
            attn = self._linear(ctx, av.view(b, hq * d), self.wo)
            self._all_reduce(ctx, attn)
            h = self._like(x)
            self._call(diopi.diopiAdd, ctx, h, x, attn, 1)
            out = self._ffn(ctx, h)
            ctx.release_workspace()
            return out
        if hq != hk:
            keys, vals = self._expand_kv(ctx, keys), self._expand_kv(ctx, vals)
        cap = keys.shape[2] if hq != hk else k_cache.shape[2]
        # [B, h, L, D] -> [B*h, L, D] is a free view as long as heads are dense in the cache
        kview = torch.as_strided(keys, (b * hq, length, d), (cap * d, d, 1), keys.storage_offset())
        vview = torch.as_strided(vals, (b * hq, length, d), (cap * d, d, 1), vals.storage_offset())
        scores = self._empty(b * hq, 1, length)
        self._call(diopi.diopiBmm, ctx, scores, q.reshape(b * hq, 1, d), kview.transpose(1, 2))
        self._call(diopi.diopiDivInpScalar, ctx, scores, math.sqrt(d), diopi.RoundModeNone)
        self._call(diopi.diopiSoftmax, ctx, scores, scores, -1)
        av = self._empty(b * hq, 1, d)
        self._call(diopi.diopiBmm, ctx, av, scores, vview)
        attn = self._linear(ctx, av.view(b, hq * d), self.wo)
        self._all_reduce(ctx, attn)
        h = self._like(x)
        self._call(diopi.diopiAdd, ctx, h, x, attn, 1)
        out = self._ffn(ctx, h)
        ctx.release_workspace()
        return out
