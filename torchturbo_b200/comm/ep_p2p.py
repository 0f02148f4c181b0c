"""Expert-parallel token dispatch / combine over peer memory (NVLink), without NCCL and without host reads.

Two forms share one workspace.  The FUSED form (`P2PTokenDispatcher.fused_experts`, default) puts the exchange inside
the grouped GEMMs of the expert MLP:
    prepare (one host call)     : counts exchange kernel (tables, send order), destination rows, receive padding cleared
    fc1 GEMM + push prologue    : two extra warps per CTA copy this rank's routed rows (+ routing weight + return tag)
                                  into the owners' expert-major buffers while the tensor cores run; the TMA producer
                                  waits per expert for "rows landed" flags; SwiGLU x weight in the epilogue
    fc2 GEMM + scatter epilogue : every output row is stored straight into the source rank's [T*k, H] return buffer;
                                  the last CTA raises "rows returned" flags
    k-sum kernel                : waits for the owners' flags, sums the k rows of a token (+ residual)
Backward is the same pair around the transposed GEMMs: d(out) rows are pushed inside the d(act) GEMM, d(x) rows (and
the routing-weight gradients) come back from the epilogue of the d(x) GEMM.  No kernel exists only to wait or to signal.
Buffer reuse needs no extra handshake: a rank starts the push of its next exchange only after its k-sum has seen every
owner's "returned" flag, which an owner raises at the end of the GEMM that follows its last read of the receive buffer;
and an owner writes a source's return buffer only in tiles whose rows that source pushed after its previous k-sum.

The UNFUSED form (`dispatch` / `combine`, `TORCHTURBO_EP_FUSED=0`) keeps exchange and GEMMs in separate kernels:

Forward of one MoE layer on every rank (all stream-ordered, nothing waits on the host):
    counts exchange kernel      : my per-expert counts -> every peer; tables for my experts and my send offsets
    rank kernel                 : destination row of each of my (token, slot) entries on its owner
    scatter kernel              : token rows + routing probabilities written into the owners' expert-major buffers,
                                  then "rows landed" flags
    wait kernel                 : all sources have delivered
    grouped GEMMs               : fc1 (SwiGLU x prob epilogue), fc2 -> symmetric output buffer, then "output ready" flags
    wait + gather kernel        : every source pulls its rows from the owners and sums its k expert outputs
Backward mirrors this: d(out) rows are scattered to the owners, d(x) rows and d(prob) scalars are pulled back.

Buffers are shared by all MoE layers of a model.  Reuse is safe because every rank waits on every other rank once
per layer in each direction: a rank that starts writing layer L+1 data has observed the owners' layer-L
"output ready" flags, which they raise after they stopped reading their receive buffers.  The same ordering lets
the expert MLP write its output (forward) and its input gradient (backward) directly into the peer-visible output
buffer, and lets its backward read d(y) in place from the receive buffer: only the forward input rows, which
backward needs again, are copied out of the workspace.

Receive capacity is `capacity_factor` x the balanced share (rows are never dropped silently: an overflow sets the
workspace status, which `check()` turns into an exception).
"""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from .. import kernels as K
from ..ops import MoEPermutation, ops
from .symm import SymmetricBuffer

_WORKSPACES: dict[tuple, "EPWorkspace"] = {}


class EPCapacityExceeded(RuntimeError):
    """Some rank's experts were routed more rows than its receive buffer holds.  No row was sent for that layer and
    the optimizer update of the step is skipped (the status poisons the gradient norm); `grow_workspaces()` followed
    by a repeat of the step makes the exchange dropless again."""


CAPACITY_MARK = "receive capacity exceeded"


class EPWorkspace:
    def __init__(self, group, hidden: int, num_experts: int, tokens: int, topk: int, capacity_factor: float):
        self.tokens, self.topk, self.capacity_factor = tokens, topk, float(capacity_factor)
        self.group = group
        self.W, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.E, self.El, self.H = num_experts, num_experts // self.W, hidden
        rows = int(tokens * topk * capacity_factor)
        self.m_tiles_cap = (rows + K.SEG_ALIGN - 1) // K.SEG_ALIGN + self.El
        self.cap = self.m_tiles_cap * K.SEG_ALIGN
        # rows of the return buffer of the fused form: this rank's own (token, expert) entries, with the same head
        # room as the receive side so that later batches may be somewhat longer than the one that sized the workspace
        self.entries = int(tokens * topk * max(capacity_factor, 1.0))
        out_rows = max(self.cap, self.entries)             # y rows (unfused) and returned rows (fused) share one region
        nbytes = (4 * self.W * self.E + self.cap * hidden * 2 + out_rows * hidden * 2 + 3 * self.cap * 4 + out_rows * 4
                  + 4 * (4 * self.W + self.E) + 24 * 256)
        self.buf = SymmetricBuffer(nbytes, group)
        self.off_counts, self.counts_all = self.buf.carve(4 * self.W * self.E, torch.int32)
        self.off_recv, self.recv_rows = self.buf.carve(self.cap * hidden * 2, torch.bfloat16, (self.cap, hidden))
        self.off_recv_vals, self.recv_vals = self.buf.carve(self.cap * 4, torch.float32)
        self.off_recv_tags, self.recv_tags = self.buf.carve(self.cap * 4, torch.int32)
        self.off_y, out_region = self.buf.carve(out_rows * hidden * 2, torch.bfloat16, (out_rows, hidden))
        self.y_rows, self.ret_rows = out_region[:self.cap], out_region[:self.entries]
        self.off_y_vals, out_vals = self.buf.carve(out_rows * 4, torch.float32)
        self.y_vals, self.ret_vals = out_vals[:self.cap], out_vals[:self.entries]
        self.ch_counts, self.ch_rows, self.ch_ready = self.buf.channel(), self.buf.channel(), self.buf.channel()
        self.ch_push, self.ch_ret = self.buf.channel(self.E), self.buf.channel()
        dev = self.buf.local.device
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        self.sent = torch.zeros(self.E + 1, dtype=torch.int32, device=dev)   # rows sent per expert + chunk counter
        self.budget_ms = int(os.environ.get("TORCHTURBO_P2P_WAIT_MS", "5000"))
        self.ptrs = self.buf.peer_ptrs

    # -- fused form -----------------------------------------------------------------------------------
    def prepare(self, expert, counts=None, tables=None):
        return K.ep_prepare(self.ptrs, off_counts=self.off_counts, off_flags_counts=self.ch_counts.offset, counts=counts,
                            expert=expert, recv_rows=self.recv_rows, recv_vals=self.recv_vals, recv_tags=self.recv_tags,
                            sent=self.sent, status=self.status, rank=self.rank, world=self.W, num_experts=self.E,
                            m_tiles_cap=self.m_tiles_cap, epoch_counts=self.ch_counts.next() if tables is None else 0,
                            budget_ms=self.budget_ms, tables=tables)

    def _fuse(self) -> "K.EpFuseArgs":
        a = K.EpFuseArgs()
        a.peer_ptrs, a.W, a.rank, a.El = C.addressof(self.ptrs), self.W, self.rank, self.El
        a.status, a.budget_ms = self.status.data_ptr(), self.budget_ms
        return a

    def push_args(self, src, order, expert, dest_row, val, counts, k) -> "K.EpFuseArgs":
        """Push prologue: rows of `src` ([T, H]) -> the owners' receive buffers, in `order`."""
        a = self._fuse()
        a.push_on = 1
        a.off_rows, a.off_vals, a.off_tags, a.off_flags = self.off_recv, self.off_recv_vals, self.off_recv_tags, self.ch_push.offset
        a.src, a.lds = src.data_ptr(), src.stride(0)
        a.order, a.expert, a.dest_row = order.data_ptr(), expert.data_ptr(), dest_row.data_ptr()
        a.val = val.data_ptr() if val is not None else None
        a.counts, a.sent = counts.data_ptr(), self.sent.data_ptr()
        a.n_entries, a.k, a.H, a.epoch, a.cap_rows = expert.numel(), k, self.H, self.ch_push.next(), self.cap
        return a

    def scatter_args(self, row_val=None) -> "K.EpFuseArgs":
        """Scatter epilogue: output rows -> the return buffer of the rank named by the row's tag."""
        a = self._fuse()
        a.scat_on = 1
        a.off_ret, a.off_ret_vals, a.off_ret_flags = self.off_y, self.off_y_vals, self.ch_ret.offset
        a.row_tag = self.recv_tags.data_ptr()
        a.row_val = row_val.data_ptr() if row_val is not None else None
        a.ret_epoch, a.done_counter, a.ret_rows = self.ch_ret.next(), self.done.data_ptr(), self.entries
        return a

    def ksum(self, T, k, residual=None):
        return K.ep_ksum(self.ptrs, self.off_y, self.ch_ret.offset, T, k, self.H, self.W, self.rank, self.ch_ret.epoch,
                         self.budget_ms, self.status, residual=residual)

    # -- primitives ---------------------------------------------------------------------------------
    def exchange(self, counts):
        return K.ep_exchange(self.ptrs, self.off_counts, self.ch_counts.offset, counts, self.rank, self.W, self.E,
                             self.ch_counts.next(), self.budget_ms, self.m_tiles_cap, self.status)

    def scatter_rows(self, src, expert, dest_row, vals, k):
        """Rows (and optional scalars) -> owners' receive buffers; returns after every source's rows have landed here."""
        epoch = self.ch_rows.next()
        K.ep_scatter(self.ptrs, self.off_recv, self.off_recv_vals, self.ch_rows.offset, src, expert, dest_row, vals, k,
                     self.El, self.rank, self.W, epoch, self.cap, self.done, self.status)
        K.flag_wait(self.ptrs, self.ch_rows.offset, self.rank, self.W, epoch, self.budget_ms, self.status)

    def publish_and_wait_ready(self):
        epoch = self.ch_ready.next()
        K.flag_signal(self.ptrs, self.ch_ready.offset, self.rank, self.W, epoch)
        K.flag_wait(self.ptrs, self.ch_ready.offset, self.rank, self.W, epoch, self.budget_ms, self.status)

    def gather_rows(self, expert, dest_row, T, k, residual=None):
        return K.ep_gather(self.ptrs, self.off_y, expert, dest_row, T, k, self.H, self.El, self.W, self.cap, self.status,
                           residual=residual)

    def gather_vals(self, expert, dest_row):
        return K.ep_gather_vals(self.ptrs, self.off_y_vals, expert, dest_row, self.El, self.W, self.cap, self.status)

    # -- one host call per direction (same kernels as the primitives above) ----------------------------
    def dispatch_all(self, src, expert, vals, k, counts=None, tables=None):
        """Forward dispatch (`counts` given) or the row scatter of combine's backward (`tables` given)."""
        return K.ep_dispatch_all(
            self.ptrs, off_counts=self.off_counts, off_flags_counts=self.ch_counts.offset, off_rows=self.off_recv,
            off_vals=self.off_recv_vals, off_flags_rows=self.ch_rows.offset, counts=counts, expert=expert, src=src, val=vals,
            recv_rows_local=self.recv_rows, recv_vals_local=self.recv_vals if vals is not None else None, rank=self.rank,
            world=self.W, num_experts=self.E, k=k, m_tiles_cap=self.m_tiles_cap, cap_rows=self.cap,
            epoch_counts=self.ch_counts.next() if tables is None else 0, epoch_rows=self.ch_rows.next(),
            budget_ms=self.budget_ms, done_counter=self.done, status=self.status, tables=tables)

    def combine_all(self, expert, dest_row, T, k, residual=None, want_vals=False):
        return K.ep_combine_all(self.ptrs, off_rows=self.off_y, off_vals=self.off_y_vals, off_flags=self.ch_ready.offset,
                                expert=expert, dest_row=dest_row, T=T, k=k, H=self.H, El=self.El, rank=self.rank, world=self.W,
                                epoch=self.ch_ready.next(), budget_ms=self.budget_ms, cap_rows=self.cap, status=self.status,
                                residual=residual, want_vals=want_vals)

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            if code in (2, 3):
                raise EPCapacityExceeded(
                    f"expert-parallel exchange on rank {self.rank}: {CAPACITY_MARK} (capacity factor "
                    f"{self.capacity_factor:g}: an owner was routed more than {self.cap} rows"
                    + (", seen here as rows addressed beyond that owner's buffer" if code == 3 else "") + ")")
            what = "receive capacity exceeded (raise capacity_factor)" if code == 2 else \
                "a row was addressed beyond its owner's receive buffer and was not sent (receive capacity exceeded on " \
                "the owner, raise capacity_factor)" if code == 3 else f"peer wait timed out (code {code:#x})"
            raise RuntimeError(f"expert-parallel exchange failed on rank {self.rank}: {what}")


def grow_workspaces(factor: float = 2.0) -> list[float]:
    """Replace every workspace by one with `factor` x the receive capacity, up to the worst case (every row of every
    rank routed to one owner).  Collective: all ranks call it at the same point (they all see the overflow status).
    Returns the new capacity factors."""
    out = []
    for key, ws in list(_WORKSPACES.items()):
        cf = min(ws.capacity_factor * factor, float(ws.W))
        if cf <= ws.capacity_factor:
            raise EPCapacityExceeded(f"expert-parallel receive buffer is already sized for the worst case ({cf:g} x the "
                                     "balanced share) and still overflowed: the batch is longer than the one that sized it "
                                     "(set TORCHTURBO_EP_MAX_TOKENS)")
        group, H, E, tokens, topk = ws.group, ws.H, ws.E, ws.tokens, ws.topk
        del _WORKSPACES[key]
        del ws
        _WORKSPACES[key] = EPWorkspace(group, H, E, tokens, topk, cf)
        out.append(cf)
    return out


def get_workspace(group, hidden, num_experts, tokens, topk, capacity_factor=2.0) -> EPWorkspace:
    """One workspace per (group, hidden, experts, top-k), created at first use.  Every rank must carve identical
    offsets, so the token count that sizes it is the maximum over the group (one all-reduce, once); it never grows
    afterwards, because a rank cannot know that a peer wants to: a later batch that does not fit raises the
    capacity status instead.  `TORCHTURBO_EP_MAX_TOKENS` presets the per-rank token count."""
    key = (id(group), hidden, num_experts, topk)
    ws = _WORKSPACES.get(key)
    if ws is None:
        preset = int(os.environ.get("TORCHTURBO_EP_MAX_TOKENS", "0"))
        t = torch.tensor([max(tokens, preset)], dtype=torch.int64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        ws = EPWorkspace(group, hidden, num_experts, int(t.item()), topk, capacity_factor)
        _WORKSPACES[key] = ws
    return ws


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, prob, idx, counts, ws: EPWorkspace):
        T, k = idx.shape
        expert = idx.reshape(-1).contiguous()
        seg_start, recv_counts, tile_group, dest_row = ws.dispatch_all(x, expert, prob.reshape(-1).contiguous(), k, counts=counts)
        xp, rp = ws.recv_rows.clone(), ws.recv_vals.clone()
        ctx.ws, ctx.dims = ws, (T, k)
        ctx.save_for_backward(expert, dest_row)
        for t in (seg_start, recv_counts, tile_group, dest_row, expert):
            ctx.mark_non_differentiable(t)
        return xp, rp, seg_start, recv_counts, tile_group, dest_row, expert

    @staticmethod
    def backward(ctx, dxp, drp, *_):
        ws, (T, k) = ctx.ws, ctx.dims
        expert, dest_row = ctx.saved_tensors
        if dxp.data_ptr() != ws.y_rows.data_ptr():   # the expert MLP normally writes d(x) straight into the buffer
            ws.y_rows.copy_(dxp)
        if drp is not None:
            ws.y_vals.copy_(drp)
        else:
            ws.y_vals.zero_()
        dx, dprob = ws.combine_all(expert, dest_row, T, k, want_vals=True)
        return dx, dprob.view(T, k), None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, expert, dest_row, seg_start, recv_counts, ws: EPWorkspace, T, k, residual):
        if y.data_ptr() != ws.y_rows.data_ptr():     # the expert MLP normally writes y straight into the buffer
            ws.y_rows.copy_(y)
        out, _ = ws.combine_all(expert, dest_row, T, k, residual=residual)
        ctx.ws, ctx.dims = ws, (T, k, residual is not None)
        ctx.save_for_backward(expert, dest_row, seg_start, recv_counts)
        return out

    @staticmethod
    def backward(ctx, dout):
        ws, (T, k, has_res) = ctx.ws, ctx.dims
        expert, dest_row, seg_start, recv_counts = ctx.saved_tensors
        dout = dout.contiguous()
        ws.dispatch_all(dout, expert, None, k, tables=(seg_start, recv_counts, dest_row))
        # no copy: the expert backward that consumes d(y) runs before this rank raises the next "ready" flag, and no
        # peer writes these rows again before it has seen that flag (it first gathers its d(x) of this layer)
        dy = ws.recv_rows.detach()
        return dy, None, None, None, None, None, None, None, (dout if has_res else None)


class _FusedExperts(torch.autograd.Function):
    """Expert MLP of one MoE layer with the token exchange inside its grouped GEMMs (module docstring, fused form)."""

    @staticmethod
    def forward(ctx, x, prob, idx32, counts, w1, w2, ws: EPWorkspace, residual):
        T, k = idx32.shape
        expert = idx32.reshape(-1)
        probf = prob.reshape(-1)
        seg_start, recv_counts, tile_group, dest_row, order = ws.prepare(expert, counts=counts)
        pre = torch.empty(ws.cap, w1.shape[-1], dtype=torch.bfloat16, device=x.device)
        act = K.gemm(ws.recv_rows, w1, b_mn=True, tile_group=tile_group, swiglu=True, row_scale=ws.recv_vals, preact=pre,
                     ep=ws.push_args(x, order, expert, dest_row, probf, counts, k))
        # the receive buffer is refilled by the next exchange: keep what backward needs
        xp, rp = K.ep_save(ws.recv_rows, ws.recv_vals, seg_start, ws.El)
        K.gemm(act, w2, b_mn=True, tile_group=tile_group, out=ws.ret_rows, ep=ws.scatter_args())
        out = ws.ksum(T, k, residual=residual)
        ctx.ws, ctx.dims = ws, (T, k, residual is not None)
        # `act` is kept as well: recomputing it in backward costs a pass over `pre`, keeping it costs cap x F bf16
        ctx.save_for_backward(xp, rp, pre, act, w1, w2, tile_group, seg_start, recv_counts, expert, dest_row, order, counts)
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops.providers.b200 import _weight_grad

        ws, (T, k, has_res) = ctx.ws, ctx.dims
        xp, rp, pre, act, w1, w2, tile_group, seg_start, recv_counts, expert, dest_row, order, counts = ctx.saved_tensors
        dout = dout.contiguous()
        ws.prepare(expert, tables=(seg_start, recv_counts))
        # d(act) = d(y) W2[e]^T with the d(out) rows pushed to the owners from inside the kernel (they land in recv_rows)
        dact = K.gemm(ws.recv_rows, w2, tile_group=tile_group, ep=ws.push_args(dout, order, expert, dest_row, None, counts, k))
        # rows past the last expert segment were never computed: the element-wise pass stops at the device-side count
        dpre, dprob_rows = K.swiglu_bwd(dact, pre, rp, want_dscale=True, nrows=seg_start[ws.El:])
        dw1 = dw2 = None
        if ctx.needs_input_grad[5]:
            dw2 = _weight_grad(w2, act, ws.recv_rows, group_rows=seg_start)
        if ctx.needs_input_grad[4]:
            dw1 = _weight_grad(w1, xp, dpre, group_rows=seg_start)
        # last reader of the received d(y) rows is done: d(x) rows and d(prob) go back to their sources from the epilogue
        K.gemm(dpre, w1, tile_group=tile_group, out=ws.ret_rows, ep=ws.scatter_args(row_val=dprob_rows))
        dx = ws.ksum(T, k)
        dprob = ws.ret_vals[:T * k].clone().view(T, k)
        return dx, dprob, None, None, dw1, dw2, None, (dout if has_res else None)


class P2PTokenDispatcher:
    """Drop-in replacement of the all-to-all dispatcher of `MoELayer` for bf16 CUDA tensors on one NVLink domain."""

    def __init__(self, config, ep_group, num_local_experts: int, capacity_factor: float | None = None):
        self.config, self.ep_group = config, ep_group
        self.ep_size = dist.get_world_size(ep_group)
        self.num_local_experts = num_local_experts
        self.capacity_factor = capacity_factor or float(os.environ.get("TORCHTURBO_EP_CAPACITY_FACTOR", "2.0"))
        self._fallback = None

    @staticmethod
    def usable(ep_group) -> bool:
        return K.available() and SymmetricBuffer.usable(ep_group) and dist.get_world_size(ep_group) > 1

    def _nccl(self):
        if self._fallback is None:
            from ..models.modules.moe.moe import MoEAlltoAllTokenDispatcher

            self._fallback = MoEAlltoAllTokenDispatcher(self.config, self.ep_group, self.num_local_experts)
        return self._fallback

    accepts_counts = True

    def fused_usable(self, x, w1, w2) -> bool:
        """bf16 CUDA rows whose width fits the scatter epilogue (whole 32-column chunks)."""
        return (os.environ.get("TORCHTURBO_EP_FUSED", "1") != "0" and x.is_cuda and x.dtype == torch.bfloat16
                and w1.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16 and x.shape[-1] % 32 == 0
                and w1.shape[-1] % 16 == 0 and not self.config.moe_swiglu_limit)

    def fused_experts(self, x, idx, prob, w1, w2, counts=None, residual=None):
        """Dispatch + expert MLP + combine of one layer: `w1` [El, H, 2F], `w2` [El, F, H]; returns [T, H]."""
        T, k = idx.shape
        E = self.config.num_moe_experts
        ws = get_workspace(self.ep_group, x.shape[-1], E, T, k, self.capacity_factor)
        if T * k > ws.entries:
            raise RuntimeError(f"expert-parallel workspace holds {ws.entries} (token, expert) entries per rank, this batch has "
                               f"{T * k}: set TORCHTURBO_EP_MAX_TOKENS to the largest per-rank token count")
        idx32 = idx if idx.dtype == torch.int32 and idx.is_contiguous() else idx.to(torch.int32).contiguous()
        if counts is None or counts.dtype != torch.int32 or counts.numel() != E:
            counts = torch.zeros(E, dtype=torch.int32, device=x.device)
            counts.scatter_add_(0, idx32.reshape(-1).long(), torch.ones(idx32.numel(), dtype=torch.int32, device=x.device))
        probf = prob if prob.dtype == torch.float32 and prob.is_contiguous() else prob.float().contiguous()
        return _FusedExperts.apply(x.contiguous(), probf, idx32, counts, w1, w2, ws, residual)

    def dispatch(self, x, idx, prob, counts=None):
        """`counts` (int32 [E], the histogram of `idx`) is taken from the routing kernel when the caller has it."""
        if not (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0):
            return self._nccl().dispatch(x, idx, prob)
        T, k = idx.shape
        E = self.config.num_moe_experts
        ws = get_workspace(self.ep_group, x.shape[-1], E, T, k, self.capacity_factor)
        idx32 = idx if idx.dtype == torch.int32 and idx.is_contiguous() else idx.to(torch.int32).contiguous()
        if counts is None or counts.dtype != torch.int32 or counts.numel() != E:
            # histogram without the host sync torch.bincount makes on CUDA (it reads the maximum back)
            counts = torch.zeros(E, dtype=torch.int32, device=x.device)
            counts.scatter_add_(0, idx32.reshape(-1).long(), torch.ones(idx32.numel(), dtype=torch.int32, device=x.device))
        xp, rp, seg_start, recv_counts, tile_group, dest_row, expert = _Dispatch.apply(
            x.contiguous(), prob if prob.dtype == torch.float32 and prob.is_contiguous() else prob.float().contiguous(), idx32,
            counts, ws)
        perm = MoEPermutation(tokens=xp, probs=rp, row_indices=dest_row.view(T, k), expert_indices=idx.long(),
                              counts=recv_counts, seg_start=seg_start, tile_group=tile_group,
                              out_buffer=ws.y_rows, grad_buffer=ws.y_rows)
        return perm, recv_counts, ("p2p", ws, expert, dest_row, seg_start, recv_counts, T, k)

    def combine(self, y, state, residual=None):
        if state[0] != "p2p":
            return self._nccl().combine(y, state)
        _, ws, expert, dest_row, seg_start, recv_counts, T, k = state
        return _Combine.apply(y, expert, dest_row, seg_start, recv_counts, ws, T, k, residual)
