"""Expert-parallel token dispatch / combine over peer memory (NVLink), without NCCL and without host reads.

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

import os

import torch
import torch.distributed as dist

from .. import kernels as K
from ..ops import MoEPermutation, ops
from .symm import SymmetricBuffer

_WORKSPACES: dict[tuple, "EPWorkspace"] = {}


class EPWorkspace:
    def __init__(self, group, hidden: int, num_experts: int, tokens: int, topk: int, capacity_factor: float):
        self.group = group
        self.W, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.E, self.El, self.H = num_experts, num_experts // self.W, hidden
        rows = int(tokens * topk * capacity_factor)
        self.m_tiles_cap = (rows + K.SEG_ALIGN - 1) // K.SEG_ALIGN + self.El
        self.cap = self.m_tiles_cap * K.SEG_ALIGN
        nbytes = 4 * self.W * self.E + 2 * self.cap * hidden * 2 + 2 * self.cap * 4 + 8 * 4 * self.W + 16 * 256
        self.buf = SymmetricBuffer(nbytes, group)
        self.off_counts, self.counts_all = self.buf.carve(4 * self.W * self.E, torch.int32)
        self.off_recv, self.recv_rows = self.buf.carve(self.cap * hidden * 2, torch.bfloat16, (self.cap, hidden))
        self.off_recv_vals, self.recv_vals = self.buf.carve(self.cap * 4, torch.float32)
        self.off_y, self.y_rows = self.buf.carve(self.cap * hidden * 2, torch.bfloat16, (self.cap, hidden))
        self.off_y_vals, self.y_vals = self.buf.carve(self.cap * 4, torch.float32)
        self.ch_counts, self.ch_rows, self.ch_ready = self.buf.channel(), self.buf.channel(), self.buf.channel()
        dev = self.buf.local.device
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        self.budget_ms = int(os.environ.get("TORCHTURBO_P2P_WAIT_MS", "5000"))
        self.ptrs = self.buf.peer_ptrs

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
            what = "receive capacity exceeded (raise capacity_factor)" if code == 2 else \
                "row index outside the receive buffer" if code == 3 else f"peer wait timed out (code {code:#x})"
            raise RuntimeError(f"expert-parallel exchange failed on rank {self.rank}: {what}")


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
