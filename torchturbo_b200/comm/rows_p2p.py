"""All-to-all-v of rows over peer memory: every rank writes its rows straight into the destination's receive buffer
(NVLink stores), no NCCL, no pack / unpack.

`p2p_all_to_all_rows(group, x, matrix)` is a drop-in for `all_to_all(group, x, out_splits, in_splits)` when every rank
knows the whole split matrix `matrix[s][d]` = rows rank `s` sends to rank `d` (the vision balancer does: all ranks
derive the same plan from gathered metadata).  Rows of `x` are ordered by destination; the result is ordered by
source.  Any dtype whose rows are a multiple of 16 bytes is moved as raw bytes.  The backward pass is the same
exchange with the transposed matrix.

Protocol per call (epoch e) on the group's shared receive buffer:
    wait   "consumed" flags of epoch e-1 from every peer   (they copied their rows out of their buffers)
    scatter rows -> owners' buffers at the row offset reserved for this source, then "landed" flags (epoch e)
    wait   "landed" flags of epoch e from every source
    copy   the received rows out, then publish "consumed" (epoch e) to every peer
The buffer grows when a call needs more rows than it holds; the decision is a function of `matrix` alone, so every
rank takes it in the same call and the (collective) re-allocation lines up.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import kernels as K
from .symm import SymmetricBuffer

_WS: dict[tuple, "_RowsWorkspace"] = {}


class _RowsWorkspace:
    def __init__(self, group, row_bytes: int, cap_rows: int):
        self.group, self.row_bytes, self.cap = group, row_bytes, cap_rows
        self.W, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.buf = SymmetricBuffer(cap_rows * row_bytes + 8 * 4 * self.W + 16 * 256, group)
        self.off_rows, self.rows = self.buf.carve(cap_rows * row_bytes, torch.bfloat16, (cap_rows, row_bytes // 2))
        self.ch_landed, self.ch_consumed = self.buf.channel(), self.buf.channel()
        dev = self.buf.local.device
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        self.budget_ms = int(os.environ.get("TORCHTURBO_P2P_WAIT_MS", "5000"))
        self.ptrs = self.buf.peer_ptrs

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"row exchange failed on rank {self.rank}: status {code:#x}")


def usable(group, x: torch.Tensor) -> bool:
    if group is None or not (x.is_cuda and K.available()):
        return False
    if os.environ.get("TORCHTURBO_ROWS_TRANSPORT", "auto") == "nccl":
        return False
    if x.dim() != 2:
        return False
    row_bytes = x.shape[1] * x.element_size()
    return row_bytes % 16 == 0 and SymmetricBuffer.usable(group) and dist.get_world_size(group) > 1


def _workspace(group, row_bytes: int, need_rows: int) -> _RowsWorkspace:
    key = (id(group), row_bytes)
    ws = _WS.get(key)
    if ws is None or ws.cap < need_rows:
        cap = max(need_rows, 1024) if ws is None else max(need_rows, 2 * ws.cap)
        if ws is not None:
            torch.cuda.synchronize()                     # nobody may still be reading the buffer that is replaced
            dist.barrier(group=group)
        ws = _RowsWorkspace(group, row_bytes, cap)
        _WS[key] = ws
    return ws


def _exchange(group, x: torch.Tensor, matrix) -> torch.Tensor:
    W, me = dist.get_world_size(group), dist.get_rank(group)
    row_bytes = x.shape[1] * x.element_size()
    recv_rows = [sum(matrix[s][d] for s in range(W)) for d in range(W)]
    ws = _workspace(group, row_bytes, max(recv_rows))
    n_send = sum(matrix[me])
    assert x.shape[0] == n_send, (x.shape, matrix[me])
    dest = torch.repeat_interleave(torch.arange(W, dtype=torch.int32), torch.tensor(matrix[me]))
    base = torch.tensor([sum(matrix[s][d] for s in range(me)) for d in range(W)], dtype=torch.int32)
    within = torch.cat([torch.arange(n, dtype=torch.int32) for n in matrix[me]]) if n_send else torch.zeros(0, dtype=torch.int32)
    dest_row = base[dest.long()] + within
    dev = x.device
    dest_d, row_d = dest.to(dev), dest_row.to(dev)
    raw = x.contiguous().view(torch.uint8).view(x.shape[0], row_bytes).view(torch.bfloat16)
    if ws.ch_landed.epoch > 0:
        K.flag_wait(ws.ptrs, ws.ch_consumed.offset, ws.rank, ws.W, ws.ch_consumed.epoch, ws.budget_ms, ws.status)
    epoch = ws.ch_landed.next()
    if n_send == 0:
        raw = torch.zeros(1, row_bytes // 2, dtype=torch.bfloat16, device=dev)
    K.ep_scatter(ws.ptrs, ws.off_rows, 0, ws.ch_landed.offset, raw, dest_d, row_d, None, 1, 1, ws.rank, ws.W, epoch, ws.cap,
                 ws.done, ws.status)
    K.flag_wait(ws.ptrs, ws.ch_landed.offset, ws.rank, ws.W, epoch, ws.budget_ms, ws.status)
    out = ws.rows[: recv_rows[me]].clone()
    K.flag_signal(ws.ptrs, ws.ch_consumed.offset, ws.rank, ws.W, ws.ch_consumed.next())
    return out.view(torch.uint8).view(recv_rows[me], row_bytes).view(x.dtype).view(recv_rows[me], x.shape[1])


class _P2PRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, matrix):
        ctx.group, ctx.matrix = group, matrix
        return _exchange(group, x, matrix)

    @staticmethod
    def backward(ctx, g):
        W = len(ctx.matrix)
        transposed = [[ctx.matrix[d][s] for d in range(W)] for s in range(W)]
        return _exchange(ctx.group, g.contiguous(), transposed), None, None


def p2p_all_to_all_rows(group, x: torch.Tensor, matrix) -> torch.Tensor:
    return _P2PRows.apply(x, group, [list(map(int, r)) for r in matrix])
