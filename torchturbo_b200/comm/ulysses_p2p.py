"""Ulysses sequence <-> head exchange over peer memory (NVLink), without NCCL.

Forward of one attention layer on every rank of the sequence-parallel group (stream-ordered, no host waits):
    qkv scatter kernel   : per-head RMSNorm + RoPE of q and k (the QKV projection's epilogue math) computed in
                           registers and stored straight into the owning ranks' `[T, heads/sp, D]` buffers, v copied
                           alongside; "rows landed" flags
    wait kernel          : every source has delivered -> attention runs on the local buffers
    output hand-off      : attention output copied to the symmetric output buffer, "output ready" flags
    wait + gather kernel : every rank pulls the heads of its own tokens from the owners -> `[T/sp, heads * D]` for o_proj
Backward mirrors it: d(output) rows are pushed to the owners, dq / dk / dv are pulled back (replicated kv heads are
summed) and flow into the QK-norm + RoPE backward kernel.

Buffers are shared by all layers: a rank starts writing layer L+1 data only after it has observed every peer's
layer-L "output ready" flag, which a peer raises after its attention stopped reading the receive buffers; forward and
backward use separate buffers and flag channels, so recomputation inside backward (activation checkpointing) keeps
the same ordering on every rank.

Replaces `gather_seq_scatter_heads` x3 + `gather_heads_scatter_seq` and their pack / unpack copies
(models/modules/attention/ulysses/ulysses.py:307-327,381-383 of the reference).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import kernels as K
from .symm import SymmetricBuffer

_WORKSPACES: dict[tuple, "UlyssesWorkspace"] = {}
D = 128


class UlyssesWorkspace:
    """Symmetric buffers for up to `cap_local` tokens per rank.  A call with `Tl` local tokens uses the first
    `Tl * W` rows of every buffer (`rows()`), so one workspace serves every sequence length up to its capacity."""

    NAMES = ("q", "k", "v", "o", "do", "dq", "dk", "dv")

    def __init__(self, group, cap_local: int, n_q: int, n_kv: int, rep: int):
        self.group = group
        self.W, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.cap_local = cap_local
        Tc = cap_local * self.W
        self.n_q, self.n_kv, self.rep = n_q, n_kv, rep
        self.Hql, self.Hkl = n_q // self.W, n_kv * rep // self.W
        qb, kb = Tc * self.Hql * D * 2, Tc * self.Hkl * D * 2
        self.buf = SymmetricBuffer(4 * qb + 4 * kb + 16 * 256 + 8 * 4 * self.W, group)
        c = self.buf.carve
        self.off_q, self._q = c(qb, torch.bfloat16, (Tc, self.Hql, D))
        self.off_k, self._k = c(kb, torch.bfloat16, (Tc, self.Hkl, D))
        self.off_v, self._v = c(kb, torch.bfloat16, (Tc, self.Hkl, D))
        self.off_o, self._o = c(qb, torch.bfloat16, (Tc, self.Hql, D))
        self.off_do, self._do = c(qb, torch.bfloat16, (Tc, self.Hql, D))
        self.off_dq, self._dq = c(qb, torch.bfloat16, (Tc, self.Hql, D))
        self.off_dk, self._dk = c(kb, torch.bfloat16, (Tc, self.Hkl, D))
        self.off_dv, self._dv = c(kb, torch.bfloat16, (Tc, self.Hkl, D))
        self.ch_qkv, self.ch_out, self.ch_dout, self.ch_dqkv = (self.buf.channel() for _ in range(4))
        dev = self.buf.local.device
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        self.budget_ms = int(os.environ.get("TORCHTURBO_P2P_WAIT_MS", "5000"))
        self.ptrs = self.buf.peer_ptrs

    def rows(self, name: str, Tl: int) -> torch.Tensor:
        """The `[Tl * W, heads, D]` part of buffer `name` that a call with `Tl` local tokens reads and writes."""
        return getattr(self, "_" + name)[:Tl * self.W]

    def wait(self, ch, epoch):
        K.flag_wait(self.ptrs, ch.offset, self.rank, self.W, epoch, self.budget_ms, self.status)

    def ready(self, ch):
        epoch = ch.next()
        K.flag_signal(self.ptrs, ch.offset, self.rank, self.W, epoch)
        self.wait(ch, epoch)

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"sequence-parallel exchange failed on rank {self.rank}: peer wait timed out (code {code:#x})")


def get_workspace(group, tokens_local: int, n_q: int, n_kv: int, rep: int) -> UlyssesWorkspace:
    """One workspace per (group, head counts), sized by a token capacity: the first request rounded up to 1024 tokens
    (or `TORCHTURBO_ULYSSES_MAX_TOKENS`), doubled when a longer row arrives.  The local token count is equal on every
    rank of the group (the row is padded to a multiple of `sp` before it is sliced), so all ranks create and grow the
    workspace at the same call without an agreement step.  A workspace that was outgrown is dropped from the table;
    autograd nodes that still hold it finish their backward on it."""
    key = (id(group), n_q, n_kv, rep)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.cap_local < tokens_local:
        preset = int(os.environ.get("TORCHTURBO_ULYSSES_MAX_TOKENS", "0"))
        cap = max((tokens_local + 1023) // 1024 * 1024, preset, 2 * ws.cap_local if ws is not None else 0)
        ws = UlyssesWorkspace(group, cap, n_q, n_kv, rep)
        _WORKSPACES[key] = ws
    return ws


def kv_replication(n_q: int, n_kv: int, sp: int) -> int | None:
    """How often each kv head is repeated so that heads divide over the group; None when the layout is unsupported."""
    if n_q % sp:
        return None
    if n_kv % sp == 0:
        rep = 1
    elif sp % n_kv == 0:
        rep = sp // n_kv
    else:
        return None
    # query heads of a rank must map onto the kv heads of the same rank
    hql, hkl = n_q // sp, n_kv * rep // sp
    return rep if hql % hkl == 0 else None


def usable(group, qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int) -> bool:
    if group is None or not (qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim == D and K.available()):
        return False
    if os.environ.get("TORCHTURBO_ULYSSES_TRANSPORT", "auto") == "nccl":
        return False
    return SymmetricBuffer.usable(group) and kv_replication(n_q, n_kv, dist.get_world_size(group)) is not None


class _QKVExchange(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, wq, wk, cos, sin, eps, n_q, n_kv, ws: UlyssesWorkspace):
        use_norm = wq is not None
        epoch = ws.ch_qkv.next()
        rstd = K.ulysses_qkv_scatter(ws.ptrs, ws.off_q, ws.off_k, ws.off_v, ws.ch_qkv.offset, qkv, n_q, n_kv, ws.rep, wq, wk,
                                     cos, sin, eps, ws.rank, ws.W, epoch, ws.done, use_norm)
        ws.wait(ws.ch_qkv, epoch)
        Tl = qkv.shape[0]
        q, k, v = ws.rows("q", Tl).clone(), ws.rows("k", Tl).clone(), ws.rows("v", Tl).clone()
        ctx.save_for_backward(qkv, wq, wk, cos, sin, rstd)
        ctx.ws, ctx.dims = ws, (n_q, n_kv, use_norm)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, wq, wk, cos, sin, rstd = ctx.saved_tensors
        ws, (n_q, n_kv, use_norm) = ctx.ws, ctx.dims
        Tl = qkv.shape[0]
        ws.rows("dq", Tl).copy_(dq)
        ws.rows("dk", Tl).copy_(dk)
        ws.rows("dv", Tl).copy_(dv)
        ws.ready(ws.ch_dqkv)
        dql = torch.empty(Tl, n_q, D, dtype=qkv.dtype, device=qkv.device)
        dkl = torch.empty(Tl, n_kv, D, dtype=qkv.dtype, device=qkv.device)
        dvl = torch.empty(Tl, n_kv, D, dtype=qkv.dtype, device=qkv.device)
        K.ulysses_move(ws.ptrs, ws.off_dq, 0, dql, n_q, 1, ws.rank, ws.W, 0, ws.done, ws.status, True)
        K.ulysses_move(ws.ptrs, ws.off_dk, 0, dkl, n_kv, ws.rep, ws.rank, ws.W, 0, ws.done, ws.status, True)
        K.ulysses_move(ws.ptrs, ws.off_dv, 0, dvl, n_kv, ws.rep, ws.rank, ws.W, 0, ws.done, ws.status, True)
        dqkv = torch.empty_like(qkv)
        dqkv[:, (n_q + n_kv) * D:] = dvl.reshape(Tl, n_kv * D)
        dwq, dwk = K.qknorm_rope_bwd(dql, dkl, qkv, n_q, n_kv, D, wq, wk, cos, sin, rstd, dqkv, use_norm)
        return (dqkv, dwq.to(wq.dtype) if use_norm else None, dwk.to(wk.dtype) if use_norm else None, None, None, None,
                None, None, None)


class _OutExchange(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o_full, ws: UlyssesWorkspace):
        Tl = o_full.shape[0] // ws.W
        ws.rows("o", Tl).copy_(o_full)
        ws.ready(ws.ch_out)
        out = torch.empty(Tl, ws.n_q, D, dtype=o_full.dtype, device=o_full.device)
        K.ulysses_move(ws.ptrs, ws.off_o, 0, out, ws.n_q, 1, ws.rank, ws.W, 0, ws.done, ws.status, True)
        ctx.ws, ctx.Tl = ws, Tl
        return out

    @staticmethod
    def backward(ctx, dout):
        ws = ctx.ws
        epoch = ws.ch_dout.next()
        K.ulysses_move(ws.ptrs, ws.off_do, ws.ch_dout.offset, dout.contiguous(), ws.n_q, 1, ws.rank, ws.W, epoch, ws.done,
                       ws.status, False)
        ws.wait(ws.ch_dout, epoch)
        return ws.rows("do", ctx.Tl).clone(), None


def qkv_exchange(qkv, n_q, n_kv, wq, wk, cos, sin, eps, group):
    """qkv [T/sp, (n_q + 2 n_kv) * 128] -> q [T, n_q/sp, 128], k, v [T, n_kv*rep/sp, 128] (normalised and rotated)."""
    sp = dist.get_world_size(group)
    ws = get_workspace(group, qkv.shape[0], n_q, n_kv, kv_replication(n_q, n_kv, sp))
    q, k, v = _QKVExchange.apply(qkv, wq, wk, cos.float().contiguous(), sin.float().contiguous(), eps, n_q, n_kv, ws)
    return q, k, v, ws


def out_exchange(o_full, ws: UlyssesWorkspace):
    """attention output [T, n_q/sp, 128] -> [T/sp, n_q, 128]"""
    return _OutExchange.apply(o_full.contiguous(), ws)
