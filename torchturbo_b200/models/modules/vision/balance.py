"""World-pooled load balancing of whole images across ranks for a vision tower.

Every step the media of all ranks are pooled (only the representative `sp_rank == 0` of each sequence-parallel group
publishes media: the members of a group hold identical batches), whole images are assigned to ranks with
longest-processing-time-first packing (weight = patches, or patches squared for attention-dominated towers), the
pixel rows travel to their owners, every owner runs the unmodified tower on what it received, and each output stream
is sent back to *every* member of the group the image came from, restored to the original image order.

Contract kept from models/modules/vision/balance.py of the reference: deterministic assignment reproduced on every
rank from gathered metadata (ties go to the lower rank), fallback to the local path when the pool holds fewer media
than ranks, a model-provided dummy medium for ranks that received nothing (so FSDP hooks and collectives stay
aligned), no balancing under `torch.no_grad()`, and gradients materialised for every stream so that all ranks run the
same backward exchanges in the same order.

Transport: on an NVLink domain the rows are written straight into the owners' buffers by a peer-memory kernel
(`comm/rows_p2p.py`); elsewhere `all_to_all` from `comm` (NCCL / gloo).  Row exchanges are all-to-all-v on dim 0.
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from ....parallel import VisionBalanceMode, VisionBalanceSpec
from ..comm import all_to_all
from .io import BaseVisionBalanceIO, VisionBatch


@dataclass
class MediaMeta:
    src: int                  # world rank that published it (an SP representative)
    index: int                # position among that rank's media
    grid: tuple[int, int, int]
    patches: int
    tokens: dict[str, int]    # output rows per stream
    weight: int
    owner: int = -1


def lpt_weight(patches: int, mode: VisionBalanceMode) -> int:
    return patches * patches if mode is VisionBalanceMode.PATCH_SQ else patches


class MediaPool:
    def __init__(self, media: list[MediaMeta]):
        self.media = media

    @classmethod
    def from_metadata(cls, metadata: list[list[list[int]]], output_names: tuple[str, ...], mode: VisionBalanceMode):
        """`metadata[rank]` holds rows `(t, h, w, *output_lengths)`; empty for non-representatives."""
        media = []
        for src, rows in enumerate(metadata):
            for i, row in enumerate(rows):
                t, h, w = (int(x) for x in row[:3])
                p = t * h * w
                media.append(MediaMeta(src, i, (t, h, w), p, dict(zip(output_names, (int(x) for x in row[3:]))),
                                       lpt_weight(p, mode)))
        return cls(media)

    def __len__(self) -> int:
        return len(self.media)

    def assign_owners(self, world_size: int) -> None:
        order = sorted(range(len(self.media)), key=lambda i: (-self.media[i].weight, i))
        heap = [(0, r) for r in range(world_size)]
        heapq.heapify(heap)
        for i in order:
            load, r = heapq.heappop(heap)
            self.media[i].owner = r
            heapq.heappush(heap, (load + self.media[i].weight, r))

    def assigned_to(self, rank: int) -> list[MediaMeta]:
        return [m for m in self.media if m.owner == rank]

    def contributed_by(self, rank: int) -> list[MediaMeta]:
        return [m for m in self.media if m.src == rank]

    def in_group(self, group: int, sp_size: int) -> list[MediaMeta]:
        return [m for m in self.media if m.src // sp_size == group]

    def pixel_matrix(self, world: int) -> list[list[int]]:
        """`m[s][d]`: pixel rows rank `s` sends to owner `d`."""
        m = [[0] * world for _ in range(world)]
        for x in self.media:
            m[x.src][x.owner] += x.patches
        return m

    def fanout_matrix(self, stream: str, world: int, sp_size: int) -> list[list[int]]:
        """`m[o][d]`: output rows of `stream` owner `o` returns to rank `d` (every member of the source group)."""
        m = [[0] * world for _ in range(world)]
        for x in self.media:
            g = x.src // sp_size
            for d in range(g * sp_size, (g + 1) * sp_size):
                m[x.owner][d] += x.tokens[stream]
        return m

    def loads(self, world_size: int) -> list[int]:
        out = [0] * world_size
        for m in self.media:
            out[m.owner] += m.weight
        return out


@dataclass
class PixelPlan:
    """Pixel exchange of one rank: rows to send per destination (in send order) and rows received per source."""

    send_order: list[MediaMeta]
    send_splits: list[int]
    recv_splits: list[int]

    @classmethod
    def build(cls, pool: MediaPool, rank: int, world: int) -> "PixelPlan":
        mine = pool.contributed_by(rank)
        send_order = sorted(mine, key=lambda m: (m.owner, m.index))
        send = [0] * world
        for m in mine:
            send[m.owner] += m.patches
        recv = [0] * world
        for m in pool.assigned_to(rank):
            recv[m.src] += m.patches
        return cls(send_order, send, recv)


@dataclass
class FanoutPlan:
    """Return path of one output stream: an owner sends each medium's rows to every member of the source group;
    a receiver gets its group's media owner-major and restores the original order."""

    send_rows: list[int] = field(default_factory=list)       # row indices into the owner's output, in send order
    send_splits: list[int] = field(default_factory=list)
    recv_splits: list[int] = field(default_factory=list)
    restore: list[int] = field(default_factory=list)         # row indices into the received buffer, original order

    @classmethod
    def build(cls, pool: MediaPool, stream: str, rank: int, world: int, sp_size: int) -> "FanoutPlan":
        mine = pool.assigned_to(rank)                         # tower output order on this rank
        starts, acc = {}, 0
        for m in mine:
            starts[(m.src, m.index)] = acc
            acc += m.tokens[stream]
        send_rows, send_splits = [], [0] * world
        for dst in range(world):
            g = dst // sp_size
            for m in mine:
                if m.src // sp_size == g:
                    s = starts[(m.src, m.index)]
                    send_rows.extend(range(s, s + m.tokens[stream]))
                    send_splits[dst] += m.tokens[stream]
        group = rank // sp_size
        gm = pool.in_group(group, sp_size)
        recv_splits = [0] * world
        pos, acc = {}, 0
        for owner in range(world):                            # receive buffer is owner-major, pooled order inside
            for m in gm:
                if m.owner == owner:
                    pos[(m.src, m.index)] = acc
                    acc += m.tokens[stream]
                    recv_splits[owner] += m.tokens[stream]
        restore = []
        for m in sorted(gm, key=lambda m: (m.src, m.index)):  # original order of the group's representative
            s = pos[(m.src, m.index)]
            restore.extend(range(s, s + m.tokens[stream]))
        return cls(send_rows, send_splits, recv_splits, restore)


class _MaterializeOutputGradients(torch.autograd.Function):
    """Identity over all streams whose backward replaces missing gradients by zeros, so that every rank runs the
    backward exchange of every stream even when its loss does not touch one of them."""

    @staticmethod
    def forward(ctx, *xs):
        ctx.meta = [(x.shape, x.dtype, x.device) for x in xs]
        return tuple(x.view_as(x) for x in xs)

    @staticmethod
    def backward(ctx, *gs):
        return tuple(g if g is not None else torch.zeros(s, dtype=dt, device=dev) for g, (s, dt, dev) in zip(gs, ctx.meta))


class VisionBalanceState:
    def __init__(self, tower: nn.Module, spec: VisionBalanceSpec, *, sp_group, sp_size: int, sp_rank: int, world_group):
        if spec.io is None or spec.mode is None:
            raise ValueError("vision balancing needs both a mode and an IO adapter")
        self.tower, self.mode, self.io = tower, spec.mode, spec.io
        self.sp_group, self.sp_size, self.sp_rank = sp_group, sp_size, sp_rank
        self.world_group = world_group
        self.world = dist.get_world_size(world_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(world_group) if dist.is_initialized() else 0
        self._ctx: dict[str, Any] | None = None
        self.last_pool: MediaPool | None = None

    # -- metadata ------------------------------------------------------------------------------------
    def _gather_metadata(self, batch: VisionBatch, names: tuple[str, ...]) -> list[list[list[int]]]:
        """Two all-gathers: media counts, then rows `(t, h, w, *lengths)` padded to the maximum count."""
        dev = batch.pixels.device
        n = batch.grid_thw.shape[0] if self.sp_rank == 0 else 0
        counts = torch.zeros(self.world, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(counts, torch.tensor([n], dtype=torch.int64, device=dev), group=self.world_group)
        counts_l = counts.tolist()
        mx = max(counts_l) if counts_l else 0
        width = 3 + len(names)
        rows = torch.zeros(max(mx, 1), width, dtype=torch.int64, device=dev)
        if n:
            rows[:n, :3] = batch.grid_thw.to(torch.int64)
            for j, name in enumerate(names):
                rows[:n, 3 + j] = torch.tensor(batch.output_lengths[name], dtype=torch.int64, device=dev)
        out = torch.zeros(self.world * max(mx, 1), width, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(out, rows, group=self.world_group)
        table = out.view(self.world, max(mx, 1), width).cpu().tolist()
        return [table[r][: counts_l[r]] for r in range(self.world)]

    # -- transport -----------------------------------------------------------------------------------
    def _exchange(self, send, recv_splits, send_splits, matrix):
        """Rows to their destinations: peer-memory stores on an NVLink domain (every rank knows the whole split matrix,
        so destination offsets need no extra exchange), NCCL / gloo all-to-all-v otherwise."""
        if send.is_cuda and send.dim() == 2:
            from ....comm import rows_p2p

            if rows_p2p.usable(self.world_group, send):
                return rows_p2p.p2p_all_to_all_rows(self.world_group, send, matrix)
        return all_to_all(self.world_group, send, recv_splits, send_splits)

    # -- hooks ---------------------------------------------------------------------------------------
    def pre_forward(self, module, args, kwargs):
        self._ctx = None
        if not torch.is_grad_enabled() or self.world == 1:
            return None
        batch = self.io.read_inputs(module, args, kwargs)
        # one element type on every rank: a rank without media feeds a dummy image that it builds itself, and the data
        # loader's type need not be the tower's (the patch embedding casts to the parameter type anyway)
        want = next((p.dtype for p in module.parameters()), batch.pixels.dtype)
        if batch.pixels.is_floating_point() and batch.pixels.dtype != want:
            batch = VisionBatch(batch.pixels.to(want), batch.grid_thw, batch.output_lengths)
        names = tuple(batch.output_lengths.keys())
        meta = self._gather_metadata(batch, names)
        pool = MediaPool.from_metadata(meta, names, self.mode)
        if len(pool) < self.world:
            return None  # sparse pool: keep the local path, no exchange
        pool.assign_owners(self.world)
        self.last_pool = pool
        plan = PixelPlan.build(pool, self.rank, self.world)
        # rows of my media in send order (non-representatives send nothing)
        starts, acc = [], 0
        for t, h, w in batch.grid_thw.tolist():
            starts.append(acc)
            acc += int(t * h * w)
        if plan.send_order:
            idx = torch.cat([torch.arange(starts[m.index], starts[m.index] + m.patches) for m in plan.send_order])
            send = batch.pixels.index_select(0, idx.to(batch.pixels.device))
        else:
            send = batch.pixels[:0]
        with torch.no_grad():
            recv = self._exchange(send.contiguous(), plan.recv_splits, plan.send_splits, pool.pixel_matrix(self.world))
        mine = pool.assigned_to(self.rank)
        # received rows are source-major with the sender's (owner, index) order == pooled order per source
        if mine:
            grid = torch.tensor([m.grid for m in mine], dtype=batch.grid_thw.dtype, device=batch.grid_thw.device)
            new = VisionBatch(recv, grid, {n_: [m.tokens[n_] for m in mine] for n_ in names})
            dummy = False
        else:
            new = self.io.make_dummy(module, batch)
            dummy = True
        self._ctx = dict(pool=pool, names=names, dummy=dummy, args=args, kwargs=kwargs)
        return self.io.write_inputs(module, args, kwargs, new)

    def post_forward(self, module, args, kwargs, output):
        ctx, self._ctx = self._ctx, None
        if ctx is None:
            return None
        pool, names = ctx["pool"], ctx["names"]
        streams = self.io.read_outputs(module, output)
        restored = []
        for name in names:
            x = streams[name]
            if ctx["dummy"]:
                x = x[:0] + 0.0 * x.sum()  # keep the graph connection of the dummy forward
            plan = FanoutPlan.build(pool, name, self.rank, self.world, self.sp_size)
            idx = torch.tensor(plan.send_rows, dtype=torch.long, device=x.device)
            send = x.index_select(0, idx) if idx.numel() else x[:0]
            recv = self._exchange(send.contiguous(), plan.recv_splits, plan.send_splits,
                                  pool.fanout_matrix(name, self.world, self.sp_size))
            ridx = torch.tensor(plan.restore, dtype=torch.long, device=x.device)
            restored.append(recv.index_select(0, ridx) if ridx.numel() else recv[:0])
        restored = _MaterializeOutputGradients.apply(*restored)
        return self.io.write_outputs(module, output, dict(zip(names, restored)))


def register_vision_balance(tower: nn.Module, spec: VisionBalanceSpec, *, sp_group=None, sp_size: int = 1,
                            sp_rank: int = 0, world_group=None) -> VisionBalanceState:
    """Install the pre/post forward hooks on `tower` (idempotent per tower)."""
    prev = getattr(tower, "_vision_balance_state", None)
    if prev is not None:
        return prev
    state = VisionBalanceState(tower, spec, sp_group=sp_group, sp_size=sp_size, sp_rank=sp_rank,
                               world_group=world_group if world_group is not None else (dist.group.WORLD if dist.is_initialized() else None))
    tower.register_forward_pre_hook(state.pre_forward, with_kwargs=True)
    tower.register_forward_hook(state.post_forward, with_kwargs=True)
    tower._vision_balance_state = state
    return state
