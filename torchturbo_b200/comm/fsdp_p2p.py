"""Peer-memory (NVLink) all-gather and reduce-scatter for FSDP2 units.

`torch.distributed.fsdp.fully_shard` lets a unit replace its two collectives (`set_custom_all_gather`,
`set_custom_reduce_scatter`): the object allocates the communication buffer and performs the collective on the
stream FSDP selected.  Here the buffers are slots of one symmetric (peer-mapped) arena per process group and the
collectives are pull kernels (`csrc/comm.cu`, `peer_allgather_kernel` / `peer_reduce_scatter_kernel`):

    all-gather      FSDP copies this rank's bf16 shard into piece `rank` of the slot (its own copy-in);
                    signal `ready`; the kernel waits for the peers' `ready` and copies their pieces over NVLink.
    reduce-scatter  FSDP packs the unit's gradients as `[W, n]` pieces into the slot (its own chunk-cat copy-in,
                    which is also the bf16 -> fp32 cast); signal `ready`; the kernel sums piece `rank` of every
                    peer's slot in fp32, applies the averaging scale and writes the sharded gradient.

Slot reuse: a rank may overwrite a slot only after every peer has read it; each kernel raises `consumed` on all
peers when it is done and the next `allocate()` of the slot enqueues the wait for those flags on the stream that
will write it.  Slots are handed out round-robin; every rank runs the same FSDP schedule, so slot numbers and
epochs agree without communication.  A request that does not fit a slot, has an unsupported dtype / reduce op, or
finds its slot still referenced locally is served by the NCCL collective instead (decided from shapes only, so all
ranks decide alike).  The number of slots bounds how many collectives FSDP may keep alive at once: an all-gather
result lives from its copy-in to its copy-out (current unit + prefetched units + the one whose buffer release is
deferred by one unit), a reduce-scatter input until the next reduce-scatter has been issued; FSDP orders a new
copy-in after the copy-out of the previous unit, so `prefetch depth + 4` all-gather slots and 3 reduce-scatter
slots are never overwritten while still being read locally.  Slots are capped at 1 GiB (all-gather) / 2 GiB
(reduce-scatter input): larger units, e.g. a 150k-row embedding of a wide model, keep NCCL.

The reference runs these collectives through NCCL inside torch FSDP2 (engine/backends/fsdp2/backend.py:420-470).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch.distributed.fsdp._fully_shard._fsdp_api import AllGather, ReduceScatter

from .. import kernels as K
from .symm import SymmetricBuffer

_ARENAS: dict[int, "PeerCollectiveArena"] = {}


class _Slot:
    def __init__(self, buf: SymmetricBuffer, nbytes: int):
        self.offset, self.bytes = buf.carve(nbytes, torch.uint8)
        self.ready, self.consumed = buf.channel(), buf.channel()
        self.epoch = 0          # epoch of the collective that last used the slot


class PeerCollectiveArena:
    """Symmetric memory for the FSDP collectives of one process group: `n_ag` all-gather slots of `ag_bytes` and
    `n_rs` reduce-scatter input slots of `rs_bytes`."""

    def __init__(self, group, ag_bytes: int, rs_bytes: int, n_ag: int = 6, n_rs: int = 3):
        self.group = group
        self.W, self.rank = dist.get_world_size(group), dist.get_rank(group)
        ag_bytes, rs_bytes = (ag_bytes + 255) // 256 * 256, (rs_bytes + 255) // 256 * 256
        total = n_ag * ag_bytes + n_rs * rs_bytes + (n_ag + n_rs) * (2 * 4 * self.W + 512) + 4096
        self.buf = SymmetricBuffer(total, group)
        self.ag = [_Slot(self.buf, ag_bytes) for _ in range(n_ag)]
        self.rs = [_Slot(self.buf, rs_bytes) for _ in range(n_rs)]
        self.ag_bytes, self.rs_bytes = ag_bytes, rs_bytes
        self._ag_next = self._rs_next = 0
        dev = self.buf.local.device
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        # one counter per stream role: kernels of one role are stream-ordered, kernels of different roles overlap
        self.done_ag = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done_rs = torch.zeros(1, dtype=torch.int32, device=dev)
        self.budget_ms = int(os.environ.get("TORCHTURBO_P2P_WAIT_MS", "5000"))
        self.grid = int(os.environ.get("TORCHTURBO_FSDP_P2P_GRID", "96"))
        self.by_ptr: dict[int, _Slot] = {s.bytes.data_ptr(): s for s in self.ag + self.rs}
        self.calls = {"all_gather": 0, "reduce_scatter": 0, "nccl": 0}

    def take(self, kind: str, nbytes: int, dtype, shape) -> torch.Tensor | None:
        slots = self.ag if kind == "ag" else self.rs
        if nbytes > slots[0].bytes.numel():
            return None
        i = self._ag_next if kind == "ag" else self._rs_next
        if kind == "ag":
            self._ag_next = (i + 1) % len(slots)
        else:
            self._rs_next = (i + 1) % len(slots)
        slot = slots[i]
        if slot.epoch:
            # every peer has finished reading what this slot held before it is written again
            K.flag_wait(self.buf.peer_ptrs, slot.consumed.offset, self.rank, self.W, slot.epoch, self.budget_ms, self.status)
        return slot.bytes[:nbytes].view(dtype).view(*shape)

    def run(self, slot: _Slot, kind: int, units: int, out=None, scale: float = 1.0) -> None:
        slot.epoch = slot.ready.next()
        slot.consumed.epoch = slot.epoch
        K.flag_signal(self.buf.peer_ptrs, slot.ready.offset, self.rank, self.W, slot.epoch)
        # the wait for the peers runs as a one-CTA kernel of its own: a peer can be milliseconds behind, and the ~100
        # CTAs of the copy kernel must not sit on the SMs spinning (and crowding out compute) for that long
        K.flag_wait(self.buf.peer_ptrs, slot.ready.offset, self.rank, self.W, slot.epoch, self.budget_ms, self.status)
        K.peer_collective(self.buf.peer_ptrs, slot.offset, slot.ready.offset, slot.consumed.offset, units, self.rank,
                          self.W, slot.epoch, self.budget_ms, self.done_ag if kind == 0 else self.done_rs, self.status,
                          kind=kind, out=out, scale=scale, grid=self.grid)

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"peer-memory FSDP collective timed out on rank {self.rank} (code {code:#x})")


def _numel(size) -> int:
    n = 1
    for s in size:
        n *= int(s)
    return n


class PeerAllGather(AllGather):
    def __init__(self, arena: PeerCollectiveArena):
        self.arena = arena

    def allocate(self, size, *, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        size = tuple(int(s) for s in size)
        nbytes = _numel(size) * dtype.itemsize
        t = None
        if (nbytes // self.arena.W) % 16 == 0 and nbytes > 0:
            t = self.arena.take("ag", nbytes, dtype, size)
        return t if t is not None else torch.empty(*size, dtype=dtype, device=device)

    def __call__(self, output_tensor, input_tensor, group, async_op: bool = False):
        a = self.arena
        slot = a.by_ptr.get(output_tensor.data_ptr())
        if slot is None:
            a.calls["nccl"] += 1
            return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)
        a.calls["all_gather"] += 1
        a.run(slot, 0, input_tensor.numel() * input_tensor.element_size() // 16)
        return None


class PeerReduceScatter(ReduceScatter):
    def __init__(self, arena: PeerCollectiveArena):
        self.arena = arena
        self._pending_input_numel = None

    def allocate(self, size, *, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        size = tuple(int(s) for s in size)
        n = _numel(size)
        if self._pending_input_numel is not None and n * self.arena.W == self._pending_input_numel:
            self._pending_input_numel = None     # the matching output: ordinary memory, written by this rank only
            return torch.empty(*size, dtype=dtype, device=device)
        self._pending_input_numel = n
        nbytes = n * dtype.itemsize
        t = None
        if dtype in (torch.float32, torch.bfloat16) and n > 0 and (nbytes // self.arena.W) % 16 == 0:
            t = self.arena.take("rs", nbytes, dtype, size)
        return t if t is not None else torch.empty(*size, dtype=dtype, device=device)

    def __call__(self, output_tensor, input_tensor, group, op, async_op: bool = False):
        a = self.arena
        slot = a.by_ptr.get(input_tensor.data_ptr())
        scale = 1.0 if op == dist.ReduceOp.SUM else (1.0 / a.W if op == dist.ReduceOp.AVG else None)
        if slot is None or scale is None or output_tensor.data_ptr() % 16:
            a.calls["nccl"] += 1
            return dist.reduce_scatter_tensor(output=output_tensor, input=input_tensor, group=group, op=op, async_op=async_op)
        a.calls["reduce_scatter"] += 1
        kind = 1 if input_tensor.dtype == torch.float32 else 2
        a.run(slot, kind, output_tensor.numel() * output_tensor.element_size() // 16, out=output_tensor, scale=scale)
        return None


def usable(group) -> bool:
    if os.environ.get("TORCHTURBO_FSDP_TRANSPORT", "p2p").lower() == "nccl":
        return False
    return K.available() and SymmetricBuffer.usable(group) and dist.get_world_size(group) > 1


def install(units, group, *, prefetch_depth: int = 1) -> PeerCollectiveArena | None:
    """Give every FSDP unit of `units` (all sharded over `group`) the peer-memory collectives.  Slot sizes come from
    the largest unit, capped by `TORCHTURBO_FSDP_P2P_MAX_SLOT_MB` (larger units keep NCCL)."""
    units = [u for u in units if hasattr(u, "set_custom_all_gather")]
    if not units or not usable(group):
        return None
    W = dist.get_world_size(group)
    biggest = 0
    for u in units:
        pg = u._get_fsdp_state()._fsdp_param_group
        if pg is None:
            continue
        n = sum(fp.padded_sharded_param_size.numel() for fp in pg.fsdp_params)
        biggest = max(biggest, n * W)
    cap = int(os.environ.get("TORCHTURBO_FSDP_P2P_MAX_SLOT_MB", "1024")) << 20
    ag_bytes = min(cap, biggest * 2 + 4096 * W)
    rs_bytes = min(2 * cap, biggest * 4 + 4096 * W)
    n_ag = int(os.environ.get("TORCHTURBO_FSDP_P2P_SLOTS", str(prefetch_depth + 4)))
    key = id(group)
    arena = _ARENAS.get(key)
    if arena is None or arena.ag_bytes < ag_bytes or arena.rs_bytes < rs_bytes:
        arena = PeerCollectiveArena(group, ag_bytes, rs_bytes, n_ag=n_ag, n_rs=3)
        _ARENAS[key] = arena
    ag, rs = PeerAllGather(arena), PeerReduceScatter(arena)
    for u in units:
        u.set_custom_all_gather(ag)
        u.set_custom_reduce_scatter(rs)
    return arena
