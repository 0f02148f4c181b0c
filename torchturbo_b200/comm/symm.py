"""Symmetric (peer-mapped) device buffers for the in-kernel NVLink paths.

`SymmetricBuffer(nbytes, group)` allocates the same number of bytes on every rank of `group` through
`torch.distributed._symmetric_memory` (CUDA VMM handles exchanged over the group's store) and exposes
  * `local`      : this rank's bytes as a uint8 tensor,
  * `peer_ptrs`  : ctypes array with the device-visible base address of every rank's buffer (index = group rank),
  * `carve(...)` : named sub-ranges (offset, tensor view) inside the buffer,
  * `channel(n)` : a flag array `[W]` int32 plus a host-side epoch counter; all ranks call the same sequence of
                   operations on a channel, so the counters stay in lock-step without communication.
Flags start at zero, epochs at one.  The reference has no counterpart (it only uses torch.distributed collectives:
engine/distributed.py, models/modules/comm/comm.py).
"""
from __future__ import annotations

import importlib

import ctypes as C
import os

import torch
import torch.distributed as dist


class Channel:
    def __init__(self, offset: int, view: torch.Tensor):
        self.offset, self.view, self.epoch = offset, view, 0

    def next(self) -> int:
        self.epoch += 1
        return self.epoch


class SymmetricBuffer:
    def __init__(self, nbytes: int, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        nbytes = (int(nbytes) + 255) // 256 * 256
        dev = torch.device("cuda", torch.cuda.current_device())
        name = self.group.group_name
        try:
            if not symm_mem.is_symm_mem_enabled_for_group(name):
                symm_mem.enable_symm_mem_for_group(name)
        except Exception:
            pass
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        self.local.zero_()
        torch.cuda.synchronize()
        self.handle = symm_mem.rendezvous(self.local, self.group)
        ptrs = list(self.handle.buffer_ptrs)
        assert len(ptrs) == self.world and ptrs[self.rank] == self.local.data_ptr()
        self.peer_ptrs = (C.c_ulonglong * self.world)(*ptrs)
        # NVSwitch multicast address of the same buffer (0 when the fabric or the driver has no multicast support):
        # `multimem.*` instructions on it reduce in the switch / store to every rank at once
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if os.environ.get("TORCHTURBO_MULTIMEM", "1") == "0" or os.environ.get("NCCL_NVLS_ENABLE", "1") == "0":
            self.multicast_ptr = 0        # multicast deliberately off (failure-detection runs keep every library off it)
        self.nbytes = nbytes
        self._cursor = 0
        dist.barrier(self.group)

    def carve(self, nbytes: int, dtype=torch.uint8, shape=None) -> tuple[int, torch.Tensor]:
        off = (self._cursor + 255) // 256 * 256
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric buffer exhausted: need {off + nbytes} of {self.nbytes} bytes")
        self._cursor = off + nbytes
        view = self.local[off:off + nbytes].view(dtype)
        if shape is not None:
            view = view.view(*shape)
        return off, view

    def channel(self, n: int | None = None) -> Channel:
        """A block of `n` epoch flags (default: one per rank)."""
        off, view = self.carve(4 * (n or self.world), torch.int32)
        return Channel(off, view)

    @staticmethod
    def usable(group=None) -> bool:
        """Peer access over NVLink needs every rank of the group on one node with one device per process."""
        if not (torch.cuda.is_available() and dist.is_initialized()):
            return False
        try:
            importlib.import_module("torch.distributed._symmetric_memory")
        except Exception:
            return False
        g = group if group is not None else dist.group.WORLD
        return dist.get_backend(g) == "nccl" and dist.get_world_size(g) <= min(16, torch.cuda.device_count())
