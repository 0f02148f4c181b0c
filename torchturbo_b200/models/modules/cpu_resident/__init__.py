"""Frozen giant lookup tables that stay in host memory.

`CPUResidentParameter` keeps a frozen tensor on the CPU (pinned when a GPU is present) and serves row lookups by
gathering the requested rows on the host and copying only those to the device, so a table far larger than HBM headroom
costs no device memory.  `NodeSharedCPUResidentParameter` additionally maps one copy per node from `/dev/shm`: local
rank 0 creates and fills the file, the other ranks of the node map it read-only after a node-local barrier
(models/modules/cpu_resident/{base,node_shared}.py of the reference).
"""
from __future__ import annotations

import mmap
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

_NP = {torch.float32: np.float32, torch.float16: np.float16, torch.int64: np.int64, torch.int32: np.int32,
       torch.uint8: np.uint8, torch.bfloat16: np.uint16}


class CPUResidentParameter(nn.Module):
    def __init__(self, num_rows: int, dim: int, dtype: torch.dtype = torch.bfloat16, pin: bool | None = None):
        super().__init__()
        self.num_rows, self.dim, self.dtype = num_rows, dim, dtype
        pin = torch.cuda.is_available() if pin is None else pin
        self._table = self._allocate(pin)

    def _allocate(self, pin: bool) -> torch.Tensor:
        t = torch.zeros(self.num_rows, self.dim, dtype=self.dtype)
        return t.pin_memory() if pin else t

    @property
    def table(self) -> torch.Tensor:
        return self._table

    def _apply(self, fn, recurse=True):  # stays on the host whatever `.to()` / FSDP do to the parent
        return self

    def load_rows(self, start: int, rows: torch.Tensor) -> None:
        """Shard I/O: copy `rows` into `[start, start + len(rows))`."""
        self._table[start:start + rows.shape[0]].copy_(rows.to(self.dtype))

    @torch.no_grad()
    def forward(self, index: torch.Tensor) -> torch.Tensor:
        idx = index.reshape(-1).cpu()
        rows = self._table.index_select(0, idx)
        if index.is_cuda:
            rows = rows.pin_memory().to(index.device, non_blocking=True) if torch.cuda.is_available() else rows
        return rows.view(*index.shape, self.dim)

    def state_dict(self, *a, **k):  # frozen and host-resident: saved through shard I/O, not through the model state
        return {}


class NodeSharedCPUResidentParameter(CPUResidentParameter):
    def __init__(self, num_rows: int, dim: int, dtype: torch.dtype = torch.bfloat16, name: str = "table",
                 local_rank: int | None = None, node_group=None, shm_dir: str = "/dev/shm"):
        self.name = name
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0")) if local_rank is None else local_rank
        self.node_group = node_group
        self.path = os.path.join(shm_dir, f"ttb200_{name}_{num_rows}x{dim}_{os.environ.get('MASTER_PORT', '0')}.bin")
        self._mm = None
        super().__init__(num_rows, dim, dtype, pin=False)

    def _barrier(self) -> None:
        if dist.is_initialized() and dist.get_world_size(self.node_group) > 1:
            dist.barrier(self.node_group)

    def _allocate(self, pin: bool) -> torch.Tensor:
        nbytes = self.num_rows * self.dim * torch.empty(0, dtype=self.dtype).element_size()
        if self.local_rank == 0:
            with open(self.path, "wb") as f:
                f.truncate(nbytes)
        self._barrier()
        fd = os.open(self.path, os.O_RDWR if self.local_rank == 0 else os.O_RDONLY)
        try:
            self._mm = mmap.mmap(fd, nbytes, access=mmap.ACCESS_WRITE if self.local_rank == 0 else mmap.ACCESS_READ)
        finally:
            os.close(fd)
        arr = np.frombuffer(self._mm, dtype=_NP[self.dtype]).reshape(self.num_rows, self.dim)
        t = torch.from_numpy(arr) if self.local_rank == 0 else torch.from_numpy(arr.view())
        return t.view(self.dtype) if self.dtype == torch.bfloat16 else t

    def load_rows(self, start: int, rows: torch.Tensor) -> None:
        if self.local_rank == 0:
            super().load_rows(start, rows)

    def finish_loading(self) -> None:
        """Make rank 0's writes visible to the readers of the node."""
        if self.local_rank == 0 and self._mm is not None:
            self._mm.flush()
        self._barrier()

    def close(self) -> None:
        self._barrier()
        if self.local_rank == 0 and os.path.exists(self.path):
            os.unlink(self.path)
