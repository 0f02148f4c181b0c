"""Park optimizer state on the host between training windows (RL loops that alternate generation and training).

`offload()` moves every state tensor to pinned CPU memory and frees the device copies; `restore()` brings them back.
While suspended, `step()`, `state_dict()` and `load_state_dict()` of the optimizer raise instead of silently
operating on missing state (engine/backends/fsdp2/optimizers/memory.py:95-279 of the reference)."""
from __future__ import annotations

import torch


class OptimizerSuspendedError(RuntimeError):
    pass


def _local(t):
    return t._local_tensor if hasattr(t, "_local_tensor") else t


class OptimizerMemoryController:
    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.suspended = False
        self._host: dict[tuple[int, str], tuple[torch.Tensor, torch.device]] = {}
        self._guarded = False

    def _children(self):
        from .container import OptimizersContainer

        return list(self.optimizer) if isinstance(self.optimizer, OptimizersContainer) else [self.optimizer]

    def _install_guards(self) -> None:
        if self._guarded:
            return
        ctl = self
        for opt in self._children():
            for name in ("step", "state_dict", "load_state_dict"):
                orig = getattr(opt, name)

                def guarded(*a, __orig=orig, __name=name, **k):
                    if ctl.suspended:
                        raise OptimizerSuspendedError(f"optimizer.{__name}() called while its state is offloaded; "
                                                      "call engine.restore_optimizer() first")
                    return __orig(*a, **k)

                setattr(opt, name, guarded)
        self._guarded = True

    @torch.no_grad()
    def offload(self) -> int:
        """Returns the number of bytes moved to the host."""
        if self.suspended:
            return 0
        self._install_guards()
        moved = 0
        for opt in self._children():
            if hasattr(opt, "_plans"):
                opt._plans.clear()  # device tables point at buffers that are about to go away
            for p, st in opt.state.items():
                for k, v in list(st.items()):
                    if isinstance(v, torch.Tensor) and _local(v).is_cuda:
                        lv = _local(v)
                        host = torch.empty(lv.shape, dtype=lv.dtype, device="cpu", pin_memory=True)
                        host.copy_(lv, non_blocking=True)
                        self._host[(id(p), k)] = (host, lv.device)
                        moved += lv.numel() * lv.element_size()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        for opt in self._children():
            for p, st in opt.state.items():
                for k, v in list(st.items()):
                    if (id(p), k) in self._host:
                        _local(v).data = torch.empty(0, dtype=_local(v).dtype, device=_local(v).device)
        self.suspended = True
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        return moved

    @torch.no_grad()
    def restore(self) -> None:
        if not self.suspended:
            return
        for opt in self._children():
            for p, st in opt.state.items():
                for k, v in st.items():
                    key = (id(p), k)
                    if key in self._host:
                        host, dev = self._host.pop(key)
                        _local(v).data = host.to(dev, non_blocking=True)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.suspended = False
