"""AdamW whose fp32 state (master weight, first and second moment) lives in pinned host memory.

`cpu_offload.mode = optimizer` keeps parameters and gradients on the GPU but parks the 12 bytes per parameter of
optimizer state on the host.  A step streams the state through a device workspace of bounded size:

    copy stream   : H2D of chunk i+1 (master, m, v) while
    compute stream: the fused AdamW kernel updates chunk i in the workspace and writes the bf16 weight, then
    copy stream   : D2H of chunk i

with two workspace slots, so transfers and updates overlap and the device never holds more than
`2 * chunk_elems * 12` bytes of state.  Parameters larger than a chunk are processed in slices.  On machines without
CUDA (and for CPU-resident parameters) the update runs on the host with the same formula.

Behavioural contract of engine/backends/fsdp2/optimizers/adamw.py:67-620 of the reference (`DeviceWorkspace`,
`AdamWSwap`): identical numerics to `torch.optim.AdamW` on fp32 state, `state_dict()` holding host tensors, workspace
size derived from `optimizer_memory_fraction` of the free device memory.
"""
from __future__ import annotations

import math

import torch

from .fused_adamw import _local


class DeviceWorkspace:
    """Two slots of `[3, chunk]` fp32 on the device plus the streams / events that pipeline them."""

    def __init__(self, device: torch.device, chunk_elems: int):
        self.device, self.chunk = device, int(chunk_elems)
        self.slots = [torch.empty(3, self.chunk, dtype=torch.float32, device=device) for _ in range(2)]
        self.copy_stream = torch.cuda.Stream(device=device)
        self.loaded = [torch.cuda.Event() for _ in range(2)]
        self.stored = [torch.cuda.Event() for _ in range(2)]
        self.computed = [torch.cuda.Event() for _ in range(2)]

    @staticmethod
    def size_for(device: torch.device, fraction: float, cap_elems: int = 256 << 20) -> int:
        free, _ = torch.cuda.mem_get_info(device)
        elems = int(free * fraction) // (2 * 3 * 4)
        return max(1 << 20, min(elems, cap_elems))


class AdamWSwap(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 memory_fraction: float = 0.8, chunk_elems: int | None = None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.memory_fraction, self.chunk_elems = memory_fraction, chunk_elems
        self._ws: DeviceWorkspace | None = None
        self._clip: torch.Tensor | None = None

    def set_clip_coef(self, coef: torch.Tensor | None) -> None:
        self._clip = coef

    # -- state -------------------------------------------------------------------------------------
    def _init_state(self, p: torch.Tensor) -> dict:
        st = self.state[p]
        if not st:
            lp = _local(p)
            pin = torch.cuda.is_available()
            st["step"] = 0
            st["master"] = torch.empty(lp.numel(), dtype=torch.float32, device="cpu", pin_memory=pin)
            st["master"].copy_(lp.detach().reshape(-1).float())
            st["exp_avg"] = torch.zeros(lp.numel(), dtype=torch.float32, device="cpu", pin_memory=pin)
            st["exp_avg_sq"] = torch.zeros(lp.numel(), dtype=torch.float32, device="cpu", pin_memory=pin)
        return st

    def _workspace(self, device: torch.device) -> DeviceWorkspace:
        if self._ws is None or self._ws.device != device:
            chunk = self.chunk_elems or DeviceWorkspace.size_for(device, self.memory_fraction)
            self._ws = DeviceWorkspace(device, chunk)
        return self._ws

    # -- update ------------------------------------------------------------------------------------
    @staticmethod
    def _update(w, m, v, g, lr, b1, b2, eps, wd, step):
        """In-place AdamW on fp32 views (device or host); `g` fp32."""
        w.mul_(1.0 - lr * wd)
        m.mul_(b1).add_(g, alpha=1.0 - b1)
        v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
        bc1, bc2 = 1.0 - b1 ** step, 1.0 - b2 ** step
        w.addcdiv_(m, (v.sqrt() / math.sqrt(bc2)).add_(eps), value=-lr / bc1)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        work = []                                            # (group, param, local param, local grad, state)
        for group in self.param_groups:
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                st = self._init_state(p)
                st["step"] += 1
                work.append((group, p, _local(p), _local(g), st))
        if not work:
            return loss
        cuda = [w for w in work if w[2].is_cuda]
        host = [w for w in work if not w[2].is_cuda]
        for group, p, lp, lg, st in host:
            g32 = lg.reshape(-1).float()
            if self._clip is not None:
                g32 = g32 * float(self._clip)
            b1, b2 = group["betas"]
            self._update(st["master"], st["exp_avg"], st["exp_avg_sq"], g32, group["lr"], b1, b2, group["eps"],
                         group["weight_decay"], st["step"])
            lp.copy_(st["master"].view_as(lp))
        if cuda:
            self._step_pipelined(cuda)
        return loss

    def _step_pipelined(self, work) -> None:
        dev = work[0][2].device
        ws = self._workspace(dev)
        main = torch.cuda.current_stream(dev)
        clip = self._clip.to(dev) if self._clip is not None else None
        # flatten the work list into (param entry, offset, length) pieces no longer than a chunk
        pieces = []
        for w in work:
            n = w[2].numel()
            for off in range(0, n, ws.chunk):
                pieces.append((w, off, min(ws.chunk, n - off)))

        def load(i):
            (group, p, lp, lg, st), off, n = pieces[i]
            s = i % 2
            with torch.cuda.stream(ws.copy_stream):
                ws.copy_stream.wait_event(ws.stored[s])      # the slot's previous contents have been written back
                for r, key in enumerate(("master", "exp_avg", "exp_avg_sq")):
                    ws.slots[s][r, :n].copy_(st[key][off:off + n], non_blocking=True)
                ws.loaded[s].record(ws.copy_stream)

        for s in range(2):
            ws.stored[s].record(main)
        load(0)
        for i, ((group, p, lp, lg, st), off, n) in enumerate(pieces):
            s = i % 2
            if i + 1 < len(pieces):
                load(i + 1)
            main.wait_event(ws.loaded[s])
            wv, mv, vv = ws.slots[s][0, :n], ws.slots[s][1, :n], ws.slots[s][2, :n]
            g32 = lg.reshape(-1)[off:off + n].float()
            if clip is not None:
                g32 = g32 * clip
            b1, b2 = group["betas"]
            self._update(wv, mv, vv, g32, group["lr"], b1, b2, group["eps"], group["weight_decay"], st["step"])
            lp.reshape(-1)[off:off + n].copy_(wv)
            ws.computed[s].record(main)
            with torch.cuda.stream(ws.copy_stream):
                ws.copy_stream.wait_event(ws.computed[s])
                for r, key in enumerate(("master", "exp_avg", "exp_avg_sq")):
                    st[key][off:off + n].copy_(ws.slots[s][r, :n], non_blocking=True)
                ws.stored[s].record(ws.copy_stream)
        main.wait_stream(ws.copy_stream)

    def zero_grad(self, set_to_none: bool = True):
        for group in self.param_groups:
            for p in group["params"]:
                if set_to_none:
                    p.grad = None
                elif p.grad is not None:
                    p.grad.zero_()
