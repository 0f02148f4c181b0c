"""AdamW on fp32 master state with one multi-tensor CUDA launch per parameter group.

Two storage schemes are handled by the same optimizer:
  * fp32 parameters (FSDP2 shards: DTensor locals): updated in place;
  * bf16 parameters (units that are not sharded, e.g. experts when the expert-data-parallel mesh has one
    rank): the optimizer owns an fp32 master copy and the kernel writes the bf16 parameter as a shadow
    in the same pass, so there is no per-step cast traffic.
The gradient-clipping coefficient is a device scalar applied inside the update kernel (no separate
"scale all gradients" pass and no host synchronisation); a non-finite norm skips the update.
On CPU (tests, oracle) the same arithmetic runs in PyTorch.  Math follows torch's fused AdamW, which the
reference calls on the shards (engine/backends/fsdp2/optimizers/adamw.py:226-251).

Overlap with the next step (`enable_overlap`, opt-in).  The update is bandwidth-bound (28 B per parameter) and the
forward pass that follows it is tensor-core-bound; in practice the persistent GEMMs leave the update only the gaps
between kernels (a 1.4 % shorter step at 1 GPU), which is why the backend does not switch it on by default.
Parameters handed over in buckets (one per decoder
layer, in forward order) are updated on a side stream, bucket after bucket, each followed by an event; the forward
pre-hook of layer i makes the compute stream wait for event i only, so layer i of the next step starts as soon as its
own weights are new while the update of the later layers is still running.  Only parameters whose gradient is a plain
`.grad` tensor take part (its memory is kept for the side stream with `record_stream`); `synchronize()` joins the
streams for anything that reads the weights outside a forward pass (checkpoints, evaluation of raw tensors).
"""
from __future__ import annotations

import weakref
from typing import Any

import torch

from ... import kernels as K


def _local(t: torch.Tensor) -> torch.Tensor:
    return t._local_tensor if hasattr(t, "_local_tensor") else t


_OVERLAPPING: "weakref.WeakSet[FusedAdamW]" = weakref.WeakSet()


def join_update_streams() -> None:
    """Order the current stream after every side-stream update in flight (call before reading weights outside a
    forward pass: checkpoints, exports, weight statistics)."""
    for opt in list(_OVERLAPPING):
        opt.synchronize()


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 **_ignored: Any):
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self._clip_coef: torch.Tensor | None = None
        # constant folded into every gradient read by `grad_sq_sum()` and by the next `step()` (then reset to 1):
        # the backend uses it for the 1/ep scaling of expert gradients instead of a pass of its own over them
        self.grad_prescale: float = 1.0
        self._plans: dict[Any, tuple[tuple, Any]] = {}
        # the clip coefficient of the last CUDA step, copied to pinned host memory without blocking: a step the kernel
        # skipped (non-finite coefficient) is taken back out of the step counters at the start of the next `step()`
        self._clip_host: torch.Tensor | None = None
        self._clip_event = None
        self._clip_pending: list[dict] | None = None
        # overlap of the update with the next forward pass
        self._buckets: list[list[torch.Tensor]] = []
        self._bucket_of: dict[int, int] = {}
        self._bucket_events: list[Any] = []
        self._side_stream = None

    # -- clipping ------------------------------------------------------------------------------------
    def set_clip_coef(self, coef: torch.Tensor | None) -> None:
        """Device scalar multiplied into every gradient by the next `step()` (then cleared)."""
        self._clip_coef = coef

    # -- state ---------------------------------------------------------------------------------------
    def _init_state(self, p: torch.Tensor) -> dict:
        st = self.state[p]
        if "exp_avg" not in st:
            lp = _local(p)
            st["step"] = torch.zeros((), dtype=torch.float32)
            st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
            if lp.dtype != torch.float32:
                st["master"] = _local(p).detach().float().clone()
        return st

    def state_dict(self):
        if self._bucket_events and torch.cuda.is_available():
            self.synchronize()
        return super().state_dict()

    def load_state_dict(self, state_dict):
        """State tensors are replaced: the cached pointer tables of the multi-tensor kernels are rebuilt."""
        if self._bucket_events and torch.cuda.is_available():
            self.synchronize()
        self._plans.clear()
        self._clip_pending = None
        return super().load_state_dict(state_dict)

    def add_param_group(self, param_group):
        if hasattr(self, "_plans"):
            self._plans.clear()
        return super().add_param_group(param_group)

    # -- overlap ---------------------------------------------------------------------------------------
    def enable_overlap(self, buckets: list[list[torch.Tensor]]) -> None:
        """`buckets[i]`: parameters of this optimizer that the forward pass first reads in its i-th stage (a decoder
        layer).  They are updated on a side stream in this order; `wait_bucket(i)` orders the caller's stream after
        bucket i.  Parameters outside every bucket are updated on the caller's stream as before."""
        mine = {id(p) for g in self.param_groups for p in g["params"]}
        self._buckets = [[p for p in b if id(p) in mine] for b in buckets]
        self._bucket_of = {id(p): i for i, b in enumerate(self._buckets) for p in b}
        self._bucket_events = [None] * len(self._buckets)
        self._plans.clear()
        _OVERLAPPING.add(self)

    def wait_bucket(self, i: int) -> None:
        ev = self._bucket_events[i] if i < len(self._bucket_events) else None
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def synchronize(self) -> None:
        """Order the current stream after every update in flight on the side stream."""
        for i in range(len(self._bucket_events)):
            self.wait_bucket(i)

    def _overlappable(self, p: torch.Tensor) -> bool:
        return (id(p) in self._bucket_of and getattr(p, "main_grad", None) is None and p.grad is not None
                and _local(p).is_cuda)

    def _settle_skipped_step(self) -> None:
        """torch's fused AdamW does not advance `step` when `found_inf` is set; the kernel here skips the same way
        on a non-finite clip coefficient, which the host learns one step later (no synchronisation inside a step)."""
        pending, self._clip_pending = self._clip_pending, None
        if pending is None:
            return
        self._clip_event.synchronize()
        v = float(self._clip_host[0])
        if v != v or v in (float("inf"), float("-inf")):
            for st in pending:
                st["step"] -= 1

    def _note_clip(self, clip: torch.Tensor | None, states: list[dict]) -> None:
        if clip is None or not clip.is_cuda:
            return
        if self._clip_host is None:
            self._clip_host = torch.empty(1, dtype=torch.float32, pin_memory=True)
            self._clip_event = torch.cuda.Event()
        self._clip_host.copy_(clip.detach().reshape(1).float(), non_blocking=True)
        self._clip_event.record()
        self._clip_pending = (self._clip_pending or []) + states

    def grad_of(self, p: torch.Tensor) -> torch.Tensor | None:
        g = getattr(p, "main_grad", None)
        return g if g is not None else p.grad

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        clip, self._clip_coef = self._clip_coef, None
        prescale, self.grad_prescale = self.grad_prescale, 1.0
        self._settle_skipped_step()
        for gi, group in enumerate(self.param_groups):
            ps = [p for p in group["params"] if self.grad_of(p) is not None]
            if not ps:
                continue
            states = [self._init_state(p) for p in ps]
            for st in states:
                st["step"] += 1
            step = int(states[0]["step"].item())
            lp0 = _local(ps[0])
            if lp0.is_cuda and K.available():
                side = [(p, st) for p, st in zip(ps, states) if self._overlappable(p)] if self._buckets else []
                if side:
                    taken = {id(p) for p, _ in side}
                    rest = [(p, st) for p, st in zip(ps, states) if id(p) not in taken]
                    if rest:
                        self._step_cuda(("rest", gi), group, [p for p, _ in rest], [st for _, st in rest], step, clip, prescale)
                    self._step_side(gi, group, side, step, clip, prescale)
                else:
                    self._step_cuda(gi, group, ps, states, step, clip, prescale)
                self._note_clip(clip, states)
            else:
                self._step_torch(group, ps, states, step, clip, prescale)
        return loss

    def _step_side(self, gi, group, side, step, clip, prescale) -> None:
        """Bucket after bucket on the side stream, an event after each."""
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream()
        S, main = self._side_stream, torch.cuda.current_stream()
        S.wait_stream(main)                       # gradients and the clip coefficient are products of the caller's stream
        by_bucket: dict[int, list] = {}
        for p, st in side:
            by_bucket.setdefault(self._bucket_of[id(p)], []).append((p, st))
        if clip is not None:
            clip.record_stream(S)
        with torch.cuda.stream(S):
            for b in sorted(by_bucket):
                ps = [p for p, _ in by_bucket[b]]
                for p in ps:
                    _local(p.grad).record_stream(S)      # `zero_grad(set_to_none)` frees it on the caller's stream
                self._step_cuda((gi, b), group, ps, [st for _, st in by_bucket[b]], step, clip, prescale)
                ev = torch.cuda.Event()
                ev.record(S)
                self._bucket_events[b] = ev

    @torch.no_grad()
    def grad_sq_sum(self) -> torch.Tensor | None:
        """Sum of squared gradients over every parameter of this optimizer as a device scalar, computed by the
        multi-tensor kernel on the same tables the update uses (CUDA only; `None` elsewhere)."""
        total = None
        for gi, group in enumerate(self.param_groups):
            ps = [p for p in group["params"] if self.grad_of(p) is not None]
            if not ps:
                continue
            if not (_local(ps[0]).is_cuda and K.available()):
                return None
            states = [self._init_state(p) for p in ps]
            plan = self._plan_for(gi, ps, states)
            s = K.grad_sqnorm_partials(plan, self.grad_prescale).sum()
            total = s if total is None else total + s
        return total

    def _plan_for(self, gi, ps, states):
        key = tuple(id(p) for p in ps) + tuple(_local(st["exp_avg"]).data_ptr() for st in states)
        cached = self._plans.get(gi)
        if cached is None or cached[0] != key:
            masters, shadows = [], []
            for p, st in zip(ps, states):
                lp = _local(p)
                if "master" in st:
                    masters.append(st["master"]); shadows.append(lp)
                else:
                    masters.append(lp); shadows.append(None)
            plan = K.MultiTensorPlan(masters, [_local(s["exp_avg"]) for s in states],
                                     [_local(s["exp_avg_sq"]) for s in states], shadows)
            self._plans[gi] = cached = (key, plan)
        plan = cached[1]
        grads = []
        for p in ps:
            g = _local(self.grad_of(p))
            grads.append(g if g.is_contiguous() else g.contiguous())
        gkey = tuple(g.data_ptr() for g in grads)
        if getattr(plan, "_gkey", None) != gkey:
            plan.refresh_grads(grads)
            plan._gkey = gkey
            plan._grads = grads  # keep contiguous copies alive until the kernels have consumed them
        return plan

    def _step_cuda(self, gi, group, ps, states, step, clip, prescale=1.0):
        plan = self._plan_for(gi, ps, states)
        b1, b2 = group["betas"]
        K.adamw_step(plan, lr=group["lr"], beta1=b1, beta2=b2, eps=group["eps"], weight_decay=group["weight_decay"],
                     step=step, clip=clip, grad_prescale=prescale)
        plan._gkey = None

    def _step_torch(self, group, ps, states, step, clip, prescale=1.0):
        b1, b2 = group["betas"]
        lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        coef = (float(clip) if clip is not None else 1.0) * prescale
        if coef != coef or coef in (float("inf"), float("-inf")):
            for st in states:
                st["step"] -= 1        # a skipped update does not advance the bias correction
            return
        for p, st in zip(ps, states):
            lp = _local(p)
            g = _local(self.grad_of(p)).float() * coef
            w = st.get("master", lp)
            m, v = _local(st["exp_avg"]), _local(st["exp_avg_sq"])
            w.mul_(1 - lr * wd)
            m.lerp_(g, 1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            denom = (v.sqrt() / (bc2 ** 0.5)).add_(eps)
            w.addcdiv_(m, denom, value=-lr / bc1)
            if w is not lp:
                lp.copy_(w)

    def zero_grad(self, set_to_none: bool = True):
        super().zero_grad(set_to_none=set_to_none)
        for group in self.param_groups:
            for p in group["params"]:
                mg = getattr(p, "main_grad", None)
                if mg is not None and getattr(mg, "_tt_flat_owner", None) is None:
                    mg.zero_()      # views of a flat buffer are cleared by its owner, once, after the step
