"""QK-clip: keep attention logits bounded under Muon by rescaling query / key projection rows.

Attention modules with a `qk_clip_state` record the per-head maximum pre-softmax logit of every forward pass
(the attention kernels emit it at no extra cost).  Before the optimizer step the controller MAX-reduces the
per-head maxima over all ranks; after the step every head whose maximum exceeded `threshold` has its query rows
scaled by `gamma^alpha` and its key rows by `gamma^(1 - alpha)` with `gamma = threshold / max_logit`, applied to the
local row shards only.  For grouped-query attention the key scale of a KV head is the smallest over its query heads.
(engine/optimizers/qk_clip.py:40-130, engine/backends/fsdp2/qk_clip.py:53-274 and
models/modules/attention/qk_clip.py:7-54 of the reference.)

Multi-head latent attention (`MLAQKClipSpec`): a query head's rows are `[NoPE | RoPE]` in the final query projection
and a key/value head's rows are `[K NoPE | V]` in `kv_b_proj`; the RoPE key is shared by all heads and cannot be
scaled per head.  The whole correction of the RoPE part therefore goes to the query (`gamma^1`), the NoPE part is
split (`gamma^alpha` on the query rows, `gamma^(1 - alpha)` on the key rows) and the value rows are left alone."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn


class QKClipState:
    """Per-attention-module running maximum of the per-head logits since the last optimizer step."""

    def __init__(self, num_heads: int):
        self.num_heads = num_heads
        self.max_logits: torch.Tensor | None = None

    def update(self, max_logits: torch.Tensor) -> None:
        m = max_logits.detach().float()
        self.max_logits = m if self.max_logits is None else torch.maximum(self.max_logits, m)

    def pop(self, device) -> torch.Tensor:
        m = self.max_logits if self.max_logits is not None else torch.full((self.num_heads,), float("-inf"), device=device)
        self.max_logits = None
        return m


@dataclass
class QKClipSpec:
    module_fqn: str            # attention module
    q_weight: str              # parameter FQN holding the query rows (may be a fused projection)
    k_weight: str
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    q_row_offset: int = 0      # first query row inside `q_weight`
    k_row_offset: int = 0


@dataclass
class MLAQKClipSpec:
    module_fqn: str
    q_weight: str              # final query projection: `num_heads * (nope + rope)` rows
    kv_weight: str             # `kv_b_proj`: `num_heads * (nope + v)` rows
    num_heads: int
    qk_nope_head_dim: int
    qk_rope_head_dim: int
    v_head_dim: int

    def __post_init__(self) -> None:
        dims = (self.num_heads, self.qk_nope_head_dim, self.qk_rope_head_dim, self.v_head_dim)
        if any(type(d) is not int or d <= 0 for d in dims):
            raise ValueError("MLA QK-clip head counts and dimensions must be positive integers")
        if not self.q_weight or not self.kv_weight or self.q_weight == self.kv_weight:
            raise ValueError("MLA QK-clip needs two distinct projection parameters")

    @property
    def num_q_heads(self) -> int:
        return self.num_heads

    @property
    def projection_rows(self) -> dict[str, int]:
        return {self.q_weight: self.num_heads * (self.qk_nope_head_dim + self.qk_rope_head_dim),
                self.kv_weight: self.num_heads * (self.qk_nope_head_dim + self.v_head_dim)}


@dataclass
class QKClipPlan:
    specs: list = field(default_factory=list)

    @classmethod
    def from_model(cls, model: nn.Module) -> "QKClipPlan":
        specs: list = []
        for name, m in model.named_modules():
            if not hasattr(m, "qk_clip_state"):
                continue
            if hasattr(m, "qkv_proj"):
                specs.append(QKClipSpec(name, f"{name}.qkv_proj.weight", f"{name}.qkv_proj.weight", m.n_q, m.n_kv,
                                        m.head_dim, 0, m.n_q * m.head_dim))
            elif hasattr(m, "kv_b_proj") and hasattr(m, "d_nope"):
                q = "q_b_proj" if hasattr(m, "q_b_proj") else "q_proj"
                specs.append(MLAQKClipSpec(name, f"{name}.{q}.weight", f"{name}.kv_b_proj.weight", int(m.n_heads),
                                           int(m.d_nope), int(m.d_rope), int(m.d_v)))
        return cls(specs)


def _scale_rows(param: torch.Tensor, row0: int, rows_per_head: int, scales: torch.Tensor) -> None:
    """Multiply global rows `[row0 + h*rows_per_head, ...)` by `scales[h]`, touching only this rank's shard."""
    local = param._local_tensor if hasattr(param, "_local_tensor") else param
    lo = 0
    if hasattr(param, "_local_tensor"):
        n = param.device_mesh.size()
        chunk = -(-param.shape[0] // n)
        lo = param.device_mesh.get_local_rank() * chunk
    n_local = local.shape[0]
    if n_local == 0:
        return
    g = torch.arange(lo, lo + n_local, device=local.device)
    head = torch.div(g - row0, rows_per_head, rounding_mode="floor")
    inside = (g >= row0) & (head < scales.numel())
    s = torch.ones(n_local, device=local.device, dtype=torch.float32)
    s[inside] = scales.to(local.device)[head[inside]]
    local.mul_(s.to(local.dtype).unsqueeze(-1))


def _local_rows(param: torch.Tensor) -> tuple[torch.Tensor, int]:
    local = param._local_tensor if hasattr(param, "_local_tensor") else param
    lo = 0
    if hasattr(param, "_local_tensor"):
        n = param.device_mesh.size()
        lo = param.device_mesh.get_local_rank() * (-(-param.shape[0] // n))
    return local, lo


def _scale_rows_pow(param: torch.Tensor, rows_per_head: int, first_rows: int, first_exp: float, rest_exp: float,
                    gamma: torch.Tensor) -> None:
    """Row r of head h is multiplied by `gamma[h] ** first_exp` when `r % rows_per_head < first_rows`, else by
    `gamma[h] ** rest_exp`; every local row is mapped on its own, because a shard boundary may cut through a head."""
    local, lo = _local_rows(param)
    if local.shape[0] == 0:
        return
    g = torch.arange(lo, lo + local.shape[0], device=local.device)
    head = torch.div(g, rows_per_head, rounding_mode="floor")
    inside = head < gamma.numel()
    expo = torch.where(g.remainder(rows_per_head) < first_rows, first_exp, rest_exp).to(torch.float32)
    s = torch.ones(local.shape[0], device=local.device, dtype=torch.float32)
    s[inside] = gamma.to(local.device)[head[inside]].float().pow(expo[inside])
    local.mul_(s.to(local.dtype).unsqueeze(-1))


class QKClipController:
    def __init__(self, model: nn.Module, threshold: float = 100.0, alpha: float = 0.5, plan: QKClipPlan | None = None,
                 group=None):
        self.model, self.threshold, self.alpha, self.group = model, float(threshold), float(alpha), group
        for m in model.modules():
            if hasattr(m, "qk_clip_state") and m.qk_clip_state is None:
                m.qk_clip_state = QKClipState(m.n_q if hasattr(m, "n_q") else m.n_heads)
        self.plan = plan or QKClipPlan.from_model(model)
        self.params = dict(model.named_parameters())
        self.last_max: torch.Tensor | None = None

    def attach(self, optimizer) -> None:
        optimizer.register_step_post_hook(lambda *_: self.apply())

    @torch.no_grad()
    def apply(self) -> torch.Tensor | None:
        if not self.plan.specs:
            return None
        dev = next(self.model.parameters()).device
        mods = dict(self.model.named_modules())
        maxima = torch.cat([mods[s.module_fqn].qk_clip_state.pop(dev) for s in self.plan.specs])
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(maxima, op=dist.ReduceOp.MAX, group=self.group)
        self.last_max = maxima
        off = 0
        for s in self.plan.specs:
            m = maxima[off: off + s.num_q_heads]
            off += s.num_q_heads
            gamma = torch.where(m > self.threshold, self.threshold / m, torch.ones_like(m))
            if bool((gamma == 1).all()):
                continue
            if isinstance(s, MLAQKClipSpec):
                _scale_rows_pow(self.params[s.q_weight], s.qk_nope_head_dim + s.qk_rope_head_dim, s.qk_nope_head_dim,
                                self.alpha, 1.0, gamma)
                _scale_rows_pow(self.params[s.kv_weight], s.qk_nope_head_dim + s.v_head_dim, s.qk_nope_head_dim,
                                1.0 - self.alpha, 0.0, gamma)
                continue
            q_scale = gamma.pow(self.alpha)
            k_scale = gamma.pow(1 - self.alpha).view(s.num_kv_heads, -1).amin(dim=1)
            _scale_rows(self.params[s.q_weight], s.q_row_offset, s.head_dim, q_scale)
            _scale_rows(self.params[s.k_weight], s.k_row_offset, s.head_dim, k_scale)
        return maxima
