"""LoRA / DoRA adapters, including adapters for fused expert tensors.

The model blocks read `module.weight` and feed it to fused kernels, so an adapted layer exposes the *effective*
weight `W + (alpha / r) * B @ A` (DoRA: column-normalised and rescaled by a learned magnitude) through the same
attribute: the low-rank factors are the only trainable tensors, gradients reach them through the merge, and the
hot kernels stay unchanged.  Fused expert tensors get one pair of factors per expert (`GroupedLoRA`), merged with a
batched matmul.  Parameter names follow the PEFT convention (`base_layer.weight`, `lora_A.<adapter>.weight`,
`lora_B.<adapter>.weight`, `lora_magnitude_vector.<adapter>.weight`) so adapter checkpoints interoperate
(engine/peft/lora.py:54-739 and engine/peft/weights.py:78-350 of the reference).
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Any

import torch
import torch.nn as nn

from ...utils.fqn import match_fqn


@dataclass
class LoraConfig:
    r: int = 8
    lora_alpha: float = 16.0
    lora_dropout: float = 0.0
    target_modules: list[str] | str = field(default_factory=lambda: ["all-linear"])
    use_dora: bool = False
    use_rslora: bool = False
    init_lora_weights: bool | str = True
    adapter_name: str = "default"
    target_experts: bool = True
    peft_type: str = "LORA"
    modules_to_save: list[str] | None = None

    @property
    def scaling(self) -> float:
        return self.lora_alpha / math.sqrt(self.r) if self.use_rslora else self.lora_alpha / self.r

    def to_dict(self) -> dict[str, Any]:
        d = asdict(self)
        if isinstance(d["target_modules"], (set, tuple)):
            d["target_modules"] = sorted(d["target_modules"])
        return d

    @classmethod
    def from_any(cls, cfg) -> "LoraConfig":
        if isinstance(cfg, cls):
            return cfg
        if isinstance(cfg, dict):
            known = {f for f in cls.__dataclass_fields__}
            return cls(**{k: v for k, v in cfg.items() if k in known})
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: getattr(cfg, k) for k in known if hasattr(cfg, k)})


def init_lora_tensor(t: torch.Tensor, kind: str, how: bool | str = True) -> None:
    """A: Kaiming-uniform (or gaussian with std 1/r), B: zeros, so the adapter starts as a no-op."""
    with torch.no_grad():
        if kind == "B" or how is False:
            t.zero_()
        elif how == "gaussian":
            t.normal_(0.0, 1.0 / t.shape[-2 if t.dim() == 3 else 0])
        else:
            nn.init.kaiming_uniform_(t.view(-1, t.shape[-1]), a=math.sqrt(5))


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Linear, cfg: LoraConfig):
        super().__init__()
        self.base_layer = base
        base.weight.requires_grad_(False)
        if base.bias is not None:
            base.bias.requires_grad_(False)
        self.cfg, name = cfg, cfg.adapter_name
        dt, dev = torch.float32 if base.weight.dtype == torch.float32 else base.weight.dtype, base.weight.device
        self.lora_A = nn.ModuleDict({name: nn.Linear(base.in_features, cfg.r, bias=False, dtype=dt, device=dev)})
        self.lora_B = nn.ModuleDict({name: nn.Linear(cfg.r, base.out_features, bias=False, dtype=dt, device=dev)})
        if not base.weight.is_meta:
            init_lora_tensor(self.lora_A[name].weight, "A", cfg.init_lora_weights)
            init_lora_tensor(self.lora_B[name].weight, "B")
        self.lora_magnitude_vector = None
        if cfg.use_dora:
            self.lora_magnitude_vector = nn.ModuleDict({name: _Magnitude(base.out_features, dt, dev)})
            if not base.weight.is_meta:
                self.reset_dora()
        self.in_features, self.out_features = base.in_features, base.out_features
        self.dropout = nn.Dropout(cfg.lora_dropout) if cfg.lora_dropout > 0 else None

    def reset_dora(self) -> None:
        with torch.no_grad():
            self.lora_magnitude_vector[self.cfg.adapter_name].weight.copy_(compute_dora_magnitude(self.delta_free_weight()))

    def delta_free_weight(self) -> torch.Tensor:
        w = self.base_layer.weight
        return (w.full_tensor() if hasattr(w, "full_tensor") else w).detach()

    def delta(self) -> torch.Tensor:
        n = self.cfg.adapter_name
        return (self.lora_B[n].weight @ self.lora_A[n].weight) * self.cfg.scaling

    @property
    def weight(self) -> torch.Tensor:
        w = self.base_layer.weight
        eff = w + self.delta().to(w.dtype)
        if self.lora_magnitude_vector is not None:
            mag = self.lora_magnitude_vector[self.cfg.adapter_name].weight
            norm = eff.detach().float().norm(dim=1, keepdim=True).clamp_min(1e-12)
            eff = eff * (mag.view(-1, 1).float() / norm).to(eff.dtype)
        return eff

    @property
    def bias(self):
        return self.base_layer.bias

    def forward(self, x):
        if self.dropout is not None and self.training:
            n = self.cfg.adapter_name
            base = nn.functional.linear(x, self.base_layer.weight, self.base_layer.bias)
            return base + self.lora_B[n](self.lora_A[n](self.dropout(x))) * self.cfg.scaling
        return nn.functional.linear(x, self.weight, self.bias)


class _Magnitude(nn.Module):
    def __init__(self, n, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n, dtype=dtype, device=device))


def compute_dora_magnitude(weight: torch.Tensor) -> torch.Tensor:
    """Per-output-row L2 norm of the (merged) weight: DoRA's initial magnitude."""
    return weight.float().norm(dim=1)


class GroupedLoRA(nn.Module):
    """Per-expert low-rank factors for one fused expert tensor `[E*rows, cols]`: A `[E, rows, r]`, B `[E, r, cols]`."""

    def __init__(self, experts: int, rows: int, cols: int, cfg: LoraConfig, dtype, device):
        super().__init__()
        self.cfg, self.E, self.rows, self.cols = cfg, experts, rows, cols
        self.lora_A = nn.Parameter(torch.empty(experts, rows, cfg.r, dtype=dtype, device=device))
        self.lora_B = nn.Parameter(torch.empty(experts, cfg.r, cols, dtype=dtype, device=device))
        if not self.lora_A.is_meta:
            init_lora_tensor(self.lora_A, "A", cfg.init_lora_weights)
            init_lora_tensor(self.lora_B, "B")

    def delta(self) -> torch.Tensor:
        return torch.bmm(self.lora_A, self.lora_B).view(self.E * self.rows, self.cols) * self.cfg.scaling


class GroupedMLPLoRA(nn.Module):
    """Wraps a `GroupedMLP`: frozen fused expert weights plus `GroupedLoRA` factors for weight1 and weight2."""

    def __init__(self, base, cfg: LoraConfig):
        super().__init__()
        self.base_layer = base
        base.weight1.requires_grad_(False)
        base.weight2.requires_grad_(False)
        E, H, Fh = base.num_local_experts, base.config.hidden_size, base.config.moe_ffn_hidden_size
        dt, dev = base.weight1.dtype, base.weight1.device
        self.lora1 = GroupedLoRA(E, H, 2 * Fh, cfg, dt, dev)
        self.lora2 = GroupedLoRA(E, Fh, H, cfg, dt, dev)
        self.num_local_experts, self.config = E, base.config

    @property
    def weight1(self):
        return self.base_layer.weight1 + self.lora1.delta().to(self.base_layer.weight1.dtype)

    @property
    def weight2(self):
        return self.base_layer.weight2 + self.lora2.delta().to(self.base_layer.weight2.dtype)

    def views(self):
        E, H, Fh = self.num_local_experts, self.config.hidden_size, self.config.moe_ffn_hidden_size
        return self.weight1.view(E, H, 2 * Fh), self.weight2.view(E, Fh, H)

    def forward(self, perm, tokens_per_expert=None):
        from ...ops import ops

        w1, w2 = self.views()
        return ops.moe_experts(perm, w1, w2, tokens_per_expert)

    def get_muon_parameter_specs(self):
        return {}


_DEFAULT_SKIP = ("lm_head", "embed_tokens", "router")


def expand_all_linear_targets(model: nn.Module, skip=_DEFAULT_SKIP) -> list[str]:
    """FQNs of every `nn.Linear` except output heads, embeddings and routers (`target_modules="all-linear"`)."""
    return [n for n, m in model.named_modules() if isinstance(m, nn.Linear) and not any(s in n.split(".") for s in skip)]


def _matches(name: str, targets) -> bool:
    leaf = name.rsplit(".", 1)[-1]
    for t in targets:
        if t == leaf or name == t or name.endswith("." + t) or match_fqn(t, name):
            return True
    return False


def apply_peft(model: nn.Module, peft_config) -> nn.Module:
    """Freeze the model, wrap the targeted linears (and expert containers) and record the config on the model."""
    cfg = LoraConfig.from_any(peft_config)
    targets = cfg.target_modules
    if isinstance(targets, str):
        targets = [targets]
    for p in model.parameters():
        p.requires_grad_(False)
    names = expand_all_linear_targets(model) if ("all-linear" in targets) else \
        [n for n, m in model.named_modules() if isinstance(m, nn.Linear) and _matches(n, targets)]
    for n in names:
        parent_name, _, child = n.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, child, LoRALinear(getattr(parent, child), cfg))
    if cfg.target_experts:
        from ...models.modules.moe import GroupedMLP

        for n, m in list(model.named_modules()):
            if isinstance(m, GroupedMLP):
                parent_name, _, child = n.rpartition(".")
                setattr(model.get_submodule(parent_name), child, GroupedMLPLoRA(m, cfg))
    for n, m in model.named_modules():
        if cfg.modules_to_save and _matches(n, cfg.modules_to_save):
            for p in m.parameters():
                p.requires_grad_(True)
    cfgs = dict(getattr(model, "peft_config", {}) or {})
    cfgs[cfg.adapter_name] = cfg
    model.peft_config = cfgs
    return model


_ADAPTER_SEGMENTS = ("lora_A", "lora_B", "lora_magnitude_vector", "lora1", "lora2")


def strip_peft_name(name: str) -> str:
    """Parameter FQN of a wrapped model -> the name the base model uses (`x.base_layer.weight` -> `x.weight`)."""
    return name.replace(".base_layer.", ".")


def is_adapter_param(name: str) -> bool:
    parts = name.split(".")
    return any(seg in parts for seg in _ADAPTER_SEGMENTS)


def _full(t: torch.Tensor) -> torch.Tensor:
    return t.full_tensor() if hasattr(t, "full_tensor") else t


def lora_merge_functions(model: nn.Module) -> dict[str, Any]:
    """{FQN of a wrapped base parameter: fn(full base tensor) -> merged tensor} for export.  The functions gather the
    adapter factors (`full_tensor()` on sharded ones), so every rank has to call them in the same order."""
    out: dict[str, Any] = {}
    for n, m in model.named_modules():
        if isinstance(m, LoRALinear):
            def merge(w, m=m):
                name = m.cfg.adapter_name
                a, b = _full(m.lora_A[name].weight).float(), _full(m.lora_B[name].weight).float()
                eff = w.float() + (b.to(w.device) @ a.to(w.device)) * m.cfg.scaling
                if m.lora_magnitude_vector is not None:
                    mag = _full(m.lora_magnitude_vector[name].weight).float().to(w.device)
                    eff = eff * (mag.view(-1, 1) / eff.norm(dim=1, keepdim=True).clamp_min(1e-12))
                return eff
            out[f"{n}.base_layer.weight"] = merge
        elif isinstance(m, GroupedMLPLoRA):
            for key, lo in (("weight1", m.lora1), ("weight2", m.lora2)):
                def merge(w, lo=lo):
                    a, b = _full(lo.lora_A).float().to(w.device), _full(lo.lora_B).float().to(w.device)
                    return w.float() + torch.bmm(a, b).view(-1, lo.cols) * lo.cfg.scaling
                out[f"{n}.base_layer.{key}"] = merge
    return out


def build_lora_delta_map(model: nn.Module) -> dict[str, torch.Tensor]:
    """{base parameter FQN (without wrapper segments): merged delta} for export-time merging."""
    out: dict[str, torch.Tensor] = {}
    for n, m in model.named_modules():
        if isinstance(m, LoRALinear):
            with torch.no_grad():
                out[f"{n}.weight"] = (m.weight - m.base_layer.weight).detach()
        elif isinstance(m, GroupedMLPLoRA):
            with torch.no_grad():
                out[f"{n}.weight1"] = m.lora1.delta().detach()
                out[f"{n}.weight2"] = m.lora2.delta().detach()
    return out


def apply_lora_delta(model: nn.Module) -> None:
    """Attach `merged_lora_delta` so that the Hugging Face exporter writes merged weights under base names."""
    model.merged_lora_delta = {k.replace(".base_layer", ""): v for k, v in build_lora_delta_map(model).items()}
