"""Typed engine configuration and its four-layer merge.

Precedence (lowest to highest), as in the reference (engine/config.py:1012-1100, README "configuration"):
built-in / adapter defaults  <  `TORCH_TURBO_*` environment  <  `--tt_config` YAML/JSON file (root key
`engine_config`, unknown keys rejected)  <  explicit `--tt_*` flags.  The reference merges with OmegaConf;
this build uses a small recursive dict merge plus a generic "dataclass from mapping" builder, so the only
dependency is PyYAML.
"""
from __future__ import annotations

import dataclasses
import json
import math
import os
import typing
from dataclasses import dataclass, field, fields, is_dataclass
from enum import Enum
from typing import Any, Iterable, Literal, Optional

from ..ops.base import OpPolicy
from ..parallel import FSDPParallelPlan


def string_to_bool(v: Any) -> bool:
    if isinstance(v, bool):
        return v
    if isinstance(v, (int, float)):
        return bool(v)
    s = str(v).strip().lower()
    if s in {"1", "true", "yes", "y", "on", "t"}:
        return True
    if s in {"0", "false", "no", "n", "off", "f", ""}:
        return False
    raise ValueError(f"cannot interpret {v!r} as a boolean")


class DistributedBackend(str, Enum):
    FSDP2 = "fsdp2"


class ParameterGroup(str, Enum):
    VISION_TOWER = "vision_tower"
    MULTI_MODAL_PROJECTOR = "multi_modal_projector"
    LANGUAGE_MODEL = "language_model"


class MixedPrecisionPolicy(str, Enum):
    """bf16 compute with fp32 master weights and fp32 gradient reduction, or pure fp32.  fp16 and fp8
    training are rejected (quantised checkpoints are dequantised offline instead)."""

    BF16 = "bf16"
    FP32 = "fp32"


def parse_mixed_precision(v: Any) -> MixedPrecisionPolicy:
    if isinstance(v, MixedPrecisionPolicy):
        return v
    s = str(v).strip().lower()
    if s in {"fp16", "float16", "half", "fp8", "float8"}:
        raise ValueError(f"mixed_precision={v!r} is not supported: training runs in bf16 or fp32")
    aliases = {"bf16": "bf16", "bfloat16": "bf16", "fp32": "fp32", "float32": "fp32", "no": "fp32"}
    if s not in aliases:
        raise ValueError(f"unknown mixed precision policy {v!r}")
    return MixedPrecisionPolicy(aliases[s])


class ShardingStrategy(str, Enum):
    FULL_SHARD = "full_shard"


class FSDPPrefetchStrategy(str, Enum):
    NATIVE = "native"            # FSDP2's implicit next-unit prefetch only
    AUTO = "auto"                # MoE-aware when the model has expert units, else native
    LAYER = "layer"              # explicit chain over decoder layers
    EXPERT_WITH_LAYER = "expert_with_layer"      # experts ride with the layer that owns them
    EXPERT_LOOKAHEAD = "expert_lookahead"        # separate rolling chain over expert units


class FSDPPrefetchDirection(str, Enum):
    FORWARD = "forward"
    FORWARD_BACKWARD = "forward_backward"


class CPUOffloadMode(str, Enum):
    FULL = "full"
    OPTIMIZER = "optimizer"


# --------------------------------------------------------------------------------------------------
# dataclasses
# --------------------------------------------------------------------------------------------------
@dataclass
class OpsConfig:
    policy: OpPolicy = OpPolicy.AUTO
    overrides: dict[str, str] = field(default_factory=dict)

    def __post_init__(self) -> None:
        self.policy = OpPolicy(self.policy)
        if not isinstance(self.overrides, dict) or any(
                not isinstance(k, str) or not isinstance(v, str) for k, v in self.overrides.items()):
            raise TypeError("ops.overrides must map op names to implementation names")
        self.overrides = dict(self.overrides)


@dataclass
class ActivationCheckpointingConfig:
    enabled: bool = True
    use_reentrant: bool = False

    def __post_init__(self) -> None:
        self.enabled = string_to_bool(self.enabled)
        self.use_reentrant = string_to_bool(self.use_reentrant)


@dataclass
class CommConfig:
    overlap_comm_compute: bool = False
    bucket_cap_mb: float = 25.0
    reduce_dtype: MixedPrecisionPolicy | None = None
    fused_collectives: bool = True
    """Use the in-kernel NVLink paths (peer stores / loads from inside the compute kernels) where one
    exists; `False` keeps every collective on NCCL (the measured baseline)."""


@dataclass
class OptimizerBucketPolicy:
    strategy: str = "parameter"
    bucket_cap_mb: float | None = None

    def __post_init__(self) -> None:
        self.strategy = str(self.strategy).lower()
        if self.strategy not in {"parameter", "size", "single"}:
            raise ValueError("optimizer bucket strategy must be parameter, size, or single")
        if self.bucket_cap_mb is not None:
            self.bucket_cap_mb = float(self.bucket_cap_mb)
            if self.bucket_cap_mb <= 0:
                raise ValueError("optimizer bucket_cap_mb must be positive")


@dataclass
class QKClipConfig:
    threshold: float = 100.0
    alpha: float = 0.5

    def __post_init__(self) -> None:
        self.threshold, self.alpha = float(self.threshold), float(self.alpha)
        if not math.isfinite(self.threshold) or self.threshold <= 0:
            raise ValueError("QK clip threshold must be finite and positive")
        if not 0.0 <= self.alpha <= 1.0:
            raise ValueError("QK clip alpha must be in [0, 1]")


def _ns_coefficients(v):
    v = tuple(v)
    if v and isinstance(v[0], (list, tuple)):
        out = tuple(tuple(float(c) for c in t) for t in v)
        if any(len(t) != 3 for t in out):
            raise ValueError("Muon ns_coefficients entries must contain three values")
        return out
    out = tuple(float(c) for c in v)
    if len(out) != 3:
        raise ValueError("Muon ns_coefficients must contain three values")
    return out


@dataclass
class MuonOptimizerConfig:
    lr: float | None = None
    weight_decay: float | None = None
    momentum: float = 0.95
    nesterov: bool = True
    ns_coefficients: Any = (3.4445, -4.7750, 2.0315)
    eps: float = 1e-7
    ns_steps: int = 5
    adjust_lr_fn: str | None = "match_rms_adamw"
    overlap_comm_compute: bool = True
    adamw_lr: float | None = None
    adamw_betas: tuple[float, float] = (0.9, 0.999)
    adamw_eps: float = 1e-8
    adamw_fused: bool | None = None
    bucket: OptimizerBucketPolicy = field(default_factory=OptimizerBucketPolicy)
    qk_clip: QKClipConfig | None = None

    def __post_init__(self) -> None:
        for n in ("lr", "adamw_lr", "weight_decay"):
            v = getattr(self, n)
            if v is not None:
                v = float(v)
                if v < 0:
                    raise ValueError(f"Muon {n} must be non-negative")
                setattr(self, n, v)
        self.momentum = float(self.momentum)
        if self.momentum < 0:
            raise ValueError("Muon momentum must be non-negative")
        self.nesterov = string_to_bool(self.nesterov)
        self.ns_coefficients = _ns_coefficients(self.ns_coefficients)
        self.eps, self.ns_steps = float(self.eps), int(self.ns_steps)
        if not 0 <= self.ns_steps < 100:
            raise ValueError("Muon ns_steps must be in [0, 100)")
        if isinstance(self.ns_coefficients[0], tuple) and len(self.ns_coefficients) != self.ns_steps:
            raise ValueError("Muon ns_coefficients must provide one triple per ns_step")
        self.overlap_comm_compute = string_to_bool(self.overlap_comm_compute)
        self.adamw_betas = tuple(float(b) for b in self.adamw_betas)
        if len(self.adamw_betas) != 2 or not all(0 <= b < 1 for b in self.adamw_betas):
            raise ValueError("Muon AdamW betas must contain two values in [0, 1)")
        self.adamw_eps = float(self.adamw_eps)
        if self.adjust_lr_fn not in {None, "original", "match_rms_adamw", "spectral_unclamped"}:
            raise ValueError(f"unsupported Muon adjust_lr_fn {self.adjust_lr_fn!r}")
        if isinstance(self.bucket, dict):
            self.bucket = OptimizerBucketPolicy(**self.bucket)
        elif self.bucket is None:
            self.bucket = OptimizerBucketPolicy()
        if isinstance(self.qk_clip, dict):
            self.qk_clip = QKClipConfig(**self.qk_clip)


@dataclass
class OptimizerConfig:
    name: str | None = None
    muon: MuonOptimizerConfig | None = None

    def __post_init__(self) -> None:
        if self.name is not None:
            self.name = str(self.name).strip().lower()
        if self.name == "muon":
            if self.muon is None:
                self.muon = MuonOptimizerConfig()
            elif isinstance(self.muon, dict):
                self.muon = MuonOptimizerConfig(**self.muon)
        elif self.name is not None:
            raise ValueError(f"unsupported engine-managed optimizer {self.name!r}; supported: 'muon'")


@dataclass
class CheckpointConfig:
    hf_export: str = "every"

    def __post_init__(self) -> None:
        if self.hf_export not in ("final", "every"):
            raise ValueError(f"checkpoint.hf_export must be 'final' or 'every', got {self.hf_export!r}")


@dataclass
class MTPConfig:
    enabled: bool = False
    loss_scaling_factor: float = 0.1
    log_loss: bool = False

    def __post_init__(self) -> None:
        self.enabled = string_to_bool(self.enabled)
        self.log_loss = string_to_bool(self.log_loss)
        self.loss_scaling_factor = float(self.loss_scaling_factor)
        if self.loss_scaling_factor < 0:
            raise ValueError("MTP loss_scaling_factor must be non-negative")


@dataclass
class DSparkTrainingConfig:
    enabled: bool = True
    loss_scaling_factor: float = 0.1
    num_anchors: int = 512
    loss_decay_gamma: float = 4.0
    ce_loss_alpha: float = 0.1
    l1_loss_alpha: float = 0.9
    confidence_loss_alpha: float = 1.0

    def __post_init__(self) -> None:
        self.enabled = string_to_bool(self.enabled)
        for n in ("loss_scaling_factor", "loss_decay_gamma", "ce_loss_alpha", "l1_loss_alpha", "confidence_loss_alpha"):
            v = float(getattr(self, n))
            if v < 0:
                raise ValueError(f"dspark {n} must be non-negative, got {v}")
            setattr(self, n, v)
        self.num_anchors = int(self.num_anchors)
        if self.num_anchors <= 0:
            raise ValueError("dspark num_anchors must be positive")


@dataclass
class LossChunkConfig:
    enabled: bool = False
    chunk_size: int = 1024

    def __post_init__(self) -> None:
        self.enabled = string_to_bool(self.enabled)
        self.chunk_size = int(self.chunk_size)
        if self.chunk_size <= 0:
            raise ValueError(f"loss_chunk.chunk_size must be positive, got {self.chunk_size}")


@dataclass
class MoEConfig:
    aux_loss_coeff: float = 0.0
    z_loss_coeff: float = 0.0
    token_dispatcher: str = "alltoall"

    def __post_init__(self) -> None:
        self.aux_loss_coeff, self.z_loss_coeff = float(self.aux_loss_coeff), float(self.z_loss_coeff)
        if self.token_dispatcher != "alltoall":
            raise ValueError("moe.token_dispatcher must be 'alltoall'")


@dataclass
class DiffusionConfig:
    cap_lambda: float = 0.0
    bd_mask_low: float = 0.3
    bd_mask_high: float = 0.8
    bd_block_size: int = 32

    def __post_init__(self) -> None:
        self.cap_lambda = float(self.cap_lambda)
        self.bd_mask_low, self.bd_mask_high = float(self.bd_mask_low), float(self.bd_mask_high)
        self.bd_block_size = int(self.bd_block_size)
        if self.bd_block_size < 1:
            raise ValueError("diffusion.bd_block_size must be a positive integer")


@dataclass
class MfuConfig:
    enabled: bool = False
    card: str | None = None

    def __post_init__(self) -> None:
        self.enabled = string_to_bool(self.enabled)


@dataclass(frozen=True)
class FreezePolicy:
    parameter_groups: tuple[ParameterGroup, ...] = ()
    patterns: tuple[str, ...] = ()

    @property
    def enabled(self) -> bool:
        return bool(self.parameter_groups or self.patterns)

    @classmethod
    def from_list(cls, entries: Iterable[ParameterGroup | str] | ParameterGroup | str | None) -> "FreezePolicy":
        """Entries naming a `ParameterGroup` become groups; anything else is an FQN pattern."""
        if entries is None:
            return cls()
        if isinstance(entries, (ParameterGroup, str)):
            entries = (entries,)
        groups, patterns = [], []
        names = {g.value for g in ParameterGroup}
        for e in entries:
            if isinstance(e, ParameterGroup) or e in names:
                g = ParameterGroup(e)
                if g not in groups:
                    groups.append(g)
            else:
                patterns.append(str(e))
        return cls(tuple(groups), tuple(patterns))


@dataclass
class CPUOffloadConfig:
    enabled: Optional[bool] = None
    mode: CPUOffloadMode = CPUOffloadMode.FULL
    optimizer_memory_fraction: float = 0.8

    def __post_init__(self) -> None:
        if self.enabled is None:
            return
        self.enabled = string_to_bool(self.enabled)
        if not self.enabled:
            self.mode, self.optimizer_memory_fraction = CPUOffloadMode.FULL, 0.8
            return
        self.mode = CPUOffloadMode(self.mode)
        self.optimizer_memory_fraction = float(self.optimizer_memory_fraction)
        if not 0 <= self.optimizer_memory_fraction <= 1:
            raise ValueError("optimizer_memory_fraction must be in [0, 1]")


@dataclass
class FSDPConfig:
    sharding_strategy: ShardingStrategy = ShardingStrategy.FULL_SHARD
    # True / False, or "auto": gathered parameters stay resident between forward and backward when all
    # FSDP-managed parameters are at most `resident_fraction` of the device memory (never on CPU meshes)
    reshard_after_forward: Any = "auto"
    resident_fraction: float = 0.10
    # consecutive decoder layers share one FSDP unit until it gathers this many bf16 bytes; "auto" = 256 MiB on
    # CUDA meshes and no merging on CPU meshes; 0 = one unit per layer
    unit_min_bytes: Any = "auto"
    # decoder layers whose world-sharded parameters are a small part of the device memory can stay REPLICATED instead
    # (bf16 weights + fp32 master + moments on every rank, one gradient all-reduce of a flat buffer per optimizer
    # step): no per-layer all-gather / reduce-scatter and none of their per-parameter host work.  True / False, or
    # "auto": replicate on CUDA meshes when those parameters with their optimizer state (18 bytes each) take at most
    # `replicate_fraction` of the device memory.  Embeddings, output head and expert containers keep their placements.
    replicate_layers: Any = "auto"
    replicate_fraction: float = 0.12
    # all-gather / reduce-scatter of FSDP units: "auto" (peer-memory NVLink kernels when every rank of the group
    # has its own GPU on one node, else NCCL), "p2p" (required), "nccl"
    transport: str = "auto"
    cpu_offload: CPUOffloadConfig = field(default_factory=lambda: CPUOffloadConfig(enabled=False))
    prefetch_strategy: FSDPPrefetchStrategy = FSDPPrefetchStrategy.AUTO
    prefetch_direction: FSDPPrefetchDirection = FSDPPrefetchDirection.FORWARD_BACKWARD
    forward_prefetch_depth: int = 1
    backward_prefetch_depth: int = 1

    def __post_init__(self) -> None:
        co = self.cpu_offload
        if co is None:
            self.cpu_offload = CPUOffloadConfig(enabled=False)
        elif isinstance(co, bool):
            raise ValueError("cpu_offload must be an object with 'enabled'; bare true/false is not accepted")
        elif isinstance(co, dict):
            if "enabled" not in co:
                raise ValueError("cpu_offload requires 'enabled'")
            self.cpu_offload = CPUOffloadConfig(**co)
        self.sharding_strategy = ShardingStrategy(self.sharding_strategy)
        self.prefetch_strategy = FSDPPrefetchStrategy(self.prefetch_strategy)
        self.prefetch_direction = FSDPPrefetchDirection(self.prefetch_direction)
        if not (isinstance(self.reshard_after_forward, str) and self.reshard_after_forward.lower() == "auto"):
            self.reshard_after_forward = string_to_bool(self.reshard_after_forward)
        else:
            self.reshard_after_forward = "auto"
        if isinstance(self.unit_min_bytes, str) and self.unit_min_bytes.lower() == "auto":
            import torch

            self.unit_min_bytes = (256 << 20) if torch.cuda.is_available() else 0
        self.unit_min_bytes = int(self.unit_min_bytes)
        self.resident_fraction = float(self.resident_fraction)
        if not (isinstance(self.replicate_layers, str) and self.replicate_layers.lower() == "auto"):
            self.replicate_layers = string_to_bool(self.replicate_layers)
        else:
            self.replicate_layers = "auto"
        self.replicate_fraction = float(self.replicate_fraction)
        if str(self.transport).lower() not in ("auto", "p2p", "nccl"):
            raise ValueError("backend_config.transport must be auto, p2p or nccl")
        self.forward_prefetch_depth, self.backward_prefetch_depth = int(self.forward_prefetch_depth), int(self.backward_prefetch_depth)
        if self.forward_prefetch_depth < 1 or self.backward_prefetch_depth < 1:
            raise ValueError("prefetch depth must be >= 1")
        if self.prefetch_direction is FSDPPrefetchDirection.FORWARD and self.backward_prefetch_depth != 1:
            raise ValueError("backward_prefetch_depth has no effect when prefetch_direction=forward")


@dataclass
class EngineConfig:
    backend: DistributedBackend = DistributedBackend.FSDP2
    parallel_plan: Any = None
    mixed_precision: MixedPrecisionPolicy = MixedPrecisionPolicy.BF16
    use_deterministic_algorithms: bool = False
    ops: OpsConfig = field(default_factory=OpsConfig)
    backend_config: Any = None
    activation_checkpointing: ActivationCheckpointingConfig = field(default_factory=ActivationCheckpointingConfig)
    comm: CommConfig = field(default_factory=CommConfig)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    mtp: MTPConfig = field(default_factory=MTPConfig)
    dspark: DSparkTrainingConfig = field(default_factory=DSparkTrainingConfig)
    moe: MoEConfig = field(default_factory=MoEConfig)
    loss_chunk: LossChunkConfig = field(default_factory=LossChunkConfig)
    freeze_policy: FreezePolicy = field(default_factory=FreezePolicy)
    diffusion: DiffusionConfig = field(default_factory=DiffusionConfig)
    mfu: MfuConfig = field(default_factory=MfuConfig)
    gbs: int | None = None
    plugin_paths: list[str] = field(default_factory=list)
    extra: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        self.backend = DistributedBackend(self.backend)
        self.mixed_precision = parse_mixed_precision(self.mixed_precision)
        self.use_deterministic_algorithms = string_to_bool(self.use_deterministic_algorithms)
        if self.backend_config is None:
            self.backend_config = FSDPConfig()
        elif isinstance(self.backend_config, dict):
            self.backend_config = FSDPConfig(**self.backend_config)
        for name, cls in _NESTED.items():
            v = getattr(self, name)
            if v is None:
                setattr(self, name, cls())
            elif isinstance(v, dict):
                setattr(self, name, build_dataclass(cls, v))
        if isinstance(self.freeze_policy, (list, tuple, str)):
            self.freeze_policy = FreezePolicy.from_list(self.freeze_policy)
        if isinstance(self.parallel_plan, dict):
            self.parallel_plan = FSDPParallelPlan.from_dict(self.parallel_plan)
        if self.gbs is not None:
            self.gbs = int(self.gbs)
            if self.gbs <= 0:
                raise ValueError(f"gbs (--tt_gbs) must be a positive integer, got {self.gbs}")

    # ------------------------------------------------------------------ (de)serialisation
    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "EngineConfig":
        """Nested dicts in the YAML schema, plus the legacy flat spellings (`sp_size`, `ep_size`,
        `gradient_checkpointing`, `cpu_offload`, `reshard_after_forward`, `aux_loss_coeff`, ...)."""
        d = dict(d)
        known = {f.name for f in fields(cls)}
        flat_moves = {
            "sp_size": ("parallel_plan", "sp_size"), "ep_size": ("parallel_plan", "ep_size"),
            "gradient_checkpointing": ("activation_checkpointing", "enabled"),
            "ac_use_reentrant": ("activation_checkpointing", "use_reentrant"),
            "op_policy": ("ops", "policy"),
            "reshard_after_forward": ("backend_config", "reshard_after_forward"),
            "prefetch_strategy": ("backend_config", "prefetch_strategy"),
            "prefetch_direction": ("backend_config", "prefetch_direction"),
            "forward_prefetch_depth": ("backend_config", "forward_prefetch_depth"),
            "backward_prefetch_depth": ("backend_config", "backward_prefetch_depth"),
            "moe_aux_loss_coeff": ("moe", "aux_loss_coeff"), "moe_z_loss_coeff": ("moe", "z_loss_coeff"),
            "moe_token_dispatcher": ("moe", "token_dispatcher"),
            "enable_chunk_loss": ("loss_chunk", "enabled"), "loss_chunk_size": ("loss_chunk", "chunk_size"),
            "enable_mtp": ("mtp", "enabled"), "mtp_loss_scaling_factor": ("mtp", "loss_scaling_factor"),
            "hf_export": ("checkpoint", "hf_export"), "log_mfu": ("mfu", "enabled"), "card_name": ("mfu", "card"),
        }
        for flat, (outer, inner) in flat_moves.items():
            if flat in d:
                tgt = d.setdefault(outer, {})
                if isinstance(tgt, dict):
                    tgt.setdefault(inner, d.pop(flat))
                else:
                    d.pop(flat)
        if "cpu_offload" in d:
            v = d.pop("cpu_offload")
            bc = d.setdefault("backend_config", {})
            if isinstance(bc, dict):
                bc.setdefault("cpu_offload", v if isinstance(v, dict) else {"enabled": v})
        # ignore keys that belong to other parallel schemes but are accepted for compatibility
        for k in ("pp_size", "tp_size", "dp_size"):
            d.pop(k, None)
        unknown = set(d) - known
        if unknown:
            raise ValueError(f"unknown engine config keys: {sorted(unknown)}")
        return build_dataclass(cls, d)

    def to_dict(self) -> dict[str, Any]:
        def conv(v):
            if isinstance(v, FSDPParallelPlan):
                pd = v.to_dict()
                for spec in pd["plan"].values():
                    if spec.get("replace_module") is not None:
                        spec["replace_module"] = getattr(spec["replace_module"], "__name__", str(spec["replace_module"]))
                    spec["module_kwargs"] = {k: repr(x) for k, x in (spec.get("module_kwargs") or {}).items()}
                    if spec.get("placement"):
                        spec["placement"]["placement"] = str(spec["placement"]["placement"])
                    if spec.get("vision_balance"):
                        vb = spec["vision_balance"]
                        vb["mode"] = vb["mode"].value if vb["mode"] is not None else None
                        vb["io"] = type(vb["io"]).__name__ if vb["io"] is not None else None
                return pd
            if is_dataclass(v) and not isinstance(v, type):
                return {f.name: conv(getattr(v, f.name)) for f in fields(v)}
            if isinstance(v, Enum):
                return v.value
            if isinstance(v, (list, tuple)):
                return [conv(x) for x in v]
            if isinstance(v, dict):
                return {k: conv(x) for k, x in v.items()}
            return v

        return conv(self)


_NESTED = {
    "ops": OpsConfig, "activation_checkpointing": ActivationCheckpointingConfig, "comm": CommConfig,
    "optimizer": OptimizerConfig, "checkpoint": CheckpointConfig, "mtp": MTPConfig, "dspark": DSparkTrainingConfig,
    "moe": MoEConfig, "loss_chunk": LossChunkConfig, "diffusion": DiffusionConfig, "mfu": MfuConfig,
}


def build_dataclass(cls, data: dict[str, Any]):
    """Instantiate `cls` from a mapping; unknown keys are errors, nested dataclass fields accept dicts."""
    if not isinstance(data, dict):
        raise TypeError(f"{cls.__name__} expects a mapping, got {type(data).__name__}")
    names = {f.name: f for f in fields(cls)}
    unknown = set(data) - set(names)
    if unknown:
        raise ValueError(f"unknown keys for {cls.__name__}: {sorted(unknown)}")
    hints = typing.get_type_hints(cls)
    kw = {}
    for k, v in data.items():
        t = hints.get(k)
        if isinstance(v, dict) and is_dataclass(t):
            v = build_dataclass(t, v)
        kw[k] = v
    return cls(**kw)


def deep_merge(base: dict, over: dict) -> dict:
    out = dict(base)
    for k, v in over.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = deep_merge(out[k], v)
        else:
            out[k] = v
    return out


def set_path(d: dict, path: str, value: Any) -> None:
    parts = path.split(".")
    for p in parts[:-1]:
        d = d.setdefault(p, {})
    d[parts[-1]] = value


_FILE_ROOT = "engine_config"

_BUILTIN_DEFAULTS: dict[str, Any] = {
    "backend": "fsdp2",
    "mixed_precision": "fp32",
    "parallel_plan": {"sp_size": 1, "ep_size": 1},
    "backend_config": {"reshard_after_forward": "auto"},
}


def load_config_file(path: str) -> dict[str, Any]:
    """Reads a YAML or JSON file whose only root key is `engine_config`; unknown keys are rejected when the
    dataclasses are built."""
    with open(path) as f:
        text = f.read()
    if path.endswith(".json"):
        data = json.loads(text)
    else:
        import yaml

        data = yaml.safe_load(text)
    if not isinstance(data, dict) or set(data) != {_FILE_ROOT}:
        raise ValueError(f"{path}: expected a single root key {_FILE_ROOT!r}, got {sorted(data or {})}")
    body = data[_FILE_ROOT] or {}
    if not isinstance(body, dict):
        raise ValueError(f"{path}: {_FILE_ROOT!r} must be a mapping")
    return body


def build_from_args(args=None, *, defaults: dict[str, Any] | None = None, env: dict[str, str] | None = None) -> EngineConfig:
    """Merge built-in defaults < `defaults` (adapter-derived) / non-explicit arg values < environment <
    config file < explicitly passed `--tt_*` flags into an `EngineConfig`."""
    from .args import ARG_SPECS, TorchTurboArgs

    env = os.environ if env is None else env
    merged: dict[str, Any] = deep_merge(_BUILTIN_DEFAULTS, defaults or {})
    args = args or TorchTurboArgs()
    explicit = set(getattr(args, "config_overrides", ()) or ())
    # layer 1: values carried on the args object that were not typed by the user
    for spec in ARG_SPECS:
        if spec.config_path is None or spec.name in explicit:
            continue
        v = getattr(args, spec.name, None)
        if v is not None:
            set_path(merged, spec.config_path, spec.convert(v))
    # layer 2: environment
    for spec in ARG_SPECS:
        if spec.env and spec.config_path and spec.env in env and env[spec.env] != "":
            set_path(merged, spec.config_path, spec.convert(env[spec.env]))
    # layer 3: file
    cfg_path = getattr(args, "config", None)
    if cfg_path:
        merged = deep_merge(merged, load_config_file(cfg_path))
    # layer 4: explicit flags
    for spec in ARG_SPECS:
        if spec.config_path and spec.name in explicit:
            set_path(merged, spec.config_path, spec.convert(getattr(args, spec.name)))
    plugins = list(getattr(args, "plugin", None) or [])
    if plugins:
        merged["plugin_paths"] = plugins
    fp = merged.get("freeze_policy")
    if isinstance(fp, dict):
        entries: list = [g for g, on in (fp.get("groups") or {}).items() if on]
        entries += list(fp.get("parameter_groups") or []) + list(fp.get("patterns") or [])
        merged["freeze_policy"] = FreezePolicy.from_list(entries)
    return EngineConfig.from_dict(merged)
