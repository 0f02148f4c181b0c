"""`--tt_*` command-line surface.

One table (`ARG_SPECS`) maps every knob to its CLI flag, environment variable and dotted config path, so
the parser, the env layer and the config merge can never drift apart (same idea as the single spec table
of the reference, engine/args.py:253-725).  `parse_torchturbo_args` consumes the `--tt_*` flags and hands
the remaining argv to the training framework; which flags were typed explicitly is remembered in
`config_overrides` because explicit flags outrank the config file.
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass, field
from typing import Any, Callable

from .config import string_to_bool


@dataclass(frozen=True)
class TurboArgSpec:
    name: str                       # attribute on TorchTurboArgs
    type: Callable[[Any], Any] = str
    env: str | None = None
    config_path: str | None = None  # None: runtime-only knob
    help: str = ""
    choices: tuple | None = None
    repeatable: bool = False

    @property
    def flag(self) -> str:
        return f"--tt_{self.name}"

    def convert(self, v: Any) -> Any:
        if self.type is bool:
            return string_to_bool(v)
        return self.type(v) if not isinstance(v, (list, tuple)) else [self.type(x) for x in v]


def _S(name, type=str, env=None, path=None, help="", choices=None, repeatable=False):
    return TurboArgSpec(name, type, env, path, help, choices, repeatable)


ARG_SPECS: tuple[TurboArgSpec, ...] = (
    _S("config", str, help="YAML/JSON file with root key `engine_config`"),
    _S("backend", str, "TORCH_TURBO_BACKEND", "backend", choices=("fsdp2",)),
    _S("mixed_precision", str, "TORCH_TURBO_MIXED_PRECISION", "mixed_precision"),
    _S("op_policy", str, "TORCH_TURBO_OP_POLICY", "ops.policy", choices=("auto", "native", "custom")),
    _S("optimizer", str, None, "optimizer.name", choices=("muon",)),
    _S("use_deterministic_algorithms", bool, "TORCH_TURBO_USE_DETERMINISTIC_ALGORITHMS", "use_deterministic_algorithms"),
    _S("sp_size", int, "TORCH_TURBO_SP_SIZE", "parallel_plan.sp_size"),
    _S("ep_size", int, "TORCH_TURBO_EP_SIZE", "parallel_plan.ep_size"),
    _S("gbs", int, "TORCH_TURBO_GBS", "gbs"),
    _S("gradient_checkpointing", bool, "TORCH_TURBO_GRADIENT_CHECKPOINTING", "activation_checkpointing.enabled"),
    _S("ac_use_reentrant", bool, "TORCH_TURBO_AC_USE_REENTRANT", "activation_checkpointing.use_reentrant"),
    _S("cpu_offload", bool, None, "backend_config.cpu_offload.enabled"),
    _S("prefetch_strategy", str, "TORCH_TURBO_PREFETCH_STRATEGY", "backend_config.prefetch_strategy"),
    _S("prefetch_direction", str, "TORCH_TURBO_PREFETCH_DIRECTION", "backend_config.prefetch_direction"),
    _S("forward_prefetch_depth", int, "TORCH_TURBO_FORWARD_PREFETCH_DEPTH", "backend_config.forward_prefetch_depth"),
    _S("backward_prefetch_depth", int, "TORCH_TURBO_BACKWARD_PREFETCH_DEPTH", "backend_config.backward_prefetch_depth"),
    _S("reshard_after_fwd", bool, "TORCH_TURBO_RESHARD_AFTER_FWD", "backend_config.reshard_after_forward"),
    _S("enable_mtp", bool, None, "mtp.enabled"),
    _S("mtp_loss_scaling_factor", float, None, "mtp.loss_scaling_factor"),
    _S("mtp_log_loss", bool, None, "mtp.log_loss"),
    _S("enable_dspark", bool, None, "dspark.enabled"),
    _S("dspark_loss_scaling_factor", float, None, "dspark.loss_scaling_factor"),
    _S("dspark_num_anchors", int, None, "dspark.num_anchors"),
    _S("dspark_loss_decay_gamma", float, None, "dspark.loss_decay_gamma"),
    _S("dspark_ce_loss_alpha", float, None, "dspark.ce_loss_alpha"),
    _S("dspark_l1_loss_alpha", float, None, "dspark.l1_loss_alpha"),
    _S("dspark_confidence_loss_alpha", float, None, "dspark.confidence_loss_alpha"),
    _S("moe_token_dispatcher", str, "TORCH_TURBO_MOE_TOKEN_DISPATCHER", "moe.token_dispatcher"),
    _S("moe_aux_loss_coeff", float, None, "moe.aux_loss_coeff"),
    _S("moe_z_loss_coeff", float, None, "moe.z_loss_coeff"),
    _S("enable_chunk_loss", bool, None, "loss_chunk.enabled"),
    _S("loss_chunk_size", int, None, "loss_chunk.chunk_size"),
    _S("freeze_vision_tower", bool, None, "freeze_policy.groups.vision_tower"),
    _S("freeze_multi_modal_projector", bool, None, "freeze_policy.groups.multi_modal_projector"),
    _S("freeze_language_model", bool, None, "freeze_policy.groups.language_model"),
    _S("cap_lambda", float, None, "diffusion.cap_lambda"),
    _S("bd_mask_low", float, None, "diffusion.bd_mask_low"),
    _S("bd_mask_high", float, None, "diffusion.bd_mask_high"),
    _S("bd_block_size", int, None, "diffusion.bd_block_size"),
    _S("log_mfu", bool, "TORCH_TURBO_LOG_MFU", "mfu.enabled"),
    _S("card_name", str, "TORCH_TURBO_CARD_NAME", "mfu.card"),
    _S("hf_export", str, None, "checkpoint.hf_export", choices=("every", "final")),
    # runtime-only knobs (no config path)
    _S("profiling", bool, help="record a torch.profiler trace"),
    _S("memory_snapshot_steps", int, help="dump an allocator snapshot at this step"),
    _S("log_level", str, help="package log level"),
    _S("plugin", str, repeatable=True, help="path[:config] of a plugin module; may be repeated"),
)

_SPEC_BY_NAME = {s.name: s for s in ARG_SPECS}


@dataclass
class TorchTurboArgs:
    """Parsed `--tt_*` values (`None` = not given) plus the names that were typed explicitly."""

    config: str | None = None
    backend: str | None = None
    mixed_precision: str | None = None
    op_policy: str | None = None
    optimizer: str | None = None
    use_deterministic_algorithms: bool | None = None
    sp_size: int | None = None
    ep_size: int | None = None
    gbs: int | None = None
    gradient_checkpointing: bool | None = None
    ac_use_reentrant: bool | None = None
    cpu_offload: bool | None = None
    prefetch_strategy: str | None = None
    prefetch_direction: str | None = None
    forward_prefetch_depth: int | None = None
    backward_prefetch_depth: int | None = None
    reshard_after_fwd: bool | None = None
    enable_mtp: bool | None = None
    mtp_loss_scaling_factor: float | None = None
    mtp_log_loss: bool | None = None
    enable_dspark: bool | None = None
    dspark_loss_scaling_factor: float | None = None
    dspark_num_anchors: int | None = None
    dspark_loss_decay_gamma: float | None = None
    dspark_ce_loss_alpha: float | None = None
    dspark_l1_loss_alpha: float | None = None
    dspark_confidence_loss_alpha: float | None = None
    moe_token_dispatcher: str | None = None
    moe_aux_loss_coeff: float | None = None
    moe_z_loss_coeff: float | None = None
    enable_chunk_loss: bool | None = None
    loss_chunk_size: int | None = None
    freeze_vision_tower: bool | None = None
    freeze_multi_modal_projector: bool | None = None
    freeze_language_model: bool | None = None
    cap_lambda: float | None = None
    bd_mask_low: float | None = None
    bd_mask_high: float | None = None
    bd_block_size: int | None = None
    log_mfu: bool | None = None
    card_name: str | None = None
    hf_export: str | None = None
    profiling: bool | None = None
    memory_snapshot_steps: int | None = None
    log_level: str | None = None
    plugin: list[str] = field(default_factory=list)
    config_overrides: tuple[str, ...] = ()


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(add_help=False, allow_abbrev=False)
    for s in ARG_SPECS:
        kw: dict[str, Any] = dict(dest=s.name, default=argparse.SUPPRESS, help=s.help)
        if s.repeatable:
            p.add_argument(s.flag, action="append", type=s.type, **kw)
        elif s.type is bool:
            p.add_argument(s.flag, nargs="?", const=True, type=string_to_bool, **kw)
        else:
            if s.choices:
                kw["choices"] = s.choices
            p.add_argument(s.flag, type=s.type, **kw)
    return p


def parse_torchturbo_args(argv: list[str] | None = None) -> tuple[TorchTurboArgs, list[str]]:
    """Returns (args, remaining argv).  Flags that were not typed stay `None`, so lower layers of the
    config merge can still fill them."""
    import sys

    argv = list(sys.argv[1:] if argv is None else argv)
    ns, rest = build_parser().parse_known_args(argv)
    given = vars(ns)
    args = TorchTurboArgs(**given, config_overrides=tuple(k for k in given if _SPEC_BY_NAME[k].config_path))
    return args, rest


_STASHED: TorchTurboArgs | None = None


def set_torchturbo_args(args: TorchTurboArgs | None) -> None:
    global _STASHED
    _STASHED = args


def get_torchturbo_args() -> TorchTurboArgs | None:
    return _STASHED
