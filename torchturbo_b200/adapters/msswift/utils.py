"""Engine config and LoRA config from swift's parsed arguments; refusal of what the engine does not implement; the
switches swift must not act on because the engine owns them (adapters/msswift/utils.py:21-119 and args.py:40-90 of the
reference)."""
from __future__ import annotations

from typing import Any

from ...engine.args import TorchTurboArgs, get_torchturbo_args
from ...engine.config import build_from_args
from ...logging import get_logger

logger = get_logger(__name__)

# the engine owns activation checkpointing, sequence parallelism and sharding: swift's own switches are turned off
FORCED_OFF = {"gradient_checkpointing": False, "sequence_parallel_size": 1, "deepspeed": None, "fsdp": "", "fsdp_config": None,
              "use_liger_kernel": False, "padding_free": False}


def raise_if_unsupported(args: Any, tt_args: TorchTurboArgs | None = None) -> None:
    tuner, rlhf = getattr(args, "tuner_type", getattr(args, "train_type", "full")), getattr(args, "rlhf_type", None)
    bad: list[str] = []
    if tuner not in ("full", "lora"):
        bad.append(f"tuner_type={tuner!r}")
    if rlhf not in (None, "dpo"):
        bad.append(f"rlhf_type={rlhf!r}")
    if rlhf == "dpo":
        if tuner != "full":
            bad.append("DPO with tuner_type != full")
        if tt_args is not None and getattr(tt_args, "enable_mtp", False):
            bad.append("DPO with multi-token prediction")
    if getattr(args, "predict_with_generate", False):
        bad.append("predict_with_generate")
    if bad:
        raise NotImplementedError("the ms-swift adapter does not support " + ", ".join(bad))


def take_over_swift_switches(args: Any) -> dict[str, Any]:
    """Turn swift's own switches off; returns what the user had asked for (the engine config is seeded from it)."""
    asked = {k: getattr(args, k) for k in FORCED_OFF if hasattr(args, k)}
    for k in ("deepspeed", "fsdp"):
        if asked.get(k):
            logger.warning_rank0("swift option %s=%r is ignored: the engine shards the model itself", k, asked[k])
    for k, v in FORCED_OFF.items():
        if hasattr(args, k):
            setattr(args, k, v)
    ta = getattr(args, "training_args", None)
    if ta is not None:
        for k in ("gradient_checkpointing", "deepspeed", "fsdp"):
            if hasattr(ta, k):
                setattr(ta, k, FORCED_OFF[k])
    return asked


def build_config_from_swift_args(args: Any, stage: str | None = None, tt_args: TorchTurboArgs | None = None):
    tt_args = tt_args or get_torchturbo_args() or TorchTurboArgs()
    raise_if_unsupported(args, tt_args)
    asked = take_over_swift_switches(args)
    precision = "bf16" if getattr(args, "bf16", False) else ("fp32" if not getattr(args, "fp16", False) else "fp16")
    defaults: dict[str, Any] = {"mixed_precision": precision,
                                "activation_checkpointing": {"enabled": bool(asked.get("gradient_checkpointing", True))}}
    sp = int(asked.get("sequence_parallel_size") or 1)
    if sp > 1:
        defaults["parallel_plan"] = {"sp_size": sp}
    if (stage == "dpo" or getattr(args, "rlhf_type", None) == "dpo") and getattr(args, "router_aux_loss_coef", None):
        defaults["moe"] = {"aux_loss_coeff": float(args.router_aux_loss_coef)}
    return build_from_args(tt_args, defaults=defaults)


def build_lora_config_from_swift_args(args: Any):
    if getattr(args, "tuner_type", getattr(args, "train_type", "full")) != "lora":
        return None
    from ...engine.peft import LoraConfig

    rank = int(getattr(args, "lora_rank", 8) or 8)
    target = getattr(args, "target_modules", None) or "all-linear"
    if isinstance(target, str):
        targets = ["all-linear"] if target in ("all", "all-linear") else [m.strip() for m in target.split(",") if m.strip()]
    else:
        names = {str(m).strip().lower() for m in target}
        targets = ["all-linear"] if names & {"all", "all-linear"} else [str(m) for m in target]
    return LoraConfig(r=rank, lora_alpha=int(getattr(args, "lora_alpha", None) or 2 * rank), target_modules=targets,
                      lora_dropout=float(getattr(args, "lora_dropout", 0.0) or 0.0),
                      use_rslora=bool(getattr(args, "use_rslora", False)), use_dora=bool(getattr(args, "use_dora", False)))
