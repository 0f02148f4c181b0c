"""Argument bridging and data helpers of the LlamaFactory adapter.

* engine config from LlamaFactory's parsed arguments (+ `--tt_*` flags, env, config file),
* the gradient-checkpointing hand-over (the engine installs activation checkpointing *before* sharding, so the
  framework's own late `gradient_checkpointing_enable()` must be switched off),
* CPU-offload resolution from the `--fsdp "... offload"` option,
* LoRA: LlamaFactory's finetuning arguments -> engine `LoraConfig`, and a copy of the arguments with LoRA stripped so
  that the framework does not wrap the model a second time,
* refusing options the engine does not implement instead of silently ignoring them,
* vision-boundary aware packing for multimodal pre-training.
(adapters/llamafactory_v0/utils.py:22-762 of the reference.)
"""
from __future__ import annotations

import copy
from itertools import chain
from typing import Any, Sequence

from ...engine.args import TorchTurboArgs, get_torchturbo_args
from ...engine.config import CPUOffloadConfig, build_from_args

SUPPORTED_STAGES = ("sft", "pt", "dpo")

# finetuning options that change the optimizer or the loss in ways the engine does not implement
_UNSUPPORTED_OPTIMIZERS = ("use_galore", "use_apollo", "use_badam", "use_adam_mini", "loraplus_lr_ratio")
_UNSUPPORTED_LOSSES = ("use_dft_loss", "use_eaft_loss", "asft_alpha")
_UNSUPPORTED_LORA = ("pissa_init", "create_new_adapter", "use_unsloth")
_UNSUPPORTED_MODEL = ("use_unsloth", "use_kt", "mixture_of_depths", "enable_liger_kernel", "quantization_bit", "shift_attn")


def fsdp_options_from_raw_args(raw_args: Any) -> Any:
    """The `fsdp` option as the user gave it, from a raw argument dict or argv-style list (None if absent)."""
    if isinstance(raw_args, dict):
        return raw_args.get("fsdp")
    if isinstance(raw_args, (list, tuple)):
        for i, tok in enumerate(raw_args):
            if tok == "--fsdp" and i + 1 < len(raw_args):
                return raw_args[i + 1]
            if isinstance(tok, str) and tok.startswith("--fsdp="):
                return tok.split("=", 1)[1]
    return None


def _fsdp_tokens(fsdp_options: Any) -> list[str]:
    if isinstance(fsdp_options, str):
        return fsdp_options.replace(",", " ").split()
    if isinstance(fsdp_options, (list, tuple)):
        out: list[str] = []
        for item in fsdp_options:
            out.extend(str(getattr(item, "value", item)).replace(",", " ").split())
        return out
    return []


def resolve_cpu_offload(fsdp_options: Any, tt_args: TorchTurboArgs | None, *, strict: bool = True) -> CPUOffloadConfig:
    """One answer for "is parameter offload on" used both when the process group is created (offload needs a
    CPU-capable backend next to NCCL) and when the engine config is built.  `--fsdp "... offload"` asks for full
    offload; an explicit engine setting that disables offload contradicts it (an error when `strict`)."""
    want = "offload" in _fsdp_tokens(fsdp_options)
    explicit = getattr(tt_args, "cpu_offload", None) if tt_args is not None else None
    enabled = getattr(tt_args, "cpu_offload_enabled", None) if tt_args is not None else None
    if isinstance(explicit, dict):
        cfg = CPUOffloadConfig(**explicit)
    elif isinstance(explicit, CPUOffloadConfig):
        cfg = copy.copy(explicit)
    elif isinstance(explicit, bool):
        mode = getattr(tt_args, "cpu_offload_mode", None)
        cfg = CPUOffloadConfig(enabled=explicit, **({"mode": mode} if mode else {}))
    elif enabled is not None:
        cfg = CPUOffloadConfig(enabled=bool(enabled))
    else:
        cfg = None
    if want:
        if cfg is not None and strict and (not cfg.enabled or str(getattr(cfg.mode, "value", cfg.mode)) != "full"):
            raise ValueError("engine cpu_offload must be enabled with mode='full' when the framework enables FSDP "
                             "parameter offload (--fsdp '... offload')")
        if cfg is None or not cfg.enabled:
            cfg = CPUOffloadConfig(enabled=True)
    return cfg if cfg is not None else CPUOffloadConfig(enabled=False)


def take_over_gradient_checkpointing(training_args: Any, model_args: Any, raw_args: Any,
                                     tt_args: TorchTurboArgs | None = None) -> tuple[bool, Any]:
    """Returns (activation checkpointing wanted, raw args with the framework's own checkpointing disabled).

    The framework enables gradient checkpointing after the model exists, which is after `fully_shard` here; recompute
    must live inside each FSDP unit, so the request is moved to the engine and switched off on the framework side."""
    wanted = bool(getattr(training_args, "gradient_checkpointing", False)) or \
        (model_args is not None and not getattr(model_args, "disable_gradient_checkpointing", True))
    explicit = getattr(tt_args, "gradient_checkpointing", None) if tt_args is not None else None
    if explicit is not None and bool(explicit) != wanted and getattr(training_args, "gradient_checkpointing", None) is not None:
        raise ValueError(f"--tt_gradient_checkpointing={bool(explicit)} contradicts the framework's gradient "
                         f"checkpointing setting ({wanted})")
    if explicit is not None:
        wanted = bool(explicit)
    if training_args is not None and hasattr(training_args, "gradient_checkpointing"):
        training_args.gradient_checkpointing = False
    if model_args is not None and hasattr(model_args, "disable_gradient_checkpointing"):
        model_args.disable_gradient_checkpointing = True
    if isinstance(raw_args, dict):
        raw_args = dict(raw_args, gradient_checkpointing=False, disable_gradient_checkpointing=True)
    elif isinstance(raw_args, list):
        out, skip = [], False
        for tok in raw_args:
            if skip:
                skip = False
                continue
            if tok in ("--gradient_checkpointing", "--disable_gradient_checkpointing"):
                skip = True
                continue
            if isinstance(tok, str) and tok.startswith(("--gradient_checkpointing=", "--disable_gradient_checkpointing=")):
                continue
            out.append(tok)
        raw_args = out + ["--gradient_checkpointing", "false", "--disable_gradient_checkpointing", "true"]
    return wanted, raw_args


def raise_if_unsupported_lf_args(model_args: Any, finetuning_args: Any, training_args: Any = None) -> None:
    bad = [k for k in _UNSUPPORTED_MODEL if getattr(model_args, k, None) not in (None, False, 0, "")]
    bad += [k for k in _UNSUPPORTED_OPTIMIZERS + _UNSUPPORTED_LOSSES if getattr(finetuning_args, k, None) not in (None, False, 0, 0.0, "")]
    if getattr(finetuning_args, "finetuning_type", "full") == "lora":
        bad += [k for k in _UNSUPPORTED_LORA if getattr(finetuning_args, k, None) not in (None, False, 0, "")]
    if getattr(finetuning_args, "finetuning_type", "full") not in ("full", "lora", "freeze"):
        bad.append(f"finetuning_type={finetuning_args.finetuning_type}")
    if training_args is not None and getattr(training_args, "deepspeed", None):
        bad.append("deepspeed")
    if getattr(finetuning_args, "stage", "sft") == "dpo":
        if getattr(finetuning_args, "pref_loss", "sigmoid") not in ("sigmoid",):
            bad.append(f"pref_loss={finetuning_args.pref_loss}")
        if getattr(finetuning_args, "use_ref_model", True) is False:
            bad.append("use_ref_model=False")
    if bad:
        raise ValueError("these LlamaFactory options are not supported by the engine: " + ", ".join(sorted(set(bad))))


def build_config_from_lf_args(model_args: Any, training_args: Any, finetuning_args: Any, tt_args: TorchTurboArgs | None = None,
                              raw_args: Any = None, gradient_checkpointing: bool | None = None):
    """Adapter-derived defaults (lowest precedence): precision follows `--bf16`, activation checkpointing follows the
    framework's gradient-checkpointing request, CPU offload follows `--fsdp offload`."""
    tt_args = tt_args or get_torchturbo_args()
    raise_if_unsupported_lf_args(model_args, finetuning_args, training_args)
    gc = gradient_checkpointing        # already taken over by the caller (the framework flags are off by then)
    if gc is None:
        gc, _ = take_over_gradient_checkpointing(training_args, model_args, None, tt_args)
    defaults: dict[str, Any] = {"mixed_precision": "bf16" if getattr(training_args, "bf16", False) else "fp32",
                                "activation_checkpointing": {"enabled": gc}}
    fsdp_opt = getattr(training_args, "fsdp", None) or fsdp_options_from_raw_args(raw_args)
    off = resolve_cpu_offload(fsdp_opt, tt_args)
    if off.enabled:
        defaults["backend_config"] = {"cpu_offload": {"enabled": True, "mode": str(getattr(off.mode, "value", off.mode))}}
    if getattr(finetuning_args, "stage", "sft") == "dpo" or getattr(finetuning_args, "disable_shuffling", False):
        pass  # sampler choices are made by the trainer, not the engine config
    return build_from_args(tt_args, defaults=defaults)


def build_lora_config_from_lf_args(finetuning_args: Any):
    if getattr(finetuning_args, "finetuning_type", "full") != "lora":
        return None
    from ...engine.peft import LoraConfig

    target = getattr(finetuning_args, "lora_target", "all")
    if target in ("all", ["all"]):
        targets = ["all-linear"]
    else:
        targets = list(target) if isinstance(target, (list, tuple)) else [t.strip() for t in str(target).split(",") if t.strip()]
    rank = int(finetuning_args.lora_rank)
    extra = getattr(finetuning_args, "additional_target", None)
    kw = {}
    if extra:
        kw["modules_to_save"] = list(extra) if isinstance(extra, (list, tuple)) else [t.strip() for t in str(extra).split(",")]
    try:
        return LoraConfig(r=rank, lora_alpha=getattr(finetuning_args, "lora_alpha", None) or 2 * rank,
                          lora_dropout=float(getattr(finetuning_args, "lora_dropout", 0.0) or 0.0), target_modules=targets,
                          use_dora=bool(getattr(finetuning_args, "use_dora", False)),
                          use_rslora=bool(getattr(finetuning_args, "use_rslora", False)), **kw)
    except TypeError:
        return LoraConfig(r=rank, lora_alpha=getattr(finetuning_args, "lora_alpha", None) or 2 * rank,
                          lora_dropout=float(getattr(finetuning_args, "lora_dropout", 0.0) or 0.0), target_modules=targets,
                          use_dora=bool(getattr(finetuning_args, "use_dora", False)),
                          use_rslora=bool(getattr(finetuning_args, "use_rslora", False)))


def strip_lora_args(args: Any) -> Any:
    """A copy of the finetuning arguments (object, dict or argv list) that says "full fine-tuning": the engine has
    already applied LoRA, the framework must not wrap the model again or look for adapter files."""
    if isinstance(args, dict):
        out = {k: v for k, v in args.items() if not k.startswith(("lora_", "use_dora", "use_rslora", "pissa_", "adapter_name_or_path"))}
        out["finetuning_type"] = "full"
        return out
    if isinstance(args, list):
        out, skip = [], False
        for tok in args:
            if skip:
                skip = False
                continue
            name = tok.split("=", 1)[0].lstrip("-") if isinstance(tok, str) and tok.startswith("--") else None
            if name and (name.startswith(("lora_", "pissa_")) or name in ("use_dora", "use_rslora", "adapter_name_or_path", "finetuning_type")):
                skip = "=" not in tok
                continue
            out.append(tok)
        return out + ["--finetuning_type", "full"]
    out = copy.copy(args)
    out.finetuning_type = "full"
    if hasattr(out, "adapter_name_or_path"):
        out.adapter_name_or_path = None
    return out


def compute_sft_loss(engine, model, inputs: dict[str, Any], *, num_items_in_batch=None, gradient_accumulation_steps: int = 1,
                     return_outputs: bool = False):
    """SFT / PT loss of one packed micro-batch through the engine (token-mean over the global batch when the trainer
    passes `num_items_in_batch`, else over the micro-batch; Ulysses ranks contribute their slice)."""
    return engine.compute_loss(model, inputs, num_items_in_batch=num_items_in_batch,
                               gradient_accumulation_steps=gradient_accumulation_steps, return_outputs=return_outputs)


def pack_with_vision_boundaries(tokenized: dict[str, list[list[int]]], images: list[list[Any]], cutoff_len: int,
                                vision_start_id: int, vision_end_id: int):
    """Cut the concatenation of tokenized samples into blocks of at most `cutoff_len` tokens without ever splitting a
    `[vision_start ... vision_end]` span: a span that would straddle a block end moves whole to the next block.
    Returns (blocked fields, images per block)."""
    flat = {k: list(chain.from_iterable(v)) for k, v in tokenized.items()}
    ids = flat.get("input_ids", [])
    if not ids:
        return {}, []
    flat_images = list(chain.from_iterable(images))
    spans, open_at = [], None
    for i, t in enumerate(ids):
        if t == vision_start_id:
            if open_at is not None:
                raise ValueError(f"nested vision span at token {i}")
            open_at = i
        elif t == vision_end_id:
            if open_at is None:
                raise ValueError(f"vision end without start at token {i}")
            spans.append((open_at, i))
            open_at = None
    if open_at is not None:
        raise ValueError("unterminated vision span")
    if len(spans) != len(flat_images):
        raise ValueError(f"{len(spans)} vision spans but {len(flat_images)} images")
    if spans and max(e - s + 1 for s, e in spans) > cutoff_len:
        raise ValueError("a vision span is longer than cutoff_len")
    blocks: dict[str, list[list[int]]] = {k: [] for k in flat}
    block_images: list[list[Any]] = []
    pos, span_i, n = 0, 0, len(ids)
    while pos < n:
        end = min(pos + cutoff_len, n)
        j, first_img = span_i, span_i
        while j < len(spans) and spans[j][0] < end:
            if spans[j][1] >= end:      # straddles the cut: the block ends right before it
                end = spans[j][0]
                break
            j += 1
        if end == pos:                   # cannot happen while every span fits a block; guards an endless loop
            raise ValueError("vision span does not fit the remaining block")
        for k in flat:
            blocks[k].append(flat[k][pos:end])
        block_images.append(flat_images[first_img:j])
        span_i, pos = j, end
    return blocks, block_images


def preprocess_multimodal_pretrain(tokenize, examples: dict[str, Sequence[Any]], cutoff_len: int, vision_start_id: int,
                                   vision_end_id: int, *, eos_token_id: int | None = None, text_key: str = "_prompt",
                                   image_key: str = "_images") -> dict[str, Any]:
    """Pre-training preprocessing for image-text documents: tokenize every document (`tokenize(text, images) ->
    list[int]` has already expanded image placeholders), append EOS, and pack with intact vision spans.  Labels equal
    the input ids (next-token loss everywhere); `images` lists the media of each packed block."""
    toks, imgs = [], []
    for text, media in zip(examples[text_key], examples.get(image_key) or [[] for _ in examples[text_key]]):
        ids = list(tokenize(text, media or []))
        if eos_token_id is not None:
            ids.append(eos_token_id)
        toks.append(ids)
        imgs.append(list(media or []))
    blocks, block_images = pack_with_vision_boundaries({"input_ids": toks}, imgs, cutoff_len, vision_start_id, vision_end_id)
    if not blocks:
        return {"input_ids": [], "attention_mask": [], "labels": [], "images": []}
    return {"input_ids": blocks["input_ids"], "attention_mask": [[1] * len(b) for b in blocks["input_ids"]],
            "labels": [list(b) for b in blocks["input_ids"]], "images": block_images}
