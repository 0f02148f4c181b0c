"""Reversible patches of LlamaFactory 0.9.x and of the pieces of transformers / accelerate it drives.

Every patch looks its target up at patch time (`importlib.import_module`), keeps the original, and restores it in
`_revert()`.  Targets that do not exist in the installed version are skipped, so one adapter serves the whole 0.9
line.  (adapters/llamafactory_v0/patches.py:37-1276 of the reference.)

  DictFieldPatch            dict-typed CLI options (`--lr_scheduler_kwargs '{"min_lr":1e-7}'`) parse as JSON strings
  RunExpPatch               builds the engine from the parsed arguments, applies the other patches, runs the stage
  PackedInputCollatorPatch  the SFT collator's output becomes one packed row with boundaries
  LoadModelPatch            `load_model` -> `engine.prepare_model` (trainable) / frozen engine model (reference)
  CreateRefModelPatch       DPO reference model built by the engine with the policy's plan
  TrainerClassPatch         stage trainers gain the engine mixins
  AcceleratorPatch          accelerate must not wrap / shard / clip: the model is already sharded
  RegisterAutoclassPatch    `register_autoclass` finds the `PreTrainedModel` class under wrappers
  LogCallbackPatch          `grad_norm` is added to `trainer_log.jsonl`
  PretrainProcessorPatch    multimodal pre-training packs with intact vision spans
"""
from __future__ import annotations

import importlib
from typing import Any

from ...logging import get_logger
from ...registry import BasePatch
from .utils import (SUPPORTED_STAGES, build_config_from_lf_args, build_lora_config_from_lf_args,
                    preprocess_multimodal_pretrain, strip_lora_args, take_over_gradient_checkpointing)

logger = get_logger(__name__)
LF_V0 = ">=0.9.0,<0.10"


def _try_import(name: str):
    try:
        return importlib.import_module(name)
    except Exception:  # noqa: BLE001 - optional target
        return None


class _AttrPatch(BasePatch):
    """Helper: remembers `(owner, attribute, original)` triples and puts them back."""

    version_spec = LF_V0

    def __init__(self) -> None:
        super().__init__()
        self._saved: list[tuple[Any, str, Any]] = []

    def _set(self, owner: Any, attr: str, new: Any) -> None:
        self._saved.append((owner, attr, getattr(owner, attr)))
        setattr(owner, attr, new)

    def _revert(self) -> None:
        for owner, attr, orig in reversed(self._saved):
            setattr(owner, attr, orig)
        self._saved.clear()


class DictFieldPatch(_AttrPatch):
    """`HfArgumentParser` gives `Union[dict, str]` fields `type=dict`, so argparse calls `dict("{...}")` and fails.
    For the listed fields the parser is told `str`; `TrainingArguments.__post_init__` then JSON-decodes the string."""

    name = "dict_field"
    fields = ("lr_scheduler_kwargs", "accelerator_config", "fsdp_config", "deepspeed", "gradient_checkpointing_kwargs")

    def _patch(self, engine=None) -> None:
        hf = _try_import("transformers.hf_argparser")
        if hf is None:
            return
        orig = hf.HfArgumentParser._parse_dataclass_field
        names = set(self.fields)

        def patched(parser, field):
            if field.name in names:
                saved = field.type
                field.type = str
                try:
                    return orig(parser, field)
                finally:
                    field.type = saved
            return orig(parser, field)

        self._set(hf.HfArgumentParser, "_parse_dataclass_field", staticmethod(patched))


class RunExpPatch(_AttrPatch):
    name = "run_exp"

    def __init__(self, adapter: Any) -> None:
        super().__init__()
        self.adapter = adapter

    def _patch(self, engine=None) -> None:
        tuner = importlib.import_module("llamafactory.train.tuner")
        orig = tuner.run_exp
        adapter = self.adapter

        def patched(args=None, callbacks=None):
            from llamafactory.hparams import get_train_args, read_args

            raw = read_args(args) if args is None or isinstance(args, (dict, list)) else args
            model_args, data_args, training_args, finetuning_args, _ = get_train_args(raw)
            if finetuning_args.stage not in SUPPORTED_STAGES:
                logger.info_rank0("stage %s is not engine-backed: running stock LlamaFactory", finetuning_args.stage)
                return orig(args, callbacks)
            from ...engine import TorchTurboEngine

            gc, raw = take_over_gradient_checkpointing(training_args, model_args, raw)
            adapter.engine = TorchTurboEngine(build_config_from_lf_args(model_args, training_args, finetuning_args, raw_args=raw,
                                                                        gradient_checkpointing=gc))
            adapter.peft_config = build_lora_config_from_lf_args(finetuning_args)
            if adapter.peft_config is not None:
                raw = strip_lora_args(raw)
            adapter.stage = finetuning_args.stage
            try:
                from ..chat_templates import register_lf_templates

                register_lf_templates()
            except Exception as e:  # noqa: BLE001 - another template API: the user's --template must exist already
                logger.warning_rank0("chat templates of the engine's model families were not registered: %s", e)
            adapter.apply_patches(adapter.engine)
            try:
                return orig(raw, callbacks)
            finally:
                adapter.revert_patches()

        self._set(tuner, "run_exp", patched)


class PackedInputCollatorPatch(_AttrPatch):
    """`SFTDataCollatorWith4DAttentionMask.__call__` (used for SFT, and for DPO through its pairwise subclass's parent)
    returns either a neat-packed row whose attention mask holds sample ids or a padded batch; both are turned into one
    packed row with `cu_seq_lens`.  Pairwise (DPO) batches are left alone: the DPO trainer packs them itself."""

    name = "packed_input_collator"

    def _patch(self, engine=None) -> None:
        coll = _try_import("llamafactory.data.collator")
        if coll is None or not hasattr(coll, "SFTDataCollatorWith4DAttentionMask"):
            return
        from ..hf_trainer import normalize_training_features

        cls = coll.SFTDataCollatorWith4DAttentionMask
        orig = cls.__call__
        pairwise = getattr(coll, "PairwiseDataCollatorWithPadding", ())

        def patched(self_, features):
            saved = getattr(self_, "block_diag_attn", False)
            self_.block_diag_attn = False       # the 4-D mask is never built: boundaries travel as cu_seq_lens
            try:
                batch = orig(self_, features)
            finally:
                self_.block_diag_attn = saved
            if pairwise and isinstance(self_, pairwise):
                return batch
            return normalize_training_features(dict(batch))

        self._set(cls, "__call__", patched)


class LoadModelPatch(_AttrPatch):
    """`load_model(tokenizer, model_args, finetuning_args, is_trainable, add_valuehead)`: trainable models are built,
    sharded and loaded by the engine (LoRA applied by the engine); non-trainable ones (reference / reward) come back
    frozen in eval mode.  Value heads are refused."""

    name = "load_model"

    def __init__(self, adapter: Any) -> None:
        super().__init__()
        self.adapter = adapter

    def _patch(self, engine=None) -> None:
        adapter = self.adapter

        def patched(tokenizer, model_args, finetuning_args, is_trainable=False, add_valuehead=False):
            if add_valuehead:
                raise NotImplementedError("value-head models (PPO / reward modelling) are not engine-backed")
            eng = adapter.engine
            path = model_args.model_name_or_path
            if not is_trainable:
                ref = eng.build_model(path)
                ref.requires_grad_(False)
                return ref.eval()
            model = eng.prepare_model(path, peft_config=adapter.peft_config)
            adapter.model = model
            return model

        for mod_name in ("llamafactory.model.loader", "llamafactory.model", "llamafactory.train.sft.workflow",
                         "llamafactory.train.pt.workflow", "llamafactory.train.dpo.workflow"):
            mod = _try_import(mod_name)
            if mod is not None and hasattr(mod, "load_model"):
                self._set(mod, "load_model", patched)


class CreateRefModelPatch(_AttrPatch):
    """`create_ref_model(model_args, finetuning_args, add_valuehead=False)`: the DPO reference is a second engine-built
    model with the policy's plan.  With `ref_model` unset it is created without loading weights and the DPO trainer
    copies the policy's shards into it; with `ref_model` set it loads that checkpoint."""

    name = "create_ref_model"

    def __init__(self, adapter: Any) -> None:
        super().__init__()
        self.adapter = adapter

    def _patch(self, engine=None) -> None:
        adapter = self.adapter

        def patched(model_args, finetuning_args, add_valuehead=False):
            if add_valuehead:
                raise NotImplementedError("value-head reference models are not engine-backed")
            if not getattr(finetuning_args, "use_ref_model", True):
                return None
            eng = adapter.engine
            path = getattr(finetuning_args, "ref_model", None)
            if path is None:
                ref = eng.build_model(model_args.model_name_or_path, load_weights=False)
            else:
                ref = eng.build_model(path)
            ref.requires_grad_(False)
            return ref.eval()

        for mod_name in ("llamafactory.train.trainer_utils", "llamafactory.train.dpo.workflow", "llamafactory.train.kto.workflow"):
            mod = _try_import(mod_name)
            if mod is not None and hasattr(mod, "create_ref_model"):
                self._set(mod, "create_ref_model", patched)


class TrainerClassPatch(_AttrPatch):
    name = "trainer_class"
    targets = {"sft": [("llamafactory.train.sft.trainer", "CustomSeq2SeqTrainer"), ("llamafactory.train.sft.workflow", "CustomSeq2SeqTrainer")],
               "pt": [("llamafactory.train.pt.trainer", "CustomTrainer"), ("llamafactory.train.pt.workflow", "CustomTrainer")],
               "dpo": [("llamafactory.train.dpo.trainer", "CustomDPOTrainer"), ("llamafactory.train.dpo.workflow", "CustomDPOTrainer")]}

    def __init__(self, adapter: Any) -> None:
        super().__init__()
        self.adapter = adapter

    def _patch(self, engine=None) -> None:
        from .trainer import make_torchturbo_trainer

        made: dict[tuple[str, type], type] = {}
        for stage, places in self.targets.items():
            for mod_name, cls_name in places:
                mod = _try_import(mod_name)
                if mod is None or not hasattr(mod, cls_name):
                    continue
                base = getattr(mod, cls_name)
                key = (stage, base)
                if key not in made:
                    made[key] = make_torchturbo_trainer(base, engine, stage)
                self._set(mod, cls_name, made[key])


class AcceleratorPatch(_AttrPatch):
    """The model arrives sharded.  accelerate must not shard or move it again, must not pick its own FSDP plugin, must
    clip through the engine (the global norm spans FSDP shards and EP-local experts), and `backward` is plain."""

    name = "accelerator"

    def _patch(self, engine=None) -> None:
        acc = _try_import("accelerate")
        if acc is None:
            return
        A = acc.Accelerator
        orig_prepare = A.prepare

        def prepare(self_, *args, **kwargs):
            if getattr(self_, "is_fsdp2", False) or getattr(getattr(self_, "state", None), "fsdp_plugin", None) is not None:
                raise RuntimeError("accelerate's own FSDP must be off (drop --fsdp / FSDP plugin options): the engine "
                                   "has already sharded the model")
            return orig_prepare(self_, *args, **kwargs)

        def prepare_model(self_, model, device_placement=None, evaluation_mode=False):
            if model not in getattr(self_, "_models", []):
                self_._models.append(model)
            return model

        def clip_grad_norm_(self_, parameters, max_norm, norm_type=2):
            if engine is None or float(norm_type) != 2.0:
                raise RuntimeError("only the L2 norm is supported for engine-backed clipping")
            model = getattr(engine, "_model", None) or (self_._models[0] if getattr(self_, "_models", None) else None)
            return engine.clip_grad_norm_(model, max_norm)

        def backward(self_, loss, **kwargs):
            ga = getattr(self_, "gradient_accumulation_steps", 1)
            if ga and ga > 1 and not kwargs.pop("_tt_prescaled", True):
                loss = loss / ga
            loss.backward(**{k: v for k, v in kwargs.items() if k in ("retain_graph", "inputs")})

        self._set(A, "prepare", prepare)
        self._set(A, "prepare_model", prepare_model)
        self._set(A, "clip_grad_norm_", clip_grad_norm_)
        self._set(A, "backward", backward)


def find_base_model_class(model: Any) -> type | None:
    """The first `PreTrainedModel` subclass with `register_for_auto_class` under PEFT / FSDP / checkpoint wrappers:
    tries the instance chain (`base_model`, `model`, `module`, `_orig_mod`) and then the class MRO."""
    seen = set()
    obj = model
    while obj is not None and id(obj) not in seen:
        seen.add(id(obj))
        for cls in type(obj).__mro__:
            if "register_for_auto_class" in cls.__dict__ or (hasattr(cls, "register_for_auto_class") and
                                                             cls.__name__ not in ("FSDPModule",) and
                                                             not cls.__name__.startswith(("FSDP", "Peft"))):
                if hasattr(cls, "register_for_auto_class"):
                    return cls
        nxt = None
        for attr in ("base_model", "model", "module", "_orig_mod"):
            cand = getattr(obj, attr, None)
            if cand is not None and cand is not obj and hasattr(cand, "parameters"):
                nxt = cand
                break
        obj = nxt
    return None


class RegisterAutoclassPatch(_AttrPatch):
    name = "register_autoclass"

    def _patch(self, engine=None) -> None:
        def patched(config, model, tokenizer):
            auto_map = getattr(config, "auto_map", None) or {}
            if "AutoConfig" in auto_map and hasattr(type(config), "register_for_auto_class"):
                type(config).register_for_auto_class()
            if "AutoModelForCausalLM" in auto_map:
                direct = "register_for_auto_class" in dir(type(model)) and not type(model).__name__.startswith("FSDP")
                cls = type(model) if direct else find_base_model_class(model)
                if cls is not None:
                    cls.register_for_auto_class()
                else:
                    logger.warning_rank0("no PreTrainedModel class found under %s; auto_map is not registered", type(model).__name__)
            init_kwargs = getattr(tokenizer, "init_kwargs", {}) or {}
            if "AutoTokenizer" in (init_kwargs.get("auto_map") or {}) and hasattr(type(tokenizer), "register_for_auto_class"):
                type(tokenizer).register_for_auto_class()

        for mod_name in ("llamafactory.model.model_utils.misc", "llamafactory.model.loader", "llamafactory.model.patcher"):
            mod = _try_import(mod_name)
            if mod is not None and hasattr(mod, "register_autoclass"):
                self._set(mod, "register_autoclass", patched)


class LogCallbackPatch(_AttrPatch):
    """`LogCallback.on_log` hands `_write_log` to a thread pool; by the time it runs, the trainer state may belong to a
    later step.  The scalar `grad_norm` of *this* log call is stashed on the callback first and merged into the
    record the worker writes."""

    name = "log_callback"

    def _patch(self, engine=None) -> None:
        cb = _try_import("llamafactory.train.callbacks")
        if cb is None or not hasattr(cb, "LogCallback"):
            return
        L = cb.LogCallback
        orig_on_log, orig_write = L.on_log, getattr(L, "_write_log", None)
        if orig_write is None:
            return

        def on_log(self_, args, state, control, **kwargs):
            last = state.log_history[-1] if getattr(state, "log_history", None) else {}
            gn = (kwargs.get("logs") or {}).get("grad_norm", last.get("grad_norm"))
            self_._tt_grad_norm = float(gn) if gn is not None else None
            return orig_on_log(self_, args, state, control, **kwargs)

        def write_log(self_, output_dir, logs):
            gn = getattr(self_, "_tt_grad_norm", None)
            if gn is not None and isinstance(logs, dict) and "grad_norm" not in logs:
                logs = dict(logs, grad_norm=round(gn, 4))
            return orig_write(self_, output_dir, logs)

        self._set(L, "on_log", on_log)
        self._set(L, "_write_log", write_log)


class PretrainProcessorPatch(_AttrPatch):
    """Stock pre-training preprocessing drops images.  Batches that carry `_images` are tokenised with the template's
    multimodal plugin and packed so that no `[vision_start .. vision_end]` span is cut."""

    name = "pretrain_processor"

    def _patch(self, engine=None) -> None:
        mod = _try_import("llamafactory.data.processor.pretrain")
        if mod is None or not hasattr(mod, "PretrainDatasetProcessor"):
            return
        P = mod.PretrainDatasetProcessor
        orig = P.preprocess_dataset

        def patched(self_, examples):
            images = examples.get("_images")
            if not images or not any(images):
                return orig(self_, examples)
            tok = self_.tokenizer
            plugin = getattr(self_.template, "mm_plugin", None)
            start = tok.convert_tokens_to_ids(getattr(plugin, "vision_bos_token", "<|vision_start|>"))
            end = tok.convert_tokens_to_ids(getattr(plugin, "vision_eos_token", "<|vision_end|>"))

            def tokenize(messages, media):
                text = messages[0]["content"] if isinstance(messages, list) else str(messages)
                if plugin is not None and media:
                    msgs = plugin.process_messages([{"role": "user", "content": text}], media, [], [], self_.processor)
                    text = msgs[0]["content"]
                return tok(text, add_special_tokens=False)["input_ids"]

            return preprocess_multimodal_pretrain(tokenize, examples, self_.data_args.cutoff_len, start, end,
                                                  eos_token_id=tok.eos_token_id)

        self._set(P, "preprocess_dataset", patched)


ENGINE_PATCHES = (PackedInputCollatorPatch, AcceleratorPatch, RegisterAutoclassPatch, LogCallbackPatch, PretrainProcessorPatch)
ADAPTER_PATCHES = (LoadModelPatch, CreateRefModelPatch, TrainerClassPatch)
