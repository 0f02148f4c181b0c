"""The contract between the engine and a model (`TurboModel`, `TurboVLMModel`).

A Turbo model is an `nn.Module` that additionally answers the questions the engine asks while building,
sharding, feeding and checkpointing it: its default parallel plan, where sequence-parallel slicing
happens, which parameters belong to which semantic group, how its checkpoint names map to Hugging Face
names, and how many FLOPs a forward pass costs.  The surface mirrors models/base.py:22-362 of the
reference so that model packages written against either are structured the same way.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Iterable, Iterator, Optional

import torch
import torch.nn as nn

from ..engine.config import EngineConfig, ParameterGroup
from ..logging import get_logger

logger = get_logger(__name__)


class TurboModel:
    is_diffusion_model = False
    base_model_prefix = "model"
    config_class: type | None = None

    # ---- structure ---------------------------------------------------------------------------------
    def get_norm(self) -> Optional[nn.Module]:
        """Final normalisation layer (placed in the resident tail FSDP unit)."""
        base = getattr(self, self.base_model_prefix, None) if self.base_model_prefix else None
        norm = getattr(base, "norm", None) if isinstance(base, nn.Module) else None
        return norm if isinstance(norm, nn.Module) else None

    def get_lm_head(self) -> Optional[nn.Module]:
        head = getattr(self, "lm_head", None)
        return head if isinstance(head, nn.Module) else None

    def get_output_embeddings(self) -> Optional[nn.Module]:
        return self.get_lm_head()

    def get_input_embeddings(self) -> Optional[nn.Module]:
        base = getattr(self, self.base_model_prefix, None)
        emb = getattr(base, "embed_tokens", None)
        return emb if isinstance(emb, nn.Module) else None

    # ---- construction ------------------------------------------------------------------------------
    @classmethod
    @contextmanager
    def init_context(cls, config: Any, engine_config: EngineConfig) -> Iterator[None]:
        """Adjust the model config for construction: multi-token-prediction layers are kept only when MTP is
        enabled, and parameters are always created in fp32 (the master copy; bf16 is a compute dtype)."""
        n_mtp = getattr(config, "num_nextn_predict_layers", 0) or 0
        if engine_config.mtp.enabled:
            if n_mtp > 0:
                logger.info_rank0("MTP enabled: %d MTP layer(s) will be built", n_mtp)
            else:
                logger.warning_rank0("MTP is enabled but the model config has no MTP layers")
        elif hasattr(config, "num_nextn_predict_layers") and n_mtp > 0:
            logger.info_rank0("MTP off: stripping %d MTP layer(s); their checkpoint weights are skipped", n_mtp)
            config.num_nextn_predict_layers = 0
        saved = cls._force_config_dtype_float32(config)
        try:
            yield
        finally:
            cls._restore_config_dtype(config, saved)
            if hasattr(config, "num_nextn_predict_layers"):
                config.num_nextn_predict_layers = n_mtp if engine_config.mtp.enabled else config.num_nextn_predict_layers

    @staticmethod
    def _force_config_dtype_float32(config: Any) -> dict[str, Any]:
        state: dict[str, Any] = {}
        for attr in ("dtype", "torch_dtype"):
            if config is not None and hasattr(config, attr):
                state[attr] = getattr(config, attr)
                try:
                    setattr(config, attr, torch.float32)
                except Exception:
                    state.pop(attr)
                break
        return state

    @staticmethod
    def _restore_config_dtype(config: Any, state: dict[str, Any]) -> None:
        for attr, v in state.items():
            setattr(config, attr, v)

    @classmethod
    def get_default_parallel_plan(cls, **kwargs: Any):
        from ..parallel import FSDPParallelPlan

        return FSDPParallelPlan()

    # ---- parallelisation hooks ---------------------------------------------------------------------
    def register_sp_attention_interface(self, sp_info: dict[str, Any]) -> None:
        """Bind the sequence-parallel group to every attention module of the model."""
        for m in self.modules():
            if hasattr(m, "set_sequence_parallel"):
                m.set_sequence_parallel(sp_info["sp_group"], sp_info["sp_size"])

    def on_parallelized(self, parallel_context: dict[str, Any]) -> None:
        self.register_sp_attention_interface(parallel_context["sp"])

    def on_materialized(self) -> None:
        """Called once parameters and buffers live on a real device (rebuild non-persistent buffers here)."""

    def get_moe_runtime_inputs(self, inputs: dict[str, Any], parallel_context: dict[str, Any]):
        """SP-local padding mask derived from the packed boundaries: tokens at or after `cu_seq_lens[-1]`
        are padding (dummy media and SP alignment tails included)."""
        from .modules.attention.ulysses import slice_input_tensor
        from .modules.moe import MoERuntimeInputs

        cu = inputs["cu_seq_lens_q"]
        ids = inputs["input_ids"]
        pos = torch.arange(ids.size(-1), device=ids.device)
        mask = (pos >= int(cu[-1])).unsqueeze(0)
        sp = parallel_context["sp"]
        if sp["sp_size"] > 1:
            mask = slice_input_tensor(mask, 1, sp["sp_group"], sp["sp_rank"])
        return MoERuntimeInputs(padding_mask=mask)

    def get_sequence_parallel_input_slicing_spec(self):
        from .modules.attention.ulysses import SequenceParallelInputSlicingSpec

        return SequenceParallelInputSlicingSpec(self, type(self).forward,
                                                sliced_inputs=(("input_ids", 1), ("position_ids", -1)))

    def on_prepare_inputs(self, inputs: dict[str, Any], *, source_inputs: dict[str, Any] | None = None) -> dict[str, Any]:
        """Enforce the packed-batch contract before SP padding: boundaries travel as `cu_seq_lens_q/k`
        (+ `max_length_q/k`); `attention_mask` batches are rejected."""
        if inputs.get("attention_mask") is not None:
            raise ValueError("training batches must express sequence boundaries with cu_seq_lens_q/k, not attention_mask")
        if inputs.get("cu_seq_lens_q") is None:
            raise ValueError("training batches must be flattened packed inputs with cu_seq_lens_q/k and max_length_q/k")
        return inputs

    # ---- optimisation / checkpoint / metrics -------------------------------------------------------
    def get_parameter_groups(self) -> dict[ParameterGroup, Iterable[tuple[str, nn.Parameter]]]:
        return {ParameterGroup.LANGUAGE_MODEL: self.named_parameters()}

    def get_optimizer_recipe(self, optimizer_name: str):
        raise NotImplementedError(f"{type(self).__name__} does not provide an optimizer recipe for {optimizer_name!r}")

    def get_weight_converter(self, parallel_context: dict[str, Any], model_path: str | None = None):
        from .weight_converter import BaseWeightConverter

        return BaseWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        raise NotImplementedError(f"{type(self).__name__} does not provide an MFU flops recipe")


class TurboVLMModel(TurboModel):
    """Multimodal models: nested text/vision configs, media inputs that stay global under SP, SP slicing
    at the fusion boundary (`inputs_embeds`), and vision / projector / language parameter groups."""

    multimodal_input_keys: tuple[str, ...] = ("pixel_values", "image_grid_thw", "pixel_values_videos", "video_grid_thw")
    vision_module_names: tuple[str, ...] = ("visual",)
    projector_module_names: tuple[str, ...] = ("visual.merger",)
    language_module_names: tuple[str, ...] = ("language_model", "lm_head")

    def on_prepare_inputs(self, inputs, *, source_inputs=None):
        inputs = super().on_prepare_inputs(inputs, source_inputs=source_inputs)
        if source_inputs is not None:
            for k in self.multimodal_input_keys:
                if k in source_inputs and k not in inputs:
                    inputs[k] = source_inputs[k]
        return inputs

    def get_sequence_parallel_input_slicing_spec(self):
        from .modules.attention.ulysses import SequenceParallelInputSlicingSpec

        lm = self.get_language_model()
        return SequenceParallelInputSlicingSpec(lm, type(lm).forward)

    def get_language_model(self) -> nn.Module:
        return getattr(getattr(self, self.base_model_prefix), "language_model")

    @staticmethod
    def _named_parameters_from_modules(root: nn.Module, prefixes: Iterable[str], exclude: Iterable[str] = ()):
        exclude = tuple(exclude)
        for name, p in root.named_parameters():
            if any(name == pre or name.startswith(pre + ".") or f".{pre}." in f".{name}" for pre in prefixes):
                if not any(f".{ex}." in f".{name}" for ex in exclude):
                    yield name, p

    def get_parameter_groups(self):
        return {
            ParameterGroup.VISION_TOWER: self._named_parameters_from_modules(self, self.vision_module_names,
                                                                             self.projector_module_names),
            ParameterGroup.MULTI_MODAL_PROJECTOR: self._named_parameters_from_modules(self, self.projector_module_names),
            ParameterGroup.LANGUAGE_MODEL: self._named_parameters_from_modules(self, self.language_module_names),
        }
