"""`qwen3_5_moe_text`: the text-only Qwen3.5 MoE causal LM (no vision tower, flat text config).  Module names keep the
`model.language_model.*` prefix, so a multimodal checkpoint loads with the tower keys ignored; a text-only checkpoint,
whose decoder sits directly under `model.` (`model.layers.*`, `mtp.*`: what models/qwen3_5_moe_text/
modeling_qwen3_5_moe_text.py:27-33 of the reference reads and writes), is recognised by its names and saved back in the
same style.  Plan as models/qwen3_5_moe_text/parallel_plan.py of the reference: the MoE plan without the vision entries."""
from __future__ import annotations

from dataclasses import replace

from ...engine.metrics.flops import MoELLMFlops
from ..base import TurboModel
from ..qwen3_5.model import Qwen3_5TurboMixin
from ..qwen3_5.modeling import Qwen3_5ForConditionalGenerationBase
from ..qwen3_5_moe.model import Qwen3_5MoeInner, Qwen3_5MoeTextConfig, get_parallel_plan
from ..registry import register_model
from ..weight_converter import FusedExpertWeightConverter


class Qwen3_5MoeTextOnlyConfig(Qwen3_5MoeTextConfig):
    model_type = "qwen3_5_moe_text"

    @property
    def text_config(self):
        return self

    @property
    def dtype(self):
        return getattr(self, "torch_dtype", None)

    @dtype.setter
    def dtype(self, v):
        self.torch_dtype = v


class Qwen3_5MoeTextWeightConverter(FusedExpertWeightConverter):
    """Fused-expert rules plus the choice of prefix: `model.language_model.` (multimodal checkpoints) or `model.`
    (text-only ones, and models built without a checkpoint)."""

    NESTED = "model.language_model."

    def __init__(self, model, parallel_context=None, model_path=None):
        super().__init__(model, parallel_context, model_path)
        infos = self.checkpoint_info.tensor_infos if self.checkpoint_info else {}
        self.flat = not any(k.startswith(self.NESTED) for k in infos)

    def _style(self, key: str) -> str:
        return "model." + key[len(self.NESTED):] if self.flat and key.startswith(self.NESTED) else key

    def _fused_in_checkpoint(self, key: str) -> bool:
        return super()._fused_in_checkpoint(self._style(key))

    def load_recipe(self, name: str):
        rec = super().load_recipe(name)
        return rec if rec is None else replace(rec, sources=[self._style(s) for s in rec.sources])

    def to_hf_tensors(self, name, tensor, expert_offset=None):
        return {self._style(k): v for k, v in super().to_hf_tensors(name, tensor, expert_offset).items()}


@register_model("qwen3_5_moe_text")
class TurboQwen3_5MoeTextForCausalLM(Qwen3_5TurboMixin, TurboModel, Qwen3_5ForConditionalGenerationBase):
    config_class = Qwen3_5MoeTextOnlyConfig
    inner_cls = Qwen3_5MoeInner
    with_vision = False
    multimodal_input_keys = ()

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan(False)

    def get_weight_converter(self, parallel_context, model_path=None):
        return Qwen3_5MoeTextWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return MoELLMFlops
