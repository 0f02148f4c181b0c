"""`qwen3_5_moe_text`: the text-only Qwen3.5 MoE causal LM (no vision tower, flat text config; module names keep the
`model.language_model.*` prefix so multimodal checkpoints load with the tower keys ignored).  Plan as
models/qwen3_5_moe_text/parallel_plan.py of the reference: the MoE plan without the vision entries."""
from __future__ import annotations

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
        return FusedExpertWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return MoELLMFlops
