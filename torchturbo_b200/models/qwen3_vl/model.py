"""`qwen3_vl`: ViT tower + Qwen3 decoder as a Turbo VLM with world-pooled vision balancing.

Plan: decoder layers and ViT blocks are checkpointed, `model.visual` is a standalone world-sharded unit whose forward
is wrapped by the vision balancer (`patch_sq` weights by default: ViT attention cost grows with the square of the
patch count), and sequence-parallel slicing happens at the language model entry on `inputs_embeds`, after the media
have been fused into the full row."""
from __future__ import annotations

from ...engine.metrics.flops import VLMFlops
from ...parallel import FSDPParallelPlan, FSDPPlanSpec, VisionBalanceMode, VisionBalanceSpec
from ..base import TurboVLMModel
from ..modules.vision import GridVisionBalanceIO
from ..registry import register_model
from ..weight_converter import BaseWeightConverter
from .modeling import Qwen3VLConfig, Qwen3VLForConditionalGenerationBase


def get_parallel_plan() -> FSDPParallelPlan:
    return FSDPParallelPlan(
        plan={
            "model.language_model.layers.*": FSDPPlanSpec(activation_checkpoint=True),
            "model.visual.blocks.*": FSDPPlanSpec(activation_checkpoint=True),
            "model.visual": FSDPPlanSpec(standalone_world_shard=True,
                                         vision_balance=VisionBalanceSpec(mode=VisionBalanceMode.PATCH_SQ,
                                                                          io=GridVisionBalanceIO(2))),
            "model.language_model.embed_tokens": FSDPPlanSpec(standalone_world_shard=True),
            "lm_head": FSDPPlanSpec(standalone_world_shard=True),
        },
        sp_size=1, ep_size=1,
    )


@register_model("qwen3_vl")
class TurboQwen3VLForConditionalGeneration(TurboVLMModel, Qwen3VLForConditionalGenerationBase):
    config_class = Qwen3VLConfig
    multimodal_input_keys = ("pixel_values", "image_grid_thw")

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan()

    def get_norm(self):
        return self.model.language_model.norm

    def get_input_embeddings(self):
        return self.model.language_model.embed_tokens

    def get_language_model(self):
        return self.model.language_model

    def get_sequence_parallel_input_slicing_spec(self):
        from ..modules.attention.ulysses import SequenceParallelInputSlicingSpec

        lm = self.model.language_model
        return SequenceParallelInputSlicingSpec(lm, type(lm).forward, sliced_inputs=(
            ("inputs_embeds", 1), ("position_ids", -1), ("deepstack_embeds", 2)))

    def on_materialized(self) -> None:
        self.model.language_model.rotary_emb.reset(self.lm_head.weight.device)
        self.tie_weights()

    def get_weight_converter(self, parallel_context, model_path=None):
        return BaseWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return VLMFlops
