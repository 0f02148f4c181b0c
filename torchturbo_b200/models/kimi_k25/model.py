"""`kimi_k25`: Kimi-K2.5, a DeepSeek-V3 language model (MLA + sigmoid group-limited MoE with shared experts) behind
the MoonViT tower (`vision.py`) whose merged, projected patch features replace the media placeholder tokens.

Module tree and parameter names as in models/kimi_k25/modeling_kimi_k25.py:901-925 of the reference: `vision_tower`
(MoonViT), `mm_projector` (patch-merger MLP) and `language_model` (`.model`, `.lm_head`), so a published checkpoint
loads tower, projector and decoder by name.  Plan (models/kimi_k25/parallel_plan.py:60-133): experts on the
expert-data-parallel mesh, MoE blocks rebuilt EP-aware, decoder layers and tower blocks checkpointed, the tower
world-sharded with vision balancing; Ulysses attention is bound per attention instance.  Muon recipe with MLA QK-clip
as for the other MLA families."""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ...engine.metrics.flops import VLMFlops
from ...parallel import FSDPPlanSpec, VisionBalanceMode, VisionBalanceSpec
from ..base import TurboVLMModel
from ..config import ModelConfig, NestedDtype
from ..modules.deepseek import DeepseekV3Config, DeepseekV3ForCausalLMBase, DeepseekWeightConverter, deepseek_plan
from ..modules.transformer import CausalLMOutput
from ..qwen3_5.modeling import as_dtype
from ..registry import register_model
from .vision import MoonViT, MoonViTConfig, PatchMergerMLP, TemporalPoolVisionBalanceIO, init_moonvit


class KimiK25Config(NestedDtype, ModelConfig):
    model_type = "kimi_k25"
    _defaults = dict(media_placeholder_token_id=163605, pad_token_id=0, ignore_index=-100, tie_word_embeddings=False,
                     initializer_range=0.02)

    def __init__(self, text_config=None, vision_config=None, **kw):
        super().__init__(**kw)
        self.text_config = text_config if isinstance(text_config, ModelConfig) else DeepseekV3Config(**(text_config or {}))
        if not isinstance(vision_config, ModelConfig):
            vc = dict(vision_config or {})
            vc.setdefault("text_hidden_size", self.text_config.hidden_size)
            vision_config = MoonViTConfig(**vc)
        self.vision_config = vision_config
        self._adopt_dtype()
        for k in ("hidden_size", "vocab_size", "num_hidden_layers", "num_attention_heads", "n_routed_experts",
                  "moe_intermediate_size", "num_experts"):
            setattr(self, k, getattr(self.text_config, k))
        self.image_token_id = self.media_placeholder_token_id



class KimiK25ForConditionalGenerationBase(nn.Module):
    def __init__(self, config: Any):
        super().__init__()
        self.config = config
        dtype = as_dtype(config.dtype)
        vc = config.vision_config
        self.vision_tower = MoonViT(vc, dtype)
        self.mm_projector = PatchMergerMLP(vc, dtype) if vc.mm_projector_type == "patchmerger" else nn.Identity()
        self.language_model = DeepseekV3ForCausalLMBase(config.text_config)
        if not any(p.is_meta for p in self.vision_tower.parameters()):
            init_moonvit(self.vision_tower, self.mm_projector, config.initializer_range)

    @property
    def lm_head(self):
        return self.language_model.lm_head

    def tie_weights(self) -> None:
        self.language_model.tie_weights()

    @property
    def all_tied_weights_keys(self):
        return {f"language_model.{k}": f"language_model.{v}" for k, v in self.language_model.all_tied_weights_keys.items()}

    def fuse_media(self, input_ids, pixel_values, grid_thw):
        emb = self.language_model.model.embed_tokens(input_ids)
        if pixel_values is None or pixel_values.shape[0] == 0:        # no media in this rank's row
            v_in, grid = self.vision_tower.dummy_inputs(emb.device, emb.dtype)
            return emb + 0.0 * self.mm_projector(self.vision_tower(v_in, grid_thw=grid)).sum()
        # patches arrive as [L, 3, p, p]; the tower (and the balancer in front of it) works on flat rows
        feats = self.mm_projector(self.vision_tower(pixel_values.reshape(pixel_values.shape[0], -1), grid_thw=grid_thw))
        mask = input_ids == self.config.media_placeholder_token_id
        n = int(mask.sum())
        if n == 0:
            return emb + 0.0 * feats.sum()
        if n != feats.shape[0]:
            raise ValueError(f"{n} media placeholder tokens but {feats.shape[0]} media features")
        return emb.masked_scatter(mask.unsqueeze(-1), feats.to(emb.dtype))

    def forward(self, input_ids=None, position_ids=None, pixel_values=None, grid_thws=None, image_grid_thw=None,
                inputs_embeds=None, skip_lm_head=False, **kw):
        grid = grid_thws if grid_thws is not None else image_grid_thw
        if inputs_embeds is None:
            inputs_embeds = self.fuse_media(input_ids, pixel_values, grid)
        out = self.language_model(input_ids=None, position_ids=position_ids, inputs_embeds=inputs_embeds,
                                  skip_lm_head=skip_lm_head, global_input_ids=input_ids, **kw)
        return CausalLMOutput(out)


def get_parallel_plan():
    plan = deepseek_plan("language_model.model")
    plan.plan.update({
        "vision_tower.encoder.blocks.*": FSDPPlanSpec(activation_checkpoint=True),
        "vision_tower": FSDPPlanSpec(standalone_world_shard=True, vision_balance=VisionBalanceSpec(
            mode=VisionBalanceMode.PATCH_SQ, io=TemporalPoolVisionBalanceIO(2))),
        "mm_projector": FSDPPlanSpec(standalone_world_shard=True),
        "language_model.model.embed_tokens": FSDPPlanSpec(standalone_world_shard=True),
        "language_model.lm_head": FSDPPlanSpec(standalone_world_shard=True),
    })
    return plan


@register_model("kimi_k25")
class TurboKimiK25ForConditionalGeneration(TurboVLMModel, KimiK25ForConditionalGenerationBase):
    config_class = KimiK25Config
    multimodal_input_keys = ("pixel_values", "grid_thws", "image_grid_thw")
    vision_tower_module_names = ("vision_tower",)
    multi_modal_projector_module_names = ("mm_projector",)

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan()

    def get_norm(self):
        return self.language_model.model.norm

    def get_lm_head(self):
        return self.language_model.lm_head

    def get_input_embeddings(self):
        return self.language_model.model.embed_tokens

    def get_language_model(self):
        return self.language_model.model

    def get_sequence_parallel_input_slicing_spec(self):
        from ..modules.attention.ulysses import SequenceParallelInputSlicingSpec

        lm = self.language_model
        return SequenceParallelInputSlicingSpec(lm, type(lm).forward)

    def on_parallelized(self, parallel_context) -> None:
        sp = parallel_context["sp"]
        self.language_model.model.set_sequence_parallel(sp["sp_group"], sp["sp_size"], sp["sp_rank"])

    def on_materialized(self) -> None:
        self.language_model.model.rotary_emb.reset(self.language_model.lm_head.weight.device)
        self.tie_weights()

    def get_weight_converter(self, parallel_context, model_path=None):
        return DeepseekWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return VLMFlops

    def get_optimizer_recipe(self, optimizer_name: str):
        from ...engine.optimizers.muon import default_decoder_muon_recipe

        if optimizer_name == "muon":
            return default_decoder_muon_recipe(self)
        return super().get_optimizer_recipe(optimizer_name)
