"""`bailing_moe_v3_vl`: the Bailing-MoE v3 hybrid decoder (MLA + KDA + MoE) with a Qwen-VL style vision tower and a
separate `linear_proj` projector in front of it.

Module tree as in models/bailing_moe_v3_vl/model.py:52-160 of the reference: the decoder's own modules sit directly
under `model` (`model.layers`, `model.embed_tokens`, `model.norm`), the tower under `model.visual`, the projector at
top level.  Plan (models/bailing_moe_v3_vl/parallel_plan.py:42-67): experts on the expert-data-parallel mesh, MoE
blocks rebuilt EP-aware, layers and tower blocks checkpointed, tower world-sharded with vision balancing, projector,
embeddings and head as standalone units.  Sequence-parallel slicing happens at the text entry
(`model.forward_text`) on the fused embeddings and positions; the prediction depths receive the global ids."""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ...engine.metrics.flops import VLMFlops
from ...ops import ops
from ...parallel import FSDPPlanSpec, VisionBalanceMode, VisionBalanceSpec
from ..bailing_hybrid.model import BailingWeightConverter, get_parallel_plan as text_plan
from ..bailing_hybrid.modeling import BailingModel, BailingMoeV3Config
from ..base import TurboVLMModel
from ..config import ModelConfig, NestedDtype
from ..modules.hybrid import run_nextn_layers
from ..modules.transformer import CausalLMOutput
from ..modules.vision import GridVisionBalanceIO
from ..qwen3.modeling import LMHead
from ..qwen3_5.modeling import as_dtype, init_hybrid_weights
from ..qwen3_vl.modeling import Qwen3VLVisionConfig, VisionTower
from ..registry import register_model


class BailingMoeV3VLConfig(NestedDtype, ModelConfig):
    model_type = "bailing_moe_v3_vl"
    _defaults = dict(image_patch_token=157157, video_patch_token=157175, tie_word_embeddings=False, initializer_range=0.02)

    def __init__(self, text_config=None, vision_config=None, **kw):
        super().__init__(**kw)
        self.text_config = text_config if isinstance(text_config, ModelConfig) else BailingMoeV3Config(**(text_config or {}))
        if not isinstance(vision_config, ModelConfig):
            vc = dict(vision_config or {})
            vc.setdefault("out_hidden_size", 3584)
            # DeepStack features of this tower are cut off before the projector (modeling_bailing_moe_v3_vl.py:2514-2520
            # of the reference keeps the first `vision_out_dim` columns), so their mergers are not built
            vc["deepstack_visual_indexes"] = ()
            vision_config = Qwen3VLVisionConfig(**{k: v for k, v in vc.items() if not k.startswith("_")})
        self.vision_config = vision_config
        self._adopt_dtype()
        for k in ("hidden_size", "vocab_size", "num_hidden_layers", "num_attention_heads", "num_experts",
                  "moe_intermediate_size", "head_dim"):
            setattr(self, k, getattr(self.text_config, k))
        self.image_token_id = self.image_patch_token



class BailingVLModel(BailingModel):
    """The text decoder plus the tower as a child module, so checkpoint prefixes stay `model.*`."""

    def __init__(self, config, dtype=None):
        super().__init__(config.text_config, dtype)
        self.visual = VisionTower(config.vision_config, dtype)

    def forward_text(self, inputs_embeds=None, position_ids=None, cu_seq_lens_q=None, max_length_q=None, input_ids=None):
        return BailingModel.forward(self, input_ids=input_ids, position_ids=position_ids, inputs_embeds=inputs_embeds,
                                    cu_seq_lens_q=cu_seq_lens_q, max_length_q=max_length_q, return_context=True)


class _Projector(nn.Sequential):
    """`Linear - GELU - Linear` under the checkpoint's names (`linear_proj.0`, `linear_proj.2`), evaluated with the fused
    bias + activation operator.  It is called as a module, never read parameter by parameter from outside: as an FSDP
    unit of its own its weights are only gathered inside its forward."""

    def forward(self, feats):
        a, b = self[0], self[2]
        return ops.bias_act(ops.linear(ops.bias_act(ops.linear(feats, a.weight), a.bias, "gelu"), b.weight), b.bias)


class BailingMoeV3VLForConditionalGenerationBase(nn.Module):
    def __init__(self, config: Any):
        super().__init__()
        self.config = config
        dtype = as_dtype(config.dtype)
        tc, vc = config.text_config, config.vision_config
        self.model = BailingVLModel(config, dtype)
        # `disable_merger_proj`: the tower hands over the joined 2x2 patch rows and this projector does all the mapping
        vin = vc.hidden_size * vc.spatial_merge_size ** 2 if getattr(vc, "disable_merger_proj", False) else vc.out_hidden_size
        self.linear_proj = _Projector(nn.Linear(vin, tc.hidden_size, bias=True, dtype=dtype), nn.GELU(),
                                      nn.Linear(tc.hidden_size, tc.hidden_size, bias=True, dtype=dtype))
        self.lm_head = LMHead(tc.hidden_size, tc.vocab_size, bias=False, dtype=dtype)
        n = int(getattr(tc, "num_nextn_predict_layers", 0) or 0)
        self.mtp = nn.ModuleList([self.model.make_nextn_layer(tc.num_hidden_layers + i, dtype) for i in range(n)]) if n else None
        if not any(p.is_meta for p in self.parameters()):
            init_hybrid_weights(self, config.initializer_range)

    def tie_weights(self) -> None:
        if getattr(self.config, "tie_word_embeddings", False):
            self.lm_head.weight = self.model.embed_tokens.weight

    @property
    def all_tied_weights_keys(self):
        return {"lm_head.weight": "model.embed_tokens.weight"} if getattr(self.config, "tie_word_embeddings", False) else {}

    def project(self, feats):
        return self.linear_proj(feats)

    def fuse_media(self, input_ids, pixel_values, grid):
        emb = self.model.embed_tokens(input_ids)
        visual = self.model.visual
        if pixel_values is None or pixel_values.shape[0] == 0:        # no media in this rank's row
            v_in, g = visual.dummy_inputs(emb.device, emb.dtype)
            return emb + 0.0 * self.project(visual(v_in, grid_thw=g)).sum()
        feats = self.project(visual(pixel_values, grid_thw=grid))
        mask = (input_ids == self.config.image_patch_token) | (input_ids == self.config.video_patch_token)
        n = int(mask.sum())
        if n == 0:
            return emb + 0.0 * feats.sum()
        if n != feats.shape[0]:
            raise ValueError(f"{n} media placeholder tokens but {feats.shape[0]} media features")
        return emb.masked_scatter(mask.unsqueeze(-1), feats.to(emb.dtype))

    def forward(self, input_ids=None, position_ids=None, pixel_values=None, image_grid_thw=None, inputs_embeds=None,
                cu_seq_lens_q=None, cu_seq_lens_k=None, max_length_q=None, max_length_k=None, skip_lm_head=False, **kw):
        if inputs_embeds is None:
            inputs_embeds = self.fuse_media(input_ids, pixel_values, image_grid_thw)
        m = self.model
        hidden, ctx = m.forward_text(inputs_embeds=inputs_embeds, position_ids=position_ids, cu_seq_lens_q=cu_seq_lens_q,
                                     max_length_q=max_length_q, input_ids=input_ids)
        out = CausalLMOutput(hidden_states=hidden)
        if self.mtp is not None and self.training and input_ids is not None:
            sp_slice = None
            if m.sp_size > 1:
                Tl = hidden.shape[1]
                sp_slice = lambda e: e[m.sp_rank * Tl:(m.sp_rank + 1) * Tl]       # noqa: E731
            hs = run_nextn_layers(self.mtp, input_ids, hidden[0], m.embed_tokens, ctx,
                                  getattr(self.config.text_config, "pad_token_id", 0) or 0, sp_slice)
            out["mtp_hidden_states"] = [h.unsqueeze(0) for h in hs]
        if not skip_lm_head:
            out["logits"] = self.lm_head(hidden)
            if out.get("mtp_hidden_states"):
                out["mtp_logits"] = [self.lm_head(h) for h in out["mtp_hidden_states"]]
        return out


class BailingVLWeightConverter(BailingWeightConverter):
    """Expert counts live in the nested text config."""

    def __init__(self, model, parallel_context=None, model_path=None):
        super().__init__(model, parallel_context, model_path)
        tc = model.config.text_config
        self.num_experts = tc.num_experts
        self.num_local_experts = self.num_experts // self.ep_size if self.num_experts else 0


def get_parallel_plan():
    plan = text_plan("model")
    plan.plan.update({
        "model.visual.blocks.*": FSDPPlanSpec(activation_checkpoint=True),
        "model.visual": FSDPPlanSpec(standalone_world_shard=True, vision_balance=VisionBalanceSpec(
            mode=VisionBalanceMode.PATCH_SQ, io=GridVisionBalanceIO(2))),
        "linear_proj": FSDPPlanSpec(standalone_world_shard=True),
        "model.embed_tokens": FSDPPlanSpec(standalone_world_shard=True),
        "lm_head": FSDPPlanSpec(standalone_world_shard=True),
    })
    return plan


@register_model("bailing_moe_v3_vl")
class TurboBailingMoeV3VLForConditionalGeneration(TurboVLMModel, BailingMoeV3VLForConditionalGenerationBase):
    config_class = BailingMoeV3VLConfig
    multimodal_input_keys = ("pixel_values", "image_grid_thw")
    vision_tower_module_names = ("model.visual",)
    multi_modal_projector_module_names = ("linear_proj",)

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan()

    def get_norm(self):
        return self.model.norm

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_language_model(self):
        return self.model

    def get_sequence_parallel_input_slicing_spec(self):
        from ..modules.attention.ulysses import SequenceParallelInputSlicingSpec

        return SequenceParallelInputSlicingSpec(self.model, BailingVLModel.forward_text, forward_name="forward_text",
                                                sliced_inputs=(("inputs_embeds", 1), ("position_ids", -1)))

    def on_parallelized(self, parallel_context) -> None:
        sp = parallel_context["sp"]
        if sp["sp_size"] > 1 and self.config.text_config.num_attention_heads % sp["sp_size"]:
            raise ValueError("attention heads must be divisible by sp_size")
        self.model.set_sequence_parallel(sp["sp_group"], sp["sp_size"], sp["sp_rank"])

    def on_materialized(self) -> None:
        self.model.rotary_emb.reset(self.lm_head.weight.device)
        self.tie_weights()

    def get_weight_converter(self, parallel_context, model_path=None):
        return BailingVLWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return VLMFlops

    def get_optimizer_recipe(self, optimizer_name: str):
        from ...engine.optimizers.muon import default_decoder_muon_recipe

        if optimizer_name == "muon":
            return default_decoder_muon_recipe(self)
        return super().get_optimizer_recipe(optimizer_name)
