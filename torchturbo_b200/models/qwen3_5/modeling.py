"""Qwen3.5: a hybrid decoder (three gated-delta-rule layers for every gated softmax-attention layer), optional
multi-token-prediction head, and a Qwen-VL vision tower feeding image features into the token embeddings.

Layer kinds come from `layer_types` (or `full_attention_interval`), RMSNorm weights are stored as offsets from one,
softmax attention rotates only `partial_rotary_factor` of each head with 3-axis multimodal positions.  Structure and
checkpoint names follow models/qwen3_5/modeling_qwen3_5.py:469-1003,1416-1494,1909-2100 of the reference; dense
projections are stored fused (`mlp.gate_up_proj`) and split by the weight converter.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ..config import ModelConfig, NestedDtype
from ..modules.hybrid import HybridDecoderLayer, HybridModel, MultiTokenPredictor
from ..modules.mixers import GatedDeltaNet, KimiDeltaAttention
from ..modules.transformer import CausalLMOutput, DenseMLP, init_weights
from ..qwen3.modeling import LMHead
from ..qwen3_vl.modeling import Qwen3VLVisionConfig, VisionTower


class Qwen3_5TextConfig(ModelConfig):
    model_type = "qwen3_5_text"
    _defaults = dict(
        vocab_size=248320, hidden_size=4096, intermediate_size=12288, num_hidden_layers=32, num_attention_heads=16,
        num_key_value_heads=4, head_dim=256, rms_norm_eps=1e-6, rope_theta=1e7, partial_rotary_factor=0.25,
        mrope_section=(11, 11, 10), mrope_interleaved=True, attention_bias=False, attn_output_gate=True,
        linear_conv_kernel_dim=4, linear_key_head_dim=128, linear_value_head_dim=128, linear_num_key_heads=16,
        linear_num_value_heads=32, full_attention_interval=4, layer_types=None, mtp_num_hidden_layers=0,
        tie_word_embeddings=False, initializer_range=0.02, hidden_act="silu", torch_dtype="bfloat16", pad_token_id=0,
        norm_one_plus_weight=True,
    )

    def __init__(self, **kw):
        rp = kw.pop("rope_parameters", None) or {}
        for k_src, k_dst in (("rope_theta", "rope_theta"), ("partial_rotary_factor", "partial_rotary_factor"),
                             ("mrope_section", "mrope_section"), ("mrope_interleaved", "mrope_interleaved")):
            if k_src in rp:
                kw[k_dst] = rp[k_src]          # what transformers reads; a top-level key next to it is a leftover default
        super().__init__(**kw)
        if not self.layer_types:
            n = self.full_attention_interval
            self.layer_types = ["full_attention" if (i + 1) % n == 0 else "linear_attention"
                                for i in range(self.num_hidden_layers)]


class Qwen3_5Config(NestedDtype, ModelConfig):
    model_type = "qwen3_5"
    text_config_class = Qwen3_5TextConfig
    _defaults = dict(image_token_id=248056, video_token_id=248057, vision_start_token_id=248053, tie_word_embeddings=False,
                     initializer_range=0.02)
    _mirrored = ("hidden_size", "vocab_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim")

    def __init__(self, text_config=None, vision_config=None, **kw):
        super().__init__(**kw)
        self.text_config = text_config if isinstance(text_config, ModelConfig) else self.text_config_class(**(text_config or {}))
        if not isinstance(vision_config, ModelConfig):
            vc = dict(vision_config or {})
            vc.setdefault("out_hidden_size", self.text_config.hidden_size)
            vision_config = Qwen3VLVisionConfig(**vc)
        self.vision_config = vision_config
        self._adopt_dtype()
        for k in self._mirrored + tuple(getattr(self, "_mirrored_extra", ())):
            if hasattr(self.text_config, k):
                setattr(self, k, getattr(self.text_config, k))



class Qwen3_5TextModel(HybridModel):
    one_plus_weight = True

    def mixer_kind(self, i: int) -> str:
        kind = self.config.layer_types[i] if i < len(self.config.layer_types) else "full_attention"
        return "gated_attention" if kind == "full_attention" else kind

    def make_mlp(self, i: int, dtype) -> nn.Module:
        return DenseMLP(self.config.hidden_size, self.config.intermediate_size, dtype)

    def make_mtp_layer(self, i: int, dtype) -> nn.Module:
        # prediction layers always use softmax attention
        return HybridDecoderLayer(self.config, i, "gated_attention", self.make_mlp(i, dtype), dtype, True)


def init_hybrid_weights(module: nn.Module, std: float) -> None:
    init_weights(module, std)
    for m in module.modules():
        if isinstance(m, nn.Conv1d):
            nn.init.normal_(m.weight, std=std)
        if isinstance(m, (GatedDeltaNet, KimiDeltaAttention)):
            m.reset_parameters_extra()


def as_dtype(dtype):
    return getattr(torch, dtype.replace("torch.", "")) if isinstance(dtype, str) else dtype


class Qwen3_5Inner(nn.Module):
    text_model_cls = Qwen3_5TextModel

    def __init__(self, config, dtype=None, with_vision: bool = True):
        super().__init__()
        if with_vision:
            self.visual = VisionTower(config.vision_config, dtype)
        self.language_model = self.text_model_cls(config.text_config, dtype)


class Qwen3_5ForConditionalGenerationBase(nn.Module):
    inner_cls = Qwen3_5Inner
    with_vision = True

    def __init__(self, config: Any):
        super().__init__()
        self.config = config
        dtype = as_dtype(config.dtype)
        tc = config.text_config
        self.model = self.inner_cls(config, dtype, self.with_vision)
        self.lm_head = LMHead(tc.hidden_size, tc.vocab_size, bias=False, dtype=dtype)
        lm = self.model.language_model
        self.mtp = MultiTokenPredictor(tc, lambda i: lm.make_mtp_layer(i, dtype), dtype, True) \
            if int(getattr(tc, "mtp_num_hidden_layers", 0) or 0) > 0 else None
        if not any(p.is_meta for p in self.parameters()):
            init_hybrid_weights(self, config.initializer_range)
        self.tie_weights()

    def tie_weights(self) -> None:
        if getattr(self.config, "tie_word_embeddings", False):
            self.lm_head.weight = self.model.language_model.embed_tokens.weight

    @property
    def all_tied_weights_keys(self):
        return {"lm_head.weight": "model.language_model.embed_tokens.weight"} \
            if getattr(self.config, "tie_word_embeddings", False) else {}

    def fuse_media(self, input_ids, pixel_values, image_grid_thw):
        emb = self.model.language_model.embed_tokens(input_ids)
        if not self.with_vision:
            return emb
        visual = self.model.visual
        if pixel_values is None or pixel_values.shape[0] == 0:        # no media in this rank's row
            v_in, grid = visual.dummy_inputs(emb.device, emb.dtype)
            return emb + 0.0 * visual(v_in, grid_thw=grid).sum()
        feats = visual(pixel_values, grid_thw=image_grid_thw)
        mask = (input_ids == self.config.image_token_id) | (input_ids == getattr(self.config, "video_token_id", -1))
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
        lm = self.model.language_model
        hidden, ctx = lm(inputs_embeds=inputs_embeds, position_ids=position_ids, cu_seq_lens_q=cu_seq_lens_q,
                         max_length_q=max_length_q, input_ids=input_ids, return_context=True)
        out = CausalLMOutput(hidden_states=hidden)
        if self.mtp is not None and self.training and input_ids is not None:
            sp_slice = None
            if lm.sp_size > 1:
                Tl = hidden.shape[1]
                sp_slice = lambda e: e[lm.sp_rank * Tl:(lm.sp_rank + 1) * Tl]     # noqa: E731
            pad = getattr(self.config.text_config, "pad_token_id", 0) or 0
            hs = self.mtp(input_ids, hidden[0], lm.embed_tokens, ctx, pad, sp_slice)
            out["mtp_hidden_states"] = [h.unsqueeze(0) for h in hs]
        if not skip_lm_head:
            out["logits"] = self.lm_head(hidden)
            if out.get("mtp_hidden_states"):
                out["mtp_logits"] = [self.lm_head(h) for h in out["mtp_hidden_states"]]
        return out
