"""Qwen3-style dense decoder (GQA, per-head QK RMSNorm, RoPE, SwiGLU) on packed inputs.

Parameter names follow the Hugging Face checkpoint layout except for the fused projections
(`self_attn.qkv_proj`, `mlp.gate_up_proj`), which the weight converter splits/joins.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ...ops import ops
from ..config import ModelConfig
from ..modules.transformer import CausalLMOutput, DecoderLayer, DenseMLP, RMSNorm, RotaryEmbedding, init_weights


class Qwen3Config(ModelConfig):
    model_type = "qwen3"
    _defaults = dict(
        vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
        num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False,
        max_position_embeddings=40960, attention_bias=False, initializer_range=0.02, qk_norm=True, torch_dtype="bfloat16",
        hidden_act="silu",
    )


class Qwen3Model(nn.Module):
    def __init__(self, config: Any, dtype=None):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, dtype=dtype)
        self.layers = nn.ModuleList([self._make_layer(config, i, dtype) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)
        self.rotary_emb = RotaryEmbedding(config.head_dim, config.rope_theta)

    def _make_layer(self, config, i, dtype):
        return DecoderLayer(config, i, DenseMLP(config.hidden_size, config.intermediate_size, dtype), dtype)

    def forward(self, input_ids=None, position_ids=None, inputs_embeds=None, cu_seq_lens_q=None, max_length_q=None,
                **_unused):
        """Packed row in, hidden states `[1, T_local, H]` out.  `cu_seq_lens_q` / `max_length_q` describe the
        global sequence (they are not sliced under sequence parallelism)."""
        if inputs_embeds is None:
            inputs_embeds = self.embed_tokens(input_ids)
        h = inputs_embeds.reshape(-1, inputs_embeds.shape[-1])
        T = h.shape[0]
        if position_ids is None:
            position_ids = torch.arange(T, device=h.device)
        cos, sin = self.rotary_emb(position_ids.reshape(-1)[-T:] if position_ids.dim() <= 2 else position_ids[0].reshape(-1))
        if cu_seq_lens_q is None:
            cu_seq_lens_q = torch.tensor([0, T], dtype=torch.int32)
            max_length_q = T
        ids = input_ids.reshape(-1) if input_ids is not None else None
        res = None
        for layer in self.layers:
            h, res = layer(h, res, cos, sin, cu_seq_lens_q, max_length_q, ids)
        h, _ = self.norm(h, res)
        return h.unsqueeze(0)


class LMHead(nn.Linear):
    """Output projection.  Called as a module (never through `.weight`) so that FSDP's forward hooks gather
    the sharded weight; with `labels` it runs the fused projection + cross entropy and returns the loss sum."""

    def forward(self, hidden, labels=None, chunk_size: int = 1024):
        if labels is None:
            return ops.linear(hidden, self.weight)
        return ops.linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), self.weight, labels.reshape(-1),
                                        chunk_size=chunk_size)


class Qwen3ForCausalLMBase(nn.Module):
    """Causal LM head on top of a decoder; shared by the dense and MoE model classes."""

    model_cls = Qwen3Model

    def __init__(self, config: Any):
        super().__init__()
        self.config = config
        dtype = getattr(config, "dtype", None) or getattr(config, "torch_dtype", None)
        if isinstance(dtype, str):
            dtype = getattr(torch, dtype.replace("torch.", ""))
        self.model = self.model_cls(config, dtype)
        self.lm_head = LMHead(config.hidden_size, config.vocab_size, bias=False, dtype=dtype)
        self.init_weights()
        self.tie_weights()

    def init_weights(self) -> None:
        if not any(p.is_meta for p in self.parameters()):
            init_weights(self, getattr(self.config, "initializer_range", 0.02))

    def tie_weights(self) -> None:
        if getattr(self.config, "tie_word_embeddings", False):
            self.lm_head.weight = self.model.embed_tokens.weight

    @property
    def all_tied_weights_keys(self) -> dict[str, str]:
        return {"lm_head.weight": "model.embed_tokens.weight"} if getattr(self.config, "tie_word_embeddings", False) else {}

    def forward(self, input_ids=None, position_ids=None, inputs_embeds=None, cu_seq_lens_q=None, cu_seq_lens_k=None,
                max_length_q=None, max_length_k=None, skip_lm_head: bool = False, **kwargs):
        hidden = self.model(input_ids=input_ids, position_ids=position_ids, inputs_embeds=inputs_embeds,
                            cu_seq_lens_q=cu_seq_lens_q, max_length_q=max_length_q, **kwargs)
        out = CausalLMOutput(hidden_states=hidden)
        if not skip_lm_head:
            out["logits"] = self.lm_head(hidden)
        return out
