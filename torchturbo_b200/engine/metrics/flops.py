"""Analytic forward-FLOP recipes per model family (matmul FLOPs = 2*m*n*k; attention counts QK^T and PV).

`ComputeProfile` describes one micro-batch (token count and per-sequence lengths); a recipe turns a model
config plus a profile into forward FLOPs.  MFU uses 3x forward, HFU 4x when activations are recomputed
(engine/metrics/mfu_estimator.py:146-177 and engine/metrics/flops.py:19-214 of the reference).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence


@dataclass
class ComputeProfile:
    num_tokens: int
    seq_lens: Sequence[int] = field(default_factory=tuple)   # lengths of the packed sequences
    causal: bool = True
    num_image_patches: Sequence[int] = field(default_factory=tuple)  # patches per image (VLM)

    @classmethod
    def from_inputs(cls, inputs: dict[str, Any]) -> "ComputeProfile":
        ids = inputs.get("input_ids")
        T = int(ids.shape[-1]) if ids is not None else int(inputs["inputs_embeds"].shape[-2])
        cu = inputs.get("cu_seq_lens_q")
        lens = [int(b - a) for a, b in zip(cu[:-1].tolist(), cu[1:].tolist())] if cu is not None else [T]
        patches = []
        grid = inputs.get("image_grid_thw")
        if grid is not None:
            patches = [int(t * h * w) for t, h, w in grid.tolist()]
        return cls(T, lens, True, patches)


def matmul_flops(m: int, n: int, k: int) -> float:
    return 2.0 * m * n * k


def attention_flops(seq_lens: Sequence[int], n_heads: int, head_dim: int, causal: bool, v_head_dim: int | None = None) -> float:
    v_head_dim = v_head_dim or head_dim
    pairs = sum(l * l for l in seq_lens)
    f = 2.0 * pairs * n_heads * (head_dim + v_head_dim)
    return f / 2 if causal else f


class BaseModelFlops:
    def __init__(self, config: Any):
        self.config = config

    def forward_flops(self, profile: ComputeProfile) -> float:
        raise NotImplementedError


class LLMFlops(BaseModelFlops):
    def _attn_proj(self, T):
        c = self.config
        D = c.head_dim
        return matmul_flops(T, (c.num_attention_heads + 2 * c.num_key_value_heads) * D, c.hidden_size) + \
            matmul_flops(T, c.hidden_size, c.num_attention_heads * D)

    def _mlp(self, T, layer_idx):
        c = self.config
        return 3 * matmul_flops(T, c.intermediate_size, c.hidden_size)

    def forward_flops(self, profile: ComputeProfile) -> float:
        c = self.config
        T = profile.num_tokens
        total = 0.0
        for i in range(c.num_hidden_layers):
            total += self._attn_proj(T) + attention_flops(profile.seq_lens, c.num_attention_heads, c.head_dim, profile.causal)
            total += self._mlp(T, i)
        total += matmul_flops(T, c.vocab_size, c.hidden_size)
        return total


class MoELLMFlops(LLMFlops):
    def _mlp(self, T, layer_idx):
        c = self.config
        dense_layers = set(getattr(c, "mlp_only_layers", ()) or ())
        if layer_idx in dense_layers or not getattr(c, "num_experts", 0):
            return super()._mlp(T, layer_idx)
        k = c.num_experts_per_tok
        f = 3 * matmul_flops(T * k, c.moe_intermediate_size, c.hidden_size) + matmul_flops(T, c.num_experts, c.hidden_size)
        shared = getattr(c, "shared_expert_intermediate_size", None)
        if shared:
            f += 3 * matmul_flops(T, shared, c.hidden_size)
        return f


class MlaLLMFlops(MoELLMFlops):
    """Multi-head latent attention: low-rank q / kv projections and separate rope / nope head dims."""

    def _attn_proj(self, T):
        c = self.config
        H, nh = c.hidden_size, c.num_attention_heads
        qk = c.qk_nope_head_dim + c.qk_rope_head_dim
        f = 0.0
        if getattr(c, "q_lora_rank", None):
            f += matmul_flops(T, c.q_lora_rank, H) + matmul_flops(T, nh * qk, c.q_lora_rank)
        else:
            f += matmul_flops(T, nh * qk, H)
        f += matmul_flops(T, c.kv_lora_rank + c.qk_rope_head_dim, H)
        f += matmul_flops(T, nh * (c.qk_nope_head_dim + c.v_head_dim), c.kv_lora_rank)
        f += matmul_flops(T, H, nh * c.v_head_dim)
        return f


class VLMFlops(BaseModelFlops):
    """Vision tower (per image, non-causal attention over its patches) + merger + a text recipe."""

    text_flops_class = LLMFlops

    def forward_flops(self, profile: ComputeProfile) -> float:
        c = self.config
        v = c.vision_config
        total = self.text_flops_class(c.text_config).forward_flops(profile)
        P = sum(profile.num_image_patches)
        if P:
            hd = v.hidden_size // v.num_heads
            per_layer = matmul_flops(P, 3 * v.hidden_size, v.hidden_size) + matmul_flops(P, v.hidden_size, v.hidden_size) + \
                2 * matmul_flops(P, v.intermediate_size, v.hidden_size) + \
                attention_flops(profile.num_image_patches, v.num_heads, hd, causal=False)
            total += v.depth * per_layer
            patch_in = v.in_channels * v.temporal_patch_size * v.patch_size ** 2
            total += matmul_flops(P, v.hidden_size, patch_in)
            merge = v.spatial_merge_size ** 2
            total += matmul_flops(P // merge, v.hidden_size * merge, v.hidden_size * merge) + \
                matmul_flops(P // merge, v.out_hidden_size, v.hidden_size * merge)
        return total
