"""Qwen-VL style vision-language model: a ViT tower over packed image patches, a 2x2 spatial merger that projects
to the language model width, and the Qwen3 decoder consuming `inputs_embeds` with image features written at the
image placeholder tokens.

Shapes of the benchmarked configuration: ViT depth 27, width 1152, 16 heads (head_dim 72), MLP 4304, patch 14,
temporal patch 2, merge 2x2 -> LLM width.  Images are variable-sized; all images of a batch are packed on dim 0
(`pixel_values [sum(t*h*w), 3*2*14*14]`, `image_grid_thw [n_images, 3]`) and attention inside the tower is
non-causal and restricted to each image (packed segments = images).
"""
from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import ops
from ..config import ModelConfig
from ..modules.transformer import CausalLMOutput, init_weights
from ..qwen3.modeling import LMHead, Qwen3Config, Qwen3Model


class Qwen3VLVisionConfig(ModelConfig):
    model_type = "qwen3_vl_vision"
    _defaults = dict(depth=27, hidden_size=1152, num_heads=16, intermediate_size=4304, patch_size=14,
                     temporal_patch_size=2, in_channels=3, spatial_merge_size=2, out_hidden_size=4096,
                     hidden_act="gelu_pytorch_tanh", initializer_range=0.02)


class Qwen3VLConfig(ModelConfig):
    model_type = "qwen3_vl"
    _defaults = dict(image_token_id=151655, video_token_id=151656, vision_start_token_id=151652, tie_word_embeddings=False,
                     initializer_range=0.02)

    def __init__(self, text_config=None, vision_config=None, **kw):
        super().__init__(**kw)
        self.text_config = text_config if isinstance(text_config, ModelConfig) else Qwen3Config(**(text_config or {}))
        vc = dict(vision_config or {}) if not isinstance(vision_config, ModelConfig) else None
        if vc is not None:
            vc.setdefault("out_hidden_size", self.text_config.hidden_size)
            vision_config = Qwen3VLVisionConfig(**vc)
        self.vision_config = vision_config
        for k in ("hidden_size", "vocab_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim"):
            setattr(self, k, getattr(self.text_config, k))

    @property
    def dtype(self):
        return getattr(self.text_config, "dtype", None) or getattr(self.text_config, "torch_dtype", None)

    @dtype.setter
    def dtype(self, v):
        self.text_config.torch_dtype = v
        self.text_config.dtype = v


def vision_rot_pos(grid_thw: torch.Tensor, merge: int, head_dim: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """2-D rotary tables `[P, head_dim/2]`: half of the rotary pairs follow the patch row, half the column, with patches
    ordered merge-window-major exactly as the processor emits them."""
    hs, ws = [], []
    for t, h, w in grid_thw.tolist():
        hp = torch.arange(h).unsqueeze(1).expand(h, w)
        wp = torch.arange(w).unsqueeze(0).expand(h, w)

        def win(x):
            return x.reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).reshape(-1)

        hs.append(win(hp).repeat(t))
        ws.append(win(wp).repeat(t))
    hpos, wpos = torch.cat(hs).to(device).float(), torch.cat(ws).to(device).float()
    n = head_dim // 4
    inv = 1.0 / (10000.0 ** (torch.arange(0, n, device=device).float() / n))
    ang = torch.cat([hpos[:, None] * inv[None], wpos[:, None] * inv[None]], dim=-1)   # [P, head_dim/2]
    return ang.cos(), ang.sin()


class VisionBlock(nn.Module):
    def __init__(self, cfg, dtype=None):
        super().__init__()
        H = cfg.hidden_size
        self.n_heads, self.head_dim = cfg.num_heads, H // cfg.num_heads
        self.norm1, self.norm2 = nn.LayerNorm(H, eps=1e-6, dtype=dtype), nn.LayerNorm(H, eps=1e-6, dtype=dtype)
        self.qkv = nn.Linear(H, 3 * H, dtype=dtype)
        self.proj = nn.Linear(H, H, dtype=dtype)
        self.fc1 = nn.Linear(H, cfg.intermediate_size, dtype=dtype)
        self.fc2 = nn.Linear(cfg.intermediate_size, H, dtype=dtype)

    def forward(self, x, cos, sin, cu, max_len):
        """Biases, GELU and residual adds ride on `ops.bias_act` (one pass after each GEMM), the norms on
        `ops.layer_norm`; attention is full (non-causal) over each image's patches."""
        P = x.shape[0]
        h = ops.layer_norm(x, self.norm1.weight, self.norm1.bias, self.norm1.eps)
        qkv = ops.bias_act(ops.linear(h, self.qkv.weight), self.qkv.bias).view(P, 3, self.n_heads, self.head_dim)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        q, k = ops.rotary_position_embedding(q, cos, sin), ops.rotary_position_embedding(k, cos, sin)
        a = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), cu, max_len, causal=False,
                          scale=1.0 / math.sqrt(self.head_dim))
        x = ops.bias_act(ops.linear(a.reshape(P, -1), self.proj.weight), self.proj.bias, residual=x)
        h = ops.layer_norm(x, self.norm2.weight, self.norm2.bias, self.norm2.eps)
        h = ops.bias_act(ops.linear(h, self.fc1.weight), self.fc1.bias, "gelu_tanh")
        return ops.bias_act(ops.linear(h, self.fc2.weight), self.fc2.bias, residual=x)


class PatchMerger(nn.Module):
    def __init__(self, cfg, dtype=None):
        super().__init__()
        self.unit = cfg.spatial_merge_size ** 2
        Hm = cfg.hidden_size * self.unit
        self.ln_q = nn.LayerNorm(cfg.hidden_size, eps=1e-6, dtype=dtype)
        self.fc1 = nn.Linear(Hm, Hm, dtype=dtype)
        self.fc2 = nn.Linear(Hm, cfg.out_hidden_size, dtype=dtype)

    def forward(self, x):
        x = ops.layer_norm(x, self.ln_q.weight, self.ln_q.bias, self.ln_q.eps).view(-1, self.unit * x.shape[-1])
        h = ops.bias_act(ops.linear(x, self.fc1.weight), self.fc1.bias, "gelu")
        return ops.bias_act(ops.linear(h, self.fc2.weight), self.fc2.bias)


class VisionTower(nn.Module):
    def __init__(self, cfg, dtype=None):
        super().__init__()
        self.config = cfg
        pin = cfg.in_channels * cfg.temporal_patch_size * cfg.patch_size ** 2
        self.patch_embed = nn.Linear(pin, cfg.hidden_size, bias=False, dtype=dtype)   # Conv3d with stride == kernel
        self.blocks = nn.ModuleList([VisionBlock(cfg, dtype) for _ in range(cfg.depth)])
        self.merger = PatchMerger(cfg, dtype)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """[P, 3*2*14*14] -> [P / merge^2, out_hidden]"""
        w = self.patch_embed.weight
        x = ops.linear(pixel_values.to(w.dtype), w)
        sizes = (grid_thw[:, 0] * grid_thw[:, 1] * grid_thw[:, 2]).to(torch.int64).cpu()
        cu = torch.cat([torch.zeros(1, dtype=torch.int64), sizes.cumsum(0)]).to(torch.int32)
        max_len = int(sizes.max()) if sizes.numel() else 0
        cos, sin = vision_rot_pos(grid_thw.cpu(), self.config.spatial_merge_size, x.shape[-1] // self.config.num_heads, x.device)
        for blk in self.blocks:
            x = blk(x, cos, sin, cu, max_len)
        return self.merger(x)

    def dummy_inputs(self, device, dtype):
        m = self.config.spatial_merge_size
        pin = self.patch_embed.weight.shape[1]
        return torch.zeros(m * m, pin, device=device, dtype=dtype), torch.tensor([[1, m, m]], device=device)


class Qwen3VLInner(nn.Module):
    def __init__(self, config, dtype=None):
        super().__init__()
        self.visual = VisionTower(config.vision_config, dtype)
        self.language_model = Qwen3Model(config.text_config, dtype)

    @property
    def embed_tokens(self):
        return self.language_model.embed_tokens

    @property
    def norm(self):
        return self.language_model.norm


class Qwen3VLForConditionalGenerationBase(nn.Module):
    def __init__(self, config: Any):
        super().__init__()
        self.config = config
        dtype = config.dtype
        if isinstance(dtype, str):
            dtype = getattr(torch, dtype.replace("torch.", ""))
        self.model = Qwen3VLInner(config, dtype)
        self.lm_head = LMHead(config.text_config.hidden_size, config.text_config.vocab_size, bias=False, dtype=dtype)
        if not any(p.is_meta for p in self.parameters()):
            init_weights(self, config.initializer_range)

    def tie_weights(self) -> None:
        if getattr(self.config, "tie_word_embeddings", False):
            self.lm_head.weight = self.model.language_model.embed_tokens.weight

    @property
    def all_tied_weights_keys(self):
        return {"lm_head.weight": "model.language_model.embed_tokens.weight"} if getattr(self.config, "tie_word_embeddings", False) else {}

    def fuse_media(self, input_ids, pixel_values, image_grid_thw):
        """Token embeddings of the *global* row with image features written at the image placeholder positions."""
        emb = self.model.language_model.embed_tokens(input_ids)
        if pixel_values is None:
            v_in, grid = self.model.visual.dummy_inputs(emb.device, emb.dtype)
            feats = self.model.visual(v_in, grid_thw=grid)
            return emb + 0.0 * feats.sum()            # keeps the tower in the graph (FSDP hooks, balanced backward)
        feats = self.model.visual(pixel_values, grid_thw=image_grid_thw)
        mask = (input_ids == self.config.image_token_id)
        n = int(mask.sum())
        if n != feats.shape[0]:
            # dummy media on media-less batches produce features that no placeholder consumes
            if n == 0:
                return emb + 0.0 * feats.sum()
            raise ValueError(f"{n} image placeholder tokens but {feats.shape[0]} image features")
        return emb.masked_scatter(mask.unsqueeze(-1), feats.to(emb.dtype))

    def forward(self, input_ids=None, position_ids=None, pixel_values=None, image_grid_thw=None, inputs_embeds=None,
                cu_seq_lens_q=None, cu_seq_lens_k=None, max_length_q=None, max_length_k=None, skip_lm_head=False, **kw):
        if inputs_embeds is None:
            inputs_embeds = self.fuse_media(input_ids, pixel_values, image_grid_thw)
        hidden = self.model.language_model(inputs_embeds=inputs_embeds, position_ids=position_ids,
                                           cu_seq_lens_q=cu_seq_lens_q, max_length_q=max_length_q)
        out = CausalLMOutput(hidden_states=hidden)
        if not skip_lm_head:
            out["logits"] = self.lm_head(hidden)
        return out
