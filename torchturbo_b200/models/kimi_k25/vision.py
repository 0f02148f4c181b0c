"""MoonViT, the vision tower of Kimi-K2.5, and its patch-merger projector, with the parameter names of the published
checkpoints (`vision_tower.patch_embed.proj`, `vision_tower.patch_embed.pos_emb.weight`,
`vision_tower.encoder.blocks.N.{norm0,norm1,wqkv,wo,mlp.fc0,mlp.fc1}`, `vision_tower.encoder.final_layernorm`,
`mm_projector.{pre_norm,proj.0,proj.2}`), so a real checkpoint's tower loads without a name map.

What the tower computes (models/kimi_k25/modeling_kimi_k25.py:271-830 of the reference):
  * patches `[L, 3, p, p]` (raster order inside each image, frames one after the other) -> a stride-`p` convolution,
    i.e. one GEMM over the flattened patch;
  * a learned `[H0, W0, C]` position table, resampled bicubically to each image's `(h, w)` grid, plus a fixed
    sin/cos code per frame for clips (`t > 1`);
  * pre-norm blocks: packed QKV with bias, 2-D rotary embedding whose rotary pairs alternate between the patch column
    and the patch row (pair `2i` turns with the column, pair `2i+1` with the row, both at `theta^(-4i/d)`), full
    attention over all `t*h*w` patches of one medium, tanh-GELU MLP; LayerNorm eps 1e-5 throughout;
  * `sd2_tpool` merge: the frames of a medium are averaged, each 2x2 window of patches becomes one row of 4 vectors;
  * projector: LayerNorm on each of the 4 vectors, concatenation, Linear -> GELU -> Linear to the language width.

Kernels: the GEMMs, LayerNorm and bias/GELU/residual tails go through `ops` (tcgen05 GEMM, `layer_norm`, `bias_act`),
attention through `ops.attention` with one segment per medium.  Checkpoints keep a rotary pair in adjacent channels;
q and k are regrouped to the half layout with the same fixed permutation before the rotation, which leaves every
score unchanged (`apply_partial_rope(..., interleaved=True)`)."""
from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import ops
from ..config import ModelConfig
from ..modules.mixers import apply_partial_rope
from ..modules.vision import GridVisionBalanceIO


class MoonViTConfig(ModelConfig):
    model_type = "moonvit3d"
    _defaults = dict(patch_size=14, init_pos_emb_height=64, init_pos_emb_width=64, init_pos_emb_time=4,
                     pos_emb_type="divided_fixed", vt_num_attention_heads=16, vt_num_hidden_layers=27, vt_hidden_size=1152,
                     vt_intermediate_size=4304, merge_kernel_size=(2, 2), video_attn_type="spatial_temporal",
                     merge_type="sd2_tpool", mm_projector_type="patchmerger", mm_hidden_size=None,
                     projector_hidden_act="gelu", projector_ln_eps=1e-5, text_hidden_size=7168, in_channels=3,
                     initializer_range=0.02)

    def __init__(self, **kw):
        super().__init__(**{k: v for k, v in kw.items() if not k.startswith("_")})
        if self.mm_hidden_size is None:
            self.mm_hidden_size = self.vt_hidden_size
        self.merge_kernel_size = tuple(int(x) for x in self.merge_kernel_size)
        if self.merge_type != "sd2_tpool" or self.pos_emb_type != "divided_fixed" or self.video_attn_type != "spatial_temporal":
            raise ValueError("MoonViT: only merge_type=sd2_tpool, pos_emb_type=divided_fixed, "
                             "video_attn_type=spatial_temporal exist in published checkpoints")
        if self.mm_projector_type not in ("patchmerger", "identity"):
            raise ValueError(f"unsupported mm_projector_type {self.mm_projector_type!r}")

    # the names the generic tower code and the balancer read
    @property
    def hidden_size(self):
        return self.vt_hidden_size

    @property
    def num_heads(self):
        return self.vt_num_attention_heads

    @property
    def spatial_merge_size(self):
        return self.merge_kernel_size[0]

    @property
    def depth(self):
        return self.vt_num_hidden_layers

    @property
    def intermediate_size(self):
        return self.vt_intermediate_size

    @property
    def temporal_patch_size(self):
        return 1

    @property
    def out_hidden_size(self):
        return self.text_hidden_size


def frame_position_code(dim: int, frames: int) -> torch.Tensor:
    """`[frames, dim]`: sin of `f * 10000^(-j / (dim/2))` in the first half of the channels, cos in the second."""
    omega = 1.0 / 10000 ** (torch.arange(dim // 2, dtype=torch.float32) / (dim / 2.0))
    ang = torch.arange(frames, dtype=torch.float32)[:, None] * omega[None]
    return torch.cat([ang.sin(), ang.cos()], dim=1)


class _PosEmb(nn.Module):
    def __init__(self, height: int, width: int, frames: int, dim: int, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(height, width, dim, dtype=dtype))
        self.register_buffer("time_weight", frame_position_code(dim, frames), persistent=False)
        self.frames = frames

    def forward(self, grid_thw: list[list[int]]) -> torch.Tensor:
        """`[sum(t*h*w), C]` additive position code for the packed patches."""
        H0, W0, C = self.weight.shape
        w = self.weight
        out, cache = [], {}
        for t, h, wd in grid_thw:
            if t > self.frames:
                raise ValueError(f"a clip of {t} frames exceeds init_pos_emb_time={self.frames}")
            if (h, wd) not in cache:
                if (h, wd) == (H0, W0):
                    cache[(h, wd)] = w.reshape(-1, C)
                else:
                    r = F.interpolate(w.permute(2, 0, 1).unsqueeze(0).float(), size=(h, wd), mode="bicubic")
                    cache[(h, wd)] = r.squeeze(0).permute(1, 2, 0).reshape(-1, C).to(w.dtype)
            e = cache[(h, wd)]
            if t > 1:
                e = (e.unsqueeze(0) + self.time_weight[:t].to(device=e.device, dtype=e.dtype).unsqueeze(1)).reshape(-1, C)
            out.append(e)
        return torch.cat(out, dim=0)


class _PatchEmbed(nn.Module):
    def __init__(self, cfg: MoonViTConfig, dtype=None):
        super().__init__()
        p = cfg.patch_size
        self.proj = nn.Conv2d(cfg.in_channels, cfg.vt_hidden_size, kernel_size=p, stride=p, dtype=dtype)
        self.pos_emb = _PosEmb(cfg.init_pos_emb_height, cfg.init_pos_emb_width, cfg.init_pos_emb_time, cfg.vt_hidden_size, dtype)

    def forward(self, pixels: torch.Tensor, grid_thw: list[list[int]]) -> torch.Tensor:
        w = self.proj.weight
        x = ops.bias_act(ops.linear(pixels.reshape(pixels.shape[0], -1).to(w.dtype), w.reshape(w.shape[0], -1)), self.proj.bias)
        return x + self.pos_emb(grid_thw)


class _MLP2(nn.Module):
    def __init__(self, d: int, hidden: int, dtype=None):
        super().__init__()
        self.fc0 = nn.Linear(d, hidden, dtype=dtype)
        self.fc1 = nn.Linear(hidden, d, dtype=dtype)


class MoonViTBlock(nn.Module):
    def __init__(self, cfg: MoonViTConfig, dtype=None):
        super().__init__()
        C = cfg.vt_hidden_size
        self.n_heads, self.head_dim = cfg.vt_num_attention_heads, C // cfg.vt_num_attention_heads
        self.norm0, self.norm1 = nn.LayerNorm(C, dtype=dtype), nn.LayerNorm(C, dtype=dtype)
        self.mlp = _MLP2(C, cfg.vt_intermediate_size, dtype)
        self.wqkv = nn.Linear(C, 3 * C, dtype=dtype)
        self.wo = nn.Linear(C, C, dtype=dtype)

    def forward(self, x, cos, sin, cu, max_len):
        P = x.shape[0]
        h = ops.layer_norm(x, self.norm0.weight, self.norm0.bias, self.norm0.eps)
        qkv = ops.bias_act(ops.linear(h, self.wqkv.weight), self.wqkv.bias).view(P, 3, self.n_heads, self.head_dim)
        q = apply_partial_rope(qkv[:, 0].contiguous(), cos, sin, interleaved=True)
        k = apply_partial_rope(qkv[:, 1].contiguous(), cos, sin, interleaved=True)
        a = ops.attention(q.contiguous(), k.contiguous(), qkv[:, 2].contiguous(), cu, max_len, causal=False,
                          scale=1.0 / math.sqrt(self.head_dim))
        x = ops.bias_act(ops.linear(a.reshape(P, -1), self.wo.weight), self.wo.bias, residual=x)
        h = ops.layer_norm(x, self.norm1.weight, self.norm1.bias, self.norm1.eps)
        h = ops.bias_act(ops.linear(h, self.mlp.fc0.weight), self.mlp.fc0.bias, "gelu_tanh")
        return ops.bias_act(ops.linear(h, self.mlp.fc1.weight), self.mlp.fc1.bias, residual=x)


class _Encoder(nn.Module):
    def __init__(self, cfg: MoonViTConfig, dtype=None):
        super().__init__()
        self.blocks = nn.ModuleList([MoonViTBlock(cfg, dtype) for _ in range(cfg.vt_num_hidden_layers)])
        self.final_layernorm = nn.LayerNorm(cfg.vt_hidden_size, dtype=dtype)


def rope_2d_tables(grid_thw: list[list[int]], head_dim: int, device, theta: float = 10000.0):
    """cos / sin `[P, head_dim / 2]`: rotary pair `2i` carries `column * theta^(-4i/d)`, pair `2i + 1` carries
    `row * theta^(-4i/d)`; the frames of a clip repeat the table of one frame."""
    n = head_dim // 4
    freqs = 1.0 / theta ** (torch.arange(0, head_dim, 4, dtype=torch.float32)[:n] / head_dim)
    parts = []
    for t, h, w in grid_thw:
        col = torch.arange(w, dtype=torch.float32).repeat(h)
        row = torch.arange(h, dtype=torch.float32).repeat_interleave(w)
        ang = torch.stack([col[:, None] * freqs[None], row[:, None] * freqs[None]], dim=-1).reshape(h * w, 2 * n)
        parts.append(ang.repeat(t, 1))
    ang = torch.cat(parts, dim=0).to(device)
    return ang.cos(), ang.sin()


class MoonViT(nn.Module):
    """`forward(pixel_values, grid_thw)` -> merged features `[sum(h*w / 4), 4, C]` flattened to `[rows, 4 * C]`."""

    def __init__(self, cfg: MoonViTConfig, dtype=None):
        super().__init__()
        if (cfg.vt_hidden_size // cfg.vt_num_attention_heads) % 4:
            raise ValueError("MoonViT: the head width must be a multiple of 4 (2-D rotary pairs)")
        self.config = cfg
        self.patch_embed = _PatchEmbed(cfg, dtype)
        self.encoder = _Encoder(cfg, dtype)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        grid = [[int(v) for v in row] for row in grid_thw.tolist()]
        x = self.patch_embed(pixel_values, grid)
        sizes = torch.tensor([t * h * w for t, h, w in grid], dtype=torch.int64)
        cu = torch.cat([torch.zeros(1, dtype=torch.int64), sizes.cumsum(0)]).to(torch.int32)
        max_len = int(sizes.max()) if sizes.numel() else 0
        cos, sin = rope_2d_tables(grid, cfg.vt_hidden_size // cfg.vt_num_attention_heads, x.device)
        for blk in self.encoder.blocks:
            x = blk(x, cos, sin, cu, max_len)
        fl = self.encoder.final_layernorm
        x = ops.layer_norm(x, fl.weight, fl.bias, fl.eps)
        kh, kw = cfg.merge_kernel_size
        out, start = [], 0
        for t, h, w in grid:
            seq = x[start:start + t * h * w].view(t, h // kh, kh, w // kw, kw, -1)
            seq = seq.permute(0, 1, 3, 2, 4, 5).float().mean(dim=0).to(x.dtype)       # frames pooled
            out.append(seq.reshape((h // kh) * (w // kw), kh * kw * x.shape[-1]))
            start += t * h * w
        return torch.cat(out, dim=0)

    def dummy_inputs(self, device, dtype):
        kh, kw = self.config.merge_kernel_size
        pin = self.config.in_channels * self.config.patch_size ** 2
        return torch.zeros(kh * kw, pin, device=device, dtype=dtype), torch.tensor([[1, kh, kw]], device=device)


class PatchMergerMLP(nn.Module):
    """`[rows, 4 * C]` (four patch vectors per row) -> `[rows, text_hidden]`."""

    def __init__(self, cfg: MoonViTConfig, dtype=None):
        super().__init__()
        C = cfg.mm_hidden_size
        self.unit = cfg.merge_kernel_size[0] * cfg.merge_kernel_size[1]
        self.pre_norm = nn.LayerNorm(C, eps=cfg.projector_ln_eps, dtype=dtype)
        self.proj = nn.Sequential(nn.Linear(C * self.unit, C * self.unit, dtype=dtype), nn.GELU(),
                                  nn.Linear(C * self.unit, cfg.text_hidden_size, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rows = x.shape[0]
        h = ops.layer_norm(x.reshape(rows * self.unit, -1), self.pre_norm.weight, self.pre_norm.bias, self.pre_norm.eps)
        h = ops.bias_act(ops.linear(h.reshape(rows, -1), self.proj[0].weight), self.proj[0].bias, "gelu")
        return ops.bias_act(ops.linear(h, self.proj[2].weight), self.proj[2].bias)


class TemporalPoolVisionBalanceIO(GridVisionBalanceIO):
    """Balancer IO of a tower that pools the frames of a medium: a medium of `(t, h, w)` patches yields
    `h * w / merge^2` rows whatever `t` is."""

    def _lengths(self, grid: torch.Tensor) -> list[int]:
        return [int(h * w) // (self.merge ** 2) for _, h, w in grid.tolist()]


def init_moonvit(tower: MoonViT, projector: nn.Module | None, std: float = 0.02, generator: Any = None) -> None:
    with torch.no_grad():
        for m in list(tower.modules()) + (list(projector.modules()) if projector is not None else []):
            if isinstance(m, (nn.Linear, nn.Conv2d)):
                m.weight.normal_(0.0, std, generator=generator)
                if m.bias is not None:
                    m.bias.zero_()
            elif isinstance(m, nn.LayerNorm):
                m.weight.fill_(1.0)
                m.bias.zero_()
            elif isinstance(m, _PosEmb):
                m.weight.normal_(0.0, 1.0, generator=generator)
