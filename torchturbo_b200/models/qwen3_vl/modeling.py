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
from ..config import ModelConfig, NestedDtype
from ..modules.transformer import CausalLMOutput, init_weights
from ..qwen3.modeling import LMHead, Qwen3Config, Qwen3Model


class Qwen3VLVisionConfig(ModelConfig):
    model_type = "qwen3_vl_vision"
    _defaults = dict(depth=27, hidden_size=1152, num_heads=16, intermediate_size=4304, patch_size=14,
                     temporal_patch_size=2, in_channels=3, spatial_merge_size=2, out_hidden_size=4096,
                     hidden_act="gelu_pytorch_tanh", initializer_range=0.02, num_position_embeddings=2304,
                     deepstack_visual_indexes=(), disable_merger_proj=False)


class Qwen3VLConfig(NestedDtype, ModelConfig):
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
        self._adopt_dtype()
        for k in ("hidden_size", "vocab_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim"):
            setattr(self, k, getattr(self.text_config, k))



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


class _PatchEmbed(nn.Module):
    """Stride == kernel 3-D convolution over `(temporal_patch, patch, patch)` voxels, i.e. one GEMM per flattened
    voxel; the parameter keeps the convolution's shape `[C, in, tp, p, p]` and name (`patch_embed.proj`)."""

    def __init__(self, cfg, dtype=None):
        super().__init__()
        k = (cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size)
        self.proj = nn.Conv3d(cfg.in_channels, cfg.hidden_size, kernel_size=k, stride=k, bias=True, dtype=dtype)

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        w = self.proj.weight
        return ops.bias_act(ops.linear(pixels.reshape(pixels.shape[0], w[0].numel()).to(w.dtype), w.reshape(w.shape[0], -1)), self.proj.bias)


class _VisionAttention(nn.Module):
    def __init__(self, H: int, dtype=None):
        super().__init__()
        self.qkv = nn.Linear(H, 3 * H, dtype=dtype)
        self.proj = nn.Linear(H, H, dtype=dtype)


class _VisionMLP(nn.Module):
    def __init__(self, H: int, hidden: int, dtype=None):
        super().__init__()
        self.linear_fc1 = nn.Linear(H, hidden, dtype=dtype)
        self.linear_fc2 = nn.Linear(hidden, H, dtype=dtype)


_ACTS = {"gelu_pytorch_tanh": "gelu_tanh", "gelu_tanh": "gelu_tanh", "gelu": "gelu"}


class VisionBlock(nn.Module):
    """Module tree of the Hugging Face block (`norm1`, `norm2`, `attn.qkv`, `attn.proj`, `mlp.linear_fc1/2`)."""

    def __init__(self, cfg, dtype=None):
        super().__init__()
        H = cfg.hidden_size
        self.n_heads, self.head_dim = cfg.num_heads, H // cfg.num_heads
        self.norm1, self.norm2 = nn.LayerNorm(H, eps=1e-6, dtype=dtype), nn.LayerNorm(H, eps=1e-6, dtype=dtype)
        self.attn = _VisionAttention(H, dtype)
        self.mlp = _VisionMLP(H, cfg.intermediate_size, dtype)
        self.act = _ACTS[getattr(cfg, "hidden_act", "gelu_pytorch_tanh")]

    def forward(self, x, cos, sin, cu, max_len):
        """Biases, GELU and residual adds ride on `ops.bias_act` (one pass after each GEMM), the norms on
        `ops.layer_norm`; attention is full (non-causal) over each frame's patches."""
        P = x.shape[0]
        a, m = self.attn, self.mlp
        h = ops.layer_norm(x, self.norm1.weight, self.norm1.bias, self.norm1.eps)
        qkv = ops.bias_act(ops.linear(h, a.qkv.weight), a.qkv.bias).view(P, 3, self.n_heads, self.head_dim)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        q, k = ops.rotary_position_embedding(q, cos, sin), ops.rotary_position_embedding(k, cos, sin)
        o = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), cu, max_len, causal=False,
                          scale=1.0 / math.sqrt(self.head_dim))
        x = ops.bias_act(ops.linear(o.reshape(P, -1), a.proj.weight), a.proj.bias, residual=x)
        h = ops.layer_norm(x, self.norm2.weight, self.norm2.bias, self.norm2.eps)
        h = ops.bias_act(ops.linear(h, m.linear_fc1.weight), m.linear_fc1.bias, self.act)
        return ops.bias_act(ops.linear(h, m.linear_fc2.weight), m.linear_fc2.bias, residual=x)


class PatchMerger(nn.Module):
    """`merge^2` neighbouring patches -> one row: LayerNorm (per patch, or over the joined row with `postshuffle`),
    then `linear_fc1` -> GELU -> `linear_fc2` (left out with `disable_merger_proj`: the joined row is the output)."""

    def __init__(self, cfg, dtype=None, postshuffle: bool = False):
        super().__init__()
        self.unit = cfg.spatial_merge_size ** 2
        Hm = cfg.hidden_size * self.unit
        self.postshuffle = postshuffle
        self.norm = nn.LayerNorm(Hm if postshuffle else cfg.hidden_size, eps=1e-6, dtype=dtype)
        self.project = not getattr(cfg, "disable_merger_proj", False)
        if self.project:
            self.linear_fc1 = nn.Linear(Hm, Hm, dtype=dtype)
            self.linear_fc2 = nn.Linear(Hm, cfg.out_hidden_size, dtype=dtype)

    def forward(self, x):
        if self.postshuffle:
            x = x.reshape(-1, self.unit * x.shape[-1])
        x = ops.layer_norm(x, self.norm.weight, self.norm.bias, self.norm.eps).view(-1, self.norm.weight.shape[0] if self.postshuffle
                                                                                   else self.unit * x.shape[-1])
        if not self.project:
            return x
        h = ops.bias_act(ops.linear(x, self.linear_fc1.weight), self.linear_fc1.bias, "gelu")
        return ops.bias_act(ops.linear(h, self.linear_fc2.weight), self.linear_fc2.bias)


def interpolated_positions(table: torch.Tensor, grid_thw: list[list[int]], merge: int) -> torch.Tensor:
    """Learned position code of every packed patch: the `[n*n, C]` table is a square grid, each image's `(h, w)` grid
    is laid over it (corners aligned) and read bilinearly; rows come out merge-window-major like the patches, and the
    frames of a clip share one image's code."""
    n = int(round(math.sqrt(table.shape[0])))
    out = []
    for t, h, w in grid_thw:
        hi = torch.linspace(0, n - 1, h, device=table.device)
        wi = torch.linspace(0, n - 1, w, device=table.device)
        hf, wf = hi.long(), wi.long()
        hc, wc = (hf + 1).clamp(max=n - 1), (wf + 1).clamp(max=n - 1)
        dh, dw = (hi - hf)[:, None], (wi - wf)[None, :]
        idx = torch.stack([hf[:, None] * n + wf[None], hf[:, None] * n + wc[None], hc[:, None] * n + wf[None],
                           hc[:, None] * n + wc[None]]).reshape(4, -1)
        wt = torch.stack([(1 - dh) * (1 - dw), (1 - dh) * dw, dh * (1 - dw), dh * dw]).reshape(4, -1, 1).to(table.dtype)
        e = (table[idx] * wt).sum(0)                                                  # [h*w, C] raster order
        e = e.view(h // merge, merge, w // merge, merge, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
        out.append(e.repeat(t, 1) if t > 1 else e)
    return torch.cat(out, dim=0)


class VisionTower(nn.Module):
    """The Qwen3-VL / Qwen3.5 / Bailing-VL tower with the module tree of its Hugging Face classes (`patch_embed.proj`,
    `pos_embed`, `blocks.N.{norm1,norm2,attn.qkv,attn.proj,mlp.linear_fc1,mlp.linear_fc2}`, `merger.{norm,linear_fc1,
    linear_fc2}`, `deepstack_merger_list.N`), so published towers load by name (transformers:
    models/qwen3_vl/modeling_qwen3_vl.py `Qwen3VLVisionModel`; models/bailing_moe_v3_vl/modeling_bailing_moe_v3_vl.py:985
    of the reference)."""

    def __init__(self, cfg, dtype=None):
        super().__init__()
        self.config = cfg
        self.patch_embed = _PatchEmbed(cfg, dtype)
        self.pos_embed = nn.Embedding(cfg.num_position_embeddings, cfg.hidden_size, dtype=dtype)
        self.blocks = nn.ModuleList([VisionBlock(cfg, dtype) for _ in range(cfg.depth)])
        self.merger = PatchMerger(cfg, dtype)
        self.deepstack_visual_indexes = [int(i) for i in (getattr(cfg, "deepstack_visual_indexes", None) or ())]
        if getattr(cfg, "disable_merger_proj", False):
            self.deepstack_visual_indexes = []
        if self.deepstack_visual_indexes:
            self.deepstack_merger_list = nn.ModuleList([PatchMerger(cfg, dtype, postshuffle=True)
                                                        for _ in self.deepstack_visual_indexes])

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor, return_deepstack: bool = False):
        """[P, in * tp * p * p] -> [P / merge^2, out_hidden] (and the list of DeepStack features when asked for)."""
        cfg = self.config
        grid = [[int(v) for v in row] for row in grid_thw.tolist()]
        x = self.patch_embed(pixel_values)
        x = x + interpolated_positions(self.pos_embed.weight, grid, cfg.spatial_merge_size).to(x.dtype)
        # attention never crosses a frame: one segment per frame of every medium
        sizes = torch.tensor([h * w for t, h, w in grid for _ in range(t)], dtype=torch.int64)
        cu = torch.cat([torch.zeros(1, dtype=torch.int64), sizes.cumsum(0)]).to(torch.int32)
        max_len = int(sizes.max()) if sizes.numel() else 0
        cos, sin = vision_rot_pos(grid_thw.cpu(), cfg.spatial_merge_size, x.shape[-1] // cfg.num_heads, x.device)
        deep = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, cu, max_len)
            if i in self.deepstack_visual_indexes:
                deep.append(self.deepstack_merger_list[self.deepstack_visual_indexes.index(i)](x))
        out = self.merger(x)
        return (out, deep) if return_deepstack else out

    def dummy_inputs(self, device, dtype):
        # sizes from the configuration: reading the (sharded) projection weight here would start a collective of its own
        c = self.config
        m = c.spatial_merge_size
        pin = c.in_channels * c.temporal_patch_size * c.patch_size ** 2
        return torch.zeros(m * m, pin, device=device, dtype=dtype), torch.tensor([[1, m, m]], device=device)


class Qwen3VLTextModel(Qwen3Model):
    """The Qwen3 decoder as Qwen3-VL runs it: interleaved multimodal rotary positions (`position_ids [3, 1, T]`:
    temporal, height, width; a plain `[1, T]` row is read as text positions) and DeepStack, i.e. the features that
    early tower blocks produce are added to the residual stream at the visual positions after decoder layers
    0, 1, ... (transformers: models/qwen3_vl/modeling_qwen3_vl.py `Qwen3VLTextModel._deepstack_process`).
    `deepstack_embeds [n, T, H]` is dense over the row (zero where there is no medium) so that sequence parallelism
    slices it like `inputs_embeds`."""

    def __init__(self, config: Any, dtype=None):
        super().__init__(config, dtype)
        from ..modules.hybrid import MRotaryEmbedding

        sec = getattr(config, "mrope_section", None)
        if sec:
            self.rotary_emb = MRotaryEmbedding(config.head_dim, config.rope_theta, sec, getattr(config, "mrope_interleaved", True))

    def forward(self, input_ids=None, position_ids=None, inputs_embeds=None, cu_seq_lens_q=None, max_length_q=None,
                deepstack_embeds=None, **_unused):
        if inputs_embeds is None:
            inputs_embeds = self.embed_tokens(input_ids)
        h = inputs_embeds.reshape(-1, inputs_embeds.shape[-1])
        T = h.shape[0]
        if position_ids is None:
            position_ids = torch.arange(T, device=h.device)
        if position_ids.dim() == 3 and position_ids.shape[0] in (3, 4):        # [3 | 4, B, T]: 4 = text row first
            pos = position_ids[-3:].reshape(3, -1)[:, -T:]
        else:
            pos = position_ids.reshape(-1)[-T:]
        cos, sin = self.rotary_emb(pos)
        if cu_seq_lens_q is None:
            cu_seq_lens_q = torch.tensor([0, T], dtype=torch.int32)
            max_length_q = T
        ids = input_ids.reshape(-1) if input_ids is not None else None
        deep = None if deepstack_embeds is None else deepstack_embeds.reshape(deepstack_embeds.shape[0], -1, h.shape[-1])
        res = None
        for i, layer in enumerate(self.layers):
            h, res = layer(h, res, cos, sin, cu_seq_lens_q, max_length_q, ids)
            if deep is not None and i < deep.shape[0]:
                h = h + deep[i].to(h.dtype)           # h is the pending update of the residual stream `res + h`
        h, _ = self.norm(h, res)
        return h.unsqueeze(0)


class Qwen3VLInner(nn.Module):
    def __init__(self, config, dtype=None):
        super().__init__()
        self.visual = VisionTower(config.vision_config, dtype)
        self.language_model = Qwen3VLTextModel(config.text_config, dtype)

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
        """Token embeddings of the *global* row with image features written at the image placeholder positions, and
        the DeepStack features of the same positions (`[n, T, H]`, or None when the tower has none)."""
        emb = self.model.language_model.embed_tokens(input_ids)
        visual = self.model.visual
        n_deep = len(visual.deepstack_visual_indexes)
        def no_media(feats, deep):
            """The tower ran on the dummy image.  Its outputs enter the graph where real features would, each DeepStack
            level at its own decoder layer, multiplied by zero: a rank without media then meets the tower's gradient
            at the same point of the backward pass as the ranks with media, so the FSDP collectives of all ranks
            stay in one order."""
            e = emb + 0.0 * feats.sum()
            if not n_deep:
                return e, None
            dense = torch.stack([emb.new_zeros(emb.shape[-2:]) + 0.0 * d.sum() for d in deep])
            return e, dense.unsqueeze(1) if emb.dim() == 3 else dense

        if pixel_values is None or pixel_values.shape[0] == 0:        # no media in this rank's row
            v_in, grid = visual.dummy_inputs(emb.device, emb.dtype)
            return no_media(*visual(v_in, grid_thw=grid, return_deepstack=True))
        feats, deep = visual(pixel_values, grid_thw=image_grid_thw, return_deepstack=True)
        mask = (input_ids == self.config.image_token_id) | (input_ids == getattr(self.config, "video_token_id", -1))
        n = int(mask.sum())
        if n != feats.shape[0]:
            # dummy media on media-less batches produce features that no placeholder consumes
            if n == 0:
                return no_media(feats, deep)
            raise ValueError(f"{n} image placeholder tokens but {feats.shape[0]} image features")
        out = emb.masked_scatter(mask.unsqueeze(-1), feats.to(emb.dtype))
        if not n_deep:
            return out, None
        dense = emb.new_zeros(n_deep, *emb.shape[-2:])
        m = mask.reshape(-1)
        for i, d in enumerate(deep):
            dense[i] = dense[i].masked_scatter(m.unsqueeze(-1), d.to(emb.dtype))
        return out, dense.unsqueeze(1) if emb.dim() == 3 else dense

    def forward(self, input_ids=None, position_ids=None, pixel_values=None, image_grid_thw=None, inputs_embeds=None,
                cu_seq_lens_q=None, cu_seq_lens_k=None, max_length_q=None, max_length_k=None, skip_lm_head=False,
                deepstack_embeds=None, **kw):
        if inputs_embeds is None:
            inputs_embeds, deepstack_embeds = self.fuse_media(input_ids, pixel_values, image_grid_thw)
        hidden = self.model.language_model(inputs_embeds=inputs_embeds, position_ids=position_ids,
                                           cu_seq_lens_q=cu_seq_lens_q, max_length_q=max_length_q,
                                           deepstack_embeds=deepstack_embeds)
        out = CausalLMOutput(hidden_states=hidden)
        if not skip_lm_head:
            out["logits"] = self.lm_head(hidden)
        return out
