"""Config-driven decoder shared by the hybrid families (Qwen3.5 dense / MoE, Bailing, Kimi, GLM, ...).

A family describes each layer by a mixer kind (`full_attention`, `gated_attention`, `linear_attention`, `mla`, `kda`)
and an MLP kind (dense SwiGLU or MoE); `HybridModel` builds the stack, computes rotary tables once per step (text
positions or 3-axis multimodal positions), and threads a `MixerContext` through the layers.  The residual stream is
carried unadded so each residual add fuses into the next RMSNorm kernel, as in `transformer.DecoderLayer`.

`MultiTokenPredictor` is the recurrent next-next-token head of the Qwen3.5 / DeepSeek style checkpoints
(models/qwen3_5/modeling_qwen3_5.py:949-1003 of the reference): per depth, roll the ids left inside every packed
sequence, embed, normalise both inputs, project `[emb | hidden]` back to the model width, run one decoder layer
and a final norm.
"""
from __future__ import annotations

from typing import Any, Callable

import torch
import torch.nn as nn

from ...ops import ops
from .mixers import GatedAttention, GatedDeltaNet, KimiDeltaAttention, MixerContext, MLAttention
from .transformer import Attention, DenseMLP, RMSNorm

MIXERS: dict[str, Callable[..., nn.Module]] = {
    "gated_attention": GatedAttention,
    "linear_attention": GatedDeltaNet,
    "mla": MLAttention,
    "kda": KimiDeltaAttention,
}


class _PlainAttentionMixer(Attention):
    """`transformer.Attention` behind the mixer call signature."""

    def forward(self, x, ctx: MixerContext):  # type: ignore[override]
        self.sp_group, self.sp_size = ctx.sp_group, ctx.sp_size
        return super().forward(x, ctx.cos, ctx.sin, ctx.cu_seqlens, ctx.max_seqlen)


MIXERS["full_attention"] = _PlainAttentionMixer


class HybridDecoderLayer(nn.Module):
    """Pre-norm block: mixer then MLP.  The mixer lives under the attribute name the checkpoints use for its kind
    (`linear_attn` for linear attention, `self_attn` otherwise)."""

    def __init__(self, config: Any, layer_idx: int, mixer_kind: str, mlp: nn.Module, dtype=None,
                 one_plus_weight: bool = False):
        super().__init__()
        self.layer_idx, self.layer_type = layer_idx, mixer_kind
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype, one_plus_weight=one_plus_weight)
        mixer = MIXERS[mixer_kind](config, layer_idx, dtype)
        if mixer_kind in ("linear_attention", "kda"):
            self.linear_attn = mixer
        else:
            self.self_attn = mixer
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype, one_plus_weight=one_plus_weight)
        self.mlp = mlp

    @property
    def mixer(self) -> nn.Module:
        return self.linear_attn if hasattr(self, "linear_attn") else self.self_attn

    def forward(self, h, residual, ctx: MixerContext):
        if residual is None:
            residual = h
            x = self.input_layernorm(h)
        else:
            x, residual = self.input_layernorm(h, residual)
        a = self.mixer(x, ctx)
        x, residual = self.post_attention_layernorm(a, residual)
        m = self.mlp(x, ctx.input_ids)
        if isinstance(m, tuple):
            m = m[0]
        return m, residual


class MRotaryEmbedding(nn.Module):
    """Rotary tables for text positions `[T]` or multimodal positions `[3, T]` (temporal, height, width): with
    `mrope_section = (t, h, w)` rotary pair `i` follows the axis whose interleaved section it falls in."""

    def __init__(self, rot_dim: int, theta: float, mrope_section=None, interleaved: bool = True):
        super().__init__()
        self.rot_dim, self.theta = rot_dim, theta
        self.mrope_section = tuple(mrope_section) if mrope_section else None
        self.interleaved = interleaved
        self.register_buffer("inv_freq", self._make(None), persistent=False)

    def _make(self, device):
        expo = torch.arange(0, self.rot_dim, 2, dtype=torch.float32, device=device) / self.rot_dim
        return 1.0 / (self.theta ** expo)

    def reset(self, device=None):
        self.inv_freq = self._make(device if device is not None else self.inv_freq.device)

    def axis_of_pair(self, n_pairs: int, device) -> torch.Tensor:
        sec = self.mrope_section
        axis = torch.zeros(n_pairs, dtype=torch.long, device=device)
        if self.interleaved:
            # pairs cycle t,h,w,t,h,w,... while the h / w budgets last; the remainder is temporal
            for ax in (1, 2):
                if sec[ax] <= 0:
                    continue
                idx = torch.arange(ax, 3 * sec[ax], 3, device=device)
                axis[idx[idx < n_pairs]] = ax
        else:
            axis[sec[0]: sec[0] + sec[1]] = 1
            axis[sec[0] + sec[1]: sec[0] + sec[1] + sec[2]] = 2
        return axis

    @torch.no_grad()
    def forward(self, position_ids: torch.Tensor):
        inv = self.inv_freq.float()
        if position_ids.dim() >= 2 and position_ids.shape[0] == 3 and self.mrope_section:
            pos = position_ids.reshape(3, -1).float()                      # [3, T]
            ang3 = pos[:, :, None] * inv[None, None, :]                    # [3, T, P]
            axis = self.axis_of_pair(inv.numel(), inv.device)
            ang = ang3.gather(0, axis.view(1, 1, -1).expand(1, ang3.shape[1], -1))[0]
        else:
            pos = (position_ids[0] if position_ids.dim() >= 2 and position_ids.shape[0] == 3 else position_ids)
            ang = pos.reshape(-1).float()[:, None] * inv[None, :]
        return ang.cos(), ang.sin()


def roll_left_in_sequences(ids: torch.Tensor, cu_seqlens, fill: int = 0) -> torch.Tensor:
    """ids[t] <- ids[t+1] inside every packed sequence; the last token of a sequence gets `fill`."""
    flat = ids.reshape(-1)
    out = torch.cat((flat[1:], flat.new_full((1,), fill)))
    ends = torch.as_tensor(cu_seqlens, dtype=torch.long)[1:] - 1
    ends = ends[(ends >= 0) & (ends < flat.numel())].to(flat.device)
    out[ends] = fill
    return out.view_as(ids)


class MultiTokenPredictor(nn.Module):
    def __init__(self, config: Any, make_layer: Callable[[int], nn.Module], dtype=None, one_plus_weight: bool = False):
        super().__init__()
        self.num_mtp_layers = int(getattr(config, "mtp_num_hidden_layers", 0) or 0)
        h, eps = config.hidden_size, config.rms_norm_eps
        self.pre_fc_norm_embedding = RMSNorm(h, eps, dtype, one_plus_weight=one_plus_weight)
        self.pre_fc_norm_hidden = RMSNorm(h, eps, dtype, one_plus_weight=one_plus_weight)
        self.fc = nn.Linear(2 * h, h, bias=False, dtype=dtype)
        self.norm = RMSNorm(h, eps, dtype, one_plus_weight=one_plus_weight)
        self.layers = nn.ModuleList([make_layer(config.num_hidden_layers + i) for i in range(self.num_mtp_layers)])

    def forward(self, input_ids, hidden, embed_tokens, ctx: MixerContext, pad_token_id: int = 0,
                sp_slice: Callable[[torch.Tensor], torch.Tensor] | None = None) -> list[torch.Tensor]:
        """`input_ids` is the global row; `hidden` `[T_local, H]`.  Returns one `[T_local, H]` per depth."""
        outs, ids, cur = [], input_ids, hidden
        for layer in self.layers:
            ids = roll_left_in_sequences(ids, ctx.cu_seqlens, pad_token_id)
            emb = embed_tokens(ids).reshape(-1, hidden.shape[-1])
            if sp_slice is not None:
                emb = sp_slice(emb)
            x = torch.cat((self.pre_fc_norm_embedding(emb), self.pre_fc_norm_hidden(cur)), -1)
            h = ops.linear(x, self.fc.weight)
            m, res = layer(h, None, ctx)
            cur, _ = self.norm(m, res)
            outs.append(cur)
        return outs


class HybridModel(nn.Module):
    """Embedding + typed layer stack + final norm.  Subclasses provide `mixer_kind(i)` and `make_mlp(i)`."""

    one_plus_weight = False

    def __init__(self, config: Any, dtype=None):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, dtype=dtype)
        self.layers = nn.ModuleList([self.make_layer(i, dtype) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype, one_plus_weight=self.one_plus_weight)
        self.rotary_emb = self.make_rotary(config)
        self.sp_group, self.sp_size, self.sp_rank = None, 1, 0

    # -- family hooks --------------------------------------------------------------------------------
    def mixer_kind(self, i: int) -> str:
        types = getattr(self.config, "layer_types", None)
        return types[i] if types else "full_attention"

    def make_mlp(self, i: int, dtype) -> nn.Module:
        return DenseMLP(self.config.hidden_size, self.config.intermediate_size, dtype)

    def make_layer(self, i: int, dtype) -> nn.Module:
        kind = self.mixer_kind(min(i, self.config.num_hidden_layers - 1)) if i >= self.config.num_hidden_layers else self.mixer_kind(i)
        return HybridDecoderLayer(self.config, i, kind, self.make_mlp(i, dtype), dtype, self.one_plus_weight)

    def make_rotary(self, config) -> nn.Module:
        rot = int(config.head_dim * getattr(config, "partial_rotary_factor", 1.0))
        return MRotaryEmbedding(rot, config.rope_theta, getattr(config, "mrope_section", None),
                                getattr(config, "mrope_interleaved", True))

    def set_sequence_parallel(self, group, size: int, rank: int | None = None) -> None:
        if rank is None:
            rank = torch.distributed.get_rank(group) if (size > 1 and group is not None) else 0
        self.sp_group, self.sp_size, self.sp_rank = group, size, rank

    # -- forward -------------------------------------------------------------------------------------
    def context(self, T: int, position_ids, cu_seq_lens_q, max_length_q, input_ids, device, extras=None) -> MixerContext:
        if position_ids is None:
            position_ids = torch.arange(T, device=device)
        elif position_ids.dim() == 3:                                       # [3, 1, T] multimodal positions
            position_ids = position_ids.reshape(3, -1)[:, -T:]
        else:
            position_ids = position_ids.reshape(-1)[-T:]
        cos, sin = self.rotary_emb(position_ids.to(device))
        if cu_seq_lens_q is None:
            cu_seq_lens_q, max_length_q = torch.tensor([0, T * self.sp_size], dtype=torch.int32), T * self.sp_size
        ids = input_ids.reshape(-1) if input_ids is not None else None
        if ids is not None and self.sp_size > 1 and ids.numel() == T * self.sp_size:
            ids = ids[self.sp_rank * T:(self.sp_rank + 1) * T]               # the global row was passed: keep the local shard
        return MixerContext(cos, sin, cu_seq_lens_q, max_length_q, self.sp_group, self.sp_size, self.sp_rank, ids, extras)

    def forward(self, input_ids=None, position_ids=None, inputs_embeds=None, cu_seq_lens_q=None, max_length_q=None,
                return_context: bool = False, **extras):
        if inputs_embeds is None:
            inputs_embeds = self.embed_tokens(input_ids)
        h = inputs_embeds.reshape(-1, inputs_embeds.shape[-1])
        ctx = self.context(h.shape[0], position_ids, cu_seq_lens_q, max_length_q, input_ids, h.device, extras or None)
        res = None
        for layer in self.layers:
            h, res = layer(h, res, ctx)
        h, _ = self.norm(h, res)
        return (h.unsqueeze(0), ctx) if return_context else h.unsqueeze(0)


class NextNPredictLayer(nn.Module):
    """DeepSeek-style prediction depth (`enorm`, `hnorm`, `eh_proj`, one decoder block, `final_layernorm`):
    `h' = block(eh_proj([enorm(emb(ids << 1)) | hnorm(h)]))` (models/bailing_hybrid/modeling_bailing_moe_v3.py:1005-1084
    and models/deepseek_v4/mtp.py of the reference)."""

    def __init__(self, config: Any, block: nn.Module, dtype=None):
        super().__init__()
        h, eps = config.hidden_size, config.rms_norm_eps
        self.enorm, self.hnorm = RMSNorm(h, eps, dtype), RMSNorm(h, eps, dtype)
        self.eh_proj = nn.Linear(2 * h, h, bias=False, dtype=dtype)
        self.block = block
        self.final_layernorm = RMSNorm(h, eps, dtype)

    def forward(self, emb, hidden, ctx: MixerContext):
        x = torch.cat((self.enorm(emb), self.hnorm(hidden)), -1)
        m, res = self.block(ops.linear(x, self.eh_proj.weight), None, ctx)
        out, _ = self.final_layernorm(m, res)
        return out


def run_nextn_layers(layers, input_ids, hidden, embed_tokens, ctx: MixerContext, pad_token_id: int = 0,
                     sp_slice: Callable[[torch.Tensor], torch.Tensor] | None = None) -> list[torch.Tensor]:
    outs, ids, cur = [], input_ids, hidden
    for layer in layers:
        ids = roll_left_in_sequences(ids, ctx.cu_seqlens, pad_token_id)
        emb = embed_tokens(ids).reshape(-1, hidden.shape[-1])
        if sp_slice is not None:
            emb = sp_slice(emb)
        cur = layer(emb, cur, ctx)
        outs.append(cur)
    return outs
