"""Token mixers of the hybrid model families, all on packed token-major activations `[T_local, H]`.

    GatedAttention        softmax attention with per-head QK norm, partial rotary and a sigmoid output gate
                          (Qwen3.5 "full_attention" layers; models/qwen3_5/modeling_qwen3_5.py:736-811 of the reference)
    GatedDeltaNet         gated delta rule linear attention with a short causal convolution and a gated RMSNorm
                          (Qwen3.5 "linear_attention" layers; modeling_qwen3_5.py:469-650)
    MLAttention           multi-head latent attention: low-rank q / kv projections, decoupled rotary key
                          (DeepSeek-V3 / Kimi / Bailing / GLM; models/kimi_k25/modeling_deepseek.py)
    KimiDeltaAttention    delta rule with per-channel decay, low-rank gate projections and an output gate
                          (models/bailing_hybrid/modeling_bailing_moe_v3.py, attention.py:23-251)

Every mixer takes a `MixerContext` (rotary tables, global packed metadata, sequence-parallel group).  Under Ulysses
sequence parallelism softmax attention trades sequence for heads around the attention op; the linear-attention
mixers do the same around convolution + recurrence and slice their per-head parameters to the local heads
(models/modules/attention/gdn/forward.py:30-237 of the reference).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import ops
from .attention.ulysses import gather_heads_scatter_seq, gather_seq_scatter_heads, ulysses_attention
from .transformer import RMSNorm


@dataclass
class MixerContext:
    cos: torch.Tensor                      # [T_local, rot/2] fp32
    sin: torch.Tensor
    cu_seqlens: torch.Tensor               # global boundaries (host int32)
    max_seqlen: int
    sp_group: Any = None
    sp_size: int = 1
    sp_rank: int = 0
    input_ids: Optional[torch.Tensor] = None
    extras: Optional[dict] = None          # family-specific side inputs (block masks, indexer caches, ...)


def apply_partial_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """Rotate the first `2 * cos.shape[-1]` channels of `[T, heads, D]`; the rest pass through.  `interleaved`
    means the checkpoint stores rotary pairs as (0,1),(2,3),... : they are regrouped to the half layout first
    (a fixed permutation applied to q and k alike, so scores are unchanged)."""
    rd = 2 * cos.shape[-1]
    xr, xp = x[..., :rd], x[..., rd:]
    if interleaved:
        xr = xr.unflatten(-1, (rd // 2, 2)).transpose(-1, -2).flatten(-2)
    xr = ops.rotary_position_embedding(xr.contiguous(), cos, sin)
    return xr if xp.shape[-1] == 0 else torch.cat((xr, xp), dim=-1)


class GatedRMSNorm(nn.Module):
    """`weight * rmsnorm(x) * silu(gate)` over the last dimension (norm first, then the gate)."""

    def __init__(self, dim: int, eps: float = 1e-6, dtype=None, activation: str = "silu"):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))
        self.eps, self.activation = eps, activation

    def forward(self, x, gate):
        y = ops.rms_norm(x, self.weight, self.eps)
        g = gate.float()
        g = F.silu(g) if self.activation == "silu" else torch.sigmoid(g)
        return (y.float() * g).to(x.dtype)


# ------------------------------------------------------------------------------------------------
# softmax attention with an output gate
# ------------------------------------------------------------------------------------------------
class GatedAttention(nn.Module):
    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.n_q, self.n_kv, self.head_dim = config.num_attention_heads, config.num_key_value_heads, config.head_dim
        H = config.hidden_size
        bias = getattr(config, "attention_bias", False)
        self.output_gate = getattr(config, "attn_output_gate", True)
        self.q_proj = nn.Linear(H, self.n_q * self.head_dim * (2 if self.output_gate else 1), bias=bias, dtype=dtype)
        self.k_proj = nn.Linear(H, self.n_kv * self.head_dim, bias=bias, dtype=dtype)
        self.v_proj = nn.Linear(H, self.n_kv * self.head_dim, bias=bias, dtype=dtype)
        self.o_proj = nn.Linear(self.n_q * self.head_dim, H, bias=bias, dtype=dtype)
        opw = getattr(config, "norm_one_plus_weight", True)
        self.q_norm = RMSNorm(self.head_dim, config.rms_norm_eps, dtype, one_plus_weight=opw)
        self.k_norm = RMSNorm(self.head_dim, config.rms_norm_eps, dtype, one_plus_weight=opw)
        self.scale = self.head_dim ** -0.5
        self.causal = True
        self.qk_clip_state = None

    @staticmethod
    def _lin(x, m: nn.Linear):
        y = ops.linear(x, m.weight)
        return y if m.bias is None else y + m.bias

    def forward(self, x, ctx: MixerContext):
        T = x.shape[0]
        qg = self._lin(x, self.q_proj).view(T, self.n_q, -1)
        if self.output_gate:
            q, gate = qg[..., : self.head_dim], qg[..., self.head_dim:].reshape(T, -1)
        else:
            q, gate = qg, None
        k = self._lin(x, self.k_proj).view(T, self.n_kv, self.head_dim)
        v = self._lin(x, self.v_proj).view(T, self.n_kv, self.head_dim)
        q, k = self.q_norm(q.contiguous()), self.k_norm(k)
        q, k = apply_partial_rope(q, ctx.cos, ctx.sin), apply_partial_rope(k, ctx.cos, ctx.sin)
        want_ml = self.qk_clip_state is not None
        out = ulysses_attention(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, sp_group=ctx.sp_group, sp_size=ctx.sp_size,
                                causal=self.causal, scale=self.scale, want_max_logits=want_ml)
        if want_ml:
            out, ml = out
            self.qk_clip_state.update(ml)
        out = out.reshape(T, -1)
        if gate is not None:
            out = out * torch.sigmoid(gate)
        return self._lin(out, self.o_proj)


# ------------------------------------------------------------------------------------------------
# gated delta rule
# ------------------------------------------------------------------------------------------------
def _head_slice(t: torch.Tensor, heads: int, sp_size: int, sp_rank: int, dim: int = 0) -> torch.Tensor:
    """Rows of a per-head parameter that belong to this rank's heads (`heads` consecutive blocks on `dim`)."""
    if sp_size <= 1:
        return t
    per = t.shape[dim] // heads
    hl = heads // sp_size
    return t.narrow(dim, sp_rank * hl * per, hl * per)


class GatedDeltaNet(nn.Module):
    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__()
        self.layer_idx = layer_idx
        H = config.hidden_size
        self.n_v, self.n_k = config.linear_num_value_heads, config.linear_num_key_heads
        self.dk, self.dv = config.linear_key_head_dim, config.linear_value_head_dim
        self.key_dim, self.value_dim = self.dk * self.n_k, self.dv * self.n_v
        self.kernel = config.linear_conv_kernel_dim
        self.in_proj_qkv = nn.Linear(H, 2 * self.key_dim + self.value_dim, bias=False, dtype=dtype)
        self.in_proj_z = nn.Linear(H, self.value_dim, bias=False, dtype=dtype)
        self.in_proj_b = nn.Linear(H, self.n_v, bias=False, dtype=dtype)
        self.in_proj_a = nn.Linear(H, self.n_v, bias=False, dtype=dtype)
        # depthwise conv taps over the concatenated [q | k | v] channels, stored as Conv1d does: [C, 1, W]
        self.conv1d = nn.Conv1d(2 * self.key_dim + self.value_dim, 2 * self.key_dim + self.value_dim, self.kernel,
                                groups=2 * self.key_dim + self.value_dim, bias=False, padding=self.kernel - 1, dtype=dtype)
        self.dt_bias = nn.Parameter(torch.ones(self.n_v, dtype=dtype))
        self.A_log = nn.Parameter(torch.zeros(self.n_v, dtype=dtype))
        self.norm = GatedRMSNorm(self.dv, config.rms_norm_eps, dtype)
        self.out_proj = nn.Linear(self.value_dim, H, bias=False, dtype=dtype)

    def reset_parameters_extra(self, generator=None) -> None:
        with torch.no_grad():
            self.dt_bias.fill_(1.0)
            self.A_log.copy_(torch.empty(self.n_v).uniform_(1e-3, 16, generator=generator).log())

    def forward(self, x, ctx: MixerContext):
        T = x.shape[0]
        sp, r = ctx.sp_size, ctx.sp_rank
        if sp > 1 and (self.n_k % sp or self.n_v % sp):
            raise ValueError(f"linear-attention heads ({self.n_k} key / {self.n_v} value) must divide by sp={sp}")
        qkv = ops.linear(x, self.in_proj_qkv.weight)
        z = ops.linear(x, self.in_proj_z.weight).view(T, self.n_v, self.dv)
        b = ops.linear(x, self.in_proj_b.weight)
        a = ops.linear(x, self.in_proj_a.weight)
        q, k, v = qkv.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q, k, v = q.reshape(T, self.n_k, self.dk), k.reshape(T, self.n_k, self.dk), v.reshape(T, self.n_v, self.dv)
        w = self.conv1d.weight.squeeze(1)
        wq, wk, wv = w.split([self.key_dim, self.key_dim, self.value_dim], dim=0)
        A_log, dt_bias = self.A_log, self.dt_bias
        if sp > 1:
            # full sequence of the local heads; per-head parameters sliced to match
            q, k, v = (gather_seq_scatter_heads(t.contiguous(), ctx.sp_group, sp) for t in (q, k, v))
            ba = gather_seq_scatter_heads(torch.stack((b, a), -1).contiguous(), ctx.sp_group, sp)
            b, a = ba[..., 0], ba[..., 1]
            wq, wk, wv = (_head_slice(t, h, sp, r) for t, h in ((wq, self.n_k), (wk, self.n_k), (wv, self.n_v)))
            A_log, dt_bias = _head_slice(A_log, self.n_v, sp, r), _head_slice(dt_bias, self.n_v, sp, r)
        Tg, hk, hv = q.shape[0], q.shape[1], v.shape[1]
        cu = ctx.cu_seqlens
        mixed = torch.cat((q.reshape(Tg, -1), k.reshape(Tg, -1), v.reshape(Tg, -1)), -1).unsqueeze(0)
        mixed, _ = ops.causal_conv1d(mixed, torch.cat((wq, wk, wv), 0), None, activation="silu", cu_seqlens=cu)
        q, k, v = mixed[0].split([hk * self.dk, hk * self.dk, hv * self.dv], dim=-1)
        q, k, v = q.reshape(1, Tg, hk, self.dk), k.reshape(1, Tg, hk, self.dk), v.reshape(1, Tg, hv, self.dv)
        beta = torch.sigmoid(b.float()).unsqueeze(0)
        g = (-A_log.float().exp() * F.softplus(a.float() + dt_bias.float())).unsqueeze(0)
        if hv // hk > 1:
            q, k = q.repeat_interleave(hv // hk, dim=2), k.repeat_interleave(hv // hk, dim=2)
        o, _ = ops.gated_delta_rule(q, k, v, g, beta, use_qk_l2norm_in_kernel=True, cu_seqlens=cu)
        o = o[0]                                                            # [Tg, hv, dv]
        if sp > 1:
            o = gather_heads_scatter_seq(o.contiguous(), ctx.sp_group, sp)  # [T_local, n_v, dv]
        o = self.norm(o.reshape(-1, self.dv), z.reshape(-1, self.dv)).reshape(T, self.value_dim)
        return ops.linear(o, self.out_proj.weight)


# ------------------------------------------------------------------------------------------------
# multi-head latent attention
# ------------------------------------------------------------------------------------------------
def yarn_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


class MLAttention(nn.Module):
    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__()
        self.layer_idx = layer_idx
        H = config.hidden_size
        self.n_heads = config.num_attention_heads
        self.q_lora, self.kv_lora = getattr(config, "q_lora_rank", None), config.kv_lora_rank
        self.d_nope, self.d_rope, self.d_v = config.qk_nope_head_dim, config.qk_rope_head_dim, config.v_head_dim
        self.d_qk = self.d_nope + self.d_rope
        # the latent norms keep the norm class's default epsilon in every published MLA implementation, whatever
        # `rms_norm_eps` says (transformers: deepseek_v3/modeling_deepseek_v3.py `DeepseekV3RMSNorm(config.q_lora_rank)`)
        eps = getattr(config, "mla_latent_norm_eps", 1e-6)
        bias = getattr(config, "attention_bias", False) or getattr(config, "use_qkv_bias", False)
        if self.q_lora:
            self.q_a_proj = nn.Linear(H, self.q_lora, bias=bias, dtype=dtype)
            self.q_a_layernorm = RMSNorm(self.q_lora, eps, dtype)
            self.q_b_proj = nn.Linear(self.q_lora, self.n_heads * self.d_qk, bias=False, dtype=dtype)
        else:
            self.q_proj = nn.Linear(H, self.n_heads * self.d_qk, bias=False, dtype=dtype)
        self.kv_a_proj_with_mqa = nn.Linear(H, self.kv_lora + self.d_rope, bias=bias, dtype=dtype)
        self.kv_a_layernorm = RMSNorm(self.kv_lora, eps, dtype)
        self.kv_b_proj = nn.Linear(self.kv_lora, self.n_heads * (self.d_nope + self.d_v), bias=False, dtype=dtype)
        self.o_proj = nn.Linear(self.n_heads * self.d_v, H, bias=bias, dtype=dtype)
        self.gate_kind = getattr(config, "gated_attention_proj_granularity_type", None)
        if self.gate_kind not in (None, "head_wise", "element_wise"):
            raise ValueError(f"unknown attention gate granularity {self.gate_kind!r}")
        self.g_proj = None if self.gate_kind is None else nn.Linear(
            H, self.n_heads * (1 if self.gate_kind == "head_wise" else self.d_v), bias=False, dtype=dtype)
        self.rope_interleaved = getattr(config, "rope_interleave", True)
        self.scale = self.d_qk ** -0.5
        rs = getattr(config, "rope_scaling", None) or {}
        if rs.get("mscale_all_dim"):
            m = yarn_mscale(rs.get("factor", 1.0), rs["mscale_all_dim"])
            self.scale *= m * m
        self.causal = True
        self.qk_clip_state = None

    def project_q(self, x):
        if self.q_lora:
            qa = ops.linear(x, self.q_a_proj.weight)
            if self.q_a_proj.bias is not None:
                qa = qa + self.q_a_proj.bias
            return ops.linear(self.q_a_layernorm(qa), self.q_b_proj.weight)
        return ops.linear(x, self.q_proj.weight)

    def forward(self, x, ctx: MixerContext):
        T = x.shape[0]
        q = self.project_q(x).view(T, self.n_heads, self.d_qk)
        ckv = ops.linear(x, self.kv_a_proj_with_mqa.weight)
        if self.kv_a_proj_with_mqa.bias is not None:
            ckv = ckv + self.kv_a_proj_with_mqa.bias
        c, k_rope = ckv[:, : self.kv_lora], ckv[:, self.kv_lora:].reshape(T, 1, self.d_rope)
        kv = ops.linear(self.kv_a_layernorm(c.contiguous()), self.kv_b_proj.weight).view(T, self.n_heads, self.d_nope + self.d_v)
        k_nope, v = kv[..., : self.d_nope], kv[..., self.d_nope:]
        q_rope = apply_partial_rope(q[..., self.d_nope:].contiguous(), ctx.cos, ctx.sin, self.rope_interleaved)
        k_rope = apply_partial_rope(k_rope.contiguous(), ctx.cos, ctx.sin, self.rope_interleaved)
        q = torch.cat((q[..., : self.d_nope], q_rope), -1)
        k = torch.cat((k_nope, k_rope.expand(T, self.n_heads, self.d_rope)), -1)
        want_ml = self.qk_clip_state is not None
        out = ulysses_attention(q, k, v.contiguous(), ctx.cu_seqlens, ctx.max_seqlen, sp_group=ctx.sp_group,
                                sp_size=ctx.sp_size, causal=self.causal, scale=self.scale, want_max_logits=want_ml)
        if want_ml:
            out, ml = out
            self.qk_clip_state.update(ml)
        if self.g_proj is not None:
            gate = torch.sigmoid(ops.linear(x, self.g_proj.weight).float()).to(out.dtype)
            out = out * gate.view(T, self.n_heads, -1)
        y = ops.linear(out.reshape(T, self.n_heads * self.d_v), self.o_proj.weight)
        return y if self.o_proj.bias is None else y + self.o_proj.bias


# ------------------------------------------------------------------------------------------------
# Kimi delta attention
# ------------------------------------------------------------------------------------------------
class KimiDeltaAttention(nn.Module):
    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__()
        self.layer_idx = layer_idx
        H = config.hidden_size
        self.n_heads = getattr(config, "linear_num_heads", None) or config.num_attention_heads
        self.dk = getattr(config, "linear_key_head_dim", None) or config.head_dim
        self.dv = getattr(config, "linear_value_head_dim", None) or self.dk
        self.kernel = getattr(config, "short_conv_kernel_size", None) or getattr(config, "linear_conv_kernel_dim", 4)
        kd, vd = self.n_heads * self.dk, self.n_heads * self.dv
        self.q_proj = nn.Linear(H, kd, bias=False, dtype=dtype)
        self.k_proj = nn.Linear(H, kd, bias=False, dtype=dtype)
        self.v_proj = nn.Linear(H, vd, bias=False, dtype=dtype)
        self.q_conv1d = nn.Conv1d(kd, kd, self.kernel, groups=kd, bias=False, padding=self.kernel - 1, dtype=dtype)
        self.k_conv1d = nn.Conv1d(kd, kd, self.kernel, groups=kd, bias=False, padding=self.kernel - 1, dtype=dtype)
        self.v_conv1d = nn.Conv1d(vd, vd, self.kernel, groups=vd, bias=False, padding=self.kernel - 1, dtype=dtype)
        rank = getattr(config, "linear_gate_low_rank_dim", None) or self.dv
        self.low_rank = not getattr(config, "no_kda_lora", False)
        if self.low_rank:
            self.f_a_proj = nn.Linear(H, rank, bias=False, dtype=dtype)
            self.f_b_proj = nn.Linear(rank, kd, bias=False, dtype=dtype)
        else:
            self.f_proj = nn.Linear(H, kd, bias=False, dtype=dtype)
        self.b_proj = nn.Linear(H, self.n_heads, bias=False, dtype=dtype)
        self.A_log = nn.Parameter(torch.zeros(self.n_heads, dtype=dtype))
        self.dt_bias = nn.Parameter(torch.zeros(kd, dtype=dtype))
        if self.low_rank:
            self.g_a_proj = nn.Linear(H, rank, bias=False, dtype=dtype)
            self.g_b_proj = nn.Linear(rank, vd, bias=False, dtype=dtype)
        else:
            self.g_proj = nn.Linear(H, vd, bias=False, dtype=dtype)
        self.o_norm = GatedRMSNorm(self.dv, config.rms_norm_eps, dtype, activation="sigmoid")
        self.o_proj = nn.Linear(vd, H, bias=False, dtype=dtype)
        self.gate_lower_bound = getattr(config, "kda_lower_bound", None) if getattr(config, "kda_safe_gate", False) \
            else getattr(config, "linear_gate_lower_bound", None)

    def reset_parameters_extra(self, generator=None) -> None:
        with torch.no_grad():
            self.A_log.copy_(torch.empty(self.n_heads).uniform_(1.0, 16.0, generator=generator).log())
            self.dt_bias.zero_()

    def forward(self, x, ctx: MixerContext):
        T = x.shape[0]
        sp, r, Hh = ctx.sp_size, ctx.sp_rank, self.n_heads
        if sp > 1 and Hh % sp:
            raise ValueError(f"KDA heads ({Hh}) must divide by sp={sp}")
        q = ops.linear(x, self.q_proj.weight).view(T, Hh, self.dk)
        k = ops.linear(x, self.k_proj.weight).view(T, Hh, self.dk)
        v = ops.linear(x, self.v_proj.weight).view(T, Hh, self.dv)
        g = ops.linear(ops.linear(x, self.f_a_proj.weight), self.f_b_proj.weight) if self.low_rank \
            else ops.linear(x, self.f_proj.weight)
        g = g.view(T, Hh, self.dk)
        beta = ops.linear(x, self.b_proj.weight)
        wq, wk, wv = (m.weight.squeeze(1) for m in (self.q_conv1d, self.k_conv1d, self.v_conv1d))
        A_log, dt_bias = self.A_log, self.dt_bias
        if sp > 1:
            q, k, v, g = (gather_seq_scatter_heads(t.contiguous(), ctx.sp_group, sp) for t in (q, k, v, g))
            beta = gather_seq_scatter_heads(beta.unsqueeze(-1).contiguous(), ctx.sp_group, sp).squeeze(-1)
            wq, wk, wv = (_head_slice(t, Hh, sp, r) for t in (wq, wk, wv))
            A_log, dt_bias = _head_slice(A_log, Hh, sp, r), _head_slice(dt_bias, Hh, sp, r)
        Tg, hl = q.shape[0], q.shape[1]
        cu = ctx.cu_seqlens
        q, _ = ops.causal_conv1d(q.reshape(1, Tg, -1), wq, None, activation="silu", cu_seqlens=cu)
        k, _ = ops.causal_conv1d(k.reshape(1, Tg, -1), wk, None, activation="silu", cu_seqlens=cu)
        v, _ = ops.causal_conv1d(v.reshape(1, Tg, -1), wv, None, activation="silu", cu_seqlens=cu)
        o, _ = ops.kda(q, k, v, g.unsqueeze(0), beta.unsqueeze(0), A_log=A_log, dt_bias=dt_bias,
                       use_qk_l2norm_in_kernel=True, use_beta_sigmoid_in_kernel=True, use_gate_in_kernel=True,
                       safe_gate=self.gate_lower_bound is not None, lower_bound=self.gate_lower_bound, cu_seqlens=cu)
        o = o[0]
        if sp > 1:
            o = gather_heads_scatter_seq(o.contiguous(), ctx.sp_group, sp)
        gate = ops.linear(ops.linear(x, self.g_a_proj.weight), self.g_b_proj.weight) if self.low_rank \
            else ops.linear(x, self.g_proj.weight)
        o = self.o_norm(o.reshape(-1, self.dv), gate.reshape(-1, self.dv)).reshape(T, -1)
        return ops.linear(o, self.o_proj.weight)
