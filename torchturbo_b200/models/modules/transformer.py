"""Decoder building blocks shared by the Qwen3-style model families.

All blocks work on packed token-major activations `[T, H]` (the batch dimension of a packed row is 1 and
is squeezed at the model boundary) and route every hot operation through `ops.*`, so the same module runs
on the torch formulations (CPU, oracle) and on the sm_100a kernels.  Projections are stored fused where a
fused GEMM pays (`qkv_proj`, `gate_up_proj`); the weight converter maps them to and from Hugging Face
per-projection tensors.

The residual stream is carried separately from the sub-layer output so that every residual add is fused
into the following RMSNorm kernel:   y, res = norm(h, residual=res)   means   res += h ; y = norm(res).
"""
from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn as nn

from ...ops import ops
from .attention.ulysses import ulysses_attention


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, dtype=None, one_plus_weight: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(dim, dtype=dtype) if one_plus_weight else torch.ones(dim, dtype=dtype))
        self.eps = eps
        self.one_plus_weight = one_plus_weight

    def forward(self, x, residual=None):
        return ops.rms_norm(x, self.weight, self.eps, residual=residual, one_plus_weight=self.one_plus_weight)


class RotaryEmbedding(nn.Module):
    """cos/sin tables `[T, D/2]` in fp32 from integer positions; `inv_freq` is a non-persistent buffer that
    is rebuilt after materialisation (meta-device construction leaves it uninitialised)."""

    def __init__(self, head_dim: int, theta: float = 1e6, inv_freq_dtype: torch.dtype = torch.float32):
        super().__init__()
        self.head_dim, self.theta, self.inv_freq_dtype = head_dim, theta, inv_freq_dtype
        self.register_buffer("inv_freq", self._make(None), persistent=False)

    def _make(self, device):
        expo = torch.arange(0, self.head_dim, 2, dtype=torch.float32, device=device) / self.head_dim
        return (1.0 / (self.theta ** expo)).to(self.inv_freq_dtype)

    def reset(self, device=None):
        self.inv_freq = self._make(device if device is not None else self.inv_freq.device)

    @torch.no_grad()
    def forward(self, position_ids: torch.Tensor):
        pos = position_ids.reshape(-1).float()
        ang = pos[:, None] * self.inv_freq.float()[None, :]
        return ang.cos(), ang.sin()


class Attention(nn.Module):
    """GQA attention with optional per-head QK RMSNorm (Qwen3) over packed variable-length sequences."""

    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.n_q, self.n_kv, self.head_dim = config.num_attention_heads, config.num_key_value_heads, config.head_dim
        H = config.hidden_size
        self.qkv_proj = nn.Linear(H, (self.n_q + 2 * self.n_kv) * self.head_dim, bias=getattr(config, "attention_bias", False), dtype=dtype)
        self.o_proj = nn.Linear(self.n_q * self.head_dim, H, bias=False, dtype=dtype)
        qk_norm = getattr(config, "qk_norm", True)
        self.q_norm = RMSNorm(self.head_dim, config.rms_norm_eps, dtype) if qk_norm else None
        self.k_norm = RMSNorm(self.head_dim, config.rms_norm_eps, dtype) if qk_norm else None
        self.scale = 1.0 / math.sqrt(self.head_dim)
        self.causal = True
        self.sp_group, self.sp_size = None, 1
        self.qk_clip_state = None  # set by the QK-clip controller when max-logit tracking is on

    def set_sequence_parallel(self, group, size: int) -> None:
        self.sp_group, self.sp_size = group, size

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        T = x.shape[0]
        qkv = ops.linear(x, self.qkv_proj.weight)
        if self.qkv_proj.bias is not None:
            qkv = qkv + self.qkv_proj.bias
        want_ml = self.qk_clip_state is not None
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        eps = self.q_norm.eps if self.q_norm is not None else 1e-6
        if self.sp_size > 1 and not want_ml and self._p2p_ok(qkv):
            # peer-memory path: QK-norm + RoPE are computed by the kernel that scatters heads to their owners
            from ...comm import ulysses_p2p

            q, k, v, ws = ulysses_p2p.qkv_exchange(qkv.contiguous(), self.n_q, self.n_kv, qw, kw, cos, sin, eps, self.sp_group)
            o = ops.attention(q, k, v, cu_seqlens, max_seqlen, causal=self.causal, scale=self.scale)
            out = ulysses_p2p.out_exchange(o, ws)
            return ops.linear(out.reshape(T, self.n_q * self.head_dim), self.o_proj.weight)
        q, k, v = ops.qk_norm_rope(qkv, self.n_q, self.n_kv, self.head_dim, qw, kw, cos, sin, eps)
        out = ulysses_attention(q, k, v, cu_seqlens, max_seqlen, sp_group=self.sp_group, sp_size=self.sp_size,
                                causal=self.causal, scale=self.scale, want_max_logits=want_ml)
        if want_ml:
            out, max_logits = out
            self.qk_clip_state.update(max_logits)
        return ops.linear(out.reshape(T, self.n_q * self.head_dim), self.o_proj.weight)

    def _p2p_ok(self, qkv) -> bool:
        if not qkv.is_cuda:
            return False
        from ...comm import ulysses_p2p

        return ulysses_p2p.usable(self.sp_group, qkv, self.n_q, self.n_kv, self.head_dim)


class DenseMLP(nn.Module):
    def __init__(self, hidden: int, inter: int, dtype=None):
        super().__init__()
        self.gate_up_proj = nn.Linear(hidden, 2 * inter, bias=False, dtype=dtype)
        self.down_proj = nn.Linear(inter, hidden, bias=False, dtype=dtype)

    def forward(self, x, input_ids=None):
        return ops.linear(ops.linear_swiglu(x, self.gate_up_proj.weight), self.down_proj.weight)


class DecoderLayer(nn.Module):
    def __init__(self, config: Any, layer_idx: int, mlp: nn.Module, dtype=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)
        self.self_attn = Attention(config, layer_idx, dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)
        self.mlp = mlp

    def forward(self, h, residual, cos, sin, cu_seqlens, max_seqlen, input_ids=None):
        """(h, residual) -> (h', residual'): `h` is the previous sub-layer output that has not been added to
        the residual stream yet (`residual is None` for the first layer)."""
        if residual is None:
            residual = h
            x = self.input_layernorm(h)
        else:
            x, residual = self.input_layernorm(h, residual)
        a = self.self_attn(x, cos, sin, cu_seqlens, max_seqlen)
        x, residual = self.post_attention_layernorm(a, residual)
        m = self.mlp(x, input_ids)
        if isinstance(m, tuple):
            m = m[0]
        return m, residual


class CausalLMOutput(dict):
    """Dict with attribute access (`out.loss`, `out.logits`, `out.hidden_states`)."""

    __getattr__ = dict.get

    def __setattr__(self, k, v):
        self[k] = v


def _register_output_pytree() -> None:
    """FSDP2 finds the tensors of a module's output with `torch.utils._pytree` (to hook the start of backward on
    them); a plain `dict` subclass would be an opaque leaf there, and a model whose only sharded unit is the root
    would never run its gradient reduction."""
    try:
        from torch.utils import _pytree as pytree

        pytree.register_pytree_node(
            CausalLMOutput,
            lambda d: (list(d.values()), list(d.keys())),
            lambda values, keys: CausalLMOutput(zip(keys, values)),
            serialized_type_name="torchturbo_b200.CausalLMOutput",
        )
    except Exception:  # noqa: BLE001 - already registered, or a torch build without the hook
        pass


_register_output_pytree()


def init_weights(module: nn.Module, std: float) -> None:
    for m in module.modules():
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=std)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=std)
        elif isinstance(m, RMSNorm):
            if m.one_plus_weight:
                nn.init.zeros_(m.weight)
            else:
                nn.init.ones_(m.weight)
