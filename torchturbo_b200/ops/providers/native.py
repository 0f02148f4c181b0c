"""Plain PyTorch formulations of every operator.

They are (a) the implementations used on CPU and under `OpPolicy.NATIVE`, and (b) the oracle every
CUDA kernel is tested against.  Each one restates the numerics contract of the corresponding
reference provider (ops/providers/native/*.py in the reference) in independent code.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..base import OpImpl, OpImplKind
from ..moe import MoEPermutation
from ..registry import register_op


def _native(op_name: str, impl_name: str | None = None, priority: int = 0):
    return register_op(op_name=op_name, impl_name=impl_name or f"torch_{op_name}", kind=OpImplKind.NATIVE,
                       priority=priority)


# ------------------------------------------------------------------------------------------------
# normalisation / activations
# ------------------------------------------------------------------------------------------------
def rms_norm_ref(x, weight, eps, residual=None, one_plus_weight=False):
    if residual is not None:
        x = x + residual
    dt = x.dtype
    xf = x.float()
    xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dt)
    w = weight.to(dt)
    y = xn * ((1.0 + w) if one_plus_weight else w)
    return (y, x) if residual is not None else y


@_native("rms_norm")
class TorchRMSNorm(OpImpl):
    """fp32 `x * rsqrt(mean(x^2) + eps)`, cast to the input dtype, then `* weight`."""

    def __call__(self, x, weight, eps=1e-6, *, residual=None, one_plus_weight=False):
        return rms_norm_ref(x, weight, eps, residual, one_plus_weight)


def layer_norm_ref(x, weight, bias, eps=1e-6):
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), bias.float(), eps).to(x.dtype)


@_native("layer_norm")
class TorchLayerNorm(OpImpl):
    """fp32 LayerNorm with affine weight and bias, cast back to the input dtype."""

    def __call__(self, x, weight, bias, eps=1e-6):
        return layer_norm_ref(x, weight, bias, eps)


def bias_act_ref(x, bias, act=None, residual=None):
    v = x.float() + bias.float()
    if act in ("gelu_tanh", "gelu_pytorch_tanh"):
        v = F.gelu(v, approximate="tanh")
    elif act in ("gelu", "gelu_erf"):
        v = F.gelu(v)
    elif act not in (None, "none", "identity"):
        raise ValueError(f"unknown activation {act!r}")
    if residual is not None:
        v = v + residual.float()
    return v.to(x.dtype)


@_native("bias_act")
class TorchBiasAct(OpImpl):
    """`act(x + bias) (+ residual)`: the elementwise tail of a biased projection."""

    def __call__(self, x, bias, act=None, *, residual=None):
        return bias_act_ref(x, bias, act, residual)


def swiglu_ref(x, probs=None):
    gate, up = x.chunk(2, dim=-1)
    y = F.silu(gate) * up
    if probs is not None:
        y = (y.float() * probs.reshape(-1, 1).float()).to(x.dtype)
    return y


@_native("swiglu")
class TorchSwiGLU(OpImpl):
    """`silu(gate) * up` on `[gate | up]` halves; optional per-row probability applied after the activation."""

    def __call__(self, x, *, probs=None):
        return swiglu_ref(x, probs)


@_native("gated_activation")
class TorchGatedActivation(OpImpl):
    """Gated activation with optional clamping (`up` to [-limit, limit]; `gate` to <= limit before the
    activation), computed in fp32 (ops/providers/native/gated_activation.py:15-44 in the reference)."""

    def __call__(self, x, *, activation: str = "silu", limit: float | None = None, probs=None):
        gate, up = x.float().chunk(2, dim=-1)
        if limit is not None:
            gate = gate.clamp(max=limit)
            up = up.clamp(min=-limit, max=limit)
        act = {"silu": F.silu, "gelu": F.gelu, "relu": F.relu, "sigmoid": torch.sigmoid}[activation]
        y = act(gate) * up
        if probs is not None:
            y = y * probs.reshape(-1, 1).float()
        return y.to(x.dtype)


# ------------------------------------------------------------------------------------------------
# GEMM-shaped ops
# ------------------------------------------------------------------------------------------------
@_native("linear")
class TorchLinear(OpImpl):
    def __call__(self, x, weight, *, residual=None):
        y = F.linear(x, weight)
        return y + residual if residual is not None else y


@_native("router_gating")
class TorchRouterGating(OpImpl):
    """Router logits `x @ W^T` returned in fp32."""

    def __call__(self, x, weight):
        return F.linear(x, weight.to(x.dtype)).float()


@_native("linear_swiglu")
class TorchLinearSwiGLU(OpImpl):
    """`swiglu(x @ W^T)` for a fused `[gate; up]` weight of shape `[2F, H]`."""

    def __call__(self, x, weight):
        return swiglu_ref(F.linear(x, weight))


def grouped_matmul_ref(x, w, tokens_per_expert):
    """`y[rows_e] = x[rows_e] @ w[e]` for densely packed expert-major rows; `w` is `[E, in, out]`."""
    counts = tokens_per_expert.tolist() if isinstance(tokens_per_expert, torch.Tensor) else list(tokens_per_expert)
    out = x.new_zeros(x.shape[0], w.shape[-1])
    start = 0
    for e, n in enumerate(counts):
        if n:
            out[start:start + n] = x[start:start + n] @ w[e]
        start += n
    return out


@_native("grouped_matmul")
class TorchGroupedMatmul(OpImpl):
    def __call__(self, x, w, tokens_per_expert):
        return grouped_matmul_ref(x, w, tokens_per_expert)


@_native("matmul_add")
class TorchMatmulAdd(OpImpl):
    """`acc += lhs^T @ rhs` accumulated in `acc`'s dtype (fp32 weight-gradient accumulator)."""

    def __call__(self, acc, lhs, rhs):
        acc.addmm_(lhs.t().to(acc.dtype), rhs.to(acc.dtype))
        return acc


@_native("moe_experts")
class TorchMoEExperts(OpImpl):
    """fc1 -> SwiGLU * prob -> fc2 over packed rows.  `w1: [E, H, 2F]`, `w2: [E, F, H]`."""

    def __call__(self, perm: MoEPermutation, w1, w2, tokens_per_expert=None):
        x = perm.tokens
        if perm.padded:
            seg, cnt = perm.seg_start.tolist(), perm.counts.tolist()
            out = x.new_zeros(x.shape[0], w2.shape[-1])
            for e, n in enumerate(cnt):
                if n:
                    r = slice(seg[e], seg[e] + n)
                    h = swiglu_ref(x[r] @ w1[e], perm.probs[r] if perm.probs is not None else None)
                    out[r] = h @ w2[e]
            return out
        h = grouped_matmul_ref(x, w1, tokens_per_expert)
        h = swiglu_ref(h, perm.probs)
        return grouped_matmul_ref(h, w2, tokens_per_expert)


# ------------------------------------------------------------------------------------------------
# losses
# ------------------------------------------------------------------------------------------------
@_native("cross_entropy_loss")
class TorchCrossEntropy(OpImpl):
    """Sum of fp32 cross entropies, `ignore_index=-100`."""

    def __call__(self, logits, labels, *, ignore_index: int = -100):
        return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1), reduction="sum",
                               ignore_index=ignore_index)


@_native("linear_cross_entropy")
class TorchLinearCrossEntropy(OpImpl):
    """`sum CE(hidden @ W^T, labels)`; the plain formulation materialises the logits chunk by chunk under
    autograd.  Returns a scalar fp32 sum."""

    def __call__(self, hidden, weight, labels, *, chunk_size: int = 1024, ignore_index: int = -100):
        total = hidden.new_zeros((), dtype=torch.float32)
        h2, l2 = hidden.reshape(-1, hidden.shape[-1]), labels.reshape(-1)
        for s in range(0, h2.shape[0], chunk_size):
            lg = F.linear(h2[s:s + chunk_size], weight).float()
            total = total + F.cross_entropy(lg, l2[s:s + chunk_size], reduction="sum", ignore_index=ignore_index)
        return total


# ------------------------------------------------------------------------------------------------
# MoE routing / permutation
# ------------------------------------------------------------------------------------------------
def router_topk_ref(logits, k, score_fn, expert_bias=None, scaling=1.0, valid_mask=None):
    """Returns (topk_idx int64 [T,k], topk_prob fp32 [T,k], stats) with the aux statistics
    `score_sum[E]` / `aux_counts[E]` over valid tokens, routing `counts[E]` and per-token `lse`."""
    lg = logits.float()
    T, E = lg.shape
    if score_fn == "softmax_post":
        sel = lg + expert_bias if expert_bias is not None else lg
        idx = torch.topk(sel, k, dim=-1).indices
        prob = torch.softmax(lg.gather(1, idx), dim=-1)
        norm_scores = torch.softmax(lg, dim=-1)
    elif score_fn == "softmax_pre":
        sc = torch.softmax(lg, dim=-1)
        idx = torch.topk(sc + expert_bias if expert_bias is not None else sc, k, dim=-1).indices
        prob = sc.gather(1, idx)
        norm_scores = sc
    elif score_fn == "sigmoid":
        sc = torch.sigmoid(lg)
        idx = torch.topk(sc + expert_bias if expert_bias is not None else sc, k, dim=-1).indices
        prob = sc.gather(1, idx)
        if k > 1:
            prob = prob / (prob.sum(-1, keepdim=True) + 1e-20)
        norm_scores = sc / (sc.sum(-1, keepdim=True) + 1e-20)
    else:
        raise ValueError(f"unknown score function {score_fn!r}")
    prob = prob * scaling
    vm = torch.ones(T, dtype=torch.bool, device=lg.device) if valid_mask is None else valid_mask.bool()
    aux_idx = idx if expert_bias is None else torch.topk(norm_scores, k, dim=-1).indices
    stats = dict(
        score_sum=(norm_scores * vm[:, None]).sum(0),
        aux_counts=torch.bincount(aux_idx[vm].reshape(-1), minlength=E),
        counts=torch.bincount(idx.reshape(-1), minlength=E),
        lse=torch.logsumexp(lg, dim=-1),
    )
    return idx, prob, stats


@_native("router_topk")
class TorchRouterTopK(OpImpl):
    def __call__(self, logits, k, score_fn="softmax_post", *, expert_bias=None, scaling=1.0, valid_mask=None):
        return router_topk_ref(logits, k, score_fn, expert_bias, scaling, valid_mask)


def moe_permutation_ref(tokens, expert_indices, probs=None, num_experts=None) -> MoEPermutation:
    T, k = expert_indices.shape
    flat_e = expert_indices.reshape(-1).long()
    order = torch.argsort(flat_e, stable=True)          # (expert, token) order: token-major input + stable sort
    src_token = torch.arange(T, device=tokens.device).repeat_interleave(k)
    packed = tokens.index_select(0, src_token[order])
    row = torch.empty_like(order)
    row[order] = torch.arange(order.numel(), device=order.device)
    return MoEPermutation(
        tokens=packed,
        probs=probs.reshape(-1)[order] if probs is not None else None,
        row_indices=row.reshape(T, k).to(torch.int32),
        expert_indices=expert_indices.long(),
    )


@_native("moe_permutation")
class TorchMoEPermutation(OpImpl):
    def __call__(self, tokens, expert_indices, *, probs=None, num_experts=None):
        return moe_permutation_ref(tokens, expert_indices, probs, num_experts)


@_native("moe_unpermutation")
class TorchMoEUnpermutation(OpImpl):
    """Scatter-add the k expert rows of every token back to `[T, H]` (optionally weighted), cast to the
    input dtype; `residual` is added in the same pass."""

    def __call__(self, expert_out, perm: MoEPermutation, *, merging_probs=None, residual=None):
        T, k = perm.row_indices.shape
        rows = expert_out.index_select(0, perm.row_indices.reshape(-1).long()).reshape(T, k, -1)
        if merging_probs is not None:
            rows = rows.float() * merging_probs.reshape(T, k, 1).float()
        out = rows.float().sum(1)
        if residual is not None:
            out = out + residual.float()
        return out.to(expert_out.dtype)


@_native("moe_sort_chunks")
class TorchMoESortChunks(OpImpl):
    """Reorder contiguous row chunks: `split_sizes[i]` rows each, emitted in `sorted_idxs` order."""

    def __call__(self, x, split_sizes, sorted_idxs, *, probs=None):
        sizes = split_sizes.tolist() if isinstance(split_sizes, torch.Tensor) else list(split_sizes)
        order = sorted_idxs.tolist() if isinstance(sorted_idxs, torch.Tensor) else list(sorted_idxs)
        chunks = torch.split(x, sizes, dim=0)
        out = torch.cat([chunks[i] for i in order], dim=0)
        if probs is None:
            return out
        pch = torch.split(probs, sizes, dim=0)
        return out, torch.cat([pch[i] for i in order], dim=0)


# ------------------------------------------------------------------------------------------------
# rotary / attention
# ------------------------------------------------------------------------------------------------
def rope_ref(x, cos, sin):
    """Half-rotation RoPE.  x: [T, heads, D]; cos/sin: [T, D/2] (fp32)."""
    D = x.shape[-1]
    x1, x2 = x[..., : D // 2].float(), x[..., D // 2:].float()
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


@_native("rotary_position_embedding")
class TorchRoPE(OpImpl):
    def __call__(self, x, cos, sin):
        return rope_ref(x, cos, sin)


@_native("qk_norm_rope")
class TorchQKNormRope(OpImpl):
    """Split a fused `[T, (n_q + 2 n_kv) D]` projection, RMS-normalise q and k per head, rotate them."""

    def __call__(self, qkv, n_q, n_kv, head_dim, q_weight, k_weight, cos, sin, eps=1e-6):
        T = qkv.shape[0]
        q, k, v = qkv.split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], dim=-1)
        q, k, v = q.reshape(T, n_q, head_dim), k.reshape(T, n_kv, head_dim), v.reshape(T, n_kv, head_dim)
        if q_weight is not None:
            q, k = rms_norm_ref(q, q_weight, eps), rms_norm_ref(k, k_weight, eps)
        return rope_ref(q, cos, sin), rope_ref(k, cos, sin), v


def attention_ref(q, k, v, cu_seqlens, causal=True, scale=None, want_max_logits=False):
    """Packed variable-length attention.  q: [T, Hq, D]; k, v: [T, Hk, D]; `cu_seqlens` (host or device ints)
    partitions the first `cu[-1]` tokens into sequences; tokens after that are padding and produce zeros.
    Returns `out [T, Hq, D]` and, optionally, the per-head maximum pre-softmax logit (fp32, detached)."""
    T, Hq, D = q.shape
    Hk = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    offs = [int(c) for c in (cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)]
    out = q.new_zeros(T, Hq, v.shape[-1])        # value heads may be narrower than q/k heads (MLA)
    max_logits = torch.full((Hq,), -float("inf"), dtype=torch.float32, device=q.device)
    rep = Hq // Hk
    pieces = []
    for a, b in zip(offs[:-1], offs[1:]):
        if b <= a:
            continue
        qs = q[a:b].transpose(0, 1).float()                      # [Hq, L, D]
        ks = k[a:b].transpose(0, 1).repeat_interleave(rep, 0).float()
        vs = v[a:b].transpose(0, 1).repeat_interleave(rep, 0).float()
        s = qs @ ks.transpose(-1, -2) * scale
        if causal:
            L = b - a
            s = s.masked_fill(~torch.ones(L, L, dtype=torch.bool, device=q.device).tril(), -float("inf"))
        if want_max_logits:
            max_logits = torch.maximum(max_logits, s.detach().amax(dim=(1, 2)))
        o = torch.softmax(s, dim=-1) @ vs
        pieces.append((a, b, o.transpose(0, 1).to(q.dtype)))
    if pieces:
        # assemble without in-place writes on a leaf so autograd stays simple
        segs, pos = [], 0
        for a, b, o in pieces:
            if a > pos:
                segs.append(out[pos:a])
            segs.append(o)
            pos = b
        if pos < T:
            segs.append(out[pos:])
        out = torch.cat(segs, dim=0)
    return (out, max_logits) if want_max_logits else out


@_native("attention")
class TorchAttention(OpImpl):
    def __call__(self, q, k, v, cu_seqlens, max_seqlen=None, *, causal=True, scale=None):
        return attention_ref(q, k, v, cu_seqlens, causal, scale)


@_native("attention_with_max_logits")
class TorchAttentionWithMaxLogits(OpImpl):
    def __call__(self, q, k, v, cu_seqlens, max_seqlen=None, *, causal=True, scale=None):
        return attention_ref(q, k, v, cu_seqlens, causal, scale, want_max_logits=True)
