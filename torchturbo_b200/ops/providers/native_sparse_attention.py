"""Plain PyTorch formulations of the sparse-attention operators: `lightning_indexer` and `sparse_attention`
(+ `sparse_flash_mla`, the shared-KV form with sink logits used by the compressed-KV families).

The reference has these operators only as Ascend vendor kernels (ops/providers/npu/lightning_indexer.py:22-140,
sparse_flash_mla.py:224) and falls back to dense masked attention inside the models elsewhere
(models/glm_moe_dsa/modeling_glm_moe_dsa.py:320-333, models/deepseek_v4/modeling_deepseek_v4.py:562-616).  Here the
same math is one operator family on packed rows, so models call one op on every device.

    lightning_indexer   score[t, s] = sum_h w[t, h] * relu(scale * q[t, h] . k[s]) over the causal keys of t's sequence;
                        returns the `topk` best key positions per query (global row indices, -1 padded)
    sparse_attention    softmax attention of each query over its listed key rows only
    sparse_flash_mla    every head attends to one shared key/value row per position (K == V), over a causal sliding
                        window of the original rows plus listed rows of a compressed stream, with a per-head sink
                        logit in the softmax denominator
"""
from __future__ import annotations

import math

import torch

from ..base import OpImpl, OpImplKind
from ..registry import register_op
from .native_linear_attention import _bounds


def _native(op_name: str, impl_name: str):
    return register_op(op_name=op_name, impl_name=impl_name, kind=OpImplKind.NATIVE, priority=0)


@torch.no_grad()
def lightning_indexer_ref(q, k, weights, topk, cu_seqlens=None, scale=None, q_offset: int = 0, chunk: int = 1024):
    """q: [Tq, Hi, D]; k: [Tk, D]; weights: [Tq, Hi].  Query row `i` is key row `q_offset + i` (queries are a
    contiguous slice of the key rows: the local shard under sequence parallelism).  Returns int32 `[Tq, topk]`."""
    Tq, Hi, D = q.shape
    Tk = k.shape[0]
    scale = D ** -0.5 if scale is None else scale
    out = torch.full((Tq, topk), -1, dtype=torch.int32, device=q.device)
    kf = k.float()
    for a, b in _bounds(cu_seqlens, Tk):
        lo, hi = max(a, q_offset), min(b, q_offset + Tq)
        for s in range(lo, hi, chunk):
            e = min(s + chunk, hi)
            qs = q[s - q_offset:e - q_offset].float()                              # [c, Hi, D]
            sc = torch.relu(torch.einsum("chd,td->cht", qs, kf[a:e]) * scale)
            sc = torch.einsum("cht,ch->ct", sc, weights[s - q_offset:e - q_offset].float())
            pos_q = torch.arange(s, e, device=q.device)[:, None]
            pos_k = torch.arange(a, e, device=q.device)[None, :]
            sc = sc.masked_fill(pos_k > pos_q, -float("inf"))
            kk = min(topk, e - a)
            # a stable sort, not `topk`: ReLU makes exact ties common, and which of two tied keys `topk` returns depends on
            # the shape of the score block, i.e. on how the queries were sliced (sequence parallelism, chunking)
            val, idx = sc.sort(dim=-1, descending=True, stable=True)
            val, idx = val[:, :kk], idx[:, :kk]
            idx = (idx + a).to(torch.int32).masked_fill(~torch.isfinite(val), -1)
            out[s - q_offset:e - q_offset, :kk] = idx
    return out


def sparse_attention_ref(q, k, v, indices, scale=None, sinks=None, chunk: int = 512):
    """q: [Tq, H, D]; k: [Tk, Hk, D]; v: [Tk, Hk, Dv]; indices: [Tq, n] key rows (-1 = unused).  GQA by head
    repetition.  `sinks` [H] adds one virtual key per head that absorbs probability mass and contributes nothing."""
    Tq, H, D = q.shape
    Hk, Dv = k.shape[1], v.shape[-1]
    rep = H // Hk
    scale = D ** -0.5 if scale is None else scale
    outs = []
    for s in range(0, Tq, chunk):
        e = min(s + chunk, Tq)
        idx = indices[s:e].long()
        valid = idx >= 0
        safe = idx.clamp_min(0)
        kg = k[safe].float()                                                      # [c, n, Hk, D]
        vg = v[safe].float()
        qs = q[s:e].float().view(e - s, Hk, rep, D)
        lg = torch.einsum("cgrd,cngd->cgrn", qs, kg) * scale
        lg = lg.masked_fill(~valid[:, None, None, :], -float("inf"))
        if sinks is not None:
            sk = sinks.float().view(1, Hk, rep, 1).expand(e - s, -1, -1, -1)
            p = torch.softmax(torch.cat((lg, sk), -1), dim=-1)[..., :-1]
        else:
            p = torch.softmax(lg, dim=-1)
        p = torch.nan_to_num(p)                                                   # rows with no valid key
        outs.append(torch.einsum("cgrn,cngd->cgrd", p, vg).reshape(e - s, H, Dv))
    return torch.cat(outs, 0).to(q.dtype) if outs else q.new_zeros(0, H, Dv)


def window_indices(T: int, window: int, cu_seqlens, device) -> torch.Tensor:
    """[T, window] rows `t-window+1 .. t` clipped to the start of t's sequence (-1 where clipped)."""
    pos = torch.arange(T, device=device)
    start = torch.zeros(T, dtype=torch.long, device=device)
    for a, b in _bounds(cu_seqlens, T):
        start[a:b] = a
    idx = pos[:, None] - torch.arange(window - 1, -1, -1, device=device)[None, :]
    return idx.masked_fill(idx < start[:, None], -1).to(torch.int32)


@_native("lightning_indexer", "torch_lightning_indexer")
class TorchLightningIndexer(OpImpl):
    def __call__(self, query, key, weights, topk, *, cu_seqlens=None, scale=None, q_offset=0, **_):
        return lightning_indexer_ref(query, key, weights, topk, cu_seqlens, scale, q_offset)


@_native("sparse_attention", "torch_sparse_attention")
class TorchSparseAttention(OpImpl):
    def __call__(self, q, k, v, indices, *, scale=None, sinks=None):
        return sparse_attention_ref(q, k, v, indices, scale, sinks)


@_native("sparse_flash_mla", "torch_sparse_flash_mla")
class TorchSparseFlashMLA(OpImpl):
    """query [T, H, D]; ori_kv [T, D]; cmp_kv [Tc, D] or None; cmp_sparse_indices [T, n] rows of `cmp_kv` (-1 unused);
    sinks [H]; window = `ori_win_left + 1` original rows ending at the query.  Returns [T, H, D]."""

    def __call__(self, query, ori_kv, cmp_kv, cmp_sparse_indices, cmp_residual_kv, sinks, softmax_scale, cmp_ratio,
                 ori_win_left, ori_win_right=0, *, cu_seq_lens_q=None, cu_seq_lens_ori_kv=None, cu_seq_lens_cmp_kv=None):
        T = query.shape[0]
        idx = window_indices(T, int(ori_win_left) + 1, cu_seq_lens_q, query.device)
        kv = ori_kv
        if cmp_kv is not None and cmp_sparse_indices is not None:
            extra = cmp_sparse_indices.to(torch.int32)
            extra = torch.where(extra >= 0, extra + T, extra)
            idx = torch.cat((idx, extra), dim=-1)
            kv = torch.cat((ori_kv, cmp_kv), dim=0)
        kv = kv.unsqueeze(1)
        return sparse_attention_ref(query, kv, kv, idx, softmax_scale, sinks)


def masked_attention_ref(q, k, v, allow, scale=None):
    """Dense attention under an explicit boolean mask.  q: [Tq, H, D]; k, v: [Tk, Hk, D]; allow: [Tq, Tk] (True =
    may attend).  Rows without any allowed key produce zeros."""
    Tq, H, D = q.shape
    Hk = k.shape[1]
    rep = H // Hk
    scale = D ** -0.5 if scale is None else scale
    qh = q.transpose(0, 1).unsqueeze(0)                                        # [1, H, Tq, D]
    kh = k.transpose(0, 1).repeat_interleave(rep, 0).unsqueeze(0)
    vh = v.transpose(0, 1).repeat_interleave(rep, 0).unsqueeze(0)
    live = allow.any(-1)
    m = allow | ~live[:, None]                                                 # dead rows: attend everywhere, zeroed below
    o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, attn_mask=m[None, None], scale=scale)
    o = o[0].transpose(0, 1)
    return o * live[:, None, None].to(o.dtype)


@_native("masked_attention", "torch_masked_attention")
class TorchMaskedAttention(OpImpl):
    def __call__(self, q, k, v, allow, *, scale=None):
        return masked_attention_ref(q, k, v, allow, scale)
