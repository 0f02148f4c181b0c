"""tcgen05 variable-length flash attention as the `attention` / `attention_with_max_logits` operators."""
from __future__ import annotations

import math
import os

import torch

from ... import kernels as K
from ...runtime import TurboDevice
from ...utils.functools import cache
from ..base import OpImplKind
from ..registry import register_op
from . import native as N
from .b200 import BF16, _B200Op, _ok


@cache
def _tiles_for(cu_seqlens, device):
    """(query-tile table on the device, number of valid tokens, boundaries on the device) for one batch; built
    once and shared by every layer (pinned staging keeps the copies asynchronous)."""
    t = K.build_q_tiles(cu_seqlens).pin_memory()
    tk = K.build_kv_tiles(cu_seqlens).pin_memory()
    cu = cu_seqlens.to(torch.int32).pin_memory()
    return (t.to(device, non_blocking=True), int(cu_seqlens[-1]), cu.to(device, non_blocking=True),
            tk.to(device, non_blocking=True))


class FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, causal, scale, want_ml):
        tiles, n_valid = _tiles_for(cu_seqlens, q.device)[:2]
        out, lse, ml = K.attn_fwd(q, k, v, tiles, scale=scale, causal=causal, want_max_logit=want_ml)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta = (cu_seqlens, max_seqlen, causal, scale, n_valid)
        if want_ml:
            ctx.mark_non_differentiable(ml)
            return out, ml
        return out

    @staticmethod
    def backward(ctx, dout, *_):
        q, k, v, out, lse = ctx.saved_tensors
        cu_seqlens, max_seqlen, causal, scale, n = ctx.meta
        if os.environ.get("TORCHTURBO_ATTN_BWD", "tcgen05") == "tcgen05":
            cached = _tiles_for(cu_seqlens, q.device)
            dq, dk, dv = K.attn_bwd(dout.contiguous(), q, k, v, out, lse, cached[3], scale=scale, causal=causal,
                                    q_tiles_dev=cached[0], deterministic=torch.are_deterministic_algorithms_enabled())
            return dq, dk, dv, None, None, None, None, None
        # library backward on this kernel's out / lse (selected with TORCHTURBO_ATTN_BWD=flash_attn2; used as a baseline)
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward

        cu = _tiles_for(cu_seqlens, q.device)[2]
        if max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max())
        dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros(k.shape, dtype=k.dtype, device=k.device)
        _flash_attn_varlen_backward(dout.contiguous()[:n], q[:n], k[:n], v[:n].contiguous(), out[:n], lse[:, :n].contiguous(),
                                    dq[:n], dk[:n], dv[:n], cu, cu, max_seqlen, max_seqlen, 0.0, scale, causal,
                                    -1, -1, 0.0, None, False)
        return dq, dk, dv, None, None, None, None, None


def _LIB_FALLBACK(q, k, v, cu_seqlens, max_seqlen, *, causal, scale):
    from .b200 import FlashAttn2Varlen

    lib = FlashAttn2Varlen()
    if lib.available():
        return lib(q, k, v, cu_seqlens, max_seqlen, causal=causal, scale=scale)
    return N.attention_ref(q, k, v, cu_seqlens, causal, scale)


def _usable(q, k, v):
    """128-wide heads, or multi-head latent attention (query / key 192 wide, value 128 wide)."""
    return _ok(q, k, v) and q.shape[-1] in (128, 192) and k.shape[-1] == q.shape[-1] and v.shape[-1] == 128 and q.dim() == 3 \
        and q.shape[1] % k.shape[1] == 0 and v.stride(2) == 1 and v.stride(1) == 128


def _paddable(q, k, v):
    """Head widths below 128 (ViT: 72, 80) run on the 128-wide kernel with zero columns: padded query / key columns add
    nothing to the logits and padded value columns only produce output columns that are sliced away."""
    return _ok(q, k, v) and q.dim() == 3 and q.shape[1] % k.shape[1] == 0 and q.shape[-1] == k.shape[-1] and \
        q.shape[-1] <= 128 and v.shape[-1] <= 128 and (q.shape[-1] < 128 or v.shape[-1] < 128)


def _padded_call(q, k, v, cu, max_seqlen, causal, scale, want_ml):
    import torch.nn.functional as F

    dqk, dv = q.shape[-1], v.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(dqk)
    qp, kp, vp = F.pad(q, (0, 128 - dqk)), F.pad(k, (0, 128 - dqk)), F.pad(v, (0, 128 - dv))
    res = FlashAttnFn.apply(qp, kp, vp, cu.cpu() if cu.is_cuda else cu, max_seqlen, causal, float(scale), want_ml)
    if want_ml:
        return res[0][..., :dv], res[1]
    return res[..., :dv]


@register_op(op_name="attention", impl_name="tcgen05_varlen_attention", kind=OpImplKind.CUSTOM, priority=100,
             devices=(TurboDevice.CUDA,))
class B200Attention(_B200Op):
    def __call__(self, q, k, v, cu_seqlens, max_seqlen=None, *, causal=True, scale=None):
        cu = cu_seqlens if isinstance(cu_seqlens, torch.Tensor) else torch.tensor(cu_seqlens, dtype=torch.int32)
        if not _usable(q, k, v):
            if _paddable(q, k, v):
                return _padded_call(q, k, v, cu, max_seqlen, causal, scale, False)
            # other head widths: the library kernel
            return _LIB_FALLBACK(q, k, v, cu_seqlens, max_seqlen, causal=causal, scale=scale)
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        return FlashAttnFn.apply(q.contiguous(), k.contiguous(), v, cu.cpu() if cu.is_cuda else cu, max_seqlen, causal,
                                 float(scale), False)


@register_op(op_name="attention_with_max_logits", impl_name="tcgen05_varlen_attention_max_logits",
             kind=OpImplKind.CUSTOM, priority=100, devices=(TurboDevice.CUDA,))
class B200AttentionWithMaxLogits(_B200Op):
    def __call__(self, q, k, v, cu_seqlens, max_seqlen=None, *, causal=True, scale=None):
        cu = cu_seqlens if isinstance(cu_seqlens, torch.Tensor) else torch.tensor(cu_seqlens, dtype=torch.int32)
        if not _usable(q, k, v):
            if _paddable(q, k, v):
                return _padded_call(q, k, v, cu, max_seqlen, causal, scale, True)
            return N.attention_ref(q, k, v, cu_seqlens, causal, scale, want_max_logits=True)
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        return FlashAttnFn.apply(q.contiguous(), k.contiguous(), v, cu.cpu() if cu.is_cuda else cu, max_seqlen, causal,
                                 float(scale), True)
