"""One entry point for softmax attention in the Hugging Face calling convention.

`attention_forward(module, query, key, value, attention_mask, ...)` takes `[B, heads, S, D]` tensors as HF attention
modules produce them and returns `([B, S, heads, D], None)`.  Sequence boundaries come, in this order, from
`cu_seq_lens_q` (flattened packed row, B == 1), a 2-D `attention_mask` (0/1 or packed sample ids) or nothing (every
row one causal sequence).  4-D masks are rejected: training batches are packed.  With `module.qk_clip_state` set the
per-head maximum logits are recorded through `ops.attention_with_max_logits` (models/modules/attention/interface.py:
52-255 of the reference).  Registered under the name `turbo_attention` when `transformers` is importable."""
from __future__ import annotations

import torch

from ....ops import ops
from ....utils.flash_attn_utils import pad_input, unpad_varlen_inputs


def attention_forward(module, query, key, value, attention_mask=None, *, scaling=None, dropout: float = 0.0,
                      cu_seq_lens_q=None, cu_seq_lens_k=None, max_length_q=None, max_length_k=None, is_causal=None,
                      **_unused):
    if dropout:
        raise ValueError("attention dropout is not supported in packed training")
    B, Hq, S, D = query.shape
    causal = bool(getattr(module, "is_causal", True)) if is_causal is None else bool(is_causal)
    q, k, v = (t.transpose(1, 2) for t in (query, key, value))             # [B, S, H, D]
    meta = None
    if cu_seq_lens_q is not None:
        if B != 1:
            raise ValueError("cu_seq_lens describe one flattened packed row (batch size 1)")
        cu, mx = cu_seq_lens_q, max_length_q
        qp, kp, vp = q[0], k[0], v[0]
    elif attention_mask is not None:
        if attention_mask.dim() != 2:
            raise ValueError("packed training expects cu_seq_lens or a 2-D mask; 4-D attention masks are not supported")
        qp, kp, vp, meta = unpad_varlen_inputs(q, k, v, attention_mask)
        cu, mx = meta["cu_seqlens"].cpu(), meta["max_seqlen"]
    else:
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32)
        mx = S
        qp, kp, vp = q.flatten(0, 1), k.flatten(0, 1), v.flatten(0, 1)
    state = getattr(module, "qk_clip_state", None)
    if state is not None:
        out, max_logits = ops.attention_with_max_logits(qp.contiguous(), kp.contiguous(), vp.contiguous(), cu, mx,
                                                        causal=causal, scale=scaling)
        state.update(max_logits)
    else:
        out = ops.attention(qp.contiguous(), kp.contiguous(), vp.contiguous(), cu, mx, causal=causal, scale=scaling)
    if meta is not None:
        out = pad_input(out, meta["indices"], meta["batch"], meta["seqlen"])
    else:
        out = out.view(B, S, Hq, out.shape[-1])
    return out, None


def register_turbo_attention(name: str = "turbo_attention") -> bool:
    """Make the function selectable as `config._attn_implementation = name` for HF models; False without transformers."""
    try:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    except Exception:
        return False
    ALL_ATTENTION_FUNCTIONS.register(name, attention_forward)
    return True
