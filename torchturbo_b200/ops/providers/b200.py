"""sm_100a implementations of the operators: autograd Functions over the hand-written CUDA kernels.

Every class here is registered as a `CUSTOM` implementation for the CUDA device.  Inputs that the
kernels do not cover (CPU tensors, non-bf16 activations) are delegated to the torch formulation of
the same op, so mixed setups (fp32 router weights, CPU reference models) keep working; bf16 CUDA
tensors always take the kernel path and raise if the library is missing.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ... import kernels as K
from ...runtime import TurboDevice
from ..base import OpImpl, OpImplKind
from ..moe import MoEPermutation
from ..registry import register_op
from . import native as N

BF16 = torch.bfloat16


def _custom(op_name: str, impl_name: str, priority: int = 100):
    return register_op(op_name=op_name, impl_name=impl_name, kind=OpImplKind.CUSTOM, priority=priority,
                       devices=(TurboDevice.CUDA,))


def _ok(*tensors) -> bool:
    return all(t is None or (t.is_cuda and t.dtype == BF16) for t in tensors)


class _B200Op(OpImpl):
    def available(self) -> bool:
        return K.available()


def _weight_grad(w: torch.Tensor, a_rows: torch.Tensor, b_rows: torch.Tensor, **kw):
    """dW = a_rows^T @ b_rows.  When the parameter carries an fp32 `main_grad` buffer the product is
    accumulated straight into it by the GEMM epilogue (no separate gradient tensor, no extra pass)."""
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        K.gemm(a_rows, b_rows, a_mn=True, b_mn=True, out=mg, accumulate=True, **kw)
        return None
    return K.gemm(a_rows, b_rows, a_mn=True, b_mn=True, out_dtype=w.dtype if w.dtype in (BF16, torch.float32) else BF16, **kw)


# ------------------------------------------------------------------------------------------------
# linear
# ------------------------------------------------------------------------------------------------
class LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual):
        x2 = x.reshape(-1, x.shape[-1])
        r2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        y = K.gemm(x2, w, residual=r2)
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        ctx.has_res = residual is not None
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm(dy2, w, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw = _weight_grad(w, dy2, x2)
        return dx, dw, (dy if ctx.has_res else None)


@_custom("linear", "tcgen05_linear")
class B200Linear(_B200Op):
    """`x @ W^T (+ residual)` on the persistent tcgen05 GEMM; backward runs the MN-major variants of the
    same kernel (dX = dY W, dW = dY^T X)."""

    def __call__(self, x, weight, *, residual=None):
        if not _ok(x, weight, residual) or x.shape[-1] % 8 or weight.shape[0] % 8:
            return N.TorchLinear()(x, weight, residual=residual)
        return LinearFn.apply(x, weight, residual)


class RouterGatingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return K.gemm(x, w, out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, dl):
        x, w = ctx.saved_tensors
        d16 = dl.to(BF16)
        dx = K.gemm(d16, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(w, d16, x) if ctx.needs_input_grad[1] else None
        return dx, dw


@_custom("router_gating", "tcgen05_router_gating")
class B200RouterGating(_B200Op):
    """bf16 operands, fp32 accumulation and fp32 logits straight from the GEMM epilogue."""

    def __call__(self, x, weight):
        if not _ok(x, weight) or x.dim() != 2 or x.shape[-1] % 8 or weight.shape[0] % 8:
            return N.TorchRouterGating()(x, weight)
        return RouterGatingFn.apply(x.contiguous(), weight)


class LinearSwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        F2 = w.shape[0]
        pre = torch.empty(x2.shape[0], F2, dtype=BF16, device=x.device)
        y = K.gemm(x2, w, swiglu=True, preact=pre)
        ctx.save_for_backward(x2, w, pre)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], F2 // 2)

    @staticmethod
    def backward(ctx, dy):
        x2, w, pre = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dpre, _ = K.swiglu_bwd(dy2, pre)
        dx = K.gemm(dpre, w, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(w, dpre, x2) if ctx.needs_input_grad[1] else None
        return dx, dw


@_custom("linear_swiglu", "tcgen05_linear_swiglu")
class B200LinearSwiGLU(_B200Op):
    """Dense-MLP gate/up projection with the SwiGLU applied in the GEMM epilogue."""

    def __call__(self, x, weight):
        if not _ok(x, weight) or x.shape[-1] % 8 or weight.shape[0] % 16:
            return N.TorchLinearSwiGLU()(x, weight)
        return LinearSwiGLUFn.apply(x, weight)


# ------------------------------------------------------------------------------------------------
# RMSNorm / SwiGLU / RoPE
# ------------------------------------------------------------------------------------------------
class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual, one_plus_w):
        y, rstd, xsum = K.rmsnorm_fwd(x.contiguous(), w, eps, residual=residual.contiguous() if residual is not None else None,
                                      one_plus_w=one_plus_w)
        ctx.save_for_backward(xsum, w, rstd)
        ctx.one_plus_w = one_plus_w
        ctx.has_res = residual is not None
        if residual is not None:
            return y, xsum
        return y

    @staticmethod
    def backward(ctx, dy, dsum=None):
        xsum, w, rstd = ctx.saved_tensors
        dx, dw = K.rmsnorm_bwd(dy.contiguous(), xsum, w, rstd, dres=dsum.contiguous() if dsum is not None else None,
                               one_plus_w=ctx.one_plus_w)
        return dx, dw.to(w.dtype), None, (dx if ctx.has_res else None), None


@_custom("rms_norm", "b200_rms_norm")
class B200RMSNorm(_B200Op):
    """Fused (residual add +) RMSNorm.  With `residual` the op returns `(y, x + residual)` and the
    backward folds the gradient of the residual stream into d(x) in the same kernel."""

    def __call__(self, x, weight, eps=1e-6, *, residual=None, one_plus_weight=False):
        H = x.shape[-1]
        if not _ok(x, weight, residual) or H % 8 or H > 8192:
            return N.rms_norm_ref(x, weight, eps, residual, one_plus_weight)
        return RMSNormFn.apply(x, weight, eps, residual, one_plus_weight)


class LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        x = x.contiguous()
        y, mean, rstd = K.layernorm_fwd(x, w, b, eps)
        ctx.save_for_backward(x, w, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        dx, dw, db = K.layernorm_bwd(dy.contiguous(), x, w, mean, rstd)
        return dx, dw.to(w.dtype), db.to(w.dtype), None


@_custom("layer_norm", "b200_layer_norm")
class B200LayerNorm(_B200Op):
    """LayerNorm with weight and bias in one pass each way (vision tower)."""

    def __call__(self, x, weight, bias, eps=1e-6):
        H = x.shape[-1]
        if not _ok(x, weight, bias) or H % 8 or H > 8192:
            return N.layer_norm_ref(x, weight, bias, eps)
        return LayerNormFn.apply(x, weight, bias, eps)


class BiasActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, act, residual):
        x = x.contiguous()
        y = K.bias_act_fwd(x, bias, act, residual.contiguous() if residual is not None else None)
        ctx.save_for_backward(x, bias)
        ctx.act, ctx.has_res = act, residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, bias = ctx.saved_tensors
        dy = dy.contiguous()
        dx, db = K.bias_act_bwd(dy, x, bias, ctx.act)
        return dx, db.to(bias.dtype), None, (dy if ctx.has_res else None)


@_custom("bias_act", "b200_bias_act")
class B200BiasAct(_B200Op):
    """`act(x + bias) (+ residual)` and its backward (d(x) and the bias gradient in one pass)."""

    def __call__(self, x, bias, act=None, *, residual=None):
        Cn = x.shape[-1]
        if not _ok(x, bias, residual) or Cn % 8 or Cn > 16384 or act not in K.ACT:
            return N.bias_act_ref(x, bias, act, residual)
        return BiasActFn.apply(x, bias, act, residual)


# ------------------------------------------------------------------------------------------------
# causal short convolution (GDN / KDA mixers)
# ------------------------------------------------------------------------------------------------
def _seq_bounds(cu_seqlens, T: int, device):
    """int32 [T] first token and one-past-last token of every token's sequence (tokens past the last boundary form
    a sequence of their own), built on the host from the packed-row boundaries and copied once."""
    if cu_seqlens is None:
        cu = torch.tensor([0, T], dtype=torch.int64)
    else:
        cu = (cu_seqlens if isinstance(cu_seqlens, torch.Tensor) else torch.tensor(cu_seqlens)).to("cpu", torch.int64)
        if int(cu[-1]) < T:
            cu = torch.cat((cu, torch.tensor([T])))
    lens = cu[1:] - cu[:-1]
    start = torch.repeat_interleave(cu[:-1], lens).to(torch.int32)
    end = torch.repeat_interleave(cu[1:], lens).to(torch.int32)
    both = torch.stack((start, end))
    if torch.device(device).type == "cuda":
        both = both.pin_memory().to(device, non_blocking=True)
    return both[0], both[1]


class CausalConv1dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, seq_start, seq_end, silu):
        y = K.causal_conv1d_fwd(x, weight, bias, seq_start, silu)
        ctx.save_for_backward(x, weight, bias, seq_start, seq_end)
        ctx.silu = silu
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias, seq_start, seq_end = ctx.saved_tensors
        dx, dw, db = K.causal_conv1d_bwd(dy.contiguous(), x, weight, bias, seq_start, seq_end, ctx.silu)
        return dx, dw.to(weight.dtype), (db.to(bias.dtype) if bias is not None else None), None, None, None


@_custom("causal_conv1d", "b200_causal_conv1d")
class B200CausalConv1d(_B200Op):
    """Packed-row training path of the depthwise short convolution (one row, no carried state); decoding-style calls
    with `initial_state` / `output_final_state` use the torch formulation."""

    def __call__(self, x, weight, bias=None, *, activation=None, initial_state=None, output_final_state=False,
                 cu_seqlens=None, packed_params=None):
        from .native_linear_attention import TorchCausalConv1d

        if packed_params is not None and cu_seqlens is None:
            cu_seqlens = packed_params.cu_seqlens
            packed_params = None
        usable = (_ok(x, weight, bias) and x.dim() == 3 and x.shape[0] == 1 and x.shape[-1] % 8 == 0 and weight.shape[1] <= 8
                  and initial_state is None and not output_final_state and activation in (None, "silu", "swish"))
        if not usable:
            return TorchCausalConv1d()(x, weight, bias, activation=activation, initial_state=initial_state,
                                       output_final_state=output_final_state, cu_seqlens=cu_seqlens, packed_params=packed_params)
        T = x.shape[1]
        start, end = _seq_bounds(cu_seqlens, T, x.device)
        y = CausalConv1dFn.apply(x[0].contiguous(), weight.contiguous(), bias, start, end, activation is not None)
        return y.unsqueeze(0), None


class SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, probs):
        x2 = x.reshape(-1, x.shape[-1])
        y = K.swiglu_fwd(x2, probs)
        ctx.save_for_backward(x2, probs)
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], x.shape[-1] // 2)

    @staticmethod
    def backward(ctx, dy):
        x2, probs = ctx.saved_tensors
        dx, ds = K.swiglu_bwd(dy.reshape(-1, dy.shape[-1]).contiguous(), x2, probs, want_dscale=probs is not None)
        return dx.view(ctx.shape), ds


@_custom("swiglu", "b200_swiglu")
class B200SwiGLU(_B200Op):
    def __call__(self, x, *, probs=None):
        if not _ok(x) or x.shape[-1] % 16 or (probs is not None and probs.dtype != torch.float32):
            return N.swiglu_ref(x, probs)
        return SwiGLUFn.apply(x, probs.reshape(-1).contiguous() if probs is not None else None)


class QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, n_q, n_kv, D, wq, wk, cos, sin, eps):
        use_norm = wq is not None
        q, k, rstd = K.qknorm_rope_fwd(qkv, n_q, n_kv, D, wq, wk, cos, sin, eps, use_norm)
        v = qkv[:, (n_q + n_kv) * D:].view(qkv.shape[0], n_kv, D)
        ctx.save_for_backward(qkv, wq, wk, cos, sin, rstd)
        ctx.dims = (n_q, n_kv, D, use_norm)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, wq, wk, cos, sin, rstd = ctx.saved_tensors
        n_q, n_kv, D, use_norm = ctx.dims
        dqkv = torch.empty_like(qkv)
        dqkv[:, (n_q + n_kv) * D:] = dv.reshape(qkv.shape[0], n_kv * D)
        dwq, dwk = K.qknorm_rope_bwd(dq.contiguous(), dk.contiguous(), qkv, n_q, n_kv, D, wq, wk, cos, sin, rstd, dqkv,
                                     use_norm)
        return (dqkv, None, None, None, dwq.to(wq.dtype) if use_norm else None, dwk.to(wk.dtype) if use_norm else None,
                None, None, None)


@_custom("qk_norm_rope", "b200_qk_norm_rope")
class B200QKNormRope(_B200Op):
    """Per-head RMSNorm of q and k plus half-rotation RoPE in one pass over the fused QKV projection."""

    def __call__(self, qkv, n_q, n_kv, head_dim, q_weight, k_weight, cos, sin, eps=1e-6):
        if not _ok(qkv, q_weight, k_weight) or head_dim != 128 or qkv.dim() != 2 or qkv.stride(1) != 1:
            return N.TorchQKNormRope()(qkv, n_q, n_kv, head_dim, q_weight, k_weight, cos, sin, eps)
        return QKNormRopeFn.apply(qkv, n_q, n_kv, head_dim, q_weight, k_weight, cos.float().contiguous(),
                                  sin.float().contiguous(), eps)


# ------------------------------------------------------------------------------------------------
# MoE: router, permutation, experts
# ------------------------------------------------------------------------------------------------
class RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, score_fn, expert_bias, scaling, valid_mask):
        out = K.router_fwd(logits, k, score_fn, expert_bias=expert_bias, valid_mask=valid_mask, scaling=scaling,
                           want_stats=True)
        ctx.save_for_backward(logits, out["topk_idx"], out["topk_prob"], valid_mask)
        ctx.cfg = (k, score_fn, scaling)
        ctx.mark_non_differentiable(out["topk_idx"], out["aux_counts"], out["counts"])
        return out["topk_idx"], out["topk_prob"], out["score_sum"], out["lse"], out["aux_counts"], out["counts"]

    @staticmethod
    def backward(ctx, _di, dprob, dscore, dlse, _da, _dc):
        logits, idx, prob, valid = ctx.saved_tensors
        k, score_fn, scaling = ctx.cfg
        dl = K.router_bwd(logits, idx, prob, k, score_fn,
                          dprob=dprob.contiguous() if dprob is not None else None,
                          aux_grad=dscore.contiguous() if dscore is not None else None,
                          dlse=dlse.contiguous() if dlse is not None else None, valid_mask=valid, scaling=scaling)
        return dl, None, None, None, None, None


@_custom("router_topk", "b200_router_topk")
class B200RouterTopK(_B200Op):
    """One warp per token: score function, top-k, weight normalisation, aux-loss statistics, logsumexp."""

    def __call__(self, logits, k, score_fn="softmax_post", *, expert_bias=None, scaling=1.0, valid_mask=None):
        E = logits.shape[-1]
        if not logits.is_cuda or E > 256 or k > 16:
            return N.router_topk_ref(logits, k, score_fn, expert_bias, scaling, valid_mask)
        lg = logits.float().contiguous()
        idx, prob, score_sum, lse, aux_counts, counts = RouterFn.apply(
            lg, k, score_fn, expert_bias.float().contiguous() if expert_bias is not None else None, float(scaling),
            valid_mask)
        return idx, prob, dict(score_sum=score_sum, aux_counts=aux_counts, counts=counts, lse=lse)


class PermuteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, probs, topk_idx, num_experts):
        T, k = topk_idx.shape
        pm = K.perm_index(topk_idx, num_experts)
        xp, row_prob = K.perm_scatter(tokens, pm["row_of"], k, pm["capacity_rows"], counts=pm["counts"],
                                      seg_start=pm["seg_start"], val=probs.reshape(-1).contiguous() if probs is not None else None)
        ctx.save_for_backward(pm["row_of"])
        ctx.dims = (T, k, probs is not None)
        for t in (pm["row_of"], pm["counts"], pm["seg_start"], pm["tile_group"]):
            ctx.mark_non_differentiable(t)
        if row_prob is None:
            row_prob = tokens.new_empty(0, dtype=torch.float32)
        return xp, row_prob, pm["row_of"], pm["counts"], pm["seg_start"], pm["tile_group"]

    @staticmethod
    def backward(ctx, dxp, drow_prob, *_):
        (row_of,) = ctx.saved_tensors
        T, k, has_p = ctx.dims
        dtok = K.perm_combine(dxp.contiguous(), row_of, T, k)
        dprobs = drow_prob.index_select(0, row_of.long()).view(T, k) if has_p and drow_prob is not None else None
        return dtok, dprobs, None, None


@_custom("moe_permutation", "b200_moe_permutation")
class B200MoEPermutation(_B200Op):
    """Stable (expert, token) packing with 128-row aligned expert segments, built entirely on the device."""

    def __call__(self, tokens, expert_indices, *, probs=None, num_experts=None):
        if not _ok(tokens) or num_experts is None or tokens.shape[-1] % 8:
            return N.moe_permutation_ref(tokens, expert_indices, probs, num_experts)
        idx32 = expert_indices.to(torch.int32).contiguous()
        p32 = probs.float() if probs is not None else None
        xp, row_prob, row_of, counts, seg_start, tile_group = PermuteFn.apply(tokens.contiguous(), p32, idx32,
                                                                              num_experts)
        return MoEPermutation(tokens=xp, probs=row_prob if probs is not None else None,
                              row_indices=row_of.view(expert_indices.shape), expert_indices=expert_indices.long(),
                              counts=counts, seg_start=seg_start, tile_group=tile_group)


class UnpermuteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, row_of, counts, seg_start, merging, residual, T, k):
        out = K.perm_combine(y, row_of, T, k, weights=merging, residual=residual)
        ctx.save_for_backward(row_of, counts, seg_start, merging, y if merging is not None else None)
        ctx.dims = (T, k, y.shape[0], residual is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        row_of, counts, seg_start, merging, y = ctx.saved_tensors
        T, k, cap, has_res = ctx.dims
        dout = dout.contiguous()
        dmerge = None
        if merging is None:
            dy, _ = K.perm_scatter(dout, row_of, k, cap, counts=counts, seg_start=seg_start)
        else:
            dy, _ = K.perm_scatter(dout, row_of, k, cap, counts=counts, seg_start=seg_start)
            w_rows = torch.zeros(cap, dtype=torch.float32, device=dout.device)
            w_rows[row_of.long()] = merging.reshape(-1)
            dmerge = (dy.float() * y.float()).sum(-1).index_select(0, row_of.long()).view(T, k)
            dy = (dy.float() * w_rows[:, None]).to(dy.dtype)
        return dy, None, None, None, dmerge, (dout if has_res else None), None, None


@_custom("moe_unpermutation", "b200_moe_unpermutation")
class B200MoEUnpermutation(_B200Op):
    """k-way gather-sum of expert rows per token, with the residual stream added in the same pass."""

    def __call__(self, expert_out, perm: MoEPermutation, *, merging_probs=None, residual=None):
        if not _ok(expert_out, residual) or not perm.padded:
            return N.TorchMoEUnpermutation()(expert_out, perm, merging_probs=merging_probs, residual=residual)
        T, k = perm.row_indices.shape
        return UnpermuteFn.apply(expert_out, perm.row_indices.reshape(-1), perm.counts, perm.seg_start,
                                 merging_probs.float().contiguous() if merging_probs is not None else None,
                                 residual.reshape(T, -1) if residual is not None else None, T, k)


class MoEExpertsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xp, row_prob, w1, w2, tile_group, seg_start, buffers=(None, None)):
        # `buffers` = (output buffer, input-gradient buffer) or Nones.  They travel inside a tuple so that autograd
        # does not treat these long-lived, reused workspaces as inputs; the results are returned as fresh aliases.
        out_buffer, grad_buffer = buffers
        cap = xp.shape[0]
        F2 = w1.shape[-1]
        pre = torch.empty(cap, F2, dtype=BF16, device=xp.device)
        act = K.gemm(xp, w1, b_mn=True, tile_group=tile_group, swiglu=True, row_scale=row_prob, preact=pre)
        y = K.gemm(act, w2, b_mn=True, tile_group=tile_group, out=out_buffer)
        ctx.save_for_backward(xp, row_prob, w1, w2, tile_group, seg_start, pre)
        ctx.grad_buffer = grad_buffer
        return y.detach() if out_buffer is not None else y

    @staticmethod
    def backward(ctx, dy):
        xp, row_prob, w1, w2, tile_group, seg_start, pre = ctx.saved_tensors
        dy = dy.contiguous()
        # d(act) = dY @ W2[e]^T  (W2[e] is [F, H] = [N, K] K-major)
        dact = K.gemm(dy, w2, tile_group=tile_group)
        dpre, dprob = K.swiglu_bwd(dact, pre, row_prob, want_dscale=row_prob is not None)
        dw1 = dw2 = None
        if ctx.needs_input_grad[3]:
            act = K.swiglu_fwd(pre, row_prob)
            dw2 = _weight_grad(w2, act, dy, group_rows=seg_start)
        if ctx.needs_input_grad[2]:
            dw1 = _weight_grad(w1, xp, dpre, group_rows=seg_start)
        # last, so that `dy` (possibly a receive buffer peers refill once they see this output) is no longer read
        dxp = K.gemm(dpre, w1, tile_group=tile_group, out=ctx.grad_buffer) if ctx.needs_input_grad[0] else None
        if dxp is not None and ctx.grad_buffer is not None:
            dxp = dxp.detach()
        return dxp, dprob, dw1, dw2, None, None, None


@_custom("moe_experts", "tcgen05_grouped_mlp")
class B200MoEExperts(_B200Op):
    """Grouped fc1 (SwiGLU x routing-prob epilogue) and grouped fc2 over the padded expert-major buffer;
    expert offsets stay on the device (`tile_group`, `seg_start`), so there is no host synchronisation."""

    def __call__(self, perm: MoEPermutation, w1, w2, tokens_per_expert=None):
        if not _ok(perm.tokens, w1, w2) or not perm.padded:
            return N.TorchMoEExperts()(perm, w1, w2, tokens_per_expert)
        return MoEExpertsFn.apply(perm.tokens, perm.probs, w1, w2, perm.tile_group, perm.seg_start,
                                  (perm.out_buffer, perm.grad_buffer))


@_custom("grouped_matmul", "tcgen05_grouped_matmul")
class B200GroupedMatmul(_B200Op):
    """`y[rows_e] = x[rows_e] @ w[e]` on a padded buffer described by a `MoEPermutation`-style tile map.
    Dense (unpadded) packings fall back to the torch loop."""

    def __call__(self, x, w, tokens_per_expert, *, tile_group=None):
        if tile_group is None or not _ok(x, w):
            return N.grouped_matmul_ref(x, w, tokens_per_expert)
        return K.gemm(x, w, b_mn=True, tile_group=tile_group)


# ------------------------------------------------------------------------------------------------
# losses
# ------------------------------------------------------------------------------------------------
class CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels):
        lg = logits.reshape(-1, logits.shape[-1])
        grad = torch.empty(lg.shape, dtype=BF16, device=lg.device) if logits.requires_grad else None
        loss = K.cross_entropy(lg, labels.reshape(-1).contiguous(), grad_out=grad)
        ctx.save_for_backward(grad)
        ctx.shape, ctx.dtype = logits.shape, logits.dtype
        return loss.sum()

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return (grad.float() * g).to(ctx.dtype).view(ctx.shape), None


@_custom("cross_entropy_loss", "b200_cross_entropy")
class B200CrossEntropy(_B200Op):
    def __call__(self, logits, labels, *, ignore_index: int = -100):
        if not logits.is_cuda or logits.dtype not in (BF16, torch.float32) or ignore_index >= 0:
            return N.TorchCrossEntropy()(logits, labels, ignore_index=ignore_index)
        return CrossEntropyFn.apply(logits.contiguous(), labels)


class LinearCrossEntropyFn(torch.autograd.Function):
    """Chunked lm_head + CE with the gradients produced during the forward pass: per chunk the logits
    GEMM writes bf16 logits, the CE kernel turns them into d(logits) in place, and two more GEMMs
    produce d(hidden) and accumulate d(W) in fp32.  Backward only scales by the incoming gradient."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, chunk_size):
        h2 = hidden.reshape(-1, hidden.shape[-1])
        lab = labels.reshape(-1).contiguous()
        T, V = h2.shape[0], weight.shape[0]
        need_h, need_w = hidden.requires_grad, weight.requires_grad
        dh = torch.empty_like(h2) if need_h else None
        mg = getattr(weight, "main_grad", None)
        dw = None
        single = T <= chunk_size
        if need_w and not single:
            dw = mg if mg is not None else torch.zeros(V, h2.shape[1], dtype=torch.float32, device=h2.device)
        total = torch.zeros((), dtype=torch.float32, device=h2.device)
        for s in range(0, T, chunk_size):
            hc = h2[s:s + chunk_size]
            logits = K.gemm(hc, weight)
            loss = K.cross_entropy(logits, lab[s:s + chunk_size], grad_out=logits if (need_h or need_w) else None)
            total += loss.sum()
            if need_h:
                K.gemm(logits, weight, b_mn=True, out=dh[s:s + chunk_size])
            if need_w:
                if single and mg is None:
                    # one chunk: the weight gradient is written once, in the weight's dtype, with no accumulator pass
                    dw = K.gemm(logits, hc, a_mn=True, b_mn=True, out_dtype=weight.dtype)
                else:
                    if dw is None:
                        dw = mg
                    K.gemm(logits, hc, a_mn=True, b_mn=True, out=dw, accumulate=True)
        ctx.save_for_backward(dh, dw if (need_w and mg is None) else None)
        ctx.meta = (hidden.shape, weight.dtype, mg is not None)
        return total

    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        shape, wdtype, fused = ctx.meta
        gh = (dh * g.to(dh.dtype)).view(shape) if dh is not None else None
        gw = (dw * g).to(wdtype) if dw is not None else None
        return gh, gw, None, None


@_custom("linear_cross_entropy", "tcgen05_linear_cross_entropy")
class B200LinearCrossEntropy(_B200Op):
    def __call__(self, hidden, weight, labels, *, chunk_size: int = 4096, ignore_index: int = -100):
        if not _ok(hidden, weight) or ignore_index >= 0 or hidden.shape[-1] % 8 or weight.shape[0] % 8:
            return N.TorchLinearCrossEntropy()(hidden, weight, labels, chunk_size=chunk_size, ignore_index=ignore_index)
        return LinearCrossEntropyFn.apply(hidden, weight, labels, chunk_size)


# ------------------------------------------------------------------------------------------------
# attention (library baseline; the tcgen05 kernel registers itself with a higher priority)
# ------------------------------------------------------------------------------------------------
@_custom("attention", "flash_attn2_varlen", priority=10)
class FlashAttn2Varlen(_B200Op):
    """flash-attn 2 `flash_attn_varlen_func`: the library baseline the reference itself uses
    (models/modules/attention/interface.py:114-158 in the reference)."""

    def available(self) -> bool:
        try:
            import flash_attn  # noqa: F401

            return torch.cuda.is_available()
        except Exception:
            return False

    def __call__(self, q, k, v, cu_seqlens, max_seqlen=None, *, causal=True, scale=None):
        D, Dv = q.shape[-1], v.shape[-1]
        if not _ok(q, k, v) or D > 256 or Dv > D:
            return N.attention_ref(q, k, v, cu_seqlens, causal, scale)
        from flash_attn import flash_attn_varlen_func

        T = q.shape[0]
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        pad_d = (-D) % 8
        if pad_d or Dv != D:
            # the library wants equal, 8-aligned head widths: zero columns change neither the scores nor the output
            q, k = F.pad(q, (0, pad_d)), F.pad(k, (0, pad_d))
            v = F.pad(v, (0, D + pad_d - Dv))
        n = int(cu_seqlens[-1])  # boundaries live on the host in the packed-batch contract
        if max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max())
        cu = cu_seqlens.to(device=q.device, dtype=torch.int32)
        out = flash_attn_varlen_func(q[:n], k[:n], v[:n], cu, cu, max_seqlen, max_seqlen, softmax_scale=scale,
                                     causal=causal)
        if out.shape[-1] != Dv:
            out = out[..., :Dv]
        if n < T:  # tokens after the last boundary are padding: zeros
            out = torch.nn.functional.pad(out, (0, 0, 0, 0, 0, T - n))
        return out
