"""ctypes bindings for the sm_100a CUDA library (`_lib/libttb200.so`).

Every function here launches hand-written kernels on the *current* CUDA stream
and takes/returns torch tensors.  Nothing falls back to PyTorch: if the library
is missing on a machine with a GPU, `lib()` raises so that a silent eager path
can never pass for the native one.  CPU-only processes never touch this module
(the op dispatcher selects the torch providers there).
"""
from __future__ import annotations

import ctypes as C
import os
from functools import lru_cache
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libttb200.so"
_lib = None

SEG_ALIGN = 128  # rows; every expert segment of a permuted buffer is padded to this
SCORE_FN = {"softmax_pre": 0, "softmax_post": 1, "sigmoid": 2}


class KernelError(RuntimeError):
    pass


class _GemmArgs(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("lda", C.c_longlong),
        ("B", C.c_void_p), ("ldb", C.c_longlong),
        ("b_group_stride", C.c_longlong), ("b_groups", C.c_int),
        ("C", C.c_void_p), ("ldc", C.c_longlong), ("c_group_stride", C.c_longlong),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("a_mn", C.c_int), ("b_mn", C.c_int),
        ("c_fp32", C.c_int), ("accumulate", C.c_int),
        ("residual", C.c_void_p), ("ldr", C.c_longlong),
        ("tile_group", C.c_void_p), ("m_tiles_cap", C.c_int),
        ("group_rows", C.c_void_p), ("groups_k", C.c_int),
        ("total_rows", C.c_longlong),
        ("epi", C.c_int), ("F", C.c_int),
        ("row_scale", C.c_void_p), ("preact", C.c_void_p), ("ld_preact", C.c_longlong),
        ("num_sms", C.c_int),
        ("ep", C.c_void_p),
    ]


class EpFuseArgs(C.Structure):
    """Expert-parallel fusion of one grouped GEMM launch (`struct EpFuseArgs` of csrc/gemm.cu): the push prologue that
    sends this rank's routed rows to their owners from inside the kernel, and / or the scatter epilogue that stores every
    output row into the return buffer of the rank it came from."""

    _fields_ = [
        ("peer_ptrs", C.c_void_p), ("W", C.c_int), ("rank", C.c_int), ("El", C.c_int),
        ("status", C.c_void_p), ("budget_ms", C.c_longlong),
        ("push_on", C.c_int),
        ("off_rows", C.c_longlong), ("off_vals", C.c_longlong), ("off_tags", C.c_longlong), ("off_flags", C.c_longlong),
        ("src", C.c_void_p), ("lds", C.c_longlong),
        ("order", C.c_void_p), ("expert", C.c_void_p), ("dest_row", C.c_void_p), ("val", C.c_void_p),
        ("counts", C.c_void_p), ("sent", C.c_void_p),
        ("n_entries", C.c_int), ("k", C.c_int), ("H", C.c_int), ("epoch", C.c_int),
        ("cap_rows", C.c_longlong),
        ("scat_on", C.c_int),
        ("off_ret", C.c_longlong), ("off_ret_vals", C.c_longlong), ("off_ret_flags", C.c_longlong),
        ("row_tag", C.c_void_p), ("row_val", C.c_void_p),
        ("ret_epoch", C.c_int),
        ("done_counter", C.c_void_p),
        ("ret_rows", C.c_int),
    ]


def lib_path() -> Path:
    return _LIB_PATH


def is_built() -> bool:
    return _LIB_PATH.exists()


def available() -> bool:
    """True when the CUDA library can be used in this process."""
    return torch.cuda.is_available() and is_built()


def lib():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise KernelError(
                f"{_LIB_PATH} is missing: run `python -m torchturbo_b200.csrc.build` "
                "(or __graft_entry__.build()) before using the CUDA ops"
            )
        _lib = C.CDLL(str(_LIB_PATH))
        _lib.ttb_gemm_bf16.argtypes = [C.POINTER(_GemmArgs), C.c_void_p]
        _lib.ttb_gemm_bf16.restype = C.c_int
    return _lib


# kernels launched per C entry point (used to report how many of this library's kernels ran in a region)
_LAUNCHES_PER_CALL = {"ttb_rmsnorm_bwd": 2, "ttb_layernorm_bwd": 2, "ttb_bias_act_bwd": 2, "ttb_causal_conv1d_bwd": 3,
                      "ttb_causal_conv1d_row_blocks": 0, "ttb_ep_dispatch_all": 5, "ttb_ep_dispatch_rows": 3,
                      "ttb_ep_combine_all": 3, "ttb_ep_combine_vals": 4, "ttb_ep_prepare": 3, "ttb_ep_prepare_bwd": 1, "ttb_router_fwd": 2, "ttb_perm_index": 3, "ttb_perm_scatter": 2,
                      "ttb_gemm_status": 0}
LAUNCH_COUNT = 0


def launch_count() -> int:
    """Number of CUDA kernels of this library launched so far in this process."""
    return LAUNCH_COUNT


def _check(code: int, what: str) -> None:
    global LAUNCH_COUNT
    if code != 0:
        raise KernelError(f"{what} failed with code {code}")
    LAUNCH_COUNT += _LAUNCHES_PER_CALL.get(what, 1)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> C.c_void_p:
    """Handle of the current stream of the current device (the raw accessor skips building a `torch.cuda.Stream`)."""
    if _raw_stream is not None:
        return C.c_void_p(_raw_stream(torch.cuda.current_device()))
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def check_device(t: torch.Tensor) -> None:
    """Kernels run on the current device's stream: an operand of another GPU would be an illegal address there."""
    if t.device.index != torch.cuda.current_device():
        raise KernelError(f"operand lives on {t.device} but the current CUDA device is {torch.cuda.current_device()}; "
                          "call torch.cuda.set_device() for this process before using the ops")


def _p(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


@lru_cache(maxsize=None)
def num_sms(device_index: int | None = None) -> int:
    return torch.cuda.get_device_properties(device_index if device_index is not None else torch.cuda.current_device()).multi_processor_count


def status(reset: bool = False) -> tuple[int, int]:
    """(first error code, number of errors) recorded by bounded in-kernel waits of the GEMM unit."""
    buf = (C.c_uint * 4)()
    _check(lib().ttb_gemm_status(buf, C.c_int(1 if reset else 0)), "ttb_gemm_status")
    return int(buf[0]), int(buf[1])


# --------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------
def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.bfloat16,
    accumulate: bool = False,
    residual: torch.Tensor | None = None,
    tile_group: torch.Tensor | None = None,
    group_rows: torch.Tensor | None = None,
    swiglu: bool = False,
    row_scale: torch.Tensor | None = None,
    preact: torch.Tensor | None = None,
    ep: "EpFuseArgs | None" = None,
) -> torch.Tensor:
    """tcgen05 GEMM ``C = op(A) @ op(B)`` on bf16 operands with fp32 accumulation.

    Memory orientation (row-major tensors):
      * ``a_mn=False``: ``a`` is ``[M, K]``;  ``a_mn=True``: ``a`` is ``[K, M]`` (used as its transpose).
      * ``b_mn=False``: ``b`` is ``[N, K]`` (``nn.Linear`` weight); ``b_mn=True``: ``b`` is ``[K, N]``.
      * grouped-M (``tile_group`` given): ``b`` is ``[G, N, K]`` / ``[G, K, N]`` and 128-row tile ``i`` of
        ``a`` multiplies ``b[tile_group[i]]`` (negative = skip the tile).
      * grouped-K (``group_rows`` given, both operands MN-major): ``C[g] = a[r_g:r_{g+1}].T @ b[r_g:r_{g+1}]``
        with ``group_rows`` an int32 ``[G+1]`` device tensor of 64-aligned row offsets.
      * ``swiglu=True``: ``b`` holds ``[gate | up]`` output columns (``2F``); the result is
        ``silu(gate) * up * row_scale`` of width ``F``; ``preact`` (``[M, 2F]``) optionally keeps gate|up.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1
    check_device(a)
    args = _GemmArgs()
    groups_k = 0
    if group_rows is not None:
        assert a_mn and b_mn and a.dim() == 2 and b.dim() == 2
        groups_k = group_rows.numel() - 1
        M, N, K = a.shape[1], b.shape[1], 0
        args.total_rows = a.shape[0]
        assert b.shape[0] == a.shape[0]
    else:
        if a_mn:
            K, M = a.shape
        else:
            M, K = a.shape
        if b_mn:
            Kb, Nmem = b.shape[-2], b.shape[-1]
        else:
            Nmem, Kb = b.shape[-2], b.shape[-1]
        assert Kb == K, (a.shape, b.shape, a_mn, b_mn)
        N = Nmem // 2 if swiglu else Nmem
    args.A, args.lda = a.data_ptr(), a.stride(0)
    args.B = b.data_ptr()
    args.ldb = b.stride(-2)
    if b.dim() == 3:
        args.b_groups, args.b_group_stride = b.shape[0], b.stride(0)
        assert tile_group is not None
    else:
        args.b_groups, args.b_group_stride = 1, 0
    if out is None:
        shape = (groups_k, M, N) if groups_k else (M, N)
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
        assert not accumulate
    assert out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    args.C, args.ldc = out.data_ptr(), out.stride(-2)
    args.c_group_stride = out.stride(0) if groups_k else 0
    args.M, args.N, args.K = M, N, K
    args.a_mn, args.b_mn = int(a_mn), int(b_mn)
    args.c_fp32, args.accumulate = int(out.dtype == torch.float32), int(accumulate)
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
        args.residual, args.ldr = residual.data_ptr(), residual.stride(0)
    if tile_group is not None:
        assert tile_group.dtype == torch.int32
        args.tile_group, args.m_tiles_cap = tile_group.data_ptr(), tile_group.numel()
        assert M <= tile_group.numel() * 128
    if group_rows is not None:
        assert group_rows.dtype == torch.int32
        args.group_rows, args.groups_k = group_rows.data_ptr(), groups_k
    args.epi = 1 if swiglu else 0
    args.F = N if swiglu else 0
    if row_scale is not None:
        assert row_scale.dtype == torch.float32
        args.row_scale = row_scale.data_ptr()
    if preact is not None:
        assert preact.dtype == torch.bfloat16
        args.preact, args.ld_preact = preact.data_ptr(), preact.stride(0)
    args.num_sms = num_sms(a.device.index)
    if ep is not None:
        args.ep = C.addressof(ep)
    _check(lib().ttb_gemm_bf16(C.byref(args), _stream()), "ttb_gemm_bf16")
    return out


# --------------------------------------------------------------------------------------
# RMSNorm
# --------------------------------------------------------------------------------------
def rmsnorm_fwd(x, weight, eps, residual=None, one_plus_w=False):
    """Returns (y, rstd, x_sum) where x_sum is ``x + residual`` (or ``x`` itself without residual)."""
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    T = x2.shape[0]
    y = torch.empty_like(x2)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    if residual is not None:
        r2 = residual.reshape(-1, H)
        xsum = torch.empty_like(x2)
    else:
        r2, xsum = None, None
    _check(lib().ttb_rmsnorm_fwd(_p(x2), _p(r2), _p(weight), _p(y), _p(xsum), _p(rstd), C.c_longlong(T), C.c_int(H),
                                 C.c_float(eps), C.c_int(int(one_plus_w)), _stream()), "ttb_rmsnorm_fwd")
    return y.view(x.shape), rstd, (xsum.view(x.shape) if xsum is not None else x)


def rmsnorm_bwd(dy, x_sum, weight, rstd, dres=None, one_plus_w=False):
    """Returns (dx, dw_fp32); ``dres`` (gradient arriving on the residual stream) is added into dx."""
    H = x_sum.shape[-1]
    x2, dy2 = x_sum.reshape(-1, H), dy.reshape(-1, H)
    T = x2.shape[0]
    grid = max(1, min(T, 2 * num_sms(x_sum.device.index)))
    dx = torch.empty_like(x2)
    partial = torch.empty(grid, H, dtype=torch.float32, device=x_sum.device)
    dw = torch.empty(H, dtype=torch.float32, device=x_sum.device)
    d2 = dres.reshape(-1, H) if dres is not None else None
    _check(lib().ttb_rmsnorm_bwd(_p(dy2), _p(x2), _p(weight), _p(rstd), _p(d2), _p(dx), _p(partial), _p(dw),
                                 C.c_longlong(T), C.c_int(H), C.c_int(int(one_plus_w)), C.c_int(grid), _stream()),
           "ttb_rmsnorm_bwd")
    return dx.view(x_sum.shape), dw


# --------------------------------------------------------------------------------------
# LayerNorm and bias + activation (vision tower)
# --------------------------------------------------------------------------------------
ACT = {None: 0, "none": 0, "identity": 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1, "gelu": 2, "gelu_erf": 2}


def layernorm_fwd(x, weight, bias, eps):
    """Returns (y, mean, rstd); statistics in fp32."""
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    T = x2.shape[0]
    y = torch.empty_like(x2)
    mean = torch.empty(T, dtype=torch.float32, device=x.device)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    _check(lib().ttb_layernorm_fwd(_p(x2), _p(weight), _p(bias), _p(y), _p(mean), _p(rstd), C.c_longlong(T), C.c_int(H),
                                   C.c_float(eps), _stream()), "ttb_layernorm_fwd")
    return y.view(x.shape), mean, rstd


def layernorm_bwd(dy, x, weight, mean, rstd):
    """Returns (dx, dw_fp32, db_fp32)."""
    H = x.shape[-1]
    x2, dy2 = x.reshape(-1, H), dy.reshape(-1, H)
    T = x2.shape[0]
    grid = max(1, min(T, 2 * num_sms(x.device.index)))
    dx = torch.empty_like(x2)
    part = torch.empty(grid, 2 * H, dtype=torch.float32, device=x.device)
    dwdb = torch.empty(2, H, dtype=torch.float32, device=x.device)
    _check(lib().ttb_layernorm_bwd(_p(dy2), _p(x2), _p(weight), _p(mean), _p(rstd), _p(dx), _p(part), _p(dwdb),
                                   C.c_longlong(T), C.c_int(H), C.c_int(grid), _stream()), "ttb_layernorm_bwd")
    return dx.view(x.shape), dwdb[0], dwdb[1]


def bias_act_fwd(x, bias, act, residual=None):
    """y = act(x + bias) (+ residual) on bf16 rows."""
    Cn = x.shape[-1]
    x2 = x.reshape(-1, Cn)
    y = torch.empty_like(x2)
    r2 = residual.reshape(-1, Cn) if residual is not None else None
    _check(lib().ttb_bias_act_fwd(_p(x2), _p(bias), _p(r2), _p(y), C.c_longlong(x2.shape[0]), C.c_int(Cn), C.c_int(ACT[act]),
                                  _stream()), "ttb_bias_act_fwd")
    return y.view(x.shape)


def bias_act_bwd(dy, x, bias, act):
    """Returns (dx, dbias_fp32); with the identity activation dx is dy itself."""
    Cn = x.shape[-1]
    x2, dy2 = x.reshape(-1, Cn), dy.reshape(-1, Cn)
    R = x2.shape[0]
    code = ACT[act]
    grid = max(1, min(R, 2 * num_sms(x.device.index)))
    dx = torch.empty_like(x2) if code else None
    part = torch.empty(grid, Cn, dtype=torch.float32, device=x.device)
    db = torch.empty(Cn, dtype=torch.float32, device=x.device)
    _check(lib().ttb_bias_act_bwd(_p(dy2), _p(x2), _p(bias), _p(dx), _p(part), _p(db), C.c_longlong(R), C.c_int(Cn),
                                  C.c_int(code), C.c_int(grid), _stream()), "ttb_bias_act_bwd")
    return (dx.view(x.shape) if dx is not None else dy), db


# --------------------------------------------------------------------------------------
# causal depthwise short convolution (linear-attention mixers)
# --------------------------------------------------------------------------------------
def causal_conv1d_fwd(x, weight, bias, seq_start, silu: bool):
    """x [T, D] bf16, weight [D, W] bf16, seq_start int32 [T] (first token of each token's sequence) -> y [T, D]."""
    T, D = x.shape
    y = torch.empty_like(x)
    _check(lib().ttb_causal_conv1d_fwd(_p(x), _p(weight), _p(bias), _p(seq_start), _p(y), C.c_longlong(T), C.c_int(D),
                                       C.c_int(weight.shape[1]), C.c_int(int(silu)), _stream()), "ttb_causal_conv1d_fwd")
    return y


def causal_conv1d_bwd(dy, x, weight, bias, seq_start, seq_end, silu: bool):
    """Returns (dx [T, D] bf16, dw [D, W] fp32, db [D] fp32)."""
    T, D = x.shape
    W = weight.shape[1]
    blocks = int(lib().ttb_causal_conv1d_row_blocks(C.c_longlong(T), C.c_int(D)))
    dpre, dx = torch.empty_like(x), torch.empty_like(x)
    part = torch.empty(blocks, (W + 1) * D, dtype=torch.float32, device=x.device)
    dwdb = torch.empty(W + 1, D, dtype=torch.float32, device=x.device)
    _check(lib().ttb_causal_conv1d_bwd(_p(dy), _p(x), _p(weight), _p(bias), _p(seq_start), _p(seq_end), _p(dpre), _p(dx),
                                       _p(part), _p(dwdb), C.c_longlong(T), C.c_int(D), C.c_int(W), C.c_int(int(silu)),
                                       _stream()), "ttb_causal_conv1d_bwd")
    # plane s holds the tap at distance s into the past = weight column W-1-s
    dw = dwdb[:W].flip(0).t().contiguous()
    return dx, dw, dwdb[W]


# --------------------------------------------------------------------------------------
# QK-norm + RoPE
# --------------------------------------------------------------------------------------
def qknorm_rope_fwd(qkv, n_q, n_kv, head_dim, wq, wk, cos, sin, eps, use_norm=True):
    """qkv: [T, (n_q + 2 n_kv) * D] -> (q [T, n_q, D], k [T, n_kv, D], rstd [T * (n_q + n_kv)])."""
    T = qkv.shape[0]
    q = torch.empty(T, n_q, head_dim, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(T, n_kv, head_dim, dtype=qkv.dtype, device=qkv.device)
    rstd = torch.empty(T * (n_q + n_kv), dtype=torch.float32, device=qkv.device)
    _check(lib().ttb_qknorm_rope_fwd(_p(qkv), C.c_longlong(qkv.stride(0)), C.c_int(n_q), C.c_int(n_kv),
                                     C.c_int(head_dim), _p(wq), _p(wk), _p(cos), _p(sin), _p(q), _p(k), _p(rstd),
                                     C.c_longlong(T), C.c_float(eps), C.c_int(int(use_norm)), _stream()),
           "ttb_qknorm_rope_fwd")
    return q, k, rstd


def qknorm_rope_bwd(dq, dk, qkv, n_q, n_kv, head_dim, wq, wk, cos, sin, rstd, dqkv, use_norm=True):
    """Writes the q and k column blocks of ``dqkv`` ([T, ld]) and returns (dwq, dwk) in fp32."""
    T = qkv.shape[0]
    dwq = torch.zeros(head_dim, dtype=torch.float32, device=qkv.device)
    dwk = torch.zeros(head_dim, dtype=torch.float32, device=qkv.device)
    grid = max(1, min((T * (n_q + n_kv) + 7) // 8, 4 * num_sms(qkv.device.index)))
    _check(lib().ttb_qknorm_rope_bwd(_p(dq), _p(dk), _p(qkv), C.c_longlong(qkv.stride(0)), C.c_int(n_q), C.c_int(n_kv),
                                     C.c_int(head_dim), _p(wq), _p(wk), _p(cos), _p(sin), _p(rstd), _p(dqkv),
                                     C.c_longlong(dqkv.stride(0)), _p(dwq), _p(dwk), C.c_longlong(T),
                                     C.c_int(int(use_norm)), C.c_int(grid), _stream()), "ttb_qknorm_rope_bwd")
    return dwq, dwk


# --------------------------------------------------------------------------------------
# SwiGLU
# --------------------------------------------------------------------------------------
def swiglu_fwd(x, row_scale=None, nrows=None):
    """`nrows` (int32 device scalar, optional): only the first `nrows[0]` rows are computed (padded buffers)."""
    R, F2 = x.shape
    F = F2 // 2
    y = torch.empty(R, F, dtype=x.dtype, device=x.device)
    _check(lib().ttb_swiglu_fwd(_p(x), C.c_longlong(x.stride(0)), _p(y), C.c_longlong(y.stride(0)), _p(row_scale),
                                C.c_longlong(R), C.c_int(F), _p(nrows), _stream()), "ttb_swiglu_fwd")
    return y


def swiglu_bwd(dy, x, row_scale=None, want_dscale=False, nrows=None):
    """`nrows` (int32 device scalar, optional): rows from `nrows[0]` on are left untouched (padded buffers)."""
    R, F2 = x.shape
    F = F2 // 2
    dx = torch.empty_like(x)
    dscale = torch.empty(R, dtype=torch.float32, device=x.device) if want_dscale else None
    _check(lib().ttb_swiglu_bwd(_p(dy), C.c_longlong(dy.stride(0)), _p(x), C.c_longlong(x.stride(0)), _p(row_scale),
                                _p(dx), C.c_longlong(dx.stride(0)), _p(dscale), C.c_longlong(R), C.c_int(F), _p(nrows),
                                _stream()), "ttb_swiglu_bwd")
    return dx, dscale


# --------------------------------------------------------------------------------------
# Cross entropy
# --------------------------------------------------------------------------------------
def cross_entropy(logits, labels, *, grad_out=None, grad_scale=None, grad_scale_host=1.0, want_lse=False):
    """Per-row CE (fp32, 0 for ignored rows).  With ``grad_out`` (bf16 [R, V]; may alias bf16 logits) also writes
    ``(softmax - onehot) * grad_scale[0] * grad_scale_host``."""
    R, V = logits.shape
    assert labels.dtype == torch.int64 and labels.numel() == R
    loss = torch.empty(R, dtype=torch.float32, device=logits.device)
    lse = torch.empty(R, dtype=torch.float32, device=logits.device) if want_lse else None
    _check(lib().ttb_cross_entropy(_p(logits), C.c_int(int(logits.dtype == torch.float32)),
                                   C.c_longlong(logits.stride(0)), _p(labels), _p(loss), _p(lse), _p(grad_out),
                                   C.c_longlong(grad_out.stride(0) if grad_out is not None else 0), _p(grad_scale),
                                   C.c_float(grad_scale_host), C.c_longlong(R), C.c_int(V), _stream()),
           "ttb_cross_entropy")
    return (loss, lse) if want_lse else loss


# --------------------------------------------------------------------------------------
# Multi-tensor AdamW / grad norm
# --------------------------------------------------------------------------------------
ADAM_CHUNK = 65536


class MultiTensorPlan:
    """Device tables for the multi-tensor AdamW / squared-norm kernels.

    ``meta`` rows are ``(p, g, m, v, shadow, numel, g_is_bf16)`` as int64; the chunk table maps each CUDA block to
    ``(tensor index, chunk index)``.  Gradient pointers are refreshed every step (autograd reallocates them).
    """

    def __init__(self, params, exp_avg, exp_avg_sq, shadows=None):
        self.params = list(params)
        self.device = self.params[0].device
        n = len(self.params)
        self.host_meta = torch.zeros(n, 7, dtype=torch.int64).pin_memory()
        chunks = []
        for i, p in enumerate(self.params):
            assert p.dtype == torch.float32 and p.is_contiguous()
            self.host_meta[i, 0] = p.data_ptr()
            self.host_meta[i, 2] = exp_avg[i].data_ptr()
            self.host_meta[i, 3] = exp_avg_sq[i].data_ptr()
            self.host_meta[i, 4] = shadows[i].data_ptr() if shadows is not None and shadows[i] is not None else 0
            self.host_meta[i, 5] = p.numel()
            for c in range((p.numel() + ADAM_CHUNK - 1) // ADAM_CHUNK):
                chunks.append((i, c))
        self.n_chunks = len(chunks)
        self.chunks = torch.tensor(chunks, dtype=torch.int32, device=self.device).reshape(-1, 2)
        self.meta = torch.empty(n, 7, dtype=torch.int64, device=self.device)
        self.partial = torch.empty(max(self.n_chunks, 1), dtype=torch.float32, device=self.device)

    def refresh_grads(self, grads):
        # the pinned table is read by the previous refresh's asynchronous copy until that copy has run on the device:
        # a host that is a whole step ahead waits here instead of overwriting pointers still to be copied
        ev = getattr(self, "_copy_event", None)
        if ev is not None:
            ev.synchronize()
        for i, g in enumerate(grads):
            assert g.is_contiguous() and g.numel() == self.host_meta[i, 5]
            self.host_meta[i, 1] = g.data_ptr()
            self.host_meta[i, 6] = int(g.dtype == torch.bfloat16)
        self.meta.copy_(self.host_meta, non_blocking=True)
        if self.device.type == "cuda":
            self._copy_event = torch.cuda.Event()
            self._copy_event.record()


def grad_sqnorm_partials(plan: MultiTensorPlan, prescale: float = 1.0) -> torch.Tensor:
    _check(lib().ttb_grad_sqnorm(_p(plan.meta), _p(plan.chunks), C.c_int(plan.n_chunks), _p(plan.partial),
                                 C.c_float(prescale), _stream()), "ttb_grad_sqnorm")
    return plan.partial[: plan.n_chunks]


def clip_coef(partials: torch.Tensor, max_norm: float, extra_sq: torch.Tensor | None = None) -> torch.Tensor:
    """Returns a device tensor ``[sum_sq, norm, coef]`` with ``coef = min(1, max_norm / (norm + 1e-6))``."""
    out = torch.empty(3, dtype=torch.float32, device=partials.device)
    _check(lib().ttb_clip_coef(_p(partials), C.c_int(partials.numel()), _p(extra_sq), C.c_float(max_norm), _p(out),
                               _stream()), "ttb_clip_coef")
    return out


def adamw_step(plan: MultiTensorPlan, *, lr, beta1, beta2, eps, weight_decay, step, clip=None, grad_prescale=1.0):
    bc1 = 1.0 - beta1 ** step
    bc2_sqrt = (1.0 - beta2 ** step) ** 0.5
    _check(lib().ttb_adamw(_p(plan.meta), _p(plan.chunks), C.c_int(plan.n_chunks), C.c_float(lr), C.c_float(beta1),
                           C.c_float(beta2), C.c_float(eps), C.c_float(weight_decay), C.c_float(bc1),
                           C.c_float(bc2_sqrt), _p(clip), C.c_float(grad_prescale), _stream()), "ttb_adamw")


# --------------------------------------------------------------------------------------
# MoE router / permutation
# --------------------------------------------------------------------------------------
def router_fwd(logits, k, score_fn, *, expert_bias=None, valid_mask=None, scaling=1.0, want_stats=False,
               want_lse=False):
    """logits fp32 [T, E] -> dict(topk_idx int32 [T,k], topk_prob fp32 [T,k], counts int32 [E],
    aux_counts int32 [E], score_sum fp32 [E], lse fp32 [T])."""
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    dev = logits.device
    idx = torch.empty(T, k, dtype=torch.int32, device=dev)
    prob = torch.empty(T, k, dtype=torch.float32, device=dev)
    counts = torch.zeros(E, dtype=torch.int32, device=dev)
    grid = max(1, min((T + 7) // 8, 2 * num_sms(dev.index)))
    lse = torch.empty(T, dtype=torch.float32, device=dev) if (want_lse or want_stats) else None
    if want_stats:
        partial = torch.empty(grid, E, dtype=torch.float32, device=dev)
        score_sum = torch.empty(E, dtype=torch.float32, device=dev)
        aux_counts = torch.zeros(E, dtype=torch.int32, device=dev)
    else:
        partial = score_sum = aux_counts = None
    vm = valid_mask.to(torch.uint8).contiguous() if valid_mask is not None else None
    _check(lib().ttb_router_fwd(_p(logits), _p(expert_bias), _p(vm), _p(idx), _p(prob), _p(lse), _p(partial),
                                _p(score_sum), _p(aux_counts), _p(counts), C.c_longlong(T), C.c_int(E), C.c_int(k),
                                C.c_int(SCORE_FN[score_fn]), C.c_float(scaling), C.c_int(grid), _stream()),
           "ttb_router_fwd")
    return dict(topk_idx=idx, topk_prob=prob, counts=counts, aux_counts=aux_counts, score_sum=score_sum, lse=lse)


def router_bwd(logits, topk_idx, topk_prob, k, score_fn, *, dprob=None, aux_grad=None, lse=None, valid_mask=None,
               dlse=None, scaling=1.0):
    """d(logits) from the gradients of the routing weights (`dprob` [T,k]), of the per-expert score sums
    (`aux_grad` [E], applied to valid tokens) and of the per-token logsumexp (`dlse` [T])."""
    T, E = logits.shape
    dlogits = torch.empty_like(logits)
    vm = valid_mask.to(torch.uint8).contiguous() if valid_mask is not None else None
    _check(lib().ttb_router_bwd(_p(logits), _p(topk_idx), _p(topk_prob), _p(dprob), _p(aux_grad), _p(lse), _p(vm),
                                _p(dlse), _p(dlogits), C.c_longlong(T), C.c_int(E), C.c_int(k),
                                C.c_int(SCORE_FN[score_fn]), C.c_float(scaling), _stream()), "ttb_router_bwd")
    return dlogits


def aux_loss(score_sum: torch.Tensor, counts: torch.Tensor, k: int, scale_num: float, coeff: float):
    """Load-balance loss from the routing kernel's statistics.  Returns (out [2] = (aux, aux / coeff), d aux / d score_sum [E])."""
    E = score_sum.numel()
    out = torch.empty(2, dtype=torch.float32, device=score_sum.device)
    coef = torch.empty(E, dtype=torch.float32, device=score_sum.device)
    _check(lib().ttb_aux_loss(_p(score_sum), _p(counts), C.c_int(E), C.c_int(k), C.c_float(scale_num), C.c_float(coeff),
                              _p(out), _p(coef), _stream()), "ttb_aux_loss")
    return out, coef


def perm_index(topk_idx: torch.Tensor, num_experts: int, m_tiles_cap: int | None = None):
    """Padded (expert, token) permutation of the [T, k] expert ids.

    Returns dict(counts [E], seg_start [E+1], tile_group [m_tiles_cap], row_of [T*k], status [1], capacity_rows).
    All int32 device tensors; nothing is synchronised with the host.
    """
    idx = topk_idx.reshape(-1)
    assert idx.dtype == torch.int32 and idx.is_contiguous()
    N = idx.numel()
    dev = idx.device
    if m_tiles_cap is None:
        m_tiles_cap = (N + SEG_ALIGN - 1) // SEG_ALIGN + num_experts
    counts = torch.empty(num_experts, dtype=torch.int32, device=dev)
    seg_start = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    tile_group = torch.empty(m_tiles_cap, dtype=torch.int32, device=dev)
    row_of = torch.empty(N, dtype=torch.int32, device=dev)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    _check(lib().ttb_perm_index(_p(idx), C.c_longlong(N), C.c_int(num_experts), _p(counts), _p(seg_start),
                                _p(tile_group), C.c_int(m_tiles_cap), _p(row_of), _p(st), _stream()),
           "ttb_perm_index")
    return dict(counts=counts, seg_start=seg_start, tile_group=tile_group, row_of=row_of, status=st,
                capacity_rows=m_tiles_cap * SEG_ALIGN)


def perm_scatter(src, row_of, k, capacity_rows, *, counts=None, seg_start=None, val=None, out=None):
    """dst[row_of[n]] = src[n // k]; pad rows of every expert segment are zeroed.  Returns (dst, row_val)."""
    T, H = src.shape
    N = row_of.numel()
    if out is None:
        out = torch.empty(capacity_rows, H, dtype=src.dtype, device=src.device)
    row_val = torch.empty(capacity_rows, dtype=torch.float32, device=src.device) if val is not None else None
    E = counts.numel() if counts is not None else 0
    _check(lib().ttb_perm_scatter(_p(src), C.c_longlong(src.stride(0)), _p(out), C.c_longlong(out.stride(0)),
                                  _p(row_of), _p(val), _p(row_val), C.c_void_p(0), _p(counts), _p(seg_start),
                                  C.c_int(E), C.c_longlong(N), C.c_int(k), C.c_int(H), _stream()), "ttb_perm_scatter")
    return out, row_val


def perm_combine(src, row_of, T, k, *, weights=None, residual=None):
    """out[t] = sum_j weights[t, j] * src[row_of[t*k+j]] (+ residual[t])."""
    H = src.shape[1]
    out = torch.empty(T, H, dtype=src.dtype, device=src.device)
    _check(lib().ttb_perm_combine(_p(src), C.c_longlong(src.stride(0)), _p(row_of), _p(weights), _p(residual),
                                  C.c_longlong(residual.stride(0) if residual is not None else 0), _p(out),
                                  C.c_longlong(out.stride(0)), C.c_longlong(T), C.c_int(k), C.c_int(H), _stream()),
           "ttb_perm_combine")
    return out


# --------------------------------------------------------------------------------------
# Flash attention (varlen, head_dim 128)
# --------------------------------------------------------------------------------------
def attn_status(reset: bool = False) -> tuple[int, int]:
    buf = (C.c_uint * 4)()
    _check(lib().ttb_attn_status(buf, C.c_int(1 if reset else 0)), "ttb_gemm_status")
    return int(buf[0]), int(buf[1])


def build_kv_tiles(cu_seqlens, block: int = 128) -> torch.Tensor:
    """Table of 128-row KV tiles for the backward pass, earliest tile of a document first (under a causal mask the
    earliest KV tiles are seen by the most query tiles, so they carry the most work)."""
    offs = cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else list(cu_seqlens)
    rows = [(k0, a, b) for a, b in zip(offs[:-1], offs[1:]) for k0 in range(a, b, block)]
    rows.sort(key=lambda r: -(r[2] - r[0]))
    return torch.tensor(rows, dtype=torch.int32).reshape(-1, 3)


def build_q_tiles(cu_seqlens, block: int = 128) -> torch.Tensor:
    """Host-side table of 128-row query tiles `[n, 3] = (first row, document start, document end)` from packed
    boundaries (a CPU tensor or list); no device synchronisation is involved."""
    offs = cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else list(cu_seqlens)
    rows = []
    for a, b in zip(offs[:-1], offs[1:]):
        # longest-first inside a document does not matter; later tiles of causal documents do more work, so
        # emit them first to shorten the tail of the launch
        for q0 in range(a + ((b - a - 1) // block) * block, a - 1, -block) if b > a else ():
            rows.append((q0, a, b))
    rows.sort(key=lambda r: -(r[0] - r[1]))          # across documents too: the tiles with the most KV blocks first
    return torch.tensor(rows, dtype=torch.int32).reshape(-1, 3)


def attn_fwd(q, k, v, q_tiles_dev, *, scale: float, causal: bool = True, want_lse: bool = True,
             want_max_logit: bool = False):
    """q: [T, Hq, D]; k: [T, Hk, D] with D = 128 or 192 (multi-head latent attention); v: [T, Hk, 128] (may be a
    row-strided view).  Returns (out [T, Hq, 128], lse [Hq, T], max_logit [Hq])."""
    T, Hq, D = q.shape
    Hk = k.shape[1]
    assert D in (128, 192) and k.shape[2] == D and v.shape[2] == 128
    assert q.stride(2) == 1 and q.stride(1) == D and k.stride(1) == D and k.stride(2) == 1 and v.stride(1) == 128 and v.stride(2) == 1
    # rows past the last sequence boundary are never written by the kernel and must read as zero
    out = torch.zeros(T, Hq, 128, dtype=q.dtype, device=q.device)
    lse = torch.full((Hq, T), float("-inf"), dtype=torch.float32, device=q.device) if want_lse else None
    ml = torch.full((Hq,), float("-inf"), dtype=torch.float32, device=q.device) if want_max_logit else None
    _check(lib().ttb_attn_fwd(_p(q), C.c_longlong(q.stride(0)), _p(k), C.c_longlong(k.stride(0)), _p(v),
                              C.c_longlong(v.stride(0)), _p(out), _p(lse), _p(ml), _p(q_tiles_dev),
                              C.c_int(q_tiles_dev.shape[0]), C.c_longlong(T), C.c_int(Hq), C.c_int(Hk), C.c_int(D),
                              C.c_float(scale), C.c_int(int(causal)), _stream()), "ttb_attn_fwd")
    return out, lse, ml


def delta_state_scan(a_tiles, b_tiles, u, decay, init, add, seq_chunks_dev, *, reverse: bool, s1: float, s2: float):
    """Chunk-state recurrence of the delta rule (csrc/delta_state.cu).  `a_tiles`, `b_tiles`: bf16 [H, NC, 64, 128];
    `u`: fp32 [H, NC, 64, 128]; `decay`: fp32 [H, NC] or [H, NC, 128]; `init`: fp32 [H, nseq, 128, 128] or None;
    `add`: fp32 [H, NC + nseq, 128, 128] (required when `reverse`); `seq_chunks_dev`: int32 [nseq, 2].
    Returns (x fp32 [H, NC, 64, 128], states fp32 [H, NC + nseq, 128, 128])."""
    H, NC, Cc, D = u.shape
    nseq = seq_chunks_dev.shape[0]
    assert Cc == 64 and D == 128 and a_tiles.shape == u.shape and b_tiles.shape == u.shape
    assert a_tiles.dtype == torch.bfloat16 and b_tiles.dtype == torch.bfloat16 and u.dtype == torch.float32
    assert a_tiles.is_contiguous() and b_tiles.is_contiguous() and u.is_contiguous() and decay.is_contiguous()
    assert decay.dtype == torch.float32 and decay.shape[:2] == (H, NC) and decay.dim() in (2, 3)
    if init is not None:
        init = init.contiguous()
        assert init.shape == (H, nseq, 128, 128) and init.dtype == torch.float32
    if add is not None:
        add = add.contiguous()
        assert add.shape == (H, NC + nseq, 128, 128) and add.dtype == torch.float32
    x = torch.empty_like(u)
    states = torch.empty(H, NC + nseq, 128, 128, dtype=torch.float32, device=u.device)
    _check(lib().ttb_delta_state_scan(_p(a_tiles), _p(b_tiles), _p(u), _p(x), _p(decay), C.c_int(int(decay.dim() == 3)),
                                      _p(init), _p(add), _p(states), _p(seq_chunks_dev), C.c_int(nseq), C.c_int(H),
                                      C.c_int(NC), C.c_int(int(reverse)), C.c_float(s1), C.c_float(s2), _stream()),
           "ttb_delta_state_scan")
    return x, states


# --------------------------------------------------------------------------------------
# Expert-parallel exchange over peer memory (see csrc/comm.cu)
# --------------------------------------------------------------------------------------
def comm_status(reset: bool = False) -> tuple[int, int]:
    buf = (C.c_uint * 4)()
    _check(lib().ttb_comm_status(buf, C.c_int(1 if reset else 0)), "ttb_gemm_status")
    return int(buf[0]), int(buf[1])


def perm_rank(idx: torch.Tensor, num_experts: int, base: torch.Tensor) -> torch.Tensor:
    flat = idx.reshape(-1)
    row_of = torch.empty_like(flat)
    _check(lib().ttb_perm_rank(_p(flat), C.c_longlong(flat.numel()), C.c_int(num_experts), _p(base), _p(row_of), _stream()),
           "ttb_perm_rank")
    return row_of


def perm_zero_pad(dst, counts, seg_start, row_val=None):
    _check(lib().ttb_perm_zero_pad(_p(dst), C.c_longlong(dst.stride(0)), _p(counts), _p(seg_start), _p(row_val),
                                   C.c_int(counts.numel()), C.c_int(dst.shape[1]), _stream()), "ttb_perm_zero_pad")


def ep_exchange(peer_ptrs, off_counts, off_flags, counts, rank, world, num_experts, epoch, budget_ms, m_tiles_cap,
                status):
    dev = counts.device
    El = num_experts // world
    seg_start = torch.empty(El + 1, dtype=torch.int32, device=dev)
    recv_counts = torch.empty(El, dtype=torch.int32, device=dev)
    tile_group = torch.empty(m_tiles_cap, dtype=torch.int32, device=dev)
    dest_base = torch.empty(num_experts, dtype=torch.int32, device=dev)
    _check(lib().ttb_ep_exchange(peer_ptrs, C.c_longlong(off_counts), C.c_longlong(off_flags), _p(counts), C.c_int(rank),
                                 C.c_int(world), C.c_int(num_experts), C.c_int(epoch), C.c_longlong(budget_ms),
                                 C.c_int(m_tiles_cap), _p(seg_start), _p(recv_counts), _p(tile_group), _p(dest_base),
                                 _p(status), _stream()), "ttb_ep_exchange")
    return seg_start, recv_counts, tile_group, dest_base


class _EpDispatchArgs(C.Structure):
    _fields_ = [
        ("peer_ptrs", C.c_void_p),
        ("off_counts", C.c_longlong), ("off_flags_counts", C.c_longlong), ("off_rows", C.c_longlong),
        ("off_vals", C.c_longlong), ("off_flags_rows", C.c_longlong),
        ("counts", C.c_void_p), ("expert", C.c_void_p), ("src", C.c_void_p), ("lds", C.c_longlong), ("val", C.c_void_p),
        ("recv_rows_local", C.c_void_p), ("recv_vals_local", C.c_void_p),
        ("seg_start", C.c_void_p), ("recv_counts", C.c_void_p), ("tile_group", C.c_void_p), ("dest_base", C.c_void_p),
        ("dest_row", C.c_void_p), ("done_counter", C.c_void_p), ("status", C.c_void_p),
        ("N", C.c_longlong), ("cap_rows", C.c_longlong), ("budget_ms", C.c_longlong),
        ("rank", C.c_int), ("W", C.c_int), ("E", C.c_int), ("k", C.c_int), ("H", C.c_int), ("m_tiles_cap", C.c_int),
        ("epoch_counts", C.c_int), ("epoch_rows", C.c_int), ("grid", C.c_int), ("exchange", C.c_int),
    ]


def ep_dispatch_all(peer_ptrs, *, off_counts, off_flags_counts, off_rows, off_vals, off_flags_rows, counts, expert, src, val,
                    recv_rows_local, recv_vals_local, rank, world, num_experts, k, m_tiles_cap, cap_rows, epoch_counts,
                    epoch_rows, budget_ms, done_counter, status, tables=None):
    """Expert-parallel row dispatch in one host call.  With `tables=None`: counts exchange, destination rows, padding
    zeroed, scatter, landed wait; returns (seg_start, recv_counts, tile_group, dest_row).  With `tables = (seg_start,
    recv_counts, dest_row)` (backward of combine) only the last three stages run."""
    dev = src.device
    N = expert.numel()
    El = num_experts // world
    a = _EpDispatchArgs()
    if tables is None:
        seg_start = torch.empty(El + 1, dtype=torch.int32, device=dev)
        recv_counts = torch.empty(El, dtype=torch.int32, device=dev)
        tile_group = torch.empty(m_tiles_cap, dtype=torch.int32, device=dev)
        dest_base = torch.empty(num_experts, dtype=torch.int32, device=dev)
        dest_row = torch.empty_like(expert)
        a.exchange, a.counts = 1, counts.data_ptr()
        a.tile_group, a.dest_base = tile_group.data_ptr(), dest_base.data_ptr()
    else:
        seg_start, recv_counts, dest_row = tables
        tile_group = None
        a.exchange = 0
    a.peer_ptrs = C.addressof(peer_ptrs)
    a.off_counts, a.off_flags_counts, a.off_rows = off_counts, off_flags_counts, off_rows
    a.off_vals, a.off_flags_rows = off_vals, off_flags_rows
    a.expert, a.src, a.lds = expert.data_ptr(), src.data_ptr(), src.stride(0)
    a.val = val.data_ptr() if val is not None else None
    a.recv_rows_local = recv_rows_local.data_ptr()
    a.recv_vals_local = recv_vals_local.data_ptr() if recv_vals_local is not None else None
    a.seg_start, a.recv_counts, a.dest_row = seg_start.data_ptr(), recv_counts.data_ptr(), dest_row.data_ptr()
    a.done_counter, a.status = done_counter.data_ptr(), status.data_ptr()
    a.N, a.cap_rows, a.budget_ms = N, cap_rows, budget_ms
    a.rank, a.W, a.E, a.k, a.H, a.m_tiles_cap = rank, world, num_experts, k, src.shape[1], m_tiles_cap
    a.epoch_counts, a.epoch_rows = epoch_counts, epoch_rows
    a.grid = max(1, min((N + 7) // 8, 8 * num_sms(dev.index)))
    _check(lib().ttb_ep_dispatch_all(C.byref(a), _stream()), "ttb_ep_dispatch_all" if tables is None else "ttb_ep_dispatch_rows")
    return seg_start, recv_counts, tile_group, dest_row


def ep_combine_all(peer_ptrs, *, off_rows, off_vals, off_flags, expert, dest_row, T, k, H, El, rank, world, epoch, budget_ms,
                   cap_rows, status, residual=None, want_vals=False):
    """Ready signal, ready wait and the k-way gather (optionally also the per-entry scalars) in one host call."""
    dev = expert.device
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    vals = torch.empty(T * k, dtype=torch.float32, device=dev) if want_vals else None
    _check(lib().ttb_ep_combine_all(peer_ptrs, C.c_longlong(off_rows), C.c_longlong(off_vals), C.c_longlong(off_flags),
                                    _p(expert), _p(dest_row), _p(residual),
                                    C.c_longlong(residual.stride(0) if residual is not None else 0), _p(out),
                                    C.c_longlong(out.stride(0)), _p(vals), C.c_longlong(T), C.c_int(k), C.c_int(H),
                                    C.c_int(El), C.c_int(rank), C.c_int(world), C.c_int(epoch), C.c_longlong(budget_ms),
                                    C.c_longlong(cap_rows), _p(status), _stream()),
           "ttb_ep_combine_vals" if want_vals else "ttb_ep_combine_all")
    return out, vals


class _EpPrepareArgs(C.Structure):
    _fields_ = [
        ("peer_ptrs", C.c_void_p), ("off_counts", C.c_longlong), ("off_flags_counts", C.c_longlong),
        ("counts", C.c_void_p), ("expert", C.c_void_p),
        ("recv_rows_local", C.c_void_p), ("recv_vals_local", C.c_void_p), ("recv_tags_local", C.c_void_p),
        ("seg_start", C.c_void_p), ("recv_counts", C.c_void_p), ("tile_group", C.c_void_p), ("dest_base", C.c_void_p),
        ("dest_row", C.c_void_p), ("send_base", C.c_void_p), ("order", C.c_void_p),
        ("sent", C.c_void_p), ("status", C.c_void_p),
        ("N", C.c_longlong), ("budget_ms", C.c_longlong),
        ("rank", C.c_int), ("W", C.c_int), ("E", C.c_int), ("H", C.c_int), ("m_tiles_cap", C.c_int),
        ("epoch_counts", C.c_int), ("exchange", C.c_int),
    ]


def ep_prepare(peer_ptrs, *, off_counts, off_flags_counts, counts, expert, recv_rows, recv_vals, recv_tags, sent, status,
               rank, world, num_experts, m_tiles_cap, epoch_counts, budget_ms, tables=None):
    """Everything a fused expert-parallel GEMM needs before it starts, in one host call.  Forward (`tables=None`):
    counts exchange with the peers, layout tables, destination row and send order of every entry, padding rows of the
    receive buffer cleared; returns `(seg_start, recv_counts, tile_group, dest_row, order)`.  Backward (`tables =
    (seg_start, recv_counts)` of the forward pass): only the receive buffer is prepared again."""
    dev = expert.device
    N = expert.numel()
    El = num_experts // world
    a = _EpPrepareArgs()
    if tables is None:
        # one int32 block: seg_start [El+1] | recv_counts [El] | tile_group [cap] | dest_base [E] | send_base [E]
        meta = torch.empty(2 * El + 1 + m_tiles_cap + 2 * num_experts, dtype=torch.int32, device=dev)
        seg_start, recv_counts = meta[:El + 1], meta[El + 1:2 * El + 1]
        o = 2 * El + 1
        tile_group = meta[o:o + m_tiles_cap]
        dest_base, send_base = meta[o + m_tiles_cap:o + m_tiles_cap + num_experts], meta[o + m_tiles_cap + num_experts:]
        rows = torch.empty(2, N, dtype=torch.int32, device=dev)
        dest_row, order = rows[0], rows[1]
        a.exchange, a.counts = 1, counts.data_ptr()
        a.tile_group, a.dest_base, a.send_base = tile_group.data_ptr(), dest_base.data_ptr(), send_base.data_ptr()
        a.dest_row, a.order = dest_row.data_ptr(), order.data_ptr()
    else:
        seg_start, recv_counts = tables
        tile_group = dest_row = order = None
        a.exchange = 0
    a.peer_ptrs = C.addressof(peer_ptrs)
    a.off_counts, a.off_flags_counts = off_counts, off_flags_counts
    a.expert = expert.data_ptr()
    a.recv_rows_local, a.recv_vals_local, a.recv_tags_local = recv_rows.data_ptr(), recv_vals.data_ptr(), recv_tags.data_ptr()
    a.seg_start, a.recv_counts = seg_start.data_ptr(), recv_counts.data_ptr()
    a.sent, a.status = sent.data_ptr(), status.data_ptr()
    a.N, a.budget_ms = N, budget_ms
    a.rank, a.W, a.E, a.H, a.m_tiles_cap = rank, world, num_experts, recv_rows.shape[1], m_tiles_cap
    a.epoch_counts = epoch_counts
    _check(lib().ttb_ep_prepare(C.byref(a), _stream()), "ttb_ep_prepare" if tables is None else "ttb_ep_prepare_bwd")
    return seg_start, recv_counts, tile_group, dest_row, order


def ep_save(recv_rows, recv_vals, seg_start, El):
    """Copies the rows (and their scalars) that landed in the receive buffer; the row count is read on the device."""
    cap, H = recv_rows.shape
    rows = torch.empty_like(recv_rows)
    vals = torch.empty_like(recv_vals) if recv_vals is not None else None
    grid = 4 * num_sms(recv_rows.device.index)
    _check(lib().ttb_ep_save(_p(recv_rows), _p(rows), _p(recv_vals), _p(vals), _p(seg_start), C.c_int(El), C.c_int(H),
                             C.c_longlong(cap), C.c_int(grid), _stream()), "ttb_ep_save")
    return rows, vals


def ep_ksum(peer_ptrs, off_ret, off_ret_flags, T, k, H, world, rank, epoch, budget_ms, status, residual=None):
    """Waits for every owner's "rows returned" flag, then sums the k returned rows of every token (+ residual)."""
    out = torch.empty(T, H, dtype=torch.bfloat16, device=status.device)
    _check(lib().ttb_ep_ksum(peer_ptrs, C.c_longlong(off_ret), C.c_longlong(off_ret_flags), _p(residual),
                             C.c_longlong(residual.stride(0) if residual is not None else 0), _p(out),
                             C.c_longlong(out.stride(0)), C.c_longlong(T), C.c_int(k), C.c_int(H), C.c_int(world),
                             C.c_int(rank), C.c_int(epoch), C.c_longlong(budget_ms), _p(status), _stream()), "ttb_ep_ksum")
    return out


def ep_scatter(peer_ptrs, off_rows, off_vals, off_flags, src, expert, dest_row, val, k, El, rank, world, epoch, cap_rows,
               done_counter, status):
    N = expert.numel()
    grid = max(1, min((N + 7) // 8, 8 * num_sms(src.device.index)))
    _check(lib().ttb_ep_scatter(peer_ptrs, C.c_longlong(off_rows), C.c_longlong(off_vals), C.c_longlong(off_flags), _p(src),
                                C.c_longlong(src.stride(0)), _p(expert), _p(dest_row), _p(val), C.c_longlong(N), C.c_int(k),
                                C.c_int(src.shape[1]), C.c_int(El), C.c_int(rank), C.c_int(world), C.c_int(epoch),
                                C.c_longlong(cap_rows), _p(done_counter), _p(status), C.c_int(grid), _stream()),
           "ttb_ep_scatter")


def flag_signal(peer_ptrs, off_flags, rank, world, epoch):
    _check(lib().ttb_flag_signal(peer_ptrs, C.c_longlong(off_flags), C.c_int(rank), C.c_int(world), C.c_int(epoch),
                                 _stream()), "ttb_flag_signal")


def flag_wait(peer_ptrs, off_flags, rank, world, epoch, budget_ms, status):
    _check(lib().ttb_flag_wait(peer_ptrs, C.c_longlong(off_flags), C.c_int(rank), C.c_int(world), C.c_int(epoch),
                               C.c_longlong(budget_ms), _p(status), _stream()), "ttb_flag_wait")


def ep_gather(peer_ptrs, off_rows, expert, dest_row, T, k, H, El, world, cap_rows, status, *, weights=None, residual=None,
              dtype=torch.bfloat16):
    out = torch.empty(T, H, dtype=dtype, device=expert.device)
    _check(lib().ttb_ep_gather(peer_ptrs, C.c_longlong(off_rows), _p(expert), _p(dest_row), _p(weights), _p(residual),
                               C.c_longlong(residual.stride(0) if residual is not None else 0), _p(out),
                               C.c_longlong(out.stride(0)), C.c_longlong(T), C.c_int(k), C.c_int(H), C.c_int(El),
                               C.c_int(world), C.c_longlong(cap_rows), _p(status), _stream()), "ttb_ep_gather")
    return out


def ep_gather_vals(peer_ptrs, off_vals, expert, dest_row, El, world, cap_rows, status):
    N = expert.numel()
    out = torch.empty(N, dtype=torch.float32, device=expert.device)
    _check(lib().ttb_ep_gather_vals(peer_ptrs, C.c_longlong(off_vals), _p(expert), _p(dest_row), _p(out), C.c_longlong(N),
                                    C.c_int(El), C.c_int(world), C.c_longlong(cap_rows), _p(status), _stream()),
           "ttb_ep_gather_vals")
    return out


def attn_bwd(dout, q, k, v, out, lse, kv_tiles_dev, *, scale: float, causal: bool = True, q_tiles_dev=None,
             deterministic: bool = False):
    """Gradients of `attn_fwd`.  Returns (dq [T,Hq,D], dk [T,Hk,D], dv [T,Hk,128]) in bf16.

    128-wide heads by default: one kernel; dQ tiles are added into an fp32 scratch buffer by TMA reductions and, with
    grouped-query attention, the dK / dV of a group's query heads are summed with atomics (the order of the adds is not
    fixed).  For 192-wide query / key heads that kernel computes dK / dV only and dQ comes from the query-major pass
    (`q_tiles_dev` required), which writes every dQ tile once.  `deterministic=True` uses that split for every width
    and lets one CTA per kv head walk the query heads of its group, so nothing is reduced with atomics and the result
    is bit-reproducible."""
    T, Hq, D = q.shape
    Hk = k.shape[1]
    assert dout.is_contiguous() and out.is_contiguous() and q.is_contiguous()
    assert k.stride(1) == D and k.stride(2) == 1 and v.stride(1) == 128 and v.stride(2) == 1
    split = deterministic or D != 128
    if split and q_tiles_dev is None:
        raise ValueError("the query-major dQ pass needs the query tile table")
    delta = torch.empty(Hq * T, dtype=torch.float32, device=q.device)
    dq_acc = None if split else torch.zeros(T, Hq, D, dtype=torch.float32, device=q.device)
    dq = torch.zeros_like(q) if split else torch.empty_like(q)
    if Hq != Hk and not deterministic:   # query heads of a group add into fp32 accumulators, converted at the end
        dk_acc = torch.zeros(T, Hk, D, dtype=torch.float32, device=q.device)
        dv_acc = torch.zeros(T, Hk, 128, dtype=torch.float32, device=q.device)
        dk = torch.empty(T, Hk, D, dtype=q.dtype, device=q.device)
        dv = torch.empty(T, Hk, 128, dtype=q.dtype, device=q.device)
    else:
        dk_acc = dv_acc = None
        dk = torch.zeros(T, Hk, D, dtype=q.dtype, device=q.device)
        dv = torch.zeros(T, Hk, 128, dtype=q.dtype, device=q.device)
    global LAUNCH_COUNT
    _check(lib().ttb_attn_bwd(_p(q), _p(k), C.c_longlong(k.stride(0)), _p(v), C.c_longlong(v.stride(0)), _p(out),
                              _p(dout), _p(lse), _p(delta), _p(dq_acc), _p(dk_acc), _p(dv_acc), _p(dq), _p(dk), _p(dv),
                              _p(kv_tiles_dev),
                              C.c_int(kv_tiles_dev.shape[0]), C.c_longlong(T), C.c_int(Hq), C.c_int(Hk), C.c_int(D),
                              C.c_float(scale), C.c_int(int(causal)), C.c_int((2 if deterministic else 0) if split else 1), _stream()),
           "ttb_attn_bwd")
    LAUNCH_COUNT += (1 if split else 2) + (0 if (Hq == Hk or deterministic) else 2)
    if split:
        _check(lib().ttb_attn_bwd_dq(_p(q), _p(k), C.c_longlong(k.stride(0)), _p(v), C.c_longlong(v.stride(0)), _p(dout),
                                     _p(lse), _p(delta), _p(dq), _p(q_tiles_dev), C.c_int(q_tiles_dev.shape[0]),
                                     C.c_longlong(T), C.c_int(Hq), C.c_int(Hk), C.c_int(D), C.c_float(scale),
                                     C.c_int(int(causal)), _stream()), "ttb_attn_bwd_dq")
    return dq, dk, dv


# --------------------------------------------------------------------------------------
# Ulysses sequence parallelism over peer memory
# --------------------------------------------------------------------------------------
def ulysses_qkv_scatter(peer_ptrs, off_q, off_k, off_v, off_flags, qkv, n_q, n_kv, rep, wq, wk, cos, sin, eps, rank, world,
                        epoch, done_counter, use_norm=True):
    """Per-head RMSNorm + RoPE of the q / k columns of `qkv` [Tl, (n_q + 2 n_kv) * 128] and a copy of the v columns,
    stored straight into the owning ranks' `[T, heads / world, 128]` buffers; publishes this rank's "landed" flag.
    Returns rstd [Tl * (n_q + n_kv)]."""
    Tl = qkv.shape[0]
    check_device(qkv)
    rstd = torch.empty(Tl * (n_q + n_kv), dtype=torch.float32, device=qkv.device)
    warps = Tl * (n_q + 2 * n_kv)
    grid = max(1, min((warps + 7) // 8, 8 * num_sms(qkv.device.index)))
    _check(lib().ttb_ulysses_qkv_scatter(peer_ptrs, C.c_longlong(off_q), C.c_longlong(off_k), C.c_longlong(off_v),
                                         C.c_longlong(off_flags), _p(qkv), C.c_longlong(qkv.stride(0)), _p(wq), _p(wk),
                                         _p(cos), _p(sin), _p(rstd), C.c_longlong(Tl), C.c_int(n_q), C.c_int(n_kv),
                                         C.c_int(rep), C.c_int(world), C.c_int(rank), C.c_int(epoch),
                                         C.c_int(int(use_norm)), C.c_float(eps), _p(done_counter), C.c_int(grid),
                                         _stream()), "ttb_ulysses_qkv_scatter")
    return rstd


def ulysses_move(peer_ptrs, off_buf, off_flags, local, heads, rep, rank, world, epoch, done_counter, status, gather: bool):
    """`gather=False`: push `local` [Tl, heads, 128] into the owners' buffers and publish the "landed" flag.
    `gather=True`: fill `local` from the owners' buffers (replicas summed)."""
    Tl = local.shape[0]
    check_device(local)
    assert local.is_contiguous() and local.dtype == torch.bfloat16 and local.shape[-1] == 128
    grid = max(1, min((Tl * heads + 7) // 8, 8 * num_sms(local.device.index)))
    _check(lib().ttb_ulysses_move(peer_ptrs, C.c_longlong(off_buf), C.c_longlong(off_flags), _p(local), C.c_longlong(Tl),
                                  C.c_int(heads), C.c_int(rep), C.c_int(world), C.c_int(rank), C.c_int(epoch),
                                  _p(done_counter), _p(status), C.c_int(int(gather)), C.c_int(grid), _stream()),
           "ttb_ulysses_move")
    return local


def multimem_allreduce_f32(mc_ptr: int, n: int, rank: int, world: int, scale: float = 1.0, grid: int = 296):
    """In-switch all-reduce (sum, then `scale`) of `n` fp32 values at multicast address `mc_ptr`; this rank handles slice
    `rank`.  The caller synchronises the ranks before (all inputs written) and after (all slices stored)."""
    _check(lib().ttb_multimem_allreduce_f32(C.c_void_p(mc_ptr), C.c_longlong(n), C.c_int(rank), C.c_int(world), C.c_float(scale),
                                            C.c_int(grid), _stream()), "ttb_multimem_allreduce_f32")


def peer_collective(peer_ptrs, off_data, off_ready, off_consumed, units, rank, world, epoch, budget_ms, done_counter,
                    status, *, kind: int, out: torch.Tensor | None = None, scale: float = 1.0, grid: int = 64):
    """Pull all-gather (kind 0) or pull reduce-scatter of fp32 (kind 1) / bf16 (kind 2) pieces over a slot of the
    symmetric buffer; `units` is the piece length in 16-byte units."""
    _check(lib().ttb_peer_collective(peer_ptrs, C.c_longlong(off_data), C.c_longlong(off_ready),
                                     C.c_longlong(off_consumed), C.c_longlong(units), C.c_int(rank), C.c_int(world),
                                     C.c_int(epoch), C.c_longlong(budget_ms), C.c_float(scale), _p(out),
                                     _p(done_counter), _p(status), C.c_int(kind), C.c_int(grid), _stream()),
           "ttb_peer_collective")
