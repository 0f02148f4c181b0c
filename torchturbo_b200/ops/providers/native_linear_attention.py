"""Plain PyTorch formulations of the linear-attention operators: `causal_conv1d`, `gated_delta_rule`, `kda`.

The reference binds these three names to the Triton kernels of the `fla` package
(ops/providers/native/causal_conv1d.py:22, gated_delta_rule.py:22, kda.py:18 of the reference); here they are
written out in torch so that they run anywhere (CPU oracle, autograd through torch ops) without that package.
Conventions follow the reference call sites: activations are `[B, T, ...]` with heads before the channel
dimension, packed rows use `B == 1` with `cu_seqlens`, and recurrent states are fp32 `[N, H, K, V]`.

Delta-rule recurrence for one head (state `S` is `[K, V]`, `a_t = exp(g_t)` scalar for the gated delta rule and
a per-channel vector for KDA):

    S  <- diag(a_t) S
    S  <- S + k_t (beta_t (v_t - S^T k_t))^T
    o_t = scale * S^T q_t

`*_recurrent` evaluates exactly that, one token at a time (test oracle).  The `chunk_*` entry points evaluate the
same map chunk-wise: inside a chunk of C tokens the rank-1 updates are folded into one unit-lower-triangular
solve (the WY form), so the sequential part runs once per chunk on `[C, C]` / `[K, V]` matmuls.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..base import OpImpl, OpImplKind
from ..registry import register_op


def _native(op_name: str, impl_name: str):
    return register_op(op_name=op_name, impl_name=impl_name, kind=OpImplKind.NATIVE, priority=0)


def _bounds(cu_seqlens, T: int) -> list[tuple[int, int]]:
    if cu_seqlens is None:
        return [(0, T)]
    offs = [int(c) for c in (cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)]
    out = [(a, b) for a, b in zip(offs[:-1], offs[1:])]
    if offs[-1] < T:
        out.append((offs[-1], T))          # a padded tail behaves as one more sequence
    return out


# ------------------------------------------------------------------------------------------------
# causal depthwise short convolution
# ------------------------------------------------------------------------------------------------
def causal_conv1d_ref(x, weight, bias=None, activation=None, initial_state=None, output_final_state=False,
                      cu_seqlens=None):
    """x: [B, T, D]; weight: [D, W] (tap W-1 multiplies the current token); bias: [D].  With `cu_seqlens`
    (B == 1) the window never crosses a sequence start.  `initial_state` / the returned final state are
    `[N, D, W]`: the last W inputs of each sequence, oldest first."""
    B, T, D = x.shape
    W = weight.shape[1]
    if cu_seqlens is not None and B != 1:
        raise ValueError("packed causal_conv1d expects a single row")
    bounds = _bounds(cu_seqlens, T) if cu_seqlens is not None else None
    pos = torch.arange(T, device=x.device)
    if bounds is not None:
        start = torch.zeros(T, dtype=torch.long, device=x.device)
        for a, b in bounds:
            start[a:b] = a
        pos = pos - start
    xf = x.float()
    y = torch.zeros_like(xf)
    wf = weight.float()
    for s in range(W):                       # s = distance into the past
        tap = wf[:, W - 1 - s]
        if s == 0:
            y = y + xf * tap
            continue
        shifted = F.pad(xf, (0, 0, s, 0))[:, :T]
        keep = (pos >= s).to(xf.dtype)[None, :, None]
        y = y + shifted * keep * tap
    if initial_state is not None:
        # rare path (decoding / chunked prefill): redo each sequence with its carried inputs in front of it
        segs = [(0, a, b) for a, b in bounds] if bounds is not None else [(r, 0, T) for r in range(B)]
        pieces: list[list[torch.Tensor]] = [[] for _ in range(B)]
        for n, (r, a, b) in enumerate(segs):
            head = initial_state[n].float().t()[1:]                              # [W-1, D], oldest first
            win = torch.cat((head, xf[r, a:b]), 0).unfold(0, W, 1)               # [L, D, W]
            pieces[r].append((win * wf).sum(-1))
        y = torch.stack([torch.cat(p, 0) for p in pieces], 0)
    if bias is not None:
        y = y + bias.float()
    if activation in ("silu", "swish"):
        y = F.silu(y)
    elif activation is not None:
        raise ValueError(f"unsupported activation {activation!r}")
    final = None
    if output_final_state:
        segs = bounds if bounds is not None else None
        if segs is None:
            padded = F.pad(xf, (0, 0, W, 0))
            if initial_state is not None and T < W:
                padded[:, : W] = initial_state.float().transpose(1, 2)
            final = padded[:, -W:].transpose(1, 2).contiguous()
        else:
            outs = []
            for n, (a, b) in enumerate(segs):
                seg = xf[0, a:b]
                head = initial_state[n].float().t() if initial_state is not None else seg.new_zeros(W, D)
                outs.append(torch.cat((head, seg), 0)[-W:].t())
            final = torch.stack(outs, 0)
    return y.to(x.dtype), final


@_native("causal_conv1d", "torch_causal_conv1d")
class TorchCausalConv1d(OpImpl):
    def __call__(self, x, weight, bias=None, *, activation=None, initial_state=None, output_final_state=False,
                 cu_seqlens=None, packed_params=None):
        if packed_params is not None:
            if cu_seqlens is not None:
                raise ValueError("pass either cu_seqlens or packed_params, not both")
            cu_seqlens = packed_params.cu_seqlens
        return causal_conv1d_ref(x, weight, bias, activation, initial_state, output_final_state, cu_seqlens)


# ------------------------------------------------------------------------------------------------
# delta rule: token-by-token oracle
# ------------------------------------------------------------------------------------------------
def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def delta_rule_recurrent(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None):
    """q, k: [B, T, H, K]; v: [B, T, H, V]; g: [B, T, H] or [B, T, H, K] (log decay); beta: [B, T, H].
    Returns (o [B, T, H, V] fp32, final_state [N, H, K, V] fp32)."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    segs = [(r, a, b) for r in range(B) for a, b in _bounds(cu_seqlens, T)] if cu_seqlens is not None \
        else [(r, 0, T) for r in range(B)]
    o = torch.zeros(B, T, H, V, dtype=torch.float32, device=q.device)
    finals = []
    for n, (r, a, b) in enumerate(segs):
        S = initial_state[n].float().clone() if initial_state is not None else q.new_zeros(H, K, V)
        for t in range(a, b):
            decay = g[r, t].exp()
            S = S * (decay[:, :, None] if decay.dim() == 2 else decay[:, None, None])
            pred = torch.einsum("hkv,hk->hv", S, k[r, t])
            S = S + torch.einsum("hk,hv->hkv", k[r, t], beta[r, t][:, None] * (v[r, t] - pred))
            o[r, t] = torch.einsum("hkv,hk->hv", S, q[r, t]) * scale
        finals.append(S)
    return o, torch.stack(finals, 0)


# ------------------------------------------------------------------------------------------------
# delta rule: chunked evaluation (differentiable through torch ops)
# ------------------------------------------------------------------------------------------------
def _chunk_one_sequence(q, k, v, g, beta, scale, S, C):
    """One sequence, head-major: q, k [H, L, K]; v [H, L, V]; g [H, L] or [H, L, K]; beta [H, L]; S [H, K, V]."""
    H, L, K = q.shape
    V = v.shape[-1]
    pad = (-L) % C
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
        beta = F.pad(beta, (0, pad))
        g = F.pad(g, (0, 0, 0, pad)) if g.dim() == 3 else F.pad(g, (0, pad))
    n = (L + pad) // C
    vec = g.dim() == 3
    q = q.view(H, n, C, K) * scale
    k = k.view(H, n, C, K)
    v = v.view(H, n, C, V)
    beta = beta.view(H, n, C)
    G = (g.view(H, n, C, K) if vec else g.view(H, n, C)).cumsum(2)          # within-chunk cumulative log decay
    eye = torch.eye(C, dtype=q.dtype, device=q.device)
    low = torch.ones(C, C, dtype=torch.bool, device=q.device).tril(-1)
    lowd = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    outs = []
    for c in range(n):
        qc, kc, vc, bc, Gc = q[:, c], k[:, c], v[:, c], beta[:, c], G[:, c]
        kb = kc * bc[..., None]
        if vec:
            # D[i, j, :] = exp(G_i - G_j) on i >= j (exponent <= 0), zero elsewhere
            D = (Gc[:, :, None, :] - Gc[:, None, :, :]).masked_fill(~lowd[None, :, :, None], -float("inf")).exp()
            kk = torch.einsum("hik,hijk,hjk->hij", kb, D, kc)
            qk = torch.einsum("hik,hijk,hjk->hij", qc, D, kc)
            k_in = kb * Gc.exp()                                            # decay from chunk start to i
            q_in = qc * Gc.exp()
            k_out = kc * (Gc[:, -1:, :] - Gc).exp()                         # decay from j to chunk end
            s_decay = Gc[:, -1].exp()[:, :, None]                           # [H, K, 1]
        else:
            D = (Gc[:, :, None] - Gc[:, None, :]).masked_fill(~lowd[None], -float("inf")).exp()
            kk = (kb @ kc.transpose(-1, -2)) * D
            qk = (qc @ kc.transpose(-1, -2)) * D
            k_in = kb * Gc.exp()[..., None]
            q_in = qc * Gc.exp()[..., None]
            k_out = kc * (Gc[:, -1:] - Gc).exp()[..., None]
            s_decay = Gc[:, -1].exp()[:, None, None]
        Lmat = kk.masked_fill(~low[None], 0.0)
        Tm = torch.linalg.solve_triangular(eye + Lmat, eye.expand(H, C, C), upper=False)   # (I + L)^-1
        u = Tm @ (vc * bc[..., None])                                       # pseudo-values without the carried state
        w = Tm @ k_in                                                       # what the carried state contributes
        v_new = u - w @ S
        outs.append(q_in @ S + qk.masked_fill(~lowd[None], 0.0) @ v_new)
        S = S * s_decay + k_out.transpose(-1, -2) @ v_new
    o = torch.stack(outs, 1).reshape(H, n * C, V)[:, :L]
    return o, S


def chunk_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
                     use_qk_l2norm=False, chunk_size=64):
    B, T, H, K = q.shape
    dt = v.dtype
    scale = K ** -0.5 if scale is None else scale
    qf, kf, vf, gf, bf = (t.float() for t in (q, k, v, g, beta))
    if use_qk_l2norm:
        qf, kf = l2norm(qf), l2norm(kf)
    if cu_seqlens is not None and B != 1:
        raise ValueError("packed delta rule expects a single row")
    segs = [(0, a, b) for a, b in _bounds(cu_seqlens, T)] if cu_seqlens is not None else [(r, 0, T) for r in range(B)]
    rows: list[list[torch.Tensor]] = [[] for _ in range(B)]
    finals = []
    for n, (r, a, b) in enumerate(segs):
        S = initial_state[n].float() if initial_state is not None else qf.new_zeros(H, K, v.shape[-1])
        if b > a:
            gs = gf[r, a:b].permute(1, 0, 2) if gf.dim() == 4 else gf[r, a:b].t()
            o, S = _chunk_one_sequence(qf[r, a:b].transpose(0, 1), kf[r, a:b].transpose(0, 1), vf[r, a:b].transpose(0, 1),
                                       gs, bf[r, a:b].t(), scale, S, chunk_size)
            rows[r].append(o.transpose(0, 1))
        finals.append(S)
    o = torch.stack([torch.cat(p, 0) for p in rows], 0).to(dt)
    return o, (torch.stack(finals, 0) if output_final_state else None)


@_native("gated_delta_rule", "torch_chunk_gated_delta_rule")
class TorchGatedDeltaRule(OpImpl):
    def __call__(self, q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False,
                 use_qk_l2norm_in_kernel=False, cu_seqlens=None, packed_params=None, chunk_size=64, **_):
        if packed_params is not None:
            if cu_seqlens is not None:
                raise ValueError("pass either cu_seqlens or packed_params, not both")
            cu_seqlens = packed_params.cu_seqlens
        return chunk_delta_rule(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                                use_qk_l2norm_in_kernel, chunk_size)


def kda_gate(g, A_log, dt_bias=None, lower_bound=None):
    """Per-channel log decay from the raw gate projection: `-exp(A_log) * softplus(g + dt_bias)`; with a
    `lower_bound` (negative) the bounded form `lower_bound * sigmoid(exp(A_log) * (g + dt_bias))` is used."""
    H, K = g.shape[-2:]
    x = g.float()
    if dt_bias is not None:
        x = x + dt_bias.float().view(H, K)
    a = A_log.float().exp().view(H, 1)
    if lower_bound is not None:
        return lower_bound * torch.sigmoid(a * x)
    return -a * F.softplus(x)


@_native("kda", "torch_chunk_kda")
class TorchKDA(OpImpl):
    """q, k: [B, T, H*K]; v: [B, T, H*V]; g: [B, T, H, K]; beta: [B, T, H].  Returns `[B, T, H, V]`."""

    def __call__(self, q, k, v, g, beta, *, A_log=None, dt_bias=None, scale=None, initial_state=None,
                 output_final_state=False, use_qk_l2norm_in_kernel=False, use_beta_sigmoid_in_kernel=True,
                 use_gate_in_kernel=False, safe_gate=False, lower_bound=None, cu_seqlens=None, chunk_size=32):
        K = g.shape[-1]
        H = beta.shape[-1]
        if q.dim() == 3:
            q, k = q.unflatten(-1, (H, K)), k.unflatten(-1, (H, K))
        if v.dim() == 3:
            v = v.unflatten(-1, (H, -1))
        if use_gate_in_kernel:
            if A_log is None:
                raise ValueError("use_gate_in_kernel needs A_log")
            g = kda_gate(g, A_log, dt_bias, lower_bound if safe_gate else None)
        if use_beta_sigmoid_in_kernel:
            beta = torch.sigmoid(beta.float())
        return chunk_delta_rule(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                                use_qk_l2norm_in_kernel, chunk_size)
