"""Chunked (gated) delta rule for GatedDeltaNet and Kimi Delta Attention layers on B200.

The chunked evaluation splits into work that is parallel over chunks and one recurrence over chunks:

  chunk-parallel (batched GEMMs and a batched triangular solve over all `[head, chunk]` pairs at once):
      G = cumsum(g) inside the chunk,  D_ij = exp(G_i - G_j) (i >= j)
      T = (I + strict_lower(k beta k^T . D))^-1,  u = T (beta v),  w = T (beta k e^G)
      q_in = q e^G,  k_out = k e^(G_last - G),  d = e^(G_last)
  recurrence (the `delta_state` tcgen05 kernel, one CTA per sequence and head, forward and reverse):
      v_new_c = u_c - w_c S_c,        S_{c+1} = d_c (.) S_c + k_out_c^T v_new_c
  chunk-parallel again:
      o_c = q_in_c S_c + tril(q k^T . D) v_new_c

`StateScan` is the autograd function around the recurrence: its backward is the same kernel run over the chunks in
reverse (dS_c = d_c (.) dS_{c+1} - w_c^T dv_new_c + gS_c, dv_new_c = g_c + k_out_c dS_{c+1}) followed by batched products
for the operand gradients; everything chunk-parallel is differentiated by autograd.  Without CUDA (or for head
widths other than 128) the recurrence runs as a torch loop, so the formulation is testable on CPU against the
token-by-token oracle.  Counterpart of the `chunk_gated_delta_rule` / `chunk_kda` operators of flash-linear-attention
used by the reference (ops/providers/native/gated_delta_rule.py, ops/providers/native/kda.py)."""
from __future__ import annotations

import torch

from ... import kernels as K
from ...runtime import TurboDevice
from ..base import OpImpl, OpImplKind
from ..registry import register_op
from .native_linear_attention import _bounds, kda_gate, l2norm

CHUNK = 64


def _kernel_ok(t: torch.Tensor, kdim: int, vdim: int) -> bool:
    return t.is_cuda and kdim == 128 and vdim == 128 and K.available()


def _scan_torch(u, w, k_out, decay, init, seq_chunks, reverse=False, add=None, s1=-1.0, s2=1.0):
    """Torch form of the recurrence (same contract as the kernel): returns (X [H, NC, C, V], states [H, NC + nseq, K, V])."""
    H, NC, C, V = u.shape
    Kd = w.shape[-1]
    nseq = len(seq_chunks)
    X = [None] * NC
    states = [None] * (NC + nseq)
    for s, (c0, n) in enumerate(seq_chunks):
        if reverse:
            S = add[:, c0 + n + s]
        else:
            S = init[:, s] if init is not None else u.new_zeros(H, Kd, V)
        states[(c0 + n if reverse else c0) + s] = S
        order = range(c0 + n - 1, c0 - 1, -1) if reverse else range(c0, c0 + n)
        for c in order:
            x = u[:, c] + s1 * (w[:, c] @ S)
            X[c] = x
            d = decay[:, c]
            S = S * (d[:, :, None] if d.dim() == 2 else d[:, None, None]) + s2 * (k_out[:, c].transpose(-1, -2) @ x)
            slot = (c if reverse else c + 1) + s
            if add is not None:
                S = S + add[:, slot]
            states[slot] = S
    return torch.stack(X, 1), torch.stack(states, 1)


class StateScan(torch.autograd.Function):
    """(u, w, k_out, decay, init) -> (v_new, states) through the `delta_state` kernel; `seq_chunks` is the host list of
    (first chunk, chunk count) per sequence and `seq_dev` the same table on the device."""

    @staticmethod
    def forward(ctx, u, w, k_out, decay, init, seq_chunks, seq_dev):
        wb, kb = w.to(torch.bfloat16).contiguous(), k_out.to(torch.bfloat16).contiguous()
        u = u.contiguous()
        decay = decay.contiguous()
        x, states = K.delta_state_scan(wb, kb, u, decay, init, None, seq_dev, reverse=False, s1=-1.0, s2=1.0)
        ctx.save_for_backward(wb, kb, decay, x, states, seq_dev)
        ctx.seq_chunks = seq_chunks
        ctx.has_init = init is not None
        ctx.w_dtype, ctx.k_dtype = w.dtype, k_out.dtype
        return x, states

    @staticmethod
    def backward(ctx, gx, gstates):
        wb, kb, decay, x, states, seq_dev = ctx.saved_tensors
        seq_chunks = ctx.seq_chunks
        H, NC = x.shape[:2]
        dev = x.device
        gx = gx.contiguous() if gx is not None else torch.zeros_like(x)
        gstates = gstates.contiguous() if gstates is not None else torch.zeros_like(states)
        # reverse recurrence: A = k_out, B = w
        dx, dS = K.delta_state_scan(kb, wb, gx, decay, None, gstates, seq_dev, reverse=True, s1=1.0, s2=-1.0)
        start = torch.tensor([c + s for s, (c0, n) in enumerate(seq_chunks) for c in range(c0, c0 + n)], device=dev)
        S_c = states.index_select(1, start)                     # state at the start of every chunk
        dS_n = dS.index_select(1, start + 1)                    # gradient of the state that leaves the chunk
        dw = -(dx @ S_c.transpose(-1, -2))
        dk_out = x @ dS_n.transpose(-1, -2)
        prod = dS_n * S_c
        ddecay = prod.sum((-1, -2)) if decay.dim() == 2 else prod.sum(-1)
        dinit = None
        if ctx.has_init:
            first = torch.tensor([c0 + s for s, (c0, n) in enumerate(seq_chunks)], device=dev)
            dinit = dS.index_select(1, first)
        return dx, dw.to(ctx.w_dtype), dk_out.to(ctx.k_dtype), ddecay, dinit, None, None


def _layout(segs, T_total: int, C: int, device):
    """Gather / scatter indices between packed tokens and the zero-padded `[chunk, C]` layout."""
    gather, seq_chunks, inv = [], [], torch.full((T_total,), -1, dtype=torch.long)
    c = 0
    for base, a, b in segs:
        L = b - a
        n = (L + C - 1) // C
        idx = torch.full((n * C,), T_total, dtype=torch.long)         # padding reads the appended zero row
        idx[:L] = torch.arange(base + a, base + b)
        inv[base + a: base + b] = c * C + torch.arange(L)
        gather.append(idx)
        seq_chunks.append((c, n))
        c += n
    gather = torch.cat(gather) if gather else torch.zeros(0, dtype=torch.long)
    return gather.to(device), inv.to(device), seq_chunks, c


def _channel_decay_products(kb, qc, kc, G, head_slab: int = 8, sub: int = 16):
    """`sum_k x[i, k] kc[j, k] exp(G[i, k] - G[j, k])` on `i >= j` (zero above the diagonal) for `x` in (kb, qc), with
    per-channel cumulative log decays `G [H, NC, C, K]` (non-increasing along C).

    The chunk is cut into sub-chunks of `sub` rows.  Between different sub-chunks the decay factorises around the first
    row `r` of the later one, `exp(G_i - G_r) exp(G_r - G_j)`, with both exponents non-positive, so those blocks are
    plain matrix products; only the `sub x sub` diagonal blocks materialise pairwise decays (`[.., sub, sub, K]`, a
    sixteenth of the `[.., C, C, K]` tensor per block row), a few heads at a time."""
    H, NC, C, Kd = G.shape
    nsb = C // sub
    x = torch.stack((kb, qc))                                              # [2, H, NC, C, K]
    rows = []
    tril = torch.ones(sub, sub, dtype=torch.bool, device=G.device).tril()
    for a in range(nsb):
        ra = slice(a * sub, (a + 1) * sub)
        Ga = G[:, :, ra]                                                    # [H, NC, sub, K]
        parts = []
        if a > 0:
            ref = Ga[:, :, :1]                                              # first row of this sub-chunk
            left = x[:, :, :, ra] * (Ga - ref).exp()
            right = kc[:, :, : a * sub] * (ref - G[:, :, : a * sub]).exp()
            parts.append(left @ right.transpose(-1, -2))                    # [2, H, NC, sub, a * sub]
        diag = []
        for h0 in range(0, H, head_slab):
            sl = slice(h0, h0 + head_slab)
            Dm = (Ga[sl, :, :, None, :] - Ga[sl, :, None, :, :]).masked_fill(~tril[None, None, :, :, None], -float("inf")).exp()
            diag.append(torch.einsum("xhnik,hnijk,hnjk->xhnij", x[:, sl, :, ra], Dm, kc[sl, :, ra]))
        parts.append(torch.cat(diag, 1))
        if a + 1 < nsb:
            parts.append(x.new_zeros(2, H, NC, sub, C - (a + 1) * sub))
        rows.append(torch.cat(parts, -1))
    out = torch.cat(rows, -2)                                               # [2, H, NC, C, C]
    return out[0], out[1]


def chunk_delta_rule_batched(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
                             use_qk_l2norm=False, head_slab: int = 8):
    """q, k: [B, T, H, K]; v: [B, T, H, V]; g: [B, T, H] (scalar log decay) or [B, T, H, K]; beta: [B, T, H].
    Returns (o [B, T, H, V] in v's dtype, final state [N, H, K, V] fp32 or None)."""
    B, T, H, Kd = q.shape
    V = v.shape[-1]
    dt = v.dtype
    dev = q.device
    C = CHUNK
    scale = Kd ** -0.5 if scale is None else scale
    qf, kf, vf, gf, bf = (t.float() for t in (q, k, v, g, beta))
    if use_qk_l2norm:
        qf, kf = l2norm(qf), l2norm(kf)
    if cu_seqlens is not None and B != 1:
        raise ValueError("packed delta rule expects a single row")
    segs = [(0, a, b) for a, b in _bounds(cu_seqlens, T)] if cu_seqlens is not None else [(r * T, 0, T) for r in range(B)]
    vec = gf.dim() == 4
    # sequences that are whole chunks and tile the rows need no gather: the chunk layout is a view of the packed rows
    aligned = all((b - a) % C == 0 for _, a, b in segs) and sum(b - a for _, a, b in segs) == B * T
    if aligned:
        seq_chunks, NC = [], 0
        for _, a, b in segs:
            seq_chunks.append((NC, (b - a) // C))
            NC += (b - a) // C
        gather = inv = None
    else:
        gather, inv, seq_chunks, NC = _layout(segs, B * T, C, dev)

    def to_chunks(x):                                   # [B, T, H, ...] -> [H, NC, C, ...]
        flat = x.reshape(B * T, *x.shape[2:])
        if not aligned:
            flat = torch.cat((flat, flat.new_zeros(1, *flat.shape[1:])), 0).index_select(0, gather)
        return flat.reshape(NC, C, *flat.shape[1:]).movedim(2, 0)

    qc, kc, vc = to_chunks(qf) * scale, to_chunks(kf), to_chunks(vf)            # [H, NC, C, K|V]
    bc = to_chunks(bf.unsqueeze(-1)).squeeze(-1)                                # [H, NC, C]
    G = (to_chunks(gf) if vec else to_chunks(gf.unsqueeze(-1)).squeeze(-1)).cumsum(2)
    eye = torch.eye(C, dtype=torch.float32, device=dev)
    low = torch.ones(C, C, dtype=torch.bool, device=dev).tril(-1)
    lowd = torch.ones(C, C, dtype=torch.bool, device=dev).tril()
    kb = kc * bc[..., None]
    if vec:
        kk, qk = _channel_decay_products(kb, qc, kc, G, head_slab)
        eG = G.exp()
        k_in, q_in = kb * eG, qc * eG
        k_out = kc * (G[:, :, -1:, :] - G).exp()
        decay = G[:, :, -1].exp()                                               # [H, NC, K]
    else:
        Dm = (G[..., :, None] - G[..., None, :]).masked_fill(~lowd, -float("inf")).exp()
        kk = (kb @ kc.transpose(-1, -2)) * Dm
        qk = (qc @ kc.transpose(-1, -2)) * Dm
        eG = G.exp()[..., None]
        k_in, q_in = kb * eG, qc * eG
        k_out = kc * (G[..., -1:] - G).exp()[..., None]
        decay = G[..., -1].exp()                                                # [H, NC]
    Tm = torch.linalg.solve_triangular(eye + kk.masked_fill(~low, 0.0), eye.expand(H, NC, C, C), upper=False)
    u = Tm @ (vc * bc[..., None])
    w = Tm @ k_in
    init = None
    if initial_state is not None:
        init = initial_state.float().transpose(0, 1).contiguous()               # [H, N, K, V]
    if _kernel_ok(q, Kd, V):
        seq_dev = torch.tensor(seq_chunks, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        v_new, states = StateScan.apply(u, w, k_out, decay, init, seq_chunks, seq_dev)
    else:
        v_new, states = _scan_torch(u, w, k_out, decay, init, seq_chunks)
    start = torch.tensor([c + s for s, (c0, n) in enumerate(seq_chunks) for c in range(c0, c0 + n)], device=dev)
    S_c = states.index_select(1, start)
    o = q_in @ S_c + qk.masked_fill(~lowd, 0.0) @ v_new                          # [H, NC, C, V]
    o = o.movedim(0, 2).reshape(NC * C, H, V)
    if aligned:
        o = o.reshape(B, T, H, V)
    else:
        covered = sum(b - a for _, a, b in segs) == B * T
        o = o.index_select(0, inv.clamp_min(0)).reshape(B, T, H, V)
        if not covered:                                                         # rows past the last boundary read as zero
            o = o * (inv >= 0).reshape(B, T, 1, 1)
    final = None
    if output_final_state:
        last = torch.tensor([c0 + n + s for s, (c0, n) in enumerate(seq_chunks)], device=dev)
        final = states.index_select(1, last).transpose(0, 1).contiguous()
    return o.to(dt), final


def _register(op_name: str, impl_name: str):
    return register_op(op_name=op_name, impl_name=impl_name, kind=OpImplKind.CUSTOM, priority=100, devices=(TurboDevice.CUDA,))


@_register("gated_delta_rule", "b200_chunk_gated_delta_rule")
class B200GatedDeltaRule(OpImpl):
    def available(self) -> bool:
        return K.available()

    def __call__(self, q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False,
                 use_qk_l2norm_in_kernel=False, cu_seqlens=None, packed_params=None, chunk_size=64, **_):
        if packed_params is not None:
            if cu_seqlens is not None:
                raise ValueError("pass either cu_seqlens or packed_params, not both")
            cu_seqlens = packed_params.cu_seqlens
        return chunk_delta_rule_batched(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                                        use_qk_l2norm_in_kernel)


@_register("kda", "b200_chunk_kda")
class B200KDA(OpImpl):
    """q, k: [B, T, H*K]; v: [B, T, H*V]; g: [B, T, H, K]; beta: [B, T, H].  Returns `[B, T, H, V]`."""

    def available(self) -> bool:
        return K.available()

    def __call__(self, q, k, v, g, beta, *, A_log=None, dt_bias=None, scale=None, initial_state=None,
                 output_final_state=False, use_qk_l2norm_in_kernel=False, use_beta_sigmoid_in_kernel=True,
                 use_gate_in_kernel=False, safe_gate=False, lower_bound=None, cu_seqlens=None, chunk_size=64):
        Kd = g.shape[-1]
        H = beta.shape[-1]
        if q.dim() == 3:
            q, k = q.unflatten(-1, (H, Kd)), k.unflatten(-1, (H, Kd))
        if v.dim() == 3:
            v = v.unflatten(-1, (H, -1))
        if use_gate_in_kernel:
            if A_log is None:
                raise ValueError("use_gate_in_kernel needs A_log")
            g = kda_gate(g, A_log, dt_bias, lower_bound if safe_gate else None)
        if use_beta_sigmoid_in_kernel:
            beta = torch.sigmoid(beta.float())
        return chunk_delta_rule_batched(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                                        use_qk_l2norm_in_kernel)


__all__ = ["B200GatedDeltaRule", "B200KDA", "StateScan", "chunk_delta_rule_batched"]
