"""Per-layer lexical embeddings (PLE) of Qwen4-Exp on packed rows.

A PLE layer looks up, for every token, hashed n-gram rows (bigrams ... `ngram_size`-grams, `heads_per_ngram` hash
heads each) in one very large frozen table, projects them to a value and one key per residual stream, gates the value
by the agreement of key and stream, and adds a dilated depthwise causal convolution of the gated values.

    * hashing (`NGramHasher`): history tokens before the sample, in another packed sample, or behind an EOS count as
      EOS; an n-gram id is the XOR of `token * multiplier[position]`, reduced modulo a per-head prime table size
      (models/qwen4_exp/ple.py:48-125 and modeling_qwen4_exp.py:1017-1110 of the reference).  The hash runs on CPU
      token ids; only the selected rows travel to the GPU.
    * the table is a frozen CPU-resident parameter shared by the ranks of a node (`cpu_resident`).
    * the convolution never crosses a packed-sample boundary; under sequence parallelism each rank receives the last
      `(kernel - 1) * dilation` inputs of its left neighbour (halo) and, in backward, the matching gradient rows of
      its right neighbour (models/qwen4_exp/ple.py:167-225,353-437).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

_MASK64 = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK64
    return x ^ (x >> 31)


def layer_multipliers(vocab: int, ngram_size: int, ple_layer_index: int, seed: int) -> torch.Tensor:
    """One odd multiplier per history position, small enough that `token * multiplier` stays inside int64."""
    bound = max(((1 << 62) // max(vocab, 1)) | 1, 3)
    out, state = [], (seed * 10007 + ple_layer_index) & _MASK64
    for _ in range(ngram_size):
        state = _splitmix64(state)
        out.append(((state % bound) | 1))
    return torch.tensor(out, dtype=torch.long)


def _is_prime(n: int) -> bool:
    if n < 2:
        return False
    if n % 2 == 0:
        return n == 2
    i = 3
    while i * i <= n:
        if n % i == 0:
            return False
        i += 2
    return True


def nth_prime_after(start: int, count: int) -> int:
    n, found = start, 0
    while True:
        n += 1
        if _is_prime(n):
            found += 1
            if found == count:
                return n


@dataclass
class NGramHasher:
    eos_token_id: int
    ngram_size: int
    heads_per_ngram: int
    multipliers: torch.Tensor        # [ngram_size]
    head_sizes: torch.Tensor         # [(ngram_size - 1) * heads_per_ngram]
    head_offsets: torch.Tensor

    @classmethod
    def build(cls, vocab: int, ngram_size: int, heads_per_ngram: int, base: int, ple_layer_index: int, seed: int, eos: int):
        heads = (ngram_size - 1) * heads_per_ngram
        sizes, offsets, total = [], [], 0
        for h in range(heads):
            size = nth_prime_after(base - 1, ple_layer_index * heads + h + 1)
            sizes.append(size)
            offsets.append(total)
            total += size
        return cls(eos, ngram_size, heads_per_ngram, layer_multipliers(vocab, ngram_size, ple_layer_index, seed),
                   torch.tensor(sizes), torch.tensor(offsets)), total

    def row_ids(self, token_ids: torch.Tensor, segment_ids: torch.Tensor) -> torch.Tensor:
        """token_ids, segment_ids: [T] (segment 0 = padding) -> table rows [T, heads]."""
        tok = token_ids.long()
        T = tok.numel()
        pos = torch.arange(T)
        eos_pos = torch.where(tok == self.eos_token_id, pos, torch.full_like(pos, -1))
        prev_eos = F.pad(eos_pos.cummax(0).values[:-1], (1, 0), value=-1)
        shifted = [tok]
        for s in range(1, self.ngram_size):
            src = pos - s
            idx = src.clamp_min(0)
            ok = (src >= 0) & segment_ids.ne(0) & segment_ids.eq(segment_ids[idx]) & (pos - prev_eos - 1 >= s)
            shifted.append(torch.where(ok, tok[idx], torch.full_like(tok, self.eos_token_id)))
        blocks = []
        for n in range(2, self.ngram_size + 1):
            mix = shifted[0] * self.multipliers[0]
            for j in range(1, n):
                mix = torch.bitwise_xor(mix, shifted[j] * self.multipliers[j])
            a = (n - 2) * self.heads_per_ngram
            b = a + self.heads_per_ngram
            blocks.append(torch.remainder(mix.unsqueeze(-1), self.head_sizes[a:b]) + self.head_offsets[a:b])
        return torch.cat(blocks, dim=-1)


# --------------------------------------------------------------------------------------------------
# segment-aware dilated causal depthwise convolution with sequence-parallel halos
# --------------------------------------------------------------------------------------------------
def _conv_window(x, seg, weight, dilation: int):
    """x [L, C], seg [L], weight [C, K] -> y [L, C]; taps never cross a segment boundary."""
    L, K = x.shape[0], weight.shape[-1]
    y = torch.zeros_like(x)
    for k in range(K):
        lag = (K - 1 - k) * dilation
        if lag >= L:
            continue
        c = x[: L - lag] * weight[:, k]
        if lag:
            c = c.masked_fill(seg[lag:].ne(seg[:-lag]).unsqueeze(-1), 0)
        y = torch.cat((y[:lag], y[lag:] + c), 0) if lag else y + c
    return y


class _HaloConv(torch.autograd.Function):
    """y_local = conv([left halo | x_local]); backward sends each rank the gradient rows its halo contributed to."""

    @staticmethod
    def forward(ctx, x, weight, seg_global, dilation, group, sp, rank):
        Tl = x.shape[0]
        hist = (weight.shape[-1] - 1) * dilation
        left = min(hist, rank * Tl) if sp > 1 else 0
        xin = x
        if sp > 1 and hist:
            h = min(hist, Tl)
            tails = x.new_empty(sp * h, x.shape[1])
            dist.all_gather_into_tensor(tails, x[-h:].contiguous(), group=group)
            stop = rank * h
            xin = torch.cat((tails[max(0, stop - hist):stop], x), 0)
            left = xin.shape[0] - Tl
        start = rank * Tl
        seg = seg_global[start - left:start + Tl]
        with torch.enable_grad():
            xin_ = xin.detach().requires_grad_(True)
            w_ = weight.detach().requires_grad_(True)
            y_all = _conv_window(xin_, seg, w_, dilation)
        ctx.save_for_backward(xin_, w_, y_all)
        ctx.meta = (Tl, left, hist, group, sp, rank)
        return y_all[left:].detach()

    @staticmethod
    def backward(ctx, gy):
        xin_, w_, y_all = ctx.saved_tensors
        Tl, left, hist, group, sp, rank = ctx.meta
        g_all = torch.cat((gy.new_zeros(left, gy.shape[1]), gy), 0)
        gx_all, gw = torch.autograd.grad(y_all, (xin_, w_), g_all)
        gx = gx_all[left:].clone()
        if sp > 1 and hist:
            # gradient that my halo rows carry belongs to the left neighbour's tail: exchange and add
            h = min(hist, Tl)
            mine = gy.new_zeros(h, gy.shape[1])
            if left:
                mine[h - left:] = gx_all[:left][-h:] if left >= h else gx_all[:left]
            gathered = gy.new_empty(sp * h, gy.shape[1])
            dist.all_gather_into_tensor(gathered, mine.contiguous(), group=group)
            if rank + 1 < sp:
                gx[-h:] += gathered[(rank + 1) * h:(rank + 2) * h]
        return gx, gw, None, None, None, None, None


def segment_causal_conv(x, weight, seg_global, dilation, sp_group=None, sp_size=1, sp_rank=0):
    """x [T_local, C]; weight [C, K] (tap K-1 = current token); seg_global [T] sample ids (0 = padding)."""
    return _HaloConv.apply(x, weight, seg_global, dilation, sp_group, sp_size, sp_rank)


# --------------------------------------------------------------------------------------------------
# the layer
# --------------------------------------------------------------------------------------------------
class GroupRMSNorm(nn.Module):
    """RMSNorm over consecutive groups of `group_size` channels with one weight per channel."""

    def __init__(self, dim: int, group_size: int, eps: float, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))
        self.group, self.eps = group_size, eps

    def forward(self, x):
        xf = x.float().unflatten(-1, (-1, self.group))
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (y.flatten(-2) * self.weight.float()).to(x.dtype)


class PLELayer(nn.Module):
    def __init__(self, config, layer_idx: int, ple_layer_index: int, dtype=None):
        super().__init__()
        c = config
        self.H, self.hc, self.ple_layer_index = c.hidden_size, c.hc_count, ple_layer_index
        heads = (c.ngram_size - 1) * c.heads_per_ngram
        eos = c.eos_token_id[0] if isinstance(c.eos_token_id, (list, tuple)) else c.eos_token_id
        self.hasher, total = NGramHasher.build(c.vocab_size, c.ngram_size, c.heads_per_ngram, c.ngram_vocab_size_base,
                                               ple_layer_index, c.seed, eos)
        div = c.make_ngram_vocab_size_divisible_by
        rows = math.ceil(total / div) * div
        self.head_dim = c.ple_embed_dim // heads
        # the big frozen table: a plain parameter here; `on_materialized` may move it to node-shared CPU memory
        self.ngram_embedding = nn.Embedding(rows, self.head_dim, dtype=dtype)
        self.ngram_embedding.weight.requires_grad_(False)
        D = c.ple_embed_dim
        self.key_proj = nn.Linear(D, self.hc * self.H, bias=False, dtype=dtype)
        self.value_proj = nn.Linear(D, self.H, bias=False, dtype=dtype)
        self.norm_key = GroupRMSNorm(self.hc * self.H, self.H, c.rms_norm_eps, dtype)
        self.norm_query = GroupRMSNorm(self.hc * self.H, self.H, c.rms_norm_eps, dtype)
        self.norm_conv = GroupRMSNorm(self.hc * self.H, self.H, c.rms_norm_eps, dtype)
        self.dilation = c.ngram_size
        self.conv1d = nn.Conv1d(self.hc * self.H, self.hc * self.H, c.ple_conv_kernel_size, groups=self.hc * self.H,
                                dilation=self.dilation, bias=False, dtype=dtype)

    def lookup(self, token_ids_cpu: torch.Tensor, segment_ids_cpu: torch.Tensor, device) -> torch.Tensor:
        """[T] ids -> [T, ple_embed_dim] rows on `device` (hash and gather on the table's device)."""
        rows = self.hasher.row_ids(token_ids_cpu, segment_ids_cpu)
        w = self.ngram_embedding.weight
        emb = w.index_select(0, rows.flatten().to(w.device)).view(rows.shape[0], -1)
        return emb.to(device)

    def forward(self, h, emb, seg_global, sp_group=None, sp_size=1, sp_rank=0):
        """h [T_local, hc*H] residual streams; emb [T_local, ple_embed_dim]; returns the increment [T_local, hc*H]."""
        Tl = h.shape[0]
        emb = emb.to(h.dtype)
        key = self.norm_key(F.linear(emb, self.key_proj.weight)).view(Tl, self.hc, self.H)
        value = F.linear(emb, self.value_proj.weight)
        query = self.norm_query(h).view(Tl, self.hc, self.H)
        gate = (key * query).sum(-1, keepdim=True) / math.sqrt(self.H)
        gate = gate.abs().clamp_min(1e-6).sqrt() * gate.sign()
        gated = (torch.sigmoid(gate) * value.unsqueeze(1)).flatten(1)
        normed = self.norm_conv(gated)
        keep = seg_global[sp_rank * Tl:(sp_rank + 1) * Tl].ne(0).unsqueeze(-1).to(h.device)
        gated, normed = gated * keep, normed * keep
        conv = segment_causal_conv(normed, self.conv1d.weight.squeeze(1), seg_global.to(h.device), self.dilation,
                                   sp_group, sp_size, sp_rank)
        return (gated + conv).to(h.dtype)
