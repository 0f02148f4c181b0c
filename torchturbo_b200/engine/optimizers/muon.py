"""Distributed Muon on FSDP-sharded storage, with AdamW for everything that is not a hidden matrix.

Muon's update needs each *complete* matrix (Newton-Schulz orthogonalisation of the momentum), while FSDP2 stores
row shards.  Per optimizer step, for every bucket of matrices:
  1. every matrix has an owner rank, chosen once by greedy load balancing of `NS flops + 2000 x bytes moved`
     (the reference's cost model: engine/backends/fsdp2/optimizers/muon.py:52-53, 1499-1605);
  2. ranks pack the momentum shards per owner and exchange them with one all-to-all (split sizes follow from shapes,
     so the host never waits on the device);
  3. owners reassemble full matrices, run Newton-Schulz in bf16 (batched for fused expert tensors and for the
     q / k / v or gate / up blocks of fused projections), and the result returns through the inverse exchange;
  4. every rank applies `p = p * (1 - lr * wd) - lr_adj * update` to its shard.
Matrices that live entirely on one rank (single-rank units, EP-local experts) skip the exchange.
`MuonParameterSpec` describes how a stored tensor decomposes into independent matrices.  All ranks hash their plan
and compare hashes before the first step so that a divergent plan fails loudly instead of deadlocking.
"""
from __future__ import annotations

import hashlib
import json
import math
from dataclasses import dataclass, field
from typing import Any, Iterable

import torch
import torch.distributed as dist
import torch.nn as nn

from ...utils.fqn import match_fqn

COLLECTIVE_FLOPS_PER_BYTE = 2000


@dataclass(frozen=True)
class MuonParameterSpec:
    """A stored 2-D tensor `[batch * rows, cols]` (or `[rows, cols]`) holding `batch` matrices; `row_blocks` /
    `col_blocks` further split each matrix into independently orthogonalised blocks (fused q|k|v rows, gate|up cols)."""

    batch: int = 1
    row_blocks: tuple[int, ...] = ()
    col_blocks: tuple[int, ...] = ()

    def matrices(self, full: torch.Tensor) -> list[torch.Tensor]:
        """Views `[b, r, c]` covering `full` ([batch*rows, cols])."""
        R, C = full.shape
        rows = R // self.batch
        x = full.view(self.batch, rows, C)
        rb = self.row_blocks or (rows,)
        cb = self.col_blocks or (C,)
        out, r0 = [], 0
        for r in rb:
            c0 = 0
            for c in cb:
                out.append(x[:, r0:r0 + r, c0:c0 + c])
                c0 += c
            r0 += r
        return out


@dataclass
class MuonRecipe:
    """Which parameters Muon owns (FQN pattern -> spec); everything else goes to AdamW."""

    matrices: dict[str, MuonParameterSpec] = field(default_factory=dict)
    exclude: tuple[str, ...] = ()

    def spec_for(self, name: str) -> MuonParameterSpec | None:
        if any(match_fqn(p, name) for p in self.exclude):
            return None
        for pat, spec in self.matrices.items():
            if match_fqn(pat, name):
                return spec
        return None


def default_decoder_muon_recipe(model: nn.Module) -> MuonRecipe:
    """Hidden matrices of a decoder: attention and MLP projections (fused ones split into their blocks) and fused
    expert tensors (one matrix per expert).  Embeddings, the output head, norms and routers stay on AdamW."""
    cfg = model.config
    tc = getattr(cfg, "text_config", cfg)
    D, nq, nkv = tc.head_dim, tc.num_attention_heads, tc.num_key_value_heads
    rec: dict[str, MuonParameterSpec] = {
        "**.self_attn.qkv_proj.weight": MuonParameterSpec(row_blocks=(nq * D, nkv * D, nkv * D)),
        "**.self_attn.o_proj.weight": MuonParameterSpec(),
        "**.mlp.gate_up_proj.weight": MuonParameterSpec(row_blocks=(tc.intermediate_size, tc.intermediate_size)),
        "**.mlp.down_proj.weight": MuonParameterSpec(),
        "**.shared_experts.gate_up_proj.weight": MuonParameterSpec(),
        "**.shared_experts.down_proj.weight": MuonParameterSpec(),
    }
    for name, mod in model.named_modules():
        if hasattr(mod, "get_muon_parameter_specs"):
            E = mod.num_local_experts
            Fh = mod.config.moe_ffn_hidden_size
            rec[f"{name}.weight1"] = MuonParameterSpec(batch=E, col_blocks=(Fh, Fh))
            rec[f"{name}.weight2"] = MuonParameterSpec(batch=E)
    return MuonRecipe(rec, exclude=("**.embed_tokens.weight", "lm_head.weight", "**.router.weight", "**.visual.**"))


def _ns_tcgen05_ok(X: torch.Tensor) -> bool:
    if not X.is_cuda or X.shape[-1] % 8 or X.shape[-2] % 8:
        return False
    from ... import kernels as K

    return K.available()


def _newton_schulz_tcgen05(X: torch.Tensor, steps: int, coeffs) -> torch.Tensor:
    """The iteration on the library's tcgen05 GEMM, one matrix of the batch at a time: `A = X X^T` and `A A` (A is
    symmetric, so both are NT products), `X <- a X + B X` with the `a X` term added by the GEMM's residual epilogue."""
    from ... import kernels as K

    per_step = isinstance(coeffs[0], (tuple, list))
    out = []
    for x in X:
        x = x.contiguous()
        for i in range(steps):
            a, b, c = coeffs[i] if per_step else coeffs
            A = K.gemm(x, x)                                     # [r, r] = x x^T
            B = K.gemm(A, A, residual=(A * (b / c)).contiguous()) * c if c != 0 else A * b     # b A + c A A
            x = K.gemm(B.contiguous(), x, b_mn=True, residual=(x * a).contiguous())            # a x + B x
        out.append(x)
    return torch.stack(out, 0)


def newton_schulz(G: torch.Tensor, steps: int, coeffs, eps: float) -> torch.Tensor:
    """Batched Newton-Schulz orthogonalisation in bf16.  G: [b, r, c] -> same shape."""
    X = G.to(torch.bfloat16)
    transposed = X.shape[-2] > X.shape[-1]
    if transposed:
        X = X.transpose(-2, -1)
    X = X / (X.float().norm(dim=(-2, -1), keepdim=True) + eps).to(X.dtype)
    if X.dim() == 3 and _ns_tcgen05_ok(X):
        X = _newton_schulz_tcgen05(X, steps, coeffs)
        return X.transpose(-2, -1) if transposed else X
    per_step = isinstance(coeffs[0], (tuple, list))
    for i in range(steps):
        a, b, c = coeffs[i] if per_step else coeffs
        A = X @ X.transpose(-2, -1)
        B = torch.baddbmm(A, A, A, beta=b, alpha=c)
        X = torch.baddbmm(X, B, X, beta=a, alpha=1.0)
    return X.transpose(-2, -1) if transposed else X


def adjusted_lr(lr: float, rows: int, cols: int, fn: str | None) -> float:
    if fn in (None, "original"):
        return lr * math.sqrt(max(1.0, rows / cols))
    if fn == "match_rms_adamw":
        return lr * 0.2 * math.sqrt(max(rows, cols))
    if fn == "spectral_unclamped":
        return lr * math.sqrt(rows / cols)
    raise ValueError(f"unknown adjust_lr_fn {fn!r}")


def _local(t):
    return t._local_tensor if hasattr(t, "_local_tensor") else t


@dataclass
class _Entry:
    name: str
    param: nn.Parameter
    spec: MuonParameterSpec
    full_rows: int
    cols: int
    sharded: bool
    owner: int = 0
    row_ranges: list[tuple[int, int]] = field(default_factory=list)  # per rank [lo, hi) of dim 0


class DistributedMuon(torch.optim.Optimizer):
    def __init__(self, named_params: Iterable[tuple[str, nn.Parameter, MuonParameterSpec]], lr: float = 2e-2,
                 weight_decay: float = 0.0, momentum: float = 0.95, nesterov: bool = True,
                 ns_coefficients=(3.4445, -4.7750, 2.0315), ns_steps: int = 5, eps: float = 1e-7,
                 adjust_lr_fn: str | None = "match_rms_adamw", group=None, bucket_cap_mb: float | None = None):
        triples = list(named_params)
        super().__init__([p for _, p, _ in triples], dict(lr=lr, weight_decay=weight_decay, momentum=momentum))
        self.nesterov, self.ns_coefficients, self.ns_steps, self.eps = nesterov, ns_coefficients, ns_steps, eps
        self.adjust_lr_fn = adjust_lr_fn
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.entries = [self._make_entry(n, p, s) for n, p, s in triples]
        self._assign_owners()
        self.buckets = self._make_buckets(bucket_cap_mb)
        self._verified = False
        self._failed = False

    # -- planning --------------------------------------------------------------------------------------
    def _make_entry(self, name, p, spec) -> _Entry:
        sharded = hasattr(p, "_local_tensor") and p.device_mesh.size() > 1
        R, C = p.shape
        e = _Entry(name, p, spec, R, C, sharded)
        if sharded:
            n = p.device_mesh.size()
            chunk = -(-R // n)
            e.row_ranges = [(min(r * chunk, R), min((r + 1) * chunk, R)) for r in range(n)]
        return e

    def _cost(self, e: _Entry) -> float:
        rows = e.full_rows // e.spec.batch
        m, n = min(rows, e.cols), max(rows, e.cols)
        flops = e.spec.batch * self.ns_steps * (2 * m * m * n * 2 + 2 * m * m * m)
        comm = 2 * e.full_rows * e.cols * 2 * COLLECTIVE_FLOPS_PER_BYTE if e.sharded else 0
        return flops + comm

    def _assign_owners(self) -> None:
        loads = [0.0] * self.world
        for e in sorted((x for x in self.entries if x.sharded), key=lambda x: (-self._cost(x), x.name)):
            o = min(range(self.world), key=lambda r: (loads[r], r))
            e.owner = o
            loads[o] += self._cost(e)

    def _make_buckets(self, cap_mb: float | None) -> list[list[_Entry]]:
        sharded = [e for e in self.entries if e.sharded]
        if not sharded:
            return []
        if cap_mb is None:
            return [[e] for e in sharded]
        cap = cap_mb * 2 ** 20
        buckets, cur, size = [], [], 0
        for e in sharded:
            b = e.full_rows * e.cols * 2
            if cur and size + b > cap:
                buckets.append(cur)
                cur, size = [], 0
            cur.append(e)
            size += b
        if cur:
            buckets.append(cur)
        return buckets

    def plan_hash(self) -> str:
        desc = [(e.name, e.full_rows, e.cols, e.sharded, e.owner, e.spec.batch, e.spec.row_blocks, e.spec.col_blocks)
                for e in self.entries]
        return hashlib.sha256(json.dumps(desc, sort_keys=True).encode()).hexdigest()

    def _verify_plan(self) -> None:
        if self._verified or self.world == 1:
            self._verified = True
            return
        hashes: list[Any] = [None] * self.world
        dist.all_gather_object(hashes, self.plan_hash(), group=self.group)
        if len(set(hashes)) != 1:
            raise RuntimeError(f"Muon plans differ across ranks: {hashes}")
        self._verified = True

    # -- step ------------------------------------------------------------------------------------------
    def _momentum(self, e: _Entry, group) -> torch.Tensor:
        p = e.param
        st = self.state[p]
        g = _local(p.grad).float()
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros_like(_local(p), dtype=torch.float32)
        buf = st["momentum_buffer"]
        buf.lerp_(g, 1 - group["momentum"])
        return g.lerp(buf, group["momentum"]) if self.nesterov else buf

    def _orthogonalise(self, e: _Entry, full: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(full, dtype=torch.bfloat16)
        for src, dst in zip(e.spec.matrices(full), e.spec.matrices(out)):
            dst.copy_(newton_schulz(src, self.ns_steps, self.ns_coefficients, self.eps))
        return out

    def _apply(self, e: _Entry, update_local: torch.Tensor, group) -> None:
        rows = (e.full_rows // e.spec.batch)
        rb = e.spec.row_blocks or (rows,)
        cb = e.spec.col_blocks or (e.cols,)
        lr = adjusted_lr(group["lr"], rb[0], cb[0], self.adjust_lr_fn)
        lp = _local(e.param)
        master = self.state[e.param].get("master")
        tgt = master if master is not None else lp
        tgt.mul_(1 - group["lr"] * group["weight_decay"])
        tgt.add_(update_local.to(tgt.dtype), alpha=-lr)
        if master is not None:
            lp.copy_(master)

    @torch.no_grad()
    def step(self, closure=None):
        if self._failed:
            raise RuntimeError("a previous Muon step failed half-way; restart from a checkpoint")
        loss = closure() if closure is not None else None
        self._verify_plan()
        group = self.param_groups[0]
        try:
            for e in self.entries:
                if e.param.grad is None or e.sharded:
                    continue
                lp = _local(e.param)
                if lp.dtype != torch.float32 and "master" not in self.state[e.param]:
                    init = getattr(e.param, "_master_init", None)
                    self.state[e.param]["master"] = init if init is not None else lp.detach().float().clone()
                m = self._momentum(e, group)
                self._apply(e, self._orthogonalise(e, m.view(e.full_rows, e.cols)), group)
            self._run_buckets(group)
        except Exception:
            self._failed = True
            raise
        return loss

    def _run_buckets(self, group) -> None:
        """Two-slot software pipeline over the buckets: while the owners run Newton-Schulz on bucket i-1, the shards
        of bucket i are already travelling (asynchronous all-to-all on the communication stream / gloo thread), and
        the updates of bucket i-2 are applied once they have come back.  At most two buckets hold exchange buffers at
        any time.  `TORCHTURBO_MUON_PIPELINE=0` runs the three phases of every bucket back to back instead (same
        arithmetic, used as the reference in tests).  The reference's counterpart is `_run_async`
        (engine/backends/fsdp2/optimizers/muon.py:2286 there)."""
        import os

        live = [b for b in self.buckets if any(e.param.grad is not None for e in b)]
        if os.environ.get("TORCHTURBO_MUON_PIPELINE", "1") == "0":
            for b in live:
                ctx = self._bucket_gather(b, group, async_op=False)
                self._bucket_compute(ctx, async_op=False)
                self._bucket_finish(ctx, group)
            return
        n = len(live)
        ctxs: list[dict | None] = [None] * n
        for i in range(n + 2):
            if i < n:
                ctxs[i] = self._bucket_gather(live[i], group, async_op=True)
            if 1 <= i <= n:
                self._bucket_compute(ctxs[i - 1], async_op=True)
            if i >= 2:
                self._bucket_finish(ctxs[i - 2], group)
                ctxs[i - 2] = None

    def _bucket_gather(self, bucket: list[_Entry], group, *, async_op: bool) -> dict:
        """Phase 1: momentum update of this rank's shards, packed by owner, sent with one all-to-all."""
        W, r = self.world, self.rank
        live = [e for e in bucket if e.param.grad is not None]
        moms = {id(e): self._momentum(e, group).to(torch.bfloat16) for e in live}
        send_chunks, send_splits = [], [0] * W
        for o in range(W):
            for e in live:
                if e.owner == o:
                    lo, hi = e.row_ranges[r]
                    chunk = moms[id(e)][: hi - lo].reshape(-1)
                    send_chunks.append(chunk)
                    send_splits[o] += chunk.numel()
        recv_splits = [0] * W
        for s_ in range(W):
            for e in live:
                if e.owner == r:
                    lo, hi = e.row_ranges[s_]
                    recv_splits[s_] += (hi - lo) * e.cols
        dev = _local(live[0].param).device
        send = torch.cat(send_chunks) if send_chunks else torch.empty(0, dtype=torch.bfloat16, device=dev)
        recv = torch.empty(sum(recv_splits), dtype=torch.bfloat16, device=dev)
        work = dist.all_to_all_single(recv, send, recv_splits, send_splits, group=self.group, async_op=async_op)
        return {"live": live, "send": send, "recv": recv, "send_splits": send_splits, "recv_splits": recv_splits, "work": work,
                "dev": dev}

    def _bucket_compute(self, ctx: dict, *, async_op: bool) -> None:
        """Phase 2 (owners): reassemble the complete matrices, orthogonalise, send the rows back."""
        W, r = self.world, self.rank
        if ctx["work"] is not None:
            ctx["work"].wait()
        live, recv, dev = ctx["live"], ctx["recv"], ctx["dev"]
        mine = [e for e in live if e.owner == r]
        fulls = {id(e): torch.empty(e.full_rows, e.cols, dtype=torch.bfloat16, device=dev) for e in mine}
        off = 0
        for s_ in range(W):
            for e in mine:
                lo, hi = e.row_ranges[s_]
                n = (hi - lo) * e.cols
                fulls[id(e)][lo:hi].copy_(recv[off:off + n].view(hi - lo, e.cols))
                off += n
        outs = {id(e): self._orthogonalise(e, fulls[id(e)]) for e in mine}
        back_chunks = []
        for s_ in range(W):
            for e in mine:
                lo, hi = e.row_ranges[s_]
                back_chunks.append(outs[id(e)][lo:hi].reshape(-1))
        back = torch.cat(back_chunks) if back_chunks else torch.empty(0, dtype=torch.bfloat16, device=dev)
        ret = torch.empty(sum(ctx["send_splits"]), dtype=torch.bfloat16, device=dev)
        ctx["back"], ctx["ret"] = back, ret
        ctx["work"] = dist.all_to_all_single(ret, back, ctx["send_splits"], ctx["recv_splits"], group=self.group,
                                             async_op=async_op)
        ctx["send"] = ctx["recv"] = None

    def _bucket_finish(self, ctx: dict, group) -> None:
        """Phase 3: the orthogonalised rows of this rank's shards are back; apply them."""
        W, r = self.world, self.rank
        if ctx["work"] is not None:
            ctx["work"].wait()
        ret, off = ctx["ret"], 0
        for o in range(W):
            for e in ctx["live"]:
                if e.owner == o:
                    lo, hi = e.row_ranges[r]
                    n = (hi - lo) * e.cols
                    upd = torch.zeros_like(_local(e.param), dtype=torch.bfloat16)
                    upd[: hi - lo].copy_(ret[off:off + n].view(hi - lo, e.cols))
                    self._apply(e, upd, group)
                    off += n


def build_muon_optimizer(model: nn.Module, cfg, backend, lr: float | None = None, weight_decay: float | None = None,
                         **adamw_kwargs: Any):
    """Muon for the recipe's matrices + fused AdamW for the rest, wrapped in one container."""
    from . import FusedAdamW, OptimizersContainer
    from .plan import OptimizerClassPlan

    recipe = model.get_optimizer_recipe("muon")
    muon_params, rest = [], []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        spec = recipe.spec_for(name) if p.ndim == 2 else None
        (muon_params if spec is not None else rest).append((name, p, spec))
    mu_lr = cfg.lr if cfg.lr is not None else (lr if lr is not None else 2e-2)
    wd = cfg.weight_decay if cfg.weight_decay is not None else (weight_decay or 0.0)
    muon = DistributedMuon(muon_params, lr=mu_lr, weight_decay=wd, momentum=cfg.momentum, nesterov=cfg.nesterov,
                           ns_coefficients=cfg.ns_coefficients, ns_steps=cfg.ns_steps, eps=cfg.eps,
                           adjust_lr_fn=cfg.adjust_lr_fn,
                           bucket_cap_mb=cfg.bucket.bucket_cap_mb if cfg.bucket.strategy == "size" else None)
    muon._tt_topology = "muon"
    adam_lr = cfg.adamw_lr if cfg.adamw_lr is not None else (lr if lr is not None else 1e-3)
    plan = OptimizerClassPlan(torch.optim.AdamW, lr=adam_lr, weight_decay=wd, betas=cfg.adamw_betas, eps=cfg.adamw_eps)
    sub = plan.resolve((n, p) for n, p, _ in rest)
    adam = backend.prepare_optimizer(_ParamView(rest), sub) if sub.groups else None
    opts, names = [muon], ["muon"]
    if adam is not None:
        if isinstance(adam, OptimizersContainer):
            opts += list(adam.optimizers)
            names += [f"adamw_{n}" for n in adam.names]
        else:
            opts.append(adam)
            names.append("adamw")
    return OptimizersContainer(opts, names)


class _ParamView(nn.Module):
    """Presents a subset of parameters as a module so the backend can validate an optimizer plan against it."""

    def __init__(self, triples):
        super().__init__()
        self._items = [(n, p) for n, p, _ in triples]

    def named_parameters(self, *a, **k):
        return iter(self._items)

    def parameters(self, *a, **k):
        return iter(p for _, p in self._items)
