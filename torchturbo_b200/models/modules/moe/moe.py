"""Dropless top-k mixture of experts with expert parallelism.

Pipeline of one layer (behavioural contract: models/modules/moe/{router,token_dispatcher,experts,moe_layer}.py
of the reference):

    router (gating GEMM -> score fn -> top-k -> aux / z losses, statistics)
      -> dispatch   local: pack rows by (expert, token)
                    EP   : counts exchange, all-to-all-v of tokens and probabilities, regroup by local expert
      -> experts    grouped fc1 -> SwiGLU * prob -> grouped fc2     (probabilities applied after the
                    activation, before fc2)
      -> combine    inverse exchange and k-way sum back to token order

Expert weights keep the fused storage layout `weight1 [E_local*H, 2F]` (per expert `[gate_proj^T | up_proj^T]`)
and `weight2 [E_local*F, H]` (`down_proj^T`), so FSDP can shard dim 0 over the expert-data-parallel mesh
and checkpoints stay interchangeable.

Two token-dispatch transports exist for EP > 1: `nccl` (torch.distributed all-to-all-v: host needs the
split sizes, so one device-to-host read per layer) and `p2p` (CUDA kernels that exchange counts and write
rows straight into the owning rank's expert-major buffer over NVLink: no host read, see
`torchturbo_b200.comm.ep_p2p`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ....ops import MoEPermutation, ops
from ....utils.recompute import in_recompute
from ..comm import all_gather_tensor, all_reduce_sum_autograd, all_to_all


# --------------------------------------------------------------------------------------------------
# configuration
# --------------------------------------------------------------------------------------------------
@dataclass
class MoELayerConfig:
    hidden_size: int = 0
    moe_ffn_hidden_size: int = 0
    num_moe_experts: int = 0
    moe_router_topk: int = 2
    expert_model_parallel_size: int = 1
    params_dtype: torch.dtype = torch.float32
    init_method_std: float = 0.02
    moe_shared_expert_intermediate_size: Optional[int] = None
    moe_shared_expert_gate: bool = False          # sigmoid(x @ w) scales the shared expert's output (Qwen MoE)
    moe_aux_loss_coeff: float = 0.0
    moe_z_loss_coeff: float = 0.0
    moe_router_num_groups: Optional[int] = None
    moe_router_group_topk: Optional[int] = None
    moe_router_pre_softmax: bool = False
    moe_router_topk_scaling_factor: Optional[float] = None
    moe_router_score_function: str = "softmax"   # softmax | sigmoid | sqrtsoftplus
    moe_swiglu_limit: Optional[float] = None      # clamp gate to <= limit and up to [-limit, limit] (0 / None = off)
    moe_router_dtype: Optional[str] = None        # None | fp32 | fp64
    moe_router_enable_expert_bias: bool = False
    moe_token_dispatcher_type: str = "alltoall"
    moe_token_dispatcher_transport: str = "auto"  # auto | nccl | p2p
    moe_apply_probs_on_input: bool = False
    num_hash_layers: int = 0
    vocab_size: int = 0

    def __post_init__(self):
        if (self.moe_router_enable_expert_bias and self.moe_router_score_function == "softmax"
                and not self.moe_router_pre_softmax):
            raise ValueError("softmax routing with an expert bias needs moe_router_pre_softmax=True "
                             "(a softmax over the selected logits would ignore the bias)")
        if self.moe_apply_probs_on_input and self.moe_router_topk != 1:
            raise ValueError("moe_apply_probs_on_input is only defined for top-1 routing")

    @property
    def score_fn(self) -> str:
        if self.moe_router_score_function in ("sigmoid", "sqrtsoftplus"):
            return "sigmoid"
        return "softmax_pre" if self.moe_router_pre_softmax else "softmax_post"


@dataclass
class MoERuntimeInputs:
    """Per-step inputs shared by every MoE layer: `padding_mask` ([1, T_local] bool, True = padding) keeps
    pad tokens out of the load-balance statistics; `aux_loss_scale` is 1/gradient-accumulation;
    `accumulate_tokens_per_expert=False` during activation-checkpoint recomputation so counters used by
    expert-bias updates are not incremented twice."""

    padding_mask: torch.Tensor | None = None
    aux_loss_scale: float = 1.0
    accumulate_tokens_per_expert: bool = True


# --------------------------------------------------------------------------------------------------
# loss helpers
# --------------------------------------------------------------------------------------------------
def _fused_aux_usable(stats) -> bool:
    s, c = stats.get("score_sum"), stats.get("aux_counts")
    if s is None or c is None or not (s.is_cuda and s.dtype == torch.float32 and c.dtype == torch.int32):
        return False
    from .... import kernels as K

    return K.available()


class _FusedAuxLoss(torch.autograd.Function):
    """aux = E * coeff * sum_e score_sum[e] * cnt[e] / (k * n^2) with n = max(sum cnt / k, 1); gradient flows to
    `score_sum` only (the counts are integers)."""

    @staticmethod
    def forward(ctx, score_sum, counts, k, scale_num, coeff):
        from .... import kernels as K

        out, coef = K.aux_loss(score_sum.contiguous(), counts.contiguous(), int(k), scale_num, coeff)
        ctx.save_for_backward(coef)
        return out[0], out[1]

    @staticmethod
    def backward(ctx, g, _g_unscaled):
        (coef,) = ctx.saved_tensors
        return coef * g, None, None, None, None
class MoEAuxLossAutoScaler(torch.autograd.Function):
    """Identity on `output` that makes `aux_loss` part of the graph: backward feeds `loss_scale` into the
    aux loss so it trains the router without changing the reported LM loss."""

    loss_scale: float = 1.0

    @staticmethod
    def forward(ctx, output, aux_loss):
        ctx.save_for_backward(aux_loss)
        return output

    @staticmethod
    def backward(ctx, g):
        (aux,) = ctx.saved_tensors
        return g, torch.full_like(aux, MoEAuxLossAutoScaler.loss_scale)

    @staticmethod
    def set_loss_scale(scale: float) -> None:
        MoEAuxLossAutoScaler.loss_scale = float(scale)


def z_loss_func(lse: torch.Tensor, coeff: float, valid: torch.Tensor | None = None) -> torch.Tensor:
    """`coeff * mean(logsumexp(logits)^2)` over valid tokens."""
    sq = lse.float().pow(2)
    if valid is None:
        return sq.mean() * coeff
    n = valid.sum().clamp(min=1)
    return (sq * valid).sum() / n * coeff


# --------------------------------------------------------------------------------------------------
# router
# --------------------------------------------------------------------------------------------------
class TopKRouter(nn.Module):
    def __init__(self, config: MoELayerConfig, sp_group=None, layer_number: int | None = None):
        super().__init__()
        self.config = config
        self.sp_group = sp_group
        self.layer_number = layer_number
        self.weight = nn.Parameter(torch.empty(config.num_moe_experts, config.hidden_size, dtype=config.params_dtype))
        nn.init.normal_(self.weight, std=config.init_method_std)
        if config.moe_router_enable_expert_bias:
            self.register_buffer("expert_bias", torch.zeros(config.num_moe_experts, dtype=torch.float32))
            self.register_buffer("local_tokens_per_expert", torch.zeros(config.num_moe_experts, dtype=torch.float32),
                                 persistent=False)
        else:
            self.expert_bias = None
        self.tid2eid = None  # token-id hash routing table [vocab, k] for hash layers
        self._metrics: dict[str, list[torch.Tensor]] = {}

    # -- metrics protocol (consumed by MetricTracker) -------------------------------------------------
    def _record(self, name: str, value: torch.Tensor) -> None:
        if in_recompute():      # the replay of a checkpointed layer reports nothing a second time
            return
        self._metrics.setdefault(name, []).append(value.detach().float())

    def pop_metrics(self) -> dict[str, torch.Tensor]:
        out = {k: torch.stack(v).mean() for k, v in self._metrics.items() if v}
        self._metrics = {}
        return out

    def gating(self, x: torch.Tensor) -> torch.Tensor:
        """Router logits in fp32 (bf16 operands accumulate in fp32 on the tensor cores; an explicit
        `moe_router_dtype` upcasts the operands too)."""
        rd = self.config.moe_router_dtype
        if rd in ("fp32", "fp64"):
            dt = torch.float32 if rd == "fp32" else torch.float64
            return F.linear(x.to(dt), self.weight.to(dt)).float()
        return ops.router_gating(x, self.weight)

    def forward(self, x: torch.Tensor, input_ids: torch.Tensor | None = None, runtime: MoERuntimeInputs | None = None):
        """x: [T, H] -> (topk_idx int [T, k], topk_prob fp32 [T, k], logits fp32 [T, E])."""
        cfg = self.config
        runtime = runtime or MoERuntimeInputs()
        logits = self.gating(x)
        T, E = logits.shape
        valid = None
        if runtime.padding_mask is not None:
            valid = ~runtime.padding_mask.reshape(-1).bool()
        scaling = cfg.moe_router_topk_scaling_factor or 1.0
        if self.tid2eid is not None and input_ids is not None:
            idx, prob, stats = self._hash_routing(logits, input_ids, scaling, valid)
        elif cfg.moe_router_num_groups:
            idx, prob, stats = self._group_limited(logits, scaling, valid)
        elif cfg.moe_router_score_function == "sqrtsoftplus":
            idx, prob, stats = self._eager_topk(logits, scaling, valid)
        else:
            idx, prob, stats = ops.router_topk(logits, cfg.moe_router_topk, cfg.score_fn, expert_bias=self.expert_bias,
                                               scaling=scaling, valid_mask=valid)
        sp = dist.get_world_size(self.sp_group) if (self.sp_group is not None and dist.is_initialized()) else 1
        if cfg.moe_z_loss_coeff > 0 and self.training:
            n_local = valid.sum() if valid is not None else torch.tensor(T, device=x.device)
            n_global = n_local.clone().float()
            if sp > 1:
                dist.all_reduce(n_global, group=self.sp_group)
            z = z_loss_func(stats["lse"], cfg.moe_z_loss_coeff, valid) * (sp * n_local.float() / n_global.clamp(min=1))
            prob = MoEAuxLossAutoScaler.apply(prob, z * runtime.aux_loss_scale)
            self._record("z_loss", z / cfg.moe_z_loss_coeff)
            self._record("z_loss_scaled", z)
        if cfg.moe_aux_loss_coeff > 0 and self.training and sp == 1 and _fused_aux_usable(stats):
            # one kernel for the loss and its gradient coefficients instead of a dozen small launches each way
            aux, aux_unscaled = _FusedAuxLoss.apply(stats["score_sum"], stats["aux_counts"], cfg.moe_router_topk,
                                                    float(E * cfg.moe_aux_loss_coeff), float(cfg.moe_aux_loss_coeff))
            prob = MoEAuxLossAutoScaler.apply(prob, aux * runtime.aux_loss_scale)
            self._record("aux_loss", aux_unscaled)
            self._record("aux_loss_scaled", aux)
        elif cfg.moe_aux_loss_coeff > 0 and self.training:
            tokens_per_expert = stats["aux_counts"].float()
            if sp > 1:
                tokens_per_expert = tokens_per_expert.clone()
                dist.all_reduce(tokens_per_expert, group=self.sp_group)
            k = cfg.moe_router_topk
            n_tokens = (tokens_per_expert.sum() / k).clamp(min=1.0)
            aux = (stats["score_sum"] * tokens_per_expert).sum() * (E * sp * cfg.moe_aux_loss_coeff) / (k * n_tokens * n_tokens)
            prob = MoEAuxLossAutoScaler.apply(prob, aux * runtime.aux_loss_scale)
            self._record("aux_loss", aux / cfg.moe_aux_loss_coeff)
            self._record("aux_loss_scaled", aux)
        if self.expert_bias is not None and self.training and runtime.accumulate_tokens_per_expert and not in_recompute():
            with torch.no_grad():
                self.local_tokens_per_expert += stats["counts"].float()
        # histogram of `idx` over the experts, as the routing kernel produced it: dispatchers reuse it
        self.last_counts = stats.get("counts") if isinstance(stats, dict) else None
        return idx, prob, logits

    # -- rarely used routing variants stay in torch ---------------------------------------------------
    def _scores(self, lg: torch.Tensor) -> torch.Tensor:
        fn = self.config.moe_router_score_function
        if fn == "sigmoid":
            return torch.sigmoid(lg)
        if fn == "sqrtsoftplus":
            return torch.sqrt(F.softplus(lg))
        return torch.softmax(lg, -1)

    def _eager_topk(self, logits, scaling, valid):
        """Score functions the fused router kernel does not cover (`sqrtsoftplus`): scores, bias-corrected selection,
        weights normalised over the selected experts."""
        from ....ops.providers.native import router_topk_ref

        cfg = self.config
        lg = logits.float()
        scores = self._scores(lg)
        sel = scores + self.expert_bias if self.expert_bias is not None else scores
        idx = sel.topk(cfg.moe_router_topk, dim=-1).indices
        prob = scores.gather(1, idx)
        if cfg.moe_router_topk > 1:
            prob = prob / (prob.sum(-1, keepdim=True) + 1e-20)
        _, _, stats = router_topk_ref(lg, cfg.moe_router_topk, "sigmoid", None, 1.0, valid)
        stats["counts"] = torch.bincount(idx.reshape(-1), minlength=lg.shape[1])
        return idx, prob * scaling, stats

    def _group_limited(self, logits, scaling, valid):
        """Group-limited top-k: keep the best `group_topk` groups (score of a group = sum of its top
        `k / group_topk` experts), then top-k inside them (models/modules/moe/utils.py:30-77 of the reference)."""
        cfg = self.config
        from ....ops.providers.native import router_topk_ref

        lg = logits.float()
        T, E = lg.shape
        G, gk, k = cfg.moe_router_num_groups, cfg.moe_router_group_topk, cfg.moe_router_topk
        scores = self._scores(lg)
        sel = scores + self.expert_bias if self.expert_bias is not None else scores
        group_scores = sel.view(T, G, E // G).topk(max(k // gk, 1), dim=-1).values.sum(-1)
        gmask = torch.zeros_like(group_scores).scatter_(1, group_scores.topk(gk, dim=-1).indices, 1.0)
        emask = gmask[:, :, None].expand(T, G, E // G).reshape(T, E).bool()
        idx = sel.masked_fill(~emask, float("-inf")).topk(k, dim=-1).indices
        prob = scores.gather(1, idx)
        if cfg.moe_router_score_function != "softmax" and k > 1:
            prob = prob / (prob.sum(-1, keepdim=True) + 1e-20)
        _, _, stats = router_topk_ref(lg, k, cfg.score_fn, None, 1.0, valid)
        stats["counts"] = torch.bincount(idx.reshape(-1), minlength=E)
        return idx, prob * scaling, stats

    def _hash_routing(self, logits, input_ids, scaling, valid):
        from ....ops.providers.native import router_topk_ref

        cfg = self.config
        idx = self.tid2eid[input_ids.reshape(-1)].long()
        lg = logits.float()
        scores = self._scores(lg)
        prob = scores.gather(1, idx)
        if cfg.moe_router_topk > 1:
            prob = prob / (prob.sum(-1, keepdim=True) + 1e-20)
        _, _, stats = router_topk_ref(lg, cfg.moe_router_topk, cfg.score_fn, None, 1.0, valid)
        stats["counts"] = torch.bincount(idx.reshape(-1), minlength=lg.shape[1])
        return idx, prob * scaling, stats


# --------------------------------------------------------------------------------------------------
# experts
# --------------------------------------------------------------------------------------------------
class GroupedMLP(nn.Module):
    """`num_local_experts` SwiGLU experts in two fused tensors (see module docstring for the layout)."""

    def __init__(self, config: MoELayerConfig, num_local_experts: int):
        super().__init__()
        self.config = config
        self.num_local_experts = num_local_experts
        H, Fh = config.hidden_size, config.moe_ffn_hidden_size
        self.weight1 = nn.Parameter(torch.empty(num_local_experts * H, 2 * Fh, dtype=config.params_dtype))
        self.weight2 = nn.Parameter(torch.empty(num_local_experts * Fh, H, dtype=config.params_dtype))
        nn.init.normal_(self.weight1, std=config.init_method_std)
        nn.init.normal_(self.weight2, std=config.init_method_std)

    def views(self):
        E, H, Fh = self.num_local_experts, self.config.hidden_size, self.config.moe_ffn_hidden_size
        return self.weight1.view(E, H, 2 * Fh), self.weight2.view(E, Fh, H)

    def forward(self, perm: MoEPermutation, tokens_per_expert=None) -> torch.Tensor:
        w1, w2 = self.views()
        if perm.tokens.shape[0] == 0:
            # keep the weights in the autograd graph on ranks that received no tokens
            return perm.tokens.new_zeros(0, w2.shape[-1]) + 0.0 * (w1.sum() + w2.sum())
        if self.config.moe_swiglu_limit:
            return self._forward_clamped(perm, w1, w2, float(self.config.moe_swiglu_limit), tokens_per_expert)
        return ops.moe_experts(perm, w1, w2, tokens_per_expert)

    @staticmethod
    def _forward_clamped(perm: MoEPermutation, w1, w2, limit: float, tokens_per_expert=None) -> torch.Tensor:
        """Clamped SwiGLU (gate <= limit, |up| <= limit).  The fused expert kernel has no clamp, so this variant runs
        per expert in torch and reads the segment table on the host."""
        x = perm.tokens
        counts = (perm.counts if perm.counts is not None else tokens_per_expert).tolist()
        starts = perm.seg_start.tolist() if perm.seg_start is not None else None
        out, pos = [], 0
        pieces = x.new_zeros(x.shape[0], w2.shape[-1])
        segs = []
        for e, n in enumerate(counts):
            a = starts[e] if starts is not None else pos
            pos += n
            if n:
                h = ops.gated_activation(x[a:a + n] @ w1[e], limit=limit,
                                         probs=perm.probs[a:a + n] if perm.probs is not None else None)
                segs.append((a, n, h @ w2[e]))
        if not segs:
            return pieces + 0.0 * (w1.sum() + w2.sum())
        idx = torch.cat([torch.arange(a, a + n, device=x.device) for a, n, _ in segs])
        return pieces.index_copy(0, idx, torch.cat([y for _, _, y in segs]).to(pieces.dtype))

    def get_muon_parameter_specs(self):
        """Each expert matrix is an independent Muon matrix inside the fused storage."""
        E, H, Fh = self.num_local_experts, self.config.hidden_size, self.config.moe_ffn_hidden_size
        return {"weight1": dict(batch=E, rows=H, cols=2 * Fh, split_cols=(Fh, Fh)), "weight2": dict(batch=E, rows=Fh, cols=H)}


# --------------------------------------------------------------------------------------------------
# token dispatcher (EP all-to-all-v over torch.distributed)
# --------------------------------------------------------------------------------------------------
class MoEAlltoAllTokenDispatcher:
    """Expert-parallel exchange.  Experts are contiguous per rank: rank r owns `[r*E_local, (r+1)*E_local)`."""

    def __init__(self, config: MoELayerConfig, ep_group, num_local_experts: int):
        self.config = config
        self.ep_group = ep_group
        self.ep_size = dist.get_world_size(ep_group) if (ep_group is not None and dist.is_initialized()) else 1
        self.ep_rank = dist.get_rank(ep_group) if self.ep_size > 1 else 0
        self.num_local_experts = num_local_experts
        self.num_experts = config.num_moe_experts

    def dispatch(self, x: torch.Tensor, idx: torch.Tensor, prob: torch.Tensor):
        """Returns (perm for the local experts, tokens_per_local_expert, state for `combine`)."""
        E = self.num_experts
        if self.ep_size == 1:
            perm = ops.moe_permutation(x, idx, probs=prob, num_experts=E)
            tpe = perm.counts if perm.padded else torch.bincount(idx.reshape(-1).long(), minlength=E)
            return perm, tpe, ("local", perm, x.shape[0])
        # ---- EP: dense (unpadded) send layout ordered by (expert, token)
        send = ops.moe_permutation(x, idx, probs=prob, num_experts=E, impl="torch_moe_permutation")
        counts = torch.bincount(idx.reshape(-1).long(), minlength=E)
        all_counts = all_gather_tensor(counts.view(1, E), self.ep_group)              # [ep, E]
        host = all_counts.cpu()                                                        # the one host read
        El, r = self.num_local_experts, self.ep_rank
        in_splits = host[r].view(self.ep_size, El).sum(1).tolist()
        mine = host[:, r * El:(r + 1) * El]                                            # [src, local expert]
        out_splits = mine.sum(1).tolist()
        recv = all_to_all(self.ep_group, send.tokens, out_splits, in_splits)
        recv_prob = all_to_all(self.ep_group, send.probs.float().view(-1, 1), out_splits, in_splits).view(-1)
        # received rows are (source rank, local expert, token); regroup by local expert with one more packing
        row_expert = torch.repeat_interleave(torch.arange(El).repeat(self.ep_size), mine.reshape(-1)).to(x.device)
        local = ops.moe_permutation(recv, row_expert.view(-1, 1), probs=recv_prob.view(-1, 1), num_experts=El)
        tpe = mine.sum(0).to(x.device)
        return local, tpe, ("ep", send, local, in_splits, out_splits, x.shape[0])

    def combine(self, y: torch.Tensor, state) -> torch.Tensor:
        if state[0] == "local":
            _, perm, T = state
            return ops.moe_unpermutation(y, perm)
        _, send, local, in_splits, out_splits, T = state
        back = ops.moe_unpermutation(y, local)                       # received order
        ret = all_to_all(self.ep_group, back, in_splits, out_splits)  # inverse exchange
        return ops.moe_unpermutation(ret, send)


# --------------------------------------------------------------------------------------------------
# layer
# --------------------------------------------------------------------------------------------------
class SharedExpertMLP(nn.Module):
    def __init__(self, hidden: int, inter: int, dtype, gated_output: bool = False, std: float = 0.02):
        super().__init__()
        self.gate_up_proj = nn.Linear(hidden, 2 * inter, bias=False, dtype=dtype)
        self.down_proj = nn.Linear(inter, hidden, bias=False, dtype=dtype)
        self.gate = nn.Linear(hidden, 1, bias=False, dtype=dtype) if gated_output else None
        for m in (self.gate_up_proj, self.down_proj):
            nn.init.normal_(m.weight, std=std)

    def forward(self, x):
        y = ops.linear(ops.linear_swiglu(x, self.gate_up_proj.weight), self.down_proj.weight)
        if self.gate is not None:
            y = torch.sigmoid(F.linear(x, self.gate.weight)) * y
        return y


class BaseMoELayer(nn.Module):
    def __init__(self, config: MoELayerConfig, ep_group=None, sp_group=None):
        super().__init__()
        self.config = config
        self.ep_group = ep_group
        self.sp_group = sp_group
        self.ep_size = dist.get_world_size(ep_group) if (ep_group is not None and dist.is_initialized()) else 1
        if config.num_moe_experts % self.ep_size:
            raise ValueError(f"{config.num_moe_experts} experts are not divisible by ep_size={self.ep_size}")
        self.num_local_experts = config.num_moe_experts // self.ep_size
        ep_rank = dist.get_rank(ep_group) if self.ep_size > 1 else 0
        self.local_expert_indices = list(range(ep_rank * self.num_local_experts, (ep_rank + 1) * self.num_local_experts))
        self._runtime_inputs = MoERuntimeInputs()

    def set_runtime_inputs(self, runtime: MoERuntimeInputs) -> None:
        self._runtime_inputs = runtime


class MoELayer(BaseMoELayer):
    def __init__(self, config: MoELayerConfig, ep_group=None, sp_group=None, layer_number: int | None = None):
        super().__init__(config, ep_group, sp_group)
        self.router = TopKRouter(config, sp_group, layer_number)
        self.experts = GroupedMLP(config, self.num_local_experts)
        self.token_dispatcher = self._build_dispatcher()
        si = config.moe_shared_expert_intermediate_size
        self.shared_experts = SharedExpertMLP(config.hidden_size, si, config.params_dtype, config.moe_shared_expert_gate,
                                              config.init_method_std) if si else None

    def _build_dispatcher(self):
        transport = self.config.moe_token_dispatcher_transport
        if self.ep_size > 1 and transport in ("auto", "p2p"):
            try:
                from ....comm.ep_p2p import P2PTokenDispatcher

                if P2PTokenDispatcher.usable(self.ep_group):
                    return P2PTokenDispatcher(self.config, self.ep_group, self.num_local_experts)
            except Exception:
                if transport == "p2p":
                    raise
        return MoEAlltoAllTokenDispatcher(self.config, self.ep_group, self.num_local_experts)

    def forward(self, hidden_states: torch.Tensor, input_ids: torch.Tensor | None = None):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1])
        idx, prob, logits = self.router(x, input_ids, self._runtime_inputs)
        xin = x
        if self.config.moe_apply_probs_on_input:
            xin = (x.float() * prob.view(-1, 1)).to(x.dtype)
            prob = torch.ones_like(prob)
        fused = getattr(self.token_dispatcher, "fused_experts", None)
        if fused is not None:
            w1, w2 = self.experts.views()
            if self.token_dispatcher.fused_usable(xin, w1, w2):
                # exchange inside the grouped GEMMs (peer-memory push prologue / scatter epilogue)
                out = fused(xin, idx, prob, w1, w2, counts=getattr(self.router, "last_counts", None)).to(x.dtype)
                if self.shared_experts is not None:
                    out = out + self.shared_experts(x)
                return out.view(shape), logits
        if getattr(self.token_dispatcher, "accepts_counts", False):
            perm, tpe, state = self.token_dispatcher.dispatch(xin, idx, prob, counts=getattr(self.router, "last_counts", None))
        else:
            perm, tpe, state = self.token_dispatcher.dispatch(xin, idx, prob)
        y = self.experts(perm, tpe)
        out = self.token_dispatcher.combine(y, state).to(x.dtype)
        if self.shared_experts is not None:
            out = out + self.shared_experts(x)
        return out.view(shape), logits
