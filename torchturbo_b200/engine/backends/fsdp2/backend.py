"""FSDP2 backend: data-parallel sharding (ZeRO-3 style) + expert-parallel mesh + Ulysses SP groups.

What it does, in the order `prepare_model` runs (phases as in engine/backends/fsdp2/backend.py:438-540 of
the reference):
  1. meshes and groups: 1-D world mesh `("dp",)`, 2-D mesh `(W/ep, ep)` named `("edp", "ep")`, SP groups of
     consecutive ranks and DP groups of strided ranks;
  2. module replacement from the plan (`replace_module`), PEFT, SP input-slicing patch;
  3. activation checkpointing per planned module;
  4. sharding: explicit plan units, every `ModuleList` child, the input-embedding unit, a resident tail unit
     (final norm + output embedding) and the root.

B200-first difference: a unit whose mesh has a single rank (everything on one GPU; experts when `ep` equals
the world size) is *not* wrapped by `fully_shard`.  Such a unit keeps bf16 parameters whose fp32 master copy
lives in the optimizer (the fused AdamW kernel writes both), which removes the per-step all-gather /
cast / reduce-scatter copies that a one-rank FSDP unit would still perform.  Units with more than one rank
use `torch.distributed.fsdp.fully_shard` with bf16 parameters, fp32 reduction and fp32 sharded masters.
"""
from __future__ import annotations

import math

import contextlib
import os
import functools
from typing import Any

import torch
import torch.distributed as dist
import torch.nn as nn

from ....logging import get_logger
from ....models.modules.attention.ulysses import patch_forward_for_sp_input_slicing, ulysses_pad_inputs
from ....models.modules.loss import chunk_loss, logits_loss, prepare_loss_labels
from ....models.modules.moe import BaseMoELayer, MoEAuxLossAutoScaler
from ....parallel import FSDPParallelPlan, FSDPPlanSpec
from ....utils.fqn import match_fqn
from ...backend_registry import register_backend
from ...config import CPUOffloadMode, EngineConfig, MixedPrecisionPolicy
from ...distributed import assert_finite, init_process_group_if_needed
from ..base import BaseBackend

logger = get_logger(__name__)

from ....utils.recompute import in_recompute, recompute_ctx as _recompute_ctx  # noqa: E402,F401  (re-exported)


def _reentrant_checkpoint(fn, args: tuple, kwargs: dict):
    """`torch.utils.checkpoint` in reentrant mode around `fn(*args, **kwargs)` with the three things that mode does
    not do by itself (engine/backends/fsdp2/backend.py:875-990 of the reference has the same glue):
      * keyword arguments: the reentrant implementation only takes positional ones, so they are bound beforehand;
      * recompute marking: the replay runs inside the checkpoint's backward with gradients enabled, the original pass
        with gradients disabled; the replay is wrapped in the recompute context so that router statistics and
        expert-bias token counts are not accumulated a second time;
      * gradient anchor: when no tensor argument requires a gradient (frozen embeddings in front of the first layer,
        LoRA), the reentrant implementation would skip the backward of the whole segment; a scalar that requires a
        gradient rides along as an extra argument."""
    from torch.utils.checkpoint import checkpoint

    def body(_anchor, *a):
        if torch.is_grad_enabled():          # the replay inside CheckpointFunction.backward
            with _recompute_ctx():
                return fn(*a, **kwargs)
        return fn(*a, **kwargs)

    tensors = [a for a in args if isinstance(a, torch.Tensor)]
    dev = tensors[0].device if tensors else None
    anchor = torch.zeros((), device=dev, requires_grad=True) if not any(t.requires_grad for t in tensors) else None
    return checkpoint(body, anchor, *args, use_reentrant=True)


def confidence_entropy_sum(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
    """(sum of softmax entropies over rows whose argmax equals the label, number of such rows): both summable, so
    they can be reduced across ranks before the division."""
    valid = labels != ignore_index
    correct = (logits.argmax(-1) == labels) & valid
    n = correct.sum()
    lp = torch.log_softmax(logits.float(), dim=-1)
    ent = -(lp.exp() * lp).sum(-1)
    return (ent * correct.to(ent.dtype)).sum(), n



class _FlatGradExchange:
    """Health view of the symmetric flat gradient buffer (status word of its flag waits), so that the engine's peer
    status checks cover it like the other peer-memory workspaces."""

    def __init__(self, parts: dict, rank: int):
        self.status, self.rank = parts["status"], rank

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"gradient all-reduce of the replicated layers timed out on rank {self.rank} (code {code:#x})")


class _HostInput:
    """A host tensor in transit through FSDP's input mover (which only moves what it recognises as a tensor)."""

    __slots__ = ("tensor",)

    def __init__(self, tensor: torch.Tensor):
        self.tensor = tensor


@register_backend("fsdp2")
class FSDP2Backend(BaseBackend):
    def __init__(self, config: EngineConfig, runtime) -> None:
        super().__init__(config, runtime)
        self.fsdp_config = config.backend_config
        offload = self.fsdp_config.cpu_offload
        init_process_group_if_needed(runtime, with_cpu_backend=bool(offload.enabled))
        self.rank, self.world_size = dist.get_rank(), dist.get_world_size()
        self.device = runtime.device
        self.world_mesh = None
        self.ep_mesh = None
        self.sp_size = self.ep_size = 1
        self.sp_group = self.dp_group = self.ep_group = self.edp_group = None
        self.sp_rank = 0
        self.dp_rank, self.dp_size = self.rank, self.world_size
        self.gradient_scaling_factor = 1.0
        self.local_units: list[nn.Module] = []
        self.replicated_units: list[nn.Module] = []      # decoder layers kept replicated (`replicate_layers`)
        self._rep_flat: torch.Tensor | None = None       # flat fp32 gradient buffer of their parameters
        self._rep_params: list[nn.Parameter] = []
        self._rep_synced = False
        self.fsdp_units: list[nn.Module] = []
        self.expert_modules: list[nn.Module] = []
        self.no_shard_names: list[str] = []
        self._model_ref = None
        self._plan: FSDPParallelPlan | None = None

    @property
    def no_shard_params(self) -> list[nn.Parameter]:
        if self._model_ref is None or not self.no_shard_names:
            return []
        table = dict(self._model_ref.named_parameters())
        return [table[n] for n in self.no_shard_names if n in table]

    @property
    def expert_param_ids(self) -> set[int]:
        """ids of the parameters owned by expert units.  Recomputed from the modules because materialisation
        (`to_empty`) and dtype changes replace parameter objects."""
        return {id(p) for m in self.expert_modules for p in m.parameters()}

    # ------------------------------------------------------------------------------------------
    # meshes and groups
    # ------------------------------------------------------------------------------------------
    def _init_mesh(self, plan: FSDPParallelPlan) -> None:
        from torch.distributed.device_mesh import init_device_mesh

        W = self.world_size
        self.sp_size, self.ep_size = int(plan.sp_size or 1), int(plan.ep_size or 1)
        if W % self.sp_size or W % self.ep_size:
            raise ValueError(f"world size {W} must be divisible by sp_size={self.sp_size} and ep_size={self.ep_size}")
        dev = self.runtime.turbo_device.value
        self.world_mesh = init_device_mesh(dev, (W,), mesh_dim_names=("dp",))
        self.ep_mesh = init_device_mesh(dev, (W // self.ep_size, self.ep_size), mesh_dim_names=("edp", "ep"))
        self.ep_group = self.ep_mesh.get_group("ep")
        self.edp_group = self.ep_mesh.get_group("edp")
        self.ep_rank = dist.get_rank(self.ep_group)
        self._create_sp_group()
        self._create_dp_group()

    def _create_sp_group(self) -> None:
        """SP groups are runs of `sp_size` consecutive ranks."""
        self.sp_group, self.sp_rank = None, 0
        if self.sp_size <= 1:
            return
        for start in range(0, self.world_size, self.sp_size):
            ranks = list(range(start, start + self.sp_size))
            g = dist.new_group(ranks)
            if self.rank in ranks:
                self.sp_group, self.sp_rank = g, self.rank - start

    def _create_dp_group(self) -> None:
        """DP groups take every `sp_size`-th rank: ranks with the same position inside their SP group."""
        self.dp_size = self.world_size // self.sp_size
        self.dp_rank = self.rank // self.sp_size
        self.dp_group = None
        if self.sp_size <= 1:
            self.dp_group = dist.group.WORLD
            return
        for off in range(self.sp_size):
            ranks = list(range(off, self.world_size, self.sp_size))
            g = dist.new_group(ranks)
            if self.rank in ranks:
                self.dp_group = g

    def get_dp_info(self) -> dict[str, Any]:
        return {"dp_group": self.dp_group, "dp_size": self.dp_size, "dp_rank": self.dp_rank}

    def get_ep_info(self) -> dict[str, Any]:
        return {"ep_group": self.ep_group, "ep_size": self.ep_size, "ep_rank": getattr(self, "ep_rank", 0),
                "edp_group": self.edp_group, "ep_mesh": self.ep_mesh}

    def get_sp_info(self) -> dict[str, Any]:
        return {"sp_group": self.sp_group, "sp_size": self.sp_size, "sp_rank": self.sp_rank}

    # ------------------------------------------------------------------------------------------
    # prepare_model
    # ------------------------------------------------------------------------------------------
    def prepare_model(self, model: nn.Module, parallel_plan: FSDPParallelPlan, peft_config: Any = None) -> nn.Module:
        self._plan = parallel_plan
        self._init_mesh(parallel_plan)
        self._replace_modules(model, parallel_plan)
        if peft_config is not None:
            from ...peft import apply_peft

            model = apply_peft(model, peft_config)
        if hasattr(model, "get_sequence_parallel_input_slicing_spec"):
            patch_forward_for_sp_input_slicing(model.get_sequence_parallel_input_slicing_spec(), self.sp_group,
                                               self.sp_size, self.sp_rank)
        compiled = self._compile_parallel_plan(model, parallel_plan)
        self._apply_activation_checkpointing(model, compiled)
        self._shard_model(model, compiled)
        self._setup_prefetch(model)
        self._install_peer_collectives()
        self._register_vision_balance(model, compiled)
        self.gradient_scaling_factor = 1.0 / self.ep_size
        return model

    def _replace_modules(self, model: nn.Module, plan: FSDPParallelPlan) -> None:
        """`spec.replace_module(original, hf_config=..., sp_info=..., ep_info=..., engine_config=..., **kwargs)`
        for every module whose FQN matches a plan entry carrying a replacement."""
        targets = []
        for fqn, mod in model.named_modules():
            for pattern, spec in plan.plan.items():
                if spec.replace_module is not None and match_fqn(pattern, fqn):
                    targets.append((fqn, mod, spec))
                    break
        for fqn, mod, spec in targets:
            parent_name, _, child = fqn.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            dev = next((p.device for p in mod.parameters()), torch.device("cpu"))
            with torch.device(dev):
                new = spec.replace_module(mod, hf_config=model.config, sp_info=self.get_sp_info(),
                                          ep_info=self.get_ep_info(), engine_config=self.config,
                                          **(spec.module_kwargs or {}))
            setattr(parent, child, new)

    def _compile_parallel_plan(self, model: nn.Module, plan: FSDPParallelPlan) -> dict[str, FSDPPlanSpec]:
        """module FQN -> first matching spec (patterns are written against the model's own names)."""
        compiled: dict[str, FSDPPlanSpec] = {}
        for fqn, _ in model.named_modules():
            spec = plan.match(fqn)
            if spec is not None:
                compiled[fqn] = spec
        return compiled

    # ------------------------------------------------------------------------------------------
    # activation checkpointing
    # ------------------------------------------------------------------------------------------
    def _apply_activation_checkpointing(self, model: nn.Module, compiled: dict[str, FSDPPlanSpec]) -> None:
        ac = self.config.activation_checkpointing
        if not ac.enabled:
            return
        from torch.utils.checkpoint import checkpoint

        n = 0
        for fqn, spec in compiled.items():
            if not spec.activation_checkpoint:
                continue
            mod = model.get_submodule(fqn)
            if getattr(mod, "_tt_ac_wrapped", False):
                continue
            orig = mod.forward

            def ac_forward(*args, __orig=orig, **kwargs):
                if not torch.is_grad_enabled():
                    return __orig(*args, **kwargs)
                if ac.use_reentrant:
                    return _reentrant_checkpoint(__orig, args, kwargs)
                return checkpoint(__orig, *args, use_reentrant=False,
                                  context_fn=lambda: (contextlib.nullcontext(), _recompute_ctx()), **kwargs)

            mod.forward = ac_forward
            mod._tt_ac_wrapped = True
            n += 1
        logger.info_rank0("activation checkpointing on %d module(s)", n)

    # ------------------------------------------------------------------------------------------
    # sharding
    # ------------------------------------------------------------------------------------------
    def _mesh_for(self, spec: FSDPPlanSpec | None):
        if spec is not None and spec.placement is not None and spec.placement.mesh_dim in ("edp", 0):
            return self.ep_mesh["edp"], True
        return self.world_mesh, False

    def _fsdp_kwargs(self, mesh, *, is_expert: bool, reshard: bool | None = None) -> dict[str, Any]:
        from torch.distributed.fsdp import CPUOffloadPolicy, MixedPrecisionPolicy as MP

        kw: dict[str, Any] = {"mesh": mesh}
        if self.config.mixed_precision is MixedPrecisionPolicy.BF16:
            kw["mp_policy"] = MP(param_dtype=torch.bfloat16, reduce_dtype=torch.float32,
                                 cast_forward_inputs=not is_expert)
        kw["reshard_after_forward"] = self.fsdp_config.reshard_after_forward if reshard is None else reshard
        off = self.fsdp_config.cpu_offload
        if off.enabled and off.mode is CPUOffloadMode.FULL:
            kw["offload_policy"] = CPUOffloadPolicy(pin_memory=True)
        return kw

    def _make_unit(self, module: nn.Module | list[nn.Module], spec: FSDPPlanSpec | None, *,
                   reshard: bool | None = None) -> None:
        """Make one unit of `module`, or of a list of sibling modules that share one all-gather / reduce-scatter
        (the first module of the list is the unit's handle; the others are marked as members)."""
        group = list(module) if isinstance(module, (list, tuple)) else [module]
        group = [m for m in group if getattr(m, "_tt_unit", None) is None]
        if not group:
            return
        mesh, is_expert = self._mesh_for(spec)
        own = [p for m in group for p in m.parameters()]
        for m in group:
            if is_expert and m not in self.expert_modules:
                self.expert_modules.append(m)
        if mesh.size() > 1:
            from torch.distributed.fsdp import fully_shard

            skip = {id(q) for q in self.no_shard_params}
            for m in group:
                for sub in m.modules():
                    if sub is not m and getattr(sub, "_tt_unit", None) in ("local", "replicated"):
                        skip.update(id(q) for q in sub.parameters())
            ignored = {p for p in own if id(p) in skip}
            kw = self._fsdp_kwargs(mesh, is_expert=is_expert, reshard=reshard)
            if ignored:
                kw["ignored_params"] = ignored
            fully_shard(group if len(group) > 1 else group[0], **kw)
            group[0]._tt_unit, group[0]._tt_group, group[0]._tt_mesh = "fsdp", group, mesh
            for m in group[1:]:
                m._tt_unit, m._tt_group = "fsdp_member", group
            self.fsdp_units.append(group[0])
        else:
            for m in group:
                m._tt_unit = "local"
                self.local_units.append(m)

    def _keep_host_inputs_on_host(self, model: nn.Module) -> None:
        """FSDP's root pre-forward hook moves every tensor argument to the GPU with a blocking copy.  The packed-row
        boundaries (`cu_seq_lens_*`) are host tensors on purpose (tile tables and loop bounds are derived from them
        on the host); moved to the GPU they cost one blocking copy per forward and then one device-to-host read per
        attention layer, which serialises host and device.  A hook in front of FSDP's wraps host tensors in a plain
        object FSDP does not recognise, a hook behind it unwraps them."""
        if getattr(model, "_tt_unit", None) != "fsdp" or getattr(model, "_tt_host_input_hooks", False):
            return

        def box(_m, args, kwargs):
            if not any(isinstance(v, torch.Tensor) and v.device.type == "cpu" for v in list(args) + list(kwargs.values())):
                return None
            wrap = lambda v: _HostInput(v) if isinstance(v, torch.Tensor) and v.device.type == "cpu" else v   # noqa: E731
            return tuple(wrap(a) for a in args), {k: wrap(v) for k, v in kwargs.items()}

        def unbox(_m, args, kwargs):
            if not any(isinstance(v, _HostInput) for v in list(args) + list(kwargs.values())):
                return None
            un = lambda v: v.tensor if isinstance(v, _HostInput) else v   # noqa: E731
            return tuple(un(a) for a in args), {k: un(v) for k, v in kwargs.items()}

        model.register_forward_pre_hook(unbox, with_kwargs=True)                 # after FSDP's (prepended) hook
        model.register_forward_pre_hook(box, prepend=True, with_kwargs=True)     # before it
        model._tt_host_input_hooks = True

    def _unit_param_bytes(self, module: nn.Module) -> int:
        """bf16 bytes one all-gather of `module` as a unit of its own would deliver: parameters that are not
        replicated and not owned by a nested unit."""
        skip = {id(q) for q in self.no_shard_params}
        for sub in module.modules():
            if sub is not module and getattr(sub, "_tt_unit", None) is not None:
                skip.update(id(q) for q in sub.parameters())
        return sum(2 * p.numel() for p in module.parameters() if id(p) not in skip)

    def _group_layers(self, layers: list[nn.Module]) -> list[list[nn.Module]]:
        """Consecutive decoder layers are merged into one FSDP unit until the unit gathers at least
        `unit_min_bytes`: a 30B-A3B layer without its experts is ~38 MB of bf16, far below the size at which the
        host cost of a unit's hooks and the latency of its two collectives stop mattering."""
        want = int(self.fsdp_config.unit_min_bytes)
        if want <= 0 or self.world_mesh.size() <= 1:
            return [[m] for m in layers]
        groups, cur, cur_bytes = [], [], 0
        for m in layers:
            cur.append(m)
            cur_bytes += self._unit_param_bytes(m)
            if cur_bytes >= want:
                groups.append(cur)
                cur, cur_bytes = [], 0
        if cur:
            if groups and cur_bytes < want // 2:
                groups[-1].extend(cur)
            else:
                groups.append(cur)
        return groups

    def _resolve_reshard(self, model: nn.Module, single_rank: list[nn.Module]) -> None:
        """`reshard_after_forward: auto` keeps gathered bf16 parameters until backward has used them whenever all
        FSDP-managed parameters together are a small part of the device memory (no second all-gather per unit)."""
        if self.fsdp_config.reshard_after_forward != "auto":
            return
        resident = False
        if torch.cuda.is_available() and self.world_mesh.size() > 1 and not self.fsdp_config.cpu_offload.enabled:
            local = {id(p) for m in single_rank for p in m.parameters()} | {id(p) for p in self.no_shard_params}
            total = sum(2 * p.numel() for p in model.parameters() if id(p) not in local)
            cap = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
            resident = total <= self.fsdp_config.resident_fraction * cap
        self.fsdp_config.reshard_after_forward = not resident
        logger.info_rank0("reshard_after_forward resolved to %s", self.fsdp_config.reshard_after_forward)

    def _resolve_replicate_layers(self, layers: list[nn.Module]) -> bool:
        """`replicate_layers`: keep the decoder layers' world-sharded parameters replicated (see `FSDPConfig`)."""
        mode = self.fsdp_config.replicate_layers
        if self.world_mesh.size() <= 1 or not layers or self.fsdp_config.cpu_offload.enabled:
            return False
        if mode != "auto":
            return bool(mode)
        if not torch.cuda.is_available():
            return False
        n = sum(self._unit_param_bytes(m) // 2 for m in layers)
        cap = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
        use = 18 * n <= self.fsdp_config.replicate_fraction * cap
        logger.info_rank0("replicate_layers resolved to %s (%.2f B parameters in %d layers)", use, n / 1e9, len(layers))
        return use

    def _collect_no_shard(self, model: nn.Module, compiled: dict[str, FSDPPlanSpec]) -> None:
        """`no_shard` entries may name modules or single parameters; their parameters stay replicated and
        get a world-average all-reduce on the gradient."""
        ids: set[int] = set()
        plan = self._plan
        for fqn, spec in compiled.items():
            if spec.no_shard:
                for p in model.get_submodule(fqn).parameters():
                    ids.add(id(p))
        for name, p in model.named_parameters():
            spec = plan.match(name) if plan is not None else None
            if spec is not None and spec.no_shard:
                ids.add(id(p))
        self.no_shard_names = [n for n, p in model.named_parameters() if id(p) in ids]
        self._model_ref = model

    def _shard_model(self, model: nn.Module, compiled: dict[str, FSDPPlanSpec]) -> None:
        self._collect_no_shard(model, compiled)
        # 1. explicit units, deepest first so children are wrapped before their parents
        explicit = [(fqn, spec) for fqn, spec in compiled.items()
                    if spec.placement is not None or spec.standalone_world_shard]
        emb = model.get_input_embeddings() if hasattr(model, "get_input_embeddings") else None
        head = model.get_output_embeddings() if hasattr(model, "get_output_embeddings") else None
        tied = emb is not None and head is not None and getattr(head, "weight", None) is getattr(emb, "weight", object())
        self._resolve_reshard(model, [model.get_submodule(fqn) for fqn, spec in explicit if self._mesh_for(spec)[0].size() <= 1])
        for fqn, spec in sorted(explicit, key=lambda kv: -kv[0].count(".")):
            mod = model.get_submodule(fqn)
            if tied and (mod is emb or mod is head):
                continue  # tied input/output embeddings must live in one unit: the root
            self._make_unit(mod, spec)
        # 2. every ModuleList child is a unit (small consecutive children share one), or stays replicated
        #    (not inside an explicit unit: a tower that is one standalone unit already owns its blocks' parameters)
        owned = {id(sub) for fqn, _ in explicit for sub in model.get_submodule(fqn).modules()
                 if getattr(model.get_submodule(fqn), "_tt_unit", None) is not None}
        lists = [[c for c in mod if any(True for _ in c.parameters()) and getattr(c, "_tt_unit", None) is None
                  and id(c) not in owned]
                 for _, mod in list(model.named_modules()) if isinstance(mod, nn.ModuleList)]
        replicate = self._resolve_replicate_layers([c for children in lists for c in children])
        for children in lists:
            if replicate:
                for c in children:
                    if getattr(c, "_tt_unit", None) is None:
                        c._tt_unit = "replicated"
                        self.replicated_units.append(c)
                continue
            for group in self._group_layers(children):
                self._make_unit(group, None)
        # 3. input embeddings, resident tail (final norm + output embedding), root
        if emb is not None and not tied:
            self._make_unit(emb, None)
        if head is not None and not tied:
            self._make_unit(head, None, reshard=False)
        self._make_unit(model, None, reshard=False)
        self._keep_host_inputs_on_host(model)
        n_fsdp, n_local = len(self.fsdp_units), len(self.local_units)
        logger.info_rank0("sharding: %d FSDP unit(s), %d single-rank unit(s), %d replicated parameter(s)", n_fsdp,
                          n_local, len(self.no_shard_params))

    def _install_peer_collectives(self) -> None:
        """All-gather / reduce-scatter of the FSDP units run as peer-memory NVLink kernels where the group allows
        it (`backend_config.transport`: auto | p2p | nccl)."""
        self.peer_arenas = []
        mode = str(self.fsdp_config.transport).lower()
        if mode == "nccl" or not self.fsdp_units or not torch.cuda.is_available():
            return
        off = self.fsdp_config.cpu_offload
        if off.enabled and off.mode is CPUOffloadMode.FULL:
            return  # sharded parameters and gradients live on the host
        from ....comm import fsdp_p2p

        by_group: dict[int, tuple[Any, list]] = {}
        for u in self.fsdp_units:
            mesh = getattr(u, "_tt_mesh", None)
            if mesh is None or mesh.ndim != 1:
                continue
            g = mesh.get_group()
            by_group.setdefault(id(g), (g, []))[1].append(u)
        depth = max(self.fsdp_config.forward_prefetch_depth, self.fsdp_config.backward_prefetch_depth)
        for g, units in by_group.values():
            if not fsdp_p2p.usable(g):
                if mode == "p2p":
                    raise RuntimeError("backend_config.transport=p2p needs one NVLink domain with one GPU per rank")
                continue
            arena = fsdp_p2p.install(units, g, prefetch_depth=depth)
            if arena is not None:
                self.peer_arenas.append(arena)
        if self.peer_arenas:
            logger.info_rank0("FSDP collectives over peer memory: %d group(s)", len(self.peer_arenas))

    def _setup_prefetch(self, model: nn.Module) -> None:
        if not self.fsdp_units:
            return
        from .prefetch import FSDPPrefetchManager

        self.prefetch_manager = FSDPPrefetchManager(self.fsdp_config)
        self.prefetch_manager.setup(model)

    def _register_vision_balance(self, model: nn.Module, compiled: dict[str, FSDPPlanSpec]) -> None:
        for fqn, spec in compiled.items():
            vb = spec.vision_balance
            if vb is not None and vb.mode is not None:
                from ....models.modules.vision import register_vision_balance

                register_vision_balance(model.get_submodule(fqn), vb, sp_group=self.sp_group, sp_size=self.sp_size,
                                        sp_rank=self.sp_rank, world_group=dist.group.WORLD)

    # ------------------------------------------------------------------------------------------
    # materialisation
    # ------------------------------------------------------------------------------------------
    def _unit_owned_params(self, model: nn.Module) -> dict[int, str]:
        """param id -> kind ('fsdp' | 'local') of the deepest unit that contains it."""
        owner: dict[int, str] = {}

        def walk(mod: nn.Module, kind: str | None):
            kind = getattr(mod, "_tt_unit", None) or kind
            for p in mod.parameters(recurse=False):
                if kind is not None:
                    owner[id(p)] = kind
            for c in mod.children():
                walk(c, kind)

        walk(model, None)
        for p in self.no_shard_params:
            owner[id(p)] = "replicated"
        return owner

    def materialize(self, model: nn.Module, *, init_weights: bool = True) -> None:
        """Allocate real storage for a meta-device model on this rank's device and (optionally) initialise it
        with the model's own initialiser, seeded identically on every rank and then sharded."""
        has_meta = any(p.is_meta for p in model.parameters()) or any(b.is_meta for b in model.buffers())
        if has_meta:
            model.to_empty(device=self.device)
        elif next(model.parameters()).device != self.device:
            model.to(self.device)
        if init_weights and has_meta:
            self._init_parameters(model)

    def _init_parameters(self, model: nn.Module, seed: int = 0) -> None:
        """normal(0, initializer_range) for matrices, ones for norm weights, zeros for biases.  Every parameter is
        drawn from its own generator (seed + CRC of its name) at its *global* shape and then cut down to this
        rank's shard / experts, so the initial model does not depend on the world size or the EP / FSDP layout."""
        import zlib

        std = float(getattr(getattr(model, "config", None), "initializer_range", 0.02))
        seed = int(getattr(self, "_init_seed", seed))
        expert_ids_cache = self.expert_param_ids
        with torch.no_grad():
            for name, p in model.named_parameters():
                lp = p._local_tensor if hasattr(p, "_local_tensor") else p
                if p.ndim <= 1:
                    if name.endswith("bias") or "expert_bias" in name:
                        lp.zero_()
                    else:
                        lp.fill_(1.0)
                    continue
                gen = torch.Generator(device=lp.device)
                expert_ids = expert_ids_cache
                gen.manual_seed(seed * 1000003 + zlib.crc32(name.encode()))
                shape = list(p.shape)
                is_expert = id(p) in expert_ids
                if is_expert and self.ep_size > 1:
                    shape[0] *= self.ep_size
                full = torch.empty(shape, dtype=torch.float32, device=lp.device).normal_(0.0, std, generator=gen)
                if is_expert and self.ep_size > 1:
                    rows = p.shape[0]
                    full = full[self.ep_rank * rows:(self.ep_rank + 1) * rows]
                if hasattr(p, "_local_tensor"):
                    from torch.distributed.tensor import Shard

                    for mesh_dim, pl in enumerate(p.placements):
                        if isinstance(pl, Shard):
                            n, r = p.device_mesh.size(mesh_dim), p.device_mesh.get_local_rank(mesh_dim)
                            chunks = torch.chunk(full, n, dim=pl.dim)
                            full = chunks[r] if r < len(chunks) else full.narrow(pl.dim, 0, 0)
                    lp.zero_()
                    lp[tuple(slice(0, s_) for s_ in full.shape)].copy_(full)
                else:
                    lp.copy_(full)
                del full
            for name, b in model.named_buffers():
                if "inv_freq" in name:
                    continue
                b.zero_()                      # integer tables too: uninitialised storage must never be used as an index
            for m in model.modules():          # buffers with content of their own (seeded routing tables, ...)
                hook = getattr(m, "reset_buffers_after_materialize", None)
                if callable(hook):
                    hook()

    def _init_adapters(self, model: nn.Module) -> None:
        """LoRA / DoRA adapters of a materialised model start as a no-op: A is uniform in +-1/sqrt(fan_in) (drawn at its
        global shape from a generator seeded by its name, then cut to this rank's shard, like the base parameters), B is
        zero, a DoRA magnitude is the row norm of the weight it scales.  Runs after the base weights are in place, for
        loaded and for freshly initialised models alike (the base initialiser knows nothing about adapters)."""
        if not getattr(model, "peft_config", None):
            return
        import zlib

        from ...peft.lora import LoRALinear, is_adapter_param

        seed = int(getattr(self, "_init_seed", 0))
        with torch.no_grad():
            for name, p in model.named_parameters():
                if not is_adapter_param(name):
                    continue
                lp = p._local_tensor if hasattr(p, "_local_tensor") else p
                parts = name.split(".")
                if "lora_B" in parts:
                    lp.zero_()
                    continue
                if "lora_magnitude_vector" in parts:
                    lp.fill_(1.0)
                    continue
                gen = torch.Generator(device=lp.device)
                gen.manual_seed(seed * 1000003 + zlib.crc32(name.encode()))
                shape = list(p.shape)
                is_expert = p.dim() == 3 and self.ep_size > 1          # grouped factors hold the local experts only
                if is_expert:
                    shape[0] *= self.ep_size
                bound = 1.0 / math.sqrt(shape[-1])
                full = torch.empty(shape, dtype=torch.float32, device=lp.device).uniform_(-bound, bound, generator=gen)
                if is_expert:
                    full = full[self.ep_rank * p.shape[0]:(self.ep_rank + 1) * p.shape[0]]
                if hasattr(p, "_local_tensor"):
                    from torch.distributed.tensor import Shard

                    for mesh_dim, pl in enumerate(p.placements):
                        if isinstance(pl, Shard):
                            n, r = p.device_mesh.size(mesh_dim), p.device_mesh.get_local_rank(mesh_dim)
                            chunks = torch.chunk(full, n, dim=pl.dim)
                            full = chunks[r] if r < len(chunks) else full.narrow(pl.dim, 0, 0)
                    lp.zero_()
                    lp[tuple(slice(0, s_) for s_ in full.shape)].copy_(full)
                else:
                    lp.copy_(full)
            for m in model.modules():
                if isinstance(m, LoRALinear) and m.lora_magnitude_vector is not None:
                    mag = m.lora_magnitude_vector[m.cfg.adapter_name].weight
                    norms = m.delta_free_weight().float().norm(dim=1)          # gathers a sharded weight: all ranks take part
                    if hasattr(mag, "_local_tensor"):
                        from torch.distributed.tensor import distribute_tensor

                        mag._local_tensor.copy_(distribute_tensor(norms.to(mag.dtype), mag.device_mesh, mag.placements)._local_tensor)
                    else:
                        mag.copy_(norms.to(mag.dtype))

    def reshard_all(self, model: nn.Module) -> None:
        """Every FSDP unit of `model` back to its sharded parameters.  A unit that is kept gathered after a forward
        (the resident tail, every unit after a forward without gradients) shows plain, unsharded tensors under the names
        of its parameters; state dictionaries must be built from the sharded ones."""
        for m in model.modules():
            if getattr(m, "_tt_unit", None) == "fsdp" and hasattr(m, "reshard"):
                m.reshard()

    def finalize_model_load(self, model: nn.Module) -> None:
        """After weights are in place: adapters get their initial values, single-rank units switch to bf16 parameters
        (their fp32 values become the optimizer's master copy), replicated parameters get their gradient all-reduce
        hook."""
        self._init_adapters(model)
        if self.config.mixed_precision is MixedPrecisionPolicy.BF16:
            owner = self._unit_owned_params(model)
            with torch.no_grad():
                for name, p in model.named_parameters():
                    if owner.get(id(p)) in ("local", "replicated") and p.dtype == torch.float32:
                        master = p.data
                        p.data = master.to(torch.bfloat16)
                        if p.requires_grad:
                            p._master_init = master
        self._register_no_shard_grad_sync()
        self._setup_replicated_grads()

    # -- replicated decoder layers: one flat fp32 gradient buffer, one all-reduce per optimizer step ------------
    def _setup_replicated_grads(self) -> None:
        """Every trainable parameter of a replicated layer gets `main_grad`, a view into one flat fp32 buffer.  Weight
        gradient GEMMs accumulate straight into it (no `.grad` tensor); gradients that autograd still delivers as
        `.grad` are folded in before the buffer is averaged over the ranks (`_sync_replicated_grads`)."""
        if not self.replicated_units or self._rep_flat is not None:
            return
        seen: set[int] = set()
        params = []
        for m in self.replicated_units:
            nested = {id(q) for sub in m.modules() if sub is not m and getattr(sub, "_tt_unit", None) is not None
                      for q in sub.parameters()}          # expert containers and other units inside the layer
            for p in m.parameters():
                if id(p) not in nested and id(p) not in seen and p.requires_grad:
                    seen.add(id(p))
                    params.append(p)
        if not params:
            return
        sizes = [(p.numel() + 3) // 4 * 4 for p in params]          # 16-byte aligned slices
        flat = self._alloc_replicated_flat(sum(sizes), params[0].device)
        off = 0
        for p, n in zip(params, sizes):
            p.main_grad = flat[off:off + p.numel()].view(p.shape)
            p.main_grad._tt_flat_owner = flat
            off += n
        self._rep_flat, self._rep_params = flat, params
        logger.info_rank0("replicated layers: %d parameters, %.1f MB flat fp32 gradient buffer", len(params), flat.numel() * 4 / 2**20)

    def _alloc_replicated_flat(self, numel: int, device: torch.device) -> torch.Tensor:
        """The flat gradient buffer lives in symmetric memory when the world is one NVLink domain: weight-gradient GEMMs
        accumulate straight into peer-visible memory and the all-reduce is the in-switch multimem kernel (no copy-in)."""
        self._rep_symm = None
        if device.type == "cuda" and self.world_size > 1:
            try:
                from ....comm.symm import SymmetricBuffer

                if SymmetricBuffer.usable(dist.group.WORLD) and os.environ.get("TORCHTURBO_REPLICATED_ALLREDUCE", "auto") != "nccl":
                    buf = SymmetricBuffer(numel * 4 + 2 * 4 * self.world_size + 4096, dist.group.WORLD)
                    if buf.multicast_ptr:
                        off, flat = buf.carve(numel * 4, torch.float32)
                        self._rep_symm = {"buf": buf, "off": off, "before": buf.channel(), "after": buf.channel(),
                                          "status": torch.zeros(1, dtype=torch.int32, device=device)}
                        self.peer_arenas = list(getattr(self, "peer_arenas", [])) + [_FlatGradExchange(self._rep_symm, self.rank)]
                        logger.info_rank0("replicated layers: gradient all-reduce in the NVSwitch (multimem), %.1f MB", numel * 4 / 2**20)
                        return flat
            except Exception as e:  # noqa: BLE001 - no symmetric memory on this system: NCCL all-reduce
                logger.info_rank0("replicated layers: symmetric gradient buffer unavailable (%s), NCCL all-reduce", e)
        return torch.zeros(numel, dtype=torch.float32, device=device)

    def _allreduce_replicated_flat(self) -> None:
        sy = self._rep_symm
        if sy is None:
            dist.all_reduce(self._rep_flat, op=dist.ReduceOp.SUM)
            self._rep_flat.div_(self.world_size)
            return
        from .... import kernels as K

        buf, W, r = sy["buf"], self.world_size, self.rank
        budget = int(os.environ.get("TORCHTURBO_P2P_WAIT_MS", "5000"))
        for ch, run in ((sy["before"], True), (sy["after"], False)):
            epoch = ch.next()
            K.flag_signal(buf.peer_ptrs, ch.offset, r, W, epoch)        # mine is written / my slice is stored
            K.flag_wait(buf.peer_ptrs, ch.offset, r, W, epoch, budget, sy["status"])
            if run:
                K.multimem_allreduce_f32(buf.multicast_ptr + sy["off"], self._rep_flat.numel(), r, W, 1.0 / W)

    @torch.no_grad()
    def _sync_replicated_grads(self) -> None:
        """Fold stray `.grad` tensors into the flat buffer and average it over the world (once per optimizer step)."""
        if self._rep_flat is None or self._rep_synced:
            return
        mains, grads = [], []
        for p in self._rep_params:
            if p.grad is not None:
                mains.append(p.main_grad)
                grads.append(p.grad if p.grad.dtype == torch.float32 else p.grad.float())
                p.grad = None
        if mains:
            torch._foreach_add_(mains, grads)
        if self.world_size > 1:
            self._allreduce_replicated_flat()
        for p in self._rep_params:
            if p.dtype == torch.float32:
                p.grad = p.main_grad      # optimizers that only know `.grad` (fp32 runs) read the averaged view
        self._rep_synced = True

    def _after_optimizer_step(self, *_args, **_kwargs) -> None:
        if self._rep_flat is not None:
            self._rep_flat.zero_()
            self._rep_synced = False

    def _register_no_shard_grad_sync(self) -> None:
        if self.world_size == 1:
            return
        W = self.world_size

        def hook(p):
            if p.grad is not None:
                dist.all_reduce(p.grad, op=dist.ReduceOp.SUM)
                p.grad.div_(W)

        for p in self.no_shard_params:
            if p.requires_grad and not getattr(p, "_tt_sync_hook", False):
                p.register_post_accumulate_grad_hook(hook)
                p._tt_sync_hook = True

    def create_checkpoint_manager(self):
        from .checkpoint import FSDP2CheckpointManager

        return FSDP2CheckpointManager(self)

    # ------------------------------------------------------------------------------------------
    # optimizer
    # ------------------------------------------------------------------------------------------
    def _topology_of(self, p: torch.Tensor, expert_ids: set[int] | None = None) -> str:
        if id(p) in (self.expert_param_ids if expert_ids is None else expert_ids):
            return "moe"
        if hasattr(p, "_local_tensor"):
            return "dense"
        return "local"

    def prepare_optimizer(self, model: nn.Module, optimizer_plan) -> torch.optim.Optimizer:
        """Build one optimizer per (class, sharding topology): fused/foreach optimizers cannot mix DTensor
        meshes, and the expert group needs its own gradient scale when clipping."""
        from ...optimizers import FusedAdamW, OptimizersContainer
        from ...optimizers.plan import OptimizerClassPlan, OptimizerPlan

        if isinstance(optimizer_plan, OptimizerClassPlan):
            optimizer_plan = optimizer_plan.resolve(model.named_parameters())
        assert isinstance(optimizer_plan, OptimizerPlan)
        optimizer_plan.validate(model)
        buckets: dict[tuple, list[dict]] = {}
        for g in optimizer_plan.groups:
            by_topo: dict[str, list] = {}
            eids = self.expert_param_ids
            for p in g.params:
                by_topo.setdefault(self._topology_of(p, eids), []).append(p)
            for topo, ps in by_topo.items():
                buckets.setdefault((g.optimizer_cls, topo), []).append({"params": ps, **g.hyperparameters})
        opts, names = [], []
        for (cls, topo), groups in buckets.items():
            off = self.fsdp_config.cpu_offload
            if cls in (torch.optim.AdamW, "adamw") and off.enabled and off.mode is CPUOffloadMode.OPTIMIZER:
                # optimizer state on the host, streamed through a bounded device workspace
                from ...optimizers.adamw_swap import AdamWSwap

                opt = AdamWSwap(groups, memory_fraction=off.optimizer_memory_fraction)
                opt._tt_topology = topo
                opts.append(opt)
                names.append(f"adamwswap_{topo}")
                continue
            if cls in (torch.optim.AdamW, "adamw") and self.runtime.turbo_device.value == "cuda":
                cls = FusedAdamW
            elif cls == "adamw":
                cls = FusedAdamW
            opt = cls(groups)
            opt._tt_topology = topo
            opts.append(opt)
            names.append(f"{getattr(cls, '__name__', str(cls)).lower()}_{topo}")
        for o in opts:
            for grp in o.param_groups:
                for p in grp["params"]:
                    init = getattr(p, "_master_init", None)
                    if init is not None and isinstance(o, FusedAdamW):
                        st = o._init_state(p)
                        st["master"] = init
                        del p._master_init
        self._enable_update_overlap(model, [o for o in opts if isinstance(o, FusedAdamW)])
        if self._rep_flat is not None:
            # replicated layers: gradients are averaged before the first optimizer touches them (normally already done
            # by `clip_grad_norm_`), the flat buffer is cleared after the last one has stepped
            opts[0].register_step_pre_hook(lambda *_a, **_k: self._sync_replicated_grads())
            opts[-1].register_step_post_hook(self._after_optimizer_step)
        return opts[0] if len(opts) == 1 else OptimizersContainer(opts, names)

    def _enable_update_overlap(self, model: nn.Module, fused: list) -> None:
        """Let the AdamW update of the decoder layers run on a side stream under the next forward pass: one bucket per
        layer of every `layers` ModuleList, and a forward pre-hook per layer that waits for its own bucket only
        (`FusedAdamW.enable_overlap`).  Off unless `TORCHTURBO_ADAMW_OVERLAP=1`: the persistent GEMMs of the forward pass
        hold every SM's registers and shared memory, so the bandwidth-bound update only gets the gaps between kernels
        (measured: 84.7 against 85.9 ms per step at 1 GPU, 12 layers)."""
        if not fused or self.device.type != "cuda" or os.environ.get("TORCHTURBO_ADAMW_OVERLAP", "0") != "1":
            return
        layers = [m for name, mod in model.named_modules() if isinstance(mod, nn.ModuleList) and name.split(".")[-1] == "layers"
                  for m in mod]
        if not layers:
            return
        buckets = [[p for p in layer.parameters() if p.requires_grad and not hasattr(p, "_local_tensor")] for layer in layers]
        for o in fused:
            o.enable_overlap(buckets)

        def make_hook(i):
            def hook(_module, _args):
                for o in fused:
                    o.wait_bucket(i)
            return hook

        for i, layer in enumerate(layers):
            layer.register_forward_pre_hook(make_hook(i))
        logger.info_rank0("AdamW update of %d decoder layers overlaps the next forward pass (side stream, one event per layer)",
                          len(layers))

    # ------------------------------------------------------------------------------------------
    # gradient clipping
    # ------------------------------------------------------------------------------------------
    def _scale_moe_gradient(self, model: nn.Module) -> None:
        """Expert gradients are sums over the tokens of all `ep` ranks; dividing by `ep` puts them on the same
        per-rank-average footing as the FSDP-averaged dense gradients."""
        if self.ep_size == 1:
            return
        with torch.no_grad():
            for m in self.expert_modules:
                for p in m.parameters():
                    if p.grad is not None and not getattr(p, "_tt_grad_scaled", False):
                        p.grad.mul_(self.gradient_scaling_factor)
                        p._tt_grad_scaled = True

    @torch.no_grad()
    def _peer_status_flag(self) -> torch.Tensor | None:
        """Device bool: any peer-memory workspace of this rank has a non-zero status word (None without workspaces)."""
        if self.device.type != "cuda":
            return None
        from ...health import peer_workspaces

        words = [ws.status.reshape(1) for ws in peer_workspaces(self) if isinstance(getattr(ws, "status", None), torch.Tensor)]
        if not words:
            return None
        return (torch.cat(words) if len(words) > 1 else words[0]).ne(0).any()

    def clip_grad_norm_(self, model: nn.Module, max_norm: float, optimizer=None) -> torch.Tensor:
        """Global L2 norm over dense (world-sharded), expert (edp-sharded, unique per EP rank) and replicated /
        single-rank parameters; every gradient is then scaled by `min(1, max_norm / (norm + 1e-6))`.
        With the fused AdamW the coefficient is handed to the optimizer as a device scalar and applied inside
        the update kernel instead of in a separate pass."""
        from ...optimizers import FusedAdamW, OptimizersContainer

        opts = list(optimizer) if isinstance(optimizer, OptimizersContainer) else ([optimizer] if optimizer is not None else [])
        dev = self.device
        # the module tree is walked once: parameter objects and their optimizer membership do not change between steps
        ckey = (id(model), tuple(id(o) for o in opts))
        cache = getattr(self, "_clip_cache", None)
        if cache is None or cache["key"] != ckey:
            params = list(model.parameters())
            fused = {id(p) for o in opts if isinstance(o, FusedAdamW) for grp in o.param_groups for p in grp["params"]}
            cache = self._clip_cache = {"key": ckey, "params": params, "fused": fused,
                                        "unfused": [p for p in params if id(p) not in fused]}
        params = cache["params"]
        self._sync_replicated_grads()
        if self.ep_size > 1:
            # the fused optimizer of the expert parameters folds the 1/ep scaling into its gradient reads
            for o in opts:
                if isinstance(o, FusedAdamW) and getattr(o, "_tt_topology", None) == "moe" and dev.type == "cuda":
                    ps = [p for grp in o.param_groups for p in grp["params"]]
                    if ps and not any(getattr(p, "_tt_grad_scaled", False) for p in ps):
                        o.grad_prescale = self.gradient_scaling_factor
                        for p in ps:
                            p._tt_grad_scaled = True
        self._scale_moe_gradient(model)
        sums = {"dense": torch.zeros((), dtype=torch.float32, device=dev), "moe": torch.zeros((), dtype=torch.float32, device=dev),
                "local": torch.zeros((), dtype=torch.float32, device=dev)}
        covered: set[int] = set()
        for o in opts:  # fused path: one multi-tensor launch per parameter group, no per-tensor norms
            if isinstance(o, FusedAdamW) and getattr(o, "_tt_topology", None) in sums:
                s_ = o.grad_sq_sum()
                if s_ is not None:
                    sums[o._tt_topology] = sums[o._tt_topology] + s_
                    covered.update(id(p) for grp in o.param_groups for p in grp["params"])
        sq = {"dense": [], "moe": [], "local": []}
        eids = cache.get("eids")
        if eids is None:
            eids = cache["eids"] = self.expert_param_ids
        for p in (params if not covered else (cache["unfused"] if covered >= cache["fused"] else params)):
            if id(p) in covered:
                continue
            g = getattr(p, "main_grad", None)
            g = g if g is not None else p.grad
            if g is None:
                continue
            lg = g._local_tensor if hasattr(g, "_local_tensor") else g
            sq[self._topology_of(p, eids)].append(lg)

        def sumsq(ts):
            if not ts:
                return torch.zeros((), dtype=torch.float32, device=dev)
            norms = torch._foreach_norm(ts, 2.0)
            return torch.stack([n.float() for n in norms]).pow(2).sum()

        dense, moe, local = (sums["dense"] + sumsq(sq["dense"]), sums["moe"] + sumsq(sq["moe"]),
                             sums["local"] + sumsq(sq["local"]))
        sharded = dense + moe
        if self.world_size > 1:
            # A peer-memory kernel that timed out or overflowed its receive buffer on ANY rank poisons the norm: the
            # status words ride on the all-reduce below (no extra collective, no host read), the coefficient becomes
            # NaN on every rank, the fused AdamW kernel skips the update, and the loop's finite check of the norm raises
            # in this very step instead of training on dropped rows until the next logging boundary.
            bad = self._peer_status_flag()
            if bad is not None:
                sharded = torch.where(bad, torch.full_like(sharded, float("nan")), sharded)
            # FSDP shards and EP-local experts are disjoint across the world; replicated ones are not summed
            dist.all_reduce(sharded)
        total = (sharded + local).sqrt()
        coef = (max_norm / (total + 1e-6)).clamp(max=1.0) if max_norm and max_norm > 0 else torch.ones_like(total)
        for o in opts:
            if isinstance(o, FusedAdamW):
                o.set_clip_coef(coef.reshape(1))
        rest = []
        for p in cache["unfused"]:
            if p.grad is not None:
                rest.append(p.grad._local_tensor if hasattr(p.grad, "_local_tensor") else p.grad)
        if rest:
            torch._foreach_mul_(rest, coef)
        if self.ep_size > 1:
            for p in params:
                if getattr(p, "_tt_grad_scaled", False):
                    p._tt_grad_scaled = False
        return total

    # ------------------------------------------------------------------------------------------
    # inputs and loss
    # ------------------------------------------------------------------------------------------
    def prepare_inputs(self, model: nn.Module, inputs: dict[str, Any]) -> dict[str, Any]:
        """Right-pad the declared batch fields to a multiple of `sp_size` and move tensors to the device
        (packed boundaries stay on the host: kernels that need them receive a device copy once per step)."""
        if self.sp_size > 1:
            inputs = ulysses_pad_inputs(inputs, model.get_sequence_parallel_input_slicing_spec(), self.sp_size)
        out = {}
        for k, v in inputs.items():
            if isinstance(v, torch.Tensor) and k not in ("cu_seq_lens_q", "cu_seq_lens_k") and v.device != self.device:
                v = v.to(self.device, non_blocking=True)
            out[k] = v
        return out

    def _moe_layers(self, model: nn.Module) -> list:
        """MoE layers of `model`, found once (the module tree does not change after preparation)."""
        cached = getattr(model, "_tt_moe_layers", None)
        if cached is None:
            cached = [m for m in model.modules() if isinstance(m, BaseMoELayer)]
            object.__setattr__(model, "_tt_moe_layers", cached)
        return cached

    def _prepare_moe_runtime(self, model: nn.Module, inputs: dict[str, Any], aux_loss_scale: float) -> None:
        layers = self._moe_layers(model)
        if not layers:
            return
        rt = model.get_moe_runtime_inputs(inputs, self.get_parallel_context())
        rt.aux_loss_scale = aux_loss_scale
        for m in layers:
            m.set_runtime_inputs(rt)

    def compute_loss(self, model: nn.Module, inputs: dict[str, Any], *, num_items_in_batch=None,
                     aux_loss_scale: float = 1.0, return_outputs: bool = False):
        """Forward + language-model loss for one packed micro-batch.  Labels are shifted inside the engine
        (the batch carries unshifted labels); under SP every rank computes the loss of its shard with a global
        normaliser and the shards are summed with an autograd-aware all-reduce."""
        from ....models.modules.comm import all_reduce_sum_autograd

        inputs = dict(inputs)
        labels = inputs.pop("labels")
        cu = inputs["cu_seq_lens_q"]
        if inputs.get("position_ids") is None:
            T = inputs["input_ids"].shape[-1]
            inputs["position_ids"] = torch.arange(T, device=inputs["input_ids"].device).unsqueeze(0)
        self._prepare_moe_runtime(model, inputs, aux_loss_scale)
        use_chunk = self.config.loss_chunk.enabled or self.runtime.turbo_device.value == "cuda" or self.world_size > 1
        head = model.get_lm_head() if hasattr(model, "get_lm_head") else None
        use_chunk = use_chunk and head is not None
        if self.config.dspark.enabled and getattr(model, "dspark", None) is not None:
            # block-draft heads (DeepSeek-V4 DSpark): trained from the same row; they need the unshifted labels
            inputs["dspark_labels"], inputs["dspark_config"] = labels, self.config.dspark
        out = model(**inputs, skip_lm_head=use_chunk)
        n_streams = 1 + (len(out.get("mtp_hidden_states") or ()) if self.config.mtp.enabled else 0)
        scales = [1.0] + [self.config.mtp.loss_scaling_factor] * (n_streams - 1)
        streams = prepare_loss_labels(labels.to(self.device), cu, num_streams=n_streams, stream_scales=scales,
                                      num_items_in_batch=num_items_in_batch, sp_size=self.sp_size, sp_rank=self.sp_rank,
                                      world_size=self.world_size)
        if use_chunk:
            hs = [out["hidden_states"]] + list(out.get("mtp_hidden_states") or ())[: n_streams - 1]
            total, comps = chunk_loss(hs, head, streams, self._loss_chunk_size(hs[0]))
        else:
            lgs = [out["logits"]] + list(out.get("mtp_logits") or ())[: n_streams - 1]
            total, comps = logits_loss(lgs, streams)
        if self.sp_size > 1:
            total = all_reduce_sum_autograd(total, self.sp_group)
            for k in comps:
                dist.all_reduce(comps[k], group=self.sp_group)
        if out.get("dspark_loss") is not None:
            total = total + self.config.dspark.loss_scaling_factor * out["dspark_loss"]
        out["loss"] = total
        out["main_loss"] = comps.get("main")
        for k, v in comps.items():
            if k != "main":
                out[f"{k}_loss"] = v
        return (total, out) if return_outputs else total

    def compute_diffusion_loss(self, model: nn.Module, inputs: dict[str, Any], *, ga: int = 1,
                               return_outputs: bool = False, **_unused):
        """Block-diffusion loss: unshifted cross entropy over the supervised (masked, noisy-half) positions of a
        `[noisy | clean]` row, plus `cap_lambda` times the mean prediction entropy over the positions the model
        already gets right (a confidence term).  Under SP the row is sliced, the block mask stays global; sums and
        counts are all-reduced over the SP group and divided globally, so the value equals the SP=1 mean.  The
        result is divided by `ga` (gradient-accumulation steps including the SP factor).  Same contract as
        engine/backends/fsdp2/backend.py:2005-2090 of the reference."""
        from ....models.modules.attention.ulysses import slice_input_tensor
        from ....models.modules.comm import all_reduce_sum_autograd

        if self.config.loss_chunk.enabled:
            raise NotImplementedError("chunked LM loss does not support diffusion training")
        inputs = dict(self.prepare_inputs(model, inputs))
        inputs.pop("bd_structure", None)
        inputs.pop("attention_mask", None)
        labels = inputs.pop("labels").to(self.device)
        self._prepare_moe_runtime_for_row(model, inputs)
        out = model(**inputs)
        logits = out["logits"]
        n_valid = (labels != -100).sum()
        if self.sp_size > 1:
            labels = slice_input_tensor(labels, 1, self.sp_group, self.sp_rank)
        flat, lab = logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1)
        loss_sum = torch.nn.functional.cross_entropy(flat, lab, ignore_index=-100, reduction="sum")
        cap = float(self.config.diffusion.cap_lambda)
        ent_sum = n_correct = None
        if cap > 0:
            ent_sum, n_correct = confidence_entropy_sum(flat, lab)
        if self.sp_size > 1:
            loss_sum = all_reduce_sum_autograd(loss_sum, self.sp_group)
            if cap > 0:
                ent_sum = all_reduce_sum_autograd(ent_sum, self.sp_group)
                n_correct = n_correct.clone()
                dist.all_reduce(n_correct, group=self.sp_group)
        loss = loss_sum / n_valid.clamp_min(1).to(loss_sum.dtype)
        if cap > 0:
            loss = loss + cap * ent_sum / n_correct.clamp_min(1).to(ent_sum.dtype)
        loss = loss / ga
        out["loss"] = loss
        return (loss, out) if return_outputs else loss

    def _prepare_moe_runtime_for_row(self, model: nn.Module, inputs: dict[str, Any]) -> None:
        """MoE statistics of a diffusion row: no packed boundaries, nothing is padding."""
        layers = [m for m in model.modules() if isinstance(m, BaseMoELayer)]
        if layers:
            from ....models.modules.moe import MoERuntimeInputs

            rt = MoERuntimeInputs()
            for m in layers:
                m.set_runtime_inputs(rt)

    def _loss_chunk_size(self, hidden: torch.Tensor) -> int:
        if self.config.loss_chunk.enabled:
            return self.config.loss_chunk.chunk_size
        return 4096  # on B200 the fused path is always used; 4096 rows keep the bf16 logits chunk near 1.2 GB
