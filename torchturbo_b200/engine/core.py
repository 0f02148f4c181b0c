"""`TorchTurboEngine`: one facade for building, sharding, loading, optimising, feeding and saving a model.

Life cycle (engine/core.py:148-1526 of the reference, same public method names):

    engine = TorchTurboEngine(config)
    model  = engine.prepare_model(path_or_config, load_weights=True)      # meta -> shard -> load -> hooks
    optim  = engine.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=..., weight_decay=...))
    sched  = engine.prepare_lr_scheduler(optim, "cosine", num_warmup_steps=..., num_training_steps=...)
    loader = engine.create_dataloader(dataset, collate_fn=..., batch_size=1)
    loss   = engine.compute_loss(model, batch); loss.backward(); engine.clip_grad_norm_(model, 1.0, optim); optim.step()
    engine.save_model(model, dir); engine.save_optimizer_and_scheduler(model, optim, sched, dir)

Unlike the reference, which delegates the training loop to external trainers, `fit()` runs the engine's own
SFT / CPT loop (see `torchturbo_b200.loops`).
"""
from __future__ import annotations

import copy
import json
import math
import os
import socket
from typing import Any, Callable, Iterator

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.data import DataLoader, DistributedSampler

from ..logging import get_logger
from ..models.config import load_config
from ..models.registry import get_model
from ..ops import get_or_create_ops
from ..parallel import FSDPParallelPlan, FSDPPlanSpec, VisionBalanceSpec
from ..runtime import get_device_runtime
from ..utils.fqn import match_fqn
from ..utils.torch_utils import has_meta_tensor
from .backend_registry import get_backend
from .config import EngineConfig, FreezePolicy, ParameterGroup
from .distributed import assert_finite
from .metrics import MetricTracker, MFUEstimator
from .plugins import PluginManager
from .rl import RLMixin

logger = get_logger(__name__)


class DPBlockDistributedSampler(DistributedSampler):
    """Block-wise data-parallel sampler whose SP ranks see identical samples.

    A global permutation (seed + epoch) is cut into blocks of `dp_size * rank_block` indices; DP rank d takes
    `[d*rank_block, (d+1)*rank_block)` of every block.  `rank_block` is the number of micro-batches a rank
    consumes per optimizer step times the micro-batch size, so one optimizer step always draws one block and
    the global batch does not depend on how it is split.  The index list is truncated (drop_last) or cycled to
    whole blocks.  Optionally each DP rank reshuffles its share with `seed + epoch + dp_rank`.
    """

    def __init__(self, dataset, dp_size: int, dp_rank: int, rank_block: int = 1, shuffle: bool = True, seed: int = 0,
                 drop_last: bool = False, per_rank_shuffle: bool = False):
        super().__init__(dataset, num_replicas=dp_size, rank=dp_rank, shuffle=shuffle, seed=seed, drop_last=drop_last)
        self.rank_block = max(1, int(rank_block))
        self.per_rank_shuffle = per_rank_shuffle
        block = dp_size * self.rank_block
        n = len(dataset)
        n_blocks = n // block if drop_last else math.ceil(n / block)
        self.num_blocks = max(n_blocks, 1 if n > 0 else 0)
        self.num_samples = self.num_blocks * self.rank_block
        self.total_size = self.num_blocks * block

    def __iter__(self) -> Iterator[int]:
        n = len(self.dataset)
        if self.shuffle:
            g = torch.Generator()
            g.manual_seed(self.seed + self.epoch)
            idx = torch.randperm(n, generator=g).tolist()
        else:
            idx = list(range(n))
        if len(idx) < self.total_size:
            reps = math.ceil(self.total_size / max(len(idx), 1))
            idx = (idx * reps)[: self.total_size]
        else:
            idx = idx[: self.total_size]
        block = self.num_replicas * self.rank_block
        mine: list[int] = []
        for b in range(self.num_blocks):
            lo = b * block + self.rank * self.rank_block
            mine.extend(idx[lo: lo + self.rank_block])
        if self.per_rank_shuffle:
            g = torch.Generator()
            g.manual_seed(self.seed + self.epoch + self.rank)
            mine = [mine[i] for i in torch.randperm(len(mine), generator=g).tolist()]
        return iter(mine)

    def __len__(self) -> int:
        return self.num_samples


class EpochDrivenDataLoader(DataLoader):
    """DataLoader that forwards `set_epoch` to its sampler."""

    def set_epoch(self, epoch: int) -> None:
        s = getattr(self, "sampler", None)
        if hasattr(s, "set_epoch"):
            s.set_epoch(epoch)
        bs = getattr(self, "batch_sampler", None)
        if bs is not None and hasattr(getattr(bs, "sampler", None), "set_epoch"):
            bs.sampler.set_epoch(epoch)


class TorchTurboEngine(RLMixin):
    def __init__(self, config: EngineConfig | dict[str, Any] | None = None) -> None:
        if config is None:
            config = EngineConfig()
        elif isinstance(config, dict):
            config = EngineConfig.from_dict(config)
        self.config = config
        self.runtime = get_device_runtime()
        if config.use_deterministic_algorithms:
            self.runtime.use_deterministic_algorithms()
        self.backend = get_backend(config.backend)(config, self.runtime)
        self.ops = get_or_create_ops(config.ops.policy, config.ops.overrides or None, self.runtime)
        self.plugins = PluginManager(config.plugin_paths)
        self.metrics = MetricTracker()
        self._checkpoint = None
        self._profiler = None
        self._mfu: MFUEstimator | None = None
        self._model_source: str | None = None
        self._optimizer = None

    # ------------------------------------------------------------------------------------------
    # model construction
    # ------------------------------------------------------------------------------------------
    def build_model(self, model_name_or_path: str | None = None, *, model_cls: type | None = None,
                    load_weights: bool = True, init_kwargs: dict[str, Any] | None = None,
                    peft_config: Any = None) -> nn.Module:
        """Construct on the meta device, apply the parallel plan, then either load a Hugging Face checkpoint
        shard-wise or materialise with seeded random initialisation (`load_weights=False`)."""
        init_kwargs = dict(init_kwargs or {})
        cfg = init_kwargs.pop("config", None)
        if cfg is None:
            if model_name_or_path is None:
                raise ValueError("either a checkpoint path or init_kwargs['config'] is required")
            cfg = load_config(model_name_or_path)
        elif isinstance(cfg, dict):
            cfg = load_config(cfg)
        model_type = getattr(cfg, "model_type", None)
        turbo_cls = model_cls or get_model(model_type)
        from ..models.base import TurboModel

        if not issubclass(turbo_cls, TurboModel):
            raise TypeError(f"{turbo_cls.__name__} is not a TurboModel")
        with turbo_cls.init_context(cfg, self.config):
            with torch.device("meta"):
                model = turbo_cls(cfg)
            plan = self._resolve_parallel_plan(model)
            model = self.backend.prepare_model(model, plan, peft_config)
        model.on_parallelized(self.backend.get_parallel_context())
        self._checkpoint = self._make_coordinator()
        if load_weights:
            if model_name_or_path is None:
                raise ValueError("load_weights=True needs a checkpoint path")
            self.backend.materialize(model, init_weights=False)
            self.checkpoint.load_pretrained(model, model_name_or_path)
            self._model_source = model_name_or_path
        else:
            seed = int(init_kwargs.get("seed", 0))
            self.runtime.manual_seed_all(seed)
            self.backend._init_seed = seed
            self.backend.materialize(model, init_weights=True)
        self.backend.finalize_model_load(model)
        model.on_materialized()
        leftover = has_meta_tensor(model)
        if leftover:
            raise RuntimeError(f"tensors still on the meta device after materialisation: {leftover[:5]}")
        return model

    def _make_coordinator(self):
        from .checkpoint import CheckpointCoordinator

        return CheckpointCoordinator(self.config, self.backend.create_checkpoint_manager(), plugins=self.plugins,
                                     parallel_context=self.backend.get_parallel_context())

    @property
    def checkpoint(self):
        if self._checkpoint is None:
            self._checkpoint = self._make_coordinator()
        return self._checkpoint

    def prepare_model(self, model_name_or_path: str | None = None, **kwargs: Any) -> nn.Module:
        model = self.build_model(model_name_or_path, **kwargs)
        self._apply_freeze_policy(model, self.config.freeze_policy)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
        self._log_info()
        self._log_model_info(model)
        return model

    # ------------------------------------------------------------------------------------------
    # plan resolution / freezing
    # ------------------------------------------------------------------------------------------
    def _resolve_parallel_plan(self, model: nn.Module) -> FSDPParallelPlan:
        """Model default plan overlaid with `EngineConfig.parallel_plan`: sizes override when given; per-FQN
        entries override field by field (only non-None fields of a partial spec); a vision-balance override may
        change the mode while inheriting the model's IO adapter."""
        base = copy.copy(type(model).get_default_parallel_plan())
        base.plan = dict(base.plan)
        over = self.config.parallel_plan
        if over is None:
            return base
        if over.sp_size is not None:
            base.sp_size = int(over.sp_size)
        if over.ep_size is not None:
            base.ep_size = int(over.ep_size)
        for fqn, ospec in (over.plan or {}).items():
            cur = base.plan.get(fqn)
            if cur is None:
                fields = {k: getattr(ospec, k) for k in vars(ospec)}
                fields = {k: v for k, v in fields.items() if v is not None}
                base.plan[fqn] = FSDPPlanSpec(**fields)
                continue
            merged = copy.copy(cur)
            for k, v in vars(ospec).items():
                if v is None or k == "vision_balance":
                    continue
                if k == "module_kwargs" and not v:
                    continue
                setattr(merged, k, v)
            ovb = getattr(ospec, "vision_balance", None)
            if ovb is not None:
                cvb = cur.vision_balance or VisionBalanceSpec()
                merged.vision_balance = VisionBalanceSpec(mode=ovb.mode if ovb.mode is not None else cvb.mode,
                                                          io=ovb.io if ovb.io is not None else cvb.io)
            base.plan[fqn] = merged
        return base

    def _apply_freeze_policy(self, model: nn.Module, policy: FreezePolicy) -> None:
        if not policy.enabled:
            return
        frozen = 0
        if policy.parameter_groups:
            groups = model.get_parameter_groups()
            for g in policy.parameter_groups:
                if g not in groups:
                    raise ValueError(f"{type(model).__name__} has no parameter group {g.value!r}")
                for _, p in groups[g]:
                    if p.requires_grad:
                        p.requires_grad_(False)
                        frozen += 1
        for name, p in model.named_parameters():
            if p.requires_grad and any(match_fqn(pat, name) for pat in policy.patterns):
                p.requires_grad_(False)
                frozen += 1
        logger.info_rank0("freeze policy: %d parameter tensor(s) frozen", frozen)

    # ------------------------------------------------------------------------------------------
    # optimizer / scheduler
    # ------------------------------------------------------------------------------------------
    def prepare_optimizer(self, model: nn.Module, optimizer_plan_or_cls=None, **kwargs: Any):
        """Accepts an `OptimizerPlan`, an `OptimizerClassPlan`, or an optimizer class plus hyper-parameters.
        With `config.optimizer.name == "muon"` the engine builds the Muon + AdamW pair from the model's recipe."""
        from .optimizers.plan import OptimizerClassPlan, OptimizerPlan

        if self.config.optimizer.name == "muon":
            from .optimizers.muon import build_muon_optimizer

            opt = build_muon_optimizer(model, self.config.optimizer.muon, self.backend, **kwargs)
        else:
            plan = optimizer_plan_or_cls
            if plan is None:
                plan = torch.optim.AdamW
            if not isinstance(plan, (OptimizerPlan, OptimizerClassPlan)):
                plan = OptimizerClassPlan(plan, **kwargs)
            opt = self.backend.prepare_optimizer(model, plan)
        self._optimizer = opt
        return opt

    def offload_optimizer(self) -> None:
        from .optimizers.memory import OptimizerMemoryController

        if self._optimizer is None:
            raise RuntimeError("no optimizer has been prepared")
        ctl = getattr(self, "_opt_memory", None) or OptimizerMemoryController(self._optimizer)
        self._opt_memory = ctl
        ctl.offload()

    def restore_optimizer(self) -> None:
        ctl = getattr(self, "_opt_memory", None)
        if ctl is not None:
            ctl.restore()

    def prepare_lr_scheduler(self, optimizer, scheduler_or_name="cosine", **kwargs: Any):
        from .optimizers.lr_scheduler import create_lr_scheduler

        if isinstance(scheduler_or_name, str):
            return create_lr_scheduler(scheduler_or_name, optimizer, **kwargs)
        return scheduler_or_name(optimizer, **kwargs)

    def clip_grad_norm_(self, model: nn.Module, max_norm: float, optimizer=None) -> torch.Tensor:
        return self.backend.clip_grad_norm_(model, max_norm, optimizer if optimizer is not None else self._optimizer)

    # ------------------------------------------------------------------------------------------
    # data
    # ------------------------------------------------------------------------------------------
    def get_dp_info(self) -> dict[str, Any]:
        return self.backend.get_dp_info()

    def get_sp_info(self) -> dict[str, Any]:
        return self.backend.get_sp_info()

    def get_ep_info(self) -> dict[str, Any]:
        return self.backend.get_ep_info()

    def _get_parallel_context(self) -> dict[str, Any]:
        return self.backend.get_parallel_context()

    @staticmethod
    def _ga_from_gbs(gbs: int, sp_size: int, world_size: int) -> int:
        num = gbs * sp_size
        if num % world_size:
            raise ValueError(f"gbs={gbs} x sp_size={sp_size} is not divisible by world_size={world_size}")
        return num // world_size

    def resolve_gradient_accumulation_steps(self, framework_ga: int = 1) -> int:
        """`gbs * sp / world` when a global batch size is configured, else the trainer's value times `sp`
        (the SP ranks of a group share one sample, so a group needs `sp` times more micro-steps)."""
        sp, W = self.backend.sp_size, self.backend.world_size
        if self.config.gbs is not None:
            return self._ga_from_gbs(self.config.gbs, sp, W)
        return int(framework_ga) * sp

    def create_dataloader(self, dataset, *, batch_size: int = 1, collate_fn: Callable | None = None, shuffle: bool = True,
                          seed: int = 0, drop_last: bool = True, gradient_accumulation_steps: int = 1,
                          num_workers: int = 0, pin_memory: bool = True, per_rank_shuffle: bool = False, **kw: Any):
        dp = self.backend.get_dp_info()
        for plugin in self.plugins.dataset_plugins():
            dataset = plugin.wrap_dataset(dataset) or dataset
        sampler = DPBlockDistributedSampler(dataset, dp["dp_size"], dp["dp_rank"],
                                            rank_block=batch_size * max(gradient_accumulation_steps, 1), shuffle=shuffle,
                                            seed=seed, drop_last=drop_last, per_rank_shuffle=per_rank_shuffle)
        return EpochDrivenDataLoader(dataset, batch_size=batch_size, sampler=sampler, collate_fn=collate_fn,
                                     num_workers=num_workers, pin_memory=pin_memory and torch.cuda.is_available(), **kw)

    # ------------------------------------------------------------------------------------------
    # loss / metrics
    # ------------------------------------------------------------------------------------------
    def compute_loss(self, model: nn.Module, inputs: dict[str, Any], *, num_items_in_batch=None,
                     gradient_accumulation_steps: int = 1, return_outputs: bool = False):
        inputs = model.on_prepare_inputs(dict(inputs), source_inputs=inputs)
        inputs = self.backend.prepare_inputs(model, inputs)
        self._record_micro(inputs)
        res = self.backend.compute_loss(model, inputs, num_items_in_batch=num_items_in_batch,
                                        aux_loss_scale=1.0 / max(gradient_accumulation_steps, 1),
                                        return_outputs=True)
        loss, out = res
        self._record_mtp_outputs(out)
        return (loss, out) if return_outputs else loss

    def compute_diffusion_loss(self, model: nn.Module, inputs: dict[str, Any], **kwargs: Any):
        inputs = self.backend.prepare_inputs(model, dict(inputs))
        return self.backend.compute_diffusion_loss(model, inputs, **kwargs)

    def collect_metrics(self, model: nn.Module) -> None:
        self.metrics.collect(model)

    def report_metrics(self, logs: dict, gather: Callable | None = None) -> dict:
        if self._mfu is not None:
            logs.update(self._mfu.pop())
        self.check_health()
        return self.metrics.report(logs, gather)

    def check_health(self) -> None:
        """Turn a timeout / overflow recorded by any rank's peer-memory kernels into an exception on every rank.
        Also orders the current stream after optimizer updates still running on their side stream, so that whatever
        follows (a checkpoint, an export) reads finished weights.
        Runs at logging and checkpoint boundaries (one small device read per workspace).  Inside a step the same
        status words poison the gradient norm on the device (`FSDP2Backend.clip_grad_norm_`), so the update of a
        failed step is skipped without a host read."""
        if self.runtime.turbo_device.value == "cuda":
            from .optimizers.fused_adamw import join_update_streams

            join_update_streams()
        if self.backend.world_size > 1 and self.runtime.turbo_device.value == "cuda":
            from .health import check_peer_status

            check_peer_status(what="peer-memory exchange since the last report")

    def recover_from_ep_overflow(self, optimizer=None) -> list[float]:
        """Collective recovery after `EPCapacityExceeded`: drop the gradients of the failed step, give the expert-parallel
        workspaces twice the receive capacity and clear the status words.  The caller then repeats the step (its
        optimizer update was skipped on every rank, so the weights are those from before the step)."""
        from ..comm.ep_p2p import grow_workspaces
        from .health import reset_peer_status

        be = self.backend
        if optimizer is not None:
            for o in getattr(optimizer, "optimizers", [optimizer]):
                if hasattr(o, "set_clip_coef"):
                    o.set_clip_coef(None)
                    o.grad_prescale = 1.0
                o.zero_grad(set_to_none=True)
        if hasattr(be, "_after_optimizer_step"):
            be._after_optimizer_step()       # flat gradient buffer of replicated layers
        torch.cuda.synchronize()
        grown = grow_workspaces(2.0)
        reset_peer_status(be)
        logger.warning_rank0("expert-parallel receive capacity exceeded: buffers grown to %s x the balanced share, step repeated",
                             ", ".join(f"{c:g}" for c in grown))
        return grown

    def close(self, model: nn.Module | None = None) -> None:
        """Orderly release of every peer-mapped (symmetric / multicast-bound) buffer this process holds: the flat
        gradient buffer of replicated layers, the FSDP arenas and the exchange workspaces.  Collective: every rank
        drops its buffers, drains its GPU and then meets the others at a barrier, so that no rank exits (or goes on to
        other work) while its memory is still bound into an NVLink multicast object that the others have mapped.
        The engine must not run another step afterwards."""
        import gc

        be = self.backend
        if model is not None:
            for p in model.parameters():
                if getattr(p, "main_grad", None) is not None and getattr(p.main_grad, "_tt_flat_owner", None) is not None:
                    p.main_grad = None
                    p.grad = None
        for name, empty in (("_rep_flat", None), ("_rep_symm", None), ("_rep_params", []), ("peer_arenas", [])):
            if hasattr(be, name):
                setattr(be, name, empty)
        if self.runtime.turbo_device.value == "cuda":
            from ..comm import ep_p2p, fsdp_p2p, rows_p2p, ulysses_p2p

            for table in (ep_p2p._WORKSPACES, fsdp_p2p._ARENAS, ulysses_p2p._WORKSPACES, rows_p2p._WS):
                table.clear()
            gc.collect()
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
        if dist.is_available() and dist.is_initialized() and be.world_size > 1:
            dist.barrier()

    def _get_mfu_estimator(self, model: nn.Module | None = None):
        if self._mfu is None and self.config.mfu.enabled and model is not None:
            recipe = model.get_flops_class()(model.config)
            self._mfu = MFUEstimator(recipe, self.config.mfu.card, self.runtime.turbo_device.value,
                                     self.config.activation_checkpointing.enabled, self.backend.world_size,
                                     self.backend.sp_size)
        return self._mfu

    def enable_mfu(self, model: nn.Module) -> None:
        self.config.mfu.enabled = True
        self._get_mfu_estimator(model)

    def _record_micro(self, inputs: Any) -> None:
        if self._mfu is not None:
            self._mfu.record_micro(inputs)

    def _record_mtp_outputs(self, out: dict[str, Any]) -> None:
        if not (self.config.mtp.enabled and self.config.mtp.log_loss):
            return
        mtp = [v for k, v in out.items() if k.startswith("mtp") and k.endswith("_loss") and v is not None]
        for i, v in enumerate(mtp, 1):
            self.metrics.add(f"mtp_loss/{i}", v)
        if mtp:
            avg = torch.stack([v.float() for v in mtp]).mean()
            self.metrics.add("mtp_loss/avg", avg)
            self.metrics.add("mtp_loss/scaled", avg * self.config.mtp.loss_scaling_factor)
            if out.get("main_loss") is not None:
                self.metrics.add("mtp_loss/main", out["main_loss"])

    # ------------------------------------------------------------------------------------------
    # checkpoint facade
    # ------------------------------------------------------------------------------------------
    def save_model(self, model: nn.Module, output_dir: str, *, final: bool = False, **kwargs: Any) -> None:
        self.check_health()   # never persist weights trained on a failed peer-memory exchange
        self.checkpoint.save_model(model, output_dir, final=final, source_path=self._model_source, **kwargs)

    def save_optimizer_and_scheduler(self, model, optimizer, scheduler, output_dir: str) -> None:
        self.check_health()
        self.checkpoint.save_optimizer_and_scheduler(model, optimizer, scheduler, output_dir)

    def load_optimizer_and_scheduler(self, model, optimizer, scheduler, checkpoint_dir: str) -> None:
        self.checkpoint.load_optimizer_and_scheduler(model, optimizer, scheduler, checkpoint_dir)

    def load_from_checkpoint(self, model: nn.Module, checkpoint_dir: str, **kwargs: Any) -> None:
        self.checkpoint.load_model(model, checkpoint_dir, **kwargs)

    # ------------------------------------------------------------------------------------------
    # profiling
    # ------------------------------------------------------------------------------------------
    def start_profiling(self, output_dir: str, *, profiling_enabled: bool = True,
                        memory_snapshot_steps: int | None = None) -> None:
        rank = dist.get_rank() if dist.is_initialized() else 0
        self._profiler = self.runtime.profiler(output_dir=output_dir, worker_name=f"rank{rank}_{socket.gethostname()}",
                                               profiling_enabled=profiling_enabled,
                                               memory_snapshot_steps=memory_snapshot_steps)
        self._profiler.start()

    def step_profiling(self) -> None:
        if self._profiler is not None:
            self._profiler.step()

    def stop_profiling(self) -> None:
        if self._profiler is not None:
            self._profiler.stop()
            self._profiler = None

    # ------------------------------------------------------------------------------------------
    # training loop
    # ------------------------------------------------------------------------------------------
    def fit(self, model: nn.Module, dataloader, optimizer, scheduler=None, **kwargs: Any):
        from ..loops.sft import run_training

        return run_training(self, model, dataloader, optimizer, scheduler, **kwargs)

    # ------------------------------------------------------------------------------------------
    # logging
    # ------------------------------------------------------------------------------------------
    def _log_info(self) -> None:
        try:
            logger.info_rank0("engine config:\n%s", json.dumps(self.config.to_dict(), indent=2, default=str))
        except Exception as e:  # configuration dumps must never break training
            logger.warning_rank0("could not serialise engine config: %s", e)
        self.ops.log_ops_selection()

    def _log_model_info(self, model: nn.Module) -> None:
        rows, total, trainable = [], 0, 0
        for name, p in model.named_parameters():
            n = p.numel()
            total += n
            trainable += n if p.requires_grad else 0
            if hasattr(p, "_local_tensor"):
                where = f"DTensor{tuple(p.placements)} mesh={tuple(p.device_mesh.mesh.shape)}"
            else:
                where = "local"
            rows.append(f"  {name:<70} {str(tuple(p.shape)):<24} {str(p.dtype).replace('torch.', ''):<9} {where}")
        head = f"model parameters: {total / 1e6:.1f}M total, {trainable / 1e6:.1f}M trainable"
        if len(rows) > 80:
            rows = rows[:40] + [f"  ... {len(rows) - 80} more ..."] + rows[-40:]
        logger.info_rank0("%s\n%s", head, "\n".join(rows))

    def __repr__(self) -> str:
        b = self.backend
        return (f"TorchTurboEngine(backend={self.config.backend.value}, world={b.world_size}, sp={b.sp_size}, "
                f"ep={b.ep_size}, precision={self.config.mixed_precision.value})")
