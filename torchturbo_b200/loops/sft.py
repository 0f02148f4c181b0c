"""The engine's own supervised fine-tuning / continued pre-training loop.

The reference leaves the loop to external trainers (LlamaFactory, ms-swift) and only overrides their hooks;
this engine ships the loop itself so that a model can be trained with nothing but this package:

    for each optimizer step:  GA micro-batches -> compute_loss -> backward   (aux-loss scale = 1/GA)
                              clip (global norm, EP aware) -> optimizer.step -> scheduler.step -> zero_grad
    periodically:             metrics (loss, grad norm, lr, tokens/s, MFU, router losses), checkpoints, profiler

Continued pre-training uses the same loop; the only difference is the data (every token is a target)."""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Any, Callable

import torch
import torch.distributed as dist

from ..engine.distributed import assert_finite
from ..logging import get_logger

logger = get_logger(__name__)


@dataclass
class TrainingArguments:
    max_steps: int = 100
    gradient_accumulation_steps: int = 1
    max_grad_norm: float = 1.0
    logging_steps: int = 10
    save_steps: int = 0
    output_dir: str | None = None
    resume_from_checkpoint: str | None = None
    check_finite: bool = True
    profiling: bool = False
    memory_snapshot_steps: int | None = None
    seed: int = 0


@dataclass
class TrainState:
    step: int = 0
    epoch: int = 0
    tokens_seen: int = 0
    history: list[dict[str, float]] = field(default_factory=list)


def _loss_multiplier(engine, num_items_in_batch) -> float:
    """The backend normalises each SP shard by `count * sp`; without a trainer-supplied global token count the
    loop multiplies by `sp` so that the world-average of gradients equals the data-parallel average."""
    return float(engine.backend.sp_size) if num_items_in_batch is None else 1.0


def train_step(engine, model, optimizer, micro_batches, *, max_grad_norm: float = 1.0, num_items_in_batch=None,
               check_finite: bool = True, ep_overflow_retries: int = 4):
    """One optimizer step over a list of micro-batches.  Returns (mean loss tensor, grad norm tensor).

    With `check_finite` the loss and the gradient norm are read on the host before the update; a step whose
    expert-parallel exchange overflowed a receive buffer is repeated with larger buffers (up to `ep_overflow_retries`
    times; each repeat doubles the capacity).  Without it nothing is read: a failed step skips its update on the device
    and the failure surfaces at the next `engine.check_health()` (logging / checkpoint boundaries)."""
    from ..comm.ep_p2p import EPCapacityExceeded

    ga = len(micro_batches)
    mult = _loss_multiplier(engine, num_items_in_batch)
    for attempt in range(1 + max(int(ep_overflow_retries), 0)):
        total = None
        for mb in micro_batches:
            loss = engine.compute_loss(model, mb, num_items_in_batch=num_items_in_batch, gradient_accumulation_steps=ga)
            (loss * (mult / ga)).backward()
            engine.collect_metrics(model)
            d = loss.detach().float() * mult
            total = d if total is None else total + d
        gnorm = engine.clip_grad_norm_(model, max_grad_norm, optimizer)
        if not check_finite:
            break
        try:
            # one host read for both; the norm is NaN on every rank when a peer-memory kernel of any rank failed
            assert_finite(torch.stack([total.reshape(()), gnorm.detach().float().reshape(())]), "loss or gradient norm")
            break
        except FloatingPointError:
            try:
                engine.check_health()     # names the failed exchange (timeout / receive overflow) when that is the cause
            except EPCapacityExceeded:
                # dropless routing without a worst-case buffer: no row of the overflowing layer was sent and no weight
                # has changed, so the receive buffers are doubled (on every rank, collectively) and the step is run again
                if attempt >= ep_overflow_retries:
                    raise
                del loss, total, gnorm, d
                engine.recover_from_ep_overflow(optimizer)
                continue
            raise
    optimizer.step()
    optimizer.zero_grad(set_to_none=True)
    return total / ga, gnorm


def run_training(engine, model, dataloader, optimizer, scheduler=None, args: TrainingArguments | None = None,
                 on_log: Callable[[dict], None] | None = None, **overrides: Any) -> TrainState:
    args = args or TrainingArguments()
    for k, v in overrides.items():
        setattr(args, k, v)
    ga = engine.resolve_gradient_accumulation_steps(args.gradient_accumulation_steps)
    state = TrainState()
    if args.resume_from_checkpoint:
        engine.load_from_checkpoint(model, args.resume_from_checkpoint)
        engine.load_optimizer_and_scheduler(model, optimizer, scheduler, args.resume_from_checkpoint)
        state.step = int(os.path.basename(os.path.normpath(args.resume_from_checkpoint)).rpartition("-")[2] or 0)
    if args.profiling or args.memory_snapshot_steps:
        engine.start_profiling(args.output_dir or ".", profiling_enabled=args.profiling,
                               memory_snapshot_steps=args.memory_snapshot_steps)
    model.train()
    it = iter(dataloader)
    t_last, tok_last = time.perf_counter(), 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    while state.step < args.max_steps:
        mbs = []
        while len(mbs) < ga:
            try:
                mbs.append(next(it))
            except StopIteration:
                state.epoch += 1
                if hasattr(dataloader, "set_epoch"):
                    dataloader.set_epoch(state.epoch)
                it = iter(dataloader)
        loss, gnorm = train_step(engine, model, optimizer, mbs, max_grad_norm=args.max_grad_norm,
                                 check_finite=args.check_finite)
        if scheduler is not None:
            scheduler.step()
        state.step += 1
        state.tokens_seen += sum(int(mb["input_ids"].numel()) for mb in mbs)
        engine.step_profiling()
        if args.logging_steps and state.step % args.logging_steps == 0:
            now = time.perf_counter()
            logs = {"step": state.step, "loss": float(loss), "grad_norm": float(gnorm),
                    "lr": optimizer.param_groups[0]["lr"],
                    "tokens_per_s_per_rank": (state.tokens_seen - tok_last) / max(now - t_last, 1e-9) / engine.backend.sp_size}
            engine.report_metrics(logs, gather=None)
            t_last, tok_last = now, state.tokens_seen
            state.history.append(logs)
            logger.info_rank0(" ".join(f"{k}={v:.6g}" if isinstance(v, float) else f"{k}={v}" for k, v in logs.items()))
            if on_log:
                on_log(logs)
        if args.save_steps and args.output_dir and (state.step % args.save_steps == 0 or state.step == args.max_steps):
            ckpt = os.path.join(args.output_dir, f"checkpoint-{state.step}")
            engine.save_model(model, ckpt, final=state.step == args.max_steps, step=state.step)
            engine.save_optimizer_and_scheduler(model, optimizer, scheduler, ckpt)
    engine.stop_profiling()
    return state
