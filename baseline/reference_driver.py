"""Runs the headline benchmark through the *unmodified* reference package (installed under `baseline/_ref`).

The reference owns no training loop and no dense-model launcher, so this driver does what its trainer adapters do,
through its public API only: `TorchTurboEngine(EngineConfig)` -> `build_model(load_weights=False)` (meta build, plan,
FSDP2 sharding, materialisation) -> seeded normal(0, 0.02) initialisation (the reference materialises with
`to_empty`) -> `prepare_optimizer(torch.optim.AdamW)` -> per step `compute_loss`, `backward`,
`backend.clip_grad_norm_`, `optimizer.step`.  The only thing added around the package is a stand-in for the
`omegaconf` import (not installable offline; the config-merge code that uses it is not on this path).
The batch, model shape, optimizer settings, timing protocol and JSON line are the same as in the other arm.
"""
from __future__ import annotations

import os
import sys


def run(args, ref_dir: str) -> dict:
    here = os.path.dirname(os.path.abspath(__file__))
    if not os.path.isdir(os.path.join(ref_dir, "torchturbo")):
        return {"impl": "reference", "unavailable": "baseline/_ref/torchturbo is not installed on this machine"}
    sys.path[:0] = [os.path.join(here, "shims"), ref_dir]
    import torch
    import torch.distributed as dist

    from bench import METRIC, ClockSampler, model_config

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29512")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        dist.init_process_group("nccl" if use_cuda else "gloo")

    from transformers import Qwen3MoeConfig

    from torchturbo.engine.config import ActivationCheckpointingConfig, EngineConfig, MixedPrecisionPolicy, MoEConfig
    from torchturbo.engine.core import TorchTurboEngine
    from torchturbo.parallel import FSDPParallelPlan

    layers = args.layers or min(48, 12 * world)
    mc = model_config(args.model, layers)
    mc.pop("model_type")
    hf = Qwen3MoeConfig(**mc)
    cfg = EngineConfig(
        mixed_precision=MixedPrecisionPolicy.BF16 if use_cuda else MixedPrecisionPolicy.FP32,
        parallel_plan=FSDPParallelPlan(sp_size=1, ep_size=world),
        moe=MoEConfig(aux_loss_coeff=1e-3),
        activation_checkpointing=ActivationCheckpointingConfig(enabled=False),
    )
    engine = TorchTurboEngine(cfg)
    model = engine.build_model(None, init_kwargs={"config": hf}, load_weights=False)
    torch.manual_seed(0)
    with torch.no_grad():
        for name, p in model.named_parameters():
            lp = p._local_tensor if hasattr(p, "_local_tensor") else p
            if lp.ndim <= 1:
                lp.fill_(1.0) if "norm" in name else lp.zero_()
            else:
                lp.normal_(0.0, 0.02)
    engine.model = model
    optim = engine.prepare_optimizer(torch.optim.AdamW, lr=1e-5, weight_decay=0.01, betas=(0.9, 0.95))

    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset

    n_batches = args.warmup + 2 * args.steps
    ds = SyntheticPackedDataset(n_batches * world, args.seq_len, mc["vocab_size"], min_doc=256, max_doc=args.seq_len, seed=1234)
    coll = PackedCollator(pin=use_cuda)
    host = [coll([ds[rank * n_batches + i]]) for i in range(n_batches)]
    dev = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")

    def to_device(b):
        # the reference's trainers hand it batches that HF `Trainer._prepare_inputs` moved to the device as a whole,
        # packed boundaries included
        return {k: (v.to(dev, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in b.items()}

    def step(b):
        loss = engine.compute_loss(model, b)
        loss.backward()
        engine.backend.clip_grad_norm_(list(model.parameters()), 1.0)
        optim.step()
        optim.zero_grad(set_to_none=True)
        return loss.detach()

    def sync():
        if world > 1:
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()

    model.train()
    for i in range(args.warmup):
        step(to_device(host[i]))
    staged = [to_device(host[args.warmup + i]) for i in range(args.steps)]
    sampler = ClockSampler(local_rank)
    sync()
    if not use_cuda:
        import time

        t0 = time.perf_counter()
        for b in staged:
            last = step(b)
        ms = (time.perf_counter() - t0) * 1e3
        clocks, e2e = {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["cpu run"]}, None
    else:
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for b in staged:
            last = step(b)
        e1.record()
        sync()
        clocks = sampler.stop()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        losses = []
        sync()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for i in range(args.steps):
            losses.append(float(step(to_device(host[args.warmup + args.steps + i])).cpu()))
        f1.record()
        sync()
        t2 = torch.tensor([f0.elapsed_time(f1)], device=dev)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        h2d = sum(v.numel() * v.element_size() for k, v in host[0].items() if isinstance(v, torch.Tensor) and not k.startswith("cu_seq"))
        e2e = {"value": args.seq_len * world * args.steps / (float(t2.item()) / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4, "ms_per_step": float(t2.item()) / args.steps,
               "final_loss": losses[-1]}
    tokens_per_step = args.seq_len * world
    out = {
        "metric": METRIC, "value": tokens_per_step * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if use_cuda else "fp32",
        "data": "synthetic (seeded random token ids, random-init weights)", "impl": "reference",
        "config": {"model": "Qwen3-30B-A3B" if args.model == "qwen3_moe_30b_a3b" else args.model, "layers": layers,
                   "layers_named": 48, "global_batch": world, "seq_len": args.seq_len,
                   "parallelism": f"fsdp2 dp{world} + ep{world}", "optimizer": "AdamW (torch) on fp32 FSDP shards"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": None, "loss": float(last),
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30 if use_cuda else None,
    }
    if world > 1:
        dist.barrier()
    return out if rank == 0 else {}
