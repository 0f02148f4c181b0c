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


def _register_dense_qwen3():
    """The reference registers no dense Qwen3 model, and its engine only builds registered `TurboModel` classes.  This
    registers Hugging Face's `Qwen3ForCausalLM` through the reference's public extension points (`register_model`,
    the `TurboModel` hooks, an `FSDPParallelPlan`), the same way its own `qwen3_moe` wrapper does for the MoE class:
    embeddings and head as stand-alone world-sharded units, every decoder layer a checkpointed unit, Ulysses attention
    interface registered for the sequence-parallel group, rotary frequencies rebuilt after materialisation.
    Returns the config class."""
    import torch
    from transformers import AutoModelForCausalLM
    from transformers.models.qwen3.modeling_qwen3 import Qwen3Config, Qwen3ForCausalLM

    from torchturbo.models.base import TurboModel
    from torchturbo.models.registry import get_model, register_model
    from torchturbo.parallel import FSDPParallelPlan, FSDPPlanSpec
    from torchturbo.runtime import get_device_runtime

    if get_model("qwen3") is not None:
        return Qwen3Config

    @register_model("qwen3", config_cls=Qwen3Config, auto_class=AutoModelForCausalLM)
    class TurboQwen3ForCausalLM(TurboModel, Qwen3ForCausalLM):
        config_class = Qwen3Config
        base_model_prefix = "model"

        @classmethod
        def get_default_parallel_plan(cls, **kwargs):
            return FSDPParallelPlan(plan={
                "model.layers.*": FSDPPlanSpec(activation_checkpoint=True),
                "model.embed_tokens": FSDPPlanSpec(standalone_world_shard=True),
                "lm_head": FSDPPlanSpec(standalone_world_shard=True),
            }, sp_size=1, ep_size=1)

        def on_parallelized(self, parallel_context):
            self.register_sp_attention_interface(parallel_context["sp"])

        def on_materialized(self):
            rotary = self.model.rotary_emb
            inv_freq, rotary.attention_scaling = rotary.compute_default_rope_parameters(rotary.config, get_device_runtime().device)
            rotary.register_buffer("inv_freq", inv_freq.to(torch.bfloat16), persistent=False)
            rotary.register_buffer("original_inv_freq", inv_freq.to(torch.bfloat16).clone(), persistent=False)

    return Qwen3Config


def run(args, ref_dir: str) -> dict:
    here = os.path.dirname(os.path.abspath(__file__))
    if not os.path.isdir(os.path.join(ref_dir, "torchturbo")):
        return {"impl": "reference", "unavailable": "baseline/_ref/torchturbo is not installed on this machine"}
    sys.path[:0] = [os.path.join(here, "shims"), ref_dir]
    import torch
    import torch.distributed as dist

    from bench import METRIC, ClockSampler, model_config, stabilise

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

    from torchturbo.engine.config import ActivationCheckpointingConfig, EngineConfig, MixedPrecisionPolicy, MoEConfig
    from torchturbo.engine.core import TorchTurboEngine
    from torchturbo.parallel import FSDPParallelPlan

    is_moe = args.model in ("qwen3_moe_30b_a3b", "tiny_moe")
    named_layers = {"qwen3_moe_30b_a3b": 48, "qwen3_8b": 36, "qwen3_14b": 40}.get(args.model, 4)
    layers = args.layers or min(named_layers, 12 * world)
    sp = max(int(getattr(args, "sp", 1)), 1)
    mc = model_config(args.model, layers)
    mc.pop("model_type")
    if is_moe:
        from transformers import Qwen3MoeConfig

        hf = Qwen3MoeConfig(**mc)
    else:
        hf = _register_dense_qwen3()(**mc)
    cfg = EngineConfig(
        mixed_precision=MixedPrecisionPolicy.BF16 if use_cuda else MixedPrecisionPolicy.FP32,
        parallel_plan=FSDPParallelPlan(sp_size=sp, ep_size=world if is_moe else 1),
        moe=MoEConfig(aux_loss_coeff=1e-3 if is_moe else 0.0),
        activation_checkpointing=ActivationCheckpointingConfig(enabled=not is_moe),
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

    n_batches = max(args.warmup, 1) + 2 * args.steps
    ds = SyntheticPackedDataset(n_batches * world, args.seq_len, mc["vocab_size"], min_doc=256, max_doc=args.seq_len, seed=1234)
    coll = PackedCollator(pin=use_cuda)
    host = [coll([ds[(rank // sp) * n_batches + i]]) for i in range(n_batches)]   # an SP group shares its row
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
    # same rule as the other arm: keep warming up until two consecutive steps agree within 3 % (bounded)
    warmup_used = args.warmup + (stabilise(lambda j: step(to_device(host[j % max(args.warmup, 1)])), sync, world, dev,
                                           4 if getattr(args, "child", False) else 12) if use_cuda else 0)
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
        e2e = {"value": args.seq_len * (world // sp) * args.steps / (float(t2.item()) / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4, "ms_per_step": float(t2.item()) / args.steps,
               "final_loss": losses[-1]}
    tokens_per_step = args.seq_len * (world // sp)
    out = {
        "metric": METRIC if args.model == "qwen3_moe_30b_a3b" else METRIC.replace("Qwen3-30B-A3B FSDP2+EP", args.model), "value": tokens_per_step * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if use_cuda else "fp32",
        "data": "synthetic (seeded random token ids, random-init weights)", "impl": "reference",
        "config": {"model": "Qwen3-30B-A3B" if args.model == "qwen3_moe_30b_a3b" else args.model, "layers": layers,
                   "layers_named": named_layers, "global_batch": world // sp, "seq_len": args.seq_len,
                   "parallelism": f"fsdp2 dp{world // sp} + ep{world if is_moe else 1}" + (f" + ulysses sp{sp}" if sp > 1 else ""),
                   "activation_checkpointing": not is_moe, "optimizer": "AdamW (torch) on fp32 FSDP shards"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": None, "loss": float(last), "warmup_used": warmup_used,
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30 if use_cuda else None,
    }
    if world > 1:
        dist.barrier()
    return out if rank == 0 else {}
