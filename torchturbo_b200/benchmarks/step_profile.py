"""Where one training step spends its time: CPU issue time per step (host-bound or not) and the torch profiler's
per-kernel device time of one step of the flagship model at a reduced depth.

    python -m torchturbo_b200.benchmarks.step_profile [--layers 4] [--model qwen3_moe_30b_a3b] [--seq-len 4096] [--rows 40] [--sort self_cpu_time_total]
    torchrun --nproc-per-node N -m torchturbo_b200.benchmarks.step_profile ...     # expert parallel over N ranks, rank 0 prints
"""
from __future__ import annotations

import argparse
import sys
import time
from pathlib import Path

import torch


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--model", default="qwen3_moe_30b_a3b")
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=40)
    ap.add_argument("--sort", default="cuda_time_total", help="profiler sort key, e.g. self_cpu_time_total")
    ap.add_argument("--cprofile", type=int, default=0, help="also print the N host functions with the most own time (cProfile over 3 steps)")
    args = ap.parse_args(argv)
    sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
    from bench import model_config  # the benchmark's model table (repository root)

    from ..data import PackedCollator, SyntheticPackedDataset
    from ..engine import EngineConfig, TorchTurboEngine
    from ..engine.optimizers import OptimizerClassPlan
    from ..loops import train_step

    import os

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    is_moe = "moe" in args.model
    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "bf16", "moe": {"aux_loss_coeff": 1e-3},
                                                   "parallel_plan": {"sp_size": 1, "ep_size": world if is_moe else 1},
                                                   "activation_checkpointing": {"enabled": False}}))
    mc = model_config(args.model, args.layers)
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": mc})
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-5))
    ds = SyntheticPackedDataset(8, args.seq_len, mc["vocab_size"], min_doc=256, max_doc=args.seq_len, seed=1)
    batches = []
    for i in range(6):
        b = PackedCollator()([ds[i]])
        batches.append({k: (v.cuda() if isinstance(v, torch.Tensor) and not k.startswith("cu_seq") else v) for k, v in b.items()})
    for i in range(3):
        # warm-up reads the loss on the host: a step whose expert exchange overflows is repeated with larger buffers
        train_step(eng, model, opt, [batches[i]], check_finite=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(3):
        train_step(eng, model, opt, [batches[3 + i]], check_finite=False)
    t1 = time.perf_counter()
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    if rank == 0:
        print(f"cpu issue time per step {(t1 - t0) / 3 * 1e3:.1f} ms, total per step {(t2 - t0) / 3 * 1e3:.1f} ms")
    if args.cprofile:
        import cProfile
        import io
        import pstats

        pr = cProfile.Profile()
        pr.enable()
        for i in range(3):
            train_step(eng, model, opt, [batches[3 + i]], check_finite=False)
        pr.disable()
        torch.cuda.synchronize()
        if rank == 0:
            buf = io.StringIO()
            pstats.Stats(pr, stream=buf).sort_stats("tottime").print_stats(args.cprofile)
            print(buf.getvalue())
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        train_step(eng, model, opt, [batches[0]], check_finite=False)
        torch.cuda.synchronize()
    eng.check_health()
    if rank == 0:
        print(prof.key_averages().table(sort_by=args.sort, row_limit=args.rows, max_name_column_width=70))
    del opt
    eng.close(model)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
