"""Spawn helpers for multi-process CPU tests: gloo backend, file rendezvous, bounded run time."""
import os
import sys
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, fn, init_file, args, err_dir):
    try:
        os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"] = str(rank), str(world), str(rank)
        import datetime

        from torchturbo_b200.runtime import CpuRuntime, set_device_runtime

        set_device_runtime(CpuRuntime())
        dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=60))
        torch.manual_seed(0)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(err_dir, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise


def run_distributed(fn, world: int, *args, timeout: float = 240.0):
    """Run `fn(rank, world, *args)` on `world` CPU ranks; raises with the first rank's traceback on failure."""
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "rdzv")
        ctx = mp.start_processes(_entry, args=(world, fn, init_file, args, d), nprocs=world, join=False,
                                 start_method="spawn")
        import time

        t0 = time.time()
        ok = False
        try:
            while not ctx.join(timeout=1.0):
                if time.time() - t0 > timeout:
                    for p in ctx.processes:
                        if p.is_alive():
                            p.terminate()
                    raise TimeoutError(f"distributed test exceeded {timeout}s")
            ok = True
        except Exception:
            errs = sorted(f for f in os.listdir(d) if f.endswith(".err"))
            if errs:
                raise AssertionError(open(os.path.join(d, errs[0])).read())
            raise
        return ok
