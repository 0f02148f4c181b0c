"""2-GPU check of the peer-memory all-to-all-v of rows (vision-balance transport) against NCCL, forward and backward,
with growing buffers, empty sends and fp32 rows."""
import os
import tempfile
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, init_file, err_dir):
    try:
        import datetime

        import torch.distributed as dist

        os.environ["NCCL_NVLS_ENABLE"] = "0"
        os.environ["LOCAL_RANK"] = str(rank)
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=120), device_id=torch.device("cuda", rank))
        from torchturbo_b200 import kernels
        from torchturbo_b200.comm import rows_p2p
        from torchturbo_b200.models.modules.comm import all_to_all

        g = dist.group.WORLD
        cases = [([[3, 5], [7, 2]], 1176, torch.bfloat16), ([[0, 4], [0, 0]], 64, torch.float32),
                 ([[1500, 900], [2000, 100]], 1176, torch.bfloat16), ([[2, 2], [2, 2]], 8, torch.bfloat16)]
        for step, (m, H, dt) in enumerate(cases):
            torch.manual_seed(step * 10 + rank)
            n = sum(m[rank])
            x = torch.randn(n, H, device="cuda").to(dt)
            xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
            assert rows_p2p.usable(g, xa)
            ya = rows_p2p.p2p_all_to_all_rows(g, xa, m)
            out_splits, in_splits = [m[s][rank] for s in range(world)], m[rank]
            yb = all_to_all(g, xb, out_splits, in_splits)
            assert ya.shape == yb.shape and torch.equal(ya, yb), (step, rank)
            w = torch.randn_like(ya.float())
            (ya.float() * w).sum().backward()
            (yb.float() * w).sum().backward()
            torch.cuda.synchronize()
            if n:
                assert torch.equal(xa.grad, xb.grad), (step, rank)
            for ws in rows_p2p._WS.values():
                ws.check()
        assert kernels.comm_status() == (0, 0)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(err_dir, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_p2p_rows_matches_nccl():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        try:
            mp.start_processes(_worker, args=(2, os.path.join(d, "rdzv"), d), nprocs=2, join=True, start_method="spawn")
        except Exception:
            errs = sorted(f for f in os.listdir(d) if f.endswith(".err"))
            if errs:
                raise AssertionError(open(os.path.join(d, errs[0])).read())
            raise
