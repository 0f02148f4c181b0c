"""In-switch all-reduce (`multimem.ld_reduce` + `multimem.st`) of a symmetric fp32 buffer against a plain fp32 sum of
the ranks' inputs, on 2 GPUs (and 4 where present): sizes that are and are not multiples of the unrolled stride, the
scale folded in, a second call on the same buffer."""
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

        os.environ.update({"LOCAL_RANK": str(rank), "RANK": str(rank), "WORLD_SIZE": str(world)})
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=120), device_id=torch.device("cuda", rank))
        from torchturbo_b200 import kernels as K
        from torchturbo_b200.comm.symm import SymmetricBuffer

        for n in (4 * 1024, 4 * (296 * 512 * 4 + 37), 4 * 3_000_001):
            buf = SymmetricBuffer(n * 4 + 4096, dist.group.WORLD)
            if not buf.multicast_ptr:
                pytest.skip("no NVSwitch multicast on this system")
            off, flat = buf.carve(n * 4, torch.float32)
            before, after = buf.channel(), buf.channel()
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            for it in range(2):
                g = torch.Generator(device="cuda").manual_seed(100 * it + rank)
                mine = torch.randn(n, device="cuda", generator=g)
                flat.copy_(mine)
                parts = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(parts, mine)
                want = torch.stack(parts).sum(0) / world
                for ch, run in ((before, True), (after, False)):
                    e = ch.next()
                    K.flag_signal(buf.peer_ptrs, ch.offset, rank, world, e)
                    K.flag_wait(buf.peer_ptrs, ch.offset, rank, world, e, 5000, status)
                    if run:
                        K.multimem_allreduce_f32(buf.multicast_ptr + off, n, rank, world, 1.0 / world)
                torch.cuda.synchronize()
                err = (flat - want).abs().max().item()
                assert err < 1e-5, (n, it, err)
                assert int(status.item()) == 0
            del flat, buf
        dist.barrier()
        dist.destroy_process_group()
    except BaseException:
        with open(os.path.join(err_dir, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise


def _run(world):
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        try:
            mp.start_processes(_worker, args=(world, os.path.join(d, "rdzv"), d), nprocs=world, join=True, start_method="spawn")
        except Exception:
            errs = sorted(f for f in os.listdir(d) if f.endswith(".err"))
            if errs:
                text = open(os.path.join(d, errs[0])).read()
                if "Skipped" in text or "no NVSwitch multicast" in text:
                    pytest.skip("no NVSwitch multicast on this system")
                raise AssertionError(text)
            raise


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_in_switch_allreduce_two_ranks():
    _run(2)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_in_switch_allreduce_four_ranks():
    _run(4)
