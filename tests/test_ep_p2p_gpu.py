"""2-GPU check of the peer-memory expert-parallel dispatcher against the NCCL all-to-all dispatcher."""
import os
import sys
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
        from torchturbo_b200.models.modules.moe import MoELayer, MoELayerConfig

        torch.manual_seed(0)
        H, F, E, k = 256, 128, 16, 4
        base = dict(hidden_size=H, moe_ffn_hidden_size=F, num_moe_experts=E, moe_router_topk=k, params_dtype=torch.bfloat16)
        with torch.device("cuda"):
            a = MoELayer(MoELayerConfig(**base, moe_token_dispatcher_transport="nccl"), ep_group=dist.group.WORLD)
            b = MoELayer(MoELayerConfig(**base, moe_token_dispatcher_transport="p2p"), ep_group=dist.group.WORLD)
        assert type(b.token_dispatcher).__name__ == "P2PTokenDispatcher"
        with torch.no_grad():
            for pa, pb in zip(a.parameters(), b.parameters()):
                pb.copy_(pa)
        for step in range(3):
            torch.manual_seed(100 + 10 * step + rank)
            T = 300 + 57 * rank + step
            x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16()
            xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
            ya, _ = a(xa)
            yb, _ = b(xb)
            g = torch.randn_like(ya)
            ya.backward(g)
            yb.backward(g)
            torch.cuda.synchronize()
            b.token_dispatcher  # noqa: B018
            from torchturbo_b200.comm.ep_p2p import _WORKSPACES

            for ws in _WORKSPACES.values():
                ws.check()

            def close(u, v, what):
                err = (u.float() - v.float()).abs().max().item()
                ref = v.float().abs().max().item()
                assert err <= 3e-2 * max(ref, 1e-3), f"{what}: err {err} ref {ref} (rank {rank}, step {step})"

            close(yb, ya, "output")
            close(xb.grad, xa.grad, "dx")
            for (n, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
                close(pb.grad, pa.grad, n)
            a.zero_grad()
            b.zero_grad()
        assert kernels.comm_status() == (0, 0)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(err_dir, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_p2p_dispatcher_matches_nccl():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        try:
            mp.start_processes(_worker, args=(2, os.path.join(d, "rdzv"), d), nprocs=2, join=True, start_method="spawn")
        except Exception:
            errs = sorted(f for f in os.listdir(d) if f.endswith(".err"))
            if errs:
                raise AssertionError(open(os.path.join(d, errs[0])).read())
            raise
