"""2-GPU check of the peer-memory Ulysses exchange (QK-norm + RoPE + head scatter kernel, output gather) against the
NCCL all-to-all formulation of the same attention block."""
import os
import tempfile
import traceback
from types import SimpleNamespace

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
        from torchturbo_b200.comm import ulysses_p2p
        from torchturbo_b200.models.modules.transformer import Attention

        for n_kv in (2, 1):                                   # 2 kv heads: one per rank; 1 kv head: replicated twice
            cfg = SimpleNamespace(num_attention_heads=8, num_key_value_heads=n_kv, head_dim=128, hidden_size=256,
                                  rms_norm_eps=1e-6, attention_bias=False, qk_norm=True)
            torch.manual_seed(0)
            with torch.device("cuda"):
                a, b = Attention(cfg, 0, torch.bfloat16), Attention(cfg, 0, torch.bfloat16)
            with torch.no_grad():
                for m in (a, b):
                    m.q_norm.weight.uniform_(0.5, 1.5)
                    m.k_norm.weight.uniform_(0.5, 1.5)
                for pa, pb in zip(a.parameters(), b.parameters()):
                    pb.copy_(pa)
            a.set_sequence_parallel(dist.group.WORLD, world)
            b.set_sequence_parallel(dist.group.WORLD, world)
            Tl = 256
            T = Tl * world
            cu = torch.tensor([0, 300, T - 20], dtype=torch.int32)     # the last 20 tokens are padding
            pos = torch.arange(T, device="cuda")[rank * Tl:(rank + 1) * Tl].float()
            inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, device="cuda").float() / 128))
            ang = pos[:, None] * inv[None, :]
            cos, sin = ang.cos(), ang.sin()
            for step in range(2):
                torch.manual_seed(10 * step + rank)
                x = (torch.randn(Tl, 256, device="cuda") * 0.5).bfloat16()
                xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
                os.environ["TORCHTURBO_ULYSSES_TRANSPORT"] = "nccl"
                ya = a(xa, cos, sin, cu, 300)
                os.environ["TORCHTURBO_ULYSSES_TRANSPORT"] = "auto"
                assert ulysses_p2p.usable(dist.group.WORLD, torch.empty(1, device="cuda", dtype=torch.bfloat16), 8, n_kv, 128)
                yb = b(xb, cos, sin, cu, 300)
                g = torch.randn_like(ya)
                ya.backward(g)
                yb.backward(g)
                torch.cuda.synchronize()
                for ws in ulysses_p2p._WORKSPACES.values():
                    ws.check()

                def close(u, v, what):
                    err = (u.float() - v.float()).abs().max().item()
                    ref = v.float().abs().max().item()
                    assert err <= 3e-2 * max(ref, 1e-3), f"{what}: err {err} ref {ref} (rank {rank}, step {step}, kv {n_kv})"

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
def test_p2p_ulysses_matches_nccl():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        try:
            mp.start_processes(_worker, args=(2, os.path.join(d, "rdzv"), d), nprocs=2, join=True, start_method="spawn")
        except Exception:
            errs = sorted(f for f in os.listdir(d) if f.endswith(".err"))
            if errs:
                raise AssertionError(open(os.path.join(d, errs[0])).read())
            raise
