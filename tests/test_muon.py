import math

import torch

from dist_utils import run_distributed
from torchturbo_b200.engine.optimizers.muon import (DistributedMuon, MuonParameterSpec, adjusted_lr, newton_schulz)


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    G = torch.randn(2, 64, 32)
    X = newton_schulz(G, 8, (3.4445, -4.7750, 2.0315), 1e-7).float()
    s = torch.linalg.svdvals(X)
    assert s.max() < 1.35 and s.min() > 0.5      # singular values pushed towards one


def test_spec_views_cover_tensor():
    full = torch.arange(4 * 6 * 8.0).view(24, 8)
    spec = MuonParameterSpec(batch=4, col_blocks=(3, 5))
    ms = spec.matrices(full)
    assert [tuple(m.shape) for m in ms] == [(4, 6, 3), (4, 6, 5)]
    spec = MuonParameterSpec(row_blocks=(16, 4, 4))
    assert [tuple(m.shape) for m in spec.matrices(full)] == [(1, 16, 8), (1, 4, 8), (1, 4, 8)]


def test_adjusted_lr():
    assert adjusted_lr(1.0, 64, 16, "original") == 2.0
    assert abs(adjusted_lr(1.0, 64, 16, "match_rms_adamw") - 0.2 * 8) < 1e-9
    assert adjusted_lr(1.0, 16, 64, "spectral_unclamped") == 0.5


def _w_muon(rank, world):
    """Sharded Muon must produce the same parameters as single-rank Muon on the full matrices."""
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    torch.manual_seed(0)
    shapes = [(48, 16), (32, 32), (20, 24)]
    specs = [MuonParameterSpec(row_blocks=(32, 8, 8)), MuonParameterSpec(), MuonParameterSpec(batch=2)]
    fulls = [torch.randn(s) for s in shapes]
    grads = [[torch.randn(s) for s in shapes] for _ in range(3)]
    ref_p = [torch.nn.Parameter(f.clone()) for f in fulls]
    ref = DistributedMuon([(f"p{i}", p, s) for i, (p, s) in enumerate(zip(ref_p, specs))], lr=0.1, weight_decay=0.01)
    ref.world, ref.rank = 1, 0
    mesh = init_device_mesh("cpu", (world,))
    sh_p = [torch.nn.Parameter(distribute_tensor(f.clone(), mesh, [Shard(0)])) for f in fulls]
    opt = DistributedMuon([(f"p{i}", p, s) for i, (p, s) in enumerate(zip(sh_p, specs))], lr=0.1, weight_decay=0.01)
    assert {e.owner for e in opt.entries} == {0, 1}
    for step in range(3):
        for p, g in zip(ref_p, grads[step]):
            p.grad = g.clone()
        ref.step()
        for p, g in zip(sh_p, grads[step]):
            p.grad = distribute_tensor(g.clone(), mesh, [Shard(0)])
        opt.step()
    for a, b in zip(ref_p, sh_p):
        assert torch.allclose(a.detach(), b.full_tensor(), rtol=2e-2, atol=2e-3), (a - b.full_tensor()).abs().max()


def test_distributed_muon_matches_single_rank():
    run_distributed(_w_muon, 2)


def _w_muon_pipeline(rank, world):
    """The two-slot pipeline (asynchronous exchanges overlapped with Newton-Schulz) must give bit-identical parameters to
    running the three phases of every bucket back to back, with several buckets in flight."""
    import os

    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    shapes = [(48, 16), (32, 32), (20, 24), (64, 8), (16, 16), (40, 12), (24, 24)]
    mesh = init_device_mesh("cpu", (world,))
    results = []
    for mode in ("0", "1"):
        os.environ["TORCHTURBO_MUON_PIPELINE"] = mode
        torch.manual_seed(0)
        fulls = [torch.randn(s) for s in shapes]
        params = [torch.nn.Parameter(distribute_tensor(f.clone(), mesh, [Shard(0)])) for f in fulls]
        opt = DistributedMuon([(f"p{i}", p, MuonParameterSpec()) for i, p in enumerate(params)], lr=0.1, weight_decay=0.01,
                              bucket_cap_mb=0.002)          # ~2 KB per bucket: several buckets
        assert len(opt.buckets) >= 3
        for step in range(2):
            for p, f in zip(params, fulls):
                p.grad = distribute_tensor(torch.randn(f.shape, generator=torch.Generator().manual_seed(step)), mesh, [Shard(0)])
            opt.step()
        results.append([p.full_tensor().clone() for p in params])
    os.environ.pop("TORCHTURBO_MUON_PIPELINE", None)
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_muon_pipeline_matches_phase_by_phase_execution():
    run_distributed(_w_muon_pipeline, 2)
