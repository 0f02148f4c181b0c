"""World-pooled vision balancing: deterministic LPT assignment, exchange plans, and the distributed forward/backward
against the unbalanced tower (including an SP group whose members share a batch, a rank without media, and the
small-pool fallback)."""
import torch
import torch.nn as nn

from dist_utils import run_distributed
from torchturbo_b200.models.modules.vision.balance import FanoutPlan, MediaPool, PixelPlan, lpt_weight, register_vision_balance
from torchturbo_b200.models.modules.vision.io import GridVisionBalanceIO
from torchturbo_b200.parallel import VisionBalanceMode, VisionBalanceSpec


def test_lpt_assignment_is_deterministic_and_balanced():
    meta = [[[1, 8, 8, 16], [1, 2, 2, 1]], [], [[1, 4, 4, 4], [1, 4, 4, 4], [1, 6, 6, 9]], []]
    pool = MediaPool.from_metadata(meta, ("pooler_output",), VisionBalanceMode.PATCH_SQ)
    assert len(pool) == 5 and lpt_weight(64, VisionBalanceMode.PATCH_SQ) == 4096 and lpt_weight(64, VisionBalanceMode.PATCH) == 64
    pool.assign_owners(4)
    owners = [m.owner for m in pool.media]
    pool2 = MediaPool.from_metadata(meta, ("pooler_output",), VisionBalanceMode.PATCH_SQ)
    pool2.assign_owners(4)
    assert owners == [m.owner for m in pool2.media]
    assert owners[0] == 0 and owners[4] == 1                      # heaviest first, ties to the lower rank
    assert max(pool.loads(4)) == 4096 and sorted(set(owners)) == [0, 1, 2, 3]
    plan = PixelPlan.build(pool, 2, 4)
    assert sum(plan.send_splits) == 16 + 16 + 36 and sum(PixelPlan.build(pool, 1, 4).send_splits) == 0
    fan = FanoutPlan.build(pool, "pooler_output", 0, 4, sp_size=2)
    # rank 0 owns image (src 0, 8x8): its 16 output rows go to both members of SP group 0
    assert fan.send_splits[0] == 16 and fan.send_splits[1] == 16 and fan.send_splits[2] == 0
    assert len(fan.restore) == 16 + 1                               # group 0 receives both of its images' rows


class TinyTower(nn.Module):
    """Per-patch linear + per-image mean mixing, 2x2 merge: enough structure that wrong routing changes the output."""

    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.proj = nn.Linear(6, 4)

    def forward(self, pixel_values, grid_thw=None):
        h = self.proj(pixel_values)
        out, a = [], 0
        for t, hh, ww in grid_thw.tolist():
            n = int(t * hh * ww)
            seg = h[a:a + n]
            seg = seg + seg.mean(0, keepdim=True)
            out.append(seg.view(n // 4, 4, 4).sum(1))
            a += n
        return torch.cat(out, 0)


def _media(rank, sp_size, n_images_by_group):
    """Members of an SP group hold identical media; a group may have none."""
    group = rank // sp_size
    g = torch.Generator().manual_seed(100 + group)
    sizes = n_images_by_group[group]
    grids = torch.tensor([[1, s, s] for s in sizes], dtype=torch.long).view(-1, 3)
    P = int(sum(s * s for s in sizes))
    return torch.randn(P, 6, generator=g), grids


def _balance_worker(rank, world, sp_size, sizes_by_group):
    import torch.distributed as dist

    pix, grid = _media(rank, sp_size, sizes_by_group)
    ref_tower, tower = TinyTower(), TinyTower()
    if pix.shape[0] == 0:                                         # the data pipeline supplies a dummy image
        pix, grid = torch.zeros(4, 6), torch.tensor([[1, 2, 2]])
        has_media = False
    else:
        has_media = True
    pr = pix.clone().requires_grad_(False)
    ref = ref_tower(pr, grid_thw=grid)
    w = torch.linspace(0.5, 1.5, ref.numel()).view_as(ref)
    (ref * w).sum().backward()
    sp_groups = [dist.new_group(list(range(g * sp_size, (g + 1) * sp_size))) for g in range(world // sp_size)]
    spec = VisionBalanceSpec(mode=VisionBalanceMode.PATCH_SQ, io=GridVisionBalanceIO(2))
    state = register_vision_balance(tower, spec, sp_group=sp_groups[rank // sp_size], sp_size=sp_size, sp_rank=rank % sp_size,
                                    world_group=dist.group.WORLD)
    out = tower(pix, grid_thw=grid)
    assert out.shape == ref.shape and torch.allclose(out, ref, atol=1e-5), (out - ref).abs().max()
    (out * w).sum().backward()
    # parameter gradients: every image's contribution is computed once per SP member on its owner; summed over the
    # world they equal the sum of the unbalanced per-rank gradients
    g_bal, g_ref = tower.proj.weight.grad.clone(), ref_tower.proj.weight.grad.clone()
    if not has_media:
        g_ref.zero_()                                             # the dummy image's own loss is not part of the batch
    dist.all_reduce(g_bal)
    dist.all_reduce(g_ref)
    if has_media or True:
        assert torch.allclose(g_bal, g_ref, atol=1e-4), (g_bal - g_ref).abs().max()
    return state


def test_balanced_tower_matches_local_tower_world4_sp2():
    run_distributed(_balance_worker, 4, 2, [[8, 2, 4], [4, 6]])


def _fallback_worker(rank, world):
    import torch.distributed as dist

    tower = TinyTower()
    spec = VisionBalanceSpec(mode=VisionBalanceMode.PATCH, io=GridVisionBalanceIO(2))
    state = register_vision_balance(tower, spec, sp_group=None, sp_size=1, sp_rank=0, world_group=dist.group.WORLD)
    pix, grid = (torch.randn(16, 6), torch.tensor([[1, 4, 4]])) if rank == 0 else (torch.zeros(4, 6), torch.tensor([[1, 2, 2]]))
    # pool of 2 media == world: balanced; then a no-grad call must stay local
    out = tower(pix, grid_thw=grid)
    assert out.shape[0] == pix.shape[0] // 4 and state.last_pool is not None
    state.last_pool = None
    with torch.no_grad():
        tower(pix, grid_thw=grid)
    assert state.last_pool is None


def test_no_grad_keeps_the_local_path():
    run_distributed(_fallback_worker, 2)
