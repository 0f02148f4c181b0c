"""CPU / gloo multi-process tests of the engine: FSDP2 dense training, EP MoE, SP (Ulysses) parity."""
import copy

import pytest
import torch

from dist_utils import run_distributed

DENSE = dict(model_type="qwen3", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
             head_dim=16, intermediate_size=128, vocab_size=512, tie_word_embeddings=True)
MOE = dict(model_type="qwen3_moe", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
           head_dim=16, intermediate_size=128, moe_intermediate_size=32, num_experts=8, num_experts_per_tok=2,
           vocab_size=512)


def _train(rank, world, mc, plan, steps, same_data, out_q=None, ac=False, backend_config=None, different_data=False):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "parallel_plan": plan,
                                                   "moe": {"aux_loss_coeff": 1e-2},
                                                   "activation_checkpointing": {"enabled": ac},
                                                   **({"backend_config": backend_config} if backend_config else {})}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(mc), "seed": 0})
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-2, weight_decay=0.0))
    ds = SyntheticPackedDataset(steps * world, 64, mc["vocab_size"], num_docs=3, seed=5)
    losses = []
    dp = eng.get_dp_info()
    for i in range(steps):
        idx = i if same_data else i * dp["dp_size"] + dp["dp_rank"]
        b = PackedCollator()([ds[idx]])
        loss, gn = train_step(eng, model, opt, [b])
        losses.append((float(loss), float(gn)))
    return losses, model, eng


def _w_dense(rank, world):
    import torch.distributed as dist

    losses, model, eng = _train(rank, world, DENSE, {"sp_size": 1, "ep_size": 1}, 4, same_data=True)
    sharded = any(hasattr(p, "_local_tensor") for p in model.parameters())
    assert sharded == (world > 1), "units are FSDP-sharded exactly when their mesh has more than one rank"
    # identical data on every rank => identical to the single-process run
    t = torch.tensor([l for l, _ in losses])
    ref = t.clone()
    dist.broadcast(ref, 0)
    assert torch.allclose(t, ref)
    assert losses[-1][0] < losses[0][0] + 0.5
    g = torch.tensor(losses)
    torch.save(g, f"/tmp/tt_dense_world{world}.pt") if rank == 0 else None


def test_fsdp2_dense_world2_matches_single_process():
    run_distributed(_w_dense, 1)
    run_distributed(_w_dense, 2)
    a, b = torch.load("/tmp/tt_dense_world1.pt"), torch.load("/tmp/tt_dense_world2.pt")
    assert torch.allclose(a, b, rtol=1e-4, atol=1e-5), (a, b)


def _w_replicated(rank, world, kind, replicate):
    """Different data per rank, two micro-batches per step: replicated decoder layers (flat gradient buffer, one
    all-reduce per step) must train exactly like FSDP-sharded ones."""
    import torch.distributed as dist

    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    mc = DENSE if kind == "dense" else MOE
    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "moe": {"aux_loss_coeff": 1e-2},
                                                   "parallel_plan": {"sp_size": 1, "ep_size": world if kind == "moe" else 1},
                                                   "activation_checkpointing": {"enabled": False},
                                                   "backend_config": {"replicate_layers": replicate}}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(mc), "seed": 0})
    assert bool(eng.backend.replicated_units) == replicate
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-2, weight_decay=0.0))
    ds = SyntheticPackedDataset(32, 64, mc["vocab_size"], num_docs=3, seed=5)
    out = []
    for i in range(3):
        mbs = [PackedCollator()([ds[(2 * i + j) * world + rank]]) for j in range(2)]
        loss, gn = train_step(eng, model, opt, mbs)
        t = torch.tensor([float(loss), float(gn)])
        dist.all_reduce(t)
        out.append(t / world)
    if rank == 0:
        torch.save(torch.stack(out), f"/tmp/tt_rep_{kind}_{int(replicate)}.pt")


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_replicated_layers_match_fsdp_sharded_layers(kind):
    run_distributed(_w_replicated, 2, kind, False)
    run_distributed(_w_replicated, 2, kind, True)
    a, b = torch.load(f"/tmp/tt_rep_{kind}_0.pt"), torch.load(f"/tmp/tt_rep_{kind}_1.pt")
    assert torch.allclose(a, b, rtol=1e-4, atol=1e-5), (a, b)


def _w_moe(rank, world, ep):
    losses, model, eng = _train(rank, world, MOE, {"sp_size": 1, "ep_size": ep}, 3, same_data=True)
    from torchturbo_b200.models.modules.moe import MoELayer

    layers = [m for m in model.modules() if isinstance(m, MoELayer)]
    assert layers and layers[0].num_local_experts == MOE["num_experts"] // ep
    if rank == 0:
        torch.save(torch.tensor(losses), f"/tmp/tt_moe_world{world}_ep{ep}.pt")


def test_moe_ep2_matches_ep1():
    run_distributed(_w_moe, 1, 1)
    run_distributed(_w_moe, 2, 2)
    run_distributed(_w_moe, 2, 1)
    a = torch.load("/tmp/tt_moe_world1_ep1.pt")
    for f in ("/tmp/tt_moe_world2_ep2.pt", "/tmp/tt_moe_world2_ep1.pt"):
        b = torch.load(f)
        # same data on both ranks: losses equal; gradient norms equal because expert grads are scaled by 1/ep
        assert torch.allclose(a[:, 0], b[:, 0], rtol=1e-4, atol=1e-5), (f, a, b)
        assert torch.allclose(a[:, 1], b[:, 1], rtol=1e-3, atol=1e-4), (f, a, b)


def _w_sp(rank, world, sp):
    losses, model, eng = _train(rank, world, DENSE, {"sp_size": sp, "ep_size": 1}, 3, same_data=True, ac=True)
    if rank == 0:
        torch.save(torch.tensor(losses), f"/tmp/tt_sp{sp}.pt")


def test_ulysses_sp2_matches_sp1():
    run_distributed(_w_sp, 2, 1)
    run_distributed(_w_sp, 2, 2)
    a, b = torch.load("/tmp/tt_sp1.pt"), torch.load("/tmp/tt_sp2.pt")
    assert torch.allclose(a[:, 0], b[:, 0], rtol=1e-4, atol=1e-5), (a, b)
    assert torch.allclose(a[:, 1], b[:, 1], rtol=1e-3, atol=1e-4), (a, b)


def _w_merged(rank, world, unit_bytes, ac, reshard, ep=1):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    mc = dict(MOE, num_hidden_layers=4)
    eng = TorchTurboEngine(EngineConfig.from_dict({
        "mixed_precision": "fp32", "parallel_plan": {"sp_size": 1, "ep_size": ep}, "moe": {"aux_loss_coeff": 1e-2},
        "activation_checkpointing": {"enabled": ac},
        "backend_config": {"unit_min_bytes": unit_bytes, "reshard_after_forward": reshard}}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": mc, "seed": 0})
    units = eng.backend.fsdp_units
    layers = [m for m in units if type(m).__name__.endswith("DecoderLayer")]
    if unit_bytes:
        assert len(layers) == 2 and all(len(m._tt_group) == 2 for m in layers), [len(m._tt_group) for m in layers]
    else:
        assert len(layers) == 4
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-2, weight_decay=0.0))
    ds = SyntheticPackedDataset(8, 64, mc["vocab_size"], num_docs=3, seed=5)
    out = []
    for i in range(3):
        loss, gn = train_step(eng, model, opt, [PackedCollator()([ds[i]])])
        out.append((float(loss), float(gn)))
    if rank == 0:
        torch.save(torch.tensor(out), f"/tmp/tt_merged_{unit_bytes}_{int(ac)}_{int(reshard)}_ep{ep}_w{world}.pt")


@pytest.mark.parametrize("ac,reshard", [(False, True), (True, True), (True, False)])
def test_merged_fsdp_units_match_per_layer_units(ac, reshard):
    """Two decoder layers per FSDP unit (one all-gather / reduce-scatter for both) train exactly like one unit per
    layer, with and without activation recomputation and with parameters kept gathered until backward."""
    # one tiny MoE layer without its experts is ~26 KB of bf16-equivalent bytes: 50 KB merges two layers
    run_distributed(_w_merged, 2, 0, ac, True)
    run_distributed(_w_merged, 2, 50_000, ac, reshard)
    a = torch.load(f"/tmp/tt_merged_0_{int(ac)}_1_ep1_w2.pt")
    b = torch.load(f"/tmp/tt_merged_50000_{int(ac)}_{int(reshard)}_ep1_w2.pt")
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-6), (a, b)


def test_merged_units_with_expert_units_sharded_over_edp():
    """4 ranks, EP=2: expert containers are FSDP units of their own on the 2-rank `edp` mesh, nested inside decoder
    layers that are merged pairwise on the world mesh; with recomputation the explicit prefetch lists (layers + the
    experts of the next merged unit) must still give the per-layer result."""
    run_distributed(_w_merged, 4, 0, True, True, 2)
    run_distributed(_w_merged, 4, 50_000, True, True, 2)
    a = torch.load("/tmp/tt_merged_0_1_1_ep2_w4.pt")
    b = torch.load("/tmp/tt_merged_50000_1_1_ep2_w4.pt")
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-6), (a, b)


VLM = dict(model_type="qwen3_vl", vocab_size=512,
           text_config=dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                            intermediate_size=128, vocab_size=512, tie_word_embeddings=False),
           vision_config=dict(depth=2, hidden_size=32, num_heads=4, intermediate_size=48, patch_size=2, temporal_patch_size=2,
                              spatial_merge_size=2, out_hidden_size=64, num_position_embeddings=16, deepstack_visual_indexes=[0]),
           image_token_id=500, vision_start_token_id=501)


def _w_vlm(rank, world, sp):
    """The vision-language family with its default plan (tower as one standalone unit, blocks listed for activation
    checkpointing, squared-patch-count balancing) on two ranks, with and without sequence parallelism."""
    from torchturbo_b200.data import SyntheticVLMDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    eng = TorchTurboEngine(EngineConfig.from_dict({
        "mixed_precision": "fp32", "activation_checkpointing": {"enabled": True},
        "parallel_plan": {"sp_size": sp, "ep_size": 1, "plan": {"model.visual": {"vision_balance": {"mode": "patch_sq"}}}}}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": copy.deepcopy(VLM), "seed": 0})
    tower = [p for n, p in model.named_parameters() if n.startswith("model.visual.")]
    assert tower and all(hasattr(p, "_local_tensor") for p in tower), "the tower is one world-sharded unit"
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-3))
    # seed 3: the first row of rank 1 (sp=1) carries no image, so a rank without media and the sparse-pool path are covered
    ds = SyntheticVLMDataset(4, 64, 512, image_token_id=500, vision_start_token_id=501, min_images=0, max_images=2, min_side=8,
                             max_side=16, patch=2, merge=2, seed=3)
    losses = []
    for i in range(2):
        loss, gn = train_step(eng, model, opt, [ds[(rank // sp) * 2 + i]])
        losses.append(float(loss))
        assert torch.isfinite(torch.as_tensor(gn))
    assert all(l == l for l in losses)


@pytest.mark.parametrize("sp", [1, 2])
def test_vision_language_family_trains_with_its_default_plan_on_two_ranks(sp):
    run_distributed(_w_vlm, 2, sp)
