"""Analytic FLOP recipes (`engine/metrics/flops.py`) against hand counts, and the optimizer construction contract
(`engine/optimizers/plan.py`, `container.py`)."""
from types import SimpleNamespace

import pytest
import torch
import torch.nn as nn

from torchturbo_b200.engine.metrics.flops import (ComputeProfile, LLMFlops, MlaLLMFlops, MoELLMFlops, VLMFlops, attention_flops,
                                                   matmul_flops)
from torchturbo_b200.engine.optimizers import OptimizerClassPlan
from torchturbo_b200.engine.optimizers.container import OptimizersContainer
from torchturbo_b200.engine.optimizers.plan import OptimizerPlan, ParamGroup, is_no_decay


def test_attention_flops_count_pairs_per_document_not_per_row():
    assert matmul_flops(3, 5, 7) == 2 * 3 * 5 * 7
    one = attention_flops([8], 2, 4, causal=False)
    assert one == 2 * 64 * 2 * (4 + 4)
    assert attention_flops([8], 2, 4, causal=True) == one / 2
    assert attention_flops([4, 4], 2, 4, causal=False) == one / 2           # two documents of half the length: half the pairs
    assert attention_flops([8], 2, 6, causal=False, v_head_dim=2) == 2 * 64 * 2 * (6 + 2)


def test_dense_recipe_matches_a_hand_count():
    c = SimpleNamespace(hidden_size=16, head_dim=4, num_attention_heads=4, num_key_value_heads=2, intermediate_size=24,
                        num_hidden_layers=3, vocab_size=50)
    prof = ComputeProfile(10, [6, 4])
    per_layer = 2 * 10 * (4 + 4) * 4 * 16 + 2 * 10 * 16 * 16 + 3 * 2 * 10 * 24 * 16 + (2 * (36 + 16) * 4 * 8) / 2
    assert LLMFlops(c).forward_flops(prof) == pytest.approx(3 * per_layer + 2 * 10 * 50 * 16)


def test_moe_recipe_counts_routed_rows_router_shared_experts_and_dense_layers():
    c = SimpleNamespace(hidden_size=16, head_dim=4, num_attention_heads=4, num_key_value_heads=2, intermediate_size=24,
                        num_hidden_layers=2, vocab_size=50, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=6,
                        shared_expert_intermediate_size=12, mlp_only_layers=[0])
    dense = LLMFlops(c)
    moe = MoELLMFlops(c)
    assert moe._mlp(10, 0) == dense._mlp(10, 0)
    assert moe._mlp(10, 1) == 3 * 2 * (10 * 2) * 6 * 16 + 2 * 10 * 8 * 16 + 3 * 2 * 10 * 12 * 16
    assert moe.forward_flops(ComputeProfile(10, [10])) < dense.forward_flops(ComputeProfile(10, [10])) + moe._mlp(10, 1)


def test_mla_projections_and_vlm_tower_terms():
    c = SimpleNamespace(hidden_size=32, num_attention_heads=4, qk_nope_head_dim=8, qk_rope_head_dim=4, v_head_dim=8, q_lora_rank=16,
                        kv_lora_rank=12)
    want = 2 * 5 * 16 * 32 + 2 * 5 * (4 * 12) * 16 + 2 * 5 * (12 + 4) * 32 + 2 * 5 * (4 * 16) * 12 + 2 * 5 * 32 * (4 * 8)
    assert MlaLLMFlops(c)._attn_proj(5) == want
    c.q_lora_rank = None
    assert MlaLLMFlops(c)._attn_proj(5) == want - (2 * 5 * 16 * 32 + 2 * 5 * 48 * 16) + 2 * 5 * 48 * 32
    text = SimpleNamespace(hidden_size=16, head_dim=4, num_attention_heads=4, num_key_value_heads=2, intermediate_size=24,
                           num_hidden_layers=1, vocab_size=50)
    vis = SimpleNamespace(hidden_size=8, num_heads=2, intermediate_size=12, depth=2, in_channels=3, temporal_patch_size=2, patch_size=2,
                          spatial_merge_size=2, out_hidden_size=16)
    both = SimpleNamespace(text_config=text, vision_config=vis)
    no_img = VLMFlops(both).forward_flops(ComputeProfile(10, [10]))
    assert no_img == LLMFlops(text).forward_flops(ComputeProfile(10, [10]))
    with_img = VLMFlops(both).forward_flops(ComputeProfile(10, [10], True, [16, 64]))
    assert with_img > no_img
    # attention inside the tower is per image: one image of 80 patches costs more than images of 16 and 64
    assert VLMFlops(both).forward_flops(ComputeProfile(10, [10], True, [80])) > with_img


def test_compute_profile_from_a_packed_batch():
    batch = {"input_ids": torch.zeros(1, 12, dtype=torch.long), "cu_seq_lens_q": torch.tensor([0, 5, 12]),
             "image_grid_thw": torch.tensor([[1, 4, 4], [2, 2, 6]])}
    p = ComputeProfile.from_inputs(batch)
    assert (p.num_tokens, list(p.seq_lens), list(p.num_image_patches)) == (12, [5, 7], [16, 24])
    p = ComputeProfile.from_inputs({"inputs_embeds": torch.zeros(1, 9, 4)})
    assert p.num_tokens == 9 and list(p.seq_lens) == [9]


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.lin = nn.Linear(4, 3)
        self.norm = nn.LayerNorm(3)
        self.frozen = nn.Linear(3, 2)
        self.frozen.requires_grad_(False)


def test_class_plan_splits_decay_and_no_decay_and_skips_frozen_parameters():
    net = _Net()
    plan = OptimizerClassPlan(torch.optim.AdamW, lr=0.1, weight_decay=0.5, betas=(0.8, 0.9)).resolve(net.named_parameters())
    by = {g.name: g for g in plan.groups}
    assert by["decay"].param_names == ["lin.weight"] and by["decay"].hyperparameters["weight_decay"] == 0.5
    assert sorted(by["no_decay"].param_names) == ["lin.bias", "norm.bias", "norm.weight"]
    assert by["no_decay"].hyperparameters == {"lr": 0.1, "betas": (0.8, 0.9), "weight_decay": 0.0}
    plan.validate(net)
    assert is_no_decay("x.bias", torch.zeros(2, 2)) and not is_no_decay("x.weight", torch.zeros(2, 2))
    opt = torch.optim.AdamW([g.as_torch_group() for g in plan.groups])
    assert [g["weight_decay"] for g in opt.param_groups] == [0.5, 0.0]


def test_plan_validation_names_duplicates_and_uncovered_parameters():
    net = _Net()
    g = ParamGroup("a", [net.lin.weight], ["lin.weight"], torch.optim.SGD, {"lr": 0.1})
    with pytest.raises(ValueError, match="without an optimizer group"):
        OptimizerPlan([g]).validate(net)
    dup = ParamGroup("b", [net.lin.weight, net.lin.bias, net.norm.weight, net.norm.bias], ["..."] * 4, torch.optim.SGD, {"lr": 0.1})
    with pytest.raises(ValueError, match="more than one optimizer group"):
        OptimizerPlan([g, dup]).validate(net)
    two = OptimizerPlan([g, ParamGroup("c", [net.lin.bias], ["lin.bias"], torch.optim.AdamW, {"lr": 0.1})])
    assert set(two.by_class()) == {torch.optim.SGD, torch.optim.AdamW}


def test_container_steps_every_optimizer_and_round_trips_its_state():
    torch.manual_seed(0)
    a, b = nn.Parameter(torch.randn(3)), nn.Parameter(torch.randn(2, 2))
    box = OptimizersContainer([torch.optim.SGD([a], lr=0.5), torch.optim.AdamW([b], lr=0.1)], ["sgd", "adamw"])
    assert len(box) == 2 and len(box.param_groups) == 2
    a.grad, b.grad = torch.ones(3), torch.ones(2, 2)
    a0, b0 = a.detach().clone(), b.detach().clone()
    calls = []
    box.register_step_post_hook(lambda *args: calls.append(1))
    box.step()
    assert torch.allclose(a, a0 - 0.5) and not torch.equal(b, b0) and calls
    box.zero_grad()
    assert a.grad is None and b.grad is None
    sd = box.state_dict()
    a2, b2 = nn.Parameter(a.detach().clone()), nn.Parameter(b.detach().clone())
    box2 = OptimizersContainer([torch.optim.SGD([a2], lr=0.5), torch.optim.AdamW([b2], lr=0.1)], ["sgd", "adamw"])
    box2.load_state_dict(sd)
    b.grad, b2.grad = torch.ones(2, 2), torch.ones(2, 2)
    a.grad, a2.grad = torch.ones(3), torch.ones(3)
    box.step(); box2.step()
    assert torch.equal(b, b2) and torch.equal(a, a2)                      # the AdamW moments and step count came along
    sched = torch.optim.lr_scheduler.LambdaLR(box, lambda s: 0.5)
    assert [g["lr"] for g in box.param_groups] == [0.25, 0.05] and sched.get_last_lr() == [0.25, 0.05]
