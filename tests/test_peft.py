"""LoRA / DoRA adapters on dense projections and on fused expert storage: no-op at init, trainable set, equivalence of
the adapted forward with merged weights, delta map for export, rank-stabilised scaling."""
import math

import pytest
import torch
import torch.nn as nn

from torchturbo_b200.engine.peft.lora import (GroupedMLPLoRA, LoRALinear, LoraConfig, apply_lora_delta, apply_peft,
                                              build_lora_delta_map, compute_dora_magnitude, expand_all_linear_targets)
from torchturbo_b200.models.registry import get_model

MOE = dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128,
           moe_intermediate_size=32, num_experts=4, num_experts_per_tok=2, vocab_size=128, torch_dtype="float32")


def _model():
    cls = get_model("qwen3_moe")
    torch.manual_seed(0)
    return cls(cls.config_class(**MOE))


def _batch():
    torch.manual_seed(1)
    return dict(input_ids=torch.randint(0, 128, (1, 20)), cu_seq_lens_q=torch.tensor([0, 8, 20], dtype=torch.int32), max_length_q=12)


def test_scaling_and_target_expansion():
    assert LoraConfig(r=8, lora_alpha=16).scaling == 2.0
    assert LoraConfig(r=16, lora_alpha=16, use_rslora=True).scaling == pytest.approx(16 / math.sqrt(16))
    m = _model()
    names = expand_all_linear_targets(m)
    assert "model.layers.0.self_attn.qkv_proj" in names and "lm_head" not in names
    assert not any("router" in n for n in names)


def test_lora_starts_as_noop_trains_only_adapters_and_merges():
    m = _model().eval()
    b = _batch()
    with torch.no_grad():
        base = m(**b).logits.clone()
    apply_peft(m, LoraConfig(r=4, lora_alpha=8, target_modules=["all-linear"], target_experts=True))
    assert isinstance(m.model.layers[0].self_attn.qkv_proj, LoRALinear)
    assert isinstance(m.model.layers[0].mlp.experts, GroupedMLPLoRA)
    with torch.no_grad():
        assert torch.allclose(m(**b).logits, base, atol=1e-6)                   # B matrices start at zero
    trainable = [n for n, p in m.named_parameters() if p.requires_grad]
    assert trainable and all("lora" in n for n in trainable)
    # make the adapters non-trivial, then compare with the model whose weights carry the merged delta
    torch.manual_seed(2)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.requires_grad:
                p.normal_(0, 0.05)
        adapted = m(**b).logits.clone()
    assert not torch.allclose(adapted, base, atol=1e-4)
    delta = build_lora_delta_map(m)
    assert "model.layers.0.self_attn.qkv_proj.weight" in delta and "model.layers.1.mlp.experts.weight1" in delta
    ref = _model().eval()
    with torch.no_grad():
        sd = dict(ref.named_parameters())
        for k, d in delta.items():
            sd[k].add_(d.view_as(sd[k]))
        assert torch.allclose(ref(**b).logits, adapted, atol=1e-4)
    apply_lora_delta(m)
    assert set(m.merged_lora_delta) == set(delta)
    # gradients reach both the dense and the expert adapters
    m.train()
    m(**b).logits.float().pow(2).mean().backward()
    g = {n: p.grad for n, p in m.named_parameters() if p.requires_grad}
    assert all(v is not None for v in g.values())
    assert any("experts" in n and float(v.abs().sum()) > 0 for n, v in g.items())


def test_dora_keeps_column_norms_at_init():
    lin = nn.Linear(12, 6, bias=False)
    w0 = lin.weight.detach().clone()
    d = LoRALinear(lin, LoraConfig(r=2, lora_alpha=4, use_dora=True))
    assert torch.allclose(compute_dora_magnitude(w0), w0.norm(dim=1))
    x = torch.randn(5, 12)
    assert torch.allclose(d(x), x @ w0.t(), atol=1e-5)                            # magnitude = |W| and B = 0
    with torch.no_grad():
        d.lora_B["default"].weight.normal_(0, 0.1)
    w = d.weight
    assert torch.allclose(w.norm(dim=1), w0.norm(dim=1), atol=1e-5)               # direction changes, magnitude stays
