"""End-to-end on the GPU: the kernel path and the torch path of the same tiny models must agree."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(policy, mc, steps=2):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "bf16", "ops": {"policy": policy},
                                                   "moe": {"aux_loss_coeff": 1e-3, "z_loss_coeff": 1e-4}}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(mc), "seed": 0})
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-3, weight_decay=0.0))
    ds = SyntheticPackedDataset(steps, 1024, mc["vocab_size"], min_doc=100, max_doc=600, seed=3)
    out = []
    for i in range(steps):
        b = PackedCollator()([ds[i]])
        b = {k: (v.cuda() if isinstance(v, torch.Tensor) and not k.startswith("cu_seq") else v) for k, v in b.items()}
        loss, gn = train_step(eng, model, opt, [b])
        out.append((float(loss), float(gn)))
    return out


MOE = dict(model_type="qwen3_moe", vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
           num_attention_heads=8, num_key_value_heads=2, head_dim=128, num_experts=16, num_experts_per_tok=4,
           moe_intermediate_size=256, norm_topk_prob=True)
DENSE = dict(model_type="qwen3", vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
             num_attention_heads=8, num_key_value_heads=2, head_dim=128)


@pytest.mark.parametrize("mc", [DENSE, MOE], ids=["dense", "moe"])
def test_kernel_path_matches_torch_path(mc):
    from torchturbo_b200 import kernels

    ref = _run("native", mc)
    ours = _run("auto", mc)
    assert kernels.status() == (0, 0)
    for (l0, g0), (l1, g1) in zip(ref, ours):
        assert abs(l0 - l1) / abs(l0) < 2e-2, (ref, ours)
        assert abs(g0 - g1) / abs(g0) < 1e-1, (ref, ours)
    assert kernels.launch_count() > 0
