"""The AdamW update of the decoder layers on a side stream under the next forward pass must train exactly like the
update on the compute stream: same kernels per parameter, only their stream and the per-layer waits differ."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _train(overlap: bool, steps: int = 5):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.engine.optimizers.fused_adamw import FusedAdamW
    from torchturbo_b200.loops import train_step

    os.environ["TORCHTURBO_ADAMW_OVERLAP"] = "1" if overlap else "0"       # opt-in: off by default
    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "bf16", "activation_checkpointing": {"enabled": False}}))
    mc = dict(model_type="qwen3_moe", vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=4,
              num_attention_heads=8, num_key_value_heads=2, head_dim=128, num_experts=8, num_experts_per_tok=2,
              moe_intermediate_size=256, norm_topk_prob=True)
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": mc, "seed": 0})
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-3, weight_decay=0.01))
    fused = [o for o in getattr(opt, "optimizers", [opt]) if isinstance(o, FusedAdamW)]
    assert fused and all(bool(o._buckets) == overlap for o in fused)
    ds = SyntheticPackedDataset(steps, 1024, mc["vocab_size"], min_doc=128, max_doc=700, seed=3)
    losses = []
    for i in range(steps):
        b = PackedCollator()([ds[i]])
        b = {k: (v.cuda() if isinstance(v, torch.Tensor) and not k.startswith("cu_seq") else v) for k, v in b.items()}
        loss, gnorm = train_step(eng, model, opt, [b], check_finite=False)      # no host read between steps
        losses.append(loss)
    eng.check_health()                                                          # joins the side stream
    torch.cuda.synchronize()
    if overlap:
        assert any(ev is not None for o in fused for ev in o._bucket_events)
    return [float(x) for x in losses], [p.detach().float().clone() for p in model.parameters()]


def test_update_on_the_side_stream_trains_identically():
    """Attention backward and the routing histograms add with atomics, so two runs differ in the last bits; the run
    with the overlap must differ from a plain run by no more than two plain runs differ from each other."""
    try:
        la, pa = _train(False)
        lc, pc = _train(False)
        lb, pb = _train(True)
    finally:
        os.environ.pop("TORCHTURBO_ADAMW_OVERLAP", None)
    noise_l = max(abs(x - y) for x, y in zip(la, lc))
    noise_p = max((a - c).abs().max().item() for a, c in zip(pa, pc))
    assert max(abs(x - y) for x, y in zip(la, lb)) <= 4 * noise_l + 1e-4, (la, lb, lc)
    assert max((a - b).abs().max().item() for a, b in zip(pa, pb)) <= 4 * noise_p + 1e-3
