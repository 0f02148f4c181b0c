"""FusedAdamW host-side behaviour: a skipped update (non-finite clip coefficient) leaves the step counters where they
were, as torch's fused AdamW does with `found_inf`; replacing the state drops the cached pointer tables."""
import pytest
import torch

from torchturbo_b200.engine.optimizers.fused_adamw import FusedAdamW


def _run(dev, finite_after):
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(64, 8, device=dev))
    q = torch.nn.Parameter(p.detach().clone())
    ours, ref = FusedAdamW([p], lr=1e-2, weight_decay=0.1), torch.optim.AdamW([q], lr=1e-2, weight_decay=0.1)
    for i in range(4):
        g = torch.randn(64, 8, device=dev)
        p.grad, q.grad = g.clone(), g.clone()
        skipped = i == 1
        ours.set_clip_coef(torch.tensor(float("nan") if skipped else 1.0, device=dev))
        ours.step()
        if not skipped:
            ref.step()
    if finite_after:
        ours._settle_skipped_step()
    assert int(ours.state[p]["step"]) == 3
    assert torch.allclose(p, q, atol=1e-6, rtol=1e-5)
    return ours, p


def test_skipped_update_keeps_step_counter_cpu():
    _run("cpu", False)


@pytest.mark.gpu
def test_skipped_update_keeps_step_counter_gpu():
    _run("cuda", True)


def test_load_state_dict_drops_cached_tables():
    ours, p = _run("cpu", False)
    ours._plans[0] = (("stale",), object())
    ours.load_state_dict(ours.state_dict())
    assert not ours._plans
    ours.add_param_group({"params": [torch.nn.Parameter(torch.zeros(3))]})
    assert not ours._plans
