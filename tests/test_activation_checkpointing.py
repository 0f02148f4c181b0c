"""Activation-checkpoint glue of the FSDP2 backend: the replay of a checkpointed segment must not count router
statistics twice, reentrant mode must accept keyword arguments and must still reach the parameters when no input
requires a gradient.  (Reference behaviour: engine/backends/fsdp2/backend.py:875-990 and activation_checkpointing.py:25-69.)"""
import contextlib

import pytest
import torch

from torchturbo_b200.engine.backends.fsdp2.backend import _recompute_ctx, _reentrant_checkpoint
from torchturbo_b200.models.modules.moe import MoELayer, MoELayerConfig

T, H, E, K = 24, 32, 8, 2


def _layer():
    torch.manual_seed(0)
    cfg = MoELayerConfig(hidden_size=H, moe_ffn_hidden_size=16, num_moe_experts=E, moe_router_topk=K, moe_aux_loss_coeff=1e-2,
                         moe_router_score_function="sigmoid", moe_router_enable_expert_bias=True)
    return MoELayer(cfg).train()


def _run(mode: str, x_requires_grad: bool):
    from torch.utils.checkpoint import checkpoint

    layer = _layer()
    x = torch.randn(T, H, requires_grad=x_requires_grad)
    fn = lambda h, scale=1.0: layer(h)[0] * scale   # noqa: E731
    if mode == "none":
        y = fn(x, scale=2.0)
    elif mode == "reentrant":
        y = _reentrant_checkpoint(fn, (x,), {"scale": 2.0})
    else:
        y = checkpoint(fn, x, use_reentrant=False, context_fn=lambda: (contextlib.nullcontext(), _recompute_ctx()), scale=2.0)
    y.square().mean().backward()
    return layer, x


@pytest.mark.parametrize("x_requires_grad", [True, False])
@pytest.mark.parametrize("mode", ["reentrant", "non_reentrant"])
def test_checkpointed_layer_counts_once_and_trains(mode, x_requires_grad):
    ref, xr = _run("none", x_requires_grad)
    got, xg = _run(mode, x_requires_grad)
    # token counters for the expert-bias update and the reported losses: one micro-batch, counted once
    assert float(got.router.local_tokens_per_expert.sum()) == T * K
    assert torch.equal(got.router.local_tokens_per_expert, ref.router.local_tokens_per_expert)
    assert {k: len(v) for k, v in got.router._metrics.items()} == {k: len(v) for k, v in ref.router._metrics.items()}
    # gradients reach every parameter (also when nothing in front of the segment requires a gradient) and match
    for (n, a), (_, b) in zip(got.named_parameters(), ref.named_parameters()):
        assert a.grad is not None, n
        assert torch.allclose(a.grad, b.grad, atol=1e-6), n
    if x_requires_grad:
        assert torch.allclose(xg.grad, xr.grad, atol=1e-6)
