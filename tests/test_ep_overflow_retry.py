"""Host-side logic of the dropless expert-parallel exchange: a step whose exchange overflowed a receive buffer is
repeated after the buffers have grown; the optimizer runs once, on the repeated step.  (The kernels and the real
buffers are covered on GPUs by tests/test_ep_fused_gpu.py.)"""
import pytest
import torch

from torchturbo_b200.comm.ep_p2p import CAPACITY_MARK, EPCapacityExceeded
from torchturbo_b200.loops import train_step


class _Engine:
    """The calls `train_step` makes, with an exchange that overflows on the first `fail` attempts."""

    def __init__(self, fail: int):
        self.fail, self.attempts, self.recovered, self.stale_grad_seen = fail, 0, 0, False

        class _B:
            sp_size = 1

        self.backend = _B()

    def compute_loss(self, model, mb, **kw):
        if any(p.grad is not None for p in model.parameters()):
            self.stale_grad_seen = True
        return model(mb["x"]).pow(2).mean()

    def collect_metrics(self, model):
        pass

    def clip_grad_norm_(self, model, max_norm, optimizer):
        self.attempts += 1
        n = torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm)
        return n * float("nan") if self.attempts <= self.fail else n

    def check_health(self):
        if self.attempts <= self.fail:
            raise EPCapacityExceeded(f"expert-parallel exchange on rank 0: {CAPACITY_MARK}")

    def recover_from_ep_overflow(self, optimizer):
        self.recovered += 1
        optimizer.zero_grad(set_to_none=True)


def _setup():
    torch.manual_seed(0)
    model = torch.nn.Linear(8, 4)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    return model, opt, [{"x": torch.randn(5, 8)}]


def test_overflowing_step_is_repeated_and_updates_once():
    model, opt, mbs = _setup()
    ref_model, ref_opt, _ = _setup()
    eng = _Engine(fail=2)
    loss, gnorm = train_step(eng, model, opt, mbs)
    assert eng.attempts == 3 and eng.recovered == 2 and not eng.stale_grad_seen
    train_step(_Engine(fail=0), ref_model, ref_opt, mbs)
    for p, q in zip(model.parameters(), ref_model.parameters()):
        assert torch.allclose(p, q)          # gradients of the failed attempts were not accumulated
    assert torch.isfinite(gnorm)


def test_overflow_without_retries_raises_and_leaves_the_weights():
    model, opt, mbs = _setup()
    before = [p.detach().clone() for p in model.parameters()]
    with pytest.raises(EPCapacityExceeded, match=CAPACITY_MARK):
        train_step(_Engine(fail=1), model, opt, mbs, ep_overflow_retries=0)
    for p, q in zip(model.parameters(), before):
        assert torch.equal(p, q)


def test_other_non_finite_steps_still_raise():
    model, opt, mbs = _setup()
    eng = _Engine(fail=1)
    eng.check_health = lambda: None                      # nothing wrong with the exchange: the numbers are bad
    with pytest.raises(FloatingPointError):
        train_step(eng, model, opt, mbs)
    assert eng.recovered == 0
