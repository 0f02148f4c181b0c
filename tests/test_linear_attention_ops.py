"""Chunked delta-rule operators and the causal short convolution against token-by-token oracles."""
import pytest
import torch
import torch.nn.functional as F

from torchturbo_b200.ops import ops
from torchturbo_b200.ops.providers import native_linear_attention as LA


def _inputs(T=70, H=2, K=8, V=6, vec=False, seed=0):
    g = torch.Generator().manual_seed(seed)
    q, k = torch.randn(1, T, H, K, generator=g), torch.randn(1, T, H, K, generator=g)
    v = torch.randn(1, T, H, V, generator=g)
    gate = -F.softplus(torch.randn(1, T, H, K, generator=g) if vec else torch.randn(1, T, H, generator=g))
    beta = torch.sigmoid(torch.randn(1, T, H, generator=g))
    return LA.l2norm(q), LA.l2norm(k), v, gate, beta


@pytest.mark.parametrize("vec", [False, True])
@pytest.mark.parametrize("cu", [None, [0, 17, 17, 50]])
def test_chunked_matches_recurrent(vec, cu):
    q, k, v, g, beta = _inputs(vec=vec)
    cu_t = torch.tensor(cu, dtype=torch.int32) if cu is not None else None
    s0 = torch.randn(4 if cu else 1, 2, 8, 6) * 0.1
    o_ref, s_ref = LA.delta_rule_recurrent(q, k, v, g, beta, initial_state=s0, cu_seqlens=cu_t)
    o, s = LA.chunk_delta_rule(q, k, v, g, beta, initial_state=s0, output_final_state=True, cu_seqlens=cu_t, chunk_size=16)
    assert torch.allclose(o, o_ref, atol=1e-4, rtol=1e-4)
    assert torch.allclose(s, s_ref, atol=1e-4, rtol=1e-4)


def test_gdn_and_kda_dispatch_and_grad():
    q, k, v, g, beta = _inputs(T=40)
    q.requires_grad_(True)
    v.requires_grad_(True)
    o, fin = ops.gated_delta_rule(q, k, v, g, beta, cu_seqlens=torch.tensor([0, 25, 40], dtype=torch.int32), chunk_size=16)
    assert o.shape == (1, 40, 2, 6) and fin is None
    o.square().sum().backward()
    assert torch.isfinite(q.grad).all() and v.grad.abs().sum() > 0
    # KDA takes flat q/k/v, raw gate + A_log / dt_bias, raw beta
    q2, k2, v2, _, _ = _inputs(T=33, vec=True, seed=1)
    raw_g, raw_b = torch.randn(1, 33, 2, 8), torch.randn(1, 33, 2)
    A_log, dt_bias = torch.randn(2) * 0.1, torch.randn(16) * 0.1
    o2, s2 = ops.kda(q2.flatten(-2), k2.flatten(-2), v2.flatten(-2), raw_g, raw_b, A_log=A_log, dt_bias=dt_bias,
                     use_gate_in_kernel=True, output_final_state=True, chunk_size=8)
    gate = LA.kda_gate(raw_g, A_log, dt_bias)
    o_ref, s_ref = LA.delta_rule_recurrent(q2, k2, v2, gate, torch.sigmoid(raw_b))
    assert o2.shape == (1, 33, 2, 6) and torch.allclose(o2, o_ref, atol=1e-4) and torch.allclose(s2, s_ref, atol=1e-4)
    assert (LA.kda_gate(raw_g, A_log, dt_bias, lower_bound=-5.0) >= -5.0).all()


def _conv_oracle(x, w, bias, cu, act, init=None):
    T, D = x.shape[1:]
    W = w.shape[1]
    y = torch.zeros(1, T, D)
    bounds = list(zip(cu[:-1], cu[1:])) + ([(cu[-1], T)] if cu[-1] < T else [])
    for n, (a, b) in enumerate(bounds):
        for t in range(a, b):
            for s in range(W):
                src = t - s
                if src >= a:
                    y[0, t] += x[0, src] * w[:, W - 1 - s]
                elif init is not None:
                    y[0, t] += init[n][:, W + (src - a)] * w[:, W - 1 - s]
    y = y + bias
    return F.silu(y) if act else y


@pytest.mark.parametrize("with_state", [False, True])
def test_causal_conv1d(with_state):
    torch.manual_seed(0)
    x, w, bias = torch.randn(1, 21, 5), torch.randn(5, 4), torch.randn(5)
    cu = [0, 2, 9, 18]
    init = torch.randn(4, 5, 4) if with_state else None
    y, fin = ops.causal_conv1d(x, w, bias, activation="silu", initial_state=init, output_final_state=True,
                               cu_seqlens=torch.tensor(cu, dtype=torch.int32))
    assert torch.allclose(y, _conv_oracle(x, w, bias, cu, True, init), atol=1e-5)
    assert fin.shape == (4, 5, 4) and torch.equal(fin[1][:, -1], x[0, 8]) and torch.equal(fin[1][:, 0], x[0, 5])
    if with_state:
        assert torch.equal(fin[0][:, :2], init[0][:, 2:])           # a 2-token sequence keeps 2 carried inputs
    else:
        assert torch.all(fin[0][:, :2] == 0)
    yb, _ = ops.causal_conv1d(x.expand(2, -1, -1), w)               # unpacked batch
    assert torch.allclose(yb[1], _conv_oracle(x, w, torch.zeros(5), [0, 21], False)[0], atol=1e-5)
