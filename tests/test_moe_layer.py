"""The MoE layer on one rank against a per-token loop over experts; routing variants (softmax before / after selection,
sigmoid with an expert bias, group-limited, token-id hash), auxiliary and z losses, the loss scaler, counters for the
bias update, shared experts, clamped SwiGLU."""
import pytest
import torch
import torch.nn.functional as F

from torchturbo_b200.models.modules.moe.moe import (MoEAuxLossAutoScaler, MoELayer, MoELayerConfig, MoERuntimeInputs, TopKRouter,
                                                    z_loss_func)


def _cfg(**kw):
    base = dict(hidden_size=16, moe_ffn_hidden_size=12, num_moe_experts=8, moe_router_topk=2, init_method_std=0.3)
    base.update(kw)
    return MoELayerConfig(**base)


def _naive(layer, x, idx, prob):
    w1, w2 = layer.experts.views()
    Fh = layer.config.moe_ffn_hidden_size
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            h = x[t] @ w1[e]
            out[t] += prob[t, j] * ((F.silu(h[:Fh]) * h[Fh:]) @ w2[e])
    return out


@pytest.mark.parametrize("kw", [dict(), dict(moe_router_pre_softmax=True), dict(moe_router_score_function="sigmoid"),
                                dict(moe_router_topk=1, moe_apply_probs_on_input=True),
                                dict(moe_shared_expert_intermediate_size=10, moe_shared_expert_gate=True)])
def test_layer_output_equals_a_loop_over_tokens_and_experts(kw):
    torch.manual_seed(0)
    layer = MoELayer(_cfg(**kw))
    x = torch.randn(2, 9, 16)
    out, logits = layer(x)
    assert out.shape == x.shape and logits.shape == (18, 8)
    flat = x.reshape(-1, 16)
    idx, prob, _ = layer.router(flat)
    if kw.get("moe_apply_probs_on_input"):
        want = _naive(layer, flat * prob, idx, torch.ones_like(prob))
    else:
        want = _naive(layer, flat, idx, prob)
    if layer.shared_experts is not None:
        want = want + layer.shared_experts(flat)
    assert torch.allclose(out.reshape(-1, 16), want, atol=1e-5)


def test_probabilities_of_the_three_score_functions():
    torch.manual_seed(1)
    x = torch.randn(7, 16)
    post = TopKRouter(_cfg())
    lg = F.linear(x, post.weight)
    idx, prob, logits = post(x)
    assert torch.allclose(logits, lg, atol=1e-6)
    top = lg.topk(2, -1)
    assert torch.equal(idx.long().sort(-1).values, top.indices.sort(-1).values)
    assert torch.allclose(prob.sum(-1), torch.ones(7), atol=1e-6)                       # softmax over the selected logits
    pre = TopKRouter(_cfg(moe_router_pre_softmax=True))
    pre.weight.data.copy_(post.weight.data)
    _, prob_pre, _ = pre(x)
    assert torch.allclose(prob_pre.sort(-1).values, torch.softmax(lg, -1).topk(2, -1).values.sort(-1).values, atol=1e-6)
    sig = TopKRouter(_cfg(moe_router_score_function="sigmoid", moe_router_topk_scaling_factor=2.5))
    sig.weight.data.copy_(post.weight.data)
    _, prob_sig, _ = sig(x)
    s = torch.sigmoid(lg).topk(2, -1).values
    assert torch.allclose(prob_sig.sort(-1).values, (s / s.sum(-1, keepdim=True) * 2.5).sort(-1).values, atol=1e-5)


def test_expert_bias_changes_the_selection_but_not_the_weights_and_counts_accumulate_once():
    torch.manual_seed(2)
    r = TopKRouter(_cfg(moe_router_score_function="sigmoid", moe_router_enable_expert_bias=True))
    x = torch.randn(11, 16)
    r.train()
    idx0, _, _ = r(x)
    assert float(r.local_tokens_per_expert.sum()) == 22
    r.expert_bias[5] = 10.0                                                              # expert 5 now wins a slot everywhere
    idx1, prob1, lg = r(x, runtime=MoERuntimeInputs(accumulate_tokens_per_expert=False))
    assert bool((idx1 == 5).any(-1).all()) and float(r.local_tokens_per_expert.sum()) == 22
    s = torch.sigmoid(lg).gather(1, idx1.long())
    assert torch.allclose(prob1, s / s.sum(-1, keepdim=True), atol=1e-5)                 # weights from the unbiased scores
    with pytest.raises(ValueError, match="pre_softmax"):
        _cfg(moe_router_enable_expert_bias=True)


def test_group_limited_routing_stays_inside_the_best_groups():
    torch.manual_seed(3)
    r = TopKRouter(_cfg(moe_router_score_function="sigmoid", moe_router_num_groups=4, moe_router_group_topk=1, moe_router_topk=2))
    x = torch.randn(13, 16)
    idx, prob, lg = r(x)
    groups = idx.long() // 2                                                            # 8 experts in 4 groups of 2
    assert bool((groups[:, 0] == groups[:, 1]).all())
    scores = torch.sigmoid(lg).view(13, 4, 2)
    best = scores.topk(2, -1).values.sum(-1).argmax(-1)                                  # group score: sum of its top k / group_topk experts
    assert torch.equal(groups[:, 0], best)
    assert torch.allclose(prob.sum(-1), torch.ones(13), atol=1e-5)


def test_hash_layers_route_by_token_id():
    torch.manual_seed(4)
    r = TopKRouter(_cfg(moe_router_score_function="sigmoid"))
    r.tid2eid = torch.stack([torch.arange(20) % 8, (torch.arange(20) + 3) % 8], -1)
    ids = torch.tensor([[0, 7, 13, 19, 7]])
    idx, prob, lg = r(torch.randn(5, 16), input_ids=ids)
    assert idx.tolist() == [[0, 3], [7, 2], [5, 0], [3, 6], [7, 2]]
    s = torch.sigmoid(lg).gather(1, idx.long())
    assert torch.allclose(prob, s / s.sum(-1, keepdim=True), atol=1e-5)


def test_aux_loss_value_padding_mask_and_metrics():
    torch.manual_seed(5)
    r = TopKRouter(_cfg(moe_aux_loss_coeff=0.01, moe_router_pre_softmax=True))
    r.train()
    x = torch.randn(10, 16)
    pad = torch.zeros(1, 10, dtype=torch.bool)
    pad[0, 7:] = True
    idx, prob, lg = r(x, runtime=MoERuntimeInputs(padding_mask=pad))
    m = r.pop_metrics()
    sc = torch.softmax(lg[:7], -1)
    counts = torch.bincount(idx[:7].reshape(-1).long(), minlength=8).float()
    want = (sc.sum(0) * counts).sum() * 8 / (2 * 7 * 7)                                  # E * sum_e f_e P_e with means over valid tokens
    assert torch.allclose(m["aux_loss"], want, atol=1e-5) and torch.allclose(m["aux_loss_scaled"], want * 0.01, atol=1e-6)
    assert r.pop_metrics() == {}


def test_z_loss_and_the_scaler_feed_the_router_gradient_without_touching_the_output():
    torch.manual_seed(6)
    lse = torch.randn(6)
    valid = torch.tensor([1, 1, 1, 0, 0, 1], dtype=torch.bool)
    assert torch.allclose(z_loss_func(lse, 0.1), lse.pow(2).mean() * 0.1)
    assert torch.allclose(z_loss_func(lse, 0.1, valid), lse[valid].pow(2).mean() * 0.1)
    out = torch.randn(3, requires_grad=True)
    aux = torch.tensor(2.0, requires_grad=True)
    MoEAuxLossAutoScaler.set_loss_scale(4.0)
    try:
        y = MoEAuxLossAutoScaler.apply(out, aux)
        assert torch.equal(y, out)
        y.sum().backward()
        assert torch.equal(out.grad, torch.ones(3)) and float(aux.grad) == 4.0
    finally:
        MoEAuxLossAutoScaler.set_loss_scale(1.0)
    r = TopKRouter(_cfg(moe_z_loss_coeff=0.1))
    r.train()
    x = torch.randn(5, 16)
    _, prob, lg = r(x)
    prob.sum().backward()                                                                # softmax-over-selected weights sum to 1: no gradient of their own
    want = torch.autograd.grad(torch.logsumexp(F.linear(x, r.weight), -1).pow(2).mean() * 0.1, r.weight)[0]
    assert torch.allclose(r.weight.grad, want, atol=1e-5)


def test_clamped_swiglu_limits_gate_and_up():
    torch.manual_seed(7)
    layer = MoELayer(_cfg(moe_swiglu_limit=0.5, init_method_std=1.0))
    x = torch.randn(6, 16)
    out, _ = layer(x)
    idx, prob, _ = layer.router(x)
    w1, w2 = layer.experts.views()
    want = torch.zeros_like(x)
    for t in range(6):
        for j in range(2):
            e = int(idx[t, j])
            h = x[t] @ w1[e]
            g, u = h[:12].clamp(max=0.5), h[12:].clamp(-0.5, 0.5)
            want[t] += prob[t, j] * ((F.silu(g) * u) @ w2[e])
    assert torch.allclose(out, want, atol=1e-5)
