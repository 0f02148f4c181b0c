"""Op dispatch, the torch oracle formulations, packed data contract, sampler, loss label preparation."""
import math

import pytest
import torch

from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset, pack_documents
from torchturbo_b200.engine.core import DPBlockDistributedSampler
from torchturbo_b200.engine.utils import assert_packed_inputs, get_packed_boundaries
from torchturbo_b200.models.modules.loss import logits_loss, prepare_loss_labels, shift_labels_packed
from torchturbo_b200.ops import MoEPermutation, OpDispatcher, OpImpl, OpImplKind, OpPolicy, get_expert_indices, ops
from torchturbo_b200.ops.packed_params import build_packed_params, get_packed_params
from torchturbo_b200.ops.providers import native as N
from torchturbo_b200.ops.registry import OpRegistry
from torchturbo_b200.runtime import CpuRuntime, TurboDevice


def test_dispatcher_policies_and_overrides():
    d = OpDispatcher(OpPolicy.AUTO, runtime=CpuRuntime())
    assert d.resolve("rms_norm").op_spec().kind is OpImplKind.NATIVE
    with pytest.raises(RuntimeError):
        OpDispatcher(OpPolicy.CUSTOM, runtime=CpuRuntime()).resolve("rms_norm")
    with pytest.raises(KeyError):
        OpDispatcher(OpPolicy.AUTO, {"nope": "x"}, runtime=CpuRuntime())
    with pytest.raises(KeyError):
        OpDispatcher(OpPolicy.AUTO, {"rms_norm": "does_not_exist"}, runtime=CpuRuntime())
    d2 = OpDispatcher(OpPolicy.AUTO, {"rms_norm": "torch_rms_norm"}, runtime=CpuRuntime())
    assert d2.resolve("rms_norm").op_spec().impl_name == "torch_rms_norm"
    with pytest.raises(AttributeError):
        d.not_an_op
    assert any(r[0] == "attention" for r in d.selection_table())


def test_registry_ranking():
    reg = OpRegistry()

    def mk(name, kind, prio, devices=()):
        from torchturbo_b200.ops.base import OpSpec

        cls = type(name, (OpImpl,), {"__call__": lambda self: name})
        cls.__op_spec__ = OpSpec("x", name, kind, prio, devices)
        reg.register(cls)
        return cls

    mk("a_native", OpImplKind.NATIVE, 0)
    mk("b_custom", OpImplKind.CUSTOM, 0)
    mk("c_dev", OpImplKind.NATIVE, 0, (TurboDevice.CPU,))
    mk("d_high", OpImplKind.NATIVE, 50)
    order = [c.op_spec().impl_name for c in reg.list("x", TurboDevice.CPU)]
    assert order == ["d_high", "c_dev", "b_custom", "a_native"]
    assert "c_dev" not in [c.op_spec().impl_name for c in reg.list("x", TurboDevice.CUDA)]


def test_native_rmsnorm_swiglu_ce():
    x, w = torch.randn(5, 16), torch.randn(16)
    y = ops.rms_norm(x, w, 1e-6)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert torch.allclose(y, ref, atol=1e-6)
    y2, s = ops.rms_norm(x, w, 1e-6, residual=x)
    assert torch.allclose(s, 2 * x)
    g = torch.randn(4, 8)
    assert torch.allclose(ops.swiglu(g), torch.nn.functional.silu(g[:, :4]) * g[:, 4:])
    p = torch.rand(4)
    assert torch.allclose(ops.swiglu(g, probs=p), torch.nn.functional.silu(g[:, :4]) * g[:, 4:] * p[:, None], atol=1e-6)
    lg, lab = torch.randn(6, 11), torch.tensor([1, -100, 3, 4, -100, 0])
    assert torch.allclose(ops.cross_entropy_loss(lg, lab), torch.nn.functional.cross_entropy(lg, lab, reduction="sum", ignore_index=-100))
    h, W = torch.randn(6, 7), torch.randn(11, 7)
    assert torch.allclose(ops.linear_cross_entropy(h, W, lab, chunk_size=4), ops.cross_entropy_loss(h @ W.t(), lab), atol=1e-5)
    acc = torch.zeros(3, 2)
    ops.matmul_add(acc, torch.ones(4, 3), torch.ones(4, 2))
    assert torch.equal(acc, torch.full((3, 2), 4.0))


def test_permutation_contract_and_roundtrip():
    torch.manual_seed(0)
    T, k, E, H = 9, 2, 4, 6
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    x, probs = torch.randn(T, H), torch.rand(T, k)
    perm = ops.moe_permutation(x, idx, probs=probs, num_experts=E)
    assert perm.row_indices.dtype == torch.int32 and perm.expert_indices.dtype == torch.int64
    rows = perm.row_indices.long()
    assert sorted(rows.reshape(-1).tolist()) == list(range(T * k))              # every packed row exactly once
    flat_e = idx.reshape(-1)
    e_of_row = torch.empty(T * k, dtype=torch.long)
    e_of_row[rows.reshape(-1)] = flat_e
    assert torch.equal(e_of_row, e_of_row.sort().values)                       # ordered by expert
    tok_of_row = torch.empty(T * k, dtype=torch.long)
    tok_of_row[rows.reshape(-1)] = torch.arange(T).repeat_interleave(k)
    for e in range(E):
        t = tok_of_row[e_of_row == e]
        assert torch.equal(t, t.sort().values)                                  # then by token
    assert torch.equal(perm.tokens[rows[:, 0]], x)
    assert torch.allclose(perm.probs[rows.reshape(-1)], probs.reshape(-1))
    out = ops.moe_unpermutation(perm.tokens, perm, merging_probs=probs)
    assert torch.allclose(out, x * probs.sum(1, keepdim=True), atol=1e-5)
    rm = torch.zeros(T, E, dtype=torch.bool).scatter_(1, idx, True)
    assert torch.equal(get_expert_indices(rm), idx.sort(1).values)
    y, p2 = ops.moe_sort_chunks(torch.arange(6.0).view(6, 1), [1, 2, 3], [2, 0, 1], probs=torch.arange(6.0))
    assert y.reshape(-1).tolist() == [3, 4, 5, 0, 1, 2] and p2.tolist() == [3, 4, 5, 0, 1, 2]


@pytest.mark.parametrize("fn", ["softmax_post", "softmax_pre", "sigmoid"])
def test_router_reference(fn):
    torch.manual_seed(0)
    lg = torch.randn(7, 8)
    idx, prob, st = N.router_topk_ref(lg, 2, fn, scaling=1.5)
    assert idx.shape == (7, 2) and torch.all(prob > 0)
    if fn != "softmax_pre":
        assert torch.allclose(prob.sum(-1), torch.full((7,), 1.5), atol=1e-5)
    assert int(st["counts"].sum()) == 14 and st["score_sum"].shape == (8,)
    bias = torch.zeros(8)
    bias[3] = 100.0
    if fn != "softmax_post":
        idx_b, _, st_b = N.router_topk_ref(lg, 2, fn, expert_bias=bias)
        assert torch.all((idx_b == 3).any(-1))                                  # bias steers selection ...
        assert int(st_b["aux_counts"][3]) < 7 or fn == "sigmoid"                # ... but not the aux statistics


def test_attention_reference_masks_and_padding():
    torch.manual_seed(0)
    T, Hq, Hk, D = 12, 4, 2, 8
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hk, D), torch.randn(T, Hk, D)
    cu = torch.tensor([0, 5, 9], dtype=torch.int32)
    out, ml = N.attention_ref(q, k, v, cu, causal=True, want_max_logits=True)
    assert torch.all(out[9:] == 0) and ml.shape == (Hq,)
    # a token only sees its own document, causally
    q2 = q.clone()
    q2[6:] += 1.0
    out2 = N.attention_ref(q2, k, v, cu, causal=True)
    assert torch.allclose(out[:6], out2[:6])
    k3 = k.clone()
    k3[4] += 5.0                                                               # last token of doc 0
    out3 = N.attention_ref(q, k3, v, cu, causal=True)
    assert torch.allclose(out[:4], out3[:4]) and torch.allclose(out[5:9], out3[5:9])


def test_packed_contract_and_boundaries():
    b = pack_documents([{"input_ids": [1, 2, 3]}, {"input_ids": [4, 5]}], pad_to=8)
    assert b["input_ids"].shape == (1, 8) and b["cu_seq_lens_q"].tolist() == [0, 3, 5]
    assert b["labels"][0].tolist() == [-100, 2, 3, -100, 5, -100, -100, -100]
    assert b["position_ids"][0].tolist()[:5] == [0, 1, 2, 0, 1] and b["max_length_q"] == 3
    assert_packed_inputs(b)
    bad = dict(b, attention_mask=torch.ones(1, 8))
    with pytest.raises(ValueError):
        assert_packed_inputs(bad)
    with pytest.raises(ValueError):
        assert_packed_inputs(dict(b, max_length_q=5))
    assert get_packed_boundaries(sample_ids=torch.tensor([[1, 1, 1, 2, 2, 0, 0]])).tolist() == [0, 3, 5]
    assert get_packed_boundaries(position_ids=torch.tensor([[0, 1, 2, 0, 1, 0]])).tolist() == [0, 3, 5, 6]
    ds = SyntheticPackedDataset(4, 64, 100, num_docs=3, seed=1)
    row = PackedCollator()([ds[0]])
    assert row["input_ids"].shape == (1, 64) and len(row["cu_seq_lens_q"]) == 4
    assert torch.equal(PackedCollator()([ds[0]])["input_ids"], row["input_ids"])   # seeded


def test_packed_params_tail_sequence():
    cu = torch.tensor([0, 10, 25], dtype=torch.int32)
    pp = build_packed_params(cu, (16,), total_tokens=32)
    assert pp.cu_seqlens_list == [0, 10, 25, 32] and pp.num_sequences == 3 and pp.max_seqlen == 15
    assert pp.chunk_indices["16"].tolist() == [[0, 0], [1, 0], [2, 0]]
    assert get_packed_params(cu, 32) is get_packed_params(cu, 32)
    assert get_packed_params(None, 3) is None


def test_label_shift_and_normalizers():
    labels = torch.arange(12).view(1, -1)
    cu = torch.tensor([0, 5, 10], dtype=torch.int32)
    s1 = shift_labels_packed(labels, cu, 1)[0].tolist()
    assert s1 == [1, 2, 3, 4, -100, 6, 7, 8, 9, -100, -100, -100]
    s2 = shift_labels_packed(labels, cu, 2)[0].tolist()
    assert s2 == [2, 3, 4, -100, -100, 7, 8, 9, -100, -100, -100, -100]
    st = prepare_loss_labels(labels, cu, num_streams=2, stream_scales=[1.0, 0.1], sp_size=2, sp_rank=1, world_size=2)
    assert st[0].labels.shape == (1, 6) and int(st[0].normalizer) == 8 * 2 and st[1].name == "mtp1"
    st2 = prepare_loss_labels(labels, cu, num_items_in_batch=17, sp_size=2, sp_rank=0, world_size=4)
    assert st2[0].normalizer == 16 / 4
    lg = torch.randn(1, 6, 20)
    total, comps = logits_loss([lg, lg], st)
    assert torch.allclose(total, comps["main"] + 0.1 * comps["mtp1"])


def test_dp_block_sampler():
    ds = list(range(20))
    per_rank = []
    for r in range(2):
        s = DPBlockDistributedSampler(ds, dp_size=2, dp_rank=r, rank_block=3, shuffle=True, seed=7, drop_last=True)
        per_rank.append(list(s))
        assert len(s) == 9
    assert not set(per_rank[0]) & set(per_rank[1])
    g = torch.Generator().manual_seed(7)
    perm = torch.randperm(20, generator=g).tolist()
    assert per_rank[0][:3] == perm[0:3] and per_rank[1][:3] == perm[3:6] and per_rank[0][3:6] == perm[6:9]
    s = DPBlockDistributedSampler(list(range(5)), 2, 0, rank_block=2, shuffle=False, drop_last=False)
    assert len(list(s)) == 4 and s.total_size == 8                                # cycled to whole blocks
    s.set_epoch(1)


def test_layer_norm_and_bias_act_torch_formulations():
    """The torch (oracle) implementations of the vision-tower elementwise operators and their dispatch by name."""
    import torch.nn.functional as F

    from torchturbo_b200.ops import ops

    torch.manual_seed(0)
    x, w, b = torch.randn(5, 16), torch.randn(16), torch.randn(16)
    assert torch.allclose(ops.layer_norm(x, w, b, 1e-6), F.layer_norm(x, (16,), w, b, 1e-6), atol=1e-6)
    r = torch.randn(5, 16)
    assert torch.allclose(ops.bias_act(x, b), x + b)
    assert torch.allclose(ops.bias_act(x, b, "gelu_tanh"), F.gelu(x + b, approximate="tanh"), atol=1e-6)
    assert torch.allclose(ops.bias_act(x, b, "gelu", residual=r), F.gelu(x + b) + r, atol=1e-6)
    with pytest.raises(ValueError, match="unknown activation"):
        ops.bias_act(x, b, "relu6")
    h = ops.bias_act(x.bfloat16(), b.bfloat16(), "gelu_tanh")
    assert h.dtype == torch.bfloat16


def test_sequence_bounds_for_the_packed_convolution():
    from torchturbo_b200.ops.providers.b200 import _seq_bounds

    s, e = _seq_bounds(torch.tensor([0, 2, 5], dtype=torch.int32), 7, torch.device("cpu"))
    assert s.tolist() == [0, 0, 2, 2, 2, 5, 5] and e.tolist() == [2, 2, 5, 5, 5, 7, 7]     # the padding tail is its own sequence
    s, e = _seq_bounds(None, 3, torch.device("cpu"))
    assert s.tolist() == [0, 0, 0] and e.tolist() == [3, 3, 3]
