"""Registry / adapter / patch lifecycle, detector, plugins, LR schedulers, FQN map, QK-clip, optimizer parking,
metrics, prefetch planning, RL packed helpers."""
import math
import os
from types import SimpleNamespace

import pytest
import torch
import torch.nn as nn


# ---------------------------------------------------------------------------------------------------------
def test_adapter_patch_lifecycle_and_version_gate():
    from torchturbo_b200.registry.adapter import BaseAdapter, _version_matches
    from torchturbo_b200.registry.patch import BasePatch

    assert _version_matches("0.9.3", ">=0.9,<1.0") and not _version_matches("1.1", ">=0.9,<1.0")
    assert _version_matches(None, None) and not _version_matches(None, ">=1") and not _version_matches("x", ">=1")
    target = SimpleNamespace(value="orig")

    class P(BasePatch):
        name = "p"

        def _patch(self, engine=None):
            self.saved, target.value = target.value, "patched"

        def _revert(self):
            target.value = self.saved

    class A(BaseAdapter):
        name = "fake"

        def detect(self):
            return True

    a = A()
    a.add_patch(P())
    applied = a.apply_patches()
    assert target.value == "patched" and applied
    a.apply_patches()                                   # idempotent
    assert target.value == "patched"
    a.revert_patches()
    assert target.value == "orig"


def test_detector_orders_by_priority(monkeypatch):
    from torchturbo_b200 import detector as D
    from torchturbo_b200.registry.adapter import BaseAdapter

    def mk(name, prio, hit):
        return type(name, (BaseAdapter,), {"name": name, "priority": prio, "detect": lambda self: hit})()

    from torchturbo_b200.registry import registry as R

    monkeypatch.setattr(R, "_ADAPTERS", {a.name: a for a in (mk("low", 1, True), mk("high", 9, True), mk("off", 99, False))})
    det = D.FrameworkDetector()
    assert det.detect_all() == ["high", "low"] and det.detect() == "high"


def test_plugins_load_from_file(tmp_path):
    from torchturbo_b200.engine.plugins import PluginManager

    f = tmp_path / "my_plugin.py"
    f.write_text("from torchturbo_b200.engine.plugins import DatasetPlugin, CheckpointExportPlugin, register_plugin\n"
                 "@register_plugin\nclass D(DatasetPlugin):\n    def wrap_dataset(self, ds):\n        return [x * 2 for x in ds]\n"
                 "@register_plugin\nclass E(CheckpointExportPlugin):\n    def on_hf_export(self, export_dir, *, step=None, final=False):\n"
                 "        open(export_dir + '/done', 'w').write(str(self.config))\n")
    pm = PluginManager([f"{f}:cfg.yaml"])
    assert len(pm.dataset_plugins()) == 1 and len(pm.export_plugins()) == 1
    assert pm.dataset_plugins()[0].wrap_dataset([1, 2]) == [2, 4]
    pm.export_plugins()[0].on_hf_export(str(tmp_path), step=3)
    assert (tmp_path / "done").read_text() == "cfg.yaml"
    with pytest.raises(FileNotFoundError):
        PluginManager([str(tmp_path / "missing.py")])


# ---------------------------------------------------------------------------------------------------------
def _opt(lrs=(1.0,)):
    ps = [nn.Parameter(torch.zeros(1)) for _ in lrs]
    return torch.optim.SGD([{"params": [p], "lr": lr} for p, lr in zip(ps, lrs)])


def _run(sched, opt, n):
    out = []
    for _ in range(n):
        out.append([g["lr"] for g in opt.param_groups])
        opt.step()
        sched.step()
    return out


def test_lr_schedulers():
    from torchturbo_b200.engine.optimizers.lr_scheduler import create_lr_scheduler

    opt = _opt()
    lrs = _run(create_lr_scheduler("linear", opt, 2, 10), opt, 10)
    assert lrs[0][0] == 0.0 and lrs[2][0] == 1.0 and lrs[6][0] == pytest.approx(0.5)
    opt = _opt()
    lrs = _run(create_lr_scheduler("cosine", opt, 0, 10), opt, 11)
    assert lrs[5][0] == pytest.approx(0.5) and lrs[10][0] == pytest.approx(0.0, abs=1e-9)
    # absolute per-group floor: both groups end at min_lr although their peaks differ
    opt = _opt((1.0, 0.1))
    lrs = _run(create_lr_scheduler("cosine_with_min_lr", opt, 2, 10, min_lr=0.05), opt, 11)
    assert lrs[10][0] == pytest.approx(0.05) and lrs[10][1] == pytest.approx(0.05) and lrs[2] == [1.0, 0.1]
    opt = _opt((1.0, 0.1))
    lrs = _run(create_lr_scheduler("cosine_with_min_lr", opt, 0, 10, min_lr_rate=0.1), opt, 11)
    assert lrs[10][0] == pytest.approx(0.1) and lrs[10][1] == pytest.approx(0.01)
    with pytest.raises(ValueError):
        create_lr_scheduler("cosine_with_min_lr", _opt(), 0, 10)
    with pytest.raises(ValueError):
        create_lr_scheduler("linear", _opt(), 0, None)


def test_model_fqn_map_strips_wrappers():
    from torchturbo_b200.engine.model_fqn import authored_name, build_model_fqn_map

    assert authored_name("base_model.model.model.layers.0._checkpoint_wrapped_module.mlp.weight") == "model.layers.0.mlp.weight"

    class Wrap(nn.Module):
        def __init__(self, m):
            super().__init__()
            self._checkpoint_wrapped_module = m

    inner = nn.Sequential(nn.Linear(2, 2))
    m = nn.ModuleDict({"layers": nn.ModuleList([Wrap(inner)])})
    mp = build_model_fqn_map(m)
    assert mp["layers.0.0.weight"] == "layers.0._checkpoint_wrapped_module.0.weight"


def test_qk_clip_scales_only_hot_heads():
    from torchturbo_b200.engine.optimizers.qk_clip import QKClipController

    class Attn(nn.Module):
        n_q, n_kv, head_dim = 4, 2, 2

        def __init__(self):
            super().__init__()
            self.qkv_proj = nn.Linear(3, (4 + 2 * 2) * 2, bias=False)
            nn.init.ones_(self.qkv_proj.weight)
            self.qk_clip_state = None

    m = nn.ModuleDict({"attn": Attn()})
    ctl = QKClipController(m, threshold=10.0, alpha=0.5)
    a = m["attn"]
    assert a.qk_clip_state is not None and len(ctl.plan.specs) == 1
    a.qk_clip_state.update(torch.tensor([5.0, 40.0, 10.0, 1000.0]))
    a.qk_clip_state.update(torch.tensor([1.0, 20.0, 10.0, 10.0]))           # running maximum since the last step
    maxima = ctl.apply()
    assert maxima.tolist() == [5.0, 40.0, 10.0, 1000.0]
    w = a.qkv_proj.weight
    g = lambda x: math.sqrt(10.0 / x)                                       # noqa: E731  gamma ** alpha per side
    assert torch.allclose(w[0:2], torch.ones(2, 3)) and torch.allclose(w[4:6], torch.ones(2, 3))
    assert torch.allclose(w[2:4], torch.full((2, 3), g(40.0))) and torch.allclose(w[6:8], torch.full((2, 3), g(1000.0)))
    # kv head 0 serves q heads 0-1, kv head 1 serves q heads 2-3: each takes the strongest shrink of its group
    assert torch.allclose(w[8:10], torch.full((2, 3), g(40.0))) and torch.allclose(w[10:12], torch.full((2, 3), g(1000.0)))
    assert torch.allclose(w[12:], torch.ones(4, 3))                         # values untouched
    assert a.qk_clip_state.max_logits is None                               # consumed


def test_qk_clip_mla_splits_nope_and_rope_rows():
    from torchturbo_b200.engine.optimizers.qk_clip import MLAQKClipSpec, QKClipController

    class MLA(nn.Module):
        n_heads, d_nope, d_rope, d_v = 2, 2, 1, 3

        def __init__(self):
            super().__init__()
            self.q_b_proj = nn.Linear(4, 2 * (2 + 1), bias=False)
            self.kv_b_proj = nn.Linear(4, 2 * (2 + 3), bias=False)
            nn.init.ones_(self.q_b_proj.weight); nn.init.ones_(self.kv_b_proj.weight)
            self.qk_clip_state = None

    m = nn.ModuleDict({"attn": MLA()})
    ctl = QKClipController(m, threshold=10.0, alpha=0.25)
    spec = ctl.plan.specs[0]
    assert isinstance(spec, MLAQKClipSpec) and spec.projection_rows == {"attn.q_b_proj.weight": 6, "attn.kv_b_proj.weight": 10}
    m["attn"].qk_clip_state.update(torch.tensor([160.0, 3.0]))              # head 0 is hot: gamma = 1/16
    ctl.apply()
    q, kv = m["attn"].q_b_proj.weight, m["attn"].kv_b_proj.weight
    g = 1.0 / 16
    assert torch.allclose(q[0:2], torch.full((2, 4), g ** 0.25)) and torch.allclose(q[2:3], torch.full((1, 4), g))   # NoPE, RoPE
    assert torch.allclose(q[3:], torch.ones(3, 4))                                                                   # cool head
    assert torch.allclose(kv[0:2], torch.full((2, 4), g ** 0.75)) and torch.allclose(kv[2:5], torch.ones(3, 4))      # K NoPE, V
    assert torch.allclose(kv[5:], torch.ones(5, 4))
    with pytest.raises(ValueError, match="distinct"):
        MLAQKClipSpec("a", "w", "w", 1, 1, 1, 1)


def test_optimizer_memory_controller_guards():
    from torchturbo_b200.engine.optimizers.memory import OptimizerMemoryController, OptimizerSuspendedError

    p = nn.Parameter(torch.ones(4))
    opt = torch.optim.AdamW([p], lr=0.1)
    p.grad = torch.ones(4)
    opt.step()
    before = {k: v.clone() for k, v in opt.state[p].items() if torch.is_tensor(v)}
    ctl = OptimizerMemoryController(opt)
    moved = ctl.offload()
    assert moved == (0 if not torch.cuda.is_available() else moved)      # only device-resident state is parked
    with pytest.raises(OptimizerSuspendedError):
        opt.step()
    with pytest.raises(OptimizerSuspendedError):
        opt.load_state_dict(opt.state_dict())
    ctl.restore()
    for k, v in before.items():
        assert torch.equal(opt.state[p][k], v)
    opt.step()


def test_metric_tracker_window_and_module_metrics():
    from torchturbo_b200.engine.metrics.tracker import MetricTracker

    class M(nn.Module):
        def pop_metrics(self):
            return {"aux_loss": torch.tensor(2.0)}

    t = MetricTracker()
    t.add("a", 1.0)
    t.add("a", torch.tensor(3.0))
    t.collect(nn.Sequential(M(), M()))
    logs = t.report({"step": 1})
    assert logs["a"] == pytest.approx(2.0) and logs["aux_loss"] == pytest.approx(2.0) and logs["step"] == 1
    assert "a" not in t.report({})                               # window cleared


def test_mfu_estimator_counts_tokens_and_flops():
    from torchturbo_b200.engine.metrics.flops import LLMFlops
    from torchturbo_b200.engine.metrics.mfu_estimator import MFUEstimator, resolve_peak_tflops

    name, peak = resolve_peak_tflops("b200")
    assert peak > 1000
    cfg = SimpleNamespace(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                          intermediate_size=128, vocab_size=100)
    est = MFUEstimator(LLMFlops(cfg), card="b200", world_size=1)
    est.record_micro({"input_ids": torch.zeros(1, 32, dtype=torch.long), "cu_seq_lens_q": torch.tensor([0, 20, 32])})
    out = est.pop()
    assert out and all(v >= 0 for v in out.values())


def test_prefetch_planning_pure_function():
    from torchturbo_b200.engine.backends.fsdp2.prefetch import FSDPPrefetchManager
    from torchturbo_b200.engine.config import FSDPConfig, FSDPPrefetchStrategy

    mgr = FSDPPrefetchManager(FSDPConfig())
    plan = mgr.build_targets(5, 2, FSDPPrefetchStrategy.EXPERT_WITH_LAYER, [False, True, True, False, True])
    assert plan[0][0] == [1, 2] and plan[0][1] == [1, 2] and plan[1][0] == [3] and plan[2][1] == [4]
    covered = [j for lt, _, _ in plan for j in lt]
    assert sorted(covered) == [1, 2, 3, 4]                       # every later layer prefetched exactly once
    look = mgr.build_targets(5, 2, FSDPPrefetchStrategy.EXPERT_LOOKAHEAD, [True, True, False, True, True])
    assert look[0][2] == [1] and look[1][2] == [3] and look[2][2] == []


# ---------------------------------------------------------------------------------------------------------
def test_rl_packed_helpers():
    from torchturbo_b200.adapters.rl.packed import gather_logprobs_entropy, prepare_packed_mb_inputs, shifted_packed_tensor

    seqs = [torch.tensor([1, 2, 3]), torch.tensor([4, 5])]
    mb = prepare_packed_mb_inputs(seqs, pad_to_multiple_of=4, pad_token_id=0)
    assert mb["input_ids"].shape == (1, 8) and mb["cu_seq_lens_q"].tolist() == [0, 3, 5]
    assert mb["position_ids"][0, :5].tolist() == [0, 1, 2, 0, 1]
    sh = shifted_packed_tensor(mb["input_ids"], mb["cu_seq_lens_q"], fill=-1)
    assert sh[0, :5].tolist() == [2, 3, -1, 5, -1]
    logits = torch.randn(1, 8, 11)
    tg = sh[0].clone()
    tg[tg < 0] = -100
    lp, ent = gather_logprobs_entropy(logits[0], tg, want_entropy=True)
    ref = torch.log_softmax(logits[0].float(), -1)
    assert torch.allclose(lp[0], ref[0, 2]) and float(lp[2]) == 0.0           # ignored targets give 0
    assert torch.allclose(ent[1], -(ref[1].exp() * ref[1]).sum(), atol=1e-5)


def test_adamw_swap_matches_torch_adamw_and_keeps_state_on_host():
    from torchturbo_b200.engine.optimizers import AdamWSwap

    torch.manual_seed(0)
    a = [nn.Parameter(torch.randn(7, 5)), nn.Parameter(torch.randn(11))]
    b = [nn.Parameter(p.detach().clone()) for p in a]
    oa = AdamWSwap(a, lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95))
    ob = torch.optim.AdamW(b, lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95))
    for _ in range(4):
        for pa, pb in zip(a, b):
            g = torch.randn_like(pa)
            pa.grad, pb.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    assert max((pa - pb).abs().max().item() for pa, pb in zip(a, b)) < 1e-6
    st = oa.state_dict()["state"][0]
    assert st["exp_avg"].device.type == "cpu" and st["master"].dtype == torch.float32 and st["step"] == 4
    oa.set_clip_coef(torch.tensor(0.5))
    a[0].grad = torch.ones_like(a[0])
    before = oa.state[a[0]]["exp_avg"].clone()
    oa.step()
    assert torch.allclose(oa.state[a[0]]["exp_avg"], before * 0.9 + 0.1 * 0.5)        # gradient scaled by the clip coefficient


def test_unpad_helpers_and_attention_interface():
    from torchturbo_b200.models.modules.attention import attention_forward
    from torchturbo_b200.ops.providers import native as N
    from torchturbo_b200.utils.flash_attn_utils import cu_seqlens_to_segment_ids, get_unpad_data, pad_input, unpad_input

    m = torch.tensor([[1, 1, 2, 2, 2, 0], [1, 1, 1, 1, 0, 0]])
    idx, cu, mx = get_unpad_data(m)
    assert idx.tolist() == [0, 1, 2, 3, 4, 6, 7, 8, 9] and cu.tolist() == [0, 2, 5, 9] and mx == 4
    x = torch.arange(12.0).view(2, 6, 1)
    assert torch.equal(pad_input(unpad_input(x, idx), idx, 2, 6), x * (m > 0).unsqueeze(-1))
    assert cu_seqlens_to_segment_ids(torch.tensor([0, 2, 5]), 7).tolist() == [1, 1, 2, 2, 2, 0, 0]
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 4, 6, 8), torch.randn(2, 2, 6, 8), torch.randn(2, 2, 6, 8)
    out, _ = attention_forward(None, q, k, v, m)
    assert out.shape == (2, 6, 4, 8) and float(out[0, 5].abs().sum()) == 0.0
    ref = N.attention_ref(q[0, :, 2:5].transpose(0, 1), k[0, :, 2:5].transpose(0, 1), v[0, :, 2:5].transpose(0, 1), [0, 3])
    assert torch.allclose(out[0, 2:5], ref, atol=1e-6)
    state = SimpleNamespace(seen=None, update=lambda ml: setattr(state, "seen", ml))
    mod = SimpleNamespace(is_causal=True, qk_clip_state=state)
    out2, _ = attention_forward(mod, q[:1], k[:1], v[:1], None, cu_seq_lens_q=torch.tensor([0, 2, 6], dtype=torch.int32), max_length_q=4)
    assert out2.shape == (1, 6, 4, 8) and state.seen.shape == (4,)
    with pytest.raises(ValueError):
        attention_forward(None, q, k, v, torch.zeros(2, 1, 6, 6))
