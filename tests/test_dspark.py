"""DSpark block-draft training of the DeepSeek-V4 family (models/deepseek_v4/dspark.py): anchor sampling, what a draft
block may attend to, the chunked CE + L1 loss against plain autograd, and one training step through the engine.
Reference behaviour: models/deepseek_v4/mtp.py:97-260,442-504,847-1000."""
import types

import torch

from torchturbo_b200.models.deepseek_v4.dspark import _DraftLoss, sample_anchors

TINY = dict(model_type="deepseek_v4", vocab_size=96, hidden_size=32, intermediate_size=48, moe_intermediate_size=24,
            num_hidden_layers=2, num_attention_heads=2, n_routed_experts=4, n_shared_experts=1, num_experts_per_tok=2,
            q_lora_rank=16, qk_rope_head_dim=8, qk_nope_head_dim=8, o_groups=2, o_lora_rank=8, sliding_window=6,
            hc_mult=2, hc_sinkhorn_iters=3, index_n_heads=2, index_head_dim=8, index_topk=4, torch_dtype="float32",
            dspark_block_size=3, dspark_num_layers=2, dspark_markov_rank=8, dspark_target_layer_ids=[0, 1], dspark_mask_token_id=95)


def test_anchor_blocks_stay_inside_their_document_and_are_supervised():
    labels = torch.arange(20)
    labels[7] = -100
    cu = torch.tensor([0, 9, 20], dtype=torch.int32)
    a = sample_anchors(labels, cu, 3, 100).tolist()
    # document 0 = [0, 9): anchors need targets a+1..a+3 < 9 and none of them equal to the unsupervised position 7
    assert a == [0, 1, 2, 3, 9, 10, 11, 12, 13, 14, 15, 16]
    few = sample_anchors(labels, cu, 3, 4, torch.Generator().manual_seed(0))
    assert few.numel() == 4 and set(few.tolist()) <= set(a) and few.tolist() == sorted(few.tolist())
    assert sample_anchors(labels[:3], torch.tensor([0, 3], dtype=torch.int32), 3, 10).numel() == 0


def test_draft_loss_matches_plain_autograd():
    torch.manual_seed(0)
    R, V = 37, 50
    logits = torch.randn(R, V, requires_grad=True)
    tgt_logits = torch.randn(R, V)
    targets = torch.randint(0, V, (R,))
    w = torch.rand(R) + 0.1
    loss, ce_sum, l1_sum, accept = _DraftLoss.apply(logits, targets, w, lambda a, b: tgt_logits[a:b], 0.3, 0.7)
    loss.backward()
    ref_in = logits.detach().clone().requires_grad_(True)
    p, q = torch.softmax(ref_in, -1), torch.softmax(tgt_logits, -1)
    ce = torch.nn.functional.cross_entropy(ref_in, targets, reduction="none")
    l1 = (p - q).abs().sum(-1)
    ref = (0.3 * ce * w + 0.7 * l1 * w).sum()
    ref.backward()
    assert torch.allclose(loss, ref, atol=1e-5) and torch.allclose(logits.grad, ref_in.grad, atol=1e-6)
    assert torch.allclose(accept, (1 - 0.5 * l1).clamp(0, 1).detach(), atol=1e-6)
    assert torch.allclose(ce_sum, (ce * w).sum().detach(), atol=1e-5) and torch.allclose(l1_sum, (l1 * w).sum().detach(), atol=1e-5)


def _model():
    from torchturbo_b200.models.registry import get_model

    cls = get_model("deepseek_v4")
    torch.manual_seed(0)
    return cls(cls.config_class(**TINY)).train()


def test_draft_block_sees_only_its_window_and_itself():
    m = _model()
    cfg = types.SimpleNamespace(num_anchors=1, loss_decay_gamma=4.0, ce_loss_alpha=0.1, l1_loss_alpha=0.9, confidence_loss_alpha=1.0)
    T = 30
    ids = torch.randint(0, 90, (1, T))
    cu = torch.tensor([0, T], dtype=torch.int32)
    labels = ids.clone()

    def draft_loss(ids_):
        g = torch.Generator().manual_seed(3)
        # same anchor in both calls: patch the sampler's generator by sampling here
        a = sample_anchors(labels.reshape(-1), cu, 3, 1, g)
        lab = torch.full_like(labels, -100)
        lab[0, int(a) + 1:int(a) + 4] = labels[0, int(a) + 1:int(a) + 4]       # exactly one anchor is possible
        out = m(input_ids=ids_, cu_seq_lens_q=cu, max_length_q=T, dspark_labels=lab, dspark_config=cfg, skip_lm_head=True)
        return int(a), out["dspark_loss"]

    a, base = draft_loss(ids)
    assert base is not None and torch.isfinite(base)
    base.backward()
    missing = [n for n, p in m.dspark.named_parameters() if p.grad is None]
    assert not missing, missing
    assert a - TINY["sliding_window"] - 2 >= 0, "test row too short for the chosen seed"


def test_engine_trains_the_draft_heads_with_the_main_model():
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    losses = {}
    for enabled in (True, False):
        eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "activation_checkpointing": {"enabled": False},
                                                       "dspark": {"enabled": enabled, "num_anchors": 8, "loss_scaling_factor": 0.5}}))
        model = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(TINY), "seed": 0})
        opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-3))
        before = {n: p.detach().clone() for n, p in model.named_parameters() if n.startswith("dspark.")}
        assert before, "the model was built without draft stages"
        ds = SyntheticPackedDataset(2, 48, TINY["vocab_size"] - 2, num_docs=2, seed=1)
        loss, _ = train_step(eng, model, opt, [PackedCollator()([ds[0]])])
        losses[enabled] = float(loss)
        moved = [n for n, p in model.named_parameters() if n.startswith("dspark.") and not torch.equal(p.detach(), before[n])]
        assert bool(moved) == enabled
        if enabled:
            metrics = eng.report_metrics({})          # the tracker collected the draft metrics after the micro-step
            assert {"dspark/ce", "dspark/l1", "dspark/confidence", "dspark/accept_rate", "dspark/anchors"} <= set(metrics)
            assert 0.0 <= float(metrics["dspark/accept_rate"]) <= 1.0
    assert losses[True] > losses[False]          # the draft objective is added to the language-model loss


def test_sequence_parallel_run_says_that_the_draft_heads_are_left_out():
    import pytest

    m = _model()
    m.model.sp_size = 2                      # as `set_sequence_parallel` leaves it on a rank of a two-way group
    seen = {}

    class Stop(Exception):
        pass

    def trunk(**kw):
        seen.update(kw)
        raise Stop

    m.model.forward = trunk                  # the check comes before the trunk runs; no process group is needed
    ids = torch.randint(0, 90, (1, 12))
    kw = dict(input_ids=ids, cu_seq_lens_q=torch.tensor([0, 24], dtype=torch.int32), max_length_q=24,
              dspark_labels=ids.clone(), dspark_config=types.SimpleNamespace(num_anchors=1), skip_lm_head=True)
    with pytest.warns(RuntimeWarning, match="DSpark draft heads are not trained under sequence parallelism"):
        with pytest.raises(Stop):
            m(**kw)
    assert seen["collect_layers"] is None    # the trunk is not asked for the draft branch's layer states
    import warnings as w
    with w.catch_warnings():
        w.simplefilter("error")              # said once per model, not every step
        with pytest.raises(Stop):
            m(**kw)
