"""Ulysses sequence parallelism on the hybrid families: two training steps on two ranks with sp = 2 give the losses and
gradient norms of sp = 1 (gated delta net and KDA with head-parallel recurrences, multi-head latent attention, sparse
attention with an indexer, prediction-depth heads)."""
import copy

import pytest
import torch

from dist_utils import run_distributed
from test_model_families import DSV3, MLA, QMOE, QWEN35, TEXT

CONFIGS = {
    "qwen3_5_moe_text": dict(QWEN35, **QMOE, model_type="qwen3_5_moe_text", num_attention_heads=4, num_key_value_heads=2),
    "bailing_hybrid": dict(TEXT, model_type="bailing_hybrid", num_hidden_layers=5, head_dim=8, num_experts=8, num_experts_per_tok=2,
                           n_group=2, topk_group=1, moe_intermediate_size=16, moe_shared_expert_intermediate_size=16,
                           layer_group_size=3, num_nextn_predict_layers=1, pad_token_id=0,
                           gated_attention_proj_granularity_type="head_wise", **MLA),
    "glm_moe_dsa": dict(DSV3, model_type="glm_moe_dsa", num_hidden_layers=4, n_group=1, num_nextn_predict_layers=0, index_topk=6,
                        index_head_dim=8, index_n_heads=2, index_topk_freq=2, index_skip_topk_offset=1,
                        mlp_layer_types=["dense", "sparse", "sparse", "sparse"]),
    "deepseek_v4": dict(TEXT, model_type="deepseek_v4", moe_intermediate_size=16, num_hidden_layers=3, n_routed_experts=8,
                        num_experts_per_tok=2, q_lora_rank=16, qk_rope_head_dim=4, qk_nope_head_dim=12, o_groups=2, o_lora_rank=8,
                        sliding_window=4, compress_ratios=[1, 4, 2], index_n_heads=2, index_head_dim=8, index_topk=2, hc_mult=2,
                        hc_sinkhorn_iters=3, swiglu_limit=7.0, num_hash_layers=1, num_mtp_layers=1),
}


def _w(rank, world, kind, sp, out):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "parallel_plan": {"sp_size": sp, "ep_size": 1},
                                                   "moe": {"aux_loss_coeff": 1e-2}, "activation_checkpointing": {"enabled": True}}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": copy.deepcopy(CONFIGS[kind]), "seed": 0})
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-2, weight_decay=0.0))
    ds = SyntheticPackedDataset(2, 64, 128, num_docs=3, seed=11)
    hist = []
    for i in range(2):
        loss, gn = train_step(eng, model, opt, [PackedCollator()([ds[i]])])       # the same rows on every rank
        hist.append([float(loss), float(gn)])
    if rank == 0:
        torch.save(torch.tensor(hist), out)


@pytest.mark.parametrize("kind", sorted(CONFIGS))
def test_sequence_parallel_two_matches_one(tmp_path, kind):
    run_distributed(_w, 2, kind, 1, str(tmp_path / "sp1.pt"), timeout=900)
    run_distributed(_w, 2, kind, 2, str(tmp_path / "sp2.pt"), timeout=900)
    a, b = torch.load(tmp_path / "sp1.pt"), torch.load(tmp_path / "sp2.pt")
    assert torch.isfinite(a).all()
    assert torch.allclose(a[:, 0], b[:, 0], rtol=2e-4, atol=2e-5), (kind, a, b)
    assert torch.allclose(a[:, 1], b[:, 1], rtol=5e-3, atol=1e-4), (kind, a, b)
