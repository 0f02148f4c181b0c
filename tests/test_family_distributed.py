"""Hybrid and vision-language families through the engine on two ranks: expert parallelism gives the losses of one expert
group, and every vision-language family trains a step with its default plan when one rank's row carries no image."""
import copy

import pytest
import torch

from dist_utils import run_distributed
from test_family_sequence_parallel import CONFIGS
from test_model_families import DSV3, MLA, QMOE, QWEN35, TEXT, VISION


def _w_ep(rank, world, kind, ep, out):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "parallel_plan": {"sp_size": 1, "ep_size": ep},
                                                   "moe": {"aux_loss_coeff": 1e-2}, "activation_checkpointing": {"enabled": False}}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": copy.deepcopy(CONFIGS[kind]), "seed": 0})
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-2, weight_decay=0.0))
    ds = SyntheticPackedDataset(4, 64, 128, num_docs=3, seed=13)
    hist = []
    for i in range(2):
        loss, gn = train_step(eng, model, opt, [PackedCollator()([ds[2 * i + rank]])])      # different rows per rank
        hist.append([float(loss), float(gn)])
    if rank == 0:
        torch.save(torch.tensor(hist), out)


@pytest.mark.parametrize("kind", ["qwen3_5_moe_text", "bailing_hybrid", "deepseek_v4"])
def test_expert_parallel_two_matches_one(tmp_path, kind):
    run_distributed(_w_ep, 2, kind, 1, str(tmp_path / "ep1.pt"), timeout=900)
    run_distributed(_w_ep, 2, kind, 2, str(tmp_path / "ep2.pt"), timeout=900)
    a, b = torch.load(tmp_path / "ep1.pt"), torch.load(tmp_path / "ep2.pt")
    assert torch.isfinite(a).all()
    assert torch.allclose(a[:, 0], b[:, 0], rtol=2e-4, atol=2e-5), (kind, a, b)
    assert torch.allclose(a[:, 1], b[:, 1], rtol=5e-3, atol=1e-4), (kind, a, b)


VLMS = {
    "qwen3_5": (dict(model_type="qwen3_5", text_config=dict(QWEN35), vision_config=dict(VISION), image_token_id=5), "image_grid_thw"),
    "qwen3_5_moe": (dict(model_type="qwen3_5_moe", text_config=dict(QWEN35, **QMOE), vision_config=dict(VISION), image_token_id=5),
                    "image_grid_thw"),
    "bailing_moe_v3_vl": (dict(model_type="bailing_moe_v3_vl", vision_config=dict(VISION), image_patch_token=5, video_patch_token=4,
                               text_config=dict(TEXT, num_hidden_layers=5, head_dim=8, num_experts=8, num_experts_per_tok=2, n_group=2,
                                                topk_group=1, moe_intermediate_size=16, moe_shared_expert_intermediate_size=16,
                                                layer_group_size=3, num_nextn_predict_layers=1, pad_token_id=0, **MLA)),
                          "image_grid_thw"),
    "kimi_k25": (dict(model_type="kimi_k25", text_config=dict(DSV3), media_placeholder_token_id=5,
                      vision_config=dict(vt_num_hidden_layers=1, vt_hidden_size=16, vt_num_attention_heads=2, vt_intermediate_size=32,
                                         patch_size=2, merge_kernel_size=(2, 2))), "grid_thws"),
}


def _w_vlm(rank, world, kind):
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    cfg, grid_key = VLMS[kind]
    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "activation_checkpointing": {"enabled": True},
                                                   "moe": {"aux_loss_coeff": 1e-2}}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": copy.deepcopy(cfg), "seed": 0})
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-3))
    g = torch.Generator().manual_seed(17 + rank)
    for step in range(2):
        ids = torch.randint(6, 128, (1, 24), generator=g)
        b = dict(input_ids=ids, labels=ids.clone(), position_ids=torch.cat((torch.arange(10), torch.arange(14)))[None],
                 cu_seq_lens_q=torch.tensor([0, 10, 24], dtype=torch.int32), cu_seq_lens_k=torch.tensor([0, 10, 24], dtype=torch.int32),
                 max_length_q=14, max_length_k=14)
        if (rank + step) % 2 == 0:               # the ranks take turns at having an image
            ids[0, 3:7] = 5
            b["labels"] = ids.clone()
            b["pixel_values"] = torch.randn(16, 3 * 1 * 2 * 2, generator=g)
            b[grid_key] = torch.tensor([[1, 4, 4]])
        loss, gn = train_step(eng, model, opt, [b])
        assert torch.isfinite(torch.as_tensor(loss)) and torch.isfinite(torch.as_tensor(gn))


@pytest.mark.parametrize("kind", sorted(VLMS))
def test_vision_language_families_train_on_two_ranks_with_a_media_less_rank(kind):
    run_distributed(_w_vlm, 2, kind, timeout=900)
