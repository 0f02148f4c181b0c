"""Adapter-side batch normalisation (ms-swift bridging, HF-trainer features) and config construction from host
framework arguments."""
from types import SimpleNamespace

import pytest
import torch

from torchturbo_b200.adapters.hf_trainer import normalize_training_features
from torchturbo_b200.adapters.msswift import (SwiftInputCollator, bake_loss_scale_into_labels, bridge_packed_inputs,
                                              bridge_unpacked_inputs, build_config_from_swift_args)


def test_bridge_packed_left_padding_and_labels():
    # two samples of 3 and 2 tokens, 3 alignment pads on the left
    ids = torch.tensor([[0, 0, 0, 11, 12, 13, 21, 22]])
    lab = ids.clone()
    pos = torch.tensor([[0, 0, 0, 0, 1, 2, 0, 1]])
    out = bridge_packed_inputs({"input_ids": ids, "labels": lab, "position_ids": pos, "attention_mask": torch.ones(1, 8)},
                               sequence_lengths=[3, 2], padding_side="left")
    assert out["input_ids"][0].tolist() == [11, 12, 13, 21, 22, 0, 0, 0]
    assert out["cu_seq_lens_q"].tolist() == [0, 3, 5] and out["max_length_q"] == 3 and "attention_mask" not in out
    assert out["labels"][0].tolist()[:5] == [-100, 12, 13, -100, 22]
    assert out["position_ids"][0].tolist()[:5] == [0, 1, 2, 0, 1]
    with pytest.raises(ValueError):
        bridge_packed_inputs({"input_ids": ids}, sequence_lengths=[9], padding_side="right")
    with pytest.raises(ValueError):
        bridge_packed_inputs({"input_ids": torch.tensor([[1, 2, 3]]), "cu_seq_lens_q": torch.tensor([0, 1, 3], dtype=torch.int32)},
                             sequence_lengths=[2, 1])


def test_bridge_unpacked_rows_become_sequences():
    ids = torch.tensor([[1, 2, 3, 0], [4, 5, 0, 0]])
    mask = torch.tensor([[1, 1, 1, 0], [1, 1, 0, 0]])
    out = bridge_unpacked_inputs({"input_ids": ids, "labels": ids.clone(), "attention_mask": mask})
    assert out["input_ids"].tolist() == [[1, 2, 3, 4, 5]] and out["cu_seq_lens_k"].tolist() == [0, 3, 5]
    assert out["position_ids"].tolist() == [[0, 1, 2, 0, 1]] and out["labels"].tolist() == [[-100, 2, 3, -100, 5]]
    pos3 = torch.arange(8).view(1, 2, 4).expand(3, 2, 4)
    out = bridge_unpacked_inputs({"input_ids": ids, "attention_mask": mask, "position_ids": pos3,
                                  "text_position_ids": torch.zeros(2, 4, dtype=torch.long)})
    assert out["position_ids"].shape == (3, 1, 5) and out["position_ids"][0, 0].tolist() == [0, 1, 2, 4, 5]
    assert out["text_position_ids"].tolist() == [[0, 1, 2, 0, 1]]


def test_loss_scale_is_folded_into_labels():
    out = bake_loss_scale_into_labels({"labels": torch.tensor([[5, 6, 7]]), "loss_scale": torch.tensor([[1.0, 0.0, 1.0]])})
    assert out["labels"].tolist() == [[5, -100, 7]] and "loss_scale" not in out
    same = {"labels": torch.tensor([[5, 6]])}
    assert bake_loss_scale_into_labels(same) is same


def test_swift_collator_dpo_orders_chosen_then_rejected():
    template = SimpleNamespace(mode="rlhf", padding_free=True, is_training=True, padding_side="right")

    def inner(batch):
        rows = [s["chosen_input_ids"] for s in batch] + [s["rejected_input_ids"] for s in batch]
        flat = [t for r in rows for t in r]
        return {"input_ids": torch.tensor([flat]), "labels": torch.tensor([flat])}

    batch = [{"chosen_input_ids": [1, 2, 3], "rejected_input_ids": [1, 9]}, {"chosen_input_ids": [4, 5], "rejected_input_ids": [4, 8, 7]}]
    out = SwiftInputCollator(inner, template)(batch)
    assert out["cu_seq_lens_q"].tolist() == [0, 3, 5, 7, 10] and out["max_length_q"] == 3


def test_hf_features_neat_packing_and_padding():
    f = normalize_training_features({"input_ids": torch.tensor([[1, 2, 3, 4, 5, 0]]), "labels": torch.tensor([[1, 2, 3, 4, 5, 0]]),
                                     "attention_mask": torch.tensor([[1, 1, 2, 2, 2, 0]])})
    assert f["cu_seq_lens_q"].tolist() == [0, 2, 5] and f["labels"][0].tolist() == [-100, 2, -100, 4, 5, -100]
    f = normalize_training_features({"input_ids": torch.tensor([[1, 2, 0], [3, 4, 5]]), "labels": torch.tensor([[1, 2, 0], [3, 4, 5]]),
                                     "attention_mask": torch.tensor([[1, 1, 0], [1, 1, 1]])})
    assert f["input_ids"].tolist() == [[1, 2, 3, 4, 5]] and f["cu_seq_lens_q"].tolist() == [0, 2, 5]


def test_swift_args_force_engine_ownership():
    from torchturbo_b200.engine.args import parse_torchturbo_args

    args = SimpleNamespace(bf16=True, gradient_checkpointing=True, sequence_parallel_size=4, deepspeed="zero3", fsdp="full_shard",
                           router_aux_loss_coef=0.01)
    tt, _ = parse_torchturbo_args(["--tt_sp_size", "2"])
    cfg = build_config_from_swift_args(args, "dpo", tt)
    assert args.gradient_checkpointing is False and args.sequence_parallel_size == 1 and args.deepspeed is None and args.fsdp == ""
    assert cfg.parallel_plan.sp_size == 2 and cfg.moe.aux_loss_coeff == pytest.approx(0.01)
    assert cfg.activation_checkpointing.enabled is True
