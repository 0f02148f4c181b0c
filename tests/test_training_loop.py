"""`loops.run_training`: gradient accumulation, scheduler stepping, logging history, periodic checkpoints and a resume that
continues exactly where the uninterrupted run went (one rank and two data-parallel ranks)."""
import os

import pytest
import torch

from dist_utils import run_distributed

DENSE = dict(model_type="qwen3", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
             intermediate_size=128, vocab_size=256, tie_word_embeddings=True)


def _w_loop(rank, world, root):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.engine.optimizers.lr_scheduler import create_lr_scheduler
    from torchturbo_b200.loops import run_training
    from torchturbo_b200.loops.sft import TrainingArguments

    ds = SyntheticPackedDataset(8, 64, 256, num_docs=3, seed=7)
    data = [PackedCollator()([ds[rank * 4 + i]]) for i in range(4)]          # a fixed cycle of four micro-batches per rank

    def run(out, max_steps, resume=None):
        eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "activation_checkpointing": {"enabled": False},
                                                       "checkpoint": {"hf_export": "final"}}))
        model = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(DENSE), "seed": 0})
        opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-2, weight_decay=0.01))
        sched = create_lr_scheduler("cosine", opt, num_warmup_steps=1, num_training_steps=6)
        logs = []
        state = run_training(eng, model, data, opt, sched, TrainingArguments(
            max_steps=max_steps, gradient_accumulation_steps=2, logging_steps=1, save_steps=2, output_dir=out,
            resume_from_checkpoint=resume), on_log=logs.append)
        return state, logs

    full, logs_full = run(os.path.join(root, "full"), 4)
    assert full.step == 4 and full.epoch == 1 and full.tokens_seen == 4 * 2 * 64
    assert [l["step"] for l in logs_full] == [1, 2, 3, 4] and logs_full[-1]["loss"] < logs_full[0]["loss"]
    assert logs_full[0]["lr"] > logs_full[-1]["lr"] > 0.0                     # cosine after one warm-up step
    for step in (2, 4):
        ck = os.path.join(root, "full", f"checkpoint-{step}")
        assert os.path.isdir(os.path.join(ck, "model_distcp")) and os.path.isdir(os.path.join(ck, "optimizer_distcp"))
        assert os.path.isdir(os.path.join(ck, "huggingface")) == (step == 4)    # Hugging Face export at the end only
    half, _ = run(os.path.join(root, "half"), 2)
    assert half.step == 2
    resumed, logs_res = run(os.path.join(root, "half"), 4, resume=os.path.join(root, "half", "checkpoint-2"))
    assert resumed.step == 4 and [l["step"] for l in logs_res] == [3, 4]
    for a, b in zip(logs_full[2:], logs_res):
        assert abs(a["loss"] - b["loss"]) < 1e-5 and abs(a["grad_norm"] - b["grad_norm"]) < 1e-4 and abs(a["lr"] - b["lr"]) < 1e-9, (a, b)


@pytest.mark.parametrize("world", [1, 2])
def test_training_loop_accumulates_checkpoints_and_resumes_exactly(tmp_path, world):
    run_distributed(_w_loop, world, str(tmp_path), timeout=900)
