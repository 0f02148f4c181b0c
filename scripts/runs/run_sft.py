"""SFT / continued pre-training with the engine's own loop.

    torchrun --nproc-per-node 8 scripts/runs/run_sft.py --model /path/to/hf_checkpoint --data train.jsonl \
        --max_steps 1000 --lr 1e-5 --seq_len 8192 --output_dir out --tt_sp_size 1 --tt_ep_size 8 --tt_mixed_precision bf16

`--data` is a JSON-lines file of `{"input_ids": [...], "labels": [...]}` (labels optional: continued pre-training);
`--synthetic` trains on seeded random tokens instead; `--model_config` builds a randomly initialised model from a
`config.json`-style file.  All `--tt_*` flags, `TORCH_TURBO_*` variables and `--tt_config` files are honoured.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402
from torch.utils.data import Dataset  # noqa: E402

from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset  # noqa: E402
from torchturbo_b200.engine import TorchTurboEngine, build_from_args, parse_torchturbo_args  # noqa: E402
from torchturbo_b200.engine.args import set_torchturbo_args  # noqa: E402
from torchturbo_b200.engine.optimizers import OptimizerClassPlan  # noqa: E402
from torchturbo_b200.logging import logging_configure  # noqa: E402
from torchturbo_b200.loops import TrainingArguments, run_training  # noqa: E402


class JsonlPackedDataset(Dataset):
    """Greedy packing of tokenised documents into rows of at most `seq_len` tokens."""

    def __init__(self, path: str, seq_len: int):
        docs = [json.loads(l) for l in open(path) if l.strip()]
        self.rows, cur, n = [], [], 0
        for d in docs:
            d = {"input_ids": d["input_ids"][:seq_len], "labels": (d.get("labels") or d["input_ids"])[:seq_len]}
            if cur and n + len(d["input_ids"]) > seq_len:
                self.rows.append(cur)
                cur, n = [], 0
            cur.append(d)
            n += len(d["input_ids"])
        if cur:
            self.rows.append(cur)

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return {"documents": self.rows[i]}


def main(argv=None):
    tt_args, rest = parse_torchturbo_args(argv)
    set_torchturbo_args(tt_args)
    p = argparse.ArgumentParser()
    p.add_argument("--model")
    p.add_argument("--model_config")
    p.add_argument("--data")
    p.add_argument("--synthetic", action="store_true")
    p.add_argument("--seq_len", type=int, default=4096)
    p.add_argument("--max_steps", type=int, default=100)
    p.add_argument("--lr", type=float, default=1e-5)
    p.add_argument("--weight_decay", type=float, default=0.01)
    p.add_argument("--warmup_steps", type=int, default=0)
    p.add_argument("--lr_scheduler", default="cosine")
    p.add_argument("--gradient_accumulation_steps", type=int, default=1)
    p.add_argument("--max_grad_norm", type=float, default=1.0)
    p.add_argument("--logging_steps", type=int, default=10)
    p.add_argument("--save_steps", type=int, default=0)
    p.add_argument("--output_dir")
    p.add_argument("--resume_from_checkpoint")
    p.add_argument("--seed", type=int, default=0)
    a = p.parse_args(rest)
    logging_configure(tt_args.log_level)
    engine = TorchTurboEngine(build_from_args(tt_args))
    engine.plugins.setup(engine)
    if a.model:
        model = engine.prepare_model(a.model)
        vocab = model.config.vocab_size
    else:
        cfg = json.load(open(a.model_config))
        model = engine.prepare_model(None, load_weights=False, init_kwargs={"config": cfg, "seed": a.seed})
        vocab = cfg["vocab_size"]
    if engine.config.mfu.enabled:
        engine.enable_mfu(model)
    optim = engine.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=a.lr, weight_decay=a.weight_decay,
                                                               betas=(0.9, 0.95)))
    sched = engine.prepare_lr_scheduler(optim, a.lr_scheduler, num_warmup_steps=a.warmup_steps, num_training_steps=a.max_steps)
    ds = SyntheticPackedDataset(4096, a.seq_len, vocab, seed=a.seed) if (a.synthetic or not a.data) else JsonlPackedDataset(a.data, a.seq_len)
    ga = engine.resolve_gradient_accumulation_steps(a.gradient_accumulation_steps)
    loader = engine.create_dataloader(ds, collate_fn=PackedCollator(pin=torch.cuda.is_available()), seed=a.seed,
                                      gradient_accumulation_steps=ga)
    args = TrainingArguments(max_steps=a.max_steps, gradient_accumulation_steps=a.gradient_accumulation_steps,
                             max_grad_norm=a.max_grad_norm, logging_steps=a.logging_steps, save_steps=a.save_steps,
                             output_dir=a.output_dir, resume_from_checkpoint=a.resume_from_checkpoint,
                             profiling=bool(tt_args.profiling), memory_snapshot_steps=tt_args.memory_snapshot_steps, seed=a.seed)
    state = run_training(engine, model, loader, optim, sched, args)
    if a.output_dir and not a.save_steps:
        engine.save_model(model, os.path.join(a.output_dir, f"checkpoint-{state.step}"), final=True)
    return state


if __name__ == "__main__":
    main()
