"""Pieces shared by adapters for Hugging Face `Trainer`-based frameworks (LlamaFactory, ms-swift).

The host framework keeps owning the loop (`Trainer.train`); the mixin below reroutes the four places where the engine
must take over: data loading (DP-block sampler whose SP ranks see identical samples), loss (packed batches through
`engine.compute_loss`), gradient clipping (EP / mesh aware) and checkpointing (native sharded state + optional HF
export).  (adapters/llamafactory_v0/trainer.py:37-500 and adapters/msswift/trainer.py:122-440 of the reference.)"""
from __future__ import annotations

from typing import Any

import torch

from ..data.packing import IGNORE_INDEX
from ..engine.distributed import assert_finite
from ..engine.utils import assert_packed_inputs, get_packed_boundaries


def normalize_training_features(features: dict[str, Any]) -> dict[str, Any]:
    """Turn what a framework collator produced into the engine's packed-row contract.

    Accepts (a) an already packed row with `cu_seq_lens_q/k`, (b) a neat-packed row whose `attention_mask` holds
    sample ids (1,1,2,2,0,0), (c) a padded `[B, S]` batch with a 0/1 `attention_mask`, which is flattened with the
    padding removed.  The first label of every document is set to -100."""
    f = dict(features)
    ids = f["input_ids"]
    if f.get("cu_seq_lens_q") is None:
        mask = f.pop("attention_mask", None)
        if ids.shape[0] == 1 and mask is not None and int(mask.max()) > 1:
            cu = get_packed_boundaries(sample_ids=mask)
        elif ids.shape[0] == 1 and mask is None:
            cu = get_packed_boundaries(position_ids=f["position_ids"]) if f.get("position_ids") is not None else \
                torch.tensor([0, ids.shape[-1]], dtype=torch.int32)
        else:
            mask = mask if mask is not None else torch.ones_like(ids)
            lens = mask.sum(-1).tolist()
            keep = mask.bool()
            for k in ("input_ids", "labels"):
                if f.get(k) is not None:
                    f[k] = f[k][keep].unsqueeze(0)
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
            f.pop("position_ids", None)
        f["cu_seq_lens_q"], f["cu_seq_lens_k"] = cu, cu.clone()
    else:
        f.pop("attention_mask", None)
    cu = f["cu_seq_lens_q"].to(torch.int32).cpu()
    f["cu_seq_lens_q"], f["cu_seq_lens_k"] = cu, cu.clone()
    mx = int((cu[1:] - cu[:-1]).max())
    f["max_length_q"] = f["max_length_k"] = mx
    if f.get("position_ids") is None:
        f["position_ids"] = torch.cat([torch.arange(int(b - a)) for a, b in zip(cu[:-1], cu[1:])] +
                                      [torch.arange(f["input_ids"].shape[-1] - int(cu[-1]))]).unsqueeze(0)
    if f.get("labels") is not None:
        lab = f["labels"].clone()
        lab[0, cu[:-1].long()] = IGNORE_INDEX
        lab[0, int(cu[-1]):] = IGNORE_INDEX
        f["labels"] = lab
    assert_packed_inputs(f)
    return f


class TurboTrainerMixin:
    """Mix into a `transformers.Trainer` subclass *before* the Trainer class.  Expects `self.turbo_engine`."""

    turbo_engine = None

    def get_train_dataloader(self):
        ga = self.turbo_engine.resolve_gradient_accumulation_steps(self.args.gradient_accumulation_steps)
        self.args.gradient_accumulation_steps = ga
        return self.turbo_engine.create_dataloader(self.train_dataset, batch_size=self.args.per_device_train_batch_size,
                                                   collate_fn=self.data_collator, seed=self.args.seed,
                                                   gradient_accumulation_steps=ga,
                                                   num_workers=self.args.dataloader_num_workers)

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        eng = self.turbo_engine
        inputs = normalize_training_features(inputs)
        res = eng.compute_loss(model, inputs, num_items_in_batch=num_items_in_batch,
                               gradient_accumulation_steps=self.args.gradient_accumulation_steps, return_outputs=True)
        loss, out = res
        if num_items_in_batch is None and eng.backend.sp_size > 1:
            loss = loss * eng.backend.sp_size
        return (loss, out) if return_outputs else loss

    def training_step(self, model, inputs, num_items_in_batch=None):
        model.train()
        loss = self.compute_loss(model, inputs, num_items_in_batch=num_items_in_batch)
        self.accelerator.backward(loss) if hasattr(self, "accelerator") else loss.backward()
        assert_finite(loss.detach(), "loss")
        self.turbo_engine.collect_metrics(model)
        return loss.detach() / self.args.gradient_accumulation_steps

    def _clip_grad_norm(self, model, max_norm):
        return self.turbo_engine.clip_grad_norm_(model, max_norm, getattr(self, "optimizer", None))

    def save_model(self, output_dir=None, _internal_call=False):
        output_dir = output_dir or self.args.output_dir
        self.turbo_engine.save_model(self.model, output_dir, final=not _internal_call)

    def _save_optimizer_and_scheduler(self, output_dir):
        self.turbo_engine.save_optimizer_and_scheduler(self.model, self.optimizer, self.lr_scheduler, output_dir)

    def _load_from_checkpoint(self, resume_from_checkpoint, model=None):
        self.turbo_engine.load_from_checkpoint(model or self.model, resume_from_checkpoint)

    def _load_optimizer_and_scheduler(self, checkpoint):
        if checkpoint:
            self.turbo_engine.load_optimizer_and_scheduler(self.model, self.optimizer, self.lr_scheduler, checkpoint)

    def log(self, logs, *args, **kwargs):
        self.turbo_engine.report_metrics(logs, gather=None)
        return super().log(logs, *args, **kwargs)
