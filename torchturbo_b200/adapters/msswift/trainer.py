"""Trainer layer of the ms-swift adapter.

`EngineTrainerMixin` goes in front of swift's `Seq2SeqTrainer` (SFT, PT) and, through `EngineDPOTrainerMixin`, in
front of swift's `DPOTrainer`.  swift / HF keep the loop, logging and callbacks; the engine owns data loading
(DP-block sampler, SP-compensated gradient accumulation resolved at construction so the run summary shows the real
value), the collator (swift's template output bridged to packed rows), loss, clipping, optimizer / schedule,
checkpoints and profiling.  accelerate is reduced to a pass-through on the instance (`prepare_model`, `backward`,
`clip_grad_norm_`), because the model arrives sharded.
(adapters/msswift/trainer.py:49-686 of the reference.)"""
from __future__ import annotations

import os
from typing import Any

import torch

from ...engine.distributed import assert_finite
from ...logging import get_logger
from . import session
from .inputs_bridging import SwiftInputCollator

logger = get_logger(__name__)


def install_clip_override(trainer: Any, engine: Any) -> None:
    """`accelerator.clip_grad_norm_` -> engine clipping (global norm over FSDP shards and EP-local experts)."""
    acc = getattr(trainer, "accelerator", None)
    if acc is None:
        return

    def clip(parameters, max_norm, *args, **kwargs):
        return engine.clip_grad_norm_(trainer.model, max_norm, getattr(trainer, "optimizer", None))

    acc.clip_grad_norm_ = clip


def install_accelerator_overrides(trainer: Any, engine: Any) -> None:
    acc = getattr(trainer, "accelerator", None)
    if acc is None:
        return
    if getattr(acc, "is_fsdp2", False) or getattr(getattr(acc, "state", None), "fsdp_plugin", None) is not None:
        raise RuntimeError("accelerate's FSDP plugin must be off: the engine has already sharded the model")

    def prepare_model(model, device_placement=None, evaluation_mode=False):
        models = getattr(acc, "_models", None)
        if models is not None and model not in models:
            models.append(model)
        return model

    def backward(loss, **kwargs):
        loss.backward(**{k: v for k, v in kwargs.items() if k in ("retain_graph", "inputs")})

    def prepare_optimizer(optimizer, device_placement=None):
        return optimizer          # optimizer-state placement belongs to the engine (sharded / host-resident states)

    acc.prepare_model, acc.backward, acc.prepare_optimizer = prepare_model, backward, prepare_optimizer


class EngineTrainerMixin:
    def __init__(self, *args, **kwargs):
        self._plugin_collator = kwargs.pop("plugin_collator", None)
        super().__init__(*args, **kwargs)
        eng = session.get_engine_or_none()
        if eng is None:
            return
        self.args.gradient_accumulation_steps = eng.resolve_gradient_accumulation_steps(self.args.gradient_accumulation_steps)
        install_clip_override(self, eng)
        install_accelerator_overrides(self, eng)
        self._profiling_callback_added = False

    # -- placement / wrapping -----------------------------------------------------------------------------
    def _move_model_to_device(self, model, _device):
        return model

    def _wrap_model(self, model, training=True, dataloader=None, **kwargs):
        return model

    # -- checkpoints ---------------------------------------------------------------------------------------
    def _is_final_save(self) -> bool:
        """swift writes its last weights through the checkpoint path: the final save is the checkpoint of the last
        step (or the one taken when training was told to stop)."""
        st = getattr(self, "state", None)
        if st is None:
            return False
        return bool(getattr(st, "global_step", 0) >= getattr(st, "max_steps", 1 << 62) or
                    getattr(getattr(self, "control", None), "should_training_stop", False))

    def _save_model(self, output_dir=None, state_dict=None):
        return None               # weights are written by save_model(); HF must not gather a DTensor state dict

    def save_model(self, output_dir=None, _internal_call=False):
        eng = session.get_engine()
        output_dir = output_dir or self.args.output_dir
        os.makedirs(output_dir, exist_ok=True)
        if _internal_call and not getattr(self.args, "save_only_model", False):
            eng.save_model(self.model, output_dir, final=self._is_final_save())
        else:
            eng.save_model(self.model, output_dir, final=True)
        parent = super()
        if hasattr(parent, "save_model"):
            parent.save_model(output_dir, _internal_call=_internal_call)   # training args, tokenizer, args.json

    def _save_optimizer_and_scheduler(self, output_dir: str) -> None:
        session.get_engine().save_optimizer_and_scheduler(self.model, self.optimizer, self.lr_scheduler, output_dir)

    def _load_from_checkpoint(self, resume_from_checkpoint, model=None):
        session.get_engine().load_from_checkpoint(self.model, resume_from_checkpoint)

    def _load_optimizer_and_scheduler(self, checkpoint):
        if checkpoint:
            session.get_engine().load_optimizer_and_scheduler(self.model, self.optimizer, self.lr_scheduler, checkpoint)

    # -- optimizer / schedule -------------------------------------------------------------------------------
    def create_optimizer(self, model=None):
        if getattr(self, "optimizer", None) is not None:
            return self.optimizer
        from ...engine.optimizers import OptimizerClassPlan

        eng, a = session.get_engine(), self.args
        opt_cfg = getattr(eng.config, "optimizer", None)
        if opt_cfg is not None and getattr(opt_cfg, "name", None):
            self.optimizer = eng.prepare_optimizer(self.model)
        else:
            self.optimizer = eng.prepare_optimizer(self.model, OptimizerClassPlan(
                torch.optim.AdamW, lr=a.learning_rate, weight_decay=a.weight_decay,
                betas=(getattr(a, "adam_beta1", 0.9), getattr(a, "adam_beta2", 0.999)), eps=getattr(a, "adam_epsilon", 1e-8)))
        return self.optimizer

    def create_scheduler(self, num_training_steps: int, optimizer=None):
        if getattr(self, "lr_scheduler", None) is None:
            a = self.args
            warm = a.get_warmup_steps(num_training_steps) if hasattr(a, "get_warmup_steps") else int(getattr(a, "warmup_steps", 0))
            self.lr_scheduler = session.get_engine().prepare_lr_scheduler(
                optimizer or self.optimizer, str(getattr(a.lr_scheduler_type, "value", a.lr_scheduler_type)),
                num_warmup_steps=warm, num_training_steps=num_training_steps, **(getattr(a, "lr_scheduler_kwargs", None) or {}))
        return self.lr_scheduler

    # -- data -------------------------------------------------------------------------------------------------
    def _get_data_collator(self, args, template):
        if self._plugin_collator is not None:
            return self._plugin_collator
        return SwiftInputCollator(super()._get_data_collator(args, template), template)

    def get_train_dataloader(self, skip_batches=0):
        eng = session.get_engine_or_none()
        if eng is None or self.train_dataset is None:
            return super().get_train_dataloader(skip_batches=skip_batches)
        a = self.args
        return eng.create_dataloader(self.train_dataset, batch_size=getattr(self, "_train_batch_size", a.per_device_train_batch_size),
                                     shuffle=getattr(a, "train_dataloader_shuffle", True), seed=getattr(a, "data_seed", None) or a.seed,
                                     collate_fn=self.data_collator, num_workers=a.dataloader_num_workers,
                                     pin_memory=getattr(a, "dataloader_pin_memory", True), drop_last=True,
                                     gradient_accumulation_steps=a.gradient_accumulation_steps)

    # -- loop bracketing ---------------------------------------------------------------------------------------
    def train(self, *args, **kwargs):
        from ...engine.args import get_torchturbo_args

        eng = session.get_engine()
        tt = get_torchturbo_args()
        profiling, snap = bool(getattr(tt, "profiling", False)), getattr(tt, "memory_snapshot_steps", None)
        started = False
        if profiling or snap:
            if not getattr(self, "_profiling_callback_added", False) and hasattr(self, "add_callback"):
                self.add_callback(self._make_profiling_callback())
                self._profiling_callback_added = True
            eng.start_profiling(self.args.output_dir, profiling_enabled=profiling, memory_snapshot_steps=snap)
            started = True
        try:
            return super().train(*args, **kwargs)
        finally:
            if started:
                eng.stop_profiling()

    def _make_profiling_callback(self):
        eng = session.get_engine()
        try:
            from transformers import TrainerCallback
        except Exception:  # noqa: BLE001
            TrainerCallback = object

        class _Step(TrainerCallback):
            def on_step_end(self, args, state, control, **kw):
                eng.step_profiling()
                return control

        return _Step()

    # -- loss / metrics -------------------------------------------------------------------------------------------
    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        eng = session.get_engine_or_none()
        if eng is None:
            return super().compute_loss(model, inputs, return_outputs, num_items_in_batch)
        for k in ("compute_loss_func", "loss_scale", "logits_to_keep"):
            inputs.pop(k, None)
        ga = getattr(self, "current_gradient_accumulation_steps", self.args.gradient_accumulation_steps) if model.training else 1
        loss, out = eng.compute_loss(model, inputs, return_outputs=True, num_items_in_batch=num_items_in_batch,
                                     gradient_accumulation_steps=ga)
        sp = eng.get_sp_info()["sp_size"]
        if num_items_in_batch is None and sp > 1:
            loss = loss * sp      # HF divides by the SP-expanded accumulation window
        return (loss, out) if return_outputs else loss

    def training_step(self, model, inputs, *args, **kwargs):
        result = super().training_step(model, inputs, *args, **kwargs)
        eng = session.get_engine_or_none()
        if eng is not None:
            assert_finite(result, "loss")
            eng.collect_metrics(model)
        return result

    def log(self, logs, *args, **kwargs):
        eng = session.get_engine_or_none()
        if eng is not None:
            acc = getattr(self, "accelerator", None)
            eng.report_metrics(logs, getattr(acc, "gather", None))
        return super().log(logs, *args, **kwargs)


class EngineDPOTrainerMixin(EngineTrainerMixin):
    """DPO over swift's packed pairwise rows (`2N` segments: chosen first, then rejected).  Log-probabilities are
    summed per segment shard by shard (`loops.dpo.sequence_logps`; SP ranks are combined with one all-reduce) and
    handed to the base trainer's `dpo_loss`, so every loss type trl defines on (policy, reference) log-probs works."""

    def __init__(self, model=None, ref_model=None, *args, **kwargs):
        super().__init__(model, ref_model, *args, **kwargs)
        if ref_model is not None:
            ref_model.requires_grad_(False)
            ref_model.eval()

    def _dpo_config(self, for_reference: bool):
        from ...loops.dpo import DPOConfig

        lt = getattr(self, "loss_type", "sigmoid")
        lt = lt[0] if isinstance(lt, (list, tuple)) else lt
        return DPOConfig(beta=float(getattr(self, "beta", 0.1)), loss_type="ipo" if lt == "ipo" else "sigmoid",
                         ld_alpha=None if for_reference else getattr(self, "ld_alpha", None))

    def concatenated_forward(self, model, batch, is_ref_model: bool = False):
        from ...loops.dpo import sequence_logps

        cfg = self._dpo_config(is_ref_model)
        grad = (not is_ref_model) and torch.is_grad_enabled()
        sums, counts = sequence_logps(session.get_engine(), model, batch, cfg, grad=grad)
        if cfg.loss_type == "ipo":
            sums = sums / counts.clamp(min=1)
        n = sums.numel() // 2
        out = {"chosen_logps": sums[:n], "rejected_logps": sums[n:], "num_chosen_tokens": counts[:n]}
        nll = -(sums[:n] if cfg.loss_type != "ipo" else sums[:n] * counts[:n].clamp(min=1)).sum() / counts[:n].sum().clamp(min=1)
        out["nll_loss"] = nll
        return out

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        pol = self.concatenated_forward(model, inputs)
        if inputs.get("ref_chosen_logps") is not None:
            rc, rr = inputs["ref_chosen_logps"], inputs["ref_rejected_logps"]
        else:
            with torch.no_grad():
                ref = self.concatenated_forward(self.ref_model, inputs, is_ref_model=True)
            rc, rr = ref["chosen_logps"], ref["rejected_logps"]
        losses, chosen_rewards, rejected_rewards = self.dpo_loss(pol["chosen_logps"], pol["rejected_logps"], rc, rr)[:3]
        loss = losses.mean()
        alpha = float(getattr(self, "rpo_alpha", 0.0) or 0.0)
        if alpha:
            loss = loss + alpha * pol["nll_loss"]
        metrics = {"rewards/chosen": chosen_rewards.mean().item(), "rewards/rejected": rejected_rewards.mean().item(),
                   "rewards/accuracies": (chosen_rewards > rejected_rewards).float().mean().item(),
                   "rewards/margins": (chosen_rewards - rejected_rewards).mean().item(),
                   "logps/chosen": pol["chosen_logps"].detach().mean().item(),
                   "logps/rejected": pol["rejected_logps"].detach().mean().item()}
        if hasattr(self, "store_metrics"):
            self.store_metrics(metrics, train_eval="train" if model.training else "eval")
        ga = getattr(self, "current_gradient_accumulation_steps", self.args.gradient_accumulation_steps) if model.training else 1
        loss = loss / max(ga, 1) * (session.get_engine().get_sp_info()["sp_size"] if num_items_in_batch is None else 1)
        return (loss, metrics) if return_outputs else loss


_CLASSES: dict[str, type] = {}


def make_engine_seq2seq_trainer() -> type:
    from swift.trainers import Seq2SeqTrainer

    return type("EngineSeq2SeqTrainer", (EngineTrainerMixin, Seq2SeqTrainer), {"__module__": __name__.rsplit(".", 1)[0] + ".trainer_factory"})


def make_engine_dpo_trainer() -> type:
    try:
        from swift.trainers import DPOTrainer
    except ImportError:
        from swift.rlhf_trainers import DPOTrainer

    return type("EngineDPOTrainer", (EngineDPOTrainerMixin, DPOTrainer), {"__module__": __name__.rsplit(".", 1)[0] + ".trainer_factory"})


def get_engine_seq2seq_trainer() -> type:
    if "sft" not in _CLASSES:
        _CLASSES["sft"] = make_engine_seq2seq_trainer()
    return _CLASSES["sft"]


def get_engine_dpo_trainer() -> type:
    if "dpo" not in _CLASSES:
        _CLASSES["dpo"] = make_engine_dpo_trainer()
    return _CLASSES["dpo"]
