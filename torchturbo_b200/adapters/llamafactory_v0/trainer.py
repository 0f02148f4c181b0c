"""Trainer layer of the LlamaFactory adapter.

`make_torchturbo_trainer(LFTrainer, engine, stage)` derives a class whose MRO is
`TorchTurboTrainerBase -> (TorchTurboDPOTrainer) -> LFTrainer -> transformers.Trainer`.  LlamaFactory / HF keep the
loop; the engine takes over:
  * data loading (DP-block sampler: the SP ranks of one group read identical samples; block-diffusion models get
    their noised / block-aligned collator),
  * optimizer and LR schedule (`engine.prepare_optimizer`, engine-managed Muon / AdamW when configured),
  * the loss (packed rows through `engine.compute_loss`; block-diffusion loss for LLaDA-style models; DPO through
    packed chosen / rejected segments),
  * clipping (EP- and mesh-aware), metrics, profiling callbacks,
  * checkpoints (native sharded state for intermediate saves, HF export for the final save).
(adapters/llamafactory_v0/trainer.py:22-842 of the reference.)
"""
from __future__ import annotations

from typing import Any

import torch

from ...engine.distributed import assert_finite
from ...logging import get_logger
from ..hf_trainer import TurboTrainerMixin, normalize_training_features

logger = get_logger(__name__)

CUSTOM_OPTIMIZER_OPTIONS = ("use_galore", "use_apollo", "use_badam", "use_adam_mini", "use_muon")


class LlamaFactoryInputCollator:
    """Wraps a framework collator: its output is turned into the engine's packed-row contract on the host, before the
    batch is moved to the device."""

    def __init__(self, inner):
        self.inner = inner

    def __call__(self, features: list[dict[str, Any]]) -> dict[str, Any]:
        return normalize_training_features(self.inner(features))


class TorchTurboTrainerBase(TurboTrainerMixin):
    engine: Any = None
    stage: str | None = None
    torchturbo_wrapped: bool = False
    base_trainer_cls: type | None = None

    def __init__(self, *args, **kwargs):
        fa = kwargs.get("finetuning_args", args[0] if args else None)
        bad = self.unsupported_options(fa)
        if bad:
            raise NotImplementedError("the engine-backed LlamaFactory trainer does not support " + ", ".join(bad))
        self._mm_processor = kwargs.get("processor")
        super().__init__(*args, **kwargs)
        if getattr(self, "optimizer", None) is not None:
            raise ValueError("externally supplied optimizers are not supported: the engine builds the optimizer over "
                             "its sharded parameters")
        self.turbo_engine = self.engine
        if self.stage in ("pt", "sft") and not isinstance(self.data_collator, LlamaFactoryInputCollator):
            self.data_collator = LlamaFactoryInputCollator(self.data_collator)
        self._profiling_callback_added = False

    # -- option screening ------------------------------------------------------------------------------
    def unsupported_options(self, finetuning_args: Any) -> list[str]:
        out = [n for n in CUSTOM_OPTIMIZER_OPTIONS if bool(getattr(finetuning_args, n, None))]
        if self.stage == "sft" and getattr(finetuning_args, "use_dft_loss", False):
            out.append("use_dft_loss")
        return out

    def _engine(self):
        if self.engine is None:
            raise RuntimeError("trainer class was not bound to an engine (use make_torchturbo_trainer)")
        return self.engine

    def _move_model_to_device(self, model, _device):
        return model  # already materialised and sharded on this rank's device

    # -- optimizer / schedule -----------------------------------------------------------------------------
    def create_optimizer(self):
        if getattr(self, "optimizer", None) is not None:
            return self.optimizer
        eng = self._engine()
        opt_cfg = getattr(eng.config, "optimizer", None)
        if opt_cfg is not None and getattr(opt_cfg, "name", None):
            self.optimizer = eng.prepare_optimizer(self.model)
            logger.info_rank0("engine-managed optimizer %s", opt_cfg.name)
            return self.optimizer
        from ...engine.optimizers import OptimizerClassPlan

        a = self.args
        plan = OptimizerClassPlan(torch.optim.AdamW, lr=a.learning_rate, weight_decay=a.weight_decay,
                                  betas=(getattr(a, "adam_beta1", 0.9), getattr(a, "adam_beta2", 0.999)),
                                  eps=getattr(a, "adam_epsilon", 1e-8))
        self.optimizer = eng.prepare_optimizer(self.model, plan)
        return self.optimizer

    def create_scheduler(self, num_training_steps: int, optimizer=None):
        if getattr(self, "lr_scheduler", None) is None:
            a = self.args
            warm = a.get_warmup_steps(num_training_steps) if hasattr(a, "get_warmup_steps") else int(getattr(a, "warmup_steps", 0))
            self.lr_scheduler = self._engine().prepare_lr_scheduler(
                optimizer or self.optimizer, str(getattr(a.lr_scheduler_type, "value", a.lr_scheduler_type)),
                num_warmup_steps=warm, num_training_steps=num_training_steps,
                **(getattr(a, "lr_scheduler_kwargs", None) or {}))
            self._created_lr_scheduler = True
        return self.lr_scheduler

    # -- checkpoints -------------------------------------------------------------------------------------
    def save_model(self, output_dir=None, _internal_call=False):
        eng = self._engine()
        output_dir = output_dir or self.args.output_dir
        if _internal_call and not getattr(self.args, "save_only_model", False):
            eng.save_model(self.model, output_dir)                 # resumable native state (+ HF export per config)
        else:
            eng.save_model(self.model, output_dir, final=True)     # the framework's last save is the HF export
        if getattr(self.args, "push_to_hub", False) and not _internal_call and hasattr(self, "push_to_hub"):
            self.push_to_hub(commit_message="Model save")

    # -- data ----------------------------------------------------------------------------------------------
    def get_train_dataloader(self):
        if self.stage not in ("sft", "pt", "dpo"):
            return super(TurboTrainerMixin, self).get_train_dataloader()
        if getattr(self.model.config, "model_type", "") == "llada2_moe" or getattr(self.model, "is_block_diffusion", False):
            return self._get_block_diffusion_dataloader()
        return TurboTrainerMixin.get_train_dataloader(self)

    def _get_block_diffusion_dataloader(self):
        """Block-diffusion models: the tokenised samples are re-laid as `[noised | clean]` rows aligned to the
        diffusion block length (`models/llada2_moe/bd.py::BDDataset`: deterministic per-sample noise, optional
        first-fit packing), one row per micro-step."""
        from ...models.llada2_moe.bd import BDDataset

        eng = self._engine()
        ga = eng.resolve_gradient_accumulation_steps(self.args.gradient_accumulation_steps)
        self.args.gradient_accumulation_steps = ga
        cfg = self.model.config
        da = getattr(self, "data_args", None)
        cutoff = int(getattr(da, "cutoff_len", 0) or getattr(self.args, "cutoff_len", 0) or 2048)
        tok = getattr(self, "processing_class", None) or getattr(self, "tokenizer", None)
        pad_id = getattr(tok, "pad_token_id", None)
        samples = [{"input_ids": ex["input_ids"],
                    "prompt_length": sum(1 for l in ex.get("labels", []) if l == -100) if "labels" in ex else 0}
                   for ex in self.train_dataset]
        ds = BDDataset(samples, cutoff, mask_id=int(getattr(cfg, "mask_token_id")), pad_id=int(pad_id if pad_id is not None else 0),
                       block_size=int(getattr(cfg, "block_size", 32) or 32), pack=bool(getattr(da, "packing", False)))
        return eng.create_dataloader(ds, batch_size=1, collate_fn=lambda rows: rows[0], seed=self.args.seed,
                                     gradient_accumulation_steps=ga, num_workers=self.args.dataloader_num_workers)

    # -- loop bracketing -----------------------------------------------------------------------------------
    def train(self, *args, **kwargs):
        """Profiling is a runtime option (`--tt_profiling`, `--tt_memory_snapshot_steps`): the engine's profiler is
        started around the framework's loop and stepped by a callback."""
        from ...engine.args import get_torchturbo_args

        eng = self._engine()
        tt = get_torchturbo_args()
        profiling, snap = bool(getattr(tt, "profiling", False)), getattr(tt, "memory_snapshot_steps", None)
        started = False
        if profiling or snap:
            if not self._profiling_callback_added and hasattr(self, "add_callback"):
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
        eng = self._engine()
        try:
            from transformers import TrainerCallback
        except Exception:  # noqa: BLE001 - stand-alone use without transformers' callback base
            TrainerCallback = object

        class _StepProfiling(TrainerCallback):
            def on_step_end(self, args, state, control, **kw):
                eng.step_profiling()
                return control

        return _StepProfiling()

    # -- loss ------------------------------------------------------------------------------------------------
    def compute_loss(self, model, inputs, return_outputs=False, **kwargs):
        if self.stage == "dpo":
            return super().compute_loss(model, inputs, return_outputs=return_outputs, **kwargs)
        if inputs.get("noisy_input_ids") is not None or inputs.get("bd_mask_info") is not None:
            return self._compute_diffusion_loss(model, inputs, return_outputs=return_outputs, **kwargs)
        return TurboTrainerMixin.compute_loss(self, model, inputs, return_outputs=return_outputs,
                                              num_items_in_batch=kwargs.get("num_items_in_batch"))

    def _compute_diffusion_loss(self, model, inputs, return_outputs=False, **kwargs):
        eng = self._engine()
        res = eng.compute_diffusion_loss(model, normalize_bd(inputs), ga=self.args.gradient_accumulation_steps)
        loss, out = res if isinstance(res, tuple) else (res, None)
        return (loss, out) if return_outputs else loss

    def training_step(self, model, inputs, *args, **kwargs):
        num_items = kwargs.get("num_items_in_batch", args[0] if args else None)
        return TurboTrainerMixin.training_step(self, model, inputs, num_items_in_batch=num_items)


def normalize_bd(inputs: dict[str, Any]) -> dict[str, Any]:
    """Block-diffusion rows come out of `BDDataset` already in the engine's layout; tensors only lose a stray batch
    dimension a default collator may have added."""
    out = {}
    for k, v in inputs.items():
        out[k] = v[0] if isinstance(v, torch.Tensor) and v.dim() == 3 and v.shape[0] == 1 and k != "bd_allow" else v
    return out


class TorchTurboDPOTrainer(TorchTurboTrainerBase):
    """DPO: LlamaFactory's pairwise collator yields `[2B, S]` padded rows (chosen first).  They are packed into one row
    of `2B` segments; policy and reference run it through `loops.dpo.sequence_logps`; LlamaFactory's own
    `compute_preference_loss` turns the four log-prob vectors into the loss, so every `pref_loss` it implements on
    summed log-probs keeps its definition."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._initialize_reference()

    def _initialize_reference(self) -> None:
        ref = getattr(self, "ref_model", None)
        if ref is None or ref is self.model:
            return
        if getattr(getattr(self, "finetuning_args", None), "ref_model", None) is None:
            copy_model_state(self.model, ref)
            logger.info_rank0("DPO reference model initialised from the policy weights")
        ref.requires_grad_(False)
        ref.eval()

    def _dpo_config(self, for_reference: bool):
        from ...loops.dpo import DPOConfig

        lt = getattr(self, "loss_type", "sigmoid")
        return DPOConfig(beta=float(getattr(self, "beta", 0.1)), loss_type="ipo" if lt in ("ipo", "orpo", "simpo") else "sigmoid",
                         ld_alpha=None if for_reference else getattr(self, "ld_alpha", None))

    @staticmethod
    def pack_pairs(inputs: dict[str, Any], pad_id: int = -100) -> dict[str, Any]:
        """`[2B, S]` padded (chosen rows then rejected rows) -> one packed row with `2B` segments."""
        ids, labels = inputs["input_ids"], inputs["labels"]
        mask = inputs.get("attention_mask")
        mask = mask.bool() if mask is not None else torch.ones_like(ids, dtype=torch.bool)
        lens = mask.sum(-1).tolist()
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32)
        flat_ids, flat_lab = ids[mask].unsqueeze(0), labels[mask].unsqueeze(0)
        pos = torch.cat([torch.arange(n) for n in lens]).unsqueeze(0)
        out = {"input_ids": flat_ids, "labels": flat_lab, "position_ids": pos, "cu_seq_lens_q": cu, "cu_seq_lens_k": cu.clone(),
               "max_length_q": max(lens), "max_length_k": max(lens)}
        for k, v in inputs.items():
            if k not in out and k not in ("attention_mask",):
                out[k] = v
        return out

    def concatenated_forward(self, model, batch, is_ref_model: bool = False):
        """(chosen logps, rejected logps, None, None, chosen valid lengths): the logits are never materialised for
        the caller (they are reduced to per-segment sums shard by shard)."""
        from ...loops.dpo import sequence_logps

        packed = batch if batch.get("cu_seq_lens_q") is not None else self.pack_pairs(batch)
        cfg = self._dpo_config(is_ref_model)
        sums, counts = sequence_logps(self._engine(), model, packed, cfg, grad=not is_ref_model and torch.is_grad_enabled())
        if cfg.loss_type == "ipo":
            sums = sums / counts.clamp(min=1)
        n = sums.numel() // 2
        return sums[:n], sums[n:], None, None, counts[:n]

    def compute_reference_log_probs(self, model, batch):
        if not getattr(self.finetuning_args, "use_ref_model", True):
            return None, None
        ref = getattr(self, "ref_model", None)
        if ref is None:
            raise NotImplementedError("DPO without a separate reference model (adapter-disabled policy) is not supported")
        with torch.no_grad():
            c, r, *_ = self.concatenated_forward(ref, batch, is_ref_model=True)
        return c, r

    def get_batch_loss_metrics(self, model, inputs, train_eval: str = "train"):
        packed = self.pack_pairs(dict(inputs)) if inputs.get("cu_seq_lens_q") is None else dict(inputs)
        pc, pr, _, _, clen = self.concatenated_forward(model, packed)
        rc, rr = self.compute_reference_log_probs(model, packed)
        losses, chosen_rewards, rejected_rewards = self.compute_preference_loss(pc, pr, rc, rr)
        sft = -pc / clen.clamp(min=1)
        gamma = float(getattr(self, "ftx_gamma", 0.0) or 0.0)
        if gamma > 1e-6:
            losses = losses + gamma * sft
        pre = "eval_" if train_eval == "eval" else ""
        m = {f"{pre}rewards/chosen": chosen_rewards.mean().item(), f"{pre}rewards/rejected": rejected_rewards.mean().item(),
             f"{pre}rewards/accuracies": (chosen_rewards > rejected_rewards).float().mean().item(),
             f"{pre}rewards/margins": (chosen_rewards - rejected_rewards).mean().item(),
             f"{pre}logps/chosen": pc.detach().mean().item(), f"{pre}logps/rejected": pr.detach().mean().item()}
        return losses.mean(), m

    def compute_loss(self, model, inputs, return_outputs=False, **kwargs):
        loss, metrics = self.get_batch_loss_metrics(model, inputs)
        if hasattr(self, "store_metrics"):
            self.store_metrics(metrics, train_eval="train")
        assert_finite(loss.detach(), "dpo loss")
        return (loss, metrics) if return_outputs else loss


def copy_model_state(src: Any, dst: Any) -> None:
    """Copy parameters and persistent buffers shard by shard (both models were built by the same engine, so their
    local shards line up); raises when the two state layouts differ."""

    def state(m):
        s = dict(m.named_parameters(remove_duplicate=False))
        non_persistent = {f"{mn}.{bn}" if mn else bn for mn, mod in m.named_modules() for bn in mod._non_persistent_buffers_set}
        s.update({k: v for k, v in m.named_buffers(remove_duplicate=False) if k not in non_persistent})
        return s

    a, b = state(src), state(dst)
    if a.keys() != b.keys():
        raise ValueError(f"reference and policy differ in state names: {sorted(a.keys() ^ b.keys())[:5]}")
    with torch.no_grad():
        for k, t in a.items():
            ls = t._local_tensor if hasattr(t, "_local_tensor") else t
            ld = b[k]._local_tensor if hasattr(b[k], "_local_tensor") else b[k]
            if ls.shape != ld.shape:
                raise ValueError(f"shape mismatch for {k}: {tuple(ls.shape)} vs {tuple(ld.shape)}")
            ld.copy_(ls)


def make_torchturbo_trainer(base_cls: type, engine: Any, stage: str) -> type:
    """Class with the engine mixins in front of `base_cls`; idempotent (an already wrapped class is rebound)."""
    base_cls = unwrap_torchturbo_trainer_class(base_cls)
    mixin = TorchTurboDPOTrainer if stage == "dpo" else TorchTurboTrainerBase
    return type(f"TorchTurbo{base_cls.__name__}", (mixin, base_cls),
                {"engine": engine, "turbo_engine": engine, "stage": stage, "torchturbo_wrapped": True, "base_trainer_cls": base_cls})


def unwrap_torchturbo_trainer_class(cls: type) -> type:
    while getattr(cls, "torchturbo_wrapped", False) and getattr(cls, "base_trainer_cls", None) is not None:
        cls = cls.base_trainer_cls
    return cls
