"""Backend-independent checkpoint life cycle: what is saved when, in which order, with which guards.

  save_model: metadata agreed on all ranks -> rank 0 resets the target and writes metadata -> native sharded
              state (always) -> Hugging Face export (`hf_export: every`, or `final` on the last save) -> plugins.
  load_model: native state preferred over HF; incomplete directories are rejected; PEFT configs must match.
  optimizer/scheduler: native sharded optimizer state + atomically written `scheduler.pt`; the EP size saved
              with the checkpoint must equal the current one.
(engine/checkpoint/coordinator.py:65-308 of the reference)"""
from __future__ import annotations

import os
import shutil
from pathlib import Path
from typing import Any

import torch.distributed as dist

from ...logging import get_logger
from .distributed import collective_check, rank_zero_call
from .layout import (HF_DIR, METADATA_DIR, MODEL_DCP_DIR, OPTIMIZER_DCP_DIR, SCHEDULER_FILE, ModelFormat, dcp_status,
                     load_scheduler, resolve_model_format, save_scheduler, validate_output_dir)
from .metadata import build_metadata, load_metadata, save_metadata, validate_peft_configs

logger = get_logger(__name__)


def _barrier() -> None:
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


class CheckpointCoordinator:
    def __init__(self, config, manager, *, plugins=None, parallel_context: dict | None = None) -> None:
        self.config = config
        self.manager = manager
        self.plugins = plugins
        self.parallel_context = parallel_context or {}

    # -- pretrained weights ----------------------------------------------------------------------
    def load_pretrained(self, model, path: str) -> None:
        self.manager.load_hf(model, path)

    # -- model -------------------------------------------------------------------------------------
    def _peft_configs(self, model) -> dict[str, Any]:
        return dict(getattr(model, "peft_config", {}) or {})

    def _reset_checkpoint(self, output_dir: str) -> None:
        """Remove only what a previous save of this engine could have written."""
        root = Path(output_dir)
        for name in (MODEL_DCP_DIR, OPTIMIZER_DCP_DIR, METADATA_DIR, HF_DIR):
            p = root / name
            if p.is_dir():
                shutil.rmtree(p)
        s = root / SCHEDULER_FILE
        if s.is_file():
            s.unlink()

    def save_model(self, model, output_dir: str, *, final: bool = False, source_path: str | None = None,
                   step: int | None = None) -> None:
        formats = [ModelFormat.NATIVE]
        if self.config.checkpoint.hf_export == "every" or final:
            formats.append(ModelFormat.HF)
        meta = collective_check(lambda: build_metadata(model, self.config, source_path=source_path,
                                                       parallel_context=self.parallel_context,
                                                       peft_configs=self._peft_configs(model)), "checkpoint metadata")

        def prepare():
            validate_output_dir(output_dir)
            self._reset_checkpoint(output_dir)
            os.makedirs(output_dir, exist_ok=True)
            save_metadata(output_dir, meta)

        rank_zero_call(prepare, "checkpoint directory preparation")
        _barrier()
        collective_check(lambda: self.manager.save_native_model(model, os.path.join(output_dir, MODEL_DCP_DIR)),
                         "native model save")
        if ModelFormat.HF in formats:
            hf_dir = os.path.join(output_dir, HF_DIR)
            collective_check(lambda: self.manager.save_hf(model, hf_dir, source_path=source_path), "HF export")
            if self.plugins is not None and (not dist.is_initialized() or dist.get_rank() == 0):
                for p in self.plugins.export_plugins():
                    p.on_hf_export(hf_dir, step=step, final=final)
        _barrier()

    def load_model(self, model, checkpoint_dir: str, **kwargs: Any) -> None:
        fmt, path = resolve_model_format(checkpoint_dir)
        meta = load_metadata(checkpoint_dir)
        if meta is not None:
            validate_peft_configs(meta.get("peft"), self._peft_configs(model))
        if fmt is ModelFormat.NATIVE:
            collective_check(lambda: self.manager.load_native_model(model, str(path)), "native model load")
        else:
            collective_check(lambda: self.manager.load_hf(model, str(path)), "HF model load")

    # -- optimizer / scheduler -----------------------------------------------------------------------
    def save_optimizer_and_scheduler(self, model, optimizer, scheduler, output_dir: str) -> None:
        collective_check(lambda: self.manager.save_native_optimizer(model, optimizer,
                                                                    os.path.join(output_dir, OPTIMIZER_DCP_DIR)),
                         "optimizer save")
        if scheduler is not None:
            rank_zero_call(lambda: save_scheduler(os.path.join(output_dir, SCHEDULER_FILE), scheduler.state_dict()),
                           "scheduler save")
        _barrier()

    def load_optimizer_and_scheduler(self, model, optimizer, scheduler, checkpoint_dir: str) -> None:
        opt_dir = os.path.join(checkpoint_dir, OPTIMIZER_DCP_DIR)

        def preflight():
            st = dcp_status(opt_dir)
            if st != "complete":
                raise RuntimeError(f"optimizer state under {opt_dir} is {st}")
            meta = load_metadata(checkpoint_dir)
            if meta is not None:
                saved_ep = meta.get("engine", {}).get("ep_size", 1)
                cur_ep = self.parallel_context.get("ep", {}).get("ep_size", 1)
                if saved_ep != cur_ep:
                    raise RuntimeError(f"checkpoint was written with ep_size={saved_ep}, current run uses {cur_ep}")

        collective_check(preflight, "optimizer checkpoint preflight")
        collective_check(lambda: self.manager.load_native_optimizer(model, optimizer, opt_dir), "optimizer load")
        sched_path = os.path.join(checkpoint_dir, SCHEDULER_FILE)
        if scheduler is not None:
            # a resume that restores the optimizer but silently restarts the learning-rate schedule trains with the
            # wrong rate: a missing file is an error, as in the reference (engine/checkpoint/coordinator.py:197-250 there)
            def load_sched():
                if not os.path.isfile(sched_path):
                    raise FileNotFoundError(f"{sched_path} is missing although {opt_dir} holds optimizer state; the checkpoint "
                                            "is incomplete (pass scheduler=None to resume without a schedule)")
                scheduler.load_state_dict(load_scheduler(sched_path))

            collective_check(load_sched, "scheduler load")
