"""`torchturbo/checkpoint.json` (schema v1): where the model came from, its config, the structural engine
settings needed to rebuild it, and the full PEFT configs (engine/checkpoint/metadata.py:58-147 of the reference)."""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any

from .layout import METADATA_DIR, METADATA_FILE, save_json

SCHEMA_VERSION = 1


def build_metadata(model, engine_config, *, source_path: str | None, parallel_context: dict | None = None,
                   peft_configs: dict[str, Any] | None = None) -> dict[str, Any]:
    cfg = getattr(model, "config", None)
    cfg_d = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(vars(cfg or {}))
    ep = (parallel_context or {}).get("ep", {}).get("ep_size", 1)
    sp = (parallel_context or {}).get("sp", {}).get("sp_size", 1)
    return {
        "schema_version": SCHEMA_VERSION,
        "source": {"model_name_or_path": source_path},
        "model": {"model_type": getattr(cfg, "model_type", None), "class": type(model).__name__, "config": cfg_d},
        "engine": {
            "backend": engine_config.backend.value,
            "mixed_precision": engine_config.mixed_precision.value,
            "ep_size": ep, "sp_size": sp,
            "mtp_enabled": engine_config.mtp.enabled,
        },
        "peft": {k: (v.to_dict() if hasattr(v, "to_dict") else dict(v)) for k, v in (peft_configs or {}).items()},
    }


def save_metadata(checkpoint_dir: str | os.PathLike, meta: dict[str, Any]) -> None:
    save_json(Path(checkpoint_dir) / METADATA_DIR / METADATA_FILE, meta)


def load_metadata(checkpoint_dir: str | os.PathLike) -> dict[str, Any] | None:
    p = Path(checkpoint_dir) / METADATA_DIR / METADATA_FILE
    if not p.is_file():
        return None
    meta = json.loads(p.read_text())
    if meta.get("schema_version") != SCHEMA_VERSION:
        raise ValueError(f"{p}: unsupported schema_version {meta.get('schema_version')!r}")
    return meta


_PEFT_STRUCTURAL = ("peft_type", "r", "lora_alpha", "target_modules", "use_dora", "use_rslora", "modules_to_save")


def validate_peft_configs(saved: dict[str, Any] | None, current: dict[str, Any] | None) -> None:
    """A checkpoint can only be resumed with the same adapters: same names and the same structural fields.
    A checkpoint saved without PEFT cannot be resumed with PEFT and vice versa."""
    saved, current = saved or {}, current or {}
    if set(saved) != set(current):
        raise ValueError(f"PEFT adapter mismatch: checkpoint has {sorted(saved)}, run has {sorted(current)}")
    for name in saved:
        a = saved[name]
        b = current[name].to_dict() if hasattr(current[name], "to_dict") else dict(current[name])
        for k in _PEFT_STRUCTURAL:
            va, vb = a.get(k), b.get(k)
            if isinstance(va, (list, tuple, set)):
                va = sorted(va)
            if isinstance(vb, (list, tuple, set)):
                vb = sorted(vb)
            if va != vb:
                raise ValueError(f"PEFT adapter {name!r}: field {k!r} differs (checkpoint {va!r}, run {vb!r})")
