"""On-disk layout of a training checkpoint and crash-safe file helpers.

    checkpoint-<step>/
        model_distcp/            sharded native model state (complete when `.metadata` exists)
        optimizer_distcp/        sharded native optimizer state
        scheduler.pt             written atomically
        torchturbo/checkpoint.json   engine metadata (schema v1)
        huggingface/             optional HF export; `model.safetensors.index.json` is written last

Commit markers make an interrupted save detectable instead of silently loadable
(engine/checkpoint/layout.py:18-180 and backends/fsdp2/checkpoint/layout.py:13-32 of the reference)."""
from __future__ import annotations

import json
import os
import tempfile
from enum import Enum
from pathlib import Path
from typing import Any

import torch

MODEL_DCP_DIR = "model_distcp"
OPTIMIZER_DCP_DIR = "optimizer_distcp"
SCHEDULER_FILE = "scheduler.pt"
METADATA_DIR = "torchturbo"
METADATA_FILE = "checkpoint.json"
HF_DIR = "huggingface"
HF_INDEX = "model.safetensors.index.json"
DCP_COMMIT = ".metadata"


class ModelFormat(str, Enum):
    NATIVE = "native"
    HF = "huggingface"


def dcp_status(path: str | os.PathLike) -> str:
    p = Path(path)
    if not p.is_dir():
        return "missing"
    return "complete" if (p / DCP_COMMIT).is_file() else "incomplete"


def hf_status(path: str | os.PathLike) -> str:
    """complete: an index (or a single `model.safetensors`) exists and every file it names is present."""
    p = Path(path)
    if not p.is_dir():
        return "missing"
    idx = p / HF_INDEX
    if idx.is_file():
        try:
            files = set(json.loads(idx.read_text())["weight_map"].values())
        except Exception:
            return "incomplete"
        return "complete" if all((p / f).is_file() for f in files) else "incomplete"
    if (p / "model.safetensors").is_file():
        return "complete"
    return "incomplete" if any(p.glob("*.safetensors")) else "missing"


def resolve_model_format(checkpoint_dir: str | os.PathLike) -> tuple[ModelFormat, Path]:
    """Prefer the native sharded state, fall back to a Hugging Face export; an incomplete directory of the
    preferred kind is an error, not a reason to fall through silently."""
    root = Path(checkpoint_dir)
    native = dcp_status(root / MODEL_DCP_DIR)
    if native == "complete":
        return ModelFormat.NATIVE, root / MODEL_DCP_DIR
    if native == "incomplete":
        raise RuntimeError(f"{root / MODEL_DCP_DIR} is incomplete (interrupted save?)")
    for cand in (root / HF_DIR, root):
        st = hf_status(cand)
        if st == "complete":
            return ModelFormat.HF, cand
        if st == "incomplete":
            raise RuntimeError(f"{cand} holds an incomplete Hugging Face export")
    raise FileNotFoundError(f"no model state found under {root}")


def fsync_dir(path: str | os.PathLike) -> None:
    try:
        fd = os.open(str(path), os.O_RDONLY)
        try:
            os.fsync(fd)
        finally:
            os.close(fd)
    except OSError:
        pass


def _atomic_write(path: Path, write) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=str(path.parent), prefix=path.name + ".tmp.")
    try:
        with os.fdopen(fd, "wb") as f:
            write(f)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
        fsync_dir(path.parent)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def save_json(path: str | os.PathLike, obj: Any) -> None:
    _atomic_write(Path(path), lambda f: f.write(json.dumps(obj, indent=2, sort_keys=True, default=str).encode()))


def save_scheduler(path: str | os.PathLike, state: dict) -> None:
    _atomic_write(Path(path), lambda f: torch.save(state, f))


def load_scheduler(path: str | os.PathLike) -> dict:
    try:
        # scheduler state is numbers, lists and dicts: nothing in it needs unpickling of arbitrary objects
        return torch.load(path, map_location="cpu", weights_only=True)
    except Exception as e:
        raise RuntimeError(f"{path} is unreadable (truncated save?): {e}") from e


def sync_directory(path: str | os.PathLike) -> None:
    for root, _, files in os.walk(path):
        for fn in files:
            try:
                fd = os.open(os.path.join(root, fn), os.O_RDONLY)
                os.fsync(fd)
                os.close(fd)
            except OSError:
                pass
        fsync_dir(root)


_OWNED = {MODEL_DCP_DIR, OPTIMIZER_DCP_DIR, SCHEDULER_FILE, METADATA_DIR, HF_DIR}


def validate_output_dir(path: str | os.PathLike) -> None:
    """Refuse to write a checkpoint into something that is clearly not a checkpoint directory: a file, the
    filesystem root / home, or a non-empty directory holding entries the engine does not own."""
    p = Path(path).resolve()
    if p.is_file():
        raise ValueError(f"{p} is a file")
    if p == Path(p.anchor) or p == Path.home():
        raise ValueError(f"refusing to use {p} as a checkpoint directory")
    if p.is_dir():
        foreign = [e.name for e in p.iterdir() if e.name not in _OWNED and not e.name.startswith(".")
                   and not e.name.endswith((".json", ".txt", ".bin", ".pt", ".pth", ".safetensors", ".model", ".jinja"))]
        if foreign:
            raise ValueError(f"{p} contains entries that do not belong to a checkpoint: {foreign[:5]}")
