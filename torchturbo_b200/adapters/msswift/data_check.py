"""Raw-dataset validation for multimodal pre-training: every row's image list must be a list of single paths and match
the number of `<image>` tags in its text.  Violations are reported with the row index before any tokenisation starts
(adapters/msswift/data_check.py:10-58 of the reference)."""
from __future__ import annotations

from typing import Any

from ...logging import get_logger

logger = get_logger(__name__)
TEXT_KEYS = ("messages", "query", "response", "text", "prompt", "conversations")


def _path_of(entry: Any) -> str:
    if isinstance(entry, str):
        return entry
    if isinstance(entry, dict):
        return entry.get("path") or ""
    return ""


def check_row(row: dict) -> str | None:
    """The violation as text, or None for a conforming (or text-only) row."""
    images = row.get("images", row.get("image"))
    if images is None:
        return None
    if isinstance(images, str):
        return "comma-joined image path" if "," in images else "images must be a list of paths"
    if not isinstance(images, (list, tuple)):
        return "images must be a list of paths"
    for entry in images:
        p = _path_of(entry)
        if not p:
            return f"image entry without a path: {str(entry)[:60]}"
        if "," in p:
            return "comma-joined image path"
    text = " ".join(str(row[k]) for k in TEXT_KEYS if k in row)
    tags = text.count("<image>")
    if tags != len(images):
        return f"<image> tag count {tags} != image count {len(images)}"
    return None


def validate_raw_dataset(dataset: Any, name: str = "train") -> None:
    if dataset is None:
        return
    cols = getattr(dataset, "column_names", None)
    if cols is not None and not ({"images", "image"} & set(cols)):
        return
    if not hasattr(dataset, "__len__"):
        return  # streaming: rows are only seen once, by the trainer
    for i, row in enumerate(dataset):
        why = check_row(row)
        if why is not None:
            raise ValueError(f"{name} dataset row {i}: {why}; normalise the data offline with "
                             "scripts/dataset/convert_lf_to_swift.py first")
    logger.info_rank0("%s dataset: %d rows conform to the swift data standard", name, len(dataset))
