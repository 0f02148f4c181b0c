"""Audit of raw multimodal rows before tokenisation starts.

A multimodal pre-training row pairs a text with media: the number of `<image>` placeholders in the text has to equal
the number of image references, and every reference has to name exactly one file.  A mismatch found later, in the
middle of a packed batch, costs a job restart, so the whole split is audited up front in ONE pass that classifies every
row and reports a per-rule tally with example row numbers (instead of stopping at the first offender), so that a data
set with several kinds of defects can be repaired in one go.

The rules come from the data contract the reference enforces in adapters/msswift/data_check.py of its tree.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field
from typing import Any, Iterable

from ...logging import get_logger

logger = get_logger(__name__)

PLACEHOLDER = "<image>"
TEXT_FIELDS = ("messages", "query", "response", "text", "prompt", "conversations")
MEDIA_FIELDS = ("images", "image")

# rule id -> what is wrong with the row
RULES = {
    "not_a_list": "the image field is not a list (one string, or another type)",
    "joined_paths": "one image reference holds several comma-separated paths",
    "empty_reference": "an image reference carries no path",
    "placeholder_mismatch": f"the text has a different number of {PLACEHOLDER} placeholders than the row has images",
}


def _reference_path(ref: Any) -> str:
    if isinstance(ref, str):
        return ref
    if isinstance(ref, dict):
        return str(ref.get("path") or "")
    return ""


def classify_row(row: dict) -> tuple[str, str] | None:
    """`(rule id, detail)` of the first rule the row breaks, or None (conforming rows and rows without media)."""
    media = next((row[f] for f in MEDIA_FIELDS if row.get(f) is not None), None)
    if media is None:
        return None
    if isinstance(media, str):
        return ("joined_paths", media[:60]) if "," in media else ("not_a_list", f"str: {media[:60]}")
    if not isinstance(media, (list, tuple)):
        return "not_a_list", type(media).__name__
    for ref in media:
        path = _reference_path(ref)
        if not path:
            return "empty_reference", str(ref)[:60]
        if "," in path:
            return "joined_paths", path[:60]
    placeholders = sum(str(row[f]).count(PLACEHOLDER) for f in TEXT_FIELDS if f in row)
    if placeholders != len(media):
        return "placeholder_mismatch", f"{placeholders} placeholder(s), {len(media)} image(s)"
    return None


def check_row(row: dict) -> str | None:
    """Human-readable violation of one row, or None."""
    hit = classify_row(row)
    return None if hit is None else f"{RULES[hit[0]]} [{hit[1]}]"


@dataclass
class AuditReport:
    rows: int = 0
    by_rule: dict[str, list[int]] = field(default_factory=lambda: defaultdict(list))
    details: dict[int, str] = field(default_factory=dict)

    @property
    def ok(self) -> bool:
        return not self.by_rule

    def summary(self, examples: int = 5) -> str:
        lines = []
        for rule, idx in sorted(self.by_rule.items(), key=lambda kv: -len(kv[1])):
            shown = ", ".join(f"#{i} ({self.details[i]})" for i in idx[:examples])
            lines.append(f"  {len(idx)} row(s): {RULES[rule]}; e.g. {shown}")
        return "\n".join(lines)


def audit_rows(rows: Iterable[dict]) -> AuditReport:
    rep = AuditReport()
    for i, row in enumerate(rows):
        rep.rows += 1
        hit = classify_row(row)
        if hit is not None:
            rep.by_rule[hit[0]].append(i)
            rep.details[i] = hit[1]
    return rep


def validate_raw_dataset(dataset: Any, name: str = "train") -> None:
    """Audit a map-style dataset that has an image column; raises one `ValueError` listing every broken rule with its
    row count.  Streaming datasets (no length) and text-only datasets are left alone."""
    if dataset is None or not hasattr(dataset, "__len__"):
        return
    columns = getattr(dataset, "column_names", None)
    if columns is not None and not set(MEDIA_FIELDS) & set(columns):
        return
    rep = audit_rows(dataset)
    if not rep.ok:
        bad = sum(len(v) for v in rep.by_rule.values())
        raise ValueError(f"{name} split: {bad} of {rep.rows} multimodal rows break the data contract\n{rep.summary()}\n"
                         "rewrite the split with scripts/dataset/convert_lf_to_swift.py (one path per image entry, one "
                         f"{PLACEHOLDER} per image) and start again")
    logger.info_rank0("%s split: all %d rows pass the multimodal data audit", name, rep.rows)
