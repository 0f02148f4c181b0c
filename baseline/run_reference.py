"""Reference arm of bench.py: drives the unmodified reference package installed under `baseline/_ref`
through its own public API.  When the package cannot be imported here, reports why in one line."""
from __future__ import annotations

import os
import sys

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def run_reference(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    try:
        from .reference_driver import run as _run
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference driver not importable: {type(e).__name__}: {e}"} if rank == 0 else {}
    try:
        return _run(args, REF_DIR)
    except Exception as e:  # noqa: BLE001
        msg = f"{type(e).__name__}: {str(e).splitlines()[0] if str(e) else ''}"[:300]
        return {"impl": "reference", "unavailable": msg} if rank == 0 else {}
