"""Model-FLOPs utilisation from analytic forward FLOPs and wall time between reports."""
from __future__ import annotations

import json
import time
from pathlib import Path

from .flops import ComputeProfile

# dense bf16 TFLOP/s per device.  The first six entries are the vendor figures the reference ships
# (engine/metrics/mfu_estimator.py:18-25); `b200` is this engine's target and uses the nominal dense figure,
# `b200_measured` the cuBLAS throughput measured on the pool when the peaks file is present.
PEAK_TFLOPS_TABLE = {
    "910b": 365.0, "910c": 376.0, "h20": 148.0, "a100": 312.0, "h100": 989.0, "h200": 989.0, "b200": 2250.0,
}


def _measured_b200() -> float | None:
    p = Path(__file__).resolve().parents[3] / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["bf16_tflops_sustained"])
    except Exception:
        return None


def resolve_peak_tflops(card: str | None, device_type: str = "cuda") -> tuple[str, float]:
    if card is None:
        card = "b200" if device_type == "cuda" else "h20"
    card = card.lower()
    if card == "b200_measured":
        v = _measured_b200()
        if v:
            return card, v
        card = "b200"
    if card not in PEAK_TFLOPS_TABLE:
        raise ValueError(f"unknown card {card!r}; known: {sorted(PEAK_TFLOPS_TABLE)}")
    return card, PEAK_TFLOPS_TABLE[card]


class MFUEstimator:
    def __init__(self, flops_recipe, card: str | None = None, device_type: str = "cuda",
                 activation_checkpointing: bool = False, world_size: int = 1, sp_size: int = 1):
        self.recipe = flops_recipe
        self.card, self.peak_tflops = resolve_peak_tflops(card, device_type)
        self.ac = activation_checkpointing
        self.world_size, self.sp_size = world_size, sp_size
        self._fwd_flops = 0.0
        self._t0 = time.perf_counter()

    def record_micro(self, inputs) -> None:
        """Accumulate the forward FLOPs of one micro-batch.  Under sequence parallelism the `sp` ranks of a
        group share one micro-batch, so each rank is charged `1/sp` of it."""
        prof = inputs if isinstance(inputs, ComputeProfile) else ComputeProfile.from_inputs(inputs)
        self._fwd_flops += self.recipe.forward_flops(prof) / self.sp_size

    def pop(self) -> dict[str, float]:
        now = time.perf_counter()
        dt, fl = max(now - self._t0, 1e-9), self._fwd_flops
        self._t0, self._fwd_flops = now, 0.0
        peak = self.peak_tflops * 1e12
        return {"mfu": 3.0 * fl / dt / peak, "hfu": (4.0 if self.ac else 3.0) * fl / dt / peak}
