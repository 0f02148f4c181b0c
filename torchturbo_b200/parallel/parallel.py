from __future__ import annotations

from dataclasses import dataclass


@dataclass
class ParallelPlan:
    """Base type of declarative, per-module parallel plans; backends define concrete subclasses."""
