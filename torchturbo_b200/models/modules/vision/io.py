"""Model-owned adapter between a vision tower's call signature and the balancer's packed view of media
(models/modules/vision/io.py:12-110 of the reference)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any

import torch
from torch import nn


@dataclass(frozen=True)
class VisionBatch:
    """`pixels`: patch rows of all media concatenated on dim 0; `grid_thw`: one `(t, h, w)` row per medium (a medium
    owns `t*h*w` consecutive pixel rows); `output_lengths[name][i]`: rows medium `i` produces in output stream
    `name` (names and order identical on every rank, known before the forward pass)."""

    pixels: torch.Tensor
    grid_thw: torch.Tensor
    output_lengths: dict[str, list[int]]


class BaseVisionBalanceIO(ABC):
    """Stateless translation of one tower boundary.  Every rank must call the tower the same number of times in the
    same order; media-less batches carry a dummy image supplied by the data pipeline."""

    @abstractmethod
    def read_inputs(self, tower: nn.Module, args: tuple, kwargs: dict) -> VisionBatch: ...

    @abstractmethod
    def write_inputs(self, tower: nn.Module, args: tuple, kwargs: dict, batch: VisionBatch) -> tuple[tuple, dict]:
        """Call arguments with the media replaced by `batch`."""

    @abstractmethod
    def read_outputs(self, tower: nn.Module, output: Any) -> dict[str, torch.Tensor]:
        """Output streams as `[rows, features]` tensors keyed by stream name."""

    @abstractmethod
    def write_outputs(self, tower: nn.Module, output: Any, streams: dict[str, torch.Tensor]) -> Any:
        """The tower's return structure with the streams replaced."""

    @abstractmethod
    def make_dummy(self, tower: nn.Module, like: VisionBatch) -> VisionBatch:
        """Smallest valid medium for a rank that was assigned nothing."""


class GridVisionBalanceIO(BaseVisionBalanceIO):
    """IO for Qwen-VL style towers: `tower(pixel_values, grid_thw=...)` returning merged patch features
    `[sum(t*h*w / merge^2), out_hidden]` (one stream, `pooler_output`)."""

    stream = "pooler_output"

    def __init__(self, spatial_merge_size: int = 2):
        self.merge = spatial_merge_size

    def _lengths(self, grid: torch.Tensor) -> list[int]:
        return [int(t * h * w) // (self.merge ** 2) for t, h, w in grid.tolist()]

    def read_inputs(self, tower, args, kwargs):
        pixels = args[0] if args else kwargs["pixel_values"]
        grid = kwargs.get("grid_thw") if "grid_thw" in kwargs else args[1]
        return VisionBatch(pixels, grid, {self.stream: self._lengths(grid)})

    def write_inputs(self, tower, args, kwargs, batch):
        kw = dict(kwargs)
        if args:
            new_args = (batch.pixels,) + tuple(args[1:])
            if "grid_thw" in kw or len(args) < 2:
                kw["grid_thw"] = batch.grid_thw
            else:
                new_args = (batch.pixels, batch.grid_thw) + tuple(args[2:])
            return new_args, kw
        kw["pixel_values"], kw["grid_thw"] = batch.pixels, batch.grid_thw
        return args, kw

    def read_outputs(self, tower, output):
        """A tower called with `return_deepstack=True` returns `(features, [per-level features, ...])`, all with one row
        per merged patch: they travel as one stream, concatenated along the feature axis (one exchange, not one per
        level)."""
        if isinstance(output, tuple):
            feats, deep = output
            return {self.stream: torch.cat([feats, *deep], dim=-1) if len(deep) else feats}
        return {self.stream: output}

    def write_outputs(self, tower, output, streams):
        x = streams[self.stream]
        if isinstance(output, tuple):
            feats, deep = output
            if not len(deep):
                return x, []
            parts = x.split([feats.shape[-1]] + [d.shape[-1] for d in deep], dim=-1)
            return parts[0].contiguous(), [p.contiguous() for p in parts[1:]]
        return x

    def make_dummy(self, tower, like):
        m = self.merge
        rows = m * m
        pixels = like.pixels.new_zeros((rows,) + tuple(like.pixels.shape[1:]))
        grid = torch.tensor([[1, m, m]], dtype=like.grid_thw.dtype, device=like.grid_thw.device)
        return VisionBatch(pixels, grid, {self.stream: [1]})
