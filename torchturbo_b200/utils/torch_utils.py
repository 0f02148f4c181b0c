from __future__ import annotations

import torch
from packaging.version import Version


def torch_version() -> Version:
    return Version(torch.__version__.split("+")[0])


def has_meta_tensor(module: torch.nn.Module) -> list[str]:
    return [n for n, p in list(module.named_parameters()) + list(module.named_buffers()) if p.is_meta]
