"""Single-entry cache keyed by tensor identity and version (utils/functools.py:41-88 in the reference)."""
from __future__ import annotations

import functools

import torch


def _key(x):
    if isinstance(x, torch.Tensor):
        return ("t", id(x), x._version, tuple(x.shape), x.device.type)
    if isinstance(x, (list, tuple)):
        return tuple(_key(v) for v in x)
    if isinstance(x, dict):
        return tuple((k, _key(v)) for k, v in sorted(x.items()))
    return x


def cache(fn):
    """Remember only the most recent call: metadata such as `cu_seq_lens` is reused by every layer of one
    step and then replaced, so one slot is enough and nothing leaks."""
    slot = {}

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        k = (_key(args), _key(kwargs))
        if slot.get("k") == k:
            return slot["v"]
        v = fn(*args, **kwargs)
        slot["k"], slot["v"] = k, v
        # keep the tensors alive so ids are not recycled while the entry is valid
        slot["refs"] = (args, kwargs)
        return v

    wrapper.cache_clear = slot.clear  # type: ignore[attr-defined]
    return wrapper
