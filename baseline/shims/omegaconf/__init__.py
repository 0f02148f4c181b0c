"""Minimal stand-in for the `omegaconf` package (not installable offline), just large enough for the reference
package to import and for its dict-style config merging.  Only used by the reference arm of bench.py."""
from __future__ import annotations

import copy
import json


class DictConfig(dict):
    pass


class ListConfig(list):
    pass


def _wrap(x):
    if isinstance(x, dict) and not isinstance(x, DictConfig):
        return DictConfig({k: _wrap(v) for k, v in x.items()})
    if isinstance(x, list) and not isinstance(x, ListConfig):
        return ListConfig([_wrap(v) for v in x])
    return x


def _merge(a, b):
    out = DictConfig(a)
    for k, v in b.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = _merge(out[k], v)
        else:
            out[k] = copy.deepcopy(v)
    return out


class OmegaConf:
    @staticmethod
    def create(obj=None):
        return _wrap(copy.deepcopy(obj) if obj is not None else {})

    @staticmethod
    def merge(*cfgs):
        out = DictConfig()
        for c in cfgs:
            out = _merge(out, c or {})
        return out

    @staticmethod
    def update(cfg, key, value, force_add=True, merge=True):
        parts = key.split(".")
        d = cfg
        for p in parts[:-1]:
            if p not in d or not isinstance(d[p], dict):
                d[p] = DictConfig()
            d = d[p]
        d[parts[-1]] = _wrap(value)

    @staticmethod
    def select(cfg, key, default=None):
        d = cfg
        for p in key.split("."):
            if not isinstance(d, dict) or p not in d:
                return default
            d = d[p]
        return d

    @staticmethod
    def to_container(cfg, resolve=True, **_):
        if isinstance(cfg, dict):
            return {k: OmegaConf.to_container(v) for k, v in cfg.items()}
        if isinstance(cfg, list):
            return [OmegaConf.to_container(v) for v in cfg]
        return cfg

    @staticmethod
    def is_dict(cfg):
        return isinstance(cfg, dict)

    @staticmethod
    def is_list(cfg):
        return isinstance(cfg, list)

    @staticmethod
    def load(path):
        with open(path) as f:
            text = f.read()
        if str(path).endswith(".json"):
            return _wrap(json.loads(text))
        import yaml

        return _wrap(yaml.safe_load(text) or {})
