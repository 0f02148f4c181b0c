"""Minimal model configuration objects compatible with Hugging Face `config.json` files.

The engine does not depend on `transformers`: a config is a plain attribute bag with the familiar key
names, `from_pretrained` reads `config.json`, and a `transformers.PretrainedConfig` is accepted anywhere
because only attribute access is used.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Any


class ModelConfig:
    model_type: str = ""
    _defaults: dict[str, Any] = {}

    def __init__(self, **kwargs: Any) -> None:
        merged = {}
        for klass in reversed(type(self).__mro__):
            merged.update(getattr(klass, "_defaults", {}) or {})
        merged.update(self._normalise_hf_keys(dict(kwargs)))
        merged.pop("model_type", None)
        for k, v in merged.items():
            setattr(self, k, v)
        if getattr(self, "head_dim", None) is None and hasattr(self, "hidden_size") and hasattr(self, "num_attention_heads"):
            self.head_dim = self.hidden_size // self.num_attention_heads

    # `config.json` spellings of recent `transformers` releases -> the attribute names the modelling code reads
    _hf_aliases = {"num_local_experts": "num_experts", "n_routed_experts": "num_experts"}

    @classmethod
    def _normalise_hf_keys(cls, d: dict[str, Any]) -> dict[str, Any]:
        """transformers 5 stores the rotary settings as `rope_parameters: {rope_theta, rope_type, ...}` (4.x:
        top-level `rope_theta` + `rope_scaling`) and writes some sizes under their attribute-map alias
        (`num_local_experts` for `num_experts`).  Explicit canonical keys win over aliases; rotary settings inside
        `rope_parameters` win over top-level keys of the same name."""
        for alias, name in cls._hf_aliases.items():
            if alias in d and name not in d:
                d[name] = d[alias]
        rp = d.get("rope_parameters")
        if isinstance(rp, dict):
            # where `rope_parameters` exists it is what transformers 5 reads; a top-level key of the same name is a
            # leftover default written next to it (`partial_rotary_factor` of the Qwen3.5 text config)
            for k in ("rope_theta", "mrope_section", "mrope_interleaved", "partial_rotary_factor"):
                if k in rp:
                    d[k] = rp[k]
            if "rope_scaling" not in d and rp.get("rope_type", "default") not in (None, "default"):
                d["rope_scaling"] = {k: v for k, v in rp.items() if k != "rope_theta"}
        return d

    # -- io ---------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "ModelConfig":
        return cls(**d)

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict[str, Any]:
        out = {"model_type": self.model_type}
        for k, v in vars(self).items():
            if k.startswith("_"):
                continue
            if isinstance(v, ModelConfig):
                v = v.to_dict()
            elif hasattr(v, "is_floating_point") or str(type(v)).startswith("<class 'torch."):
                v = str(v).replace("torch.", "")
            out[k] = copy.deepcopy(v)
        return out

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=2, sort_keys=True)

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.to_dict()})"


class NestedDtype:
    """`dtype` of a composite (text + vision) config lives in its text config.  A `dtype` key at the top level of
    `config.json` reaches the setter before the text config exists: it is kept and applied by `_adopt_dtype()`, which
    the subclass calls once `text_config` is built (a dtype stated in the text config itself wins)."""

    @property
    def dtype(self):
        tc = self.__dict__.get("text_config")
        if tc is None:
            return self.__dict__.get("_dtype_pending")
        return getattr(tc, "dtype", None) or getattr(tc, "torch_dtype", None)

    @dtype.setter
    def dtype(self, v):
        tc = self.__dict__.get("text_config")
        if tc is None:
            self.__dict__["_dtype_pending"] = v
            return
        tc.torch_dtype = v
        tc.dtype = v

    torch_dtype = dtype

    def _adopt_dtype(self) -> None:
        v = self.__dict__.pop("_dtype_pending", None)
        if v is not None and self.dtype is None:
            self.dtype = v


def load_config(path_or_dict) -> ModelConfig:
    """Build the registered config class for a checkpoint directory, a dict, or pass an object through."""
    from .registry import get_model

    if isinstance(path_or_dict, (str, os.PathLike)):
        with open(os.path.join(path_or_dict, "config.json")) as f:
            d = json.load(f)
    elif isinstance(path_or_dict, dict):
        d = dict(path_or_dict)
    else:
        return path_or_dict
    cls = get_model(d["model_type"])
    return cls.config_class.from_dict(d)
