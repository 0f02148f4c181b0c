"""Streaming conversion of a quantised Hugging Face checkpoint directory to bf16 safetensors.

Plan first, then stream: the index (or, without one, the shard headers) gives every tensor name and its shard; the
profile pairs each value tensor with its companions (scales, shape) wherever they live.  A companion in ANOTHER shard
file than its weight is normal in published checkpoints (shards are cut by size, not by module), so companions are
fetched through a small cache of open shard readers.  Output shards keep the input file names (a logical tensor lands
in the shard of its value tensor); non-tensor files are carried over; `config.json` loses its `quantization_config`
and declares bf16; the index is written LAST, so an interrupted run never looks complete.

The reference's tool with the same job: scripts/dequant/converter.py (plus one format class per model).
"""
from __future__ import annotations

import json
import os
import shutil
from collections import OrderedDict
from dataclasses import dataclass

import torch

try:
    from .formats import PROFILES, QuantProfile
except ImportError:  # run as a script from this directory
    from formats import PROFILES, QuantProfile

INDEX = "model.safetensors.index.json"


@dataclass
class LogicalTensor:
    name: str                      # output key
    parts: dict[str, str]          # role -> physical key ("weight" only for tensors copied as they are)
    quantised: bool


@dataclass
class Summary:
    tensors: int = 0
    dequantised: int = 0
    cross_shard: int = 0           # quantised tensors with a companion in another shard file
    shards: int = 0


def read_weight_map(model_dir: str) -> dict[str, str]:
    idx = os.path.join(model_dir, INDEX)
    if os.path.exists(idx):
        wm = json.load(open(idx)).get("weight_map")
        if wm:
            return dict(wm)
    from safetensors import safe_open

    out = {}
    for fn in sorted(os.listdir(model_dir)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, fn), framework="pt") as f:
                out.update({k: fn for k in f.keys()})
    if not out:
        raise FileNotFoundError(f"{model_dir} holds neither {INDEX} nor *.safetensors files")
    return out


def plan(weight_map: dict[str, str], profile: QuantProfile) -> list[LogicalTensor]:
    """Pair value tensors with their companions; anything unpaired is copied.  Half-described tensors are an error."""
    keys = set(weight_map)
    used: set[str] = set()
    out: list[LogicalTensor] = []
    vrole = profile.value_role
    companions = [r for r in profile.roles if r != vrole]
    for key in sorted(keys):
        vs = next((s for s in profile.roles[vrole] if key.endswith(s)), None)
        if vs is None:
            continue
        stem = key[: -len(vs)]
        found: dict[str, str] = {}
        for role in companions:
            hits = [stem + s for s in profile.roles[role] if stem + s in keys]
            if len(hits) > 1:
                raise ValueError(f"{key}: several {role} tensors ({', '.join(hits)})")
            if hits:
                found[role] = hits[0]
        if not found:
            if vrole == "packed":
                raise ValueError(f"{key}: packed values without {' / '.join(companions)} tensors")
            continue                                   # an ordinary (unquantised) weight
        missing = [r for r in companions if r not in found]
        if missing:
            raise ValueError(f"{key}: quantised tensor lacks its {', '.join(missing)} tensor")
        logical = stem + profile.logical_suffix
        if logical != key and logical in keys:
            raise ValueError(f"{logical} exists both packed and unpacked")
        out.append(LogicalTensor(logical, {vrole: key, **found}, True))
        used.update([key, *found.values()])
    orphans = [k for k in keys - used if any(k.endswith(s) for r in companions for s in profile.roles[r])
               and not k.endswith((".weight", ".bias"))]
    if orphans:
        raise ValueError(f"scale / shape tensors without a quantised weight: {sorted(orphans)[:4]}")
    out.extend(LogicalTensor(k, {"weight": k}, False) for k in sorted(keys - used))
    return out


class ShardReaders:
    """At most `limit` shard files open at a time (least recently used closed first)."""

    def __init__(self, model_dir: str, limit: int = 4):
        self.dir, self.limit, self.open = model_dir, limit, OrderedDict()

    def get(self, shard: str, key: str) -> torch.Tensor:
        from safetensors import safe_open

        f = self.open.pop(shard, None)
        if f is None:
            f = safe_open(os.path.join(self.dir, shard), framework="pt", device="cpu")
            f.__enter__()
            while len(self.open) >= self.limit:
                self.open.popitem(last=False)[1].__exit__(None, None, None)
        self.open[shard] = f
        return f.get_tensor(key)

    def close(self) -> None:
        for f in self.open.values():
            f.__exit__(None, None, None)
        self.open.clear()


def convert_checkpoint(model_dir: str, output_dir: str, profile: str | QuantProfile) -> Summary:
    from safetensors.torch import save_file

    prof = PROFILES[profile] if isinstance(profile, str) else profile
    src, dst = os.path.realpath(model_dir), os.path.realpath(output_dir)
    if src == dst or dst.startswith(src + os.sep):
        raise ValueError("the output directory must not be (inside) the input directory")
    os.makedirs(dst, exist_ok=True)
    wmap = read_weight_map(src)
    cfg = prof.settings(src)
    by_shard: dict[str, list[LogicalTensor]] = {}
    for lt in plan(wmap, prof):
        by_shard.setdefault(wmap[lt.parts[prof.value_role if lt.quantised else "weight"]], []).append(lt)
    readers, summary, out_map = ShardReaders(src), Summary(), {}
    try:
        for shard in sorted(by_shard):
            tensors = {}
            for lt in by_shard[shard]:
                parts = {role: readers.get(wmap[k], k) for role, k in lt.parts.items()}
                if lt.quantised:
                    tensors[lt.name] = prof.decode(parts, cfg)
                    summary.dequantised += 1
                    summary.cross_shard += int(len({wmap[k] for k in lt.parts.values()}) > 1)
                else:
                    tensors[lt.name] = parts["weight"].contiguous()
                out_map[lt.name] = shard
            save_file(tensors, os.path.join(dst, shard), metadata={"format": "pt"})
            summary.tensors += len(tensors)
            summary.shards += 1
    finally:
        readers.close()
    for fn in os.listdir(src):
        p = os.path.join(src, fn)
        if os.path.isfile(p) and not fn.endswith(".safetensors") and fn != INDEX:
            shutil.copy2(p, os.path.join(dst, fn))
    cpath = os.path.join(dst, "config.json")
    if os.path.exists(cpath):
        c = json.load(open(cpath))
        for node in (c, c.get("text_config") if isinstance(c.get("text_config"), dict) else None):
            if node is not None:
                node.pop("quantization_config", None)
                node["torch_dtype"] = "bfloat16"
        json.dump(c, open(cpath, "w"), indent=2)
    json.dump({"metadata": {"format": "pt"}, "weight_map": dict(sorted(out_map.items()))}, open(os.path.join(dst, INDEX), "w"),
              indent=2)
    return summary


def cli(profile: str, in_flag: str, out_flag: str, argv=None) -> Summary:
    import argparse

    ap = argparse.ArgumentParser(description=f"{profile}: quantised Hugging Face checkpoint -> bf16")
    ap.add_argument(in_flag, dest="src", required=True)
    ap.add_argument(out_flag, dest="dst", required=True)
    a = ap.parse_args(argv)
    s = convert_checkpoint(a.src, a.dst, profile)
    print(f"{profile}: {s.tensors} tensors in {s.shards} shard(s), {s.dequantised} dequantised "
          f"({s.cross_shard} with scales in another shard) -> {a.dst}")
    return s
