"""Numeric side of offline dequantisation: what a quantised tensor and its companions (scales, shape) decode to.

Each model family is a `QuantProfile`: how companion tensors are named next to a `.weight`, and a decode function
`(tensors by role, settings) -> bf16 matrix`.  The decoders cover
  * block-scaled fp8 (one fp32 or ue8m0 scale per 128x128 / 32x32 block, or per row and 32-column group),
  * packed fp4 / mxfp4 (two e2m1 values per byte, low nibble first, one scale per row and 32-column group),
  * packed int4 (eight offset-binary nibbles per int32, low nibble first, one scale per row and column group).
Numerics follow scripts/dequant/{deepseekv4,deepseekv4_1,bailing,kimik26}.py of the reference: decode to fp32, multiply
by the expanded scale in fp32, round once to bf16.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from math import ceil
from typing import Callable, Mapping

import torch

E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def _matrix(name: str, t: torch.Tensor) -> None:
    if t.ndim != 2:
        raise ValueError(f"{name} must be a matrix, got shape {tuple(t.shape)}")


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    """uint8 / int8 [R, C/2] -> fp32 [R, C]; the low nibble holds the even column."""
    b = packed.view(torch.uint8)
    pair = torch.stack((b & 0x0F, b >> 4), dim=-1)
    return E2M1[pair.long()].reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def unpack_int4(packed: torch.Tensor, shape: tuple[int, int]) -> torch.Tensor:
    """int32 [R, ceil(C/8)] -> fp32 [R, C]: eight 4-bit values per word, low nibble first, stored with an offset of 8."""
    shifts = torch.arange(0, 32, 4, device=packed.device)
    nib = ((packed.to(torch.int32).unsqueeze(-1) >> shifts) & 0xF) - 8
    return nib.flatten(-2)[:, : shape[1]].float()


def decode_ue8m0(scale: torch.Tensor) -> torch.Tensor:
    """One-byte power-of-two scales (stored as uint8 or as a one-byte float dtype): 2 ** (byte - 127)."""
    if scale.dtype != torch.uint8:
        if scale.element_size() != 1:
            raise ValueError(f"ue8m0 scales are one byte wide, got {scale.dtype}")
        scale = scale.view(torch.uint8)
    return torch.exp2(scale.float() - 127.0)


def expand_scale(scale: torch.Tensor, shape: tuple[int, int], *, allowed: tuple[tuple[int, int], ...]) -> torch.Tensor:
    """Broadcast a per-block scale to `shape`.  `allowed` lists the (row block, column block) geometries a format may use
    (row block 1 = one scale row per weight row); the first one whose scale shape matches is taken."""
    _matrix("scale", scale)
    rows, cols = shape
    for rb, cb in allowed:
        if tuple(scale.shape) == (ceil(rows / rb), ceil(cols / cb)):
            out = scale.repeat_interleave(cb, dim=1)
            if rb > 1:
                out = out.repeat_interleave(rb, dim=0)
            return out[:rows, :cols]
    want = [(ceil(rows / rb), ceil(cols / cb)) for rb, cb in allowed]
    raise ValueError(f"scale shape {tuple(scale.shape)} fits none of {want} for a {shape} weight")


def finish(values: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    if values.shape != scales.shape:
        raise ValueError(f"decoded weight {tuple(values.shape)} and expanded scale {tuple(scales.shape)} differ")
    return (values.float() * scales.float()).to(torch.bfloat16).contiguous()


# ------------------------------------------------------------------------------------------------------------------
# decoders
# ------------------------------------------------------------------------------------------------------------------
def decode_deepseek_v4(t: Mapping[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """fp8 with fp32 128x128 block scales, or packed mxfp4 with one fp32 scale per row and 32 columns."""
    w, s = t["weight"], t["scale"]
    _matrix("weight", w)
    if w.dtype in (torch.int8, torch.uint8):
        v = unpack_e2m1(w)
        s = s.float().unsqueeze(0) if (s.ndim == 1 and v.shape[0] == 1) else s.float()
        return finish(v, expand_scale(s, tuple(v.shape), allowed=((1, 32),)))
    if not (w.is_floating_point() and w.element_size() == 1):
        raise ValueError(f"expected fp8 or packed fp4 bytes, got {w.dtype}")
    return finish(w, expand_scale(s.float(), tuple(w.shape), allowed=((128, 128),)))


def decode_deepseek_v41(t: Mapping[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """ue8m0 scales throughout: packed fp4 per row and 32 columns; fp8 e4m3 per row and 32 columns, or 32x32 / 128x128 blocks."""
    w, s = t["weight"], t["scale"]
    _matrix("weight", w)
    if w.dtype in (torch.int8, torch.uint8):
        v = unpack_e2m1(w)
        return finish(v, expand_scale(decode_ue8m0(s), tuple(v.shape), allowed=((1, 32),)))
    if w.dtype != torch.float8_e4m3fn:
        raise ValueError(f"expected fp8 e4m3 or packed fp4 bytes, got {w.dtype}")
    return finish(w, expand_scale(decode_ue8m0(s), tuple(w.shape), allowed=((1, 32), (32, 32), (128, 128))))


def decode_fp8_block128(t: Mapping[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    w, s = t["weight"], t["scale"]
    _matrix("weight", w)
    if not (w.is_floating_point() and w.element_size() == 1):
        raise ValueError(f"expected an fp8 weight, got {w.dtype}")
    return finish(w, expand_scale(s.float(), tuple(w.shape), allowed=((128, 128),)))


def decode_int4_group(t: Mapping[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    shape = tuple(int(v) for v in t["shape"].reshape(-1).tolist())
    if len(shape) != 2 or min(shape) <= 0:
        raise ValueError(f"weight_shape must hold two positive sizes, got {shape}")
    v = unpack_int4(t["packed"], shape)
    if tuple(v.shape) != shape:
        raise ValueError(f"unpacked int4 weight is {tuple(v.shape)}, the checkpoint says {shape}")
    s = t["scale"].float()
    s = s.unsqueeze(1) if s.ndim == 1 else s
    g = int(cfg.get("group_size", 32))
    s = expand_scale(s, shape, allowed=((1, g),)) if g > 0 else s.reshape(shape)
    return finish(v, s)


# ------------------------------------------------------------------------------------------------------------------
# profiles
# ------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class QuantProfile:
    name: str
    # role -> suffixes that may follow the logical tensor's stem (the key without its `.weight`); the role "weight" /
    # "packed" names the tensor that carries the values
    roles: dict[str, tuple[str, ...]]
    decode: Callable[[Mapping[str, torch.Tensor], dict], torch.Tensor]
    settings: Callable[[str], dict] = field(default=lambda model_dir: {})
    logical_suffix: str = ".weight"     # appended to the stem to name the bf16 result

    @property
    def value_role(self) -> str:
        return "packed" if "packed" in self.roles else "weight"


def _kimi_settings(model_dir: str) -> dict:
    """Group size of the int4 scheme from `quantization_config` (compressed-tensors layout), default 32."""
    try:
        q = json.load(open(os.path.join(model_dir, "config.json")))
    except OSError:
        return {"group_size": 32}
    q = q.get("quantization_config") or (q.get("text_config") or {}).get("quantization_config") or {}
    for grp in (q.get("config_groups") or {}).values():
        gs = (grp.get("weights") or {}).get("group_size")
        if gs:
            return {"group_size": int(gs)}
    return {"group_size": int(q.get("group_size", 32))}


def decode_mxfp4_blocks(t: Mapping[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """`*_blocks` uint8 [..., G, 16] (32 e2m1 values per group) with `*_scales` ue8m0 [..., G]; any leading dimensions."""
    vals = unpack_e2m1(t["weight"])                                   # [..., G, 32]
    return (vals * decode_ue8m0(t["scale"]).unsqueeze(-1)).flatten(-2).to(torch.bfloat16).contiguous()


PROFILES = {
    "mxfp4_blocks": QuantProfile("mxfp4_blocks", {"weight": ("_blocks",), "scale": ("_scales",)}, decode_mxfp4_blocks,
                                 logical_suffix=""),
    "deepseek_v4": QuantProfile("deepseek_v4", {"weight": (".weight",), "scale": (".scale",)}, decode_deepseek_v4),
    "deepseek_v4_1": QuantProfile("deepseek_v4_1", {"weight": (".weight",), "scale": (".scale", ".weight_scale_inv")},
                                  decode_deepseek_v41),
    "bailing": QuantProfile("bailing", {"weight": (".weight",), "scale": (".weight_scale_inv",)}, decode_fp8_block128),
    "kimi_k26": QuantProfile("kimi_k26", {"packed": (".weight_packed",), "scale": (".weight_scale",),
                                          "shape": (".weight_shape",)}, decode_int4_group, _kimi_settings),
}
