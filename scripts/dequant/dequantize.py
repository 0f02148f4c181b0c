"""Offline dequantisation of quantised Hugging Face checkpoints to bf16 safetensors (training runs in bf16 only).

    python scripts/dequant/dequantize.py --input /ckpt/fp8 --output /ckpt/bf16 --format fp8_block

Formats:
  fp8_block  : e4m3 weights with one fp32 `weight_scale_inv` per 128x128 block (DeepSeek / Bailing style)
  mxfp4      : e2m1 values packed two per byte with one ue8m0 scale per 32 values (`*_blocks`, `*_scales`)
  int4_group : symmetric int4 packed eight per int32 with per-group scales (`weight_packed`, `weight_scale`)
Non-quantised tensors are copied unchanged; the index and every non-tensor file are carried over.  Model-specific
front ends with the reference's command lines: deepseekv4.py, deepseekv4_1.py, bailing.py, kimik26.py
(scripts/dequant/{dequantize,converter,deepseekv4,bailing,kimik26}.py of the reference)."""
from __future__ import annotations

import argparse
import json
import os
import shutil

import torch

FP4_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def dequant_fp8_block(w: torch.Tensor, scale_inv: torch.Tensor, block: int = 128) -> torch.Tensor:
    R, C = w.shape
    s = scale_inv.float().repeat_interleave(block, 0)[:R].repeat_interleave(block, 1)[:, :C]
    return (w.float() * s).to(torch.bfloat16)


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """blocks: uint8 [..., G, 16] (32 fp4 values per group), scales: uint8 ue8m0 [..., G]."""
    lo, hi = blocks & 0x0F, blocks >> 4
    vals = torch.stack([FP4_VALUES[lo.long()], FP4_VALUES[hi.long()]], dim=-1).flatten(-2)   # [..., G, 32]
    exp = (scales.to(torch.int32) - 127).float()
    return (vals * torch.exp2(exp).unsqueeze(-1)).flatten(-2).to(torch.bfloat16)


def dequant_int4_group(packed: torch.Tensor, scale: torch.Tensor, group: int = 32) -> torch.Tensor:
    """packed: int32 [R, C/8] (eight 4-bit values, low nibble first, offset-binary), scale: [R, C/group]."""
    shifts = torch.arange(0, 32, 4, device=packed.device)
    nib = ((packed.unsqueeze(-1) >> shifts) & 0xF).to(torch.int8) - 8
    vals = nib.flatten(-2).float()
    return (vals * scale.float().repeat_interleave(group, -1)).to(torch.bfloat16)


def convert_state(tensors: dict[str, torch.Tensor], fmt: str) -> dict[str, torch.Tensor]:
    out = {}
    for name, t in tensors.items():
        if fmt == "fp8_block":
            if name.endswith("weight_scale_inv"):
                continue
            s = tensors.get(name + "_scale_inv")
            out[name] = dequant_fp8_block(t, s) if (s is not None and t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)) else t
        elif fmt == "mxfp4":
            if name.endswith("_scales"):
                continue
            if name.endswith("_blocks"):
                out[name[: -len("_blocks")]] = dequant_mxfp4(t, tensors[name[: -len("_blocks")] + "_scales"])
            else:
                out[name] = t
        elif fmt == "int4_group":
            if name.endswith(("weight_scale", "weight_shape")):
                continue
            if name.endswith("weight_packed"):
                base = name[: -len("_packed")]
                out[base] = dequant_int4_group(t, tensors[base + "_scale"])
            else:
                out[name] = t
        else:
            raise ValueError(f"unknown format {fmt!r}")
    return out


PROFILE_OF = {"fp8_block": "bailing", "mxfp4": "mxfp4_blocks", "int4_group": "kimi_k26"}


def main(argv=None):
    """Generic front end: picks the profile by format name.  Scales are looked up through the checkpoint index, so a
    scale tensor stored in another shard file than its weight is found (`convert.convert_checkpoint`)."""
    import sys

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from convert import convert_checkpoint

    p = argparse.ArgumentParser()
    p.add_argument("--input", required=True)
    p.add_argument("--output", required=True)
    p.add_argument("--format", required=True, choices=sorted(PROFILE_OF))
    a = p.parse_args(argv)
    return convert_checkpoint(a.input, a.output, PROFILE_OF[a.format])


if __name__ == "__main__":
    main()
