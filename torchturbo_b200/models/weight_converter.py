"""Name and layout mapping between Hugging Face checkpoints and engine storage.

Engine-side differences that need conversion:
  * fused attention projection   `self_attn.qkv_proj.weight`  = cat(q_proj, k_proj, v_proj) on dim 0
  * fused dense MLP projection   `mlp.gate_up_proj.weight`    = cat(gate_proj, up_proj) on dim 0
  * router                       `mlp.router.weight`          = `mlp.gate.weight`
                                 `mlp.router.expert_bias`     = `mlp.gate.e_score_correction_bias`
  * fused experts                `mlp.experts.weight1 [E_local*H, 2F]` : per expert cat(gate_proj^T, up_proj^T) on the last dim
                                 `mlp.experts.weight2 [E_local*F, H]`  : per expert down_proj^T
    where the local experts of EP rank r are the global experts `[r*E_local, (r+1)*E_local)`.
  * tied output embeddings are omitted from Hugging Face checkpoints.
The layouts match models/weight_converter.py:54-450 of the reference, so its checkpoints load here and
exports from here load there.  `FusedExpertWeightConverter` handles checkpoints that already store experts
as 3-D fused tensors (`experts.gate_up_proj [E, H, 2F]`, `experts.down_proj [E, F, H]`).
"""
from __future__ import annotations

import json
import re
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

import torch

_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
    "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
    "F8_E4M3": getattr(torch, "float8_e4m3fn", None), "F8_E5M2": getattr(torch, "float8_e5m2", None),
}


class CheckpointInfo:
    """Tensor name -> (shape, dtype, file) read from safetensors headers only (no tensor data is touched)."""

    def __init__(self, model_path: str | Path):
        self.path = Path(model_path)
        if not self.path.is_dir():
            raise FileNotFoundError(f"model path not found: {self.path}")
        index = self.path / "model.safetensors.index.json"
        if index.exists():
            files = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        else:
            files = sorted(p.name for p in self.path.glob("*.safetensors"))
            if not files:
                raise FileNotFoundError(f"no safetensors files under {self.path}")
        self.tensor_infos: dict[str, tuple[tuple[int, ...], torch.dtype]] = {}
        self.tensor_files: dict[str, str] = {}
        for fn in files:
            with (self.path / fn).open("rb") as f:
                n = struct.unpack("<Q", f.read(8))[0]
                header = json.loads(f.read(n))
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                self.tensor_infos[name] = (tuple(meta["shape"]), _ST_DTYPES[meta["dtype"]])
                self.tensor_files[name] = fn

    def get_tensor_infos(self):
        return self.tensor_infos


@dataclass
class LoadRecipe:
    """How one engine tensor is assembled: `sources` are Hugging Face tensor names, `assemble` maps the
    loaded tensors (same order) to the *full local* engine tensor (before FSDP sharding)."""

    sources: list[str]
    assemble: Callable[[list[torch.Tensor]], torch.Tensor]


class BaseWeightConverter:
    expert_gate, expert_up, expert_down = "gate_proj", "up_proj", "down_proj"
    hf_router_name, router_name = "gate", "router"
    hf_shared_expert_name = "shared_expert"          # DeepSeek-style checkpoints call it `shared_experts`
    # family-specific (engine regex, Hugging Face replacement) pairs applied to every name before the generic rules
    extra_renames: tuple[tuple[str, str], ...] = ()

    def __init__(self, model, parallel_context: dict | None = None, model_path: str | None = None):
        self.model = model
        self.config = model.config
        ep = (parallel_context or {}).get("ep") or {"ep_size": 1, "ep_rank": 0, "ep_group": None}
        self.ep_size, self.ep_rank, self.ep_group = ep["ep_size"], ep["ep_rank"], ep.get("ep_group")
        self.checkpoint_info = CheckpointInfo(model_path) if model_path else None
        self.tied = dict(getattr(model, "all_tied_weights_keys", {}) or {})
        self.n_q = getattr(self.config, "num_attention_heads", 0)
        self.n_kv = getattr(self.config, "num_key_value_heads", 0)
        self.head_dim = getattr(self.config, "head_dim", 0)
        self.num_experts = getattr(self.config, "num_experts", 0) or 0
        self.num_local_experts = self.num_experts // self.ep_size if self.num_experts else 0

    # ---- names --------------------------------------------------------------------------------------
    def is_expert_param(self, name: str) -> bool:
        return name.endswith("experts.weight1") or name.endswith("experts.weight2")

    def to_hf_name(self, name: str) -> str:
        """Engine FQN -> Hugging Face name for tensors that map one-to-one."""
        for pat, repl in self.extra_renames:
            name = re.sub(pat, repl, name)
        name = re.sub(r"\.mlp\.router\.weight$", f".mlp.{self.hf_router_name}.weight", name)
        name = re.sub(r"\.mlp\.router\.expert_bias$", f".mlp.{self.hf_router_name}.e_score_correction_bias", name)
        name = re.sub(r"\.mlp\.shared_experts\.gate\.weight$", f".mlp.{self.hf_shared_expert_name}_gate.weight", name)
        name = re.sub(r"\.mlp\.shared_experts\.", f".mlp.{self.hf_shared_expert_name}.", name)
        return name

    def local_expert_ids(self) -> range:
        return range(self.ep_rank * self.num_local_experts, (self.ep_rank + 1) * self.num_local_experts)

    # ---- load ---------------------------------------------------------------------------------------
    def load_recipe(self, name: str) -> LoadRecipe | None:
        """Recipe for the engine tensor `name`, or `None` when the tensor is a tied alias that the checkpoint omits."""
        infos = self.checkpoint_info.tensor_infos if self.checkpoint_info else None
        if name in self.tied:
            src = self.to_hf_name(self.tied[name])
            if infos is None or (name not in infos and src in infos):
                return None
        m = re.match(r"(.*)\.self_attn\.qkv_proj\.(weight|bias)$", name)
        if m:
            pre, kind = m.groups()
            return LoadRecipe([f"{pre}.self_attn.{p}_proj.{kind}" for p in "qkv"], lambda ts: torch.cat(ts, dim=0))
        m = re.match(r"(.*)\.gate_up_proj\.weight$", name)
        if m and not self.is_expert_param(name):
            pre = self.to_hf_name(m.group(1) + ".x")[:-2]
            return LoadRecipe([f"{pre}.gate_proj.weight", f"{pre}.up_proj.weight"], lambda ts: torch.cat(ts, dim=0))
        m = re.match(r"(.*)\.experts\.weight1$", name)
        if m:
            pre = m.group(1)
            ids = list(self.local_expert_ids())
            srcs = [f"{pre}.experts.{e}.{p}.weight" for e in ids for p in (self.expert_gate, self.expert_up)]

            def asm(ts, n=len(ids)):
                per = [torch.cat([ts[2 * i].t(), ts[2 * i + 1].t()], dim=-1) for i in range(n)]   # [H, 2F] each
                return torch.cat(per, dim=0)

            return LoadRecipe(srcs, asm)
        m = re.match(r"(.*)\.experts\.weight2$", name)
        if m:
            pre = m.group(1)
            srcs = [f"{pre}.experts.{e}.{self.expert_down}.weight" for e in self.local_expert_ids()]
            return LoadRecipe(srcs, lambda ts: torch.cat([t.t() for t in ts], dim=0))
        return LoadRecipe([self.to_hf_name(name)], lambda ts: ts[0])

    # ---- export -------------------------------------------------------------------------------------
    def to_hf_tensors(self, name: str, tensor: torch.Tensor, expert_offset: int | None = None) -> dict[str, torch.Tensor]:
        """Full local engine tensor -> Hugging Face tensors.  For expert tensors `expert_offset` is the global
        id of the first local expert (defaults to this rank's)."""
        if name in self.tied:
            return {}
        m = re.match(r"(.*)\.self_attn\.qkv_proj\.(weight|bias)$", name)
        if m:
            pre, kind = m.groups()
            D = self.head_dim
            q, k, v = tensor.split([self.n_q * D, self.n_kv * D, self.n_kv * D], dim=0)
            return {f"{pre}.self_attn.q_proj.{kind}": q, f"{pre}.self_attn.k_proj.{kind}": k,
                    f"{pre}.self_attn.v_proj.{kind}": v}
        m = re.match(r"(.*)\.gate_up_proj\.weight$", name)
        if m and not self.is_expert_param(name):
            pre = self.to_hf_name(m.group(1) + ".x")[:-2]
            g, u = tensor.chunk(2, dim=0)
            return {f"{pre}.gate_proj.weight": g, f"{pre}.up_proj.weight": u}
        off = self.ep_rank * self.num_local_experts if expert_offset is None else expert_offset
        m = re.match(r"(.*)\.experts\.weight1$", name)
        if m:
            pre = m.group(1)
            H = self.config.hidden_size
            n = tensor.shape[0] // H
            out = {}
            for i, w in enumerate(tensor.view(n, H, -1)):
                g, u = w.chunk(2, dim=-1)
                out[f"{pre}.experts.{off + i}.{self.expert_gate}.weight"] = g.t().contiguous()
                out[f"{pre}.experts.{off + i}.{self.expert_up}.weight"] = u.t().contiguous()
            return out
        m = re.match(r"(.*)\.experts\.weight2$", name)
        if m:
            pre = m.group(1)
            Fh = self.config.moe_intermediate_size
            n = tensor.shape[0] // Fh
            return {f"{pre}.experts.{off + i}.{self.expert_down}.weight": w.t().contiguous()
                    for i, w in enumerate(tensor.view(n, Fh, -1))}
        return {self.to_hf_name(name): tensor}


class FusedExpertWeightConverter(BaseWeightConverter):
    """For checkpoints whose experts are 3-D fused tensors in the Hugging Face layout: `experts.gate_up_proj
    [E, 2F, H]` and `experts.down_proj [E, H, F]` (nn.Linear orientation per expert; the engine keeps `[E*H, 2F]` and
    `[E*F, H]`, so each expert is transposed on the way in and out).  A rank loads only its expert slice (`narrow` on
    dim 0).  Tensors whose fused key is absent from the checkpoint (the prediction-depth layers of Qwen3.5 ship per
    expert; `transformers` writes per-expert files for the whole model) use the per-expert rules of the base class,
    in both directions (models/weight_converter.py:477-560 of the reference)."""

    def _fused_in_checkpoint(self, key: str) -> bool:
        infos = self.checkpoint_info.tensor_infos if self.checkpoint_info else None
        return infos is None or key in infos

    def load_recipe(self, name: str):
        m = re.match(r"(.*)\.experts\.weight([12])$", name)
        if not m:
            return super().load_recipe(name)
        pre, which = m.groups()
        src = f"{pre}.experts.gate_up_proj" if which == "1" else f"{pre}.experts.down_proj"
        if not self._fused_in_checkpoint(src):
            return super().load_recipe(name)
        lo, n = self.ep_rank * self.num_local_experts, self.num_local_experts

        def asm(ts):
            w = ts[0].narrow(0, lo, n).transpose(1, 2)          # [n, H, 2F] / [n, F, H]
            return w.reshape(-1, w.shape[-1])

        return LoadRecipe([src], asm)

    def to_hf_tensors(self, name, tensor, expert_offset=None):
        m = re.match(r"(.*)\.experts\.weight([12])$", name)
        if not m:
            return super().to_hf_tensors(name, tensor, expert_offset)
        pre, which = m.groups()
        rows = self.config.hidden_size if which == "1" else self.config.moe_intermediate_size
        key = f"{pre}.experts.gate_up_proj" if which == "1" else f"{pre}.experts.down_proj"
        if not self._fused_in_checkpoint(key):
            return super().to_hf_tensors(name, tensor, expert_offset)
        off = self.ep_rank * self.num_local_experts if expert_offset is None else expert_offset
        # a virtual per-EP-rank key; the saver concatenates the `__ep<N>` pieces in rank order
        return {f"{key}__ep{off // max(self.num_local_experts, 1)}":
                tensor.view(-1, rows, tensor.shape[-1]).transpose(1, 2).contiguous()}
