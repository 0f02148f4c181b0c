"""`deepseek_v4`: hyper-connected decoder with shared-KV sliding-window + compressed sparse attention and a
`sqrtsoftplus` / hash-routed MoE.

Plan (models/deepseek_v4/parallel_plan.py:9-20,96-131 of the reference): layers and prediction depths checkpointed,
experts on the expert-data-parallel mesh with MoE blocks rebuilt EP-aware, and the small fp32 parameters that every
rank needs whole (`hc_*` mixers, `attn_sink`) kept out of FSDP sharding (`no_shard`, gradients averaged over the
world).  Sequence parallelism gathers the shared key/value stream over the group instead of trading heads
(models/deepseek_v4/model.py:251-569)."""
from __future__ import annotations

from ...engine.metrics.flops import MlaLLMFlops
from ...parallel import FSDPParallelPlan, FSDPPlacementSpec, FSDPPlanSpec
from ..bailing_hybrid.model import HybridTurboMixin
from ..base import TurboModel
import re

import torch

from ..registry import register_model
from ..weight_converter import BaseWeightConverter, LoadRecipe
from .modeling import DeepseekV4Config, DeepseekV4ForCausalLMBase, replace_v4_moe

NO_SHARD_PARAMETERS = ("hc_attn.fn", "hc_attn.base", "hc_attn.scale", "hc_ffn.fn", "hc_ffn.base", "hc_ffn.scale",
                       "hc_head.fn", "hc_head.base", "hc_head.scale", "attn_sink")


class DeepseekV4WeightConverter(BaseWeightConverter):
    """Engine names <-> the flat names of DeepSeek-V4 checkpoints (models/deepseek_v4/model.py:30-62 and the module
    tree of models/deepseek_v4/modeling_deepseek_v4.py:1360-1392 of the reference): `embed`, `layers.N.attn.*`,
    `layers.N.ffn.{gate.weight,gate.bias,gate.tid2eid,experts.E.w1|w2|w3,shared_experts.w1|w2|w3}`, `layers.N.attn_norm`,
    `layers.N.ffn_norm`, `layers.N.hc_{attn,ffn}_{fn,base,scale}`, `norm`, `head`, `hc_head_{fn,base,scale}`; a prediction
    depth `mtp.N` is a decoder layer with `e_proj`, `h_proj`, `enorm`, `hnorm`, `norm`, `hc_head_*` beside its own
    sub-modules (here: `mtp.N.block.*` and one `eh_proj = [e_proj | h_proj]`)."""

    expert_gate, expert_up, expert_down = "w1", "w3", "w2"

    def __init__(self, model, parallel_context=None, model_path=None):
        super().__init__(model, parallel_context, model_path)
        self.num_experts = getattr(self.config, "n_routed_experts", 0) or 0
        self.num_local_experts = self.num_experts // self.ep_size if self.num_experts else 0

    _RULES = (
        (r"^model\.embed_tokens\.", "embed."), (r"^model\.norm\.", "norm."), (r"^lm_head\.", "head."),
        (r"^model\.hc_head\.(fn|base|scale)$", r"hc_head_\1"), (r"^model\.layers\.", "layers."),
        (r"^(mtp\.\d+)\.block\.", r"\1."), (r"^(mtp\.\d+)\.hc_head\.(fn|base|scale)$", r"\1.hc_head_\2"),
        (r"\.self_attn\.", ".attn."), (r"\.hc_(attn|ffn)\.(fn|base|scale)$", r".hc_\1_\2"),
        (r"\.input_layernorm\.", ".attn_norm."), (r"\.post_attention_layernorm\.", ".ffn_norm."),
        (r"\.mlp\.router\.weight$", ".ffn.gate.weight"), (r"\.mlp\.router\.expert_bias$", ".ffn.gate.bias"),
        (r"\.mlp\.router\.tid2eid$", ".ffn.gate.tid2eid"), (r"\.down_proj\.weight$", ".w2.weight"), (r"\.mlp\.", ".ffn."),
    )

    def to_hf_name(self, name: str) -> str:
        for pat, repl in self._RULES:
            name = re.sub(pat, repl, name)
        return name

    def load_recipe(self, name: str):
        m = re.match(r"(.*)\.gate_up_proj\.weight$", name)
        if m and not self.is_expert_param(name):
            pre = self.to_hf_name(m.group(1) + ".x")[:-2]
            return LoadRecipe([f"{pre}.w1.weight", f"{pre}.w3.weight"], lambda ts: torch.cat(ts, dim=0))
        m = re.match(r"(mtp\.\d+)\.eh_proj\.weight$", name)
        if m:
            return LoadRecipe([f"{m.group(1)}.e_proj.weight", f"{m.group(1)}.h_proj.weight"], lambda ts: torch.cat(ts, dim=1))
        m = re.match(r"(.*)\.experts\.weight([12])$", name)
        if m:
            pre, ids = self.to_hf_name(m.group(1) + ".x")[:-2], list(self.local_expert_ids())
            if m.group(2) == "1":
                srcs = [f"{pre}.experts.{e}.{p}.weight" for e in ids for p in ("w1", "w3")]
                return LoadRecipe(srcs, lambda ts, n=len(ids): torch.cat(
                    [torch.cat([ts[2 * i].t(), ts[2 * i + 1].t()], dim=-1) for i in range(n)], dim=0))
            return LoadRecipe([f"{pre}.experts.{e}.w2.weight" for e in ids], lambda ts: torch.cat([t.t() for t in ts], dim=0))
        return LoadRecipe([self.to_hf_name(name)], lambda ts: ts[0])

    def to_hf_tensors(self, name, tensor, expert_offset=None):
        if name in self.tied:
            return {}
        m = re.match(r"(.*)\.gate_up_proj\.weight$", name)
        if m and not self.is_expert_param(name):
            pre = self.to_hf_name(m.group(1) + ".x")[:-2]
            g, u = tensor.chunk(2, dim=0)
            return {f"{pre}.w1.weight": g, f"{pre}.w3.weight": u}
        m = re.match(r"(mtp\.\d+)\.eh_proj\.weight$", name)
        if m:
            e, h = tensor.chunk(2, dim=1)
            return {f"{m.group(1)}.e_proj.weight": e.contiguous(), f"{m.group(1)}.h_proj.weight": h.contiguous()}
        m = re.match(r"(.*)\.experts\.weight([12])$", name)
        if m:
            pre = self.to_hf_name(m.group(1) + ".x")[:-2]
            off = self.ep_rank * self.num_local_experts if expert_offset is None else expert_offset
            if m.group(2) == "1":
                H, out = self.config.hidden_size, {}
                for i, w in enumerate(tensor.view(tensor.shape[0] // H, H, -1)):
                    g, u = w.chunk(2, dim=-1)
                    out[f"{pre}.experts.{off + i}.w1.weight"] = g.t().contiguous()
                    out[f"{pre}.experts.{off + i}.w3.weight"] = u.t().contiguous()
                return out
            Fh = self.config.moe_intermediate_size
            return {f"{pre}.experts.{off + i}.w2.weight": w.t().contiguous()
                    for i, w in enumerate(tensor.view(tensor.shape[0] // Fh, Fh, -1))}
        return {self.to_hf_name(name): tensor}


def get_parallel_plan() -> FSDPParallelPlan:
    from torch.distributed.tensor import Shard

    plan = {
        "model.layers.*.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
        "model.layers.*.mlp": FSDPPlanSpec(replace_module=replace_v4_moe),
        "model.layers.*": FSDPPlanSpec(activation_checkpoint=True),
        "mtp.*.block.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
        "mtp.*.block.mlp": FSDPPlanSpec(replace_module=replace_v4_moe),
        "mtp.*": FSDPPlanSpec(activation_checkpoint=True),
        "model.embed_tokens": FSDPPlanSpec(standalone_world_shard=True),
        "lm_head": FSDPPlanSpec(standalone_world_shard=True),
    }
    for leaf in ("hc_attn", "hc_ffn"):
        plan[f"model.layers.*.{leaf}"] = FSDPPlanSpec(no_shard=True)
        plan[f"mtp.*.block.{leaf}"] = FSDPPlanSpec(no_shard=True)
    plan["model.hc_head"] = FSDPPlanSpec(no_shard=True)
    plan["mtp.*.hc_head"] = FSDPPlanSpec(no_shard=True)
    return FSDPParallelPlan(plan=plan, sp_size=1, ep_size=1)


@register_model("deepseek_v4")
class TurboDeepseekV4ForCausalLM(HybridTurboMixin, TurboModel, DeepseekV4ForCausalLMBase):
    config_class = DeepseekV4Config

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan()

    def on_materialized(self) -> None:
        self.tie_weights()

    def on_prepare_inputs(self, inputs, *, source_inputs=None):
        inputs = TurboModel.on_prepare_inputs(self, inputs, source_inputs=source_inputs)
        inputs.setdefault("global_input_ids", inputs["input_ids"])
        if inputs.get("position_ids") is not None:
            inputs.setdefault("global_position_ids", inputs["position_ids"])
        return inputs

    def get_weight_converter(self, parallel_context, model_path=None):
        return DeepseekV4WeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return MlaLLMFlops
