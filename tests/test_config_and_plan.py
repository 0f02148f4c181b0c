import json
import os

import pytest
import torch

from torchturbo_b200.engine.args import ARG_SPECS, TorchTurboArgs, parse_torchturbo_args
from torchturbo_b200.engine.config import (EngineConfig, FreezePolicy, FSDPConfig, MixedPrecisionPolicy, ParameterGroup,
                                           build_from_args, parse_mixed_precision)
from torchturbo_b200.parallel import (FSDPParallelPlan, FSDPPlacementSpec, FSDPPlanSpec, VisionBalanceMode,
                                      VisionBalanceSpec)
from torchturbo_b200.utils.fqn import match_fqn


def test_match_fqn():
    assert match_fqn("layers.*.weight", "layers.0.weight")
    assert not match_fqn("layers.*.weight", "layers.0.attn.weight")
    assert match_fqn("layers.**.weight", "layers.0.attn.q.weight")
    assert not match_fqn("layers.*", "model.layers.0")
    assert match_fqn("model.layers.*.mlp.experts", "model.layers.12.mlp.experts")


def test_plan_normalisation_and_match():
    from torch.distributed.tensor import Shard

    plan = FSDPParallelPlan(plan={"a.*": (Shard(0), "edp"), "b": FSDPPlacementSpec(Shard(0)), "c": Shard(1),
                                  "d": FSDPPlanSpec(no_shard=True)}, sp_size=2, ep_size=4)
    assert all(isinstance(v, FSDPPlanSpec) for v in plan.plan.values())
    assert plan.plan["a.*"].placement.mesh_dim == "edp"
    assert plan.match("a.3").placement.mesh_dim == "edp"
    assert plan.match("zzz") is None
    with pytest.raises(ValueError):
        FSDPPlanSpec(no_shard=True, standalone_world_shard=True)
    with pytest.raises(ValueError):
        FSDPPlanSpec(standalone_world_shard=True, placement=FSDPPlacementSpec(Shard(0)))
    with pytest.raises(TypeError):
        VisionBalanceSpec(mode="patch")


def test_plan_roundtrip_partial_override():
    d = {"sp_size": 2, "plan": {"model.visual": {"vision_balance": {"mode": "patch_sq"}}}}
    p = FSDPParallelPlan.from_dict(d)
    spec = p.plan["model.visual"]
    assert spec.vision_balance.mode is VisionBalanceMode.PATCH_SQ and spec.vision_balance.io is None
    assert spec.no_shard is None and p.ep_size is None and p.sp_size == 2
    full = FSDPParallelPlan(plan={"x": FSDPPlanSpec(activation_checkpoint=True)}, sp_size=1, ep_size=2)
    again = FSDPParallelPlan.from_dict(full.to_dict())
    assert again.plan["x"].activation_checkpoint is True and again.ep_size == 2


def test_mixed_precision_rejects_fp16_fp8():
    assert parse_mixed_precision("bfloat16") is MixedPrecisionPolicy.BF16
    for bad in ("fp16", "fp8"):
        with pytest.raises(ValueError):
            parse_mixed_precision(bad)


def test_engine_config_from_dict_flat_and_nested():
    c = EngineConfig.from_dict({"sp_size": 2, "ep_size": 4, "gradient_checkpointing": False, "cpu_offload": True,
                                "moe": {"aux_loss_coeff": 0.01}, "mixed_precision": "bf16", "pp_size": 1})
    assert c.parallel_plan.sp_size == 2 and c.parallel_plan.ep_size == 4
    assert c.activation_checkpointing.enabled is False
    assert c.backend_config.cpu_offload.enabled is True
    assert c.moe.aux_loss_coeff == 0.01
    with pytest.raises(ValueError):
        EngineConfig.from_dict({"nonsense": 1})
    with pytest.raises(ValueError):
        EngineConfig.from_dict({"moe": {"token_dispatcher": "allgather"}})
    d = c.to_dict()
    json.dumps(d)
    assert d["parallel_plan"]["sp_size"] == 2


def test_fsdp_config_validation():
    with pytest.raises(ValueError):
        FSDPConfig(cpu_offload=True)
    with pytest.raises(ValueError):
        FSDPConfig(cpu_offload={"mode": "full"})
    with pytest.raises(ValueError):
        FSDPConfig(prefetch_direction="forward", backward_prefetch_depth=2)
    assert FSDPConfig(cpu_offload={"enabled": True, "mode": "optimizer"}).cpu_offload.mode.value == "optimizer"


def test_freeze_policy_from_list():
    p = FreezePolicy.from_list(["vision_tower", "model.layers.0.*", ParameterGroup.LANGUAGE_MODEL])
    assert p.parameter_groups == (ParameterGroup.VISION_TOWER, ParameterGroup.LANGUAGE_MODEL)
    assert p.patterns == ("model.layers.0.*",) and p.enabled
    assert not FreezePolicy.from_list(None).enabled


def test_four_layer_merge_precedence(tmp_path):
    cfg_file = tmp_path / "c.yaml"
    cfg_file.write_text("engine_config:\n  parallel_plan:\n    sp_size: 4\n    ep_size: 8\n  moe:\n    aux_loss_coeff: 0.5\n")
    # explicit flag beats file beats env beats defaults
    args, rest = parse_torchturbo_args(["--tt_config", str(cfg_file), "--tt_sp_size", "2", "--model_name", "x",
                                        "--tt_plugin", "a.py", "--tt_plugin", "b.py:cfg", "--tt_enable_chunk_loss"])
    assert rest == ["--model_name", "x"] and args.plugin == ["a.py", "b.py:cfg"]
    assert "sp_size" in args.config_overrides and "config" not in args.config_overrides
    c = build_from_args(args, env={"TORCH_TURBO_EP_SIZE": "2", "TORCH_TURBO_MIXED_PRECISION": "bf16", "TORCH_TURBO_SP_SIZE": "16"})
    assert c.parallel_plan.sp_size == 2       # explicit CLI
    assert c.parallel_plan.ep_size == 8       # file over env
    assert c.mixed_precision is MixedPrecisionPolicy.BF16   # env over default
    assert c.moe.aux_loss_coeff == 0.5 and c.loss_chunk.enabled is True
    assert c.plugin_paths == ["a.py", "b.py:cfg"]
    # built-in defaults
    d = build_from_args(TorchTurboArgs(), env={})
    assert d.mixed_precision is MixedPrecisionPolicy.FP32 and d.backend_config.reshard_after_forward == "auto"
    assert d.activation_checkpointing.enabled is True and d.checkpoint.hf_export == "every"


def test_config_file_rejects_unknown_root(tmp_path):
    f = tmp_path / "bad.json"
    f.write_text(json.dumps({"engine": {}}))
    args, _ = parse_torchturbo_args(["--tt_config", str(f)])
    with pytest.raises(ValueError):
        build_from_args(args, env={})
    f.write_text(json.dumps({"engine_config": {"bogus": 1}}))
    with pytest.raises(ValueError):
        build_from_args(args, env={})


def test_freeze_flags_map_to_policy():
    args, _ = parse_torchturbo_args(["--tt_freeze_vision_tower", "--tt_freeze_language_model", "false"])
    c = build_from_args(args, env={})
    assert c.freeze_policy.parameter_groups == (ParameterGroup.VISION_TOWER,)


def test_arg_specs_unique():
    names = [s.name for s in ARG_SPECS]
    assert len(names) == len(set(names))
    envs = [s.env for s in ARG_SPECS if s.env]
    assert len(envs) == len(set(envs))
    for s in ARG_SPECS:
        assert hasattr(TorchTurboArgs(), s.name)
