"""Name and layout rules between engine parameters and Hugging Face checkpoints (`models/weight_converter.py`): fused
attention / MLP projections, per-expert and fused expert tensors under expert parallelism, router and shared-expert
names, tied heads, safetensors header reading."""
from types import SimpleNamespace

import pytest
import torch
from safetensors.torch import save_file

from torchturbo_b200.models.weight_converter import BaseWeightConverter, CheckpointInfo, FusedExpertWeightConverter


def _model(**cfg):
    base = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=8, hidden_size=16, moe_intermediate_size=6, num_experts=4)
    base.update(cfg)
    return SimpleNamespace(config=SimpleNamespace(**base), all_tied_weights_keys={"lm_head.weight": "model.embed_tokens.weight"})


def _ep(size, rank):
    return {"ep": {"ep_size": size, "ep_rank": rank, "ep_group": None}}


def test_fused_qkv_and_gate_up_split_back_into_the_checkpoint_tensors():
    conv = BaseWeightConverter(_model())
    q, k, v = torch.randn(32, 16), torch.randn(16, 16), torch.randn(16, 16)
    rec = conv.load_recipe("model.layers.3.self_attn.qkv_proj.weight")
    assert rec.sources == [f"model.layers.3.self_attn.{p}_proj.weight" for p in "qkv"]
    fused = rec.assemble([q, k, v])
    out = conv.to_hf_tensors("model.layers.3.self_attn.qkv_proj.weight", fused)
    assert torch.equal(out["model.layers.3.self_attn.q_proj.weight"], q) and torch.equal(out["model.layers.3.self_attn.v_proj.weight"], v)
    g, u = torch.randn(10, 16), torch.randn(10, 16)
    rec = conv.load_recipe("model.layers.0.mlp.gate_up_proj.weight")
    assert rec.sources == ["model.layers.0.mlp.gate_proj.weight", "model.layers.0.mlp.up_proj.weight"]
    out = conv.to_hf_tensors("model.layers.0.mlp.gate_up_proj.weight", rec.assemble([g, u]))
    assert torch.equal(out["model.layers.0.mlp.up_proj.weight"], u)
    bias = conv.load_recipe("model.layers.3.self_attn.qkv_proj.bias")
    assert bias.sources[0].endswith("q_proj.bias") and bias.assemble([torch.ones(32), torch.ones(16), torch.ones(16)]).shape == (64,)


def test_router_and_shared_expert_names():
    conv = BaseWeightConverter(_model())
    assert conv.to_hf_name("model.layers.1.mlp.router.weight") == "model.layers.1.mlp.gate.weight"
    assert conv.to_hf_name("model.layers.1.mlp.router.expert_bias") == "model.layers.1.mlp.gate.e_score_correction_bias"
    assert conv.to_hf_name("model.layers.1.mlp.shared_experts.gate.weight") == "model.layers.1.mlp.shared_expert_gate.weight"
    rec = conv.load_recipe("model.layers.1.mlp.shared_experts.gate_up_proj.weight")
    assert rec.sources == ["model.layers.1.mlp.shared_expert.gate_proj.weight", "model.layers.1.mlp.shared_expert.up_proj.weight"]

    class DeepSeekStyle(BaseWeightConverter):
        hf_shared_expert_name = "shared_experts"
        extra_renames = ((r"^model\.norm_f\.", "model.norm."),)

    ds = DeepSeekStyle(_model())
    assert ds.to_hf_name("model.layers.1.mlp.shared_experts.down_proj.weight") == "model.layers.1.mlp.shared_experts.down_proj.weight"
    assert ds.to_hf_name("model.norm_f.weight") == "model.norm.weight"


@pytest.mark.parametrize("ep_size", [1, 2, 4])
def test_per_expert_tensors_of_a_rank_round_trip(ep_size):
    H, Fh, E = 16, 6, 4
    full = {}
    for e in range(E):
        full[f"model.layers.0.mlp.experts.{e}.gate_proj.weight"] = torch.randn(Fh, H)
        full[f"model.layers.0.mlp.experts.{e}.up_proj.weight"] = torch.randn(Fh, H)
        full[f"model.layers.0.mlp.experts.{e}.down_proj.weight"] = torch.randn(H, Fh)
    seen = {}
    for rank in range(ep_size):
        conv = BaseWeightConverter(_model(), _ep(ep_size, rank))
        assert list(conv.local_expert_ids()) == list(range(rank * E // ep_size, (rank + 1) * E // ep_size))
        r1 = conv.load_recipe("model.layers.0.mlp.experts.weight1")
        w1 = r1.assemble([full[s] for s in r1.sources])
        assert w1.shape == (E // ep_size * H, 2 * Fh)                  # engine layout: [local experts * H, gate | up]
        e0 = rank * E // ep_size
        assert torch.equal(w1[:H, :Fh], full[f"model.layers.0.mlp.experts.{e0}.gate_proj.weight"].t())
        r2 = conv.load_recipe("model.layers.0.mlp.experts.weight2")
        w2 = r2.assemble([full[s] for s in r2.sources])
        assert w2.shape == (E // ep_size * Fh, H)
        seen.update(conv.to_hf_tensors("model.layers.0.mlp.experts.weight1", w1))
        seen.update(conv.to_hf_tensors("model.layers.0.mlp.experts.weight2", w2))
    assert set(seen) == set(full) and all(torch.equal(seen[k], full[k]) for k in full)


def test_fused_expert_checkpoints_are_sliced_by_rank_and_fall_back_to_per_expert_names(tmp_path):
    H, Fh, E = 16, 6, 4
    gu, dn = torch.randn(E, 2 * Fh, H), torch.randn(E, H, Fh)
    save_file({"model.layers.0.mlp.experts.gate_up_proj": gu, "model.layers.0.mlp.experts.down_proj": dn,
               "mtp.layers.0.mlp.experts.0.gate_proj.weight": torch.randn(Fh, H)}, str(tmp_path / "model.safetensors"))
    conv = FusedExpertWeightConverter(_model(), _ep(2, 1), str(tmp_path))
    r1 = conv.load_recipe("model.layers.0.mlp.experts.weight1")
    assert r1.sources == ["model.layers.0.mlp.experts.gate_up_proj"]
    w1 = r1.assemble([gu])
    assert w1.shape == (2 * H, 2 * Fh) and torch.equal(w1[:H], gu[2].t())
    out = conv.to_hf_tensors("model.layers.0.mlp.experts.weight1", w1)
    (key, piece), = out.items()
    assert key == "model.layers.0.mlp.experts.gate_up_proj__ep1" and torch.equal(piece, gu[2:4])
    w2 = conv.load_recipe("model.layers.0.mlp.experts.weight2").assemble([dn])
    assert torch.equal(w2[:Fh], dn[2].t())
    # the prediction-depth layer of this checkpoint ships per expert: per-expert rules in both directions
    r = conv.load_recipe("mtp.layers.0.mlp.experts.weight1")
    assert r.sources[0] == "mtp.layers.0.mlp.experts.2.gate_proj.weight" and len(r.sources) == 4
    assert "mtp.layers.0.mlp.experts.3.up_proj.weight" in conv.to_hf_tensors("mtp.layers.0.mlp.experts.weight1", torch.randn(2 * H, 2 * Fh))


def test_tied_head_is_skipped_when_the_checkpoint_omits_it(tmp_path):
    save_file({"model.embed_tokens.weight": torch.randn(5, 4)}, str(tmp_path / "model.safetensors"))
    conv = BaseWeightConverter(_model(), None, str(tmp_path))
    assert conv.load_recipe("lm_head.weight") is None
    assert conv.to_hf_tensors("lm_head.weight", torch.randn(5, 4)) == {}
    save_file({"model.embed_tokens.weight": torch.randn(5, 4), "lm_head.weight": torch.randn(5, 4)}, str(tmp_path / "model.safetensors"))
    conv = BaseWeightConverter(_model(), None, str(tmp_path))
    assert conv.load_recipe("lm_head.weight").sources == ["lm_head.weight"]       # an untied copy in the file is loaded


def test_checkpoint_info_reads_headers_of_sharded_and_single_file_checkpoints(tmp_path):
    a, b = tmp_path / "a", tmp_path / "b"
    a.mkdir(); b.mkdir()
    save_file({"x": torch.zeros(2, 3, dtype=torch.bfloat16)}, str(a / "model.safetensors"))
    info = CheckpointInfo(a)
    assert info.tensor_infos["x"] == ((2, 3), torch.bfloat16) and info.tensor_files["x"] == "model.safetensors"
    save_file({"x": torch.zeros(2)}, str(b / "model-00001-of-00002.safetensors"))
    save_file({"y": torch.zeros(3, dtype=torch.int64)}, str(b / "model-00002-of-00002.safetensors"))
    save_file({"z": torch.zeros(1)}, str(b / "stale.safetensors"))                # not in the index: ignored
    import json
    (b / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "model-00001-of-00002.safetensors",
                                                                                "y": "model-00002-of-00002.safetensors"}}))
    info = CheckpointInfo(b)
    assert set(info.get_tensor_infos()) == {"x", "y"} and info.tensor_infos["y"][1] == torch.int64
    with pytest.raises(FileNotFoundError):
        CheckpointInfo(tmp_path / "missing")
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError):
        CheckpointInfo(tmp_path / "empty")
