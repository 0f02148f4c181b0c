"""Stand-alone scripts: offline dequantisation numerics and file handling, dataset converters, native -> HF export
argument guards, launcher argument splitting."""
import importlib.util
import json
import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _load(rel: str, name: str):
    spec = importlib.util.spec_from_file_location(name, ROOT / rel)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_fp8_block_dequantisation_scales_each_128_block():
    dq = _load("scripts/dequant/dequantize.py", "tt_dequant")
    torch.manual_seed(0)
    w = torch.randn(200, 300).to(torch.float8_e4m3fn)
    s = torch.rand(2, 3) + 0.5
    out = dq.dequant_fp8_block(w, s)
    assert out.dtype == torch.bfloat16 and out.shape == (200, 300)
    ref = w.float().clone()
    for i in range(2):
        for j in range(3):
            ref[i * 128:(i + 1) * 128, j * 128:(j + 1) * 128] *= s[i, j]
    assert torch.equal(out, ref.to(torch.bfloat16))


def test_mxfp4_and_int4_dequantisation():
    dq = _load("scripts/dequant/dequantize.py", "tt_dequant")
    # mxfp4: byte 0x21 = low nibble 1 (0.5), high nibble 2 (1.0); scale byte 128 = 2^1
    blocks = torch.full((1, 2, 16), 0x21, dtype=torch.uint8)
    blocks[0, 1, 0] = 0x9F                              # low nibble 0xF (-6.0), high nibble 0x9 (-0.5)
    scales = torch.tensor([[128, 126]], dtype=torch.uint8)
    out = dq.dequant_mxfp4(blocks, scales)
    assert out.shape == (1, 64) and out.dtype == torch.bfloat16
    assert out[0, 0] == 1.0 and out[0, 1] == 2.0         # 0.5 * 2, 1.0 * 2
    assert out[0, 32] == -3.0 and out[0, 33] == -0.25    # -6 * 0.5, -0.5 * 0.5
    # int4: eight offset-binary nibbles per int32, low nibble first
    vals = torch.tensor([[-8, -1, 0, 1, 7, 3, -3, 2] * 4], dtype=torch.int32)        # [1, 32]
    packed = torch.zeros(1, 4, dtype=torch.int32)
    for c in range(32):
        packed[0, c // 8] |= ((vals[0, c] + 8) & 0xF) << (4 * (c % 8))
    out = dq.dequant_int4_group(packed, torch.tensor([[0.5]]), group=32)
    assert torch.equal(out.float(), vals.float() * 0.5)


def test_dequantize_cli_rewrites_shards_index_and_config(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file

    dq = _load("scripts/dequant/dequantize.py", "tt_dequant")
    src, dst = tmp_path / "q", tmp_path / "bf16"
    src.mkdir()
    w = torch.randn(128, 256).to(torch.float8_e4m3fn)
    save_file({"model.layers.0.w.weight": w, "model.layers.0.w.weight_scale_inv": torch.tensor([[2.0, 0.5]]),
               "model.norm.weight": torch.ones(4, dtype=torch.bfloat16)}, str(src / "model-00001-of-00001.safetensors"))
    (src / "config.json").write_text(json.dumps({"hidden_size": 4, "quantization_config": {"quant_method": "fp8"}}))
    (src / "tokenizer.json").write_text("{}")
    (src / "model.safetensors.index.json").write_text("{}")
    dq.main(["--input", str(src), "--output", str(dst), "--format", "fp8_block"])
    with safe_open(str(dst / "model-00001-of-00001.safetensors"), framework="pt") as f:
        keys = set(f.keys())
        got = f.get_tensor("model.layers.0.w.weight")
    assert keys == {"model.layers.0.w.weight", "model.norm.weight"}              # scales are consumed
    assert got.dtype == torch.bfloat16
    assert torch.equal(got[:, :128], (w.float()[:, :128] * 2.0).to(torch.bfloat16))
    assert torch.equal(got[:, 128:], (w.float()[:, 128:] * 0.5).to(torch.bfloat16))
    cfg = json.loads((dst / "config.json").read_text())
    assert "quantization_config" not in cfg and cfg["torch_dtype"] == "bfloat16"
    idx = json.loads((dst / "model.safetensors.index.json").read_text())
    assert idx["weight_map"] == {"model.layers.0.w.weight": "model-00001-of-00001.safetensors",
                                 "model.norm.weight": "model-00001-of-00001.safetensors"}
    assert (dst / "tokenizer.json").exists()
    with pytest.raises(ValueError, match="unknown format"):
        dq.convert_state({"a": torch.zeros(1)}, "nf4")


def test_dataset_converters(tmp_path):
    lf = _load("scripts/dataset/convert_lf_to_swift.py", "tt_lf2swift")
    r = lf.convert_record({"system": "S", "instruction": "do", "input": "x", "output": "done", "images": ["a.png"]})
    assert r == {"messages": [{"role": "system", "content": "S"}, {"role": "user", "content": "do\nx"},
                              {"role": "assistant", "content": "done"}], "images": ["a.png"]}
    r = lf.convert_record({"conversations": [{"from": "human", "value": "q"}, {"from": "gpt", "value": "a"}]})
    assert [m["role"] for m in r["messages"]] == ["user", "assistant"]
    r = lf.convert_record({"instruction": "q", "chosen": {"from": "gpt", "value": "good"}, "rejected": "bad"}, dpo=True)
    assert r["messages"][-1] == {"role": "assistant", "content": "good"} and r["rejected_response"] == "bad"
    src, dst = tmp_path / "in.json", tmp_path / "out.jsonl"
    src.write_text(json.dumps([{"instruction": "a", "output": "b"}, {"instruction": "c", "output": "d"}]))
    assert lf.main([str(src), str(dst)]) == 2
    rows = [json.loads(l) for l in dst.read_text().splitlines()]
    assert len(rows) == 2 and rows[1]["messages"][1]["content"] == "d"
    dpo = _load("scripts/dataset/convert_text_dpo_to_swift.py", "tt_dpo2swift")
    src2 = tmp_path / "p.jsonl"
    src2.write_text(json.dumps({"prompt": "p", "chosen": "c", "rejected": "r"}) + "\n\n")
    assert dpo.main([str(src2), str(dst)]) == 1
    assert json.loads(dst.read_text())["rejected_response"] == "r"


def test_dcp_to_hf_guards_and_export_config(tmp_path):
    mod = _load("scripts/checkpoint/dcp_to_hf.py", "tt_dcp2hf")
    cfg = mod.build_export_config({"engine": {"mixed_precision": "fp32", "ep_size": 2, "mtp_enabled": True}})
    assert cfg.mixed_precision.value == "fp32" and cfg.parallel_plan.ep_size == 2 and cfg.parallel_plan.sp_size == 1
    assert cfg.mtp.enabled is True and cfg.activation_checkpointing.enabled is False
    with pytest.raises(FileNotFoundError):
        mod.main(["--checkpoint_dir", str(tmp_path / "nope"), "--output_dir", str(tmp_path / "o")])
    ck = tmp_path / "ck"
    ck.mkdir()
    with pytest.raises(ValueError, match="must differ"):
        mod.main(["--checkpoint_dir", str(ck), "--output_dir", str(ck)])
    with pytest.raises(FileNotFoundError, match="checkpoint.json"):
        mod.main(["--checkpoint_dir", str(ck), "--output_dir", str(tmp_path / "o")])


def test_launchers_split_engine_flags_from_framework_arguments(monkeypatch):
    from torchturbo_b200.engine.args import parse_torchturbo_args

    tt, rest = parse_torchturbo_args(["--tt_sp_size", "2", "--model", "m", "--tt_profiling", "--dataset", "d", "--tt_ep_size=4"])
    assert rest == ["--model", "m", "--dataset", "d"] and tt.sp_size == 2 and tt.ep_size == 4 and tt.profiling is True
    for script in ("run_lf.py", "run_swift.py", "run_sft.py"):
        src = (ROOT / "scripts" / "runs" / script).read_text()
        compile(src, script, "exec")                                   # launchers at least parse
    assert "adapter.main(stage, rest)" in (ROOT / "scripts" / "runs" / "run_swift.py").read_text()
