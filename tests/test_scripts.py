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
    sys.modules[name] = mod            # dataclasses resolve annotations through sys.modules
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


def _pack_e2m1(codes):
    """uint8 codes [R, C] (0..15) -> packed bytes [R, C/2], low nibble = even column."""
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8)


def test_model_dequant_profiles_decode_their_formats():
    fm = _load("scripts/dequant/formats.py", "tt_formats")
    torch.manual_seed(0)
    # fp8 with fp32 128x128 block scales (DeepSeek V4 dense weights, Bailing)
    w = torch.randn(200, 300).to(torch.float8_e4m3fn)
    s = torch.rand(2, 3) + 0.5
    want = (w.float() * s.repeat_interleave(128, 0)[:200].repeat_interleave(128, 1)[:, :300]).bfloat16()
    for prof in ("deepseek_v4", "bailing"):
        assert torch.equal(fm.PROFILES[prof].decode({"weight": w, "scale": s}, {}), want)
    # packed mxfp4 with one fp32 scale per row and 32 columns (DeepSeek V4 experts)
    codes = torch.randint(0, 16, (4, 64), dtype=torch.uint8)
    s = torch.rand(4, 2) + 0.5
    want = (fm.E2M1[codes.long()] * s.repeat_interleave(32, 1)).bfloat16()
    assert torch.equal(fm.PROFILES["deepseek_v4"].decode({"weight": _pack_e2m1(codes), "scale": s}, {}), want)
    # DeepSeek V4.1: ue8m0 scales; fp4 per row / 32 columns, fp8 per row / 32 columns or square blocks
    e = torch.randint(120, 134, (4, 2), dtype=torch.uint8)
    want = (fm.E2M1[codes.long()] * torch.exp2(e.float() - 127).repeat_interleave(32, 1)).bfloat16()
    assert torch.equal(fm.PROFILES["deepseek_v4_1"].decode({"weight": _pack_e2m1(codes), "scale": e}, {}), want)
    w = torch.randn(64, 96).to(torch.float8_e4m3fn)
    for shape, (rb, cb) in (((64, 3), (1, 32)), ((2, 3), (32, 32)), ((1, 1), (128, 128))):
        e = torch.randint(120, 134, shape, dtype=torch.uint8)
        full = torch.exp2(e.float() - 127).repeat_interleave(cb, 1)
        full = (full.repeat_interleave(rb, 0) if rb > 1 else full)[:64, :96]
        assert torch.equal(fm.PROFILES["deepseek_v4_1"].decode({"weight": w, "scale": e}, {}), (w.float() * full).bfloat16())
    with pytest.raises(ValueError, match="fits none"):
        fm.PROFILES["deepseek_v4_1"].decode({"weight": w, "scale": torch.zeros(5, 5, dtype=torch.uint8)}, {})
    # Kimi: eight offset-binary nibbles per int32, group scales
    vals = torch.randint(-8, 8, (3, 64))
    words = torch.zeros(3, 8, dtype=torch.int64)
    for i in range(8):
        words |= ((vals[:, i::8] + 8) & 0xF) << (4 * i)
    packed = words.to(torch.int32) if int(words.max()) < 2 ** 31 else (words - (words >= 2 ** 31) * 2 ** 32).to(torch.int32)
    s = torch.rand(3, 2) + 0.5
    got = fm.PROFILES["kimi_k26"].decode({"packed": packed, "scale": s, "shape": torch.tensor([3, 64])}, {"group_size": 32})
    assert torch.equal(got, (vals.float() * s.repeat_interleave(32, 1)).bfloat16())


def test_dequant_converter_finds_scales_in_other_shards_and_rejects_half_described_tensors(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file

    cv = _load("scripts/dequant/convert.py", "tt_convert")
    src, dst = tmp_path / "q", tmp_path / "bf16"
    src.mkdir()
    wa, wb = torch.randn(128, 128).to(torch.float8_e4m3fn), torch.randn(128, 256).to(torch.float8_e4m3fn)
    sa, sb = torch.tensor([[3.0]]), torch.tensor([[0.25, 4.0]])
    # shards cut by size: the scale of `a` sits in shard 2, the scale of `b` in shard 1
    save_file({"l.a.weight": wa, "l.b.weight_scale_inv": sb, "l.norm.weight": torch.ones(8, dtype=torch.bfloat16)}, str(src / "m-1.safetensors"))
    save_file({"l.b.weight": wb, "l.a.weight_scale_inv": sa, "l.a.bias": torch.zeros(4)}, str(src / "m-2.safetensors"))
    wmap = {"l.a.weight": "m-1.safetensors", "l.b.weight_scale_inv": "m-1.safetensors", "l.norm.weight": "m-1.safetensors",
            "l.b.weight": "m-2.safetensors", "l.a.weight_scale_inv": "m-2.safetensors", "l.a.bias": "m-2.safetensors"}
    (src / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wmap}))
    (src / "config.json").write_text(json.dumps({"quantization_config": {"x": 1}, "text_config": {"quantization_config": {}}}))
    bl = _load("scripts/dequant/bailing.py", "tt_bailing")
    summary = bl.main(["--input-fp8-hf-path", str(src), "--output-hf-path", str(dst)])
    assert (summary.tensors, summary.dequantised, summary.cross_shard, summary.shards) == (4, 2, 2, 2)
    idx = json.loads((dst / "model.safetensors.index.json").read_text())["weight_map"]
    assert idx == {"l.a.bias": "m-2.safetensors", "l.a.weight": "m-1.safetensors", "l.b.weight": "m-2.safetensors",
                   "l.norm.weight": "m-1.safetensors"}
    with safe_open(str(dst / "m-1.safetensors"), framework="pt") as f:
        assert torch.equal(f.get_tensor("l.a.weight"), (wa.float() * 3.0).bfloat16())
    with safe_open(str(dst / "m-2.safetensors"), framework="pt") as f:
        got = f.get_tensor("l.b.weight")
    assert torch.equal(got[:, :128], (wb.float()[:, :128] * 0.25).bfloat16()) and torch.equal(got[:, 128:], (wb.float()[:, 128:] * 4.0).bfloat16())
    cfg = json.loads((dst / "config.json").read_text())
    assert "quantization_config" not in cfg and "quantization_config" not in cfg["text_config"] and cfg["torch_dtype"] == "bfloat16"
    # planning errors: a packed tensor without its scale, an orphan scale, output inside input
    kimi = cv.PROFILES["kimi_k26"]
    with pytest.raises(ValueError, match="lacks its scale"):
        cv.plan({"x.weight_packed": "a", "x.weight_shape": "a"}, kimi)
    with pytest.raises(ValueError, match="without a quantised weight"):
        cv.plan({"y.weight_scale_inv": "a", "z.weight": "a"}, cv.PROFILES["bailing"])
    with pytest.raises(ValueError, match="must not be"):
        cv.convert_checkpoint(str(src), str(src / "out"), "bailing")


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


def test_every_run_recipe_parses_against_the_engine_schema():
    """Every `scripts/runs/<model>/*.yaml` must load through the same path `--tt_config` uses (unknown keys are
    rejected there), every launcher must be valid bash and name a recipe that exists."""
    import subprocess

    from torchturbo_b200.engine.config import EngineConfig, load_config_file

    runs = ROOT / "scripts" / "runs"
    recipes = sorted(runs.glob("*/*.yaml"))
    assert len(recipes) >= 14
    for y in recipes:
        cfg = EngineConfig.from_dict(load_config_file(str(y)))
        assert cfg.parallel_plan.ep_size in (1, 8) and cfg.parallel_plan.sp_size in (1, 2, 8), y
    launchers = sorted(runs.glob("*/*.sh")) + [runs / "common.sh"]
    assert len(launchers) >= 25
    for sh in launchers:
        assert subprocess.run(["bash", "-n", str(sh)]).returncode == 0, sh
        text = sh.read_text()
        for tok in text.split():
            if tok.endswith(".yaml}") and "/" in tok:
                name = tok.split("/")[-1].rstrip("}")
                assert (sh.parent / name).exists() or (runs / "qwen3" / name).exists(), (sh, name)
    for j in ("moe_30b_a3b", "dense_14b", "dense_8b"):
        shape = json.loads((runs / "qwen3" / f"{j}.json").read_text())
        assert shape["vocab_size"] == 151936 and shape["model_type"] in ("qwen3", "qwen3_moe")
