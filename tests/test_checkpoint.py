"""Checkpoint layer: HF export / reload, native sharded save / resume, commit markers, EP stamping, layout guards."""
import json
import os

import pytest
import torch

from dist_utils import run_distributed
from torchturbo_b200.engine.checkpoint import (dcp_status, hf_status, resolve_model_format, save_scheduler,
                                               validate_output_dir, validate_peft_configs)
from torchturbo_b200.engine.checkpoint.layout import ModelFormat, load_scheduler

MOE = dict(model_type="qwen3_moe", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
           head_dim=16, intermediate_size=128, moe_intermediate_size=32, num_experts=8, num_experts_per_tok=2,
           vocab_size=256)


def _build(ep, seed=0):
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan

    eng = TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "parallel_plan": {"sp_size": 1, "ep_size": ep},
                                                   "activation_checkpointing": {"enabled": False}}))
    model = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(MOE), "seed": seed})
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-2, weight_decay=0.0))
    return eng, model, opt


def _step(eng, model, opt, i=0):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.loops import train_step

    ds = SyntheticPackedDataset(8, 48, MOE["vocab_size"], num_docs=2, seed=9)
    return float(train_step(eng, model, opt, [PackedCollator()([ds[i]])])[0])


def _full(p):
    return p.full_tensor() if hasattr(p, "full_tensor") else p


def _w_roundtrip(rank, world, ep, root):
    import torch.distributed as dist

    eng, model, opt = _build(ep)
    _step(eng, model, opt, 0)
    sched = eng.prepare_lr_scheduler(opt, "linear", num_warmup_steps=1, num_training_steps=10)
    sched.step()
    ckpt = os.path.join(root, "checkpoint-1")
    eng.save_model(model, ckpt, final=True)
    eng.save_optimizer_and_scheduler(model, opt, sched, ckpt)
    assert dcp_status(os.path.join(ckpt, "model_distcp")) == "complete"
    assert hf_status(os.path.join(ckpt, "huggingface")) == "complete"
    meta = json.load(open(os.path.join(ckpt, "torchturbo", "checkpoint.json")))
    assert meta["schema_version"] == 1 and meta["engine"]["ep_size"] == ep
    ref_loss = _step(eng, model, opt, 1)
    ref_params = {n: _full(p).detach().clone() for n, p in model.named_parameters()}
    # ---- resume into a differently initialised model
    eng2, model2, opt2 = _build(ep, seed=123)
    sched2 = eng2.prepare_lr_scheduler(opt2, "linear", num_warmup_steps=1, num_training_steps=10)
    eng2.load_from_checkpoint(model2, ckpt)
    eng2.load_optimizer_and_scheduler(model2, opt2, sched2, ckpt)
    assert sched2.last_epoch == sched.last_epoch
    loss2 = _step(eng2, model2, opt2, 1)
    assert abs(loss2 - ref_loss) < 1e-5, (loss2, ref_loss)
    for n, p in model2.named_parameters():
        assert torch.allclose(_full(p), ref_params[n], atol=1e-6), n
    # ---- reload the HF export as pretrained weights (EP layout preserved through per-expert HF tensors)
    eng3, model3, _ = _build(ep, seed=7)
    eng3.checkpoint.load_pretrained(model3, os.path.join(ckpt, "huggingface"))
    eng4, model4, _ = _build(ep, seed=0)
    eng4.load_from_checkpoint(model4, ckpt)
    for (n, a), (_, b) in zip(model3.named_parameters(), model4.named_parameters()):
        assert torch.allclose(_full(a).float(), _full(b).float(), atol=1e-2, rtol=1e-2), n   # export is bf16
    if rank == 0:
        idx = json.load(open(os.path.join(ckpt, "huggingface", "model.safetensors.index.json")))["weight_map"]
        assert "model.layers.0.self_attn.q_proj.weight" in idx and "model.layers.1.mlp.experts.7.down_proj.weight" in idx
        assert "model.layers.0.mlp.gate.weight" in idx and not any("qkv_proj" in k or "weight1" in k for k in idx)
    dist.barrier()


@pytest.mark.parametrize("world,ep", [(1, 1), (2, 2), (2, 1)])
def test_save_resume_and_hf_roundtrip(tmp_path, world, ep):
    run_distributed(_w_roundtrip, world, ep, str(tmp_path))


def _w_split_load(rank, world, root):
    """HF load on 2 ranks: every shared tensor is read by exactly one rank and broadcast (also with a budget so small
    that every broadcast is its own window), experts are read by their owners only; the result equals the source."""
    import torch.distributed as dist

    eng, model, opt = _build(2)
    ckpt = os.path.join(root, "checkpoint-1")
    eng.save_model(model, ckpt, final=True)
    ref = {n: _full(p).detach().clone() for n, p in model.named_parameters()}
    for budget in ("0", "1"):
        if budget == "1":
            os.environ["TORCHTURBO_LOAD_BROADCAST_BYTES"] = "1"
        eng2, model2, _ = _build(2, seed=31)
        eng2.checkpoint.load_pretrained(model2, os.path.join(ckpt, "huggingface"))
        st = eng2.checkpoint.manager.last_load_stats
        t = torch.tensor([st["read_here"], st["received"], st["direct"]])
        both = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(both, t)
        shared = int(both[0][0] + both[0][1])
        assert all(int(b[0] + b[1]) == shared for b in both)                 # same shared tensors on every rank
        assert sum(int(b[0]) for b in both) == shared                        # each one read exactly once
        assert all(int(b[2]) > 0 for b in both)                              # experts: direct reads by their owner
        for n, p in model2.named_parameters():
            assert torch.allclose(_full(p).float(), ref[n].float(), atol=1e-2, rtol=1e-2), n   # export is bf16
    os.environ.pop("TORCHTURBO_LOAD_BROADCAST_BYTES", None)


def test_hf_load_splits_reads_across_ranks(tmp_path):
    run_distributed(_w_split_load, 2, str(tmp_path))


def _w_ep_mismatch(rank, world, root):
    eng, model, opt = _build(2)
    ckpt = os.path.join(root, "checkpoint-1")
    _step(eng, model, opt)
    eng.save_model(model, ckpt)
    eng.save_optimizer_and_scheduler(model, opt, None, ckpt)
    eng1, model1, opt1 = _build(1)
    with pytest.raises(Exception, match="ep_size|lacks"):
        eng1.load_optimizer_and_scheduler(model1, opt1, None, ckpt)


def test_optimizer_resume_rejects_other_ep_size(tmp_path):
    run_distributed(_w_ep_mismatch, 2, str(tmp_path))


def test_commit_markers_and_layout_guards(tmp_path):
    d = tmp_path / "ckpt"
    (d / "model_distcp").mkdir(parents=True)
    assert dcp_status(d / "model_distcp") == "incomplete"
    with pytest.raises(RuntimeError):
        resolve_model_format(d)
    (d / "model_distcp" / ".metadata").write_bytes(b"x")
    assert resolve_model_format(d)[0] is ModelFormat.NATIVE
    hf = tmp_path / "hf"
    hf.mkdir()
    (hf / "model-00001.safetensors").write_bytes(b"")
    assert hf_status(hf) == "incomplete"                       # shards without an index: interrupted export
    (hf / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "model-00001.safetensors", "b": "missing.safetensors"}}))
    assert hf_status(hf) == "incomplete"
    (hf / "missing.safetensors").write_bytes(b"")
    assert hf_status(hf) == "complete"
    with pytest.raises(FileNotFoundError):
        resolve_model_format(tmp_path / "nothing")
    # scheduler file: atomic write, truncated file is reported
    save_scheduler(tmp_path / "scheduler.pt", {"last_epoch": 3})
    assert load_scheduler(tmp_path / "scheduler.pt")["last_epoch"] == 3
    (tmp_path / "scheduler.pt").write_bytes(b"\x80\x02")
    with pytest.raises(RuntimeError):
        load_scheduler(tmp_path / "scheduler.pt")
    # destructive-path guards
    with pytest.raises(ValueError):
        validate_output_dir("/")
    junk = tmp_path / "project"
    (junk / "src").mkdir(parents=True)
    with pytest.raises(ValueError):
        validate_output_dir(junk)
    validate_output_dir(d)


def test_peft_compat_rule():
    a = {"default": {"peft_type": "LORA", "r": 8, "lora_alpha": 16, "target_modules": ["q", "k"], "use_dora": False}}
    validate_peft_configs(a, {"default": dict(a["default"], target_modules=["k", "q"])})
    with pytest.raises(ValueError):
        validate_peft_configs(a, {})
    with pytest.raises(ValueError):
        validate_peft_configs(a, {"default": dict(a["default"], r=16)})
