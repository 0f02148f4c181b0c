"""LoRA / DoRA through the engine: fine-tuning from a base checkpoint (wrapped parameters are read under their base names,
adapters start as a no-op), training touches adapters only, and the Hugging Face export is a plain checkpoint of the base
architecture with the adapters merged in, on one rank and with expert parallelism on two."""
import os

import pytest
import torch

from dist_utils import run_distributed

MOE = dict(model_type="qwen3_moe", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
           intermediate_size=128, moe_intermediate_size=32, num_experts=8, num_experts_per_tok=2, vocab_size=512)
DENSE = dict(model_type="qwen3", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
             intermediate_size=128, vocab_size=512, tie_word_embeddings=False)
PEFT = {"r": 4, "lora_alpha": 8, "target_modules": ["qkv_proj", "o_proj"], "target_parameters": ["experts.weight1", "experts.weight2"]}


def _logits(model, b):
    cu = b["cu_seq_lens_q"]
    with torch.no_grad():
        return model(input_ids=b["input_ids"], position_ids=b["position_ids"], cu_seq_lens_q=cu, cu_seq_lens_k=cu,
                     max_length_q=b["max_length_q"], max_length_k=b["max_length_q"])["logits"].float()


def _names(hf_dir):
    from safetensors import safe_open

    out = set()
    for fn in os.listdir(hf_dir):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(hf_dir, fn), "pt") as sf:
                out |= set(sf.keys())
    return out


def _effective(model):
    """{base parameter name: the weight the adapted model computes with}."""
    from torchturbo_b200.engine.peft.lora import GroupedMLPLoRA, LoRALinear, is_adapter_param, strip_peft_name

    out = {}
    for n, m in model.named_modules():
        if isinstance(m, LoRALinear):
            out[f"{n}.weight"] = m.weight.detach()
        elif isinstance(m, GroupedMLPLoRA):
            out[f"{n}.weight1"], out[f"{n}.weight2"] = m.weight1.detach(), m.weight2.detach()
    for n, p in model.named_parameters():
        if not is_adapter_param(n):
            out.setdefault(strip_peft_name(n), p.detach())
    return out


def _w_finetune(rank, world, root, ep, peft, mc):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.engine.peft.lora import is_adapter_param
    from torchturbo_b200.loops import train_step

    def engine():        # one engine per model: an engine's backend keeps the sharding state of the model it built
        return TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "parallel_plan": {"sp_size": 1, "ep_size": ep},
                                                        "activation_checkpointing": {"enabled": False},
                                                        "checkpoint": {"hf_export": "every"}}))

    eng = engine()
    base = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(mc), "seed": 0})
    eng.save_model(base, os.path.join(root, "base", "checkpoint-0"), final=True)
    src = os.path.join(root, "base", "checkpoint-0", "huggingface")
    base_names = _names(src)
    b = PackedCollator()([SyntheticPackedDataset(2, 64, 512, num_docs=3, seed=5)[0]])
    plain = engine().build_model(src)                             # the bf16-rounded base, as the fine-tune will see it
    plain.eval()
    start = _logits(plain, b)
    eng = engine()
    model = eng.build_model(src, peft_config=dict(peft))
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all(is_adapter_param(n) for n in trainable)
    model.eval()
    assert torch.allclose(_logits(model, b), start, atol=1e-5), "adapters start as a no-op on the loaded base weights"
    def whole(p):      # a unit that stays gathered after a forward shows its parameters unsharded: compare whole tensors
        return (p.full_tensor() if hasattr(p, "full_tensor") else p).detach().clone()

    frozen = {n: whole(p) for n, p in model.named_parameters() if not p.requires_grad}
    model.train()
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-2))
    losses = [float(train_step(eng, model, opt, [b])[0]) for _ in range(4)]
    assert losses[-1] < losses[0]
    for n, p in model.named_parameters():
        if n in frozen:
            assert torch.equal(whole(p), frozen[n]), n
    model.eval()
    adapted = _logits(model, b)
    assert (adapted - start).abs().max() > 1e-2
    out = os.path.join(root, "tuned", "checkpoint-4")
    eng.save_model(model, out, final=True)
    hf = os.path.join(out, "huggingface")
    assert _names(hf) == base_names, "the export is a plain checkpoint: base names only, no wrapper or adapter tensors"
    merged = engine().build_model(hf)
    merged.eval()
    want = _effective(model)
    for n, p in merged.named_parameters():
        w = want[n]
        assert (whole(p).float() - whole(w).float()).abs().max() <= 1e-2 * max(float(whole(w).abs().max()), 1e-3), n   # bf16 export
    if "num_experts" not in mc:
        # (with experts a weight rounded to bf16 can flip a token's routing, which moves logits by much more)
        err = (_logits(merged, b) - adapted).abs().max()
        assert err <= 2e-2 * max(1.0, float(adapted.abs().max())), f"merged export differs from the adapted model by {err}"


@pytest.mark.parametrize("peft,mc", [(PEFT, MOE), (dict(PEFT, use_dora=True, target_parameters=[]), DENSE),
                                     (dict(PEFT, target_modules="all-linear", target_parameters=[]), DENSE)],
                         ids=["lora+experts", "dora-dense", "all-linear-dense"])
def test_finetune_from_a_checkpoint_trains_adapters_only_and_exports_merged_weights(tmp_path, peft, mc):
    run_distributed(_w_finetune, 1, str(tmp_path), 1, peft, mc, timeout=600)


def test_expert_parallel_lora_exports_one_merged_checkpoint(tmp_path):
    run_distributed(_w_finetune, 2, str(tmp_path), 2, PEFT, MOE, timeout=600)


def test_fsdp_sharded_dora_exports_one_merged_checkpoint(tmp_path):
    run_distributed(_w_finetune, 2, str(tmp_path), 1, dict(PEFT, use_dora=True, target_parameters=[]), DENSE, timeout=600)


def _w_resume(rank, world, root):
    from torchturbo_b200.data import PackedCollator, SyntheticPackedDataset
    from torchturbo_b200.engine import EngineConfig, TorchTurboEngine
    from torchturbo_b200.engine.optimizers import OptimizerClassPlan
    from torchturbo_b200.loops import train_step

    def engine():
        return TorchTurboEngine(EngineConfig.from_dict({"mixed_precision": "fp32", "parallel_plan": {"sp_size": 1, "ep_size": 2},
                                                        "activation_checkpointing": {"enabled": False},
                                                        "checkpoint": {"hf_export": "every"}}))

    eng = engine()
    base = eng.build_model(None, load_weights=False, init_kwargs={"config": dict(MOE), "seed": 0})
    eng.save_model(base, os.path.join(root, "base", "checkpoint-0"), final=True)
    src = os.path.join(root, "base", "checkpoint-0", "huggingface")
    b = PackedCollator()([SyntheticPackedDataset(2, 64, 512, num_docs=3, seed=5)[0]])
    eng = engine()
    model = eng.build_model(src, peft_config=dict(PEFT))
    opt = eng.prepare_optimizer(model, OptimizerClassPlan(torch.optim.AdamW, lr=1e-2))
    for _ in range(3):
        train_step(eng, model, opt, [b])
    ck = os.path.join(root, "tuned", "checkpoint-3")
    eng.save_model(model, ck, final=False)
    eng.save_optimizer_and_scheduler(model, opt, None, ck)
    model.eval()
    want = _logits(model, b)
    model.train()
    step4 = train_step(eng, model, opt, [b])
    eng2 = engine()
    again = eng2.build_model(src, peft_config=dict(PEFT))
    opt2 = eng2.prepare_optimizer(again, OptimizerClassPlan(torch.optim.AdamW, lr=1e-2))
    eng2.load_from_checkpoint(again, ck)
    eng2.load_optimizer_and_scheduler(again, opt2, None, ck)
    again.eval()
    assert torch.equal(_logits(again, b), want), "adapters and wrapped base weights come back from the sharded checkpoint"
    again.train()
    step4b = train_step(eng2, again, opt2, [b])
    assert float(step4[0]) == float(step4b[0]) and abs(float(step4[1]) - float(step4b[1])) < 1e-6     # AdamW moments too


def test_adapter_training_resumes_exactly_from_a_sharded_checkpoint(tmp_path):
    run_distributed(_w_resume, 2, str(tmp_path), timeout=600)
