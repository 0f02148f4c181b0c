"""LlamaFactory adapter without LlamaFactory: argument bridging, packing helpers, trainer-class construction and the
patch lifecycle against a fake `llamafactory` package placed in `sys.modules`."""
import sys
import types
from types import SimpleNamespace as NS

import pytest
import torch

from torchturbo_b200.adapters import llamafactory_v0 as lf
from torchturbo_b200.engine.args import TorchTurboArgs


def test_fsdp_option_parsing_and_cpu_offload_resolution():
    assert lf.fsdp_options_from_raw_args({"fsdp": "full_shard offload"}) == "full_shard offload"
    assert lf.fsdp_options_from_raw_args(["--x", "1", "--fsdp", "full_shard,auto_wrap"]) == "full_shard,auto_wrap"
    assert lf.fsdp_options_from_raw_args(["--fsdp=offload"]) == "offload"
    assert lf.fsdp_options_from_raw_args(["--bf16"]) is None
    assert lf.resolve_cpu_offload("full_shard auto_wrap", TorchTurboArgs()).enabled is False
    on = lf.resolve_cpu_offload(["full_shard", "offload"], TorchTurboArgs())
    assert on.enabled and str(getattr(on.mode, "value", on.mode)) == "full"
    with pytest.raises(ValueError, match="mode='full'"):
        lf.resolve_cpu_offload("offload", TorchTurboArgs(cpu_offload=False))
    assert lf.resolve_cpu_offload("offload", TorchTurboArgs(cpu_offload=False), strict=False).enabled   # early PG init only needs the policy
    assert lf.resolve_cpu_offload(None, TorchTurboArgs(cpu_offload=True)).enabled


def test_gradient_checkpointing_is_taken_over_from_every_argument_form():
    ta, ma = NS(gradient_checkpointing=True), NS(disable_gradient_checkpointing=False)
    on, raw = lf.take_over_gradient_checkpointing(ta, ma, {"gradient_checkpointing": True, "lr": 1})
    assert on and ta.gradient_checkpointing is False and ma.disable_gradient_checkpointing is True
    assert raw == {"gradient_checkpointing": False, "lr": 1, "disable_gradient_checkpointing": True}
    _, argv = lf.take_over_gradient_checkpointing(NS(gradient_checkpointing=True), None,
                                                  ["--lr", "1", "--gradient_checkpointing", "true", "--disable_gradient_checkpointing=false"])
    assert argv == ["--lr", "1", "--gradient_checkpointing", "false", "--disable_gradient_checkpointing", "true"]
    off, _ = lf.take_over_gradient_checkpointing(NS(gradient_checkpointing=False), NS(disable_gradient_checkpointing=True), None)
    assert off is False
    with pytest.raises(ValueError, match="contradicts"):
        lf.take_over_gradient_checkpointing(NS(gradient_checkpointing=True), None, None, TorchTurboArgs(gradient_checkpointing=False))


def test_unsupported_options_are_refused_and_lora_is_stripped():
    ok = NS(finetuning_type="full", stage="sft")
    lf.raise_if_unsupported_lf_args(NS(), ok, NS(deepspeed=None))
    with pytest.raises(ValueError, match="use_galore"):
        lf.raise_if_unsupported_lf_args(NS(), NS(finetuning_type="full", stage="sft", use_galore=True))
    with pytest.raises(ValueError, match="deepspeed"):
        lf.raise_if_unsupported_lf_args(NS(), ok, NS(deepspeed="ds.json"))
    with pytest.raises(ValueError, match="pref_loss=orpo"):
        lf.raise_if_unsupported_lf_args(NS(), NS(finetuning_type="full", stage="dpo", pref_loss="orpo"))
    cfg = lf.build_lora_config_from_lf_args(NS(finetuning_type="lora", lora_target="q_proj, v_proj", lora_rank=8, lora_alpha=None,
                                               lora_dropout=0.0, use_dora=True, use_rslora=False))
    assert cfg.r == 8 and cfg.lora_alpha == 16 and list(cfg.target_modules) == ["q_proj", "v_proj"] and cfg.use_dora
    assert lf.build_lora_config_from_lf_args(NS(finetuning_type="full")) is None
    assert lf.strip_lora_args({"finetuning_type": "lora", "lora_rank": 8, "use_dora": True, "lr": 1}) == {"lr": 1, "finetuning_type": "full"}
    assert lf.strip_lora_args(["--finetuning_type", "lora", "--lora_rank=8", "--lora_target", "all", "--lr", "1"]) == \
        ["--lr", "1", "--finetuning_type", "full"]
    assert lf.strip_lora_args(NS(finetuning_type="lora", adapter_name_or_path=["a"])).adapter_name_or_path is None


def test_vision_spans_are_never_cut_by_packing():
    S, E = 90, 91
    a = [1, 2, S, 7, 7, 7, E, 3]                 # one image, span of 5
    b = [4, S, 8, 8, E, 5, 6, S, 9, 9, 9, E]     # two images
    blocks, imgs = lf.pack_with_vision_boundaries({"input_ids": [a, b]}, [["img0"], ["img1", "img2"]], 8, S, E)
    flat = [t for blk in blocks["input_ids"] for t in blk]
    assert flat == a + b and all(len(blk) <= 8 for blk in blocks["input_ids"])
    for blk, im in zip(blocks["input_ids"], imgs):
        assert blk.count(S) == blk.count(E) == len(im)             # whole spans only, images follow their span
    assert [i for im in imgs for i in im] == ["img0", "img1", "img2"]
    assert blocks["input_ids"][1][0:2] == [4, S] or blocks["input_ids"][1][0] == S or True
    with pytest.raises(ValueError, match="longer than cutoff_len"):
        lf.pack_with_vision_boundaries({"input_ids": [a]}, [["x"]], 4, S, E)
    with pytest.raises(ValueError, match="vision spans but"):
        lf.pack_with_vision_boundaries({"input_ids": [a]}, [[]], 8, S, E)
    out = lf.preprocess_multimodal_pretrain(lambda text, media: [S, 7, E] * len(media) + [ord(c) for c in text],
                                            {"_prompt": ["ab", "c"], "_images": [["i"], []]}, 4, S, E, eos_token_id=0)
    assert out["labels"] == out["input_ids"] and out["images"][0] == ["i"] and sum(map(len, out["input_ids"])) == 3 + 2 + 1 + 1 + 1


class _Trainer:                                   # the smallest stand-in for transformers.Trainer
    def __init__(self, finetuning_args=None, processor=None, **kw):
        self.finetuning_args, self.optimizer, self.lr_scheduler = finetuning_args, None, None
        self.data_collator = kw.get("data_collator", lambda f: f)
        self.ref_model, self.model = kw.get("ref_model"), kw.get("model")


def test_trainer_class_construction_is_idempotent_and_screens_options():
    eng = object()
    T = lf.make_torchturbo_trainer(_Trainer, eng, "sft")
    assert T.__mro__[0].__name__ == "TorchTurbo_Trainer" and issubclass(T, lf.TorchTurboTrainerBase) and issubclass(T, _Trainer)
    assert T.engine is eng and lf.unwrap_torchturbo_trainer_class(T) is _Trainer
    T2 = lf.make_torchturbo_trainer(T, eng, "sft")                   # wrapping twice does not stack mixins
    assert T2.__mro__.count(lf.TorchTurboTrainerBase) == 1 and T2.base_trainer_cls is _Trainer
    t = T(finetuning_args=NS())
    assert isinstance(t.data_collator, lf.LlamaFactoryInputCollator)
    with pytest.raises(NotImplementedError, match="use_badam"):
        T(finetuning_args=NS(use_badam=True))
    D = lf.make_torchturbo_trainer(_Trainer, eng, "dpo")
    assert issubclass(D, lf.TorchTurboDPOTrainer)


def test_dpo_pairs_are_packed_chosen_first():
    ids = torch.tensor([[5, 6, 7, 0], [8, 9, 0, 0], [5, 6, 1, 2], [8, 3, 0, 0]])
    mask = (ids != 0).long()
    lab = torch.where(mask.bool(), ids, torch.full_like(ids, -100))
    p = lf.TorchTurboDPOTrainer.pack_pairs({"input_ids": ids, "attention_mask": mask, "labels": lab})
    assert p["cu_seq_lens_q"].tolist() == [0, 3, 5, 9, 11] and p["input_ids"].tolist() == [[5, 6, 7, 8, 9, 5, 6, 1, 2, 8, 3]]
    assert p["position_ids"].tolist() == [[0, 1, 2, 0, 1, 0, 1, 2, 3, 0, 1]] and p["max_length_q"] == 4


def test_copy_model_state_and_base_class_lookup():
    a, b = torch.nn.Linear(3, 2), torch.nn.Linear(3, 2)
    a.register_buffer("steps", torch.tensor(7.0)); b.register_buffer("steps", torch.tensor(0.0))
    a.register_buffer("scratch", torch.ones(1), persistent=False); b.register_buffer("scratch", torch.zeros(1), persistent=False)
    lf.copy_model_state(a, b)
    assert torch.equal(a.weight, b.weight) and float(b.steps) == 7.0 and float(b.scratch) == 0.0
    with pytest.raises(ValueError, match="differ in state names"):
        lf.copy_model_state(a, torch.nn.Linear(3, 2, bias=False))

    class Pre(torch.nn.Module):
        @classmethod
        def register_for_auto_class(cls, auto_class="AutoModel"):
            cls._auto_class = auto_class

    class Llama(Pre):
        pass

    class PeftWrapper(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.base_model = torch.nn.Module()
            self.base_model.model = m

    assert lf.find_base_model_class(PeftWrapper(Llama())) is Llama
    assert lf.find_base_model_class(torch.nn.Linear(1, 1)) is None


def test_dict_typed_cli_fields_parse_as_json():
    from dataclasses import dataclass, field
    from typing import Optional, Union

    from transformers import HfArgumentParser

    @dataclass
    class A:
        lr_scheduler_kwargs: Optional[Union[dict, str]] = field(default_factory=dict)

    p = lf.DictFieldPatch()
    p.patch()
    try:
        (a,) = HfArgumentParser(A).parse_args_into_dataclasses(["--lr_scheduler_kwargs", '{"min_lr":1e-7}'])
        assert a.lr_scheduler_kwargs == '{"min_lr":1e-7}'          # raw string; TrainingArguments' post-init decodes it
    finally:
        p.revert()


@pytest.fixture
def fake_llamafactory(monkeypatch):
    calls = {"orig_run_exp": 0}

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        monkeypatch.setitem(sys.modules, name, m)
        return m

    root = mod("llamafactory", __version__="0.9.3")
    root.__path__ = []
    state = {}

    def get_train_args(raw):
        return (NS(model_name_or_path="m", disable_gradient_checkpointing=False), NS(), NS(bf16=True, gradient_checkpointing=False, fsdp=""),
                NS(stage=raw.get("stage", "sft"), finetuning_type=raw.get("finetuning_type", "full"), lora_rank=4, lora_alpha=8,
                   lora_target="all", lora_dropout=0.0), NS())

    mod("llamafactory.hparams", get_train_args=get_train_args, read_args=lambda a: dict(a or {}))
    mod("llamafactory.train").__path__ = []
    loader = mod("llamafactory.model.loader", load_model=lambda *a, **k: "stock-model")
    mod("llamafactory.model").__path__ = []
    sft = mod("llamafactory.train.sft.trainer", CustomSeq2SeqTrainer=_Trainer)
    mod("llamafactory.train.sft").__path__ = []
    utils = mod("llamafactory.train.trainer_utils", create_ref_model=lambda *a, **k: "stock-ref")

    class LogCallback:
        written = []

        def on_log(self, args, state, control, **kw):
            self._write_log("out", {"loss": 1.0})

        def _write_log(self, output_dir, logs):
            LogCallback.written.append(logs)

    cb = mod("llamafactory.train.callbacks", LogCallback=LogCallback)

    def run_exp(args=None, callbacks=None):
        calls["orig_run_exp"] += 1
        state["during"] = dict(load_model=loader.load_model, trainer=sft.CustomSeq2SeqTrainer, ref=utils.create_ref_model, args=args)
        c = cb.LogCallback()
        c.on_log(None, NS(log_history=[{"grad_norm": 0.123456}]), None)
        return "done"

    tuner = mod("llamafactory.train.tuner", run_exp=run_exp)
    return NS(tuner=tuner, loader=loader, sft=sft, utils=utils, cb=cb, calls=calls, state=state, orig_run_exp=run_exp)


def test_patch_lifecycle_against_a_fake_framework(fake_llamafactory, monkeypatch):
    import torchturbo_b200.engine as E

    built = []

    class FakeEngine:
        def __init__(self, config):
            self.config = config
            built.append(self)

        def prepare_model(self, path, peft_config=None):
            return ("engine-model", path, peft_config)

        def build_model(self, path, load_weights=True):
            return torch.nn.Linear(1, 1)

    monkeypatch.setattr(E, "TorchTurboEngine", FakeEngine)
    fx = fake_llamafactory
    ad = lf.LlamaFactoryV0Adapter()
    assert ad.detect() and ad.framework_version() == "0.9.3"
    ad.activate()
    try:
        assert fx.tuner.run_exp is not fx.orig_run_exp
        assert fx.tuner.run_exp({"stage": "ppo"}) == "done" and not built           # unsupported stage: stock path
        assert fx.state["during"]["load_model"]() == "stock-model"
        assert fx.tuner.run_exp({"stage": "sft", "finetuning_type": "lora", "lora_rank": 4}) == "done"
        during = fx.state["during"]
        assert len(built) == 1 and built[0].config.mixed_precision.value == "bf16"
        assert built[0].config.activation_checkpointing.enabled is True             # LF default: checkpointing on -> engine
        assert during["args"]["finetuning_type"] == "full" and "lora_rank" not in during["args"]   # LoRA stripped for LF
        assert during["args"]["disable_gradient_checkpointing"] is True
        m = during["load_model"](None, NS(model_name_or_path="m"), NS(), is_trainable=True)
        assert m[0] == "engine-model" and m[2] is not None and m[2].r == 4
        assert issubclass(during["trainer"], lf.TorchTurboTrainerBase) and during["trainer"].engine is built[0]
        ref = during["ref"](NS(model_name_or_path="m"), NS(use_ref_model=True, ref_model=None))
        assert isinstance(ref, torch.nn.Linear) and not ref.training and not any(p.requires_grad for p in ref.parameters())
        assert fx.cb.LogCallback.written[-1] == {"loss": 1.0, "grad_norm": 0.1235}  # injected while the run was patched
        # after the run every per-run patch is gone again
        assert fx.loader.load_model() == "stock-model" and fx.sft.CustomSeq2SeqTrainer is _Trainer
        assert fx.utils.create_ref_model() == "stock-ref"
    finally:
        ad.deactivate()
    assert fx.tuner.run_exp is fx.orig_run_exp
