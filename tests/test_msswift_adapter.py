"""ms-swift adapter without ms-swift: data validation, stage table, session slot, plugin bridge, and pipeline / loader /
trainer construction against a fake `swift` package in `sys.modules`."""
import sys
import types
from types import SimpleNamespace as NS

import pytest
import torch

from torchturbo_b200.adapters import msswift as sw
from torchturbo_b200.adapters.msswift import session


def test_raw_dataset_rows_are_audited_before_tokenisation():
    from torchturbo_b200.adapters.msswift.data_check import audit_rows, classify_row

    assert sw.check_row({"messages": "hello"}) is None
    assert sw.check_row({"messages": "<image> a <image>", "images": ["a.png", {"path": "b.png"}]}) is None
    assert classify_row({"messages": "<image>", "images": "a.png,b.png"})[0] == "joined_paths"
    assert classify_row({"messages": "<image>", "images": ["a.png,b.png"]})[0] == "joined_paths"
    assert classify_row({"messages": "<image>", "images": "a.png"})[0] == "not_a_list"
    assert classify_row({"messages": "<image>", "images": [{"bytes": b"x"}]})[0] == "empty_reference"
    assert classify_row({"messages": "<image>", "images": ["a", "b"]}) == ("placeholder_mismatch", "1 placeholder(s), 2 image(s)")
    assert "different number" in sw.check_row({"messages": "<image>", "images": ["a", "b"]})

    class DS(list):
        column_names = ["messages", "images"]

    good = {"messages": "<image>", "images": ["a"]}
    sw.validate_raw_dataset(DS([good]))
    # every broken rule is reported with its count, not just the first offender
    rows = DS([good, {"messages": "x", "images": ["a"]}, {"messages": "<image>", "images": "p,q"}, {"messages": "y", "images": ["b"]}])
    rep = audit_rows(rows)
    assert rep.rows == 4 and rep.by_rule["placeholder_mismatch"] == [1, 3] and rep.by_rule["joined_paths"] == [2]
    with pytest.raises(ValueError, match=r"3 of 4 multimodal rows(.|\n)*2 row\(s\)(.|\n)*#1 (.|\n)*1 row\(s\)"):
        sw.validate_raw_dataset(rows, "train")
    sw.validate_raw_dataset(iter([{"images": "bad,bad"}]))        # streaming datasets are not walked
    text_only = DS([{"messages": "x"}])
    text_only.column_names = ["messages"]
    sw.validate_raw_dataset(text_only)


def test_stage_table_and_session_slot():
    names = [s.name for s in sw.iter_stages()]
    assert names == ["sft", "pt", "dpo"] and sw.get_stage("dpo").pipeline_attr == "SwiftRLHF"
    sw.register_stage(sw.SwiftStageSpec("sft", "x", "y", "z", "causal_lm"))          # idempotent on the name
    assert len(sw.iter_stages()) == 3
    session.clear()
    with pytest.raises(RuntimeError, match="no active engine"):
        session.get_engine()
    session.set_engine("E", stage="pt")
    assert session.get_engine() == "E" and session.get_stage() == "pt" and session.get_loading_role() is None
    with session.loading_role("reference"):
        assert session.get_loading_role() == "reference"
        with session.loading_role(None):
            assert session.get_loading_role() is None
        assert session.get_loading_role() == "reference"
    assert session.get_loading_role() is None
    session.clear()


def test_unsupported_swift_options_and_lora_config():
    with pytest.raises(NotImplementedError, match="tuner_type='adalora'"):
        sw.raise_if_unsupported(NS(tuner_type="adalora"))
    with pytest.raises(NotImplementedError, match="DPO with tuner_type"):
        sw.raise_if_unsupported(NS(tuner_type="lora", rlhf_type="dpo"))
    with pytest.raises(NotImplementedError, match="rlhf_type='kto'"):
        sw.raise_if_unsupported(NS(rlhf_type="kto"))
    cfg = sw.build_lora_config_from_swift_args(NS(tuner_type="lora", lora_rank=16, lora_alpha=None, target_modules=["ALL-LINEAR"]))
    assert cfg.r == 16 and cfg.lora_alpha == 32 and list(cfg.target_modules) == ["all-linear"]
    assert sw.build_lora_config_from_swift_args(NS(tuner_type="full")) is None
    a = NS(gradient_checkpointing=True, sequence_parallel_size=2, training_args=NS(gradient_checkpointing=True, deepspeed="z"))
    asked = sw.take_over_swift_switches(a)
    assert asked["sequence_parallel_size"] == 2 and a.sequence_parallel_size == 1 and a.training_args.deepspeed is None


def test_dataset_plugin_bridge_routes_and_refuses_mixtures():
    from torchturbo_b200.engine.plugins import DatasetPlugin

    class P(DatasetPlugin):
        dataset_names = ["mine_a", "mine_b"]

        def load(self, name, ctx):
            return [{"t": f"{name}{i}"} for i in range(2)]

        def encode(self, row, ctx):
            return {"input_ids": [len(row["t"])], "max_length": ctx["max_length"]}

        def collate(self, rows):
            return {"n": len(rows)}

    b = sw.DatasetPluginBridge()
    p = P()
    b.add(p)
    assert b.resolve(NS(dataset=["other"])) is None and b.collator_for(NS(dataset=["other"])) is None
    args = NS(dataset=["mine_a#100", "mine_b"], max_length=77, seed=1)
    train, val = b.try_takeover(args=args, template=None)
    assert len(train) == 4 and train[3] == {"input_ids": [7], "max_length": 77} and val is None
    assert b.collator_for(args)([1, 2]) == {"n": 2}
    with pytest.raises(ValueError, match="mix plugin-provided and native"):
        b.resolve(NS(dataset=["mine_a", "alpaca"]))


@pytest.fixture
def fake_swift(monkeypatch):
    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        if "." not in name or name.count(".") < 3:
            m.__path__ = []
        monkeypatch.setitem(sys.modules, name, m)
        return m

    log = []

    class SwiftPipeline:
        def __init__(self, args=None):
            self.args = args
            log.append("parse")

    class SwiftSft(SwiftPipeline):
        def __init__(self, args=None):
            raise AssertionError("the native constructor would load the model before the engine exists")

        def _prepare_model_tokenizer(self):
            log.append("model")
            self.model = session.get_engine().prepare_model("dir")

        def _prepare_template(self):
            log.append("template")
            self.template = "tpl"

        def _prepare_dataset(self):
            return ["native-train", None]

        def _get_trainer_kwargs(self):
            return {"x": 1}

    class SwiftRLHF(SwiftSft):
        def _prepare_single_model(self, key, origin_key, model_type, model_revision):
            return session.get_loading_role()

    class ModelLoader:
        def __init__(self, *a, **k):
            pass

        def get_processor(self):
            return "native-processor"

        def _postprocess_model(self, model_dir, model):
            self.post = model

    class Seq2SeqTrainer:
        def __init__(self, *a, **k):
            self.args = k.get("args")
            self.kw = k
            self.accelerator = NS(_models=[], state=NS(fsdp_plugin=None))
            self.model = k.get("model")

        def _get_data_collator(self, args, template):
            return lambda rows: rows

        def save_model(self, output_dir=None, _internal_call=False):
            self.saved_aux = output_dir

    registered = {}
    mod("swift", __version__="4.0.1")
    mod("swift.pipelines")
    mod("swift.pipelines.base", SwiftPipeline=SwiftPipeline)
    mod("swift.pipelines.train")
    sft = mod("swift.pipelines.train.sft", SwiftSft=SwiftSft, sft_main=lambda a=None: sys.modules["swift.pipelines.train.sft"].SwiftSft(a))
    rl = mod("swift.pipelines.train.rlhf", SwiftRLHF=SwiftRLHF)
    mod("swift.model", Model=lambda *a, **k: NS(), ModelGroup=lambda models, template=None: NS(models=models, template=template),
        ModelMeta=lambda **k: NS(**k), register_model=lambda meta, exist_ok=False: registered.__setitem__(meta.model_type, meta),
        ModelLoader=ModelLoader)

    class NativeQwenLoader(ModelLoader):
        def get_processor(self):
            return "qwen-processor"

    mod("swift.model.model_meta", MODEL_MAPPING={"qwen3": NS(loader=NativeQwenLoader, template="qwen3", requires=[], tags=[], task_type="causal_lm")})
    mod("swift.trainers", TrainerFactory=NS(TRAINER_MAPPING={}), Seq2SeqTrainer=Seq2SeqTrainer)
    return NS(sft=sft, rl=rl, log=log, SwiftSft=SwiftSft, registered=registered, NativeQwenLoader=NativeQwenLoader, Seq2SeqTrainer=Seq2SeqTrainer)


def test_pipeline_loader_and_trainer_against_a_fake_swift(fake_swift, monkeypatch):
    import torchturbo_b200.engine as E
    from torchturbo_b200.adapters.msswift import loader as L
    from torchturbo_b200.adapters.msswift import pipeline as PL
    from torchturbo_b200.adapters.msswift import trainer as TR
    from torchturbo_b200.engine.plugins import PluginManager

    calls = []

    class FakeEngine:
        def __init__(self, config):
            self.config, self.plugins, self.peft_config = config, PluginManager([]), None

        def prepare_model(self, path, peft_config=None, init_kwargs=None):
            calls.append(("prepare", path, peft_config))
            return torch.nn.Linear(2, 2)

        def build_model(self, path, init_kwargs=None):
            calls.append(("build", path))
            return torch.nn.Linear(2, 2)

        def resolve_gradient_accumulation_steps(self, ga):
            return ga * 2

        def clip_grad_norm_(self, model, max_norm, optimizer=None):
            return ("clipped", max_norm)

        def save_model(self, model, out, final=False):
            calls.append(("save", out, final))

    monkeypatch.setattr(E, "TorchTurboEngine", FakeEngine)
    PL._CACHE.clear(); L._CACHE.clear(); TR._CLASSES.clear()
    fx = fake_swift
    ad = sw.MSSwiftAdapter()
    assert ad.detect() and ad.framework_version() == "4.0.1"
    ad.activate()
    try:
        Pipe = sys.modules["swift.pipelines.train.sft"].SwiftSft
        assert Pipe is not fx.SwiftSft and issubclass(Pipe, fx.SwiftSft) and Pipe.turbo_stage == "sft"
        args = NS(bf16=True, gradient_checkpointing=True, sequence_parallel_size=1, tuner_type="lora", lora_rank=4, model_type="qwen3",
                  dataset=["alpaca"])
        pipe = fx.sft.sft_main(args)                     # swift's own entry point now builds the engine-backed pipeline
        assert fx.log == ["parse", "model", "template"]  # engine first, then swift's usual preparation
        assert isinstance(ad.engine, FakeEngine) and ad.engine.peft_config.r == 4 and args.gradient_checkpointing is False
        assert args.model_type == "turbo_qwen3" and "turbo_qwen3" in fx.registered and "turbo_qwen3_moe" in fx.registered
        assert sys.modules["swift.trainers"].TrainerFactory.TRAINER_MAPPING["dpo"].endswith("trainer_factory.EngineDPOTrainer")
        assert pipe.prepare_model(model="m") == "m" and pipe._prepare_dataset() == ["native-train", None]
        assert pipe._get_trainer_kwargs() == {"x": 1, "plugin_collator": None}
        # loader: engine get_model in front of the model's native loader, whose processor path stays intact
        loader_cls = fx.registered["turbo_qwen3"].loader
        assert issubclass(loader_cls, fx.NativeQwenLoader) and loader_cls.__mro__[1] is L.EngineModelMixin or loader_cls.__mro__[0].__name__.startswith("EngineModelLoader")
        ld = loader_cls()
        assert ld.get_processor() == "qwen-processor"
        m = ld.get_model("dir", {"c": 1}, None, {})
        assert calls[-1][0] == "prepare" and calls[-1][2] is ad.engine.peft_config and any(p.requires_grad for p in m.parameters())
        with session.loading_role("reference"):
            ref = ld.get_model("ref-dir", {"c": 1}, None, {})
        assert calls[-1] == ("build", "ref-dir") and not ref.training and not any(p.requires_grad for p in ref.parameters())
        assert getattr(L, loader_cls.__name__) is loader_cls            # importable by name for pickling by reference
        # DPO pipeline marks the reference load
        RL = sys.modules["swift.pipelines.train.rlhf"].SwiftRLHF
        rl = RL.__new__(RL)
        assert rl._prepare_single_model("ref_model", "ref", None, None) == "reference"
        assert rl._prepare_single_model("model", None, None, None) is None
        # trainer: built lazily under a module-level name, GA resolved at construction, accelerate reduced to pass-through
        from torchturbo_b200.adapters.msswift import trainer_factory

        T = trainer_factory.EngineSeq2SeqTrainer
        assert issubclass(T, fx.Seq2SeqTrainer) and T.__mro__[1] is TR.EngineTrainerMixin and trainer_factory.EngineSeq2SeqTrainer is T
        t = T(args=NS(gradient_accumulation_steps=3, output_dir="/tmp/x", save_only_model=False), model=m, plugin_collator=None)
        assert t.args.gradient_accumulation_steps == 6 and "plugin_collator" not in t.kw
        assert t.accelerator.clip_grad_norm_(None, 1.5) == ("clipped", 1.5) and t.accelerator.prepare_model(m) is m
        assert isinstance(t._get_data_collator(None, "tpl"), sw.SwiftInputCollator)
        t.state, t.control = NS(global_step=5, max_steps=10), NS(should_training_stop=False)
        t.save_model("/tmp/tt_swift_ck", _internal_call=True)
        assert calls[-1] == ("save", "/tmp/tt_swift_ck", False) and t.saved_aux == "/tmp/tt_swift_ck"
        t.state.global_step = 10
        t.save_model("/tmp/tt_swift_ck", _internal_call=True)
        assert calls[-1] == ("save", "/tmp/tt_swift_ck", True)
    finally:
        ad.deactivate()
    assert sys.modules["swift.pipelines.train.sft"].SwiftSft is fx.SwiftSft and session.get_engine_or_none() is None
