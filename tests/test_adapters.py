"""Adapter-side batch normalisation (ms-swift bridging, HF-trainer features) and config construction from host
framework arguments."""
from types import SimpleNamespace

import pytest
import torch

from torchturbo_b200.adapters.hf_trainer import normalize_training_features
from torchturbo_b200.adapters.msswift import (SwiftInputCollator, bake_loss_scale_into_labels, bridge_packed_inputs,
                                              bridge_unpacked_inputs, build_config_from_swift_args)


def test_bridge_packed_left_padding_and_labels():
    # two samples of 3 and 2 tokens, 3 alignment pads on the left
    ids = torch.tensor([[0, 0, 0, 11, 12, 13, 21, 22]])
    lab = ids.clone()
    pos = torch.tensor([[0, 0, 0, 0, 1, 2, 0, 1]])
    out = bridge_packed_inputs({"input_ids": ids, "labels": lab, "position_ids": pos, "attention_mask": torch.ones(1, 8)},
                               sequence_lengths=[3, 2], padding_side="left")
    assert out["input_ids"][0].tolist() == [11, 12, 13, 21, 22, 0, 0, 0]
    assert out["cu_seq_lens_q"].tolist() == [0, 3, 5] and out["max_length_q"] == 3 and "attention_mask" not in out
    assert out["labels"][0].tolist()[:5] == [-100, 12, 13, -100, 22]
    assert out["position_ids"][0].tolist()[:5] == [0, 1, 2, 0, 1]
    with pytest.raises(ValueError):
        bridge_packed_inputs({"input_ids": ids}, sequence_lengths=[9], padding_side="right")
    with pytest.raises(ValueError):
        bridge_packed_inputs({"input_ids": torch.tensor([[1, 2, 3]]), "cu_seq_lens_q": torch.tensor([0, 1, 3], dtype=torch.int32)},
                             sequence_lengths=[2, 1])


def test_bridge_unpacked_rows_become_sequences():
    ids = torch.tensor([[1, 2, 3, 0], [4, 5, 0, 0]])
    mask = torch.tensor([[1, 1, 1, 0], [1, 1, 0, 0]])
    out = bridge_unpacked_inputs({"input_ids": ids, "labels": ids.clone(), "attention_mask": mask})
    assert out["input_ids"].tolist() == [[1, 2, 3, 4, 5]] and out["cu_seq_lens_k"].tolist() == [0, 3, 5]
    assert out["position_ids"].tolist() == [[0, 1, 2, 0, 1]] and out["labels"].tolist() == [[-100, 2, 3, -100, 5]]
    pos3 = torch.arange(8).view(1, 2, 4).expand(3, 2, 4)
    out = bridge_unpacked_inputs({"input_ids": ids, "attention_mask": mask, "position_ids": pos3,
                                  "text_position_ids": torch.zeros(2, 4, dtype=torch.long)})
    assert out["position_ids"].shape == (3, 1, 5) and out["position_ids"][0, 0].tolist() == [0, 1, 2, 4, 5]
    assert out["text_position_ids"].tolist() == [[0, 1, 2, 0, 1]]


def test_loss_scale_is_folded_into_labels():
    out = bake_loss_scale_into_labels({"labels": torch.tensor([[5, 6, 7]]), "loss_scale": torch.tensor([[1.0, 0.0, 1.0]])})
    assert out["labels"].tolist() == [[5, -100, 7]] and "loss_scale" not in out
    same = {"labels": torch.tensor([[5, 6]])}
    assert bake_loss_scale_into_labels(same) is same


def test_swift_collator_dpo_orders_chosen_then_rejected():
    template = SimpleNamespace(mode="rlhf", padding_free=True, is_training=True, padding_side="right")

    def inner(batch):
        rows = [s["chosen_input_ids"] for s in batch] + [s["rejected_input_ids"] for s in batch]
        flat = [t for r in rows for t in r]
        return {"input_ids": torch.tensor([flat]), "labels": torch.tensor([flat])}

    batch = [{"chosen_input_ids": [1, 2, 3], "rejected_input_ids": [1, 9]}, {"chosen_input_ids": [4, 5], "rejected_input_ids": [4, 8, 7]}]
    out = SwiftInputCollator(inner, template)(batch)
    assert out["cu_seq_lens_q"].tolist() == [0, 3, 5, 7, 10] and out["max_length_q"] == 3


def test_hf_features_neat_packing_and_padding():
    f = normalize_training_features({"input_ids": torch.tensor([[1, 2, 3, 4, 5, 0]]), "labels": torch.tensor([[1, 2, 3, 4, 5, 0]]),
                                     "attention_mask": torch.tensor([[1, 1, 2, 2, 2, 0]])})
    assert f["cu_seq_lens_q"].tolist() == [0, 2, 5] and f["labels"][0].tolist() == [-100, 2, -100, 4, 5, -100]
    f = normalize_training_features({"input_ids": torch.tensor([[1, 2, 0], [3, 4, 5]]), "labels": torch.tensor([[1, 2, 0], [3, 4, 5]]),
                                     "attention_mask": torch.tensor([[1, 1, 0], [1, 1, 1]])})
    assert f["input_ids"].tolist() == [[1, 2, 3, 4, 5]] and f["cu_seq_lens_q"].tolist() == [0, 2, 5]


def test_swift_args_force_engine_ownership():
    from torchturbo_b200.engine.args import parse_torchturbo_args

    args = SimpleNamespace(bf16=True, gradient_checkpointing=True, sequence_parallel_size=4, deepspeed="zero3", fsdp="full_shard",
                           router_aux_loss_coef=0.01)
    tt, _ = parse_torchturbo_args(["--tt_sp_size", "2"])
    cfg = build_config_from_swift_args(args, "dpo", tt)
    assert args.gradient_checkpointing is False and args.sequence_parallel_size == 1 and args.deepspeed is None and args.fsdp == ""
    assert cfg.parallel_plan.sp_size == 2 and cfg.moe.aux_loss_coeff == pytest.approx(0.01)
    assert cfg.activation_checkpointing.enabled is True


def test_chat_formats_render_and_register_with_a_fake_llamafactory(monkeypatch):
    import sys
    import types

    from torchturbo_b200.adapters import chat_templates as C

    conv = [{"role": "system", "content": "S"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"},
            {"role": "observation", "content": "42"}]
    assert C.render(C.FORMATS["bailing_v3"], conv) == (
        "<role>SYSTEM</role>\nS<|role_end|>\n\n<role>HUMAN</role>\nhi<|role_end|>\n\n<role>ASSISTANT</role>yo<|role_end|>\n\n"
        "<role>OBSERVATION</role>\n\n```result\n42\n```\n<|role_end|>\n\n<role>ASSISTANT</role>")
    assert C.render(C.FORMATS["deepseek_v4"], conv[1:3], bos="<B>") == "<B><｜User｜>hi<｜Assistant｜>yo<｜end▁of▁sentence｜>"
    assert C.render(C.FORMATS["kimi_k25"], conv[1:2]).startswith("<|im_system|>system<|im_middle|>You are a helpful assistant<|im_end|>")
    assert C.render(C.FORMATS["glm5"], conv[1:3]) == "[gMASK]<sop><|user|>\nhi<|assistant|>\nyo"
    with pytest.raises(ValueError, match="no tool-result turn"):
        C.render(C.FORMATS["qwen3_5_nothink"], conv)
    assert set(C.MODEL_FORMATS.values()) <= set(C.FORMATS)
    assert '"name": "f"' in C.ling_v3_tool_text([{"name": "f", "parameters": {}}]) and "<tools>" in C.ling_v3_tool_text([])

    registered = {}

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        m.__path__ = []
        monkeypatch.setitem(sys.modules, name, m)
        return m

    class Fmt:
        def __init__(self, slots=None, tool_format=None):
            self.slots, self.tool_format = slots, tool_format

    mod("llamafactory")
    mod("llamafactory.data")
    mod("llamafactory.data.formatter", EmptyFormatter=Fmt, FunctionFormatter=Fmt, StringFormatter=Fmt, ToolFormatter=Fmt)
    mod("llamafactory.data.tool_utils", TOOLS={"qwen": object(), "glm4_moe": object()}, QwenToolUtils=object)
    plugins = {}
    mod("llamafactory.data.mm_plugin", get_mm_plugin=lambda name, **kw: (name, kw), PLUGINS=plugins,
        BasePlugin=type("BasePlugin", (), {}), register_mm_plugin=plugins.__setitem__)
    mod("llamafactory.data.template", TEMPLATES=registered, ReasoningTemplate=type("ReasoningTemplate", (), {}),
        register_template=lambda **kw: registered.__setitem__(kw["name"], kw))
    done = C.register_lf_templates()
    assert set(done) == set(C.FORMATS) and C.register_lf_templates() == []            # idempotent
    b = registered["bailing_v3"]
    assert b["format_user"].slots == ["<role>HUMAN</role>\n{{content}}<|role_end|>\n\n<role>ASSISTANT</role>"] and b["efficient_eos"]
    assert b["format_tools"].tool_format == "ling_v3" and "ling_v3" in sys.modules["llamafactory.data.tool_utils"].TOOLS
    d = registered["deepseek_v4_thinking"]
    assert d["format_prefix"].slots == [{"bos_token"}] and d["template_class"].__name__ == "ReasoningTemplate"
    assert "format_tools" not in d                                                    # its tool format is not known to this LF
    assert registered["qwen3_5"]["mm_plugin"][0] == "qwen3_vl" and registered["kimi_k25"]["default_system"]
    assert set(plugins) == {"kimi_k25", "bailing_vl"}                                 # plugin classes registered first
    assert registered["bailing_v3_vl"]["mm_plugin"] == ("bailing_vl", {"image_token": "<|image_pad|>", "video_token": "<|video_pad|>"})


def test_chat_formats_register_with_a_fake_swift(monkeypatch):
    import sys
    import types

    from torchturbo_b200.adapters import chat_templates as C

    metas = {}

    class TemplateMeta:
        def __init__(self, template_type, prefix, prompt, chat_sep, suffix=None, system_prefix=None, default_system=None, stop_words=None):
            self.template_type, self.prefix, self.prompt, self.chat_sep = template_type, prefix, prompt, chat_sep
            self.suffix, self.system_prefix, self.default_system, self.stop_words = suffix, system_prefix, default_system, stop_words

    for name, attrs in (("swift", {}), ("swift.template", {"register_template": lambda m, exist_ok=False: metas.__setitem__(m.template_type, m)}),
                        ("swift.template.template_meta", {"TemplateMeta": TemplateMeta})):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        m.__path__ = []
        monkeypatch.setitem(sys.modules, name, m)
    done = C.register_swift_templates(["bailing_v3", "kimi_k25", "glm5"])
    assert done == ["turbo_bailing_v3", "turbo_kimi_k25", "turbo_glm5"]
    b = metas["turbo_bailing_v3"]
    assert b.prompt == ["<role>HUMAN</role>\n{{QUERY}}<|role_end|>\n\n<role>ASSISTANT</role>"] and b.chat_sep == ["<|role_end|>\n\n"]
    assert b.system_prefix == ["<role>SYSTEM</role>\n{{SYSTEM}}<|role_end|>\n\n"] and b.suffix == ["<|role_end|>"] and b.stop_words == []
    k = metas["turbo_kimi_k25"]
    assert k.default_system == "You are a helpful assistant" and k.stop_words == ["<|im_end|>"]
    g = metas["turbo_glm5"]
    assert g.prefix == ["[gMASK]<sop>"] and g.system_prefix[0] == "[gMASK]<sop>" and g.chat_sep == ["\n"]


def test_ling_vl_tool_serialisers():
    from torchturbo_b200.adapters import chat_templates as C

    t = C.ling_vl_tool_call_text([{"name": "get", "arguments": {"city": "Paris", "days": 3}}, '{"name": "f", "arguments": {}}'])
    assert t == ("<tool_call>get\n<arg_key>city</arg_key>\n<arg_value>Paris</arg_value>\n<arg_key>days</arg_key>\n"
                 "<arg_value>3</arg_value>\n</tool_call>\n<tool_call>f\n</tool_call>")
    with pytest.raises(ValueError):
        C.ling_vl_tool_call_text([{"name": " ", "arguments": {}}])
    with pytest.raises(ValueError):
        C.ling_vl_tool_call_text([{"name": "f", "arguments": [1]}])
    o = C.ling_vl_observation_text(["a", "b"])
    assert o == "<role>OBSERVATION</role>\n<tool_response>\na\n</tool_response>\n<tool_response>\nb\n</tool_response>"
    with pytest.raises(ValueError):
        C.ling_vl_observation_text([])


def test_swift_template_wrap_keeps_input_ids_and_merges_mrope(monkeypatch):
    import sys
    import types

    from torchturbo_b200.adapters import chat_templates as C

    class Native:
        def pre_forward_hook(self, model, args, kwargs):
            kwargs = dict(kwargs)
            kwargs.pop("input_ids")                      # what swift does once vision is folded into the embeddings
            kwargs["inputs_embeds"] = "E"
            return args, kwargs

    K = C.keep_inputs_template(Native)
    assert C.keep_inputs_template(K) is K
    ids = torch.arange(6).view(1, 6)
    pos = torch.arange(18).view(3, 1, 6)
    _, kw = K().pre_forward_hook(None, (), {"input_ids": ids, "position_ids": pos, "text_position_ids": torch.arange(6).view(1, 6)})
    assert kw["input_ids"] is ids and kw["inputs_embeds"] == "E" and "text_position_ids" not in kw
    assert kw["position_ids"].shape == (4, 1, 6) and torch.equal(kw["position_ids"][0, 0], torch.arange(6))
    plain = {"position_ids": torch.arange(6).view(1, 6)}
    assert C.merge_mrope_rows(dict(plain))["position_ids"].shape == (1, 6)

    mapping = {"qwen3_5": types.SimpleNamespace(template_cls=Native, template_type="qwen3_5")}
    reg = types.ModuleType("swift.template.register")
    reg.TEMPLATE_MAPPING = mapping
    reg.register_template = lambda meta, exist_ok=False: mapping.__setitem__(meta.template_type, meta)
    for name, mod in (("swift", types.ModuleType("swift")), ("swift.template", types.ModuleType("swift.template")),
                      ("swift.template.register", reg)):
        monkeypatch.setitem(sys.modules, name, mod)
    assert C.wrap_swift_native_templates(("qwen3_5", "unknown")) == ["qwen3_5"]
    assert mapping["qwen3_5"].template_cls._tt_keeps_inputs
    assert C.wrap_swift_native_templates(("qwen3_5",)) == []       # already wrapped
