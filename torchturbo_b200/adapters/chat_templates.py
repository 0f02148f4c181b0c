"""Chat formats of the model families, as data, and their registration with LlamaFactory and ms-swift.

A `ChatFormat` lists the literal wrappers a family's tokenizer expects around each role (`{content}` marks the text).
The two `register_*` functions translate the table into the host framework's own template objects; nothing of either
framework is imported until they are called.  Families whose format is the stock Qwen ChatML (qwen3, qwen3_moe, qwen3_vl)
use the framework's own templates and are not listed.  (models/*/lf_template.py and models/*/swift_template.py of the
reference: one file per family and framework.)
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any

from ..logging import get_logger
from .mm_tokens import register_lf_mm_plugins

logger = get_logger(__name__)


@dataclass(frozen=True)
class ChatFormat:
    name: str
    user: str                       # wraps a user turn and opens the assistant turn
    assistant: str                  # closes an assistant turn
    system: str
    observation: str | None = None  # tool result turn (opens the next assistant turn)
    prefix: str | None = None       # once, in front of the conversation ("{bos}" = the tokenizer's BOS token)
    default_system: str | None = None
    stop_words: tuple[str, ...] = ()
    thought_words: tuple[str, str] | None = None
    efficient_eos: bool = False     # the assistant wrapper already ends the turn; EOS is appended only at the very end
    replace_eos: bool = False       # the first stop word becomes the tokenizer's EOS
    reasoning: bool = False         # thinking content is stripped from history turns
    tool_format: str | None = None
    mm_plugin: tuple[str, dict] | None = None      # (LlamaFactory mm plugin name, its keyword arguments)
    swift_suffix: tuple[str, ...] = field(default=())


FORMATS: dict[str, ChatFormat] = {f.name: f for f in (
    ChatFormat("qwen3_5", user="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n", assistant="{content}<|im_end|>\n",
               system="<|im_start|>system\n{content}<|im_end|>\n", observation="<|im_start|>user\n<tool_response>\n{content}\n</tool_response><|im_end|>\n<|im_start|>assistant\n",
               stop_words=("<|im_end|>",), replace_eos=True, reasoning=True, thought_words=("<think>\n", "\n</think>\n\n"),
               tool_format="qwen", mm_plugin=("qwen3_vl", {"image_token": "<|image_pad|>", "video_token": "<|video_pad|>"}),
               swift_suffix=("<|im_end|>",)),
    ChatFormat("qwen3_5_nothink", user="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n", assistant="{content}<|im_end|>\n",
               system="<|im_start|>system\n{content}<|im_end|>\n", stop_words=("<|im_end|>",), replace_eos=True, tool_format="qwen",
               mm_plugin=("qwen3_vl", {"image_token": "<|image_pad|>", "video_token": "<|video_pad|>"}), swift_suffix=("<|im_end|>",)),
    ChatFormat("bailing_v3", user="<role>HUMAN</role>\n{content}<|role_end|>\n\n<role>ASSISTANT</role>", assistant="{content}<|role_end|>\n\n",
               system="<role>SYSTEM</role>\n{content}<|role_end|>\n\n",
               observation="<role>OBSERVATION</role>\n\n```result\n{content}\n```\n<|role_end|>\n\n<role>ASSISTANT</role>",
               stop_words=("",), efficient_eos=True, tool_format="ling_v3", swift_suffix=("<|role_end|>",)),
    ChatFormat("bailing_v3_vl", user="<role>HUMAN</role>{content}<|role_end|><role>ASSISTANT</role>\n", assistant="{content}<|role_end|>",
               system="<role>SYSTEM</role>{content}<|role_end|>", stop_words=("<|role_end|>",), thought_words=("<think>", "</think>"),
               mm_plugin=("bailing_vl", {"image_token": "<|image_pad|>", "video_token": "<|video_pad|>"}), swift_suffix=("<|role_end|>",)),
    ChatFormat("kimi_k25", user="<|im_user|>user<|im_middle|>{content}<|im_end|><|im_assistant|>assistant<|im_middle|>",
               assistant="{content}<|im_end|>", system="<|im_system|>system<|im_middle|>{content}<|im_end|>",
               default_system="You are a helpful assistant", stop_words=("<|im_end|>",), replace_eos=True,
               mm_plugin=("kimi_k25", {"image_token": "<|media_pad|>"}), swift_suffix=("<|im_end|>",)),
    ChatFormat("deepseek_v4", user="<｜User｜>{content}<｜Assistant｜>", assistant="{content}<｜end▁of▁sentence｜>", system="{content}\n\n",
               observation="\n<function_results>\n<result>{content}</result>\n</function_results>", prefix="{bos}",
               stop_words=("<｜end▁of▁sentence｜>",), thought_words=("<think>", "</think>"), tool_format="deepseek_v4",
               swift_suffix=("<｜end▁of▁sentence｜>",)),
    ChatFormat("deepseek_v4_thinking", user="<｜User｜>{content}<｜Assistant｜>", assistant="{content}<｜end▁of▁sentence｜>", system="{content}\n\n",
               observation="\n<function_results>\n<result>{content}</result>\n</function_results>", prefix="{bos}",
               stop_words=("<｜end▁of▁sentence｜>",), thought_words=("<think>", "</think>"), reasoning=True, tool_format="deepseek_v4",
               swift_suffix=("<｜end▁of▁sentence｜>",)),
    ChatFormat("glm5", user="<|user|>\n{content}<|assistant|>", assistant="\n{content}", system="<|system|>\n{content}",
               observation="<|observation|>\n{content}<|assistant|>", prefix="[gMASK]<sop>", stop_words=("<|user|>", "<|observation|>"),
               thought_words=("<think>", "</think>"), efficient_eos=True, reasoning=True, tool_format="glm4_moe",
               swift_suffix=("<|user|>",)),
)}

# model_type -> default format
MODEL_FORMATS = {"qwen3_5": "qwen3_5", "qwen3_5_moe": "qwen3_5", "qwen3_5_moe_text": "qwen3_5", "qwen4_exp": "qwen3_5",
                 "bailing_hybrid": "bailing_v3", "bailing_moe_v3": "bailing_v3", "bailing_moe_v3_vl": "bailing_v3_vl",
                 "kimi_k25": "kimi_k25", "deepseek_v4": "deepseek_v4", "glm_moe_dsa": "glm5", "llada2_moe": "bailing_v3"}

LING_V3_TOOL_PROMPT = ("# Tools\nYou may call one or more functions to assist with the user query.\n"
                       "You are provided with function signatures within <tools></tools> XML tags:\n<tools>{tool_text}"
                       "\n</tools>\nIf none of the functions can be used, point it out. "
                       "If the given question lacks the parameters required by the function, also point it out.\n"
                       "If you need to use a function, for each function call, output the function name and arguments "
                       "within the following XML format:\n"
                       "<function=func_name>\n<parameter=arg_key>\narg_value\n</parameter>\n...\n</function>\n")


def ling_v3_tool_text(tools: list[dict[str, Any]]) -> str:
    """The tool section of a Bailing / Ling v3 system prompt: one JSON function signature per line."""
    lines = ""
    for tool in tools:
        wrapped = tool if tool.get("type") == "function" else {"type": "function", "function": tool}
        lines += "\n" + json.dumps(wrapped, ensure_ascii=False)
    return LING_V3_TOOL_PROMPT.format(tool_text=lines)


def ling_vl_tool_call_text(calls: list[dict[str, Any]]) -> str:
    """Tool calls the way the Bailing VL checkpoints render them: `<tool_call>name`, one `<arg_key>` / `<arg_value>`
    pair per argument (non-string values as JSON), `</tool_call>`; calls separated by a newline.  Each call is a
    dict with `name` and `arguments` (or a JSON string of such a dict).
    (BailingVLAgentTemplate._format_tool_calls, models/bailing_moe_v3_vl/swift_template.py:60-80 in the reference.)"""
    out = []
    for call in calls:
        if isinstance(call, str):
            call = json.loads(call)
        name, args = call.get("name"), call.get("arguments")
        if isinstance(args, str):
            args = json.loads(args)
        if not isinstance(name, str) or not name.strip() or not isinstance(args, dict):
            raise ValueError("a tool call needs a non-empty name and an arguments object")
        lines = [f"<tool_call>{name}"]
        for k, v in args.items():
            lines += [f"<arg_key>{k}</arg_key>", f"<arg_value>{v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)}</arg_value>"]
        lines.append("</tool_call>")
        out.append("\n".join(lines))
    return "\n".join(out)


def ling_vl_observation_text(results: list[str]) -> str:
    """A group of consecutive tool results as one OBSERVATION turn body (without the closing role marker)."""
    if not results:
        raise ValueError("an observation turn needs at least one tool result")
    return "<role>OBSERVATION</role>" + "".join(f"\n<tool_response>\n{r}\n</tool_response>" for r in results)


def render(fmt: ChatFormat, messages: list[dict[str, str]], *, bos: str = "", add_generation_prompt: bool = False) -> str:
    """Plain-text rendering of a conversation (used by tests and by dataset plugins that tokenise offline).  The user
    wrapper opens the assistant turn, so a trailing user message already ends with the generation prompt."""
    out = (fmt.prefix or "").replace("{bos}", bos)
    msgs = list(messages)
    if msgs and msgs[0]["role"] == "system":
        out += fmt.system.replace("{content}", msgs.pop(0)["content"])
    elif fmt.default_system:
        out += fmt.system.replace("{content}", fmt.default_system)
    for m in msgs:
        if m["role"] == "user":
            out += fmt.user.replace("{content}", m["content"])
        elif m["role"] == "assistant":
            out += fmt.assistant.replace("{content}", m["content"])
        elif m["role"] in ("observation", "tool"):
            if fmt.observation is None:
                raise ValueError(f"format {fmt.name} has no tool-result turn")
            out += fmt.observation.replace("{content}", m["content"])
        else:
            raise ValueError(f"unknown role {m['role']!r}")
    if add_generation_prompt and msgs and msgs[-1]["role"] == "assistant":
        raise ValueError("a generation prompt after an assistant turn is not defined")
    return out


def _lf_slots(text: str) -> list:
    """LlamaFactory slot list: `{{content}}` placeholders inside strings, special tokens as one-element sets."""
    if text == "{bos}":
        return [{"bos_token"}]
    return [text.replace("{content}", "{{content}}")]


def register_lf_templates(names: list[str] | None = None) -> list[str]:
    from llamafactory.data import template as T
    from llamafactory.data.formatter import EmptyFormatter, FunctionFormatter, StringFormatter, ToolFormatter

    done = []
    register_lf_mm_plugins()      # the plugin names the formats below refer to
    tools = getattr(__import__("llamafactory.data.tool_utils", fromlist=["TOOLS"]), "TOOLS", None)
    if isinstance(tools, dict) and "ling_v3" not in tools:
        base = getattr(__import__("llamafactory.data.tool_utils", fromlist=["QwenToolUtils"]), "QwenToolUtils", None)
        if base is not None:
            tools["ling_v3"] = type("LingV3ToolUtils", (base,), {"tool_formatter": staticmethod(ling_v3_tool_text)})()
    for name in names or list(FORMATS):
        f = FORMATS[name]
        if name in getattr(T, "TEMPLATES", {}):
            continue
        kw: dict[str, Any] = dict(name=name, format_user=StringFormatter(slots=_lf_slots(f.user)),
                                  format_assistant=StringFormatter(slots=_lf_slots(f.assistant)),
                                  format_system=StringFormatter(slots=_lf_slots(f.system)),
                                  stop_words=list(f.stop_words), efficient_eos=f.efficient_eos, replace_eos=f.replace_eos)
        if f.observation is not None:
            kw["format_observation"] = StringFormatter(slots=_lf_slots(f.observation))
        if f.prefix is not None:
            kw["format_prefix"] = EmptyFormatter(slots=_lf_slots(f.prefix))
        if f.default_system:
            kw["default_system"] = f.default_system
        if f.thought_words:
            kw["thought_words"] = f.thought_words
        known_tools = tools if isinstance(tools, dict) else {}
        if f.tool_format and f.tool_format in known_tools:
            kw["format_function"] = FunctionFormatter(slots=_lf_slots(f.assistant), tool_format=f.tool_format)
            kw["format_tools"] = ToolFormatter(tool_format=f.tool_format)
        if f.reasoning and hasattr(T, "ReasoningTemplate"):
            kw["template_class"] = T.ReasoningTemplate
        if f.mm_plugin is not None:
            try:
                from llamafactory.data.mm_plugin import get_mm_plugin

                kw["mm_plugin"] = get_mm_plugin(name=f.mm_plugin[0], **f.mm_plugin[1])
            except Exception:  # noqa: BLE001 - plugin of another LlamaFactory version: text-only template
                logger.warning_rank0("LlamaFactory has no mm plugin %s: template %s is registered text-only", f.mm_plugin[0], name)
        T.register_template(**kw)
        done.append(name)
    return done


def register_swift_templates(names: list[str] | None = None) -> list[str]:
    from swift.template import register_template
    from swift.template.template_meta import TemplateMeta

    done = []
    for name in names or list(FORMATS):
        f = FORMATS[name]
        head, _, tail = f.user.partition("{content}")
        prompt = [f.user.replace("{content}", "{{QUERY}}")]
        chat_sep = [f.assistant.replace("{content}", "")] if f.assistant.replace("{content}", "") else []
        prefix = [(f.prefix or "").replace("{bos}", "")] if f.prefix and f.prefix != "{bos}" else []
        system_prefix = prefix + [f.system.replace("{content}", "{{SYSTEM}}")]
        meta = TemplateMeta(f"turbo_{name}", prefix=prefix, prompt=prompt, chat_sep=chat_sep or None,
                            suffix=list(f.swift_suffix) or None, system_prefix=system_prefix, default_system=f.default_system,
                            stop_words=[w for w in f.stop_words if w])
        try:
            register_template(meta, exist_ok=True)
        except TypeError:
            register_template(meta)
        done.append(meta.template_type if hasattr(meta, "template_type") else f"turbo_{name}")
    return done


# ---- ms-swift: keep what the models need across swift's own pre-forward step -----------------------------------------
def merge_mrope_rows(inputs: dict[str, Any]) -> dict[str, Any]:
    """swift delivers the text positions `[B, S]` and the three mRoPE rows `[3, B, S]` separately; the hybrid models
    take one `[4, B, S]` tensor (text row first).  In place; other layouts pass through."""
    tpos, pos = inputs.get("text_position_ids"), inputs.get("position_ids")
    if tpos is not None and pos is not None and pos.dim() == 3 and pos.shape[0] == 3:
        import torch

        inputs["position_ids"] = torch.cat((tpos.reshape(1, *pos.shape[1:]), pos), dim=0)
        inputs.pop("text_position_ids", None)
    return inputs


def keep_inputs_template(template_cls: type, keep: tuple[str, ...] = ("input_ids",)) -> type:
    """Subclass of a swift template class whose `pre_forward_hook` puts back the keyword arguments swift drops when
    it folds the vision features into `inputs_embeds` (the multi-token-prediction heads embed the shifted token ids
    themselves), then merges the mRoPE rows.  Wrapping twice returns the class unchanged.
    (models/qwen3_5/swift_template.py:33-52 in the reference.)"""
    if getattr(template_cls, "_tt_keeps_inputs", False):
        return template_cls

    class KeepInputs(template_cls):  # type: ignore[misc, valid-type]
        _tt_keeps_inputs = True

        def pre_forward_hook(self, model, args, kwargs):
            saved = {k: kwargs[k] for k in keep if k in kwargs}
            args, kwargs = super().pre_forward_hook(model, args, kwargs)
            for k, v in saved.items():
                kwargs.setdefault(k, v)
            return args, merge_mrope_rows(kwargs)

    KeepInputs.__name__ = f"{template_cls.__name__}KeepInputs"
    return KeepInputs


def wrap_swift_native_templates(names: tuple[str, ...] = ("qwen3_5",)) -> list[str]:
    """Re-register swift's own templates of the families the models of this package replace, with
    `keep_inputs_template` around their class.  Names swift does not know are skipped."""
    from copy import deepcopy

    from swift.template.register import TEMPLATE_MAPPING, register_template

    done = []
    for name in names:
        native = TEMPLATE_MAPPING.get(name)
        if native is None or getattr(native.template_cls, "_tt_keeps_inputs", False):
            continue
        meta = deepcopy(native)
        meta.template_cls = keep_inputs_template(native.template_cls)
        register_template(meta, exist_ok=True)
        done.append(name)
    return done
