"""Which swift pipeline class each engine-backed stage replaces (adapters/msswift/stages.py:14-90 of the reference)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SwiftStageSpec:
    name: str              # sft | pt | dpo
    pipeline_module: str   # module whose global is swapped
    pipeline_attr: str     # name of that global
    main_attr: str         # the module's entry function (`sft_main`, ...)
    trainer_key: str       # swift's trainer-registry key the stage resolves through


_STAGES: list[SwiftStageSpec] = []


def register_stage(spec: SwiftStageSpec) -> None:
    if not any(s.name == spec.name for s in _STAGES):
        _STAGES.append(spec)


def iter_stages() -> tuple[SwiftStageSpec, ...]:
    return tuple(_STAGES)


def get_stage(name: str) -> SwiftStageSpec:
    for s in _STAGES:
        if s.name == name:
            return s
    raise KeyError(name)


register_stage(SwiftStageSpec("sft", "swift.pipelines.train.sft", "SwiftSft", "sft_main", "causal_lm"))
register_stage(SwiftStageSpec("pt", "swift.pipelines.train.pretrain", "SwiftPretrain", "pretrain_main", "causal_lm"))
register_stage(SwiftStageSpec("dpo", "swift.pipelines.train.rlhf", "SwiftRLHF", "rlhf_main", "dpo"))
