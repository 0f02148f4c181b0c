"""ms-swift launcher: `torchrun scripts/runs/run_swift.py [sft|pt|dpo] --tt_* <swift arguments>`."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import torchturbo_b200
    from torchturbo_b200.engine.args import parse_torchturbo_args, set_torchturbo_args

    stage = sys.argv[1] if len(sys.argv) > 1 and sys.argv[1] in ("sft", "pt", "dpo") else "sft"
    argv = sys.argv[2:] if len(sys.argv) > 1 and sys.argv[1] == stage else sys.argv[1:]
    tt_args, rest = parse_torchturbo_args(argv)
    set_torchturbo_args(tt_args)
    adapter = torchturbo_b200.activate("msswift")
    if adapter is None:            # TORCH_TURBO_DISABLE: stock swift
        import importlib

        from torchturbo_b200.adapters.msswift import get_stage

        spec = get_stage(stage)
        return getattr(importlib.import_module(spec.pipeline_module), spec.main_attr)(rest)
    # swift's own entry function of the stage (`sft_main`, `pretrain_main`, `rlhf_main`) now builds the engine-backed
    # pipeline, because the adapter swapped the pipeline class in that module
    return adapter.main(stage, rest)


if __name__ == "__main__":
    main()
