"""LlamaFactory launcher: `torchrun scripts/runs/run_lf.py --tt_* <LlamaFactory arguments>`.
Consumes the `--tt_*` flags, activates the LlamaFactory adapter and hands the remaining argv to `run_exp`."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import torchturbo_b200
    from torchturbo_b200.engine.args import parse_torchturbo_args, set_torchturbo_args

    tt_args, rest = parse_torchturbo_args()
    set_torchturbo_args(tt_args)
    torchturbo_b200.activate("llamafactory_v0")
    sys.argv = [sys.argv[0]] + rest
    from llamafactory.train.tuner import run_exp

    run_exp()


if __name__ == "__main__":
    main()
