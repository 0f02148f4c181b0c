"""Ling / Bailing MoE V3 (fp8 128x128 blocks) -> bf16 safetensors.

    python scripts/dequant/bailing.py --input-fp8-hf-path /ckpt/quantised --output-hf-path /ckpt/bf16

Same command line as scripts/dequant/bailing.py of the reference; the work is done by `convert.convert_checkpoint` with the
`bailing` profile of `formats.py`."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from convert import cli  # noqa: E402


def main(argv=None):
    return cli("bailing", "--input-fp8-hf-path", "--output-hf-path", argv)


if __name__ == "__main__":
    main()
