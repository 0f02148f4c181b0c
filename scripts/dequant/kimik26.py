"""Kimi-K2.6 (packed int4 with group scales) -> bf16 safetensors.

    python scripts/dequant/kimik26.py --model-dir /ckpt/quantised --output-dir /ckpt/bf16

Same command line as scripts/dequant/kimik26.py of the reference; the work is done by `convert.convert_checkpoint` with the
`kimi_k26` profile of `formats.py`."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from convert import cli  # noqa: E402


def main(argv=None):
    return cli("kimi_k26", "--model-dir", "--output-dir", argv)


if __name__ == "__main__":
    main()
