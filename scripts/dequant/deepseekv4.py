"""DeepSeek V4 (fp8 128x128 blocks, packed mxfp4 experts) -> bf16 safetensors.

    python scripts/dequant/deepseekv4.py --input-fp8-hf-path /ckpt/quantised --output-hf-path /ckpt/bf16

Same command line as scripts/dequant/deepseekv4.py of the reference; the work is done by `convert.convert_checkpoint` with the
`deepseek_v4` profile of `formats.py`."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from convert import cli  # noqa: E402


def main(argv=None):
    return cli("deepseek_v4", "--input-fp8-hf-path", "--output-hf-path", argv)


if __name__ == "__main__":
    main()
