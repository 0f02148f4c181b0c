"""DeepSeek V4.1 Flash (fp8 / packed fp4 with ue8m0 scales) -> bf16 safetensors.

    python scripts/dequant/deepseekv4_1.py --input-fp8-hf-path /ckpt/quantised --output-hf-path /ckpt/bf16

Same command line as scripts/dequant/deepseekv4_1.py of the reference; the work is done by `convert.convert_checkpoint` with the
`deepseek_v4_1` profile of `formats.py`."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from convert import cli  # noqa: E402


def main(argv=None):
    return cli("deepseek_v4_1", "--input-fp8-hf-path", "--output-hf-path", argv)


if __name__ == "__main__":
    main()
