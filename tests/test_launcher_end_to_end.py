"""The stand-alone launcher (`scripts/runs/run_sft.py`) started the way a user starts it, `torchrun` with two CPU ranks:
training from a model configuration on a JSON-lines file, periodic checkpoints, resume, then fine-tuning from the exported
Hugging Face checkpoint with expert parallelism switched on by a `--tt_*` flag."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MOE = dict(model_type="qwen3_moe", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
           intermediate_size=128, moe_intermediate_size=32, num_experts=4, num_experts_per_tok=2, vocab_size=256)


def _run(args, port, timeout=600):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", TORCH_TURBO_DEVICE="cpu", OMP_NUM_THREADS="1",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "scripts", "runs", "run_sft.py")] + args
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, (res.stdout[-1500:], res.stderr[-3000:])
    return res.stdout + res.stderr


@pytest.mark.timeout(1500)
def test_launcher_trains_checkpoints_resumes_and_finetunes_its_own_export(tmp_path):
    g = torch.Generator().manual_seed(0)
    with open(tmp_path / "train.jsonl", "w") as f:
        for _ in range(40):
            n = int(torch.randint(10, 60, (1,), generator=g))
            f.write(json.dumps({"input_ids": torch.randint(1, 256, (n,), generator=g).tolist()}) + "\n")
    with open(tmp_path / "config.json", "w") as f:
        json.dump(MOE, f)
    common = ["--data", str(tmp_path / "train.jsonl"), "--seq_len", "64", "--lr", "1e-2", "--logging_steps", "1",
              "--tt_mixed_precision", "fp32", "--tt_hf_export", "final"]
    out = str(tmp_path / "run")
    log = _run(["--model_config", str(tmp_path / "config.json"), "--max_steps", "4", "--save_steps", "2", "--output_dir", out] + common, 29711)
    assert "step=4" in log
    assert os.path.isdir(os.path.join(out, "checkpoint-2", "model_distcp")) and os.path.isdir(os.path.join(out, "checkpoint-4", "huggingface"))
    log = _run(["--model_config", str(tmp_path / "config.json"), "--max_steps", "6", "--save_steps", "6", "--output_dir", out,
                "--resume_from_checkpoint", os.path.join(out, "checkpoint-4")] + common, 29713)
    assert "step=5" in log and "step=6" in log and "step=4 " not in log
    hf = os.path.join(out, "checkpoint-6", "huggingface")
    assert os.path.isfile(os.path.join(hf, "config.json")) and any(fn.endswith(".safetensors") for fn in os.listdir(hf))
    # fine-tune the export with the experts spread over the two ranks
    out2 = str(tmp_path / "run2")
    log = _run(["--model", hf, "--max_steps", "2", "--output_dir", out2, "--tt_ep_size", "2"] + common, 29715)
    assert "step=2" in log and os.path.isdir(os.path.join(out2, "checkpoint-2", "huggingface"))
