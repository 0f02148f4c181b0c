"""Convert a native sharded checkpoint into a Hugging Face safetensors export.

    torchrun --nproc-per-node N scripts/checkpoint/dcp_to_hf.py --checkpoint_dir out/checkpoint-100 --output_dir export

The model is rebuilt from `torchturbo/checkpoint.json` (model config + structural engine settings: EP / SP sizes and
precision must match the run that wrote the checkpoint, because EP-local tensors are stored per EP rank), the sharded
state is loaded, and the export is written with the index last (scripts/checkpoint/dcp_to_hf.py of the reference)."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def build_export_config(meta: dict):
    from torchturbo_b200.engine import EngineConfig

    eng = meta.get("engine", {})
    return EngineConfig.from_dict({
        "mixed_precision": eng.get("mixed_precision", "bf16"),
        "parallel_plan": {"sp_size": 1, "ep_size": eng.get("ep_size", 1)},
        "mtp": {"enabled": bool(eng.get("mtp_enabled", False))},
        "activation_checkpointing": {"enabled": False},
    })


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--checkpoint_dir", required=True)
    p.add_argument("--output_dir", required=True)
    a = p.parse_args(argv)
    from torchturbo_b200.engine import TorchTurboEngine
    from torchturbo_b200.engine.checkpoint import MODEL_DCP_DIR, dcp_status, load_metadata, validate_output_dir

    if not os.path.isdir(a.checkpoint_dir):
        raise FileNotFoundError(a.checkpoint_dir)
    if os.path.abspath(a.output_dir) == os.path.abspath(a.checkpoint_dir):
        raise ValueError("output_dir must differ from checkpoint_dir")
    meta = load_metadata(a.checkpoint_dir)
    if meta is None:
        raise FileNotFoundError(f"{a.checkpoint_dir} has no torchturbo/checkpoint.json")
    if dcp_status(os.path.join(a.checkpoint_dir, MODEL_DCP_DIR)) != "complete":
        raise RuntimeError(f"{a.checkpoint_dir}/{MODEL_DCP_DIR} is missing or incomplete")
    validate_output_dir(a.output_dir)
    engine = TorchTurboEngine(build_export_config(meta))
    model = engine.build_model(None, load_weights=False, init_kwargs={"config": meta["model"]["config"]})
    engine.load_from_checkpoint(model, a.checkpoint_dir)
    engine.checkpoint.manager.save_hf(model, a.output_dir, source_path=meta.get("source", {}).get("model_name_or_path"))
    return a.output_dir


if __name__ == "__main__":
    main()
