from .coordinator import CheckpointCoordinator
from .distributed import RemoteRankError, collective_check, rank_zero_call
from .layout import (HF_DIR, MODEL_DCP_DIR, OPTIMIZER_DCP_DIR, SCHEDULER_FILE, ModelFormat, dcp_status, hf_status,
                     resolve_model_format, save_json, save_scheduler, sync_directory, validate_output_dir)
from .metadata import build_metadata, load_metadata, save_metadata, validate_peft_configs

__all__ = ["CheckpointCoordinator", "RemoteRankError", "collective_check", "rank_zero_call", "HF_DIR", "MODEL_DCP_DIR",
           "OPTIMIZER_DCP_DIR", "SCHEDULER_FILE", "ModelFormat", "dcp_status", "hf_status", "resolve_model_format",
           "save_json", "save_scheduler", "sync_directory", "validate_output_dir", "build_metadata", "load_metadata",
           "save_metadata", "validate_peft_configs"]
