from .dpo import DPOConfig, build_reference_model, dpo_loss, dpo_step, sequence_logps
from .sft import TrainingArguments, TrainState, run_training, train_step

__all__ = ["DPOConfig", "build_reference_model", "dpo_loss", "dpo_step", "sequence_logps", "TrainingArguments",
           "TrainState", "run_training", "train_step"]
