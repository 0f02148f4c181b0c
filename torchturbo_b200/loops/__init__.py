from .sft import TrainingArguments, TrainState, run_training, train_step

__all__ = ["TrainingArguments", "TrainState", "run_training", "train_step"]
