from .lm_loss import IGNORE_INDEX, LossStream, chunk_loss, logits_loss, prepare_loss_labels, shift_labels_packed

__all__ = ["IGNORE_INDEX", "LossStream", "chunk_loss", "logits_loss", "prepare_loss_labels", "shift_labels_packed"]
