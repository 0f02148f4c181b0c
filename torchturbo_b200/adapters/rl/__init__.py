from .packed import gather_logprobs_entropy, prepare_packed_mb_inputs, shifted_packed_tensor
from .sp import gather_logprobs_and_shift, gather_vocab_logits_stats

__all__ = ["gather_logprobs_entropy", "prepare_packed_mb_inputs", "shifted_packed_tensor", "gather_logprobs_and_shift",
           "gather_vocab_logits_stats"]
