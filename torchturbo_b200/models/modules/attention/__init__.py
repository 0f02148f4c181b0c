from .interface import attention_forward, register_turbo_attention
from .ulysses import (SeqAllToAll, SequencePadding, SequenceParallelInputSlicingSpec, all_gather_sp_with_grad_reduce,
                      gather_heads_scatter_seq, gather_seq_scatter_heads, patch_forward_for_sp_input_slicing,
                      repeat_kv, slice_input_tensor, ulysses_attention, ulysses_pad_inputs)

__all__ = ["attention_forward", "register_turbo_attention", "SeqAllToAll", "SequencePadding", "SequenceParallelInputSlicingSpec", "all_gather_sp_with_grad_reduce",
           "gather_heads_scatter_seq", "gather_seq_scatter_heads", "patch_forward_for_sp_input_slicing", "repeat_kv",
           "slice_input_tensor", "ulysses_attention", "ulysses_pad_inputs"]
