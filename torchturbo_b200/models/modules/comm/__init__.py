from .comm import (all_gather_tensor, all_gather_tensor_chunked, all_reduce_sum_autograd, all_to_all,
                   gather_from_sequence_parallel_region)

__all__ = ["all_gather_tensor", "all_gather_tensor_chunked", "all_reduce_sum_autograd", "all_to_all",
           "gather_from_sequence_parallel_region"]
