from .flops import BaseModelFlops, ComputeProfile, LLMFlops, MlaLLMFlops, MoELLMFlops, VLMFlops
from .mfu_estimator import PEAK_TFLOPS_TABLE, MFUEstimator
from .tracker import MetricTracker

__all__ = ["BaseModelFlops", "ComputeProfile", "LLMFlops", "MlaLLMFlops", "MoELLMFlops", "VLMFlops",
           "PEAK_TFLOPS_TABLE", "MFUEstimator", "MetricTracker"]
