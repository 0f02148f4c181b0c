from .model import BailingMoeV3VLConfig, TurboBailingMoeV3VLForConditionalGeneration

__all__ = ["BailingMoeV3VLConfig", "TurboBailingMoeV3VLForConditionalGeneration"]
