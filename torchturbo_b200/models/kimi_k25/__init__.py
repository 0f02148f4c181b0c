from .model import KimiK25Config, TurboKimiK25ForConditionalGeneration

__all__ = ["KimiK25Config", "TurboKimiK25ForConditionalGeneration"]
