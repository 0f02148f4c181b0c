from .model import GlmMoeDsaConfig, TurboGlmMoeDsaForCausalLM

__all__ = ["GlmMoeDsaConfig", "TurboGlmMoeDsaForCausalLM"]
