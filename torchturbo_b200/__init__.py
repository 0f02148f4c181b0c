"""torchturbo_b200: a B200-native (sm_100a) LLM/VLM post-training engine."""
__version__ = "0.1.0"
