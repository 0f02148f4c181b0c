from .backend import FSDP2Backend, in_recompute

__all__ = ["FSDP2Backend", "in_recompute"]
