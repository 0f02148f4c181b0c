from .symm import Channel, SymmetricBuffer

__all__ = ["Channel", "SymmetricBuffer"]
