from .base import BaseBackend, BaseCheckpointManager

__all__ = ["BaseBackend", "BaseCheckpointManager"]
