from .adapter import BaseAdapter
from .patch import BasePatch
from .registry import get_adapter, list_adapters, register_adapter

__all__ = ["BaseAdapter", "BasePatch", "get_adapter", "list_adapters", "register_adapter"]
