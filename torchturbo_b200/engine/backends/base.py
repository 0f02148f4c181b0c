"""Backend and checkpoint-manager contracts (engine/backends/base.py:24-230 of the reference)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any

import torch
import torch.nn as nn


class BaseCheckpointManager(ABC):
    """Backend-specific persistence: Hugging Face safetensors in/out and native sharded state."""

    @abstractmethod
    def load_hf(self, model: nn.Module, path: str) -> None: ...

    @abstractmethod
    def save_hf(self, model: nn.Module, path: str, *, source_path: str | None = None) -> None: ...

    @abstractmethod
    def save_native_model(self, model: nn.Module, path: str) -> None: ...

    @abstractmethod
    def load_native_model(self, model: nn.Module, path: str) -> None: ...

    @abstractmethod
    def save_native_optimizer(self, model: nn.Module, optimizer, path: str) -> None: ...

    @abstractmethod
    def load_native_optimizer(self, model: nn.Module, optimizer, path: str) -> None: ...

    @abstractmethod
    def native_model_status(self, path: str) -> str:
        """'complete' | 'incomplete' | 'missing'"""

    @abstractmethod
    def native_optimizer_status(self, path: str) -> str: ...


class BaseBackend(ABC):
    def __init__(self, config: Any, runtime: Any) -> None:
        self.config = config
        self.runtime = runtime

    @abstractmethod
    def prepare_model(self, model: nn.Module, parallel_plan: Any, peft_config: Any = None) -> nn.Module: ...

    @abstractmethod
    def materialize(self, model: nn.Module, *, init_weights: bool = True) -> None: ...

    def finalize_model_load(self, model: nn.Module) -> None:
        pass

    @abstractmethod
    def create_checkpoint_manager(self) -> BaseCheckpointManager: ...

    @abstractmethod
    def prepare_optimizer(self, model: nn.Module, optimizer_plan: Any) -> torch.optim.Optimizer: ...

    def offload_optimizer(self, optimizer) -> None:
        raise NotImplementedError

    def restore_optimizer(self, optimizer) -> None:
        raise NotImplementedError

    @abstractmethod
    def get_dp_info(self) -> dict[str, Any]: ...

    @abstractmethod
    def get_ep_info(self) -> dict[str, Any]: ...

    @abstractmethod
    def get_sp_info(self) -> dict[str, Any]: ...

    def get_parallel_context(self) -> dict[str, Any]:
        return {"dp": self.get_dp_info(), "ep": self.get_ep_info(), "sp": self.get_sp_info()}

    @abstractmethod
    def prepare_inputs(self, model: nn.Module, inputs: dict[str, Any]) -> dict[str, Any]: ...

    @abstractmethod
    def compute_loss(self, model: nn.Module, inputs: dict[str, Any], **kwargs: Any) -> Any: ...

    def compute_diffusion_loss(self, model: nn.Module, inputs: dict[str, Any], **kwargs: Any) -> Any:
        raise NotImplementedError

    @abstractmethod
    def clip_grad_norm_(self, model: nn.Module, max_norm: float, optimizer=None) -> torch.Tensor: ...
