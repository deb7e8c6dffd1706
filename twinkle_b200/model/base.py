"""The trainable-model contract.

Parity: reference ``src/twinkle/model/base.py:21-178`` — the method set every
backend exposes (and every HTTP twin mirrors), plus process-group bootstrap.
"""
from __future__ import annotations

import datetime
import os
from abc import ABC, abstractmethod
from typing import Any, Dict, Optional

from ..utils.platform import Platform


class TwinkleModel(ABC):
    """Methods take ``adapter_name=`` where multi-tenancy applies."""

    @abstractmethod
    def forward(self, *, inputs, **kwargs): ...

    @abstractmethod
    def forward_only(self, *, inputs, **kwargs): ...

    @abstractmethod
    def calculate_loss(self, **kwargs): ...

    @abstractmethod
    def backward(self, **kwargs): ...

    @abstractmethod
    def forward_backward(self, *, inputs, **kwargs): ...

    @abstractmethod
    def clip_grad_norm(self, max_grad_norm: float = 1.0, norm_type=2, **kwargs): ...

    @abstractmethod
    def step(self, **kwargs): ...

    @abstractmethod
    def zero_grad(self, **kwargs): ...

    @abstractmethod
    def lr_step(self, **kwargs): ...

    @abstractmethod
    def clip_grad_and_step(self, max_grad_norm: float = 1.0, norm_type=2, **kwargs): ...

    @abstractmethod
    def set_loss(self, loss_cls, **kwargs): ...

    @abstractmethod
    def set_optimizer(self, optimizer_cls, **kwargs): ...

    @abstractmethod
    def set_lr_scheduler(self, scheduler_cls, **kwargs): ...

    @abstractmethod
    def save(self, name: str, output_dir: Optional[str] = None, **kwargs) -> str: ...

    @abstractmethod
    def load(self, name: str, output_dir: Optional[str] = None, **kwargs) -> None: ...

    @abstractmethod
    def get_state_dict(self, **kwargs) -> Dict[str, Any]: ...

    @abstractmethod
    def resume_from_checkpoint(self, checkpoint_dir: str, **kwargs) -> Dict[str, Any]: ...

    @abstractmethod
    def apply_patch(self, patch_cls, **kwargs) -> None: ...

    @abstractmethod
    def add_metric(self, metric_cls, is_training: Optional[bool] = None, **kwargs) -> None: ...

    @abstractmethod
    def calculate_metric(self, is_training: bool, **kwargs) -> Dict[str, Any]: ...

    @abstractmethod
    def add_adapter_to_model(self, adapter_name: str, config_or_dir, **kwargs) -> None: ...

    @abstractmethod
    def set_template(self, template_cls, **kwargs) -> None: ...

    @abstractmethod
    def set_processor(self, processor_cls, **kwargs) -> None: ...

    @abstractmethod
    def get_train_configs(self, **kwargs) -> str: ...

    def upload_to_hub(self, checkpoint_dir: str, hub_model_id: str, hub_token: Optional[str] = None, async_upload: bool = True):
        from ..hub import HubOperation
        return HubOperation.push_to_hub(hub_model_id, checkpoint_dir, token=hub_token, async_upload=async_upload)

    # --------------------------------------------------------------------
    @staticmethod
    def _try_init_process_group() -> None:
        """``init_process_group(backend, env://)`` bound to this rank's device,
        when launched with more than one rank and not yet initialised."""
        import torch
        import torch.distributed as dist
        if not dist.is_available() or dist.is_initialized():
            return
        if Platform.get_world_size() <= 1 and 'MASTER_ADDR' not in os.environ:
            return
        backend = Platform.device_backend()
        timeout = datetime.timedelta(seconds=int(os.environ.get('TWINKLE_DIST_TIMEOUT_SECONDS', '7200')))
        kw = {}
        if backend == 'nccl':
            Platform.set_device()
            kw['device_id'] = Platform.current_device()
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29500')
        dist.init_process_group(backend=backend, init_method='env://', timeout=timeout, rank=Platform.get_rank(),
                                world_size=Platform.get_world_size(), **kw)
