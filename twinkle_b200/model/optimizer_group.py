"""Per-adapter training state.

Parity: reference ``src/twinkle/model/optimizer_group.py:16-91`` and
``model/transformers/transformers.py:71-141``: every adapter (tenant) — and the
default un-named one — owns its optimizer hyper-parameters, scheduler, loss,
template, processor, metrics, gradient-accumulation counter and the running
``TrainStatus`` of the current accumulation window.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

from ..loss import CrossEntropyLoss, Loss
from ..metric import LossMetric, Metric, TrainMetric


@dataclass
class TrainStatus:
    inputs: Any = None
    outputs: Any = None
    loss_value: Any = None  # graph-connected loss of the last forward
    loss_sum: float = 0.0
    num_tokens: float = 0.0  # this rank's denominator contribution of the window
    metrics: List[Metric] = field(default_factory=list)
    forward_kwargs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class AdamHyper:
    lr: float = 1e-5
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.01


@dataclass
class OptimizerGroup:
    adapter_name: str = ''
    hyper: AdamHyper = field(default_factory=AdamHyper)
    optimizer: Any = None  # engine optimizer facade (exposes param_groups for schedulers)
    lr_scheduler: Any = None
    loss_instance: Optional[Callable] = None
    template: Any = None
    processor: Any = None
    train_status: TrainStatus = field(default_factory=TrainStatus)
    eval_status: TrainStatus = field(default_factory=TrainStatus)
    gradient_accumulation_steps: int = 1
    cur_step: int = 0  # number of backward calls
    optim_steps: int = 0  # number of optimizer steps (Adam bias correction)
    consumed_train_samples: int = 0
    _last_grad_norm: Optional[float] = None
    adapter_config: Any = None
    grad_ready: bool = False

    def __post_init__(self):
        if self.loss_instance is None:
            self.set_loss(CrossEntropyLoss())
        if not self.train_status.metrics:
            self.train_status.metrics = [LossMetric(), TrainMetric()]
        if not self.eval_status.metrics:
            self.eval_status.metrics = [LossMetric()]

    def set_loss(self, loss) -> None:
        from ..utils.nccl_safe import safe_loss
        self.loss_instance = safe_loss(loss)

    def do_grad_sync(self, gradient_accumulation_steps: Optional[int] = None) -> bool:
        g = gradient_accumulation_steps or self.gradient_accumulation_steps
        return self.cur_step % max(g, 1) == 0

    def status(self, is_training: bool) -> TrainStatus:
        return self.train_status if is_training else self.eval_status

    def current_lr(self):
        if self.optimizer is not None:
            return [g['lr'] for g in self.optimizer.param_groups]
        return [self.hyper.lr]
