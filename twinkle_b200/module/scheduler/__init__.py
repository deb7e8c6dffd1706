"""Warm-up learning-rate schedules.  Parity: reference
``src/twinkle/module/scheduler/*.py`` (LambdaLR-based cosine / linear)."""
from __future__ import annotations

import math

from torch.optim.lr_scheduler import LambdaLR


class CosineWarmupScheduler(LambdaLR):

    def __init__(self, optimizer, num_warmup_steps: int = 0, num_training_steps: int = 1000, min_lr_ratio: float = 0.0,
                 num_cycles: float = 0.5, last_epoch: int = -1):
        self.num_warmup_steps, self.num_training_steps = num_warmup_steps, num_training_steps

        def f(step: int) -> float:
            if step < num_warmup_steps:
                return step / max(1, num_warmup_steps)
            p = min((step - num_warmup_steps) / max(1, num_training_steps - num_warmup_steps), 1.0)
            c = 0.5 * (1.0 + math.cos(math.pi * 2.0 * num_cycles * p))
            return min_lr_ratio + (1.0 - min_lr_ratio) * max(0.0, c)

        super().__init__(optimizer, f, last_epoch)


class LinearWarmupScheduler(LambdaLR):

    def __init__(self, optimizer, num_warmup_steps: int = 0, num_training_steps: int = 1000, min_lr_ratio: float = 0.0,
                 last_epoch: int = -1):

        def f(step: int) -> float:
            if step < num_warmup_steps:
                return step / max(1, num_warmup_steps)
            p = min((step - num_warmup_steps) / max(1, num_training_steps - num_warmup_steps), 1.0)
            return min_lr_ratio + (1.0 - min_lr_ratio) * (1.0 - p)

        super().__init__(optimizer, f, last_epoch)


class ConstantWarmupScheduler(LambdaLR):

    def __init__(self, optimizer, num_warmup_steps: int = 0, last_epoch: int = -1, **_):
        super().__init__(optimizer, lambda s: min(1.0, s / max(1, num_warmup_steps)) if num_warmup_steps else 1.0, last_epoch)


scheduler_mapping = {
    'cosine': CosineWarmupScheduler, 'linear': LinearWarmupScheduler, 'constant': ConstantWarmupScheduler,
    'CosineWarmupScheduler': CosineWarmupScheduler, 'LinearWarmupScheduler': LinearWarmupScheduler,
    'ConstantWarmupScheduler': ConstantWarmupScheduler,
}


def resolve_scheduler(name: str):
    """A scheduler class by name: the ones of this module first, then any class of ``torch.optim.lr_scheduler`` (reference
    ``model/transformers/transformers.py:975-992`` looks names up in both places)."""
    if name in scheduler_mapping:
        return scheduler_mapping[name]
    import torch.optim.lr_scheduler as tls
    cls = getattr(tls, name, None)
    if isinstance(cls, type) and issubclass(cls, tls.LRScheduler):
        return cls
    raise KeyError(f'unknown lr scheduler {name!r}; known: {sorted(scheduler_mapping)} and the classes of torch.optim.lr_scheduler')
