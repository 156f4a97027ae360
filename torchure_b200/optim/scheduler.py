"""Learning-rate schedules.

``WarmupStableDecay`` reproduces reference ``torchure/optimizer/scheduler.py:10-35``: with
``W = max(1, round(total * warmup_ratio))`` and ``D0 = total * (1 - decay_ratio)``, the lr
used by (0-based) optimizer step k is ``base * (k+1)/W`` for ``k < W``,
``base * max(0, 1 - (k - D0) / (decay_ratio * total))`` for ``k >= D0`` and ``base`` between.
``last_epoch`` is the step index, so ``state_dict()`` interchanges with the reference.

``CosineWithWarmup`` is a working cosine schedule (the reference's is a stub that returns 0).
"""

from __future__ import annotations

import math

from torch.optim.lr_scheduler import LRScheduler


def wsd_scale(step: int, total_steps: int, warmup_ratio: float, decay_ratio: float) -> float:
    warmup = max(1, round(total_steps * warmup_ratio))
    decay_from = total_steps * (1 - decay_ratio)
    if step < warmup:
        return (step + 1) / warmup
    if step >= decay_from:
        return max(0.0, 1.0 - (step - decay_from) / (decay_ratio * total_steps))
    return 1.0


class WarmupStableDecay(LRScheduler):
    def __init__(self, optimizer, total_steps: int, warmup_ratio: float, decay_ratio: float, last_epoch: int = -1):
        self.total_steps = total_steps
        self.warmup_ratio = warmup_ratio
        self.decay_ratio = decay_ratio
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        s = wsd_scale(self.last_epoch, self.total_steps, self.warmup_ratio, self.decay_ratio)
        return [base * s for base in self.base_lrs]


def cosine_scale(step: int, total_steps: int, warmup_ratio: float, min_ratio: float) -> float:
    warmup = max(1, round(total_steps * warmup_ratio))
    if step < warmup:
        return (step + 1) / warmup
    span = max(1, total_steps - warmup)
    t = min(1.0, (step - warmup) / span)
    return min_ratio + (1.0 - min_ratio) * 0.5 * (1.0 + math.cos(math.pi * t))


class CosineWithWarmup(LRScheduler):
    def __init__(self, optimizer, total_steps: int, warmup_ratio: float = 0.0, min_ratio: float = 0.0,
                 last_epoch: int = -1):
        self.total_steps = total_steps
        self.warmup_ratio = warmup_ratio
        self.min_ratio = min_ratio
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        s = cosine_scale(self.last_epoch, self.total_steps, self.warmup_ratio, self.min_ratio)
        return [base * s for base in self.base_lrs]


# the reference spells the class name with a typo; keep an alias so configs and pickles resolve
WarmupStableDecaySchedulder = WarmupStableDecay
