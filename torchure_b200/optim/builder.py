"""Optimizer / scheduler registries (reference ``torchure/optimizer/builder.py:20-59``).

Parameters are split into two groups: tensors with ``dim >= 2`` take the configured weight
decay, 1-D tensors (norm gains) take none.  Remaining config keys pass straight through.
"""

from __future__ import annotations

import torch.nn as nn
import torch.optim as optim

from torchure_b200.optim.adamw import AdamW
from torchure_b200.optim.scheduler import CosineWithWarmup, WarmupStableDecay

OPTIMIZERS = {"adamw": AdamW, "sgd": optim.SGD}
SCHEDULERS = {"wsd": WarmupStableDecay, "cosine": CosineWithWarmup}


def build_optimizer(model: nn.Module | None, name: str, cfg: dict, params=None) -> optim.Optimizer:
    """`params` overrides ``model.parameters()``: sharded strategies hand in their shard parameters instead."""
    cfg = dict(cfg)
    weight_decay = cfg.pop("weight_decay", 0.0)
    if name == "sgd":
        cfg.pop("betas", None)
        cfg.pop("fused", None)
    params = [p for p in (params if params is not None else model.parameters()) if p.requires_grad]
    groups = [
        {"params": [p for p in params if p.dim() >= 2], "weight_decay": weight_decay},
        {"params": [p for p in params if p.dim() < 2], "weight_decay": 0.0},
    ]
    if name not in OPTIMIZERS:
        raise KeyError(f"unknown optimizer {name!r}; known: {sorted(OPTIMIZERS)}")
    return OPTIMIZERS[name](groups, **cfg)


def build_scheduler(optimizer: optim.Optimizer, cfg: dict):
    cfg = dict(cfg)
    kind = cfg.pop("type")
    if kind not in SCHEDULERS:
        raise KeyError(f"unknown scheduler {kind!r}; known: {sorted(SCHEDULERS)}")
    return SCHEDULERS[kind](optimizer, **cfg)
