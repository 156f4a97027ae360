"""Plain next-token cross entropy on materialised logits (reference ``torchure/loss/cross_entropy.py:7-35``)."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def shift_labels(ids: torch.Tensor, ignore_index: int) -> torch.Tensor:
    """labels[t] = ids[t+1]; the last position of every row has no target."""
    labels = torch.full_like(ids, ignore_index)
    labels[:, :-1] = ids[:, 1:]
    return labels


def cross_entropy_loss(ids: torch.Tensor, logits: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    labels = shift_labels(ids, ignore_index)
    return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1),
                           ignore_index=ignore_index)
