"""Autoregressive next-token objective (reference ``torchure/objectives/autoregressive.py:16-47``)."""

from __future__ import annotations

import torch

from torchure_b200.loss import cross_entropy_loss, fused_linear_cross_entropy, shift_labels


class ARObjective:
    def __init__(self, ignore_index: int = -100, fused_linear_ce: bool = True, ce_chunk_size: int = 4096):
        self.ignore_index = ignore_index
        self.fused_linear_ce = fused_linear_ce
        self.ce_chunk_size = ce_chunk_size

    def compute_loss(self, model, batch: dict[str, torch.Tensor], loss_scale: float = 1.0) -> torch.Tensor:
        """Mean next-token CE times `loss_scale` (1/micro-batches under gradient accumulation: folding it here
        keeps the loss the root of backward, which the fused gradient paths rely on)."""
        if self.fused_linear_ce:
            hidden = model(batch["input_ids"], return_final_hidden=True)
            labels = shift_labels(batch["labels"], self.ignore_index)
            return fused_linear_cross_entropy(hidden, model.lm_head.weight, labels, self.ignore_index,
                                              self.ce_chunk_size, loss_scale)
        logits = model(batch["input_ids"])
        loss = cross_entropy_loss(batch["labels"], logits, self.ignore_index)
        return loss if loss_scale == 1.0 else loss * loss_scale
