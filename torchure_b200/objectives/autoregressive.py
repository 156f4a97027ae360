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
        cp = getattr(model, "cp", None)
        if cp is not None:
            return self._compute_loss_cp(model, batch, loss_scale, *cp)
        coef = getattr(model, "aux_loss_coef", 0.0)
        if coef:      # mixture-of-experts model: add the routers' load-balancing term of this forward pass
            return self._lm_loss(model, batch, loss_scale) + (coef * loss_scale) * model.aux_loss()
        return self._lm_loss(model, batch, loss_scale)

    def eval_loss(self, model, batch: dict[str, torch.Tensor]) -> torch.Tensor:
        """The language-model loss alone (no auxiliary terms), for held-out evaluation."""
        cp = getattr(model, "cp", None)
        if cp is not None:
            return self._compute_loss_cp(model, batch, 1.0, *cp)
        return self._lm_loss(model, batch, 1.0)

    def _lm_loss(self, model, batch, loss_scale: float) -> torch.Tensor:
        if self.fused_linear_ce:
            hidden = model(batch["input_ids"], return_final_hidden=True)
            labels = shift_labels(batch["labels"], self.ignore_index)
            # (mesh, axis) when the run asked for a loss-parallel head over its tensor-parallel axis
            return fused_linear_cross_entropy(hidden, model.lm_head.weight, labels, self.ignore_index,
                                              self.ce_chunk_size, loss_scale,
                                              vocab_parallel=getattr(model, "vocab_parallel", None))
        logits = model(batch["input_ids"])
        loss = cross_entropy_loss(batch["labels"], logits, self.ignore_index)
        return loss if loss_scale == 1.0 else loss * loss_scale

    def loss_from_output(self, out: torch.Tensor, head_weight: torch.Tensor, label_ids: torch.Tensor) -> torch.Tensor:
        """Mean next-token CE from what the last pipeline stage produced: the normalised hidden state when the head
        is fused into the loss (``fused_linear_ce``), logits otherwise."""
        if self.fused_linear_ce:
            labels = shift_labels(label_ids, self.ignore_index)
            return fused_linear_cross_entropy(out, head_weight, labels, self.ignore_index, self.ce_chunk_size)
        return cross_entropy_loss(label_ids, out, self.ignore_index)

    def _compute_loss_cp(self, model, batch, loss_scale, mesh, dim) -> torch.Tensor:
        """Context parallelism: every rank of the axis receives the whole batch, keeps its part of every sequence
        (two zigzag chunks for ring attention, one contiguous chunk for Ulysses; tokens and the already shifted
        targets alike) and divides its summed loss by 1/n of the GLOBAL target
        count, so that the average over the axis (which the gradient reduction takes anyway) is the mean over all
        targets whatever the chunks' own counts are."""
        import torch.nn.functional as F

        from torchure_b200.parallel.context_parallel import zigzag_split

        n, r = mesh.size(dim), mesh.coordinate(dim)
        full = shift_labels(batch["labels"], self.ignore_index)
        normalizer = (full != self.ignore_index).sum().clamp_min(1).float() / n
        if getattr(model, "cp_kind", "ring") == "ulysses":
            ids, labels = batch["input_ids"].chunk(n, dim=1)[r].contiguous(), full.chunk(n, dim=1)[r].contiguous()
        else:
            ids, labels = zigzag_split(batch["input_ids"], n, r).contiguous(), zigzag_split(full, n, r).contiguous()
        if self.fused_linear_ce:
            hidden = model(ids, return_final_hidden=True)
            return fused_linear_cross_entropy(hidden, model.lm_head.weight, labels, self.ignore_index,
                                              self.ce_chunk_size, loss_scale, normalizer)
        logits = model(ids)
        total = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1),
                                ignore_index=self.ignore_index, reduction="sum")
        return total * (loss_scale / normalizer)
