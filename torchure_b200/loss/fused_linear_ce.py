"""Chunked fused linear + cross-entropy: never holds the (N, V) logits of the whole batch.

Semantics are ``F.cross_entropy(hidden @ weight.T, labels, ignore_index, reduction="mean")``
with the divisor clamped to at least 1 (reference ``torchure/loss/fused_linear_ce.py:63-136``).
Gradients w.r.t. ``hidden`` and ``weight`` are produced during the forward pass, one row
chunk at a time, and only rescaled by ``grad_out / n_valid`` in backward, so a chunk's
logits die before the next chunk starts.

On CUDA with the sm_100a extension the three GEMMs per chunk are tcgen05 kernels and the
softmax / target-gather / loss / dlogits step is one fused kernel that rewrites the bf16
logits in place with the bf16 gradient (``torchure_b200/ops/linear_ce.py``).  The code
below is the plain PyTorch statement of the same algorithm (CPU path and test oracle).
"""

from __future__ import annotations

import torch


def _chunk_torch(h: torch.Tensor, w: torch.Tensor, y: torch.Tensor, ignore_index: int):
    logits = (h @ w.t()).float()
    keep = y != ignore_index
    tgt = torch.where(keep, y, torch.zeros_like(y))
    lse = torch.logsumexp(logits, dim=-1)
    picked = logits.gather(1, tgt[:, None]).squeeze(1)
    loss_sum = torch.where(keep, lse - picked, torch.zeros_like(lse)).sum()
    dlogits = torch.exp(logits - lse[:, None])
    dlogits[torch.arange(h.shape[0], device=h.device), tgt] -= 1.0
    dlogits = (dlogits * keep[:, None]).to(h.dtype)
    return loss_sum, dlogits @ w, dlogits.t() @ h


def vocab_slice(vocab: int, mesh, dim: str) -> tuple[int, int]:
    """(first row, rows) of the head weight that this rank of `dim` owns under a vocabulary-parallel loss."""
    n = mesh.size(dim)
    assert vocab % n == 0, f"vocabulary {vocab} is not divisible by the {dim!r} axis ({n})"
    return mesh.coordinate(dim) * (vocab // n), vocab // n


def _chunk_torch_vocab_parallel(h, w_local, y, ignore_index, v0, mesh, dim):
    """One chunk with the vocabulary sharded over `dim`: this rank's logits cover rows [v0, v0 + len(w_local)) of the
    head.  Two all-reduces over (chunk,)-sized fp32 vectors: the row maxima, then the sums of exponentials packed with
    the target logits; the (chunk, V) logits never exist on any rank."""
    from torchure_b200.core.collective import all_reduce

    logits = (h @ w_local.t()).float()
    keep = y != ignore_index
    mine = keep & (y >= v0) & (y < v0 + w_local.shape[0])
    idx = torch.where(mine, y - v0, torch.zeros_like(y))
    mx = logits.max(dim=-1).values
    all_reduce(mx, mesh, dim, "max")
    ex = torch.exp(logits - mx[:, None])
    tgt = torch.where(mine, logits.gather(1, idx[:, None]).squeeze(1), torch.zeros_like(mx))
    packed = torch.stack([ex.sum(-1), tgt])
    all_reduce(packed, mesh, dim, "sum")
    loss_sum = torch.where(keep, torch.log(packed[0]) + mx - packed[1], torch.zeros_like(mx)).sum()
    dlogits = ex / packed[0][:, None]
    rows = torch.arange(h.shape[0], device=h.device)[mine]
    dlogits[rows, idx[mine]] -= 1.0
    dlogits = (dlogits * keep[:, None]).to(h.dtype)
    return loss_sum, dlogits @ w_local, dlogits.t() @ h


class _LinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, chunk_size, normalizer=None, vocab_parallel=None):
        n = hidden.shape[0]
        loss_sum = torch.zeros((), dtype=torch.float32, device=hidden.device)
        d_hidden = torch.empty_like(hidden)
        d_weight = torch.zeros_like(weight, dtype=torch.float32) if weight.requires_grad else None
        if vocab_parallel is not None:
            v0, rows = vocab_slice(weight.shape[0], *vocab_parallel)
            w = weight[v0:v0 + rows].to(hidden.dtype)
        else:
            w = weight.to(hidden.dtype)
        for lo in range(0, n, chunk_size):
            hi = min(n, lo + chunk_size)
            if vocab_parallel is not None:
                ls, dh, dw = _chunk_torch_vocab_parallel(hidden[lo:hi], w, labels[lo:hi], ignore_index, v0,
                                                         *vocab_parallel)
            else:
                ls, dh, dw = _chunk_torch(hidden[lo:hi], w, labels[lo:hi], ignore_index)
            loss_sum += ls
            d_hidden[lo:hi] = dh
            if d_weight is not None:
                (d_weight if vocab_parallel is None else d_weight[v0:v0 + rows]).add_(dw)
        if vocab_parallel is not None:
            # every rank holds the contribution of its vocabulary rows to dL/dhidden; the rows of d_weight outside the
            # rank's slice stay zero (the caller gathers the slices once per step)
            from torchure_b200.core.collective import all_reduce

            all_reduce(d_hidden, *vocab_parallel, "sum")
        n_valid = (labels != ignore_index).sum().clamp_min(1) if normalizer is None else normalizer
        ctx.stash = (d_hidden, d_weight, n_valid)
        ctx.weight_dtype = weight.dtype
        return loss_sum / n_valid

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.stash is None:
            raise RuntimeError("fused_linear_cross_entropy: backward ran twice; its grads are consumed in place")
        d_hidden, d_weight, n_valid = ctx.stash
        ctx.stash = None
        scale = grad_out / n_valid
        d_hidden.mul_(scale.to(d_hidden.dtype))
        if d_weight is not None:
            d_weight.mul_(scale)
            d_weight = d_weight.to(ctx.weight_dtype)
        return d_hidden, d_weight, None, None, None, None, None


def fused_linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                               ignore_index: int = -100, chunk_size: int = 1024, loss_scale: float = 1.0,
                               normalizer: torch.Tensor | None = None, vocab_parallel=None) -> torch.Tensor:
    """hidden (B,S,D) or (N,D); weight (V,D); labels already shifted, (B,S) or (N,).  Returns mean CE * loss_scale
    (the scale is folded into the gradients that are computed during the forward pass).  `normalizer` (a 0-d device
    tensor) replaces the count of valid labels as the divisor: a rank that holds only part of every sequence divides
    by its share of the global count, so that averaging the ranks' losses and gradients gives the global mean.

    `vocab_parallel` = (mesh, axis): the loss-parallel form for tensor parallelism.  `hidden` and `weight` are
    replicated over the axis; every rank computes the logits of ITS V/n rows of the head only, and inside each chunk
    the ranks combine row maxima, sums of exponentials and target logits with two small all-reduces.  The returned
    loss and dL/dhidden are complete on every rank; dL/dweight is complete in the rank's rows and zero elsewhere, so
    the owner of the step gathers the row slices over the axis before the optimizer (``Trainer`` does)."""
    if hidden.dim() == 3:
        hidden = hidden.reshape(-1, hidden.shape[-1])
        labels = labels.reshape(-1)
    if hidden.is_cuda:
        from torchure_b200 import ops

        if ops.available():
            from torchure_b200.ops.linear_ce import linear_ce_sm100

            return linear_ce_sm100(hidden, weight, labels, ignore_index, chunk_size, loss_scale, normalizer,
                                   vocab_parallel)
    loss = _LinearCE.apply(hidden, weight, labels, ignore_index, chunk_size, normalizer, vocab_parallel)
    return loss if loss_scale == 1.0 else loss * loss_scale
