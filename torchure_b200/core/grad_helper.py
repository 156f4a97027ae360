"""Global L2 gradient-norm measurement and clipping.

``clip_grad_norm`` keeps the reference contract (``torchure/core/grad_helper.py:8-34``):
it returns the PRE-clip norm, scales ``.grad`` in place by
``min(1, max_norm / (norm + 1e-6))``, measures only when ``max_norm is None``, refuses an
empty grad list (so no rank silently skips a collective), and for sharded grads sums the
squared norm over the given mesh axes before the square root.

``grad_norm_and_coef`` is the device-resident variant the trainer uses on GPUs: it returns
the norm and the clip coefficient as 0-d device tensors and leaves the grads untouched;
the fused AdamW kernel multiplies by the coefficient while it reads the grads, so neither
a separate scaling pass nor a host synchronisation happens.
"""

from __future__ import annotations

import torch

from torchure_b200.core.collective import all_reduce

_EPS = 1e-6


def _collect(params) -> list[torch.Tensor]:
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        raise AssertionError("clip_grad_norm got no grads: backward did not run or every param is frozen")
    return grads


def _local_sq_norm(grads: list[torch.Tensor]) -> torch.Tensor:
    if grads[0].is_cuda:
        from torchure_b200.ops import multi_tensor

        if multi_tensor.available():
            return multi_tensor.sq_norm(grads)
    norms = torch._foreach_norm(grads, 2.0)
    return torch.linalg.vector_norm(torch.stack(norms), 2.0).float() ** 2


def _total_norm(grads, mesh, shard_dims, presummed_sq: torch.Tensor | None = None) -> torch.Tensor:
    sq = presummed_sq if presummed_sq is not None else _local_sq_norm(grads)
    for dim in shard_dims:
        all_reduce(sq, mesh, dim, "sum")
    return sq.sqrt()


def grad_norm_and_coef(params, mesh, max_norm, shard_dims=(), presummed_sq=None):
    """Return ``(pre-clip norm, clip coefficient)`` as device scalars; grads are not modified."""
    grads = _collect(params)
    total = _total_norm(grads, mesh, shard_dims, presummed_sq)
    if max_norm is None:
        return total, torch.ones_like(total)
    coef = torch.clamp(max_norm / (total + _EPS), max=1.0)
    return total, coef


def clip_grad_norm(params, mesh, max_norm, shard_dims=()) -> torch.Tensor:
    """Clip grads in place to a global L2 norm of `max_norm`; returns the norm before clipping."""
    grads = _collect(params)
    total = _total_norm(grads, mesh, shard_dims)
    if max_norm is None:
        return total
    coef = torch.clamp(max_norm / (total + _EPS), max=1.0)
    if grads[0].is_cuda:
        from torchure_b200.ops import multi_tensor

        if multi_tensor.available():
            multi_tensor.scale_(grads, coef)
            return total
    torch._foreach_mul_(grads, coef)
    return total
