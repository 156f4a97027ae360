"""Ulysses sequence parallelism: all-to-all between sequence shards and head shards around attention.

Absent from the reference (its ``all_to_all`` docstring names only redistribution and the EP shuffle); here it is
the second consumer of that primitive.  Each rank holds S/n tokens of all heads; before attention an all-to-all
gives it all S tokens of H/n heads, attention runs unsharded per head, and the inverse all-to-all restores the
sequence sharding.  Both directions are autograd functions whose backward is the opposite exchange.
"""

from __future__ import annotations

import torch

from torchure_b200.core.collective import all_to_all


class _SeqToHead(torch.autograd.Function):
    """(B, S/n, H, d) -> (B, S, H/n, d)"""

    @staticmethod
    def forward(ctx, x, mesh, dim):
        ctx.mesh, ctx.dim = mesh, dim
        return all_to_all(x.contiguous(), mesh, dim, split_dim=2, concat_dim=1)

    @staticmethod
    def backward(ctx, g):
        return all_to_all(g.contiguous(), ctx.mesh, ctx.dim, split_dim=1, concat_dim=2), None, None


class _HeadToSeq(torch.autograd.Function):
    """(B, S, H/n, d) -> (B, S/n, H, d)"""

    @staticmethod
    def forward(ctx, x, mesh, dim):
        ctx.mesh, ctx.dim = mesh, dim
        return all_to_all(x.contiguous(), mesh, dim, split_dim=1, concat_dim=2)

    @staticmethod
    def backward(ctx, g):
        return all_to_all(g.contiguous(), ctx.mesh, ctx.dim, split_dim=2, concat_dim=1), None, None


def ulysses_attention(q, k, v, mesh, dim: str, attn_fn=None):
    """q (B, S/n, Hq, d), k/v (B, S/n, Hkv, d), sequence-sharded in rank order.  `attn_fn(q, k, v)` is any
    full-sequence attention on (B, S, h, d) tensors; the default is causal ``ops.attention.flash_attention``: the
    tcgen05 kernels on Blackwell (bf16, d = 128), SDPA elsewhere.  On GPUs the two exchanges are the NVLink
    all-to-all kernel of ``core.collective``."""
    if attn_fn is None:
        from torchure_b200.ops.attention import flash_attention

        attn_fn = flash_attention
    n = mesh.size(dim)
    assert q.shape[2] % n == 0 and k.shape[2] % n == 0, "head counts must be divisible by the Ulysses degree"
    qh, kh, vh = (_SeqToHead.apply(t, mesh, dim) for t in (q, k, v))
    oh = attn_fn(qh, kh, vh)
    return _HeadToSeq.apply(oh, mesh, dim)
