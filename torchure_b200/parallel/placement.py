"""Placement bookkeeping for sharded tensors (a deliberately small stand-in for DTensor).

Roadmap-only in the reference: "a bookkeeping wrapper with an explicit redistribute table, no __torch_dispatch__".
``ShardedTensor`` records how a logical tensor is laid out along ONE mesh axis (``Replicate`` or ``Shard(d)``) and
``redistribute`` moves between layouts with exactly one collective from the table below.

    Replicate -> Shard(d)        local slice (no communication)
    Shard(d)  -> Replicate       all_gather(gather_dim=d)
    Shard(i)  -> Shard(j)        all_to_all(split_dim=j, concat_dim=i)
    Partial   -> Replicate       all_reduce(sum)
    Partial   -> Shard(d)        reduce_scatter(scatter_dim=d)
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from torchure_b200.core.collective import all_gather, all_reduce, all_to_all, reduce_scatter


@dataclass(frozen=True)
class Replicate:
    pass


@dataclass(frozen=True)
class Shard:
    dim: int


@dataclass(frozen=True)
class Partial:
    """Every rank holds a full-shape addend of the logical tensor."""


class ShardedTensor:
    def __init__(self, local: torch.Tensor, mesh, axis: str, placement):
        self.local, self.mesh, self.axis, self.placement = local, mesh, axis, placement

    @classmethod
    def from_full(cls, full: torch.Tensor, mesh, axis: str, placement):
        if isinstance(placement, Shard):
            n, r = mesh.size(axis), mesh.coordinate(axis)
            assert full.shape[placement.dim] % n == 0
            return cls(full.chunk(n, dim=placement.dim)[r].contiguous(), mesh, axis, placement)
        return cls(full, mesh, axis, placement)

    def redistribute(self, target) -> "ShardedTensor":
        src = self.placement
        m, a = self.mesh, self.axis
        if src == target:
            return self
        if isinstance(src, Replicate) and isinstance(target, Shard):
            return ShardedTensor.from_full(self.local, m, a, target)
        if isinstance(src, Shard) and isinstance(target, Replicate):
            return ShardedTensor(all_gather(self.local, m, a, src.dim), m, a, target)
        if isinstance(src, Shard) and isinstance(target, Shard):
            return ShardedTensor(all_to_all(self.local, m, a, split_dim=target.dim, concat_dim=src.dim), m, a, target)
        if isinstance(src, Partial) and isinstance(target, Replicate):
            return ShardedTensor(all_reduce(self.local.clone(), m, a, "sum"), m, a, target)
        if isinstance(src, Partial) and isinstance(target, Shard):
            return ShardedTensor(reduce_scatter(self.local, m, a, "sum", target.dim), m, a, target)
        raise ValueError(f"no redistribution from {src} to {target}")

    def full(self) -> torch.Tensor:
        return self.redistribute(Replicate()).local
