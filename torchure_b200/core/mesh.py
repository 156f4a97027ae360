"""Named device mesh over the flat rank space.

A mesh is an ordered mapping ``axis name -> size`` whose product equals the world size.
Ranks are laid out row-major with the LAST axis varying fastest, so on one NVSwitch node
the innermost axis gets neighbouring GPUs.  Every axis owns one process group per
"line" of the grid; a rank keeps the group it belongs to.  ``flatten`` registers a
virtual axis that spans several real axes (HSDP's ``dp = dp_replicate x dp_shard``).

Behavioural parity: reference ``torchure/core/mesh.py:8-114`` (spec assert, row-major
strides, every rank creates every group, flatten with spec-order check).

Each axis can additionally carry a symmetric-memory communicator (peer pointers and an
NVSwitch multicast mapping) used by the sm_100a collectives; see ``core/symm.py``.
"""

from __future__ import annotations

import itertools
import math

import torch
import torch.distributed as dist


class Mesh:
    def __init__(self, spec: dict[str, int]):
        if not dist.is_initialized():
            raise AssertionError("init_process_group() must run before a Mesh is built")
        self.world_size = dist.get_world_size()
        self.rank = dist.get_rank()
        spec = {str(k): int(v) for k, v in spec.items()}
        total = math.prod(spec.values())
        if total != self.world_size:
            raise AssertionError(f"mesh {spec} covers {total} ranks, world size is {self.world_size}")
        self.sizes: dict[str, int] = dict(spec)
        self._real_axes: tuple[str, ...] = tuple(spec)
        # stride of an axis = number of ranks one step along it skips
        self.strides: dict[str, int] = {}
        acc = 1
        for name in reversed(self._real_axes):
            self.strides[name] = acc
            acc *= spec[name]
        self._coords: dict[str, int] = {
            name: (self.rank // self.strides[name]) % spec[name] for name in self._real_axes
        }
        self.groups: dict[str, dist.ProcessGroup] = {}
        self._members: dict[str, list[int]] = {}
        for name in self._real_axes:
            self._make_groups(name, (name,))

    # -- group construction ------------------------------------------------------------
    def _lines(self, axes: tuple[str, ...]):
        """Yield, in an order identical on every rank, the rank lists that vary only along `axes`."""
        fixed = [a for a in self._real_axes if a not in axes]
        fixed_ranges = [range(self.sizes[a]) for a in fixed]
        moving_ranges = [range(self.sizes[a]) for a in axes]
        for fixed_idx in itertools.product(*fixed_ranges):
            base = sum(i * self.strides[a] for i, a in zip(fixed_idx, fixed))
            yield [
                base + sum(i * self.strides[a] for i, a in zip(mv, axes))
                for mv in itertools.product(*moving_ranges)
            ]

    @staticmethod
    def _world_timeout():
        """The timeout the world group was initialised with; axis groups inherit it, so that a rank that stops
        joining collectives ends its peers' next collective after that bound instead of the library default
        (tens of minutes).  None when the backend does not expose it."""
        try:
            pg = dist.distributed_c10d._get_default_group()
            dev = torch.device("cuda" if dist.get_backend(pg) == "nccl" else "cpu")
            return pg._get_backend(dev).options._timeout
        except Exception:
            return None

    def _make_groups(self, name: str, axes: tuple[str, ...]) -> None:
        # new_group is collective: all ranks create all groups, in the same order
        timeout = self._world_timeout()
        for members in self._lines(axes):
            group = dist.new_group(members, timeout=timeout) if timeout is not None else dist.new_group(members)
            if self.rank in members:
                self.groups[name] = group
                self._members[name] = members

    def flatten(self, axes: tuple[str, ...], name: str) -> None:
        """Register virtual axis `name` = row-major product of real `axes` (given in spec order)."""
        axes = tuple(axes)
        if not axes or len(set(axes)) != len(axes):
            raise AssertionError(f"bad axes {axes}")
        for a in axes:
            if a not in self._real_axes:
                raise AssertionError(f"unknown (or virtual) axis {a!r}")
        in_spec_order = tuple(a for a in self._real_axes if a in axes)
        if axes != in_spec_order:
            raise AssertionError(f"{axes} must follow spec order {in_spec_order}")
        if name in self.sizes:
            raise AssertionError(f"axis {name!r} already exists")
        self._make_groups(name, axes)
        self.sizes[name] = math.prod(self.sizes[a] for a in axes)
        # members are enumerated row-major over `axes`, so the index is the flat coordinate
        self._coords[name] = self._members[name].index(self.rank)

    # -- queries -----------------------------------------------------------------------
    def size(self, dim: str) -> int:
        return self.sizes[dim]

    def get_group(self, dim: str) -> dist.ProcessGroup:
        return self.groups[dim]

    def coordinate(self, dim: str) -> int:
        return self._coords[dim]

    def members(self, dim: str) -> list[int]:
        """Global ranks of my `dim` group, ordered by coordinate."""
        return list(self._members[dim])

    def axes(self) -> tuple[str, ...]:
        return self._real_axes

    def __repr__(self) -> str:
        return f"Mesh({self.sizes}, rank={self.rank}, coords={self._coords})"
