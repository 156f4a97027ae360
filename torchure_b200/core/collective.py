"""Mesh-aware collectives: the only module that issues communication.

Callers pass ``(tensor, mesh, axis name)`` and never see a ProcessGroup.  Contracts
(parity with reference ``torchure/core/collective.py:87-363``):

* ops are lowercase strings ``"sum" | "avg" | "max" | "min"``;
* ``all_reduce`` and ``broadcast`` work in place and return their input; ``all_gather``,
  ``reduce_scatter``, ``all_to_all`` and ``ring_send_recv`` return a new tensor;
* a synchronous call returns the tensor, ``async_op=True`` returns ``(tensor, work)`` and
  the tensor may only be read after ``work.wait()``;
* ``broadcast(src=)`` is a coordinate inside the axis group, not a global rank;
* no autograd.

Two transports sit behind the same signatures:

``torch``  ``torch.distributed`` (gloo on CPU, NCCL on CUDA).  Used for CPU tests, for
           bootstrap, for ``ring_send_recv`` and as the measured baseline.
``sm100``  hand-written kernels that load/store peer GPUs' memory over NVLink/NVSwitch
           (plain P2P or ``multimem`` in-switch reduction), chosen per message size.
           Active for CUDA tensors once ``enable_sm100(mesh, dim)`` has attached a
           symmetric-memory communicator to the axis.
"""

from __future__ import annotations

from typing import Literal, Protocol

import torch
import torch.distributed as dist

ReduceOpName = Literal["sum", "avg", "max", "min"]

_TORCH_OPS = {
    "sum": dist.ReduceOp.SUM,
    "avg": dist.ReduceOp.AVG,
    "max": dist.ReduceOp.MAX,
    "min": dist.ReduceOp.MIN,
}


class MeshLike(Protocol):
    def size(self, dim: str) -> int: ...

    def get_group(self, dim: str) -> dist.ProcessGroup: ...

    def coordinate(self, dim: str) -> int: ...


class _Done:
    """Work handle for operations that were already ordered on the current stream."""

    def wait(self) -> bool:
        return True

    def is_completed(self) -> bool:
        return True


# (id(mesh), dim) -> SymmComm; filled by enable_sm100
_SM100: dict[tuple[int, str], object] = {}


def enable_sm100(mesh: MeshLike, dim: str, max_bytes: int = 64 << 20, persistent_bytes: int = 0):
    """Attach a symmetric-memory communicator to `dim`; CUDA collectives then use our kernels.

    Collective over the axis group.  Returns the communicator (None when the axis has one
    rank or the tensor lives on the CPU, in which case the torch transport stays active).
    `persistent_bytes` reserves room for long-lived symmetric tensors (operands of the fused
    GEMM+collective kernels, gradient buckets).
    """
    if mesh.size(dim) == 1 or not torch.cuda.is_available():
        return None
    key = (id(mesh), dim)
    if key not in _SM100:
        from torchure_b200.core.symm import SymmComm

        _SM100[key] = SymmComm(mesh.get_group(dim), mesh.coordinate(dim), mesh.size(dim), max_bytes, persistent_bytes)
    return _SM100[key]


def disable_sm100(mesh: MeshLike, dim: str) -> None:
    _SM100.pop((id(mesh), dim), None)


def _sm100_for(tensor: torch.Tensor, mesh: MeshLike, dim: str):
    if not tensor.is_cuda:
        return None
    return _SM100.get((id(mesh), dim))


def _is_nccl(group) -> bool:
    return dist.get_backend(group) == "nccl"


def _check_op(op: str) -> None:
    if op not in _TORCH_OPS:
        raise ValueError(f"unknown reduce op {op!r}; expected one of {sorted(_TORCH_OPS)}")


def all_reduce(tensor, mesh: MeshLike, dim: str, op: ReduceOpName = "sum", *, async_op: bool = False):
    """Reduce `tensor` over the `dim` group in place; every member ends with the same values."""
    _check_op(op)
    comm = _sm100_for(tensor, mesh, dim)
    if comm is not None and comm.supports(tensor):
        comm.all_reduce_(tensor, op)
        return (tensor, _Done()) if async_op else tensor
    group = mesh.get_group(dim)
    if op == "avg" and not _is_nccl(group):
        # gloo has no AVG: dividing first keeps the call a single (async-capable) sum
        tensor.div_(mesh.size(dim))
        op = "sum"
    work = dist.all_reduce(tensor, _TORCH_OPS[op], group=group, async_op=async_op)
    return (tensor, work) if async_op else tensor


def broadcast(tensor, mesh: MeshLike, dim: str, src: int = 0, *, async_op: bool = False):
    """Overwrite `tensor` on every member with the values held at coordinate `src` of the group."""
    comm = _sm100_for(tensor, mesh, dim)
    if comm is not None and comm.supports(tensor):
        comm.broadcast_(tensor, src)
        return (tensor, _Done()) if async_op else tensor
    group = mesh.get_group(dim)
    work = dist.broadcast(tensor, group=group, group_src=src, async_op=async_op)
    return (tensor, work) if async_op else tensor


def _stacked_output(output_tensor, expected_shape, like: torch.Tensor, axis: int, what: str):
    if output_tensor is None:
        return torch.empty(expected_shape, dtype=like.dtype, device=like.device)
    if axis != 0:
        raise AssertionError(f"a caller-provided output_tensor requires {what}=0, got {axis}")
    if tuple(output_tensor.shape) != tuple(expected_shape):
        raise AssertionError(f"output_tensor shape {tuple(output_tensor.shape)} != {tuple(expected_shape)}")
    if output_tensor.dtype != like.dtype or output_tensor.device != like.device:
        raise AssertionError("output_tensor dtype/device differ from the input's")
    if not output_tensor.is_contiguous():
        raise AssertionError("output_tensor must be contiguous")
    return output_tensor


def all_gather(tensor, mesh: MeshLike, dim: str, gather_dim: int = 0, *, async_op: bool = False,
               output_tensor: torch.Tensor | None = None):
    """Concatenate every member's `tensor` along `gather_dim`, ordered by coordinate."""
    n = mesh.size(dim)
    src = tensor.movedim(gather_dim, 0).contiguous()
    out = _stacked_output(output_tensor, (n * src.shape[0], *src.shape[1:]), tensor, gather_dim, "gather_dim")
    comm = _sm100_for(tensor, mesh, dim)
    if comm is not None and comm.supports(src, copies=comm.world + 0.01):
        comm.all_gather(src, out)
        work = _Done()
    else:
        work = dist.all_gather_into_tensor(out, src, group=mesh.get_group(dim), async_op=async_op)
    res = out.movedim(0, gather_dim)
    return (res, work) if async_op else res


def reduce_scatter(tensor, mesh: MeshLike, dim: str, op: ReduceOpName = "sum", scatter_dim: int = 0, *,
                   async_op: bool = False, output_tensor: torch.Tensor | None = None):
    """Reduce over the group; each member keeps its coordinate-th slice along `scatter_dim`."""
    _check_op(op)
    n = mesh.size(dim)
    if tensor.shape[scatter_dim] % n != 0:
        raise AssertionError(f"shape[{scatter_dim}]={tensor.shape[scatter_dim]} is not divisible by group size {n}")
    src = tensor.movedim(scatter_dim, 0).contiguous()
    out = _stacked_output(output_tensor, (src.shape[0] // n, *src.shape[1:]), tensor, scatter_dim, "scatter_dim")
    comm = _sm100_for(tensor, mesh, dim)
    if comm is not None and comm.supports(src, copies=1.01):
        comm.reduce_scatter(src, out, op)
        res = out.movedim(0, scatter_dim)
        return (res, _Done()) if async_op else res
    group = mesh.get_group(dim)
    if op == "avg" and not _is_nccl(group):
        if async_op:
            raise AssertionError("async 'avg' reduce_scatter needs a backend with ReduceOp.AVG")
        dist.reduce_scatter_tensor(out, src, op=dist.ReduceOp.SUM, group=group)
        out.div_(n)
        return out.movedim(0, scatter_dim)
    work = dist.reduce_scatter_tensor(out, src, op=_TORCH_OPS[op], group=group, async_op=async_op)
    res = out.movedim(0, scatter_dim)
    return (res, work) if async_op else res


def all_to_all(tensor, mesh: MeshLike, dim: str, split_dim: int = 0, concat_dim: int = 0, *,
               async_op: bool = False):
    """Split along `split_dim` into `size` chunks, send chunk j to coordinate j, concatenate the
    received chunks (ordered by sender) along `concat_dim`.  Even splits, synchronous."""
    n = mesh.size(dim)
    if tensor.shape[split_dim] % n != 0:
        raise AssertionError(f"shape[{split_dim}]={tensor.shape[split_dim]} is not divisible by group size {n}")
    if async_op:
        raise AssertionError("all_to_all is synchronous")
    src = tensor.movedim(split_dim, 0).contiguous()
    recv = torch.empty_like(src)
    comm = _sm100_for(tensor, mesh, dim)
    if comm is not None and comm.supports(src, copies=1.01):
        comm.all_to_all(src, recv)
    else:
        dist.all_to_all_single(recv, src, group=mesh.get_group(dim))
    pieces = [c.movedim(0, split_dim) for c in recv.chunk(n, dim=0)]
    return torch.cat(pieces, dim=concat_dim)


def ring_send_recv(tensor, mesh: MeshLike, dim: str, *, async_op: bool = False):
    """Send to coordinate+1 and receive from coordinate-1 (mod size); returns the received tensor.

    Stays on the library transport (NCCL p2p on GPUs): context-parallel attention overlaps
    it with compute by issuing it on a side stream.
    """
    if async_op:
        raise AssertionError("ring_send_recv is synchronous")
    n = mesh.size(dim)
    if n == 1:
        return tensor.clone()
    group = mesh.get_group(dim)
    me = mesh.coordinate(dim)
    nxt = dist.get_global_rank(group, (me + 1) % n)
    prv = dist.get_global_rank(group, (me - 1) % n)
    out_buf = tensor.contiguous()
    in_buf = torch.empty_like(out_buf)
    ops = [dist.P2POp(dist.isend, out_buf, nxt, group=group), dist.P2POp(dist.irecv, in_buf, prv, group=group)]
    for req in dist.batch_isend_irecv(ops):
        req.wait()
    return in_buf


def send_recv(send: torch.Tensor | None, recv: torch.Tensor | None, mesh: MeshLike, dim: str,
              dst: int | None = None, src: int | None = None) -> torch.Tensor | None:
    """Directed point-to-point exchange inside the `dim` group (pipeline stages).

    `dst`/`src` are coordinates in the group.  Either side may be None.
    """
    group = mesh.get_group(dim)
    ops = []
    if send is not None and dst is not None:
        ops.append(dist.P2POp(dist.isend, send.contiguous(), dist.get_global_rank(group, dst), group=group))
    if recv is not None and src is not None:
        ops.append(dist.P2POp(dist.irecv, recv, dist.get_global_rank(group, src), group=group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return recv


def isend(tensor: torch.Tensor, mesh: MeshLike, dim: str, dst: int):
    """Start sending `tensor` to coordinate `dst` of the `dim` group; returns a work handle to ``wait()`` on later.
    The tensor must stay alive and unmodified until then (pipeline schedules post sends and move on)."""
    group = mesh.get_group(dim)
    return dist.isend(tensor.contiguous(), dist.get_global_rank(group, dst), group=group)


def recv(tensor: torch.Tensor, mesh: MeshLike, dim: str, src: int) -> torch.Tensor:
    """Blocking receive into `tensor` from coordinate `src` of the `dim` group."""
    group = mesh.get_group(dim)
    dist.recv(tensor, dist.get_global_rank(group, src), group=group)
    return tensor


def barrier(mesh: MeshLike | None = None, dim: str | None = None) -> None:
    """Block until every rank of the `dim` group (the world without a mesh) has arrived."""
    dist.barrier(group=None if mesh is None else mesh.get_group(dim))
