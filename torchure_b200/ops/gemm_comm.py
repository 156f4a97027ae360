"""Fused tensor-core GEMM + NVLink collective (one kernel each).

``ag_gemm``   all-gather -> GEMM.  Every rank holds a row block ``A_r`` of the activation in the symmetric
              allocation; the kernel computes ``concat_r(A_r) @ B^T``.  Copy warps in its CTAs push this rank's shard
              over NVLink into the gathered copy of every rank (one ``multimem.st`` through the switch, or a posted
              store per peer) while the tensor cores already work on the rows this rank owns; a tile on remote rows
              starts as soon as the owner's arrival words for its row block are set.  The
              gathered copy is returned too (the backward pass needs it for the weight gradient).  (FSDP parameter
              all-gather fused into the first consuming GEMM: pass the weight shard as ``A`` and the activation as
              ``B`` to get the transposed product.)
``gemm_rs``   GEMM -> reduce-scatter.  Every rank multiplies its K-slice (``A [M, K/n] @ B [N, K/n]^T``) and the
              epilogue adds each fp32 tile into the row block of the rank that owns it with TMA reduce-add over
              NVLink; after the kernel rank r holds ``sum_ranks(partial)[rows of r]``.  (Row-parallel TP output, FSDP
              gradient reduce-scatter.)

Both handshake with the same CTA index on every peer before touching remote memory and after the last remote access
(bounded waits, status word on expiry).  Operands are bf16, ``M`` must be a multiple of ``128 * world``.
"""

from __future__ import annotations

import torch

from torchure_b200 import ops


class SymmetricOperand:
    """A tensor allocated inside a communicator's symmetric region (same offset on every rank)."""

    def __init__(self, comm, shape, dtype):
        self.comm = comm
        numel = 1
        for s in shape:
            numel *= s
        self.tensor = comm.alloc(numel, dtype).view(*shape)
        self.offset = comm.offset_of(self.tensor)


def ag_gemm(comm, a_shard: SymmetricOperand, b: torch.Tensor, out: torch.Tensor | None = None,
            gathered: SymmetricOperand | None = None, return_gathered: bool = False, b_mn: bool = False):
    """out[M, N] = concat_ranks(a_shard)[M, K] @ b[N, K]^T, bf16 (`b_mn`: b is stored [K, N] and used untransposed).

    `gathered` ([M, K], symmetric: every rank pushes its shard into every rank's copy) receives the assembled A; one
    is allocated per (M, K) and kept on the communicator when none is passed.
    """
    rows, K = a_shard.tensor.shape
    M = rows * comm.world
    if out is None:
        out = torch.empty(M, b.shape[1] if b_mn else b.shape[0], dtype=torch.bfloat16, device=b.device)
    if gathered is None:
        cache = comm.__dict__.setdefault("_ag_gathered", {})
        if (M, K) not in cache:
            cache[(M, K)] = SymmetricOperand(comm, (M, K), torch.bfloat16)
        gathered = cache[(M, K)]
    comm.ag_epoch = getattr(comm, "ag_epoch", 0) + 1
    ops.ext().ag_gemm(*comm._ctx(), a_shard.offset, gathered.offset, comm.ag_epoch, b, out, M, K, b_mn)
    ops.count_launch()
    return (out, gathered.tensor) if return_gathered else out


def gemm_rs(comm, a: torch.Tensor, b: torch.Tensor, out_shard: SymmetricOperand, b_mn: bool = False) -> torch.Tensor:
    """out_shard[M/world, N] (fp32, zeroed here) = rows of this rank of sum_ranks(a @ b^T) (`b_mn`: b stored [K, N])."""
    out_shard.tensor.zero_()
    ops.ext().gemm_rs(*comm._ctx(), a, b, out_shard.offset, b_mn)
    ops.count_launch()
    return out_shard.tensor
