"""Fused gradient-bucket reducer for DDP on sm_100a.

All buckets are slices of ONE fp32 main-gradient buffer.  With more than one rank that buffer lives in the
symmetric allocation of the dp axis, so peers read and write it directly over NVLink.

Gradients reach a bucket in one of two ways:

* **sink** (models that run on the sm_100a engine): the wgrad GEMM epilogue, the norm-gain kernels and the fused
  linear+CE write their fp32 results STRAIGHT into the bucket slice (``grad_dest`` / ``grad_written``).  The first
  write of a step stores, later micro-batches accumulate through the TMA reduce-add epilogue, so the bf16->fp32
  cast, the no_sync accumulation and the placement into the flat buffer cost no kernel and no extra HBM pass.
* **hook** (any other parameter): the post-accumulate-grad hook copies or adds the autograd gradient into the slice
  (``absorb``).

When the last gradient of a bucket has arrived in the sync micro-batch, ONE kernel on the communication stream
all-reduces it: every rank reduces its 1/world slice with ``multimem.ld_reduce`` (NVSwitch in-fabric reduction; peer
loads without a multicast mapping), applies the 1/world scale, publishes the slice's sum of squares into every rank's
partial table and broadcasts the slice with ``multimem.st``.  No NCCL call, no separate scale or norm kernel.
``sq_norm()`` sums the partial table in a fixed order, so every rank derives bit-identical clip coefficients; with one
rank it is a single multi-tensor reduction over the flat buffer.  After a sync launch ``p.grad`` is a view of the bucket.

The communication kernel needs almost no shared memory and few registers, so its CTAs become resident NEXT TO the
persistent GEMM CTAs (one per SM, shared-memory bound) instead of waiting for them; ``sm_reserve`` > 0 additionally
keeps that many SMs free of GEMM CTAs (``ops.set_compute_sm_reserve``) for fabrics where co-residency is not enough.
"""

from __future__ import annotations

import torch

from torchure_b200 import ops
from torchure_b200.ops import multi_tensor


class FusedReducer:
    fused = True

    def __init__(self, ddp, comm_sms: int = 16, sm_reserve: int = 0):
        self.ddp = ddp
        self.world = ddp.group_size
        dev = ddp.buckets[0].params[0].device
        # 64-element alignment keeps every bucket 256-byte aligned and 16-byte divisible per rank
        offs, total = [], 0
        for b in ddp.buckets:
            offs.append(total)
            total += (b.numel + 63) // 64 * 64
        self.comm = None
        self.embed_rows = self.embed_ids = None
        if self.world > 1:
            from torchure_b200.core.symm import SymmComm

            table = ddp.early_table
            extra = 0
            if table is not None:
                extra = ddp.embed_tokens * (table.shape[1] * 4 + 8) + 1024
            self.comm = SymmComm(ddp.mesh.get_group(ddp.dim), ddp.mesh.coordinate(ddp.dim), self.world,
                                 staging_bytes=4096, persistent_bytes=total * 4 + 4096 + extra)
            self.comm_sms = comm_sms
            self.flat = self.comm.alloc(total, torch.float32)
            self.flat.zero_()
            self.flat_tail = self.comm.alloc(4, torch.float32)     # the step's loss, averaged in place over the ranks
            self.flat_tail.zero_()
            # one slot of sum-of-squares partials per bucket, plus one for the embedding-row exchange's correction
            self.partials = self.comm.partials(len(ddp.buckets) + 1)
            self.partials.zero_()
            if table is not None:
                self.embed_rows = self.comm.alloc(ddp.embed_tokens * table.shape[1], torch.float32)
                self.embed_ids = self.comm.alloc(ddp.embed_tokens, torch.int64)
                self.embed_ids_all = torch.empty(self.world * ddp.embed_tokens, dtype=torch.int64, device=dev)
            self.stream = torch.cuda.Stream(device=dev, priority=-1)
            ops.set_compute_sm_reserve(sm_reserve)
        else:
            self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
            self.partials = None
            self.stream = None
        self.padded = []
        self._view_of: dict[torch.Tensor, torch.Tensor] = {}
        for b, off in zip(ddp.buckets, offs):
            b.bind(self.flat[off:off + b.numel])
            self.padded.append(self.flat[off:off + (b.numel + 63) // 64 * 64])
            for p, v in zip(b.params, b.views):
                self._view_of[p] = v
        self._written: set[int] = set()
        self._table_done: torch.cuda.Event | None = None

    # -- sink API: the producer writes into the bucket itself ------------------------------------------------
    def grad_dest(self, p: torch.Tensor) -> tuple[torch.Tensor, bool]:
        """(fp32 destination shaped like p, accumulate?) for the gradient of `p` in this backward."""
        return self._view_of[p], id(p) in self._written

    def grad_written(self, p: torch.Tensor) -> None:
        """The gradient of `p` for this micro-batch is in its destination (the writes are ordered on the
        current stream)."""
        self._written.add(id(p))
        self.ddp._count_down(p)

    # -- tied embedding / head bucket: reduce early, exchange the embedding rows afterwards ---------------------
    # The tied gradient is dW_head (complete when the loss head's backward ends, before any block runs backward)
    # plus at most one row per token from the embedding lookup (known only after the LAST kernel of backward).  An
    # all-reduce is linear, so the big dense part is launched at once and hides under the whole backward; the rows
    # are exchanged at the end: every rank leaves its (ids, rows) in symmetric memory and adds ALL ranks' rows,
    # scaled by 1/world, into its reduced bucket with the deterministic scatter kernel (same order of additions on
    # every rank, so the replicas keep identical bits).
    def early_table(self, p: torch.Tensor) -> bool:
        """True when `p` is the tied table, the exchange is configured and this micro-batch synchronises."""
        return self.embed_rows is not None and p is self.ddp.early_table and self.ddp.requires_sync

    def embed_rows_dest(self, M: int, D: int) -> torch.Tensor:
        assert M * D <= self.embed_rows.numel(), (
            f"{M} tokens per micro-batch exceed ddp.embed_tokens = {self.ddp.embed_tokens}")
        return self.embed_rows[: M * D].view(M, D)

    def exchange_embedding(self, ids: torch.Tensor, table: torch.Tensor) -> None:
        """`embed_rows_dest` holds this rank's embedding-row gradients for tokens `ids`; the table's bucket was
        launched by ``grad_written(table)`` when the loss head finished."""
        from torchure_b200.ops import kernels as K

        M = ids.numel()
        done = self._table_done
        assert done is not None, "the tied bucket must have been launched before the embedding rows are exchanged"
        torch.cuda.current_stream().wait_event(done)       # the bucket holds avg(dW_head) now
        self.embed_ids[:M].copy_(ids.reshape(-1))
        self.comm.barrier(phase=2)                          # every rank's rows and ids are in place
        ro, io = self.comm.offset_of(self.embed_rows), self.comm.offset_of(self.embed_ids)
        sources = [(self.comm.peers[p] + io, self.comm.peers[p] + ro) for p in range(self.world)]
        K.embedding_scatter_(sources, self._view_of[table], M, scale=1.0 / self.world,
                             sq_delta=self.partials[len(self.ddp.buckets)], blocks=592, ids_scratch=self.embed_ids_all)
        self.comm.barrier(phase=3)                          # nobody reads my rows any more
        ops.count_launch(2)
        self._table_done = None

    # -- hook path: a gradient arrived through autograd -------------------------------------------------------
    def absorb(self, p: torch.Tensor) -> bool:
        """Move an autograd-delivered gradient into its slice.  Returns False when there is none (``p.grad`` is
        unset or already the slice itself), which is what a hook sees for a parameter served by the sink."""
        g, v = p.grad, self._view_of[p]
        if g is None or g.data_ptr() == v.data_ptr():
            return False
        if id(p) in self._written:
            v.add_(g)
        else:
            v.copy_(g)
        self._written.add(id(p))
        return True

    def launch(self, b, sync: bool):
        if not sync:
            for p in b.params:
                p.grad = None  # the running sum lives in the bucket
            return None
        for p, v in zip(b.params, b.views):
            p.grad = v
        if self.world == 1:
            return _Ready()
        ready = torch.cuda.Event()
        ready.record()
        early = self.embed_rows is not None and b.params[0] is self.ddp.early_table
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            # buckets reduced under the rest of backward share the SMs with it; the last bucket has the GPU to itself
            last = b.index == len(self.ddp.buckets) - 1 and not early
            self.comm.all_reduce_symmetric_(self.padded[b.index], "avg", sq_slot=b.index,
                                            blocks=self.comm.blocks if last else self.comm_sms)
            done = torch.cuda.Event()
            done.record()
        if early:
            self._table_done = done
        return _Ready(done)

    def wait(self, works) -> None:
        for w in works:
            w.wait()
        self._written.clear()

    def sq_norm(self) -> torch.Tensor:
        if self.world == 1:
            return multi_tensor.sq_norm([self.flat])
        return self.partials.sum()

    def norm_and_coef(self, max_norm: float | None) -> tuple[torch.Tensor, torch.Tensor]:
        """(global gradient norm, clip coefficient) on the device, one finalisation launch over the per-bucket
        partials the all-reduce kernels published (identical bits on every rank)."""
        src = self.partials if self.world > 1 else multi_tensor.sq_norm([self.flat]).reshape(1)
        return multi_tensor.finalize_norm(src, max_norm)

    def loss_slot(self) -> torch.Tensor | None:
        """A 4-float tensor inside the symmetric region: accumulating the step's loss there lets the data-parallel
        average run as an in-place symmetric all-reduce (no padding copy, capturable in the step's graph)."""
        if self.comm is None:
            return None
        if getattr(self, "_loss_slot", None) is None:
            self._loss_slot = self.flat_tail
        return self._loss_slot


class _Ready:
    def __init__(self, event: torch.cuda.Event | None = None):
        self.event = event

    def wait(self) -> bool:
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)
        return True
