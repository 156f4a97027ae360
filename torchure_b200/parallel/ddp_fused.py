"""Fused gradient-bucket reducer for DDP on sm_100a.

All buckets are slices of ONE fp32 main-gradient buffer.  With more than one rank that buffer lives in the
symmetric allocation of the dp axis, so peers read and write it directly over NVLink.

Per bucket, when its last gradient arrives (post-accumulate-grad hook, i.e. while backward is still running):

1. ``bucket_pack``   one multi-tensor kernel casts the autograd gradients (fp32 or bf16) to fp32 and stores or
                     accumulates them into the bucket (accumulation over no_sync micro-batches happens here, in
                     fp32).  With one rank the same kernel also emits the bucket's sum of squares.
2. ``all_reduce``    (world > 1, sync micro-batch only) one kernel on the communication stream: every rank reduces
                     its 1/world slice with ``multimem.ld_reduce`` (NVSwitch in-fabric reduction; peer loads when
                     no multicast mapping exists), applies the 1/world scale, adds the slice's sum of squares to the
                     shared partial table of every rank and broadcasts the slice with ``multimem.st``.

There is no NCCL call and no separate scale or norm kernel; ``sq_norm()`` sums the partial table in a fixed order,
so every rank derives bit-identical clip coefficients.  After a sync launch ``p.grad`` is a view of the bucket.

GEMM kernels are persistent and occupy every SM they are given, so while a backward is in flight the reducer
asks them to leave ``comm_sms`` SMs free for the communication kernels (``ops.set_compute_sm_reserve``).
"""

from __future__ import annotations

import torch

from torchure_b200 import ops
from torchure_b200.ops import multi_tensor


class FusedReducer:
    fused = True

    def __init__(self, ddp, comm_sms: int = 16):
        self.ddp = ddp
        self.world = ddp.group_size
        params0 = ddp.buckets[0].params
        dev = params0[0].device
        # 64-element alignment keeps every bucket 256-byte aligned and 16-byte divisible per rank
        offs, total = [], 0
        for b in ddp.buckets:
            offs.append(total)
            total += (b.numel + 63) // 64 * 64
        self.comm = None
        if self.world > 1:
            from torchure_b200.core.symm import SymmComm

            self.comm = SymmComm(ddp.mesh.get_group(ddp.dim), ddp.mesh.coordinate(ddp.dim), self.world,
                                 staging_bytes=4096, persistent_bytes=total * 4 + 4096, blocks=comm_sms)
            self.flat = self.comm.alloc(total, torch.float32)
            self.flat.zero_()
            self.partials = self.comm.partials(len(ddp.buckets))
            self.partials.zero_()
            self.stream = torch.cuda.Stream(device=dev, priority=-1)
            ops.set_compute_sm_reserve(comm_sms)
        else:
            self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
            self.partials = torch.zeros(len(ddp.buckets), dtype=torch.float32, device=dev)
            self.stream = None
        self.padded = []
        for b, off in zip(ddp.buckets, offs):
            b.bind(self.flat[off:off + b.numel])
            self.padded.append(self.flat[off:off + (b.numel + 63) // 64 * 64])
            b.fresh = True  # the next pack stores instead of accumulating
        self._events: list[torch.cuda.Event] = []

    def launch(self, b, sync: bool):
        grads = [p.grad for p in b.params]
        local_sq = self.partials[b.index] if (sync and self.world == 1) else None
        if local_sq is not None:
            local_sq.zero_()
        multi_tensor.bucket_pack(grads, b.views, accumulate=not b.fresh, post_scale=1.0, sq_out=local_sq)
        b.fresh = False
        if not sync:
            for p in b.params:
                p.grad = None  # the next micro-batch produces a fresh gradient; the sum lives in the bucket
            return None
        for p, v in zip(b.params, b.views):
            p.grad = v
        b.fresh = True
        if self.world == 1:
            return _Ready()
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            self.comm.all_reduce_symmetric_(self.padded[b.index], "avg", sq_slot=b.index)
            done = torch.cuda.Event()
            done.record()
        return _Ready(done)

    def wait(self, works) -> None:
        for w in works:
            w.wait()

    def sq_norm(self) -> torch.Tensor:
        return self.partials.sum()


class _Ready:
    def __init__(self, event: torch.cuda.Event | None = None):
        self.event = event

    def wait(self) -> bool:
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)
        return True
