"""Multi-tensor kernels (AdamW, grad norm, scaling, DDP bucket fill) driven by device-resident tables.

A ``TensorTable`` records, for a fixed list of tensors, up to five pointer columns, the element counts,
per-tensor flags and the (tensor, chunk) assignment of every thread block.  It is uploaded once; while the
underlying storages stay where they are (parameters, optimizer state, bucket views), every later launch
reuses it.  Tables are rebuilt only when a pointer changes (fresh autograd grads).  A table holds addresses, not
tensors: it keeps nothing alive, and there is one live table per (operation, tensor sizes, flags) slot, so fresh
gradients arriving at new addresses every step replace the previous table instead of piling up.
"""

from __future__ import annotations

import torch

from torchure_b200 import ops

CHUNK = 16384


def available() -> bool:
    return ops.available()


class TensorTable:
    def __init__(self, columns: list[list[torch.Tensor | None]], flags: list[int] | None = None):
        """columns: up to 5 equally long tensor lists (None entries become null pointers)."""
        n = len(columns[0])
        assert n > 0 and all(len(c) == n for c in columns)
        dev = next(t for t in columns[0] if t is not None).device
        ptrs = [[(t.data_ptr() if t is not None else 0) for t in col] for col in columns]
        while len(ptrs) < 5:
            ptrs.append([0] * n)
        numel = [t.numel() for t in columns[0]]
        import numpy as np

        chunks = [(ne + CHUNK - 1) // CHUNK for ne in numel]
        bt = np.repeat(np.arange(n, dtype=np.int32), chunks)
        bc = np.concatenate([np.arange(c, dtype=np.int32) for c in chunks]) if chunks else np.zeros(0, np.int32)
        self.key = tuple(tuple(p) for p in ptrs)
        # uploads go through pinned staging that lives as long as the table: an asynchronous copy from pinned memory
        # is legal while a stream is being captured (the copy node re-reads the same, unchanged, host bytes)
        host = [torch.tensor(ptrs, dtype=torch.int64), torch.tensor(numel, dtype=torch.int64),
                torch.tensor(flags if flags is not None else [0] * n, dtype=torch.int32),
                torch.from_numpy(bt), torch.from_numpy(bc)]
        if dev.type == "cuda":
            host = [h.pin_memory() for h in host]
        self.host = host
        self.ptrs, self.numel, self.flags, self.bt, self.bc = (h.to(dev, non_blocking=True) for h in host)

    def args(self):
        return self.ptrs, self.numel, self.flags, self.bt, self.bc


_CACHE: dict[tuple, TensorTable] = {}


def _table(tag: str, columns, flags=None) -> TensorTable:
    first = columns[0]
    slot = (tag, len(columns), tuple(t.numel() for t in first), tuple(flags) if flags is not None else (),
            first[0].device.index)
    ptrs = [tuple((t.data_ptr() if t is not None else 0) for t in col) for col in columns]
    while len(ptrs) < 5:
        ptrs.append((0,) * len(first))
    tab = _CACHE.get(slot)
    if tab is None or tab.key != tuple(ptrs):
        if len(_CACHE) > 256:
            _CACHE.clear()
        tab = TensorTable(columns, flags)   # replaces (and thereby drops) the slot's previous table
        _CACHE[slot] = tab
    return tab


def _bf16_flags(ts) -> list[int]:
    return [1 if t.dtype == torch.bfloat16 else 0 for t in ts]


def sq_norm(tensors: list[torch.Tensor]) -> torch.Tensor:
    """0-d fp32 tensor: sum of squares over all `tensors` (fp32 or bf16)."""
    out = torch.zeros((), dtype=torch.float32, device=tensors[0].device)
    tab = _table("sq", [tensors], _bf16_flags(tensors))
    ops.ext().sqnorm_multi(*tab.args(), out)
    ops.count_launch()
    return out


def finalize_norm(partials: torch.Tensor, max_norm: float | None, eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor]:
    """(norm, clip coefficient) as 0-d device tensors from partial sums of squares, in ONE launch with a fixed
    summation order: sqrt(sum(partials)) and min(1, max_norm / (norm + eps)) (1 without a max_norm)."""
    out = torch.empty(2, dtype=torch.float32, device=partials.device)
    ops.ext().finalize_norm(partials.reshape(-1), float(max_norm) if max_norm is not None else -1.0, eps, out)
    ops.count_launch()
    return out[0], out[1]


def scale_(tensors: list[torch.Tensor], scale: torch.Tensor) -> None:
    tab = _table("scale", [tensors], _bf16_flags(tensors))
    ops.ext().scale_multi(*tab.args(), scale.to(torch.float32))
    ops.count_launch()


def zero_(tensors: list[torch.Tensor]) -> None:
    """fp32 tensors := 0 in one launch."""
    assert all(t.dtype == torch.float32 for t in tensors)
    tab = _table("zero", [tensors])
    ops.ext().zero_multi(*tab.args())
    ops.count_launch()


def adamw_step(params, grads, exp_avgs, exp_avg_sqs, shadows, lr, beta1, beta2, eps, weight_decay, step,
               grad_scale=None, maximize=False, hyper=None) -> None:
    """`hyper`: optional device tensor {lr, 1 - beta1^t, 1 - beta2^t} that overrides lr/step at run time (graph replay)."""
    tab = _table("adamw", [params, grads, exp_avgs, exp_avg_sqs, shadows], _bf16_flags(grads))
    bias1 = 1.0 - beta1 ** step
    bias2 = 1.0 - beta2 ** step
    gs = grad_scale.to(torch.float32) if grad_scale is not None else None
    ops.ext().adamw_multi(*tab.args(), lr, beta1, beta2, eps, weight_decay, bias1, bias2, gs, maximize, hyper)
    ops.count_launch()


def bucket_pack(grads, dst_views, accumulate: bool, post_scale: float, sq_out: torch.Tensor | None) -> None:
    tab = _table("pack", [grads, dst_views], _bf16_flags(grads))
    ops.ext().bucket_pack_multi(*tab.args(), accumulate, post_scale, sq_out)
    ops.count_launch()
