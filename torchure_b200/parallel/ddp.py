"""Data parallelism: replicate along a mesh axis, average gradients per bucket during backward.

Contract (reference ``torchure/parallelism/data_parallel.py:53-147``):

* the constructor broadcasts every parameter and buffer from coordinate 0 of the axis;
* parameters are bucketed in reverse ``model.parameters()`` order (roughly the order in
  which backward finishes them); a post-accumulate-grad hook per parameter counts a
  bucket down and launches its reduction when the last gradient arrives, so reductions
  overlap the rest of backward;
* after the launch ``p.grad`` points into the bucket's flat buffer, so the reduced values
  are what the optimizer reads;
* ``requires_sync = False`` turns a backward into pure accumulation (no_sync); the last
  micro-batch sets it back to True;
* ``sync()`` waits for every bucket and fails loudly when a bucket never filled.

Two reducers implement a bucket launch:

``TorchReducer``   copy the grads into the flat buffer and call ``collective.all_reduce``
                   ("avg", async).  CPU/gloo path and NCCL baseline.
``FusedReducer``   (CUDA, sm_100a) ONE kernel per bucket reads the bf16/fp32 autograd grads,
                   casts to fp32, accumulates into the fp32 main-grad bucket that lives in
                   symmetric memory, all-reduces it over NVLink with the 1/world scale
                   folded in (multimem in-switch reduction or peer loads) and emits the
                   bucket's sum of squares for gradient clipping.  No NCCL call, no separate
                   cast/scale/norm kernel.  In no_sync micro-batches the same kernel runs
                   with the communication phase off, so accumulation happens in fp32.
                   It is used at world size 1 too (cast + accumulate + sum of squares).

The planner differs from the reference's greedy rule in one way: a run of tiny tensors
(norm gains) is never flushed as its own bucket in front of a matrix that exceeds the cap;
it rides along with that matrix.  At Qwen3-4B this removes every bucket under 1 MiB
(254 launches become 217).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from torchure_b200.core.collective import MeshLike, all_reduce, broadcast


def plan_buckets(params: list[torch.Tensor], cap_bytes: int, merge_small: bool = True,
                 small_bytes: int | None = None, groups=(), solo=()) -> list[list[torch.Tensor]]:
    """Group `params` (already in launch order) into buckets of about `cap_bytes`.

    A bucket closes when the next tensor would overflow it or has another dtype.  With
    `merge_small`, a running bucket smaller than `small_bytes` (default cap/16) is never
    closed by an overflow: the tensor joins it instead.  `groups` lists tuples of parameters
    that must sit next to each other, in the given order, inside one bucket (the rows of a
    fused projection, so one GEMM can write all of their gradients); a group is placed where
    its first member appears in `params`.  `solo` lists parameters that get a bucket of their own (one that must be
    launchable before its neighbours' gradients exist).
    """
    if small_bytes is None:
        small_bytes = cap_bytes // 16
    group_of = {id(p): tuple(g) for g in groups for p in g}
    units: list[list[torch.Tensor]] = []
    seen: set[int] = set()
    for p in params:
        if id(p) in seen:
            continue
        unit = list(group_of.get(id(p), (p,)))
        seen.update(id(q) for q in unit)
        units.append(unit)
    out: list[list[torch.Tensor]] = []
    run: list[torch.Tensor] = []
    run_bytes = 0
    solo_ids = {id(p) for p in solo}
    for unit in units:
        nbytes = sum(p.numel() * p.element_size() for p in unit)
        if any(id(p) in solo_ids for p in unit):
            if run:
                out.append(run)
                run, run_bytes = [], 0
            out.append(list(unit))
            continue
        if run:
            dtype_change = unit[0].dtype != run[0].dtype
            overflow = run_bytes + nbytes > cap_bytes
            keep_small = merge_small and run_bytes < small_bytes and not dtype_change
            if dtype_change or (overflow and not keep_small):
                out.append(run)
                run, run_bytes = [], 0
        run.extend(unit)
        run_bytes += nbytes
    if run:
        out.append(run)
    return out


class Bucket:
    def __init__(self, index: int, params: list[nn.Parameter]):
        self.index = index
        self.params = params
        self.pending = len(params)
        self.numel = sum(p.numel() for p in params)
        self.flat: torch.Tensor | None = None
        self.views: list[torch.Tensor] | None = None

    def bind(self, flat: torch.Tensor) -> None:
        self.flat = flat
        self.views = []
        at = 0
        for p in self.params:
            self.views.append(flat[at:at + p.numel()].view_as(p))
            at += p.numel()


class TorchReducer:
    """Library transport: flat fp32/param-dtype buffers, one async all_reduce("avg") per bucket."""

    fused = False

    def __init__(self, ddp: "DDP"):
        self.ddp = ddp
        for b in ddp.buckets:
            if len(b.params) > 1:
                b.bind(torch.empty(b.numel, dtype=b.params[0].dtype, device=b.params[0].device))

    def launch(self, b: Bucket, sync: bool):
        if not sync:
            return None
        if b.flat is None:
            buf = b.params[0].grad  # a tensor at or over the cap is reduced where it lies
        else:
            torch._foreach_copy_(b.views, [p.grad for p in b.params])
            for p, v in zip(b.params, b.views):
                p.grad = v
            buf = b.flat
        _, work = all_reduce(buf, self.ddp.mesh, self.ddp.dim, "avg", async_op=True)
        return work

    def wait(self, works) -> None:
        for w in works:
            w.wait()


class DDP:
    def __init__(self, model: nn.Module, mesh: MeshLike, dim: str = "dp", bucket_mb: float = 25,
                 fused: bool | None = None, merge_small: bool = True, comm_sms: int = 16, sm_reserve: int = 0,
                 embed_tokens: int = 0, params: list | None = None):
        """`embed_tokens` (tokens per micro-batch, fused reducer with a tied embedding only): size of the symmetric
        buffer through which the ranks exchange embedding-row gradients, which lets the tied embedding / head bucket
        be reduced as soon as the loss head has produced its weight gradient instead of after the last kernel of
        backward (see ``FusedReducer.exchange_embedding``).  0 keeps the bucket where it is."""
        self.mesh, self.dim = mesh, dim
        self.group_size = mesh.size(dim)
        self.requires_sync = True
        self._works: list = []
        self._accum_launches = 0
        # `params` restricts the wrapper to a subset of the model's parameters (expert parallelism reduces expert and
        # shared parameters over different axes, with one wrapper each)
        self._subset = params is not None
        params = [p for p in (params if params is not None else model.parameters()) if p.requires_grad]
        on_gpu = bool(params) and params[0].is_cuda
        if fused is None:
            fused = False
            if on_gpu:
                from torchure_b200 import ops

                fused = ops.available()
        self.fused = bool(fused)
        self.active = self.group_size > 1 or self.fused
        if not self.active:
            return
        self._subset_params = list(params)
        if self.group_size > 1:
            self._replicate(model)
        params.reverse()
        groups = model.fused_param_groups() if (self.fused and hasattr(model, "fused_param_groups")) else ()
        self.early_table = None
        if (self.fused and self.group_size > 1 and embed_tokens > 0 and hasattr(model, "token_emb")
                and getattr(model, "lm_head", None) is not None and model.lm_head.weight is model.token_emb.weight
                and model.token_emb.weight.shape[1] % 4 == 0):
            self.early_table = model.token_emb.weight
        self.embed_tokens = embed_tokens
        self.buckets = [Bucket(i, ps) for i, ps in
                        enumerate(plan_buckets(params, int(bucket_mb * 1024 * 1024), merge_small, groups=groups,
                                               solo=(self.early_table,) if self.early_table is not None else ()))]
        self._bucket_of = {p: b for b in self.buckets for p in b.params}
        if self.fused:
            from torchure_b200.parallel.ddp_fused import FusedReducer

            self.reducer = FusedReducer(self, comm_sms=comm_sms, sm_reserve=sm_reserve)
            if hasattr(model, "set_grad_sink"):
                model.set_grad_sink(self.reducer)
        else:
            self.reducer = TorchReducer(self)
        for p in params:
            p.register_post_accumulate_grad_hook(self._on_grad_ready)

    def _replicate(self, model: nn.Module) -> None:
        tensors = self._subset_params if self._subset else [*model.parameters(), *model.buffers()]
        for t in tensors:
            broadcast(t.detach(), self.mesh, self.dim, src=0)

    def _on_grad_ready(self, param: nn.Parameter) -> None:
        if not self.requires_sync and not self.fused:
            return  # library path: autograd itself accumulates into .grad
        if self.fused and not self.reducer.absorb(param):
            return  # nothing arrived through autograd: the producer wrote into the bucket itself (gradient sink)
        self._count_down(param)

    def _count_down(self, param: nn.Parameter) -> None:
        b = self._bucket_of[param]
        b.pending -= 1
        if b.pending == 0:
            b.pending = len(b.params)
            work = self.reducer.launch(b, self.requires_sync)
            if work is not None:
                self._works.append(work)

    def sync(self) -> None:
        """Wait for every bucket of the step; call between the last backward and the optimizer."""
        if not self.active:
            return
        if len(self._works) != len(self.buckets):
            raise AssertionError(
                f"only {len(self._works)}/{len(self.buckets)} gradient buckets launched: a parameter got no "
                "gradient in this backward (frozen?), or requires_sync was still False on the last "
                "micro-batch of the step")
        self.reducer.wait(self._works)
        self._works.clear()

    # -- fused extras ------------------------------------------------------------------------
    def norm_and_coef(self, max_norm):
        """(gradient norm, clip coefficient) from ONE finalisation kernel over the fused reducer's partials; None
        on the library path."""
        if self.active and self.fused:
            return self.reducer.norm_and_coef(max_norm)
        return None

    def loss_slot(self):
        """Symmetric 4-float tensor for the step's loss (fused reducer with more than one rank), else None."""
        if self.active and self.fused:
            return self.reducer.loss_slot()
        return None

    def sq_norm(self) -> torch.Tensor | None:
        """Sum of squares of the reduced gradients, from the fused kernels' per-bucket partials
        (identical bits on every rank).  None on the library path."""
        if self.active and self.fused:
            return self.reducer.sq_norm()
        return None
