"""Tensor parallelism (Megatron-style column/row split) and sequence parallelism for the decoder block.

The reference has no TP code (roadmap only: column-wise q/k/v/gate/up, row-wise o/down, vocab-parallel head with
loss-parallel CE, SP as all-gather / reduce-scatter pairs).  Building blocks here:

* ``ColumnParallelLinear``  y_local = x W_local^T, W split along the output dim.  forward: identity on x (or
  all-gather along the sequence when ``sequence_parallel``); backward: all-reduce of dx (or reduce-scatter).
* ``RowParallelLinear``     y = sum_ranks x_local W_local^T, W split along the input dim.  forward: all-reduce (or
  reduce-scatter along the sequence); backward: identity (or all-gather).
* ``parallelize_block``     rewrites a ``TransformerBlock`` in place: q/k/v/gate/up become column-parallel (whole KV
  heads per rank), o/down row-parallel; per-head q/k norms are replicated.
* ``vocab_parallel_cross_entropy``  loss-parallel CE on vocabulary shards: two all-reduces per call (max, then
  sum-exp and target logit together).

Collectives go through ``core.collective`` (NVLink kernels on GPUs, gloo on CPU).

On GPUs with an sm_100a communicator attached to the axis (``collective.enable_sm100``), bf16 activations and one
sequence per micro-batch (token-major rows, a multiple of 128 per rank), the sequence-parallel linears run as ONE
kernel each: ``ag_gemm`` (all-gather -> GEMM) for the column-parallel forward and the row-parallel input gradient,
``gemm_rs`` (GEMM -> reduce-scatter) for the row-parallel forward and the column-parallel input gradient
(``ops/gemm_comm.py``).  Everything else falls back to collective + matmul.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from torchure_b200.core.collective import all_gather, all_reduce, reduce_scatter


class _CopyToTP(torch.autograd.Function):
    """identity forward, all-reduce backward"""

    @staticmethod
    def forward(ctx, x, mesh, dim):
        ctx.mesh, ctx.dim = mesh, dim
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        all_reduce(g, ctx.mesh, ctx.dim, "sum")
        return g, None, None


class _ReduceFromTP(torch.autograd.Function):
    """all-reduce forward, identity backward"""

    @staticmethod
    def forward(ctx, x, mesh, dim):
        x = x.contiguous()
        all_reduce(x, mesh, dim, "sum")
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None, None


class _GatherSeq(torch.autograd.Function):
    """sequence-parallel entry: all-gather along dim 1 forward, reduce-scatter backward"""

    @staticmethod
    def forward(ctx, x, mesh, dim):
        ctx.mesh, ctx.dim = mesh, dim
        return all_gather(x.contiguous(), mesh, dim, gather_dim=1)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter(g.contiguous(), ctx.mesh, ctx.dim, "sum", scatter_dim=1), None, None


class _ScatterSeq(torch.autograd.Function):
    """sequence-parallel exit: reduce-scatter along dim 1 forward, all-gather backward"""

    @staticmethod
    def forward(ctx, x, mesh, dim):
        ctx.mesh, ctx.dim = mesh, dim
        return reduce_scatter(x.contiguous(), mesh, dim, "sum", scatter_dim=1)

    @staticmethod
    def backward(ctx, g):
        return all_gather(g.contiguous(), ctx.mesh, ctx.dim, gather_dim=1), None, None


class _ShardSeq(torch.autograd.Function):
    """Entry of a sequence-parallel region whose input is REPLICATED over the axis (the embedding output): keep this
    rank's slice of dim 1 forward; backward all-gathers the slices, so the replicated producer sees the full gradient
    on every rank (its weight gradient then needs no sum over the axis)."""

    @staticmethod
    def forward(ctx, x, mesh, dim):
        ctx.mesh, ctx.dim = mesh, dim
        n, r = mesh.size(dim), mesh.coordinate(dim)
        assert x.shape[1] % n == 0, f"sequence length {x.shape[1]} is not divisible by tp={n}"
        return x.chunk(n, dim=1)[r].contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather(g.contiguous(), ctx.mesh, ctx.dim, gather_dim=1), None, None


class _UnshardSeq(torch.autograd.Function):
    """Exit of a sequence-parallel region into REPLICATED computation (final norm, head, loss run identically on every
    rank of the axis): all-gather dim 1 forward; every rank then holds the same full gradient, of which backward keeps
    this rank's slice (no sum: the replicas compute one loss, not n of them)."""

    @staticmethod
    def forward(ctx, x, mesh, dim):
        ctx.mesh, ctx.dim = mesh, dim
        return all_gather(x.contiguous(), mesh, dim, gather_dim=1)

    @staticmethod
    def backward(ctx, g):
        n, r = ctx.mesh.size(ctx.dim), ctx.mesh.coordinate(ctx.dim)
        return g.chunk(n, dim=1)[r].contiguous(), None, None


def shard_sequence(x: torch.Tensor, mesh, dim: str = "tp") -> torch.Tensor:
    return _ShardSeq.apply(x, mesh, dim)


def unshard_sequence(x: torch.Tensor, mesh, dim: str = "tp") -> torch.Tensor:
    return _UnshardSeq.apply(x, mesh, dim)


def _autocast_input(x: torch.Tensor) -> torch.Tensor:
    """What F.linear would do to its input under autocast, done up front so that the fused kernels see bf16 rows."""
    if x.is_cuda and torch.is_autocast_enabled() and x.is_floating_point():
        return x.to(torch.get_autocast_gpu_dtype())
    return x


def _fused_comm(x: torch.Tensor, mesh, dim: str):
    """The axis' sm_100a communicator if the fused GEMM+collective kernels can take `x` (tokens of ONE sequence shard
    as rows), else None."""
    from torchure_b200.core.collective import _sm100_for

    if not x.is_cuda or x.dtype != torch.bfloat16:
        return None
    comm = _sm100_for(x, mesh, dim)
    if comm is None:
        return None
    rows = x.numel() // x.shape[-1]
    lead_ok = x.dim() == 2 or all(d == 1 for d in x.shape[:-2])
    return comm if lead_ok and rows % 128 == 0 and x.shape[-1] % 64 == 0 else None


def _workspace(comm, kind: str, shape, dtype):
    """Persistent symmetric operand per (kind, shape): reused by every layer (calls are ordered on one stream and
    every fused kernel handshakes with its peers before it touches their memory)."""
    from torchure_b200.ops.gemm_comm import SymmetricOperand

    cache = comm.__dict__.setdefault("_tp_workspaces", {})
    key = (kind, tuple(shape), dtype)
    if key not in cache:
        cache[key] = SymmetricOperand(comm, shape, dtype)
    return cache[key]


class _ColumnSPFused(torch.autograd.Function):
    """y[M, N/tp] = all_gather_rows(x_shard)[M, K] @ w[N/tp, K]^T in one kernel; backward: one GEMM->reduce-scatter
    kernel for dx, a re-gather plus the wgrad GEMM for dw."""

    @staticmethod
    def forward(ctx, x, w, comm, mesh, dim):
        from torchure_b200.ops.gemm_comm import ag_gemm

        rows, K = x.shape
        a = _workspace(comm, "ag_in", (rows, K), torch.bfloat16)
        a.tensor.copy_(x)
        g = _workspace(comm, "ag_full", (rows * comm.world, K), torch.bfloat16)
        wb = w.to(torch.bfloat16)
        y = ag_gemm(comm, a, wb, gathered=g)
        ctx.save_for_backward(x, wb)
        ctx.comm, ctx.mesh, ctx.dim, ctx.w_dtype = comm, mesh, dim, w.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        from torchure_b200.ops import kernels
        from torchure_b200.ops.gemm_comm import gemm_rs

        x, wb = ctx.saved_tensors
        comm = ctx.comm
        dy = dy.contiguous()
        c = _workspace(comm, "rs_out", (x.shape[0], x.shape[1]), torch.float32)
        dx = gemm_rs(comm, dy, wb, c, b_mn=True).to(torch.bfloat16)   # dy [M, N/tp] @ w [N/tp, K]
        xg = all_gather(x, ctx.mesh, ctx.dim, gather_dim=0)
        dw = kernels.linear_wgrad(dy, xg, out_dtype=torch.float32).to(ctx.w_dtype)
        return dx, dw, None, None, None


class _RowSPFused(torch.autograd.Function):
    """y_shard[M/tp, N] = reduce_scatter_rows(x[M, K/tp] @ w[N, K/tp]^T) in one kernel; backward: one all-gather->GEMM
    kernel for dx whose gathered dy also feeds the wgrad GEMM."""

    @staticmethod
    def forward(ctx, x, w, comm, mesh, dim):
        from torchure_b200.ops.gemm_comm import gemm_rs

        M = x.shape[0]
        wb = w.to(torch.bfloat16)
        c = _workspace(comm, "rs_out", (M // comm.world, wb.shape[0]), torch.float32)
        y = gemm_rs(comm, x.contiguous(), wb, c).to(torch.bfloat16)
        ctx.save_for_backward(x, wb)
        ctx.comm, ctx.w_dtype = comm, w.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        from torchure_b200.ops import kernels
        from torchure_b200.ops.gemm_comm import ag_gemm

        x, wb = ctx.saved_tensors
        comm = ctx.comm
        rows, N = dy.shape
        a = _workspace(comm, "ag_in", (rows, N), torch.bfloat16)
        a.tensor.copy_(dy)
        g = _workspace(comm, "ag_full", (rows * comm.world, N), torch.bfloat16)
        dx, dyg = ag_gemm(comm, a, wb, gathered=g, return_gathered=True, b_mn=True)  # dy_full [M, N] @ w [N, K/tp]
        dw = kernels.linear_wgrad(dyg, x, out_dtype=torch.float32).to(ctx.w_dtype)
        return dx, dw, None, None, None


class ColumnParallelLinear(nn.Module):
    def __init__(self, full: nn.Linear, mesh, dim: str, sequence_parallel: bool = False, split_sizes=None):
        super().__init__()
        n, r = mesh.size(dim), mesh.coordinate(dim)
        rows = full.weight.shape[0]
        assert rows % n == 0, f"output dim {rows} is not divisible by tp={n}"
        per = rows // n
        self.weight = nn.Parameter(full.weight.detach()[r * per:(r + 1) * per].clone())
        self.mesh, self.dim, self.sp = mesh, dim, sequence_parallel

    @property
    def in_features(self) -> int:
        return self.weight.shape[1]

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    def forward(self, x):
        if self.sp:
            x = _autocast_input(x)
            comm = _fused_comm(x, self.mesh, self.dim)
            if comm is not None:
                y = _ColumnSPFused.apply(x.reshape(-1, x.shape[-1]), self.weight, comm, self.mesh, self.dim)
                return y.view(*x.shape[:-2], -1, y.shape[-1])
        x = _GatherSeq.apply(x, self.mesh, self.dim) if self.sp else _CopyToTP.apply(x, self.mesh, self.dim)
        return F.linear(x, self.weight.to(x.dtype))


class RowParallelLinear(nn.Module):
    def __init__(self, full: nn.Linear, mesh, dim: str, sequence_parallel: bool = False):
        super().__init__()
        n, r = mesh.size(dim), mesh.coordinate(dim)
        cols = full.weight.shape[1]
        assert cols % n == 0, f"input dim {cols} is not divisible by tp={n}"
        per = cols // n
        self.weight = nn.Parameter(full.weight.detach()[:, r * per:(r + 1) * per].clone())
        self.mesh, self.dim, self.sp = mesh, dim, sequence_parallel

    def forward(self, x):
        if self.sp:
            n = self.mesh.size(self.dim)
            x = _autocast_input(x)
            comm = _fused_comm(x, self.mesh, self.dim)
            if comm is not None and (x.numel() // x.shape[-1]) % (128 * n) == 0:
                y = _RowSPFused.apply(x.reshape(-1, x.shape[-1]), self.weight, comm, self.mesh, self.dim)
                return y.view(*x.shape[:-2], -1, y.shape[-1])
        y = F.linear(x, self.weight.to(x.dtype))
        return _ScatterSeq.apply(y, self.mesh, self.dim) if self.sp else _ReduceFromTP.apply(y, self.mesh, self.dim)


def parallelize_block(block, mesh, dim: str = "tp", sequence_parallel: bool = False) -> None:
    """Shard one TransformerBlock over the `dim` axis in place (heads and FFN columns split evenly)."""
    n = mesh.size(dim)
    g = block.gqa
    assert g.num_heads % n == 0 and g.num_kv_heads % n == 0, "tp must divide the query and KV head counts"
    g.q_proj = ColumnParallelLinear(g.q_proj, mesh, dim, sequence_parallel)
    g.k_proj = ColumnParallelLinear(g.k_proj, mesh, dim, sequence_parallel)
    g.v_proj = ColumnParallelLinear(g.v_proj, mesh, dim, sequence_parallel)
    g.o_proj = RowParallelLinear(g.o_proj, mesh, dim, sequence_parallel)
    g.num_heads //= n
    g.num_kv_heads //= n
    if getattr(g, "qk_norm", False) and n > 1:
        # the per-head gains are shared by all heads while each rank only sees its own: sum their gradients over the
        # axis (autograd path; the sm_100a engine does the same inside its block function)
        def _sum_over_axis(grad):   # on the incoming gradient, so accumulation over micro-batches stays correct
            if grad is None:          # the sm_100a engine delivers these gradients through its sink, already summed
                return None
            grad = grad.contiguous().clone()
            all_reduce(grad, mesh, dim, "sum")
            return grad

        for w in (g.q_norm.weight, g.k_norm.weight):
            w.register_hook(_sum_over_axis)
    f = block.ffn
    f.gate_proj = ColumnParallelLinear(f.gate_proj, mesh, dim, sequence_parallel)
    f.up_proj = ColumnParallelLinear(f.up_proj, mesh, dim, sequence_parallel)
    f.down_proj = RowParallelLinear(f.down_proj, mesh, dim, sequence_parallel)


class EngineTP:
    """What the sm_100a engine needs to run a tensor-parallel block: the partial sums of the two row-parallel GEMMs
    (attention output, MLP output) and of the two column-parallel input gradients are all-reduced over the axis with
    the NVLink all-reduce kernel, and the per-head QK-norm gain gradients (each rank sees only its heads) are summed."""

    def __init__(self, mesh, dim: str):
        self.mesh, self.dim = mesh, dim
        self.size = mesh.size(dim)

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            all_reduce(t, self.mesh, self.dim, "sum")
        return t


def parallelize_model(model, mesh, dim: str = "tp", sequence_parallel: bool = False) -> None:
    """Tensor-parallel decoder: every block sharded (whole KV heads and FFN columns per rank), embedding / norms /
    head replicated.

    Without sequence parallelism the model keeps its execution path: on Blackwell the sm_100a engine runs each block
    on the rank's heads and FFN columns with its own kernels (the fused projections are simply narrower) and
    all-reduces the four partial sums (``EngineTP``).  With ``sequence_parallel`` the blocks run through the
    module-level column / row linears, whose sequence-parallel form is ONE fused kernel each on GPUs (``ag_gemm`` /
    ``gemm_rs``), around the PyTorch attention and norms."""
    n = mesh.size(dim)
    for b in model.blocks:
        parallelize_block(b, mesh, dim, sequence_parallel)
    for b in model.blocks:
        for lin in (b.gqa.q_proj, b.gqa.k_proj, b.gqa.v_proj, b.gqa.o_proj, b.ffn.gate_proj, b.ffn.up_proj,
                    b.ffn.down_proj):
            lin.weight._tp_sharded = True
    if sequence_parallel:
        # The module path runs with the activations between the linears sharded along the sequence: the model slices
        # the embedding output (`shard_sequence`) and gathers before its final norm (`unshard_sequence`); the norms
        # inside the blocks see 1/n of the tokens each, so their gain gradients are summed over the axis.
        model.impl = "torch"
        model.sp = (mesh, dim)

        def _sum_partial(grad):
            if grad is None:
                return None
            grad = grad.contiguous().clone()
            all_reduce(grad, mesh, dim, "sum")
            return grad

        if n > 1:
            for b in model.blocks:
                for norm in (b.norm1, b.norm2):
                    norm.weight.register_hook(_sum_partial)
        return
    # the engine reads head counts and the FFN width from the model's config: make them this rank's
    model.cfg = dict(model.cfg, num_heads=model.cfg["num_heads"] // n, num_kv_heads=model.cfg["num_kv_heads"] // n,
                     ffn_dim=model.cfg["ffn_dim"] // n)
    model._engine = None
    model.tp = EngineTP(mesh, dim)


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits_local, labels, mesh, dim, ignore_index):
        n, r = mesh.size(dim), mesh.coordinate(dim)
        vloc = logits_local.shape[-1]
        lo = r * vloc
        lf = logits_local.float()
        mx = lf.max(dim=-1).values
        all_reduce(mx, mesh, dim, "max")
        ex = torch.exp(lf - mx[:, None])
        keep = labels != ignore_index
        mine = keep & (labels >= lo) & (labels < lo + vloc)
        idx = torch.where(mine, labels - lo, torch.zeros_like(labels))
        tgt = torch.where(mine, lf.gather(1, idx[:, None]).squeeze(1), torch.zeros_like(mx))
        packed = torch.stack([ex.sum(-1), tgt], dim=0)  # one all-reduce for both
        all_reduce(packed, mesh, dim, "sum")
        sumexp, tgt = packed[0], packed[1]
        n_valid = keep.sum().clamp_min(1)
        loss = torch.where(keep, torch.log(sumexp) + mx - tgt, torch.zeros_like(mx)).sum() / n_valid
        probs = ex / sumexp[:, None]
        probs[torch.arange(labels.numel(), device=labels.device)[mine], idx[mine]] -= 1.0
        ctx.save_for_backward((probs * keep[:, None] / n_valid).to(logits_local.dtype))
        return loss

    @staticmethod
    def backward(ctx, g):
        (d,) = ctx.saved_tensors
        return d * g, None, None, None, None


def vocab_parallel_cross_entropy(logits_local: torch.Tensor, labels: torch.Tensor, mesh, dim: str = "tp",
                                 ignore_index: int = -100) -> torch.Tensor:
    """Mean CE where `logits_local` (N, V/tp) holds this rank's vocabulary slice [r*V/tp, (r+1)*V/tp)."""
    return _VocabParallelCE.apply(logits_local, labels, mesh, dim, ignore_index)
