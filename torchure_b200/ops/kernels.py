"""Thin Python wrappers over the sm_100a kernels (allocation + launch counting); no math here.

Every function launches exactly the kernels its docstring names.  Plain PyTorch statements of the
same operations live in ``ops/oracle.py`` and are what the GPU tests compare against.
"""

from __future__ import annotations

import torch

from torchure_b200 import ops
from torchure_b200.ops.debug import new_output

BF16 = torch.bfloat16


def _C():
    ext = ops.ext()
    if ext is None:
        raise RuntimeError("the torchure_b200 CUDA extension is not built (python -m torchure_b200.build)")
    return ext


def check_error() -> None:
    """Synchronise and raise if any kernel recorded an expired wait."""
    word = _C().error_word()
    code = int(word[0].item())
    if code != 0:
        word.zero_()
        names = {1: "GEMM producer waited for a free stage", 2: "GEMM MMA warp waited for a full stage",
                 3: "GEMM MMA warp waited for a free accumulator", 4: "GEMM epilogue waited for an accumulator",
                 5: "a collective waited for a peer flag", 6: "attention pipeline wait",
                 7: "a row staged into shared memory by a bulk copy never arrived"}
        raise RuntimeError(f"sm_100a kernel reported an expired wait: code {code} ({names.get(code, 'unknown')})")


def check_comm_error(rank: int | None = None) -> None:
    """Synchronise and raise if a collective or fused GEMM+collective kernel gave up waiting for a peer."""
    word = _C().comm_error_word()
    code = int(word[0].item())
    if code != 0:
        word.zero_()
        where = "" if rank is None else f" on rank {rank}"
        raise RuntimeError(f"a collective gave up waiting for a peer flag{where} (code {code}); its output is "
                           "incomplete and every later collective bails out until the word is cleared")


# ---- GEMM ---------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: torch.Tensor | None = None,
         out_dtype=BF16, accumulate: bool = False, splits: int = 0) -> torch.Tensor:
    """out[M,N] (+)= A * B^T on tcgen05 tensor cores, fp32 accumulation.

    a: [M,K] (or [K,M] when a_mn), b: [N,K] (or [K,N] when b_mn); bf16, innermost stride 1.
    """
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        assert not accumulate
        out = new_output("gemm", M, N, dtype=out_dtype, device=a.device)
    mode = 0 if out.dtype == BF16 else (2 if accumulate else 1)
    assert not (accumulate and out.dtype == BF16), "accumulation needs an fp32 output"
    _C().gemm(a, b, out, a_mn, b_mn, mode, splits)
    ops.count_launch()
    return out


def linear_fwd(x: torch.Tensor, w: torch.Tensor, out=None) -> torch.Tensor:
    """y[M,N] = x[M,K] @ w[N,K]^T"""
    return gemm(x, w, out=out)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, out=None) -> torch.Tensor:
    """dx[M,K] = dy[M,N] @ w[N,K]   (w is the MN-major B operand)"""
    return gemm(dy, w, b_mn=True, out=out)


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, out=None, out_dtype=BF16, accumulate=False) -> torch.Tensor:
    """dw[N,K] = dy[M,N]^T @ x[M,K]   (both operands MN-major)"""
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, out_dtype=out_dtype, accumulate=accumulate)


# ---- norms / rope / mlp -----------------------------------------------------------------------------
def add_rmsnorm(x, y, w, eps, *, ids=None, table=None, need_x_out=True):
    """(x_new, h, rstd) with x_new = x + y (or table[ids]); h = rmsnorm(x_new) * w in bf16."""
    if ids is not None:
        M, D = ids.numel(), table.shape[1]
        dev = table.device
    else:
        M, D = x.shape
        dev = x.device
    h = new_output("add_rmsnorm.h", M, D, dtype=BF16, device=dev)
    rstd = new_output("add_rmsnorm.rstd", M, dtype=torch.float32, device=dev)
    x_out = None
    if (y is not None or ids is not None) and need_x_out:
        x_out = new_output("add_rmsnorm.x_out", M, D, dtype=torch.float32, device=dev)
    _C().add_rmsnorm_fwd(x, y, ids, table, w, x_out, h, rstd, eps)
    ops.count_launch()
    return (x_out if x_out is not None else x), h, rstd


def rmsnorm_bwd(dh, x, w, rstd, dx_in, dw, want_bf16=True, dx_out=None):
    """dx = dx_in + d rmsnorm(x)^T dh (fp32), optional bf16 copy; dw += sum_rows(dh * xhat).  `dx_out`: caller-owned
    destination of dx (a symmetric buffer the peers will read)."""
    dx = dx_out if dx_out is not None else new_output("rmsnorm_bwd.dx", x.shape, dtype=x.dtype, device=x.device)
    dxb = new_output("rmsnorm_bwd.dx_bf16", x.shape, dtype=BF16, device=x.device) if want_bf16 else None
    _C().rmsnorm_bwd(dh, x, w, rstd, dx_in, dx, dxb, dw)
    ops.count_launch()
    return dx, dxb


def qknorm_rope(qkv, qw, kw, cos, sin, S, Hq, Hkv, eps, use_norm=True):
    out = new_output("qknorm_rope", qkv.shape[0], (Hq + Hkv) * 128, dtype=BF16, device=qkv.device)
    _C().qknorm_rope_fwd(qkv, qw, kw, cos, sin, out, S, Hq, Hkv, eps, use_norm)
    ops.count_launch()
    return out


def qknorm_rope_bwd_(dqkv, qkv, qw, kw, cos, sin, dqw, dkw, S, Hq, Hkv, eps, use_norm=True, dq_acc=None):
    """In place on the q / k columns of dqkv.  `dq_acc` (fp32 [B, Hq, S, 128]): dq is read from there instead of the
    q columns (what the single-pass attention backward leaves behind), saving its conversion pass."""
    _C().qknorm_rope_bwd(dqkv, qkv, qw, kw, cos, sin, dqw, dkw, S, Hq, Hkv, eps, use_norm, dq_acc)
    ops.count_launch()
    return dqkv


def swiglu(gu):
    act = new_output("swiglu", gu.shape[0], gu.shape[1] // 2, dtype=BF16, device=gu.device)
    _C().swiglu_fwd(gu, act)
    ops.count_launch()
    return act


def swiglu_bwd(dact, gu):
    dgu = new_output("swiglu_bwd", gu.shape, dtype=gu.dtype, device=gu.device)
    _C().swiglu_bwd(dact, gu, dgu)
    ops.count_launch()
    return dgu


def embedding_bwd_(dx, ids, dtable):
    _C().embedding_bwd(dx, ids, dtable)
    ops.count_launch()
    return dtable


def embedding_scatter_(sources, dtable, M, scale=1.0, sq_delta=None, blocks=592, ids_scratch=None):
    """Deterministic dtable[id] += scale * rows, over `sources` = [(ids (M,) int64, rows (M, D) fp32) or
    (ids address, rows address), ...] in list order; no atomics.  Addresses let a source live on a peer GPU; then pass
    `ids_scratch` (local int64, len(sources) * M): a first kernel copies every source's ids there, because every CTA
    of the scatter scans all of them."""
    ids_ptrs = [s[0] if isinstance(s[0], int) else s[0].data_ptr() for s in sources]
    rows_ptrs = [s[1] if isinstance(s[1], int) else s[1].data_ptr() for s in sources]
    _C().embedding_scatter(ids_ptrs, rows_ptrs, dtable, M, float(scale), sq_delta, blocks, ids_scratch)
    ops.count_launch(2 if ids_scratch is not None else 1)
    return dtable


def ce_softmax_grad_(logits, labels, row_loss, inv_n_valid, ignore_index):
    _C().ce_softmax_grad(logits, labels, row_loss, inv_n_valid, ignore_index)
    ops.count_launch()


def ce_row_stats_(logits, labels, stats, vocab_lo, ignore_index):
    """Vocabulary-sharded CE, first pass: stats (fp32 [3, rows]) <- row maximum, sum of exponentials relative to it,
    target logit (0 when the target lies outside columns [vocab_lo, vocab_lo + V))."""
    _C().ce_row_stats(logits, labels, stats, vocab_lo, ignore_index)
    ops.count_launch()


def ce_grad_from_lse_(logits, labels, lse, inv_n_valid, vocab_lo, ignore_index):
    """Second pass: logits <- (exp(logits - lse[row]) - onehot) * inv_n_valid in place, zeros for ignored rows."""
    _C().ce_grad_from_lse(logits, labels, lse, inv_n_valid, vocab_lo, ignore_index)
    ops.count_launch()


def cast_to_bf16(src, dst=None):
    if dst is None:
        dst = torch.empty(src.shape, dtype=BF16, device=src.device)
    _C().cast_to_bf16(src, dst)
    ops.count_launch()
    return dst


def scale_inplace_(x, scale):
    _C().scale_inplace(x, scale)
    ops.count_launch()
    return x
