"""Causal GQA attention over the fused projection layout.

Inputs are the buffers the surrounding kernels produce, no transposes or copies:

* ``qk``   (M, (Hq+Hkv)*hd) bf16: normalised, rotated queries then keys, token-major
* ``qkv``  (M, (Hq+2Hkv)*hd) bf16: the raw QKV projection; only its V columns are read
* output  ``o`` (M, Hq*hd) bf16 (what o_proj consumes) and ``lse`` (B, Hq, S) fp32 (natural log)

Backward writes dq | dk | dv into one (M, (Hq+2Hkv)*hd) buffer laid out like ``qkv``, which the
QK-norm/RoPE backward kernel then transforms in place and the QKV dgrad/wgrad GEMMs consume.

``impl="sm100"`` is the hand-written tcgen05 kernel set: ``csrc/attention_fwd_sm100.cu`` forward and, for
backward, either the single-pass kernel ``csrc/attention_bwd_fused_sm100.cu`` (default: five tile products per
block pair, dQ partial tiles added into an fp32 accumulator, so dQ is not bitwise repeatable) or the two-kernel
path ``csrc/attention_bwd_dq_sm100.cu`` + ``csrc/attention_bwd_dkv_sm100.cu`` (seven products, no atomics, bitwise
repeatable; ``set_backward("split")`` or ``TORCHURE_B200_ATTN_BWD=split``).
``impl="sdpa"`` routes through ``torch.nn.functional.scaled_dot_product_attention``.  It exists for A/B comparison
only and must be asked for (``TORCHURE_B200_ATTN=sdpa``): a shape the kernels do not cover (S % 128 != 0, an odd
number of query heads per KV head) raises instead of silently running the library kernel on the hot path.  Models
whose head_dim is not 128 never reach this module: they run on the PyTorch path (``models/qwen3.py::_use_sm100``).
"""

from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from torchure_b200 import ops
from torchure_b200.ops.debug import new_output

_FORCE = os.environ.get("TORCHURE_B200_ATTN", "")  # "sdpa" forces the library path
_BWD = os.environ.get("TORCHURE_B200_ATTN_BWD", "fused")


def set_backward(mode: str) -> None:
    """Choose the backward of the sm100 path: "fused" (single pass, fp32 dQ reductions) or "split" (two kernels,
    deterministic)."""
    global _BWD
    assert mode in ("fused", "split")
    _BWD = mode


def kernel_supported(S: int, Hq: int, Hkv: int, hd: int) -> bool:
    ext = ops.ext()
    if _FORCE == "sdpa" or ext is None or not (hasattr(ext, "attn_fwd") and hasattr(ext, "attn_bwd")):
        return False
    return hd == 128 and S % 128 == 0 and Hq % Hkv == 0 and (Hq // Hkv) % 2 == 0


def _views(qk, qkv, B, S, Hq, Hkv, hd):
    q = qk[:, :Hq * hd].view(B, S, Hq, hd).transpose(1, 2)
    k = qk[:, Hq * hd:].view(B, S, Hkv, hd).transpose(1, 2)
    v = qkv[:, (Hq + Hkv) * hd:].view(B, S, Hkv, hd).transpose(1, 2)
    return q, k, v


class AttnState:
    """What backward needs; differs per implementation."""

    __slots__ = ("impl", "o", "lse", "graph")

    def __init__(self, impl, o=None, lse=None, graph=None):
        self.impl, self.o, self.lse, self.graph = impl, o, lse, graph


def attn_fwd(qk, qkv, B, S, Hq, Hkv, hd, need_grad=True):
    """Returns (o (M, Hq*hd) bf16, state)."""
    if _FORCE != "sdpa" and not kernel_supported(S, Hq, Hkv, hd):
        raise RuntimeError(
            f"the sm_100a attention kernels cover head_dim 128, sequence lengths in multiples of 128 and an even "
            f"number of query heads per KV head; got head_dim {hd}, S {S}, {Hq}/{Hkv} heads.  Pad the sequence, or run "
            f"the model with impl='torch', or set TORCHURE_B200_ATTN=sdpa to use the library kernel on purpose")
    if kernel_supported(S, Hq, Hkv, hd):
        ext = ops.ext()
        o = new_output("attn_fwd.o", B * S, Hq * hd, dtype=torch.bfloat16, device=qk.device)
        lse = new_output("attn_fwd.lse", B, Hq, S, dtype=torch.float32, device=qk.device)
        ext.attn_fwd(qk, qkv, o, lse, B, S, Hq, Hkv)
        ops.count_launch()
        return o, AttnState("sm100", o, lse)
    q, k, v = _views(qk, qkv, B, S, Hq, Hkv, hd)
    if need_grad:
        with torch.enable_grad():
            ql, kl, vl = (t.detach().requires_grad_() for t in (q, k, v))
            out = F.scaled_dot_product_attention(ql, kl, vl, is_causal=True, enable_gqa=Hq != Hkv)
        o = out.detach().transpose(1, 2).reshape(B * S, Hq * hd)
        return o, AttnState("sdpa", graph=(out, ql, kl, vl))
    out = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=Hq != Hkv)
    return out.transpose(1, 2).reshape(B * S, Hq * hd), AttnState("sdpa")


def attn_bwd(d_o, qk, qkv, state: AttnState, B, S, Hq, Hkv, hd, keep_dq_fp32: bool = False):
    """Returns dqkv (M, (Hq+2Hkv)*hd) bf16 = [dq (post-rope) | dk (post-rope) | dv].

    With `keep_dq_fp32` the result is ``(dqkv, dq_acc)``: when the single-pass kernel ran, ``dq_acc`` is its head-major
    fp32 dQ accumulator (B, Hq, S, hd) and the q columns of ``dqkv`` are left unwritten for the consumer that reads
    the accumulator (``kernels.qknorm_rope_bwd_(..., dq_acc=)``); otherwise ``dq_acc`` is None."""
    M = B * S
    dqkv = new_output("attn_bwd.dqkv", M, (Hq + 2 * Hkv) * hd, dtype=torch.bfloat16, device=d_o.device)
    if state.impl == "sm100":
        dq_acc = None
        if _BWD == "fused":
            acc = ops.ext().attn_bwd_fused(d_o, qk, qkv, state.o, state.lse, dqkv, B, S, Hq, Hkv, not keep_dq_fp32)
            ops.count_launch(2 if keep_dq_fp32 else 3)  # statistics (+ accumulator clear), fused kernel, conversion
            dq_acc = acc if keep_dq_fp32 else None
        else:
            ops.ext().attn_bwd(d_o, qk, qkv, state.o, state.lse, dqkv, B, S, Hq, Hkv)
            ops.count_launch(3)
        return (dqkv, dq_acc) if keep_dq_fp32 else dqkv
    out, ql, kl, vl = state.graph
    g = d_o.view(B, S, Hq, hd).transpose(1, 2)
    dq, dk, dv = torch.autograd.grad(out, (ql, kl, vl), g)
    dqkv[:, :Hq * hd].view(B, S, Hq, hd).copy_(dq.transpose(1, 2))
    dqkv[:, Hq * hd:(Hq + Hkv) * hd].view(B, S, Hkv, hd).copy_(dk.transpose(1, 2))
    dqkv[:, (Hq + Hkv) * hd:].view(B, S, Hkv, hd).copy_(dv.transpose(1, 2))
    return (dqkv, None) if keep_dq_fp32 else dqkv


# ---- attention on caller-owned (B, S, H, 128) tensors ---------------------------------------------------------------
def pair_supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    """True when the block-pair kernels can take these (B, S, H, d) tensors: CUDA bf16, head_dim 128, sequence
    lengths in whole 128-token blocks, an even number of query heads per KV head."""
    ext = ops.ext() if ops.available() else None
    if ext is None or not hasattr(ext, "attn_fwd_pair"):
        return False
    if not (q.is_cuda and q.dtype == k.dtype == v.dtype == torch.bfloat16):
        return False
    return (q.shape[-1] == 128 and q.shape[1] % 128 == 0 and k.shape[1] % 128 == 0 and q.shape[2] % k.shape[2] == 0
            and (q.shape[2] // k.shape[2]) % 2 == 0)


def _rows(t: torch.Tensor) -> torch.Tensor:
    """(B, S, H, d) -> the token-major 2-D view (B*S, H*d) the kernels index (copy only if not contiguous)."""
    return t.contiguous().view(t.shape[0] * t.shape[1], t.shape[2] * t.shape[3])


class _FlashAttention(torch.autograd.Function):
    """Full-sequence attention on separate q / k / v tensors through the block-pair entry points of the sm_100a
    kernels: ``attn_fwd_pair`` forward, ``attn_bwd_stats`` + ``attn_bwd_pair`` + ``attn_dq_convert`` backward."""

    @staticmethod
    def forward(ctx, q, k, v, causal):
        B, Sq, Hq, _ = q.shape
        Skv, Hkv = k.shape[1], k.shape[2]
        q2, k2, v2 = _rows(q), _rows(k), _rows(v)
        o = torch.empty(B * Sq, Hq * 128, dtype=torch.bfloat16, device=q.device)
        lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=q.device)
        ops.ext().attn_fwd_pair(q2, 0, k2, 0, v2, 0, o, lse, B, Sq, Skv, Hq, Hkv, Sq, 0, Skv, 0, bool(causal))
        ops.count_launch()
        ctx.save_for_backward(q2, k2, v2, o, lse)
        ctx.dims = (B, Sq, Skv, Hq, Hkv, bool(causal))
        return o.view(B, Sq, Hq, 128)

    @staticmethod
    def backward(ctx, d_o):
        q2, k2, v2, o, lse = ctx.saved_tensors
        B, Sq, Skv, Hq, Hkv, causal = ctx.dims
        ext = ops.ext()
        d_o2 = _rows(d_o.to(torch.bfloat16))
        dev = q2.device
        nds = torch.empty(B, Hq, Sq, dtype=torch.float32, device=dev)
        nlse2 = torch.empty_like(nds)
        dq_acc = torch.empty(B, Hq, Sq, 128, dtype=torch.float32, device=dev)
        ext.attn_bwd_stats(d_o2, o, lse, nds, nlse2, dq_acc, B, Sq, Hq)
        dk = torch.empty(B * Skv, Hkv * 128, dtype=torch.bfloat16, device=dev)
        dv = torch.empty_like(dk)
        ext.attn_bwd_pair(q2, 0, k2, 0, v2, 0, d_o2, dq_acc, dk, dv, nds, nlse2, B, Sq, Skv, Hq, Hkv, Sq, 0, Skv, 0, Sq, 0,
                          causal)
        dq = torch.empty(B * Sq, Hq * 128, dtype=torch.bfloat16, device=dev)
        ext.attn_dq_convert(dq_acc, dq, B, Sq, Hq)
        ops.count_launch(3)
        return dq.view(B, Sq, Hq, 128), dk.view(B, Skv, Hkv, 128), dv.view(B, Skv, Hkv, 128), None


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """Attention of q (B, Sq, Hq, 128) over k / v (B, Skv, Hkv, 128), bf16, differentiable.  ``causal`` needs
    Sq == Skv.  What Ulysses sequence parallelism calls between its two all-to-alls; falls back to SDPA for tensors
    the kernels do not cover."""
    if pair_supported(q, k, v):
        return _FlashAttention.apply(q, k, v, causal)
    out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal,
                                         enable_gqa=q.shape[2] != k.shape[2])
    return out.transpose(1, 2)
