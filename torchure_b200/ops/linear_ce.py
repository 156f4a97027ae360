"""Chunked fused linear + cross-entropy on sm_100a kernels.

Per chunk of ``chunk_size`` rows (reference algorithm: ``torchure/loss/fused_linear_ce.py:31-93``):

1. ``logits = h_chunk @ W^T``         tcgen05 GEMM, bf16 out (the only (chunk, V) buffer, reused by every chunk)
2. ``ce_softmax_grad``                one kernel: online max/sum, target gather, per-row loss and, in place,
                                      ``dlogits = (softmax - onehot) / n_valid`` in bf16 (zero for ignored rows)
3. ``dH_chunk = dlogits @ W``         tcgen05 GEMM, B operand read MN-major
4. ``dW (+)= dlogits^T @ h_chunk``    tcgen05 GEMM with fp32 output; the first chunk stores, later chunks
                                      accumulate through TMA reduce-add, so there is no separate ``+=`` pass

With the vocabulary sharded over a tensor-parallel axis (``vocab_parallel``) every rank runs steps 1, 3 and 4 on its
V/n rows of the head, and step 2 becomes ``ce_row_stats`` (row maximum, sum of exponentials, target logit of the
rank's columns), two all-reduces over (chunk,)-sized fp32 vectors (maxima; rescaled sums packed with the target
logits) and ``ce_grad_from_lse``; ``dH`` is summed over the axis once after the loop.

``n_valid`` is counted on the device before the loop, so the mean is folded into step 2 and backward only has
to multiply by the incoming gradient, which a conditional kernel skips when it is exactly 1.
"""

from __future__ import annotations

import torch

from torchure_b200.ops import kernels as K

BF16 = torch.bfloat16


class _LinearCESm100(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, chunk_size, w_bf16, engine, loss_scale, sink_dest,
                normalizer=None, vocab_parallel=None):
        N, D = hidden.shape
        V_all = w_bf16.shape[0]   # a sharded strategy may have released the fp32 weight's own storage
        v0, V = 0, V_all
        if vocab_parallel is not None:
            # loss-parallel: this rank's logits cover rows [v0, v0 + V) of the head; steps 1, 3 and 4 run on that
            # slice, step 2 becomes statistics -> two small all-reduces -> gradient (see the module docstring)
            from torchure_b200.core.collective import all_reduce
            from torchure_b200.loss.fused_linear_ce import vocab_slice

            v0, V = vocab_slice(V_all, *vocab_parallel)
            w_bf16 = w_bf16[v0:v0 + V]
        dev = hidden.device
        h = hidden if hidden.dtype == BF16 else hidden.to(BF16)
        h = h.contiguous()
        n_valid = (labels != ignore_index).sum().clamp_min(1) if normalizer is None else normalizer
        inv_n = (loss_scale / n_valid.float()).reshape(1)
        row_loss = torch.empty(N, dtype=torch.float32, device=dev)
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        d_hidden = torch.empty(N, D, dtype=BF16, device=dev) if need_dh else None
        acc0 = False
        if need_dw and sink_dest is not None:
            d_weight, acc0 = sink_dest  # the fused DDP bucket slice of the weight: written in place
        else:
            d_weight = torch.empty(V_all, D, dtype=torch.float32, device=dev) if need_dw else None
        d_weight_all = d_weight
        if vocab_parallel is not None and need_dw:
            if not acc0:    # rows of the other ranks' slices: zero here, filled by the caller's gather over the axis
                d_weight[:v0].zero_()
                d_weight[v0 + V:].zero_()
            d_weight = d_weight[v0:v0 + V]
        chunk = min(chunk_size, N)
        ldl = (V + 7) // 8 * 8
        logits_buf = torch.empty(chunk, ldl, dtype=BF16, device=dev)
        for lo in range(0, N, chunk):
            hi = min(N, lo + chunk)
            hc = h[lo:hi]
            logits = logits_buf[: hi - lo, :V]
            K.gemm(hc, w_bf16, out=logits)
            if vocab_parallel is None:
                K.ce_softmax_grad_(logits, labels[lo:hi], row_loss[lo:hi], inv_n, ignore_index)
            else:
                yc = labels[lo:hi]
                stats = torch.empty(3, hi - lo, dtype=torch.float32, device=dev)
                K.ce_row_stats_(logits, yc, stats, v0, ignore_index)
                mx = stats[0].clone()
                all_reduce(mx, *vocab_parallel, "max")
                packed = torch.stack([stats[1] * torch.exp(stats[0] - mx), stats[2]])
                all_reduce(packed, *vocab_parallel, "sum")
                lse = mx + torch.log(packed[0])
                row_loss[lo:hi] = torch.where(yc != ignore_index, lse - packed[1], torch.zeros_like(lse))
                K.ce_grad_from_lse_(logits, yc, lse, inv_n, v0, ignore_index)
            if need_dh:
                K.gemm(logits, w_bf16, b_mn=True, out=d_hidden[lo:hi])
            if need_dw:
                K.gemm(logits, hc, a_mn=True, b_mn=True, out=d_weight, accumulate=acc0 or lo > 0)
        if vocab_parallel is not None and need_dh:
            all_reduce(d_hidden, *vocab_parallel, "sum")     # each rank contributed its vocabulary rows
        loss = row_loss.sum() * inv_n[0]
        ctx.stash = (d_hidden, d_weight_all)
        ctx.engine = engine
        ctx.in_sink = sink_dest is not None
        ctx.hidden_dtype = hidden.dtype
        return loss

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.stash is None:
            raise RuntimeError("fused_linear_cross_entropy: backward ran twice; its grads are consumed in place")
        d_hidden, d_weight = ctx.stash
        ctx.stash = None
        scale = grad_out.float().reshape(1)
        if d_hidden is not None:
            K.scale_inplace_(d_hidden, scale)
            if ctx.hidden_dtype != BF16:
                d_hidden = d_hidden.to(ctx.hidden_dtype)
        if d_weight is not None:
            if not ctx.in_sink:  # a sink slice may hold earlier micro-batches: the loss must be the root there
                K.scale_inplace_(d_weight, scale)
            eng = ctx.engine
            if eng is not None and eng.expect_tied_grad:
                eng.expect_tied_grad = False
                sink = eng.model._grad_sink
                head = eng.model.lm_head.weight
                if ctx.in_sink and hasattr(sink, "early_table") and sink.early_table(head):
                    # tied embedding under DDP: the dense part of the gradient is complete, reduce it now (under the
                    # whole block backward); the embedding rows are exchanged when the gather's backward has them
                    from torchure_b200.ops.block import EARLY_TABLE

                    sink.grad_written(head)
                    eng.pending_tied_grad = EARLY_TABLE
                else:
                    # hand the buffer to the gather's backward, which adds its rows and returns it
                    eng.pending_tied_grad = d_weight
                d_weight = None
            elif ctx.in_sink:
                eng.model._grad_sink.grad_written(eng.model.lm_head.weight)
                d_weight = None
        return d_hidden, d_weight, None, None, None, None, None, None, None, None, None


def linear_ce_sm100(hidden, weight, labels, ignore_index, chunk_size, loss_scale=1.0, normalizer=None,
                    vocab_parallel=None):
    from torchure_b200.ops.block import engine_for_weight

    eng = engine_for_weight(weight)
    sink_dest = None
    if eng is not None:
        eng.refresh()
        w_bf16 = eng.head_shadow
        sink = eng.model._grad_sink
        if sink is not None and weight.requires_grad and torch.is_grad_enabled():
            sink_dest = sink.grad_dest(weight)
    else:
        w_bf16 = K.cast_to_bf16(weight.detach().contiguous()) if weight.dtype != BF16 else weight.detach()
    return _LinearCESm100.apply(hidden, weight, labels, ignore_index, chunk_size, w_bf16, eng, float(loss_scale),
                                sink_dest, normalizer, vocab_parallel)
