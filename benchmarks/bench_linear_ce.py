"""Standalone fused linear + cross-entropy: forward + backward time, this repo against the reference.

    python -m benchmarks.bench_linear_ce [--impl ours|reference|both] [--chunk 4096] [--iters 10]

Shapes of the headline model's head: hidden states 8192 x 1024 bf16 ~ N(0, 1), weight 151936 x 1024 ~ N(0, 0.02),
uniform int64 targets; the weight is the fp32 master both trainers hold (each casts it to bf16 itself).  "ours" is
``loss.fused_linear_cross_entropy`` (tcgen05 logits / dgrad / wgrad GEMMs around the ``ce_softmax_grad`` kernel,
fp32 dW accumulated by TMA reduce-add); "reference" is the unmodified
``torchure.loss.fused_linear_ce.fused_linear_cross_entropy`` imported from ``baseline/_ref`` (torch.compile'd chunk
function, cuBLAS).  Each timed iteration is loss forward + ``loss.backward()``; CUDA events, after warm-up.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _time(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference", "both"], default="both")
    ap.add_argument("--chunk", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=4)
    args = ap.parse_args(argv)
    torch.manual_seed(0)
    N, D, V = 8192, 1024, 151936
    dev = "cuda"
    labels = torch.randint(0, V, (N,), device=dev)
    flops = 3 * 2.0 * N * D * V
    out = {"N": N, "D": D, "V": V, "chunk": args.chunk}
    if args.impl in ("ours", "both"):
        from torchure_b200.loss import fused_linear_cross_entropy

        h = torch.randn(N, D, device=dev).bfloat16().requires_grad_(True)
        w = (torch.randn(V, D, device=dev) * 0.02).requires_grad_(True)   # fp32 master, as both trainers hold it

        def ours():
            h.grad = w.grad = None
            fused_linear_cross_entropy(h, w, labels, -100, args.chunk).backward()

        ms = _time(ours, args.iters, args.warmup)
        out["ours_ms"] = ms
        out["ours_tflops"] = flops / ms / 1e9
    if args.impl in ("reference", "both"):
        ref_root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_root, "torchure")):
            out["reference_unavailable"] = "baseline/_ref/torchure is not installed"
        else:
            sys.path.insert(0, ref_root)
            from torchure.loss.fused_linear_ce import fused_linear_cross_entropy as ref_fn

            h2 = torch.randn(N, D, device=dev).bfloat16().requires_grad_(True)
            w2 = (torch.randn(V, D, device=dev) * 0.02).requires_grad_(True)

            def ref():
                h2.grad = w2.grad = None
                ref_fn(h2, w2, labels, -100, args.chunk).backward()

            ms = _time(ref, args.iters, args.warmup + 2)  # torch.compile warms up in the first calls
            out["reference_ms"] = ms
            out["reference_tflops"] = flops / ms / 1e9
    print(json.dumps(out))


if __name__ == "__main__":
    main()
