"""Small, self-contained launches of single kernels for profiling and timing.

    python -m benchmarks.profile_case <case> [--iters N]

Cases: gemm_fwd, gemm_dgrad, gemm_wgrad, attn_fwd, attn_bwd (single pass), attn_bwd_split, attn_prep, rmsnorm, rmsnorm_bwd, qknorm_rope,
qknorm_rope_bwd, qknorm_rope_bwd_acc, swiglu, swiglu_bwd, ce, adamw.  Each case builds inputs
larger than the 126 MB L2 but well under a few GB, launches the kernel `iters` times (default 4) and prints the
CUDA-event time of the last launch with the achieved FLOP/s or bytes/s, so the same command serves a plain timing run
and an `ncu -k regex:<kernel> -s 2 -c 1` capture.
"""

from __future__ import annotations

import argparse

import torch


def main(argv=None) -> None:
    from torchure_b200 import ops
    from torchure_b200.models.qwen3 import RotaryEmbedding
    from torchure_b200.ops import kernels as K
    from torchure_b200.ops import multi_tensor

    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=4)
    args = ap.parse_args(argv)
    torch.manual_seed(0)
    dev = "cuda"
    M, D, F_, Hq, Hkv, hd, S, B = 8192, 1024, 3072, 16, 8, 128, 4096, 2
    flops = bytes_ = 0.0
    if args.case == "gemm_fwd":        # gate|up projection: [8192,1024] x [6144,1024]^T
        a, b = torch.randn(M, D, device=dev).bfloat16(), torch.randn(2 * F_, D, device=dev).bfloat16()
        out = torch.empty(M, 2 * F_, dtype=torch.bfloat16, device=dev)
        fn = lambda: K.gemm(a, b, out=out)
        flops = 2.0 * M * 2 * F_ * D
    elif args.case == "gemm_dgrad":    # d_h2 = d_gu [8192,6144] x Wgu [6144,1024]
        a, b = torch.randn(M, 2 * F_, device=dev).bfloat16(), torch.randn(2 * F_, D, device=dev).bfloat16()
        out = torch.empty(M, D, dtype=torch.bfloat16, device=dev)
        fn = lambda: K.gemm(a, b, b_mn=True, out=out)
        flops = 2.0 * M * 2 * F_ * D
    elif args.case == "gemm_wgrad":    # dWgu [6144,1024] = d_gu^T h2, fp32 out, split-K
        a, b = torch.randn(M, 2 * F_, device=dev).bfloat16(), torch.randn(M, D, device=dev).bfloat16()
        out = torch.empty(2 * F_, D, dtype=torch.float32, device=dev)
        fn = lambda: K.gemm(a, b, a_mn=True, b_mn=True, out=out)
        flops = 2.0 * M * 2 * F_ * D
    elif args.case in ("attn_fwd", "attn_bwd", "attn_bwd_split"):
        qk = torch.randn(M, (Hq + Hkv) * hd, device=dev).bfloat16()
        qkv = torch.randn(M, (Hq + 2 * Hkv) * hd, device=dev).bfloat16()
        o = torch.empty(M, Hq * hd, dtype=torch.bfloat16, device=dev)
        lse = torch.empty(B, Hq, S, device=dev)
        unit = 2.0 * S * S * hd * Hq * B / 2  # one causal S x S x hd product over all heads
        if args.case == "attn_fwd":
            fn = lambda: ops.ext().attn_fwd(qk, qkv, o, lse, B, S, Hq, Hkv)
            flops = 2 * unit
        else:
            ops.ext().attn_fwd(qk, qkv, o, lse, B, S, Hq, Hkv)
            d_o = torch.randn(M, Hq * hd, device=dev).bfloat16()
            dqkv = torch.empty_like(qkv)
            if args.case == "attn_bwd":
                fn = lambda: ops.ext().attn_bwd_fused(d_o, qk, qkv, o, lse, dqkv, B, S, Hq, Hkv)
                flops = 5 * unit
            else:
                fn = lambda: ops.ext().attn_bwd(d_o, qk, qkv, o, lse, dqkv, B, S, Hq, Hkv)
                flops = 7 * unit  # S and dP are recomputed in both gradient kernels: 3 + 4 products
    elif args.case == "rmsnorm":
        x, y = torch.randn(4 * M, D, device=dev), torch.randn(4 * M, D, device=dev).bfloat16()
        w = torch.ones(D, device=dev)
        fn = lambda: K.add_rmsnorm(x, y, w, 1e-6)
        bytes_ = 4 * M * D * (4 + 2 + 4 + 2)
    elif args.case == "qknorm_rope":
        qkv = torch.randn(M, (Hq + 2 * Hkv) * hd, device=dev).bfloat16()
        cos, sin = RotaryEmbedding(hd).tables(S, dev)
        w = torch.ones(hd, device=dev)
        fn = lambda: K.qknorm_rope(qkv, w, w, cos, sin, S, Hq, Hkv, 1e-6, True)
        bytes_ = 2 * M * (Hq + Hkv) * hd * 2
    elif args.case in ("qknorm_rope_bwd", "qknorm_rope_bwd_acc"):
        qkv = torch.randn(M, (Hq + 2 * Hkv) * hd, device=dev).bfloat16()
        dqkv = torch.randn(M, (Hq + 2 * Hkv) * hd, device=dev).bfloat16()
        cos, sin = RotaryEmbedding(hd).tables(S, dev)
        w = torch.ones(hd, device=dev)
        dqw, dkw = torch.zeros(hd, device=dev), torch.zeros(hd, device=dev)
        # _acc: dq comes from the head-major fp32 accumulator of the single-pass attention backward (the engine's path)
        acc = torch.randn(M // S, Hq, S, hd, device=dev) if args.case.endswith("_acc") else None
        fn = lambda: K.qknorm_rope_bwd_(dqkv, qkv, w, w, cos, sin, dqw, dkw, S, Hq, Hkv, 1e-6, True, dq_acc=acc)
        bytes_ = 3 * M * (Hq + Hkv) * hd * 2   # read dqkv and qkv (q, k columns), write dqkv
        if acc is not None:
            bytes_ += M * Hq * hd * 2          # dq is read as fp32 instead of bf16
    elif args.case == "rmsnorm_bwd":
        rows = 4 * M
        x, dh = torch.randn(rows, D, device=dev), torch.randn(rows, D, device=dev).bfloat16()
        dx_in = torch.randn(rows, D, device=dev)
        w, dw = torch.ones(D, device=dev), torch.zeros(D, device=dev)
        rstd = torch.rsqrt(x.pow(2).mean(-1) + 1e-6)
        fn = lambda: K.rmsnorm_bwd(dh, x, w, rstd, dx_in, dw)
        bytes_ = rows * D * (2 + 4 + 4 + 4 + 2)   # dh, x, dx_in read; dx fp32 and bf16 written
    elif args.case == "attn_prep":
        d_o, o = (torch.randn(4 * M, Hq * hd, device=dev).bfloat16() for _ in range(2))
        lse = torch.randn(4 * B, Hq, S, device=dev)
        delta, lse2 = torch.empty_like(lse), torch.empty_like(lse)
        fn = lambda: ops.ext().attn_bwd_prep(d_o, o, lse, delta, lse2, 4 * B, S, Hq)
        bytes_ = 2 * 4 * M * Hq * hd * 2
    elif args.case in ("swiglu", "swiglu_bwd"):
        rows = 2 * M
        gu = torch.randn(rows, 2 * F_, device=dev).bfloat16()
        if args.case == "swiglu":
            fn = lambda: K.swiglu(gu)
            bytes_ = rows * F_ * 2 * 3          # gate, up read; act written
        else:
            dact = torch.randn(rows, F_, device=dev).bfloat16()
            fn = lambda: K.swiglu_bwd(dact, gu)
            bytes_ = rows * F_ * 2 * 5          # dact, gate, up read; dgate, dup written
    elif args.case == "ce":
        V, C = 151936, 1024
        logits = torch.randn(C, V, device=dev).bfloat16()
        labels = torch.randint(0, V, (C,), device=dev)
        loss, inv = torch.empty(C, device=dev), torch.ones(1, device=dev)
        fn = lambda: K.ce_softmax_grad_(logits, labels, loss, inv, -100)
        bytes_ = 2 * C * V * 2
    elif args.case == "adamw":
        n = 64 << 20
        p, g, m, v = (torch.randn(n, device=dev) for _ in range(4))
        v.abs_()
        sh = torch.empty(n, dtype=torch.bfloat16, device=dev)
        fn = lambda: multi_tensor.adamw_step([p], [g], [m], [v], [sh], 1e-3, 0.9, 0.95, 1e-8, 0.1, 3)
        bytes_ = n * (16 + 14)
    else:
        raise SystemExit(f"unknown case {args.case}")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(args.iters - 1):
        fn()
    torch.cuda.synchronize()
    start.record()
    fn()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    K.check_error()
    rate = f"{flops / ms / 1e9:.0f} TFLOP/s" if flops else f"{bytes_ / ms / 1e6:.0f} GB/s"
    print(f"{args.case}: {ms * 1e3:.1f} us  {rate}")


if __name__ == "__main__":
    main()
