"""Causal GQA attention, forward and backward: the sm_100a kernels against the library path the reference calls.

    python -m benchmarks.bench_attention [--B 2] [--S 4096] [--Hq 16] [--Hkv 8] [--iters 20]

"ours" are ``attn_fwd``, the single-pass backward ``attn_bwd_fused`` (statistics pass, accumulator clear, fused
kernel and dQ conversion all inside the timed region) and the two-kernel backward ``attn_bwd``; "sdpa" is
``torch.nn.functional.scaled_dot_product_attention`` (reference call site: ``torchure/models/qwen3/qwen3.py:184-185``)
and its autograd backward.  CUDA events around `iters` back-to-back launches after warm-up; the inputs of one call
(B=2, S=4096: 270 MB with outputs) exceed the L2, and a 256 MB buffer is rewritten between timed launches when
``--flush`` is given.  FLOP counts are algorithmic: 2 causal products forward, 5 backward.
"""

from __future__ import annotations

import argparse
import json

import torch
import torch.nn.functional as F


def main(argv=None) -> None:
    from torchure_b200 import ops
    from torchure_b200.ops import kernels

    ap = argparse.ArgumentParser()
    ap.add_argument("--B", type=int, default=2)
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--Hq", type=int, default=16)
    ap.add_argument("--Hkv", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--flush", action="store_true")
    args = ap.parse_args(argv)
    B, S, Hq, Hkv, hd = args.B, args.S, args.Hq, args.Hkv, 128
    torch.manual_seed(0)
    qk = torch.randn(B * S, (Hq + Hkv) * hd, device="cuda").bfloat16()
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * hd, device="cuda").bfloat16()
    o = torch.empty(B * S, Hq * hd, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, Hq, S, device="cuda")
    d_o = torch.randn(B * S, Hq * hd, device="cuda").bfloat16()
    dqkv = torch.empty(B * S, (Hq + 2 * Hkv) * hd, dtype=torch.bfloat16, device="cuda")
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if args.flush else None

    def timed(fn) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        if scrub is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / args.iters
        for _ in range(args.iters):
            scrub.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / args.iters

    unit = 2.0 * S * S * hd * Hq * B / 2  # one causal S x S x hd product over all heads
    res = {"shape": {"B": B, "S": S, "Hq": Hq, "Hkv": Hkv, "hd": hd}, "flush_l2": bool(args.flush)}
    ext = ops.ext()
    res["fwd_ours_ms"] = timed(lambda: ext.attn_fwd(qk, qkv, o, lse, B, S, Hq, Hkv))
    res["bwd_fused_ms"] = timed(lambda: ext.attn_bwd_fused(d_o, qk, qkv, o, lse, dqkv, B, S, Hq, Hkv))
    res["bwd_split_ms"] = timed(lambda: ext.attn_bwd(d_o, qk, qkv, o, lse, dqkv, B, S, Hq, Hkv))
    kernels.check_error()
    q = qk[:, :Hq * hd].view(B, S, Hq, hd).transpose(1, 2)
    k = qk[:, Hq * hd:].view(B, S, Hkv, hd).transpose(1, 2)
    v = qkv[:, (Hq + Hkv) * hd:].view(B, S, Hkv, hd).transpose(1, 2)
    res["fwd_sdpa_ms"] = timed(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=Hq != Hkv))
    ql, kl, vl = (x.detach().requires_grad_() for x in (q, k, v))
    out = F.scaled_dot_product_attention(ql, kl, vl, is_causal=True, enable_gqa=Hq != Hkv)
    g = d_o.view(B, S, Hq, hd).transpose(1, 2)
    res["bwd_sdpa_ms"] = timed(lambda: torch.autograd.grad(out, (ql, kl, vl), g, retain_graph=True))
    for key, mult in (("fwd_ours", 2), ("fwd_sdpa", 2), ("bwd_fused", 5), ("bwd_split", 5), ("bwd_sdpa", 5)):
        res[key + "_tflops"] = mult * unit / res[key + "_ms"] / 1e9
    print(json.dumps(res))


if __name__ == "__main__":
    main()
