"""Fused GEMM+collective kernels against their unfused equivalents (one rank per GPU, launched with torchrun).

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 -m benchmarks.bench_gemm_comm

For every shape: ``ag_gemm`` vs NCCL ``all_gather_into_tensor`` followed by the tcgen05 GEMM, and ``gemm_rs`` vs the
GEMM followed by NCCL ``reduce_scatter_tensor`` of the fp32 product.  Device time with CUDA events, max over ranks,
and the roofline bound max(FLOPs / GEMM peak, NVLink bytes / link bandwidth) for each fused kernel.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

GEMM_PEAK = 1.4e15   # sustained bf16 dense FLOP/s used for the bound
LINK_BW = 770e9      # measured peer-copy bandwidth per direction


def timed(fn, iters=20, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, dist.ReduceOp.MAX)
    return t.item()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.core.symm import SymmComm
    from torchure_b200.ops import kernels
    from torchure_b200.ops.gemm_comm import SymmetricOperand, ag_gemm, gemm_rs

    mesh = Mesh({"tp": world})
    comm = SymmComm(mesh.get_group("tp"), rank, world, staging_bytes=1 << 20, persistent_bytes=3 << 29)
    group = mesh.get_group("tp")
    rows = []
    # (M total tokens, K, N): column-parallel up-projections (ag_gemm) and row-parallel down-projections (gemm_rs)
    shapes = [(8192, 1024, 4096), (8192, 1024, 6144), (8192, 2560, 9728), (16384, 4096, 4096)]
    for M, K, N in shapes:
        if M % (128 * world):
            continue
        Nl = N // world
        a_sh = SymmetricOperand(comm, (M // world, K), torch.bfloat16)
        a_sh.tensor.normal_()
        b = torch.randn(Nl, K, device="cuda").bfloat16()
        out = torch.empty(M, Nl, device="cuda", dtype=torch.bfloat16)
        gathered = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)

        def unfused_ag():
            dist.all_gather_into_tensor(gathered, a_sh.tensor, group=group)
            kernels.gemm(gathered, b, out=out)

        g_sh = SymmetricOperand(comm, (M, K), torch.bfloat16)
        t_f = timed(lambda: ag_gemm(comm, a_sh, b, out, g_sh))
        t_u = timed(unfused_ag)
        t_g = timed(lambda: kernels.gemm(gathered, b, out=out))
        flops = 2.0 * M * K * Nl
        bound = max(flops / GEMM_PEAK, (M // world) * K * 2 * (world - 1) / LINK_BW) * 1e3
        rows.append({"op": "ag_gemm", "M": M, "K": K, "N_local": Nl, "fused_ms": t_f, "nccl_then_gemm_ms": t_u,
                     "gemm_only_ms": t_g, "bound_ms": bound, "of_bound": bound / t_f})
        # row-parallel: A [M, K/world] local, out fp32 [M/world, N]
        Kl = N // world  # reuse N as the (large) contraction dim, K as the output width
        a = torch.randn(M, Kl, device="cuda").bfloat16()
        w = torch.randn(K, Kl, device="cuda").bfloat16()
        c_sh = SymmetricOperand(comm, (M // world, K), torch.float32)
        full = torch.empty(M, K, device="cuda", dtype=torch.float32)
        shard = torch.empty(M // world, K, device="cuda", dtype=torch.float32)

        def unfused_rs():
            kernels.gemm(a, w, out=full, out_dtype=torch.float32)
            dist.reduce_scatter_tensor(shard, full, group=group)

        t_f = timed(lambda: gemm_rs(comm, a, w, c_sh))
        t_u = timed(unfused_rs)
        t_g = timed(lambda: kernels.gemm(a, w, out=full, out_dtype=torch.float32))
        flops = 2.0 * M * Kl * K
        bound = max(flops / GEMM_PEAK, (M // world) * K * 4 * (world - 1) / LINK_BW) * 1e3
        rows.append({"op": "gemm_rs", "M": M, "K_local": Kl, "N": K, "fused_ms": t_f, "gemm_then_nccl_ms": t_u,
                     "gemm_only_ms": t_g, "bound_ms": bound, "of_bound": bound / t_f})
        del a_sh, c_sh
    comm.check()
    kernels.check_error()
    if rank == 0:
        for r in rows:
            print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()}))
        if args.out:
            with open(args.out, "w") as f:
                json.dump({"world": world, "rows": rows}, f, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
