"""Bus-bandwidth sweep of the mesh collectives: our NVLink kernels against the NCCL path of the same call.

    torchrun --nproc-per-node N -m benchmarks.bench_collectives [--max-mb 1024] [--stride 1] [--out sweep.json]

For every op (all_reduce, all_gather, reduce_scatter, all_to_all), dtype (bf16, fp32) and per-rank message size
(powers of two from 1 KiB, N(0,1) values) it times both transports with CUDA events after warm-up, takes the
maximum over ranks and reports bus bandwidth with the usual conventions (all_reduce: 2(n-1)/n * bytes / t;
all_gather / reduce_scatter: (n-1)/n * total bytes / t; all_to_all: (n-1)/n * bytes / t).

``--symmetric`` adds the in-place paths on tensors that live in the symmetric allocation, which are what training
uses (no staging copy): ``ar_symm`` is the DDP bucket all-reduce (two-shot, 1/world scale and sum of squares fused),
``ag_inplace`` / ``rs_symm`` are FSDP's weight all-gather and gradient reduce-scatter.  Their NCCL column is the
library collective on an ordinary tensor of the same size.  For ``ar_symm`` the line also gives the fraction of the
NVLink bound at ``--link-gbs`` per direction (default 770 GB/s, the measured peer copy rate): 2 (n-1)/n of the
message per direction with peer loads and stores, one message per direction with multimem (the switch reduces and
replicates).
"""

from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist


def _time(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    t = torch.tensor([start.elapsed_time(stop) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None) -> None:
    from torchure_b200.core import collective as C
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.train.train import init_distributed

    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--out", default=None)
    ap.add_argument("--stride", type=int, default=1, help="take every stride-th power of two (a quick sweep)")
    ap.add_argument("--symmetric", action="store_true", help="also time the in-place symmetric-memory paths")
    ap.add_argument("--symmetric-mb", type=float, nargs="*", default=[24, 594],
                    help="message sizes (MiB, fp32) of the symmetric paths: a DDP bucket and the tied embedding")
    ap.add_argument("--blocks", type=int, nargs="*", default=[16, 128], help="CTAs of the symmetric kernels")
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--only-symmetric", action="store_true")
    args = ap.parse_args(argv)
    rank, _, world = init_distributed()
    mesh = Mesh({"dp": world})
    ours = Mesh({"dp": world})
    comm = C.enable_sm100(ours, "dp", max_bytes=(args.max_mb << 20) * (world + 2) + (64 << 20))
    rows = []
    sizes = [1 << k for k in range(10, 31, args.stride) if (1 << k) <= (args.max_mb << 20)]
    if args.only_symmetric:
        sizes = []
    if args.symmetric or args.only_symmetric:
        from torchure_b200.core.symm import SymmComm

        top = int(max(args.symmetric_mb) * (1 << 20))
        sc = SymmComm(mesh.get_group("dp"), rank, world, staging_bytes=4096, persistent_bytes=2 * top + (1 << 20))
        buf = sc.alloc(top // 4, torch.float32)
        buf.normal_()
        for mb in args.symmetric_mb:
            n = int(mb * (1 << 20)) // 4 // (64 * world) * (64 * world)
            nbytes = n * 4
            t = buf[:n]
            shard = torch.empty(n // world, device="cuda")
            plain = torch.randn(n, device="cuda")
            out_g = torch.empty(n, device="cuda")
            nccl = {"ar_symm": _time(lambda: dist.all_reduce(plain), 5),
                    "ag_inplace": _time(lambda: dist.all_gather_into_tensor(out_g, plain[: n // world]), 5),
                    "rs_symm": _time(lambda: dist.reduce_scatter_tensor(shard, plain), 5)}
            for blocks in args.blocks:
                cases = {"ar_symm": (lambda: sc.all_reduce_symmetric_(t, "avg", sq_slot=0, blocks=blocks),
                                     2 * (world - 1) / world * nbytes),
                         "ag_inplace": (lambda: sc.all_gather_inplace_([t], blocks=blocks), (world - 1) / world * nbytes),
                         "rs_symm": (lambda: sc.reduce_scatter_symmetric([t], [shard], "avg", sq_slot=0, blocks=blocks),
                                     (world - 1) / world * nbytes)}
                for op, (fn, bus_bytes) in cases.items():
                    t_ours = _time(fn, 5)
                    one_way = (world - 1) / world * nbytes      # bytes over this rank's links, each direction
                    bound_ms = one_way / (args.link_gbs * 1e6) * (2 if op == "ar_symm" else 1)
                    if op == "ar_symm" and sc.mc:
                        # in-switch reduction and replication: (n-1)/n out + 1/n back for the reduce, 1/n out +
                        # (n-1)/n back for the broadcast = one message per direction
                        bound_ms = nbytes / (args.link_gbs * 1e6)
                    rows.append({"op": op, "dtype": "float32", "bytes": nbytes, "world": world, "blocks": blocks,
                                 "ours_ms": t_ours, "nccl_ms": nccl[op], "ours_busbw_gbs": bus_bytes / t_ours / 1e6,
                                 "nccl_busbw_gbs": bus_bytes / nccl[op] / 1e6, "nvlink_bound_ms": bound_ms,
                                 "fraction_of_bound": bound_ms / t_ours})
                    if rank == 0:
                        r = rows[-1]
                        print(f"{op:11s} {mb:6.0f} MiB {blocks:4d} CTAs  ours {t_ours:8.3f} ms {r['ours_busbw_gbs']:7.1f} GB/s"
                              f" | nccl {nccl[op]:8.3f} ms {r['nccl_busbw_gbs']:7.1f} GB/s | bound {bound_ms:.3f} ms "
                              f"({r['fraction_of_bound']:.2f})", flush=True)
        sc.check()
    for dtype in (torch.bfloat16, torch.float32):
        es = 2 if dtype == torch.bfloat16 else 4
        for nbytes in sizes:
            n = nbytes // es
            x = torch.randn(n, device="cuda").to(dtype)
            big = torch.randn(n * world, device="cuda").to(dtype) if nbytes * world <= (2 << 30) else None
            iters = 20 if nbytes <= (16 << 20) else 5
            cases = {
                "all_reduce": (lambda m: C.all_reduce(x, m, "dp", "sum"), 2 * (world - 1) / world * nbytes),
                "all_gather": (lambda m: C.all_gather(x, m, "dp", 0), (world - 1) / world * nbytes * world),
                "all_to_all": (lambda m: C.all_to_all(x[: n // world * world], m, "dp", 0, 0), (world - 1) / world * nbytes),
            }
            if big is not None:
                cases["reduce_scatter"] = (lambda m: C.reduce_scatter(big, m, "dp", "sum"),
                                           (world - 1) / world * nbytes * world)
            for op, (fn, bus_bytes) in cases.items():
                if op == "all_to_all" and n < world:
                    continue
                t_ours = _time(lambda: fn(ours), iters)
                t_nccl = _time(lambda: fn(mesh), iters)
                rows.append({"op": op, "dtype": str(dtype).split(".")[-1], "bytes": nbytes, "world": world,
                             "ours_ms": t_ours, "nccl_ms": t_nccl, "ours_busbw_gbs": bus_bytes / t_ours / 1e6,
                             "nccl_busbw_gbs": bus_bytes / t_nccl / 1e6})
                if rank == 0:
                    r = rows[-1]
                    print(f"{op:14s} {r['dtype']:8s} {nbytes:>11d} B  ours {t_ours * 1e3:9.1f} us {r['ours_busbw_gbs']:7.1f} GB/s"
                          f" | nccl {t_nccl * 1e3:9.1f} us {r['nccl_busbw_gbs']:7.1f} GB/s", flush=True)
    comm.check()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
