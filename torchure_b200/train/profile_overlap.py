"""Communication/compute overlap profiler.

    python -m torchure_b200.train.profile_overlap --config cfg.json --out trace.json [--warmup 10 --steps 2]
    python -m torchure_b200.train.profile_overlap --analyze trace.json [--steps 2]

``capture`` runs warm-up steps, synchronises, records ``steps`` optimizer steps under ``torch.profiler`` (CPU+CUDA)
and rank 0 exports a chrome trace; ``analyze`` is pure JSON post-processing (no GPU, no rendezvous) and prints, per
step: device time of compute kernels, of communication kernels, how much communication was hidden under compute,
how much was exposed, GPU idle time, the top kernels with their exposure, and per-stream busy time
(reference: ``torchure/train/profile_overlap.py:97-190``).

The reference classifies communication by the substring "nccl".  Here the gradient all-reduce is our own kernel, so
a kernel counts as communication when its name matches one of ``COMM_PATTERNS`` (our collective kernels and NCCL).
"""

from __future__ import annotations

import argparse
import json
import os

COMM_PATTERNS = ("nccl", "all_reduce_kernel", "all_gather_kernel", "reduce_scatter_kernel", "all_to_all_kernel",
                 "broadcast_kernel", "barrier_kernel", "ag_gemm", "gemm_rs", "all_gather_inplace_kernel",
                 "reduce_scatter_symm_kernel", "embedding_scatter_kernel")
GPU_CATS = ("kernel", "gpu_memcpy", "gpu_memset")


def union(intervals: list[tuple[float, float]]) -> list[tuple[float, float]]:
    out: list[list[float]] = []
    for lo, hi in sorted(intervals):
        if out and lo <= out[-1][1]:
            out[-1][1] = max(out[-1][1], hi)
        else:
            out.append([lo, hi])
    return [(a, b) for a, b in out]


def total_len(intervals) -> float:
    return sum(b - a for a, b in intervals)


def intersect_len(a, b) -> float:
    """Length of the intersection of two sorted, disjoint interval lists."""
    i = j = 0
    acc = 0.0
    while i < len(a) and j < len(b):
        lo, hi = max(a[i][0], b[j][0]), min(a[i][1], b[j][1])
        if hi > lo:
            acc += hi - lo
        if a[i][1] < b[j][1]:
            i += 1
        else:
            j += 1
    return acc


def short_name(name: str) -> str:
    """Kernel name without the anonymous-namespace marker and the parameter list (template arguments are kept)."""
    name = name.replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
    if name.startswith("void "):
        name = name[5:]
    depth = 0
    for i, ch in enumerate(name):
        if ch == "<":
            depth += 1
        elif ch == ">":
            depth -= 1
        elif ch == "(" and depth == 0:
            return name[:i][:70]
    return name[:70]


def is_comm(name: str) -> bool:
    low = name.lower()
    return any(p in low for p in COMM_PATTERNS)


def analyze(path: str, steps: int = 2, top: int = 8) -> dict:
    with open(path) as f:
        trace = json.load(f)
    events = [e for e in trace["traceEvents"] if e.get("ph") == "X" and e.get("cat") in GPU_CATS]
    if not events:
        raise SystemExit("no GPU events in the trace")
    comp = [(e["ts"], e["ts"] + e["dur"]) for e in events if not is_comm(e["name"])]
    comm = [(e["ts"], e["ts"] + e["dur"]) for e in events if is_comm(e["name"])]
    ucomp, ucomm = union(comp), union(comm)
    span = max(e["ts"] + e["dur"] for e in events) - min(e["ts"] for e in events)
    busy = total_len(union(comp + comm))
    hidden = intersect_len(ucomm, ucomp)
    comm_t, comp_t = total_len(ucomm), total_len(ucomp)
    res = {
        "steps": steps, "span_ms": span / 1e3 / steps, "compute_ms": comp_t / 1e3 / steps,
        "comm_ms": comm_t / 1e3 / steps, "hidden_ms": hidden / 1e3 / steps,
        "exposed_ms": (comm_t - hidden) / 1e3 / steps, "idle_ms": (span - busy) / 1e3 / steps,
        "hidden_pct": 100.0 * hidden / comm_t if comm_t else 0.0, "n_comm_kernels": len(comm) // max(1, steps),
    }
    print(f"per step over {steps} steps: span {res['span_ms']:.2f} ms | compute {res['compute_ms']:.2f} | "
          f"comm {res['comm_ms']:.2f} | hidden {res['hidden_ms']:.2f} ({res['hidden_pct']:.1f} %) | "
          f"exposed {res['exposed_ms']:.2f} | idle {res['idle_ms']:.2f} | comm kernels {res['n_comm_kernels']}")
    # kernels by total device time
    by_name: dict[str, list[float]] = {}
    for e in events:
        by_name.setdefault(short_name(e["name"]), []).append(e["dur"])
    print("top kernels by device time (per step):")
    for name, durs in sorted(by_name.items(), key=lambda kv: -sum(kv[1]))[:top * 2]:
        print(f"  {sum(durs) / 1e3 / steps:8.3f} ms  x{len(durs) // max(1, steps):4d}  {name}")
    # longest communication kernels and how exposed each is
    if comm:
        print("largest communication kernels (duration, exposed share):")
        big = sorted((e for e in events if is_comm(e["name"])), key=lambda e: -e["dur"])[:top]
        biggest = big[0]["dur"]
        for e in big:
            iv = [(e["ts"], e["ts"] + e["dur"])]
            exposed = e["dur"] - intersect_len(iv, ucomp)
            print(f"  {e['dur'] / 1e3:8.3f} ms  exposed {100 * exposed / e['dur']:5.1f} %  {e['name'][:60]}")
        tail = [e for e in events if is_comm(e["name"]) and e["dur"] >= 0.9 * biggest]
        tail_exposed = sum(e["dur"] - intersect_len([(e["ts"], e["ts"] + e["dur"])], ucomp) for e in tail)
        res["structural_tail_ms"] = tail_exposed / 1e3 / steps
        print(f"structural tail (kernels >= 90 % of the largest): {res['structural_tail_ms']:.3f} ms exposed per step")
    streams: dict = {}
    for e in events:
        streams.setdefault(e.get("args", {}).get("stream", e.get("tid")), []).append((e["ts"], e["ts"] + e["dur"]))
    print("device time per stream (per step):")
    for sid, iv in sorted(streams.items(), key=lambda kv: -total_len(union(kv[1]))):
        print(f"  stream {sid}: {total_len(union(iv)) / 1e3 / steps:.2f} ms")
    return res


def capture(config: str, out: str, warmup: int, steps: int) -> None:
    import torch
    import torch.distributed as dist
    from torch.profiler import ProfilerActivity, profile

    from torchure_b200.train.train import init_distributed
    from torchure_b200.train.trainer import Trainer

    rank, local_rank, world = init_distributed()
    try:
        trainer = Trainer(config, rank, local_rank, world, benchmark=True)
        for _ in range(warmup):
            trainer.train_step_untimed()
        torch.cuda.synchronize()
        dist.barrier()
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            for _ in range(steps):
                trainer.train_step_untimed()
            torch.cuda.synchronize()
        if rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
            prof.export_chrome_trace(out)
            print(f"trace written to {out}")
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config")
    ap.add_argument("--out", default="traces/overlap_trace.json")
    ap.add_argument("--analyze", metavar="TRACE", default=None)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--steps", type=int, default=2)
    args = ap.parse_args(argv)
    if args.analyze:
        analyze(args.analyze, args.steps)
        return
    if not args.config:
        ap.error("--config is required to capture")
    capture(args.config, args.out, args.warmup, args.steps)
    if int(os.environ.get("RANK", "0")) == 0:
        analyze(args.out, args.steps)


if __name__ == "__main__":
    main()
