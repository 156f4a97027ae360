"""Headline benchmark: Qwen3-0.6B bf16 training tokens/sec at seq 4096, micro-batch 2 per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model 0.6b|4b]

For N > 1 launch under torchrun (one rank per GPU); when started as a plain process with
``--gpus N`` it re-launches itself under ``python -m torch.distributed.run``.

Both arms run the same configuration (28 layers, hidden 1024, 16/8 heads, head_dim 128,
ffn 3072, vocab 151936, tied embeddings; synthetic packed tokens; random init; fused
linear+CE chunk 4096; AdamW lr 3e-4 + WSD; grad clip 1.0; DDP bucket 25 MB; weak scaling)
through each side's public ``Trainer``:

* ``--impl ours``       ``torchure_b200.train.trainer.Trainer`` (hand-written sm_100a kernels).
* ``--impl reference``  the unmodified reference installed under ``baseline/_ref`` driven
  through its own ``Trainer.train_step`` (``baseline/run_reference.py``); only its network
  dependent tokenizer/dataset constructors are replaced by the synthetic source.

Timing: W >= 3 untimed steps, then exactly K steps between CUDA events, bracketed by a
barrier and a device synchronise on both sides; the reported time is the maximum over
ranks.  The working set of a step (>10 GB of weights and activations) is far larger than
the 126 MB L2, so no explicit L2 flush is needed.  ``e2e`` repeats the K steps with the
per-step host-to-device batch copy from pinned memory (always part of a step) and a
device-to-host read of the step's loss inside the timed region.  Neither arm synchronises
inside the timed steps of ``value`` and ``e2e`` (``config.sync_per_step`` false: the reference's
step body is called without its ``record_time`` bracket); ``synced`` repeats the K steps through
each side's public sync-bracketed ``train_step``.  ``kernel_census`` comes from one extra
untimed step under ``torch.profiler``.  SM clocks and throttle reasons are sampled with
nvidia-smi during the timed region.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODELS = {
    "0.6b": dict(num_layers=28, num_heads=16, num_kv_heads=8, emb_dim=1024, head_dim=128, vocab_size=151936,
                 ffn_dim=3072),
    "4b": dict(num_layers=36, num_heads=32, num_kv_heads=8, emb_dim=2560, head_dim=128, vocab_size=151936,
               ffn_dim=9728),
}
MICRO_BATCH = {"0.6b": 2, "4b": 1}
SEQ_LEN = 4096
# no B200 number is published for the reference; the only published single-GPU figure is H100 NVL
PUBLISHED_TPS_1GPU_H100 = 54_500.0


def bench_mesh(parallel: str, n_gpus: int) -> dict:
    """dp: DDP (the headline).  fsdp / hsdp2 / tp2 / cp2: the other strategies the mesh can select, for comparison rows."""
    if parallel == "fsdp":
        return {"dp_shard": n_gpus}
    if parallel == "hsdp2":
        return {"dp_replicate": 2, "dp_shard": n_gpus // 2}
    if parallel in ("tp2", "tp2sp", "tp2lp"):
        return {"dp": n_gpus // 2, "tp": 2}
    if parallel == "cp2":
        return {"dp": n_gpus // 2, "cp": 2}
    return {"dp": n_gpus}


def bench_config(model: str, n_gpus: int, total_steps: int, micro_batch: int | None = None, chunk: int = 4096,
                 parallel: str = "dp") -> dict:
    mbs = micro_batch or MICRO_BATCH[model]
    mesh = bench_mesh(parallel, n_gpus)
    replicas = n_gpus // (mesh.get("tp", 1) * mesh.get("cp", 1))      # ranks that see different data
    return {
        "model": {"name": "qwen3_dense", "config": dict(MODELS[model])},
        "mesh": mesh,
        "optimizer": {"name": "adamw",
                      "config": {"lr": 3e-4, "weight_decay": 0.1, "betas": [0.9, 0.95], "fused": True},
                      "max_norm": 1.0,
                      "scheduler": {"type": "wsd", "warmup_ratio": 0.001, "decay_ratio": 0.1,
                                    "total_steps": max(100, total_steps)}},
        "objective": {"name": "AR", "config": {"ignore_index": -100, "fused_linear_ce": True, "ce_chunk_size": chunk}},
        "data": {"name": "synthetic", "synthetic": True, "seed": 42, "mean_doc_len": 1024, "eos_id": 151643,
                 "tokenizer": "synthetic", "eos_token": "<eos>", "pad_token": "<pad>", "text_field": "text",
                 "shuffle_buffer": 0, "num_workers": 0, "global_batch_size": mbs * replicas, "micro_batch_size": mbs,
                 "seq_len": SEQ_LEN},
        "ddp": {"bucket_mb": 25},
        "checkpointing": {"save_steps": 10 ** 9, "resume": None},
        "run_name": f"bench_{model}_dp{n_gpus}",
    }


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampler for the local GPU (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self) -> None:
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                    power.append(float(parts[3]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def relaunch_under_torchrun(args) -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
    return subprocess.call(cmd)


def timed_steps(step_fn, k: int, read_loss: bool):
    """Run k steps between CUDA events; returns device milliseconds (this rank).

    With `read_loss` every step's loss is brought to the host inside the timed region: an asynchronous copy into
    pinned memory right after the step is enqueued, consumed (event wait + read) after the NEXT step has been
    enqueued, so the host never drains the device queue to log a number; the last one is read before the stop event.
    """
    import torch
    import torch.distributed as dist

    dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    slots = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)] if read_loss else None
    ready = [torch.cuda.Event(), torch.cuda.Event()] if read_loss else None
    t0 = time.perf_counter()
    start.record()
    last = None
    for i in range(k):
        out = step_fn()
        if read_loss:
            slots[i % 2].copy_(out["loss"].detach().reshape(1), non_blocking=True)  # device-to-host read of the result
            ready[i % 2].record()
            if i > 0:
                ready[(i - 1) % 2].synchronize()
                last = float(slots[(i - 1) % 2][0])
    if read_loss:
        ready[(k - 1) % 2].synchronize()
        last = float(slots[(k - 1) % 2][0])
    stop.record()
    enqueue_ms = (time.perf_counter() - t0) * 1e3  # host time to enqueue the k steps
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    timed_steps.last_enqueue_ms = enqueue_ms
    dist.barrier()
    return start.elapsed_time(stop), wall_ms, last


def shared_config(model: str, cfg: dict, world: int, ce_chunk: int) -> dict:
    """The `config` object both arms print: identical keys and values for identical work."""
    mbs = cfg["data"]["micro_batch_size"]
    mesh = cfg["mesh"]
    par = f"dp{world}" if list(mesh) == ["dp"] else "x".join(f"{k}{v}" for k, v in mesh.items())
    par += "".join(f"+{k}" for k, v in sorted(cfg.get("tp", {}).items()) if v)    # sequence_parallel / loss_parallel
    return {"model": f"qwen3-{model}", "ffn_dim": cfg["model"]["config"]["ffn_dim"],
            "global_batch": cfg["data"]["global_batch_size"],
            "micro_batch": mbs, "seq_len": cfg["data"]["seq_len"], "parallelism": par, "ce_chunk": ce_chunk,
            "grad_clip": 1.0, "ddp_bucket_mb": cfg["ddp"]["bucket_mb"], "sync_per_step": False,
            "l2": "per-step working set (>10 GB) exceeds the 126 MB L2; no explicit flush"}


def kernel_census(step_fn, top: int = 40) -> dict:
    """One extra, untimed step under torch.profiler: launches and device time per kernel name, with the kernels
    of this repository, NCCL's and everything else (library / framework kernels) counted apart."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step_fn()
        torch.cuda.synchronize()
    rows = {}
    for ev in prof.events():
        if ev.device_type.name != "CUDA" or not ev.name or ev.name.startswith(("Memcpy", "Memset")):
            continue
        r = rows.setdefault(ev.name, [0, 0.0])
        r[0] += 1
        r[1] += ev.device_time if hasattr(ev, "device_time") else ev.cuda_time
    own_marks = ("tb::", "gemm_bf16_kernel", "gemm_comm_kernel", "attn_", "rmsnorm", "qknorm", "swiglu", "ce_softmax",
                 "adamw_kernel", "all_reduce_kernel", "all_gather_kernel", "reduce_scatter_kernel", "all_to_all_kernel",
                 "broadcast_kernel", "barrier_kernel", "embedding_bwd", "cast_", "scale_", "sqnorm", "bucket_pack",
                 "finalize_kernel")

    def kind(name: str) -> str:
        if "nccl" in name.lower():
            return "nccl"
        return "own" if any(m in name for m in own_marks) else "other"

    out = {"own": {"launches": 0, "us": 0.0}, "nccl": {"launches": 0, "us": 0.0}, "other": {"launches": 0, "us": 0.0}}
    for name, (n, us) in rows.items():
        k = kind(name)
        out[k]["launches"] += n
        out[k]["us"] += us
    ranked = sorted(rows.items(), key=lambda kv: -kv[1][1])[:top]
    out["top"] = [{"name": n[:96], "kind": kind(n), "launches": c, "us": round(us, 1)} for n, (c, us) in ranked]
    for k in ("own", "nccl", "other"):
        out[k]["us"] = round(out[k]["us"], 1)
    return out


def max_over_ranks(x: float) -> float:
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from torchure_b200 import ops
    from torchure_b200.train.train import init_distributed
    from torchure_b200.train.trainer import Trainer

    if not torch.cuda.is_available():
        # the benchmark is a GPU measurement: without a device say so instead of grinding through the model on CPU
        print(json.dumps({"impl": "ours", "unavailable": "no CUDA device"}))
        return
    rank, local_rank, world = init_distributed()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    cfg = bench_config(args.model, world, args.steps * 2 + args.warmup + 8, args.micro_batch, args.ce_chunk,
                       args.parallel)
    if args.torch_path:
        cfg["compile"] = False
    if args.parallel == "tp2sp":
        # sequence parallelism: the block linears run as the fused all-gather -> GEMM and GEMM -> reduce-scatter kernels
        cfg["tp"] = {"sequence_parallel": True}
    if args.parallel == "tp2lp":
        # loss-parallel head: every rank computes V / tp rows of the logits inside the chunked CE
        cfg["tp"] = {"loss_parallel": True}
        cfg["comm"] = {"max_bytes": 1 << 30}    # room for the gather of the head-gradient row slices (311 MB per rank)
    cfg["cuda_graph"] = bool(args.graph) and not args.torch_path and args.parallel not in ("tp2sp", "cp2")
    trainer = Trainer(cfg, rank, local_rank, world, benchmark=True)
    step = trainer.train_step_untimed
    for _ in range(max(5, args.warmup)):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ops.reset_launches()
    dev_ms, _, _ = timed_steps(step, args.steps, read_loss=False)
    launches = ops.launches()
    host_enqueue_ms = timed_steps.last_enqueue_ms / args.steps
    e2e_ms, _, last_loss = timed_steps(step, args.steps, read_loss=True)
    # the same steps through the public sync-bracketed `train_step` (how the reference times itself)
    sync_ms, _, _ = timed_steps(lambda: trainer.train_step()[0], args.steps, read_loss=False)
    clocks = sampler.stop() if rank == 0 else None
    trainer.check_device_errors()   # an expired device-side wait would make every number above meaningless
    dev_ms, e2e_ms, sync_ms = max_over_ranks(dev_ms), max_over_ranks(e2e_ms), max_over_ranks(sync_ms)
    census = None
    if args.census:
        eager = trainer.use_cuda_graph
        trainer.use_cuda_graph = False        # kernels inside a replayed graph carry no names in the profiler
        step()
        census = kernel_census(step) if rank == 0 else step()
        trainer.use_cuda_graph = eager
    tokens = SEQ_LEN * cfg["data"]["global_batch_size"] * args.steps
    if rank == 0:
        value = tokens / (dev_ms / 1e3)
        print(json.dumps({
            "metric": "Qwen3-0.6B bf16 global tokens/sec @seq4096 bs2/GPU" if args.model == "0.6b"
                      else "Qwen3-4B bf16 global tokens/sec @seq4096 bs1/GPU",
            "impl": "ours", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(5, args.warmup), "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": value / (PUBLISHED_TPS_1GPU_H100 * world) if args.model == "0.6b" else None,
            "vs_baseline_note": "published reference number is 54.5k tok/s on 1x H100 NVL (no B200 number exists)",
            "dtype": "bf16", "data": "synthetic packed uniform tokens, random-init weights",
            "config": shared_config(args.model, cfg, world, args.ce_chunk),
            "kernels": "sm100" if ops.available() and not args.torch_path else "torch-oracle",
            "launch": "cuda-graph replay" if trainer.use_cuda_graph else "eager",
            "synced": {"value": tokens / (sync_ms / 1e3), "unit": "tokens/s", "ms_per_step": sync_ms / args.steps,
                       "note": "device synchronize before and after every step (Trainer.train_step)"},
            "kernel_census": census,
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": trainer.prefetcher.h2d_bytes * trainer.microbatches_per_step,
                    "d2h_bytes_per_step": 4, "last_loss": last_loss,
                    "loss_read": "async copy to pinned memory every step, consumed one step later"},
            "gpu_launches": launches, "host_enqueue_ms_per_step": host_enqueue_ms, "clocks": clocks,
            "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
        }), flush=True)
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", choices=sorted(MODELS), default="0.6b")
    ap.add_argument("--micro-batch", type=int, default=None)
    ap.add_argument("--ce-chunk", type=int, default=4096)
    ap.add_argument("--torch-path", action="store_true", help="ours: run the PyTorch oracle path (A/B)")
    ap.add_argument("--graph", type=int, default=1, help="ours: replay the device step from one CUDA graph (1) or launch eagerly (0)")
    ap.add_argument("--parallel", choices=["dp", "fsdp", "hsdp2", "tp2", "tp2sp", "tp2lp", "cp2"], default="dp",
                    help="ours: strategy selected through the mesh (dp = DDP is the headline configuration)")
    ap.add_argument("--census", type=int, default=1, help="one extra untimed step under torch.profiler: kernel census")
    args = ap.parse_args()
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        sys.exit(relaunch_under_torchrun(args))
    if args.impl == "reference":
        from baseline.run_reference import run_reference

        run_reference(args, bench_config(args.model, args.gpus, args.steps * 2 + args.warmup + 8,
                                         args.micro_batch, args.ce_chunk), timed_steps, max_over_ranks, ClockSampler,
                      shared_config, kernel_census)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
