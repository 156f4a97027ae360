"""Entry point: ``python -m torchure_b200.train.train --config cfg.json [--steps N]``.

Same code path for one process and for torchrun: missing rendezvous variables default to a
single local rank, the device is selected before the process group is created, and the
group is destroyed on the way out (reference ``torchure/train/train.py:45-87``).
``--steps N`` runs N optimizer steps in benchmark mode (no checkpoints, no wandb).
"""

from __future__ import annotations

import argparse
import os
from datetime import timedelta

import torch
import torch.distributed as dist


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description="torchure_b200 trainer")
    ap.add_argument("--config", required=True, help="path to the JSON run config")
    ap.add_argument("--steps", type=int, default=None, help="benchmark mode: run this many steps and exit")
    ap.add_argument("--backend", default=None, help="process-group backend (default: nccl on GPUs, gloo on CPU)")
    return ap.parse_args(argv)


def init_distributed(backend: str | None = None, timeout_s: int = 600):
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    rank, local_rank, world = (int(os.environ[k]) for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"))
    on_gpu = torch.cuda.is_available()
    if on_gpu:
        torch.cuda.set_device(local_rank)
    if backend is None:
        backend = "nccl" if on_gpu else "gloo"
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device(f"cuda:{local_rank}")
        dist.init_process_group(backend=backend, timeout=timedelta(seconds=timeout_s), **kw)
    return rank, local_rank, world


def main(argv=None) -> None:
    args = parse_args(argv)
    rank, local_rank, world = init_distributed(args.backend)
    try:
        from torchure_b200.train.trainer import Trainer

        trainer = Trainer(args.config, rank, local_rank, world, benchmark=args.steps is not None)
        if args.steps is not None:
            trainer.train_n_step_test(args.steps)
        else:
            trainer.train()
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
