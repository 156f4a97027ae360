"""Spawn N gloo ranks on this host and run a function in each (CPU multi-rank tests).

Failures are produced on the host only: a rank raising makes the parent raise with that
rank's traceback; a deadlock ends by the process-group timeout instead of hanging.
"""

from __future__ import annotations

import os
import socket
import traceback
from datetime import timedelta

import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errq, timeout_s):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank),
                      WORLD_SIZE=str(world))
    try:
        import torch

        # the ranks share this host's cores: without a cap every rank starts one thread per core and they fight.  The
        # same count for every world size, so that a single-process reference sums its products in the same order
        torch.set_num_threads(2)
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=timeout_s))
        fn(rank, world, *args)
        dist.barrier()
    except Exception:
        errq.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_distributed(fn, world_size: int, *args, timeout_s: int = 60, join_s: int | None = None):
    # a fork server that has torch imported already: every rank starts as a fork of that single-threaded server
    # instead of a fresh interpreter that imports torch again (seconds per rank, dozens of ranks per session)
    ctx = mp.get_context("forkserver")
    ctx.set_forkserver_preload(["torch", "torch.distributed", "torch.multiprocessing"])
    errq = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world_size, port, fn, args, errq, timeout_s))
             for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(join_s or timeout_s * 3)   # process start-up (spawn + import torch) counts against this, not timeout_s
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            errors.append((-1, "a rank did not exit"))
        elif p.exitcode != 0 and not errors:
            errors.append((-1, f"a rank exited with code {p.exitcode}"))
    if errors:
        raise AssertionError("\n".join(f"[rank {r}]\n{tb}" for r, tb in errors))
