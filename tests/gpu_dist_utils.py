"""Spawn one process per GPU on this node (NCCL bootstrap) and run a function in each."""

from __future__ import annotations

import os
import tempfile
import traceback
from datetime import timedelta

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.dist_utils import free_port


def _entry(rank, world, port, fn, args, errq, env, store_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank),
                      WORLD_SIZE=str(world), **env)
    try:
        torch.cuda.set_device(rank)
        # a file store: no listening socket, so a port that another process grabbed cannot fail the rendezvous
        store = dist.FileStore(store_path, world)
        dist.init_process_group("nccl", store=store, rank=rank, world_size=world, timeout=timedelta(seconds=120),
                                device_id=torch.device(f"cuda:{rank}"))
        fn(rank, world, *args)
        torch.cuda.synchronize()
        dist.barrier()
    except Exception:
        errq.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_on_gpus(fn, world: int, *args, timeout_s: int = 150, env: dict | None = None):
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = free_port()
    store_dir = tempfile.mkdtemp(prefix="tb_gpu_store_")
    store_path = os.path.join(store_dir, "store")
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq, env or {}, store_path))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout_s)
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            errors.append((-1, "a rank did not exit in time"))
        elif p.exitcode != 0 and not errors:
            errors.append((-1, f"a rank exited with code {p.exitcode}"))
    if errors:
        raise AssertionError("\n".join(f"[rank {r}]\n{tb}" for r, tb in errors))
