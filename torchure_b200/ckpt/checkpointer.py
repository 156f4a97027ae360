"""Step-directory checkpoints with a completion marker.

Layout (reference ``torchure/checkpoint/checkpointer.py:18-102`` and ``trainer.py:298-327``)::

    <root>/<completed_steps>/model.pt            model.state_dict() (fp32 master weights)
                             optimizer.pt        AdamW state_dict
                             scheduler.pt        LR scheduler state_dict
                             trainer.pt          {"step", "cpu_rng", "cuda_rng", "config", "wandb_id"}
                             dataloader_dp{r}.pt loader position of dp coordinate r
                             .complete           written last; a step without it does not exist

Files are written to a temporary name and renamed, so a crash leaves either the old file
or the new one.  ``latest()`` / ``valid_step()`` only see completed steps.  Sharded
strategies store per-shard files (``model_shard{r}.pt``, ``optimizer_shard{r}.pt``) in the
same directory.  With ``background=True`` (config ``checkpointing.async``) the files are written by a worker thread from
host snapshots while training goes on; the marker is only written once every rank's files are on disk.
``prune(keep_last)`` (config ``checkpointing.keep_last``) bounds the disk a long run uses.
"""

from __future__ import annotations

import os
from pathlib import Path

import torch

MARKER = ".complete"


def _host_snapshot(obj):
    """A copy of `obj` that later training steps cannot change: tensors copied to host memory, containers rebuilt,
    everything else deep-copied."""
    import copy

    if isinstance(obj, torch.Tensor):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return type(obj)((k, _host_snapshot(v)) for k, v in obj.items())
    if isinstance(obj, (list, tuple)):
        return type(obj)(_host_snapshot(v) for v in obj)
    return copy.deepcopy(obj)


class Checkpointer:
    def __init__(self, root: str, background: bool = False):
        """`background`: ``_write`` takes a host snapshot of its payload and returns; one worker thread serialises and
        renames the files in order.  ``wait()`` blocks until everything queued is on disk (and re-raises a failed
        write); the owner calls it before it marks a step complete."""
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)
        self.background = background
        self._queue = None
        self._worker = None
        self._failure: BaseException | None = None

    # -- background writer -------------------------------------------------------------------
    def _ensure_worker(self) -> None:
        import queue
        import threading

        if self._worker is not None:
            return
        self._queue = queue.Queue()

        def run():
            while True:
                job = self._queue.get()
                try:
                    if job is None:
                        return
                    if self._failure is None:
                        self._write_now(*job)
                except BaseException as e:      # reported by wait()
                    self._failure = e
                finally:
                    self._queue.task_done()

        self._worker = threading.Thread(target=run, name="checkpoint-writer", daemon=True)
        self._worker.start()

    def wait(self) -> None:
        if self._queue is not None:
            self._queue.join()
        if self._failure is not None:
            failure, self._failure = self._failure, None
            raise RuntimeError("a background checkpoint write failed") from failure

    # -- discovery -------------------------------------------------------------------------
    def _steps(self) -> list[int]:
        found = []
        for child in self.root.iterdir():
            if child.name.isdigit() and (child / MARKER).exists():
                found.append(int(child.name))
        return found

    def latest(self) -> int | None:
        steps = self._steps()
        return max(steps) if steps else None

    def valid_step(self, step: int) -> int | None:
        return step if step in self._steps() else None

    def step_dir(self, step: int, create: bool = False) -> Path:
        d = self.root / str(step)
        if create:
            d.mkdir(parents=True, exist_ok=True)
        return d

    def mark_complete(self, step: int) -> None:
        (self.step_dir(step, create=True) / MARKER).touch()

    def is_complete(self, step: int) -> bool:
        return (self.step_dir(step) / MARKER).exists()

    def prune(self, keep_last: int) -> list[int]:
        """Delete all but the newest `keep_last` COMPLETE steps (one caller per run: rank 0, after the newest step was
        marked).  A step loses its marker first, so an interrupted deletion leaves a directory that does not count
        as a checkpoint.  Incomplete directories older than the newest complete step are leftovers of a crashed
        writer and go as well.  Returns the steps removed."""
        import shutil

        assert keep_last >= 1
        steps = sorted(self._steps())
        doomed = steps[:-keep_last]
        newest = steps[-1] if steps else None
        for child in self.root.iterdir():
            if child.name.isdigit() and not (child / MARKER).exists() and newest is not None and int(child.name) < newest:
                doomed.append(int(child.name))
        for step in doomed:
            d = self.step_dir(step)
            marker = d / MARKER
            if marker.exists():
                marker.unlink()
            shutil.rmtree(d, ignore_errors=True)
        return sorted(doomed)

    # -- raw io ----------------------------------------------------------------------------
    def _write(self, payload, step: int, name: str) -> None:
        if self.background:
            self._ensure_worker()
            self._queue.put((_host_snapshot(payload), step, name))
        else:
            self._write_now(payload, step, name)

    def _write_now(self, payload, step: int, name: str) -> None:
        final = self.step_dir(step, create=True) / name
        tmp = final.with_name(final.name + ".tmp")
        torch.save(payload, tmp)
        os.replace(tmp, final)

    def _read(self, step: int, name: str, weights_only: bool = True):
        return torch.load(self.step_dir(step) / name, map_location="cpu", weights_only=weights_only)

    # -- components ------------------------------------------------------------------------
    def save_model(self, model, step: int, shard: int | None = None) -> None:
        self._write(model.state_dict(), step, "model.pt" if shard is None else f"model_shard{shard}.pt")

    def load_model(self, model, step: int, shard: int | None = None) -> None:
        model.load_state_dict(self._read(step, "model.pt" if shard is None else f"model_shard{shard}.pt"))

    def save_optimizer(self, optimizer, step: int, shard: int | None = None) -> None:
        self._write(optimizer.state_dict(), step, "optimizer.pt" if shard is None else f"optimizer_shard{shard}.pt")

    def load_optimizer(self, optimizer, step: int, shard: int | None = None) -> None:
        optimizer.load_state_dict(
            self._read(step, "optimizer.pt" if shard is None else f"optimizer_shard{shard}.pt"))

    def save_scheduler(self, scheduler, step: int) -> None:
        self._write(scheduler.state_dict(), step, "scheduler.pt")

    def load_scheduler(self, scheduler, step: int) -> None:
        scheduler.load_state_dict(self._read(step, "scheduler.pt"))

    def save_dataloader(self, dataloader, step: int, dp_rank: int = 0) -> None:
        """`dataloader` is anything with ``state_dict()`` (a loader or the prefetcher that wraps it)."""
        self._write(dataloader.state_dict(), step, f"dataloader_dp{dp_rank}.pt")

    def load_dataloader(self, dataloader, step: int, dp_rank: int = 0) -> None:
        dataloader.load_state_dict(self._read(step, f"dataloader_dp{dp_rank}.pt", weights_only=False))

    def save_trainer(self, state: dict, step: int) -> None:
        self._write(state, step, "trainer.pt")

    def load_trainer(self, step: int) -> dict:
        return self._read(step, "trainer.pt")
