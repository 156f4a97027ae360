"""Host-to-device prefetch on a side stream (reference ``torchure/dataloader/prefetcher.py:18-66``).

Batch N+1 is copied from pinned host memory on a dedicated stream while batch N computes;
``__next__`` makes the compute stream wait for the copy and records the tensors on it.

Unlike the reference, the prefetcher also tracks the loader position of the batch it has
NOT yet handed out: ``state_dict()`` returns the loader state from before the look-ahead
batch was pulled, so a resumed run continues with exactly the next unseen batch instead of
skipping one.
"""

from __future__ import annotations

import copy

import torch


class CUDAPrefetcher:
    def __init__(self, loader, device: torch.device):
        self.loader = loader
        self.loader_iter = iter(loader)
        self.device = torch.device(device)
        self.on_gpu = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.on_gpu else None
        self._state_before_next = None
        self.next_batch: dict[str, torch.Tensor] | None = None
        self.h2d_bytes = 0
        self._preload()

    def _loader_state(self):
        fn = getattr(self.loader, "state_dict", None)
        return copy.deepcopy(fn()) if fn is not None else None

    def _preload(self) -> None:
        self._state_before_next = self._loader_state()
        try:
            batch = next(self.loader_iter)
        except StopIteration:
            self.next_batch = None
            return
        if not self.on_gpu:
            self.next_batch = batch
            return
        with torch.cuda.stream(self.stream):
            self.next_batch = {k: v.to(self.device, non_blocking=True) for k, v in batch.items()}
        self.h2d_bytes = sum(v.numel() * v.element_size() for v in batch.values())

    def __iter__(self):
        return self

    def __next__(self) -> dict[str, torch.Tensor]:
        if self.next_batch is None:
            raise StopIteration
        batch = self.next_batch
        if self.on_gpu:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_stream(self.stream)
            for v in batch.values():
                v.record_stream(cur)
        self._preload()
        return batch

    def state_dict(self):
        """Loader state such that the next batch produced after a restore is the one not yet consumed."""
        return self._state_before_next
