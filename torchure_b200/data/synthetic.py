"""Synthetic packed-token source for benchmarks and tests (no network, no tokenizer).

Every row is a slice of an endless stream of documents whose lengths are geometric with
the configured mean, tokens uniform over the vocabulary, each document closed by the EOS
id.  Row ``r`` of dp coordinate ``c`` is a pure function of ``(seed, c, r)`` (counter-based
Philox), so the loader is deterministic, shards never overlap, and resuming is restoring
one integer.  Batches have the collator's format: ``{"input_ids": int64 (B, S),
"labels": clone}`` (reference ``torchure/dataloader/builder.py:44-47``).
"""

from __future__ import annotations

import numpy as np
import torch


def synthetic_row(seed: int, dp_rank: int, row: int, seq_len: int, vocab_size: int, eos_id: int,
                  mean_doc_len: float) -> np.ndarray:
    # the row index and the shard go into the KEY: counters of one key are consecutive blocks of the same stream,
    # so keying by seed alone and offsetting the counter would make neighbouring rows shifted copies of each other
    rng = np.random.Generator(np.random.Philox(key=[seed & 0xFFFFFFFFFFFFFFFF, (dp_rank << 44) | row]))
    toks = rng.integers(0, vocab_size, size=seq_len, dtype=np.int64)
    # document ends: gaps are geometric(1/mean); the row starts inside a document
    p = 1.0 / max(1.0, mean_doc_len)
    n_draw = max(8, int(4 * seq_len * p) + 8)
    ends = np.cumsum(rng.geometric(p, size=n_draw)) - 1
    while ends[-1] < seq_len:
        more = np.cumsum(rng.geometric(p, size=n_draw)) + ends[-1]
        ends = np.concatenate([ends, more])
    toks[ends[ends < seq_len]] = eos_id
    return toks


class SyntheticLoader:
    """Stateful iterable of synthetic batches; ``state_dict`` is the number of batches handed out."""

    def __init__(self, seq_len: int, micro_batch_size: int, vocab_size: int, eos_id: int = 0, seed: int = 0,
                 mean_doc_len: float = 1024.0, dp_rank: int = 0, dp_size: int = 1, pin_memory: bool = True):
        self.seq_len, self.mbs = seq_len, micro_batch_size
        self.vocab_size, self.eos_id, self.seed = vocab_size, eos_id, seed
        self.mean_doc_len = mean_doc_len
        self.dp_rank, self.dp_size = dp_rank, dp_size
        self.pin = pin_memory and torch.cuda.is_available()
        self.batches_served = 0

    def __iter__(self):
        return self

    def __next__(self) -> dict[str, torch.Tensor]:
        first = self.batches_served * self.mbs
        rows = [synthetic_row(self.seed, self.dp_rank, first + i, self.seq_len, self.vocab_size, self.eos_id,
                              self.mean_doc_len) for i in range(self.mbs)]
        ids = torch.from_numpy(np.stack(rows))
        if self.pin:
            ids = ids.pin_memory()
        self.batches_served += 1
        labels = ids.clone()
        if self.pin:
            labels = labels.pin_memory()
        return {"input_ids": ids, "labels": labels}

    def state_dict(self) -> dict:
        return {"batches_served": self.batches_served, "seed": self.seed, "dp_rank": self.dp_rank,
                "dp_size": self.dp_size}

    def load_state_dict(self, state: dict) -> None:
        assert state["dp_size"] == self.dp_size and state["dp_rank"] == self.dp_rank, "dataloader shard mismatch"
        self.batches_served = int(state["batches_served"])
