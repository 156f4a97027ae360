"""Sequence packers: turn a batch of tokenised documents into fixed ``seq_len`` rows.

Stream packers (``ListPacker``, ``NumpyPacker``, ``TensorPacker``) join documents with an
EOS after each, cut the stream into back-to-back rows and drop the tail shorter than a row;
all three emit identical rows (reference ``torchure/dataloader/packers.py:100-112,191-238``).
``ListPackerBestFit`` splits long documents into full rows plus a remainder and bin-packs
remainders and short documents best-fit-decreasing, padding open bins with ``pad_id``
(reference ``packers.py:114-188``).  Packers are top-level picklable classes so DataLoader
workers can receive them.
"""

from __future__ import annotations

import numpy as np
import torch

from torchure_b200.utils.segtree import MarkedKeys


class Packer:
    def __init__(self, tokenizer, seq_len: int, eos_id: int, pad_id: int | None = None, verbose: bool = False):
        self.tokenizer = tokenizer
        self.seq_len = seq_len
        self.eos_id = eos_id
        self.pad_id = eos_id if pad_id is None else pad_id
        self.verbose = verbose

    def __call__(self, examples: dict[str, list]) -> dict[str, list]:
        docs = [enc.ids for enc in self.tokenizer.encode_batch(examples["text"])]
        return {"input_ids": self.pack(docs)}

    def pack(self, docs: list[list[int]]) -> list[list[int]]:
        raise NotImplementedError

    def pack_to_tensor(self, docs: list[list[int]]) -> torch.Tensor:
        rows = self.pack(docs)
        if not rows:
            return torch.empty((0, self.seq_len), dtype=torch.long)
        return torch.tensor(rows, dtype=torch.long)

    def _note_dropped(self, n_tokens: int, n_rows: int) -> None:
        if self.verbose:
            print(f"{type(self).__name__}: dropped {n_tokens - n_rows * self.seq_len} tail tokens")


class ListPacker(Packer):
    def pack(self, docs):
        L = self.seq_len
        stream: list[int] = []
        for d in docs:
            stream += d
            stream.append(self.eos_id)
        n_rows = len(stream) // L
        self._note_dropped(len(stream), n_rows)
        return [stream[r * L:(r + 1) * L] for r in range(n_rows)]


class NumpyPacker(Packer):
    def _rows(self, docs) -> np.ndarray:
        L = self.seq_len
        total = sum(len(d) for d in docs) + len(docs)
        stream = np.empty(total, dtype=np.int64)
        at = 0
        for d in docs:
            n = len(d)
            stream[at:at + n] = d
            stream[at + n] = self.eos_id
            at += n + 1
        n_rows = total // L
        self._note_dropped(total, n_rows)
        return stream[: n_rows * L].reshape(n_rows, L)

    def pack(self, docs):
        return self._rows(docs).tolist()

    def pack_to_tensor(self, docs):
        return torch.from_numpy(self._rows(docs))


class TensorPacker(Packer):
    def _rows(self, docs) -> torch.Tensor:
        L = self.seq_len
        if not docs:
            return torch.empty((0, L), dtype=torch.long)
        eos = torch.tensor([self.eos_id], dtype=torch.long)
        stream = torch.cat([t for d in docs for t in (torch.tensor(d, dtype=torch.long), eos)])
        n_rows = stream.numel() // L
        self._note_dropped(stream.numel(), n_rows)
        return stream[: n_rows * L].view(n_rows, L)

    def pack(self, docs):
        return self._rows(docs).tolist()

    def pack_to_tensor(self, docs):
        return self._rows(docs)


class ListPackerBestFit(Packer):
    def pack(self, docs):
        L = self.seq_len
        rows: list[list[int]] = []
        pieces: list[list[int]] = []
        for d in docs:
            whole = len(d) // L
            rows.extend(d[i * L:(i + 1) * L] for i in range(whole))
            pieces.append(d[whole * L:] + [self.eos_id])  # 1..L tokens
        pieces.sort(key=len, reverse=True)

        open_space = MarkedKeys(L + 1)          # key s marked <=> some bin has s free slots
        bins_with: dict[int, list[int]] = {}    # free slots -> bin ids
        bins: list[list[int]] = []
        for piece in pieces:
            need = len(piece)
            have = open_space.smallest_at_least(need)
            if have is None:
                bins.append([])
                which, have = len(bins) - 1, L
            else:
                which = bins_with[have].pop()
                if not bins_with[have]:
                    open_space.set(have, False)
            bins[which] += piece
            left = have - need
            if left:
                ids = bins_with.setdefault(left, [])
                if not ids:
                    open_space.set(left, True)
                ids.append(which)
        for b in bins:
            b += [self.pad_id] * (L - len(b))
        return rows + bins


PACKERS: dict[str, type[Packer]] = {"list": ListPacker, "numpy": NumpyPacker, "tensor": TensorPacker}
BESTFIT_PACKERS: dict[str, type[Packer]] = {"bestfit": ListPackerBestFit}
