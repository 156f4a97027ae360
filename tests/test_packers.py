"""Packers on a seeded synthetic corpus (coverage of the reference's ``tests/dataloader_packing.py``):
stream packers emit identical rows (list == numpy == tensor, tensor path, empty input); best-fit rows
are all exactly seq_len and conserve the multiset of real tokens."""

import random
from collections import Counter

import torch

EOS, PAD, SEQ = 1, 2, 64


def corpus(n_docs=300, seed=0, max_len=300):
    rng = random.Random(seed)
    docs = []
    for _ in range(n_docs):
        n = int(min(max_len, max(1, rng.lognormvariate(3.5, 1.0))))
        docs.append([rng.randrange(3, 1000) for _ in range(n)])
    return docs


def test_stream_packers_agree():
    from torchure_b200.data import PACKERS

    docs = corpus()
    outs = {name: cls(None, SEQ, EOS, PAD).pack(docs) for name, cls in PACKERS.items()}
    assert outs["list"] == outs["numpy"] == outs["tensor"]
    stream = [t for d in docs for t in d + [EOS]]
    assert len(outs["list"]) == len(stream) // SEQ
    assert [t for row in outs["list"] for t in row] == stream[: len(outs["list"]) * SEQ]
    for name, cls in PACKERS.items():
        t = cls(None, SEQ, EOS, PAD).pack_to_tensor(docs)
        assert t.dtype == torch.long and t.tolist() == outs["list"], name
        assert cls(None, SEQ, EOS, PAD).pack([]) == []
        assert cls(None, SEQ, EOS, PAD).pack_to_tensor([]).shape == (0, SEQ)


def test_bestfit_conserves_tokens():
    from torchure_b200.data import ListPackerBestFit

    docs = corpus(seed=1)
    rows = ListPackerBestFit(None, SEQ, EOS, PAD).pack(docs)
    assert all(len(r) == SEQ for r in rows)
    real_in = Counter(t for d in docs for t in d)
    real_out = Counter(t for r in rows for t in r if t not in (EOS, PAD))
    assert real_in == real_out
    assert sum(1 for r in rows for t in r if t == EOS) == len(docs)
    # best fit wastes less than one-document-per-row
    pad = sum(1 for r in rows for t in r if t == PAD)
    assert pad < 0.2 * len(rows) * SEQ


def test_marked_keys():
    from torchure_b200.utils import MarkedKeys

    mk = MarkedKeys(65)
    assert mk.smallest_at_least(1) is None
    for k in (5, 17, 40):
        mk.set(k, True)
    assert mk.smallest_at_least(1) == 5 and mk.smallest_at_least(6) == 17 and mk.smallest_at_least(18) == 40
    assert mk.smallest_at_least(41) is None
    mk.set(17, False)
    assert mk.smallest_at_least(6) == 40


def test_synthetic_loader_deterministic_and_sharded():
    from torchure_b200.data import SyntheticLoader

    a = SyntheticLoader(256, 2, 4096, eos_id=0, seed=1, mean_doc_len=32, dp_rank=0, dp_size=2, pin_memory=False)
    b = SyntheticLoader(256, 2, 4096, eos_id=0, seed=1, mean_doc_len=32, dp_rank=0, dp_size=2, pin_memory=False)
    c = SyntheticLoader(256, 2, 4096, eos_id=0, seed=1, mean_doc_len=32, dp_rank=1, dp_size=2, pin_memory=False)
    x, y, z = next(a), next(b), next(c)
    assert torch.equal(x["input_ids"], y["input_ids"]) and not torch.equal(x["input_ids"], z["input_ids"])
    assert x["input_ids"].shape == (2, 256) and x["input_ids"].dtype == torch.long
    assert torch.equal(x["labels"], x["input_ids"]) and x["labels"].data_ptr() != x["input_ids"].data_ptr()
    n_eos = (torch.cat([next(a)["input_ids"] for _ in range(20)]) == 0).float().mean().item()
    assert 1 / 64 < n_eos < 1 / 16  # about one EOS per 32 tokens
