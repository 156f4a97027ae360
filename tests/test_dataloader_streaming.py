"""The streaming text path (reference ``torchure/dataloader/builder.py:50-113``) without a network: a local JSONL
directory as the dataset, a word-level tokenizer built in the test, the stateful loader's position saved and restored,
and a Trainer run on it with an exact resume."""

import json
import os

import pytest
import torch

from tests.dist_utils import run_distributed
from tests.tiny import parity_config

pytest.importorskip("datasets")
pytest.importorskip("torchdata.stateful_dataloader")
tokenizers = pytest.importorskip("tokenizers")

WORDS = [f"w{i}" for i in range(50)]


def _corpus(root) -> str:
    d = os.path.join(root, "corpus")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "train.jsonl"), "w") as f:
        for i in range(600):
            n = 3 + (i * 7) % 23
            f.write(json.dumps({"content": " ".join(WORDS[(i + j) % 50] for j in range(n))}) + "\n")
    return d


def _tokenizer(root) -> str:
    vocab = {"<pad>": 0, "<eos>": 1, "<unk>": 2, **{w: 3 + i for i, w in enumerate(WORDS)}}
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    path = os.path.join(root, "tokenizer.json")
    tok.save(path)
    return path


def _data_cfg(root, **kw):
    cfg = dict(name=_corpus(root), tokenizer=_tokenizer(root), text_field="content", shuffle_buffer=16, seed=3,
               eos_token="<eos>", pad_token="<pad>", seq_len=32, micro_batch_size=2, num_workers=0, pack_batch=50)
    cfg.update(kw)
    return cfg


def test_streaming_loader_shards_packs_and_resumes(tmp_path):
    from torchure_b200.data import build_dataloader

    cfg = _data_cfg(str(tmp_path))
    tok = tokenizers.Tokenizer.from_file(cfg["tokenizer"])
    firsts = []
    for r in range(2):
        dl = build_dataloader(cfg, tok, -100, r, 2)
        it = iter(dl)
        batch = next(it)
        assert batch["input_ids"].shape == (2, 32) and torch.equal(batch["input_ids"], batch["labels"])
        assert (batch["input_ids"] == 1).any(), "documents are separated by the eos token"
        assert (batch["input_ids"] != 0).all(), "the stream packer fills rows completely (no padding)"
        firsts.append(batch["input_ids"])
        state = dl.state_dict()          # position after one batch
        want = next(it)
        again = build_dataloader(cfg, tok, -100, r, 2)
        again.load_state_dict(state)
        assert torch.equal(next(iter(again))["input_ids"], want["input_ids"])
    assert not torch.equal(firsts[0], firsts[1]), "the two data-parallel coordinates read different documents"


def _train_and_resume(rank, world, home, out):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    def cfg(run_name, **kw):
        c = parity_config(1, steps=5, run_name=run_name, accumulation=2, **kw)
        c["model"]["config"]["vocab_size"] = 64
        c["data"] = dict(_data_cfg(home), global_batch_size=4)
        return c

    def weights(tr):
        return {n: p.detach().clone() for n, p in tr.model.named_parameters()}

    straight = Trainer(cfg("text_straight"), rank, rank, world, device="cpu")
    assert straight.tokenizer is not None and type(straight.dataloader).__name__ == "StatefulDataLoader"
    straight.train()
    first = Trainer(cfg("text_resumed", save_steps=3), rank, rank, world, device="cpu")
    first.num_train_steps = 3
    first.train()
    second = Trainer(cfg("text_resumed", resume="auto", save_steps=1000), rank, rank, world, device="cpu")
    assert second.start_step == 3
    second.train()
    torch.save({"a": weights(straight), "b": weights(second)}, out)


def test_trainer_on_local_text_resumes_exactly(tmp_path):
    """Three steps, a checkpoint (with the stateful loader's position), two resumed steps: the same weights, bit for
    bit, as five straight steps on the same stream."""
    run_distributed(_train_and_resume, 1, str(tmp_path), str(tmp_path / "r.pt"), timeout_s=240)
    got = torch.load(tmp_path / "r.pt")
    for n in got["a"]:
        assert torch.equal(got["a"][n], got["b"][n]), n
