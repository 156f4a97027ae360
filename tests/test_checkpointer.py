"""Checkpoint layout, round trips and `.complete` semantics (coverage of the reference's
``tests/checkpointer.py``: component round trips, overwrite of a step, RNG replay, torn newest
step falls back, explicit torn step refused, non-numeric directories ignored)."""

import os

import torch

from tests.tiny import TINY


def _parts():
    from torchure_b200.models import Qwen3
    from torchure_b200.optim import build_optimizer, build_scheduler

    torch.manual_seed(0)
    m = Qwen3(**TINY)
    m.init_weights()
    opt = build_optimizer(m, "adamw", {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95]})
    sch = build_scheduler(opt, {"type": "wsd", "warmup_ratio": 0.1, "decay_ratio": 0.2, "total_steps": 10})
    return m, opt, sch


def _train(m, opt, sch, n):
    ids = torch.randint(0, TINY["vocab_size"], (2, 16), generator=torch.Generator().manual_seed(1))
    for _ in range(n):
        opt.zero_grad()
        m(ids).float().pow(2).mean().backward()
        opt.step()
        sch.step()


def test_roundtrip_and_layout(tmp_path):
    from torchure_b200.ckpt import Checkpointer
    from torchure_b200.data import SyntheticLoader

    ck = Checkpointer(str(tmp_path / "run"))
    m, opt, sch = _parts()
    _train(m, opt, sch, 3)
    dl = SyntheticLoader(16, 2, 64, seed=3, pin_memory=False)
    next(dl), next(dl)
    for _ in range(2):  # saving the same step twice overwrites
        ck.save_model(m, 3)
        ck.save_optimizer(opt, 3)
        ck.save_scheduler(sch, 3)
        ck.save_dataloader(dl, 3, 0)
        ck.save_trainer({"step": 3, "cpu_rng": torch.get_rng_state(), "cuda_rng": None, "config": {"mesh": {"dp": 1}},
                         "wandb_id": None}, 3)
    ck.mark_complete(3)
    assert sorted(os.listdir(tmp_path / "run" / "3")) == sorted(
        [".complete", "model.pt", "optimizer.pt", "scheduler.pt", "trainer.pt", "dataloader_dp0.pt"])
    sd = torch.load(tmp_path / "run" / "3" / "model.pt")
    assert "lm_head.weight" in sd and "token_emb.weight" in sd and "rope.inv_freq" not in sd
    assert "blocks.1.gqa.q_norm.weight" in sd and "blocks.0.ffn.down_proj.weight" in sd
    expected_next = next(dl)["input_ids"]

    m2, opt2, sch2 = _parts()
    dl2 = SyntheticLoader(16, 2, 64, seed=3, pin_memory=False)
    ck.load_model(m2, 3)
    ck.load_optimizer(opt2, 3)
    ck.load_scheduler(sch2, 3)
    ck.load_dataloader(dl2, 3, 0)
    assert torch.equal(next(dl2)["input_ids"], expected_next)
    for p, q in zip(m.parameters(), m2.parameters()):
        assert torch.equal(p, q)
    assert sch2.last_epoch == sch.last_epoch
    # continuing both gives the same weights => optimizer state restored exactly
    _train(m, opt, sch, 2)
    _train(m2, opt2, sch2, 2)
    for p, q in zip(m.parameters(), m2.parameters()):
        torch.testing.assert_close(p, q, rtol=0, atol=0)
    st = ck.load_trainer(3)
    torch.set_rng_state(st["cpu_rng"])
    a = torch.rand(3)
    torch.set_rng_state(st["cpu_rng"])
    assert torch.equal(a, torch.rand(3))


def test_complete_marker_semantics(tmp_path):
    from torchure_b200.ckpt import Checkpointer

    ck = Checkpointer(str(tmp_path / "run"))
    assert ck.latest() is None
    m, _, _ = _parts()
    ck.save_model(m, 5)
    ck.mark_complete(5)
    ck.save_model(m, 10)  # torn: no marker
    os.makedirs(tmp_path / "run" / "notes")
    os.makedirs(tmp_path / "run" / "7x")
    assert ck.latest() == 5
    assert ck.valid_step(10) is None and ck.valid_step(5) == 5
    assert not ck.is_complete(10)
    ck.mark_complete(10)
    assert ck.latest() == 10
    assert not list((tmp_path / "run" / "10").glob("*.tmp"))


def test_prefetcher_position_is_exact(tmp_path):
    """The look-ahead batch must not be skipped by a save/restore through the prefetcher."""
    from torchure_b200.data import CUDAPrefetcher, SyntheticLoader

    dl = SyntheticLoader(16, 2, 64, seed=5, pin_memory=False)
    pf = CUDAPrefetcher(dl, torch.device("cpu"))
    next(pf), next(pf)
    state = pf.state_dict()
    want = next(pf)["input_ids"]
    dl2 = SyntheticLoader(16, 2, 64, seed=5, pin_memory=False)
    dl2.load_state_dict(state)
    pf2 = CUDAPrefetcher(dl2, torch.device("cpu"))
    assert torch.equal(next(pf2)["input_ids"], want)


def test_prune_keeps_the_newest_complete_steps(tmp_path):
    from torchure_b200.ckpt import Checkpointer

    ck = Checkpointer(str(tmp_path))
    for step in (2, 4, 6, 8):
        ck.save_trainer({"step": step}, step)
        ck.mark_complete(step)
    ck.save_trainer({"step": 5}, 5)          # a writer died here before the marker
    ck.save_trainer({"step": 10}, 10)        # ... and one is being written right now
    assert ck.prune(2) == [2, 4, 5]
    assert sorted(p.name for p in tmp_path.iterdir()) == ["10", "6", "8"]
    assert ck.latest() == 8 and ck.valid_step(6) == 6 and ck.valid_step(4) is None
    assert ck.prune(2) == []
