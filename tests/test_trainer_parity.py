"""End-to-end trainer on CPU/gloo.

* Parity: tiny Qwen3-style decoder (hidden 256, 4 layers, 4/2 heads, head_dim 64, ffn 768, vocab 4096),
  seq 256, micro-batch 2 per rank, 2 accumulation steps via no_sync, 5 AdamW steps with clip 1.0:
  world_size=2 DDP must match one process fed the same rows.
* Resume exactness: 3 steps + checkpoint + 2 resumed steps == 5 straight steps, bitwise.
"""

import os

import torch

from tests.dist_utils import run_distributed
from tests.tiny import parity_config

STEPS = 5


class _Interleaved:
    """Feeds a single process the rows the two DDP ranks would see, micro-batch by micro-batch."""

    def __init__(self, cfg, world):
        from torchure_b200.data import SyntheticLoader

        d = cfg["data"]
        self.loaders = [SyntheticLoader(d["seq_len"], d["micro_batch_size"], cfg["model"]["config"]["vocab_size"],
                                        d["eos_id"], d["seed"], d["mean_doc_len"], r, world, pin_memory=False)
                        for r in range(world)]
        self.k = 0

    def __iter__(self):
        return self

    def __next__(self):
        b = next(self.loaders[self.k % len(self.loaders)])
        self.k += 1
        return b


def _run(rank, world, cfg, home, out, emulate_world):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    tr = Trainer(cfg, rank, rank, world, benchmark=True, device="cpu")
    if emulate_world:
        tr.prefetcher = _Interleaved(cfg, emulate_world)
    hist = tr.train_n_step_test(STEPS)
    if rank == 0:
        torch.save({"hist": hist, "params": {n: p.detach().clone() for n, p in tr.model.named_parameters()}}, out)


def test_ddp_world2_matches_single_process(tmp_path):
    ddp_cfg = parity_config(world=2, steps=STEPS, accumulation=2)
    one_cfg = parity_config(world=1, steps=STEPS, accumulation=4)
    assert ddp_cfg["data"]["global_batch_size"] == one_cfg["data"]["global_batch_size"] == 8
    run_distributed(_run, 2, ddp_cfg, str(tmp_path), str(tmp_path / "ddp.pt"), 0, timeout_s=240)
    run_distributed(_run, 1, one_cfg, str(tmp_path), str(tmp_path / "one.pt"), 2, timeout_s=240)
    a, b = torch.load(tmp_path / "ddp.pt"), torch.load(tmp_path / "one.pt")
    for x, y in zip(a["hist"], b["hist"]):
        assert abs(x["loss"] - y["loss"]) < 1e-4 * max(1.0, abs(y["loss"]))
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, abs(y["grad_norm"]))
    assert a["hist"][0]["loss"] > 8.0  # ~ln(4096) = 8.3 at init
    for n in a["params"]:
        torch.testing.assert_close(a["params"][n], b["params"][n], rtol=1e-4, atol=1e-5, msg=lambda m: f"{n}: {m}")  # Adam amplifies summation-order noise on near-zero gradients


def _run_resume(rank, world, home, out):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    def weights(tr):
        return {n: p.detach().clone() for n, p in tr.model.named_parameters()}

    straight = Trainer(parity_config(1, steps=5, run_name="straight", accumulation=1), rank, rank, world, device="cpu")
    straight.train()
    first = Trainer(parity_config(1, steps=5, run_name="resumed", accumulation=1, save_steps=3), rank, rank, world,
                    device="cpu")
    first.num_train_steps = 3  # stop after the step-3 checkpoint, schedule still spans 5 steps
    first.train()
    second = Trainer(parity_config(1, steps=5, run_name="resumed", accumulation=1, resume="auto", save_steps=1000),
                     rank, rank, world, device="cpu")
    assert second.start_step == 3
    second.train()
    torch.save({"a": weights(straight), "b": weights(second)}, out)


def test_resume_is_exact(tmp_path):
    run_distributed(_run_resume, 1, str(tmp_path), str(tmp_path / "r.pt"), timeout_s=240)
    got = torch.load(tmp_path / "r.pt")
    for n in got["a"]:
        assert torch.equal(got["a"][n], got["b"][n]), n
    assert (tmp_path / "checkpoints" / "resumed" / "5" / ".complete").exists()
    assert sorted(os.listdir(tmp_path / "checkpoints" / "resumed")) == ["3", "5"]
