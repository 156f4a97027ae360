"""Optional parts of the Trainer.  Metrics sinks (reference ``torchure/train/trainer.py:404-441``): the wandb run (a
stand-in object here: init arguments, one log call per step, finish, run id kept in the checkpoint and passed back on
resume) and the JSONL sink.  Per-block ``torch.compile`` of the PyTorch path (reference ``trainer.py:223-244``)."""

import json
import os

import torch

from tests.dist_utils import run_distributed
from tests.tiny import parity_config


class _FakeRun:
    def __init__(self, calls, run_id):
        self.calls, self.id = calls, run_id

    def log(self, payload, step=None):
        self.calls.append(("log", step, sorted(payload)))

    def finish(self):
        self.calls.append(("finish",))


class _FakeWandb:
    def __init__(self):
        self.calls = []

    def init(self, **kw):
        self.calls.append(("init", {k: kw[k] for k in ("project", "entity", "id", "resume")}, "config" in kw))
        return _FakeRun(self.calls, kw.get("id") or "run-abc")


def _run(rank, world, home, out):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train import trainer as T

    fake = _FakeWandb()
    T.wandb, T.HAS_WANDB = fake, True

    def cfg(**kw):
        c = parity_config(1, steps=4, run_name="logged", accumulation=1, **kw)
        c["wandb"] = {"enabled": True, "project": "proj", "entity": "me"}
        c["logging"] = {"jsonl": os.path.join(home, "metrics", "log.jsonl")}
        return c

    first = T.Trainer(cfg(save_steps=2), rank, rank, world, device="cpu")
    first.num_train_steps = 2
    first.train()
    second = T.Trainer(cfg(resume="auto", save_steps=1000), rank, rank, world, device="cpu")
    second.train()
    torch.save(fake.calls, out)


def test_wandb_run_and_jsonl_sink(tmp_path):
    run_distributed(_run, 1, str(tmp_path), str(tmp_path / "calls.pt"), timeout_s=240)
    calls = torch.load(tmp_path / "calls.pt", weights_only=False)
    inits = [c for c in calls if c[0] == "init"]
    assert inits[0][1] == {"project": "proj", "entity": "me", "id": None, "resume": None} and inits[0][2]
    # the resumed run continues the SAME wandb run: the id travelled through trainer.pt
    assert inits[1][1] == {"project": "proj", "entity": "me", "id": "run-abc", "resume": "must"}
    logs = [c for c in calls if c[0] == "log"]
    assert [c[1] for c in logs] == [1, 2, 3, 4]
    assert {"train/loss", "train/grad_norm", "train/lr", "train/tokens", "perf/tps", "perf/step_time"} <= set(logs[0][2])
    assert sum(1 for c in calls if c[0] == "finish") == 2
    with open(tmp_path / "metrics" / "log.jsonl") as f:
        recs = [json.loads(line) for line in f]
    assert [r["step"] for r in recs] == [1, 2, 3, 4]
    assert all(r["loss"] > 0 and r["tps"] > 0 and r["lr"] >= 0 for r in recs)
    assert recs[-1]["tokens"] == 4 * 256 * 2       # steps x seq_len x global batch


def _per_block_compile(rank, world, home, out):
    os.environ["TORCHURE_B200_HOME"] = home
    import torch._dynamo

    from torchure_b200.train.trainer import Trainer

    def cfg(name, **kw):
        c = parity_config(1, steps=3, run_name=name, accumulation=1)
        c["compile"] = False            # the PyTorch path
        c.update(kw)
        return c

    compiled = Trainer(cfg("pbc", torch_compile=True, compile_backend="aot_eager"), rank, rank, world, benchmark=True,
                       device="cpu")
    # one compiled region per transformer block plus the final norm, as the reference compiles (not the whole model)
    assert all(b._compiled_call_impl is not None for b in compiled.model.blocks)
    assert compiled.model.norm._compiled_call_impl is not None and compiled.model._compiled_call_impl is None
    a = compiled.train_n_step_test(3)
    b = Trainer(cfg("pbe"), rank, rank, world, benchmark=True, device="cpu").train_n_step_test(3)
    torch.save({"compiled": a, "eager": b}, out)


def test_per_block_compile_of_the_pytorch_path(tmp_path):
    """`torch_compile: true` (with `compile: false`): every block and the final norm become compiled regions; the run
    follows the eager one.  `compile_backend: "aot_eager"` keeps the test independent of a host C++ toolchain."""
    run_distributed(_per_block_compile, 1, str(tmp_path), str(tmp_path / "c.pt"), timeout_s=240)
    got = torch.load(tmp_path / "c.pt")
    for x, y in zip(got["compiled"], got["eager"]):
        assert abs(x["loss"] - y["loss"]) < 1e-5 * max(1.0, abs(y["loss"])), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-4 * max(1.0, abs(y["grad_norm"])), (x, y)


def test_command_line_entrypoint_under_torchrun(tmp_path):
    """`python -m torch.distributed.run ... -m torchure_b200.train.train --config C --steps N` (the reference's
    interface, ``torchure/train/train.py:45-87``): two CPU ranks over gloo, benchmark mode, rank 0 prints one line per
    step, both ranks exit 0 after destroying the process group."""
    import subprocess
    import sys

    from tests.dist_utils import free_port

    cfg = parity_config(2, steps=3, run_name="cli", accumulation=1)
    path = tmp_path / "cli.json"
    path.write_text(json.dumps(cfg))
    env = dict(os.environ, TORCHURE_B200_HOME=str(tmp_path), OMP_NUM_THREADS="2")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", str(free_port()), "-m", "torchure_b200.train.train", "--config", str(path),
         "--steps", "3"],
        capture_output=True, text=True, timeout=240, env=env, cwd=os.path.dirname(os.path.dirname(__file__)))
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("step=")]
    assert len(lines) == 3 and "loss=" in lines[0] and "tps=" in lines[0], out.stdout[-1000:]


def _with_eval(rank, world, home, out):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    def cfg(name, mesh, **kw):
        c = parity_config(world, steps=4, run_name=name, accumulation=1, mesh=mesh)
        c["logging"] = {"jsonl": os.path.join(home, f"{name}.jsonl")}
        c.update(kw)
        return c

    def weights(tr):
        if getattr(tr, "sharded", False):
            return {n: v.detach().clone() for n, v in tr.ddp.full_state_dict().items()}
        return {n: p.detach().clone() for n, p in tr.model.named_parameters()}

    result = {}
    for name, mesh in (("ddp", {"dp": world}), ("fsdp", {"dp_shard": world})):
        plain = Trainer(cfg(f"{name}_plain", mesh), rank, rank, world, device="cpu")
        plain.train()
        evald = Trainer(cfg(f"{name}_eval", mesh, eval={"every": 2, "batches": 3}), rank, rank, world, device="cpu")
        first = evald.evaluate().item()
        assert evald.evaluate().item() == first           # the held-out stream restarts at every call
        evald.train()
        last = evald.evaluate().item()
        a, b = weights(plain), weights(evald)
        assert all(torch.equal(a[n], b[n]) for n in a), f"{name}: evaluating changed the training trajectory"
        result[name] = (first, last)
    if rank == 0:
        torch.save(result, out)


def test_held_out_evaluation(tmp_path):
    """`eval: {every, batches}`: the loss on a held-out synthetic stream is logged at the cadence, is the same on
    repeated calls, and leaves training untouched (bitwise the weights of a run without it), for DDP and FSDP."""
    run_distributed(_with_eval, 2, str(tmp_path), str(tmp_path / "e.pt"), timeout_s=300)
    got = torch.load(tmp_path / "e.pt")
    assert abs(got["ddp"][0] - got["fsdp"][0]) < 1e-4 and got["ddp"][0] > 8.0      # ~ln(4096) at initialisation
    with open(tmp_path / "ddp_eval.jsonl") as f:
        recs = [json.loads(line) for line in f]
    assert [("eval_loss" in r) for r in recs] == [False, True, False, True]
    assert all(r["eval_loss"] > 0 for r in recs if "eval_loss" in r)


def _keep_last(rank, world, home):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    cfg = parity_config(1, steps=5, run_name="pruned", accumulation=1, save_steps=1)
    cfg["checkpointing"]["keep_last"] = 2
    Trainer(cfg, rank, rank, world, device="cpu").train()


def test_keep_last_bounds_the_checkpoints_on_disk(tmp_path):
    run_distributed(_keep_last, 1, str(tmp_path), timeout_s=240)
    assert sorted(os.listdir(tmp_path / "checkpoints" / "pruned")) == ["4", "5"]
    assert (tmp_path / "checkpoints" / "pruned" / "5" / ".complete").exists()


def _preempted(rank, world, home, out):
    import signal

    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    def cfg(name, **kw):
        c = parity_config(2, steps=5, run_name=name, accumulation=1, **kw)
        c["checkpointing"]["on_signal"] = True
        return c

    def weights(tr):
        return {n: p.detach().clone() for n, p in tr.model.named_parameters()}

    straight = Trainer(cfg("pre_straight"), rank, rank, world, device="cpu")
    straight.train()
    first = Trainer(cfg("pre_resumed"), rank, rank, world, device="cpu")
    calls = []

    def in_second_step(mod, args):      # ONE rank is told to stop, in the middle of its second step
        calls.append(1)
        if rank == 1 and len(calls) == 2:
            os.kill(os.getpid(), signal.SIGTERM)

    first.model.register_forward_pre_hook(in_second_step)
    first.train()
    assert len(calls) == 2, "both ranks must leave after the step in which the signal arrived"
    second = Trainer(cfg("pre_resumed", resume="auto"), rank, rank, world, device="cpu")
    assert second.start_step == 2
    second.train()
    if rank == 0:
        torch.save({"a": weights(straight), "b": weights(second)}, out)


def test_signal_checkpoints_and_leaves_at_a_step_boundary(tmp_path):
    """`checkpointing.on_signal`: SIGTERM on one rank during a step; every rank finishes the step, all write a
    checkpoint of it and leave; the resumed run ends, bit for bit, where an undisturbed run does."""
    run_distributed(_preempted, 2, str(tmp_path), str(tmp_path / "p.pt"), timeout_s=240)
    got = torch.load(tmp_path / "p.pt")
    for n in got["a"]:
        assert torch.equal(got["a"][n], got["b"][n]), n
    assert sorted(os.listdir(tmp_path / "checkpoints" / "pre_resumed")) == ["2", "5"]


def _async_ckpt(rank, world, home, out):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    def cfg(name, **kw):
        c = parity_config(2, steps=5, run_name=name, accumulation=1, **kw)
        c["checkpointing"]["async"] = True
        return c

    def weights(tr):
        return {n: p.detach().clone() for n, p in tr.model.named_parameters()}

    # the files hold the state at the moment of checkpoint(), whatever training does while they are written, and the
    # step exists only after finish_checkpoint()
    probe = Trainer(cfg("async_probe"), rank, rank, world, device="cpu")
    probe.train_step()
    probe.train_step()
    at_two = weights(probe)
    probe.checkpoint(2)
    assert not probe.checkpointer.is_complete(2)
    probe.train_step()
    probe.finish_checkpoint()
    torch.distributed.barrier()          # rank 0 writes the marker after every rank's files are on disk
    assert probe.checkpointer.is_complete(2)
    saved = probe.checkpointer._read(2, "model.pt")
    assert all(torch.equal(saved[n], at_two[n]) for n in at_two)
    assert not torch.equal(saved["norm.weight"], weights(probe)["norm.weight"])
    # and a run interrupted after step 3 resumes exactly
    straight = Trainer(cfg("async_straight"), rank, rank, world, device="cpu")
    straight.train()
    first = Trainer(cfg("async_resumed", save_steps=3), rank, rank, world, device="cpu")
    first.num_train_steps = 3
    first.train()
    second = Trainer(cfg("async_resumed", resume="auto", save_steps=1000), rank, rank, world, device="cpu")
    assert second.start_step == 3
    second.train()
    if rank == 0:
        torch.save({"a": weights(straight), "b": weights(second)}, out)


def test_asynchronous_checkpoints(tmp_path):
    run_distributed(_async_ckpt, 2, str(tmp_path), str(tmp_path / "a.pt"), timeout_s=240)
    got = torch.load(tmp_path / "a.pt")
    for n in got["a"]:
        assert torch.equal(got["a"][n], got["b"][n]), n
    assert sorted(os.listdir(tmp_path / "checkpoints" / "async_resumed")) == ["3", "5"]
