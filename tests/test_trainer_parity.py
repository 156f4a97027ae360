"""End-to-end trainer on CPU/gloo.

* Parity: tiny Qwen3-style decoder (hidden 256, 4 layers, 4/2 heads, head_dim 64, ffn 768, vocab 4096),
  seq 256, micro-batch 2 per rank, 2 accumulation steps via no_sync, 5 AdamW steps with clip 1.0:
  world_size=2 DDP must match one process fed the same rows.
* The same comparison for FSDP2 (mesh ``dp_shard: 2``) and HSDP (``dp_replicate: 2, dp_shard: 2``), selected by
  the mesh of the config alone.
* Resume exactness: 3 steps + checkpoint + 2 resumed steps == 5 straight steps, bitwise; for FSDP the checkpoint
  holds an unsharded ``model.pt`` and one ``optimizer_shard{r}.pt`` per shard.
"""

import os

import pytest
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
    params = _weights(tr)
    if rank == 0:
        torch.save({"hist": hist, "params": params}, out)


_REFERENCE: dict = {}


def _single_process(tmp_path, accumulation: int, emulate_world: int | None = None) -> dict:
    """What ONE process does with the same global batch (computed once per test session and kind): with
    `emulate_world` the run is fed the rows that many data-parallel ranks would read and returns the loss / norm
    history and the final weights; without it, the history only."""
    key = (accumulation, emulate_world)
    if key not in _REFERENCE:
        cfg = parity_config(world=1, steps=STEPS, accumulation=accumulation)
        out = str(tmp_path / f"single_{accumulation}_{emulate_world}.pt")
        if emulate_world is None:
            run_distributed(_run_hist_only, 1, cfg, str(tmp_path), out, timeout_s=240)
        else:
            run_distributed(_run, 1, cfg, str(tmp_path), out, emulate_world, timeout_s=240)
        _REFERENCE[key] = torch.load(out)
    return _REFERENCE[key]



def _weights(tr):
    """Unsharded fp32 weights under the model's keys (a collective when the strategy shards them)."""
    if getattr(tr, "sharded", False):
        sd = tr.ddp.full_state_dict()
        return {n: sd[n].detach().clone() for n, _ in tr.model.named_parameters()}
    return {n: p.detach().clone() for n, p in tr.model.named_parameters()}


def _compare(a, b):
    for x, y in zip(a["hist"], b["hist"]):
        assert abs(x["loss"] - y["loss"]) < 1e-4 * max(1.0, abs(y["loss"]))
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, abs(y["grad_norm"]))
    assert a["hist"][0]["loss"] > 8.0  # ~ln(4096) = 8.3 at init
    for n in b["params"]:
        x, y = a["params"][n], b["params"][n]
        diff = (x - y).abs()
        off = (diff > 1e-5 + 1e-4 * y.abs()).float().mean().item()
        # Adam moves a weight by up to lr per step whatever the size of its gradient, so a gradient that is zero up
        # to summation order may step the other way: a handful of elements differ by a few lr, nothing else may
        assert off < 1e-5, f"{n}: {off:.2e} of the elements differ"
        assert diff.max().item() < 5 * 3e-4, f"{n}: max difference {diff.max().item():.2e}"


def test_fsdp_and_hsdp_match_single_process(tmp_path):
    """The mesh alone selects the strategy: dp_shard -> FSDP2 units, dp_replicate x dp_shard -> HSDP."""
    fsdp_cfg = parity_config(world=2, steps=STEPS, accumulation=2, mesh={"dp_shard": 2})
    run_distributed(_run, 2, fsdp_cfg, str(tmp_path), str(tmp_path / "fsdp.pt"), 0, timeout_s=240)
    _compare(torch.load(tmp_path / "fsdp.pt"), _single_process(tmp_path, 4, 2))
    hsdp_cfg = parity_config(world=4, steps=STEPS, accumulation=1, mesh={"dp_replicate": 2, "dp_shard": 2})
    run_distributed(_run, 4, hsdp_cfg, str(tmp_path), str(tmp_path / "hsdp.pt"), 0, timeout_s=240)
    _compare(torch.load(tmp_path / "hsdp.pt"), _single_process(tmp_path, 4, 4))


def _run_hist_only(rank, world, cfg, home, out):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    tr = Trainer(cfg, rank, rank, world, benchmark=True, device="cpu")
    assert (getattr(tr.model, "vocab_parallel", None) is not None) == bool(cfg.get("tp", {}).get("loss_parallel"))
    seen = []
    tr.model.register_forward_pre_hook(lambda mod, args: seen.append(tuple(args[0].shape)))
    hist = tr.train_n_step_test(STEPS)
    if rank == 0:
        torch.save({"hist": hist, "input_shapes": sorted(set(seen))}, out)


def test_tensor_parallel_trainer_matches_single_process(tmp_path):
    """mesh {dp: 1, tp: 2}: both ranks see the same batches and hold half of every block; loss and the global
    gradient norm (sharded tensors summed over tp, replicated ones counted once) must follow the single-process run,
    which also pins the clip coefficient and therefore every later step."""
    tp_cfg = parity_config(world=1, steps=STEPS, accumulation=2, mesh={"dp": 1, "tp": 2})
    run_distributed(_run_hist_only, 2, tp_cfg, str(tmp_path), str(tmp_path / "tp.pt"), timeout_s=240)
    a, b = torch.load(tmp_path / "tp.pt"), _single_process(tmp_path, 2)
    for x, y in zip(a["hist"], b["hist"]):
        assert abs(x["loss"] - y["loss"]) < 1e-4 * max(1.0, abs(y["loss"])), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, abs(y["grad_norm"])), (x, y)


def test_loss_parallel_trainer_matches_single_process(tmp_path):
    """mesh {dp: 1, tp: 2} with `tp.loss_parallel`: each rank computes half of the vocabulary's logits inside the
    chunked CE, the row slices of the tied embedding / head gradient are gathered before the clip norm."""
    lp_cfg = parity_config(world=1, steps=STEPS, accumulation=2, mesh={"dp": 1, "tp": 2})
    lp_cfg["tp"] = {"loss_parallel": True}
    run_distributed(_run_hist_only, 2, lp_cfg, str(tmp_path), str(tmp_path / "lp.pt"), timeout_s=240)
    a, b = torch.load(tmp_path / "lp.pt"), _single_process(tmp_path, 2)
    for x, y in zip(a["hist"], b["hist"]):
        assert abs(x["loss"] - y["loss"]) < 1e-4 * max(1.0, abs(y["loss"])), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, abs(y["grad_norm"])), (x, y)


def test_sequence_parallel_trainer_matches_single_process(tmp_path):
    """mesh {dp: 1, tp: 2} with `tp.sequence_parallel`: the activations between the column / row linears are sharded
    along the sequence, the embedding output is sliced on entry and the hidden state gathered before the final norm;
    the norm gains inside the blocks see half of the tokens each and their gradients are summed over the axis.  Loss
    and global gradient norm must follow the single-process run."""
    sp_cfg = parity_config(world=1, steps=STEPS, accumulation=2, mesh={"dp": 1, "tp": 2})
    sp_cfg["tp"] = {"sequence_parallel": True}
    run_distributed(_run_hist_only, 2, sp_cfg, str(tmp_path), str(tmp_path / "sp.pt"), timeout_s=240)
    a, b = torch.load(tmp_path / "sp.pt"), _single_process(tmp_path, 2)
    for x, y in zip(a["hist"], b["hist"]):
        assert abs(x["loss"] - y["loss"]) < 1e-4 * max(1.0, abs(y["loss"])), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, abs(y["grad_norm"])), (x, y)


def test_context_parallel_trainer_matches_single_process(tmp_path):
    """mesh {dp: 1, cp: 2}: both ranks read the same rows, keep two zigzag chunks of every sequence, rotate by the
    chunks' global positions and run attention as a ring; each divides its summed loss by half of the global target
    count and the gradients are averaged over dp x cp.  Loss and gradient norm must follow the single-process run."""
    cp_cfg = parity_config(world=1, steps=STEPS, accumulation=2, mesh={"dp": 1, "cp": 2})
    run_distributed(_run_hist_only, 2, cp_cfg, str(tmp_path), str(tmp_path / "cp.pt"), timeout_s=240)
    a, b = torch.load(tmp_path / "cp.pt"), _single_process(tmp_path, 2)
    d = cp_cfg["data"]
    assert a["input_shapes"] == [(d["micro_batch_size"], d["seq_len"] // 2)], a["input_shapes"]   # half of every row
    for x, y in zip(a["hist"], b["hist"]):
        assert abs(x["loss"] - y["loss"]) < 1e-4 * max(1.0, abs(y["loss"])), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, abs(y["grad_norm"])), (x, y)


@pytest.mark.parametrize("mesh,extra", [({"dp": 2, "cp": 2}, {}),
                                        ({"dp": 2, "tp": 2}, {"tp": {"loss_parallel": True}})])
def test_model_parallel_axes_with_data_parallel_replicas(tmp_path, mesh, extra):
    """Four ranks: two data-parallel replicas of a context-parallel (or tensor-parallel, loss-parallel) pair, against
    one process fed both replicas' rows.  Pins the flattened gradient axis, the per-replica loss divisor and the
    gather of the head-gradient rows when the axes combine."""
    cfg = parity_config(world=2, steps=STEPS, accumulation=2, mesh=mesh)
    cfg.update(extra)
    run_distributed(_run_hist_only, 4, cfg, str(tmp_path), str(tmp_path / "four.pt"), timeout_s=300)
    a, b = torch.load(tmp_path / "four.pt"), _single_process(tmp_path, 4, 2)
    for x, y in zip(a["hist"], b["hist"]):
        assert abs(x["loss"] - y["loss"]) < 1e-4 * max(1.0, abs(y["loss"])), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, abs(y["grad_norm"])), (x, y)


def test_ulysses_trainer_matches_single_process(tmp_path):
    """mesh {dp: 1, cp: 2} with `cp.kind: "ulysses"`: contiguous halves of every sequence, all heads of the half
    exchanged for half of the heads of the whole sequence around attention."""
    u_cfg = parity_config(world=1, steps=STEPS, accumulation=2, mesh={"dp": 1, "cp": 2})
    u_cfg["cp"] = {"kind": "ulysses"}
    run_distributed(_run_hist_only, 2, u_cfg, str(tmp_path), str(tmp_path / "u.pt"), timeout_s=240)
    a, b = torch.load(tmp_path / "u.pt"), _single_process(tmp_path, 2)
    d = u_cfg["data"]
    assert a["input_shapes"] == [(d["micro_batch_size"], d["seq_len"] // 2)], a["input_shapes"]
    for x, y in zip(a["hist"], b["hist"]):
        assert abs(x["loss"] - y["loss"]) < 1e-4 * max(1.0, abs(y["loss"])), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, abs(y["grad_norm"])), (x, y)


def _moe_config(world, accumulation, mesh=None, **kw):
    cfg = parity_config(world=world, steps=STEPS, accumulation=accumulation, mesh=mesh, **kw)
    cfg["model"] = {"name": "qwen3_moe", "config": dict(cfg["model"]["config"], num_experts=4, top_k=2,
                                                        moe_ffn_dim=256, capacity_factor=8.0)}
    return cfg


def _run_moe(rank, world, cfg, home, out, emulate_world):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    tr = Trainer(cfg, rank, rank, world, benchmark=True, device="cpu")
    if emulate_world:
        tr.prefetcher = _Interleaved(cfg, emulate_world)
    hist = tr.train_n_step_test(STEPS)
    torch.save({"hist": hist, "params": _weights(tr)}, f"{out}.{rank}")


def test_expert_parallel_trainer_matches_single_process(tmp_path):
    """mesh {dp: 1, ep: 2} on the mixture-of-experts model: each rank keeps two of the four experts of every layer
    and reads its own rows; tokens travel to their experts and back.  One process that holds all experts and is fed
    both ranks' rows must see the same loss and gradient norm and end with the same weights (shared tensors on every
    rank, each rank's experts equal to the matching slice)."""
    run_distributed(_run_moe, 1, _moe_config(1, 2), str(tmp_path), str(tmp_path / "one.pt"), 2, timeout_s=240)
    run_distributed(_run_moe, 2, _moe_config(2, 1, mesh={"dp": 1, "ep": 2}), str(tmp_path), str(tmp_path / "ep.pt"), 0,
                    timeout_s=240)
    one = torch.load(f"{tmp_path}/one.pt.0")
    parts = [torch.load(f"{tmp_path}/ep.pt.{r}") for r in range(2)]
    for x, y in zip(parts[0]["hist"], one["hist"]):
        assert abs(x["loss"] - y["loss"]) < 1e-4 * max(1.0, abs(y["loss"])), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, abs(y["grad_norm"])), (x, y)
    for r, part in enumerate(parts):
        for n, v in part["params"].items():
            want = one["params"][n]
            if v.shape != want.shape:               # stacked expert weights: this rank's half
                assert n.split(".")[-1] in ("w_gate", "w_up", "w_down"), n
                want = want[r * v.shape[0]:(r + 1) * v.shape[0]]
            assert (v - want).abs().max().item() < 5 * 3e-4, (n, (v - want).abs().max().item())
            assert ((v - want).abs() > 1e-5 + 1e-4 * want.abs()).float().mean().item() < 1e-4, n


def test_expert_parallel_with_data_parallel_replicas(tmp_path):
    """mesh {dp: 2, ep: 2} on four ranks: the experts' gradients are averaged over the two replicas that hold the same
    experts (and divided by the ep size), the shared parameters over all four ranks.  One process with all experts,
    fed the four ranks' rows, must give the same losses and norms; replicas must stay identical."""
    run_distributed(_run_moe, 1, _moe_config(1, 4), str(tmp_path), str(tmp_path / "one.pt"), 4, timeout_s=240)
    run_distributed(_run_moe, 4, _moe_config(4, 1, mesh={"dp": 2, "ep": 2}), str(tmp_path), str(tmp_path / "ep.pt"), 0,
                    timeout_s=300)
    one = torch.load(f"{tmp_path}/one.pt.0")
    parts = [torch.load(f"{tmp_path}/ep.pt.{r}") for r in range(4)]      # rank = dp * 2 + ep
    for x, y in zip(parts[0]["hist"], one["hist"]):
        assert abs(x["loss"] - y["loss"]) < 1e-4 * max(1.0, abs(y["loss"])), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 1e-3 * max(1.0, abs(y["grad_norm"])), (x, y)
    for ep in range(2):
        for n, v in parts[ep]["params"].items():
            assert torch.equal(v, parts[2 + ep]["params"][n]), n         # same ep coordinate, other replica
            want = one["params"][n]
            if v.shape != want.shape:
                want = want[ep * v.shape[0]:(ep + 1) * v.shape[0]]
            assert (v - want).abs().max().item() < 5 * 3e-4, (n, (v - want).abs().max().item())


def _run_moe_resume(rank, world, home, out):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    mesh = {"dp": 1, "ep": 2}
    straight = Trainer(_moe_config(2, 1, mesh=mesh, run_name="ep_straight"), rank, rank, world, device="cpu")
    straight.train()
    first = Trainer(_moe_config(2, 1, mesh=mesh, run_name="ep_resumed", save_steps=3), rank, rank, world, device="cpu")
    first.num_train_steps = 3
    first.train()
    second = Trainer(_moe_config(2, 1, mesh=mesh, run_name="ep_resumed", resume="auto", save_steps=1000), rank, rank,
                     world, device="cpu")
    assert second.start_step == 3
    second.train()
    torch.save({"a": _weights(straight), "b": _weights(second)}, f"{out}.{rank}")


def test_expert_parallel_resume_is_exact(tmp_path):
    run_distributed(_run_moe_resume, 2, str(tmp_path), str(tmp_path / "r.pt"), timeout_s=240)
    for r in range(2):
        got = torch.load(f"{tmp_path}/r.pt.{r}")
        for n in got["a"]:
            assert torch.equal(got["a"][n], got["b"][n]), n
    files = sorted(os.listdir(tmp_path / "checkpoints" / "ep_resumed" / "3"))
    assert "model_shard0.pt" in files and "model_shard1.pt" in files and "optimizer_shard1.pt" in files, files
    assert "dataloader_rank0.pt" in " ".join(files) or any(f.startswith("dataloader") for f in files), files


def _run_pp(rank, world, cfg, home, out, emulate_world):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    tr = Trainer(cfg, rank, rank, world, benchmark=True, device="cpu")
    assert type(tr.model).__name__ == "PipelineStage" and tr.model.stages == cfg["mesh"]["pp"]
    hist = tr.train_n_step_test(STEPS)
    params = _weights(tr)          # the stage's tensors under the keys of the whole model
    torch.save({"hist": hist, "params": params}, f"{out}.{rank}")


def test_pipeline_trainer_matches_single_process(tmp_path, schedule="1f1b"):
    """mesh {dp: 1, pp: 2}: two stages of two blocks, the tied embedding / head held by both (gradients summed,
    values equal), four micro-batches per step through the schedule, the clip norm taken over both stages.  Loss,
    gradient norm and the final weights of BOTH stages must follow the single-process run."""
    pp_cfg = parity_config(world=1, steps=STEPS, accumulation=4, mesh={"dp": 1, "pp": 2})
    pp_cfg["pp"] = {"schedule": schedule}
    run_distributed(_run_pp, 2, pp_cfg, str(tmp_path), str(tmp_path / "pp.pt"), 0, timeout_s=240)
    one = _single_process(tmp_path, 4, 0)
    parts = [torch.load(f"{tmp_path}/pp.pt.{r}") for r in range(2)]
    assert "token_emb.weight" in parts[0]["params"] and "lm_head.weight" in parts[1]["params"]
    assert "blocks.0.norm1.weight" in parts[0]["params"] and "blocks.3.norm1.weight" in parts[1]["params"]
    merged = {**parts[0]["params"], **parts[1]["params"]}
    # the whole model lists its tied tensor once, as the embedding; the last stage holds it as the head
    assert torch.equal(parts[0]["params"]["token_emb.weight"], merged.pop("lm_head.weight"))
    assert set(merged) == set(one["params"])
    for part in parts:      # every stage reports the same loss and norm
        assert [h["loss"] for h in part["hist"]] == [h["loss"] for h in parts[0]["hist"]]
    _compare({"hist": parts[0]["hist"], "params": merged}, one)


def test_pipeline_with_data_parallel_replicas(tmp_path):
    """mesh {dp: 2, pp: 2} on four ranks (GPipe order) against one process fed the rows of both replicas."""
    pp_cfg = parity_config(world=2, steps=STEPS, accumulation=2, mesh={"dp": 2, "pp": 2})
    pp_cfg["pp"] = {"schedule": "gpipe"}
    run_distributed(_run_pp, 4, pp_cfg, str(tmp_path), str(tmp_path / "pp.pt"), 0, timeout_s=300)
    one = _single_process(tmp_path, 4, 2)
    parts = [torch.load(f"{tmp_path}/pp.pt.{r}") for r in range(4)]    # ranks 0 / 1: stages 0 / 1 of replica 0
    merged = {**parts[0]["params"], **parts[1]["params"]}
    merged.pop("lm_head.weight")
    _compare({"hist": parts[0]["hist"], "params": merged}, one)
    for n, v in parts[2]["params"].items():
        assert torch.equal(v, parts[0]["params"][n]), n      # the replicas stay identical


def _run_pp_resume(rank, world, home, out):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    mesh = {"dp": 1, "pp": 2}
    straight = Trainer(parity_config(1, steps=5, run_name="pp_straight", accumulation=2, mesh=mesh), rank, rank, world,
                       device="cpu")
    straight.train()
    first = Trainer(parity_config(1, steps=5, run_name="pp_resumed", accumulation=2, save_steps=3, mesh=mesh), rank,
                    rank, world, device="cpu")
    first.num_train_steps = 3
    first.train()
    second = Trainer(parity_config(1, steps=5, run_name="pp_resumed", accumulation=2, resume="auto", save_steps=1000,
                                   mesh=mesh), rank, rank, world, device="cpu")
    assert second.start_step == 3
    second.train()
    torch.save({"a": _weights(straight), "b": _weights(second)}, f"{out}.{rank}")


def test_pipeline_resume_is_exact(tmp_path):
    run_distributed(_run_pp_resume, 2, str(tmp_path), str(tmp_path / "r.pt"), timeout_s=240)
    for r in range(2):
        got = torch.load(f"{tmp_path}/r.pt.{r}")
        for n in got["a"]:
            assert torch.equal(got["a"][n], got["b"][n]), n
    files = sorted(os.listdir(tmp_path / "checkpoints" / "pp_resumed" / "3"))
    assert "model_shard0.pt" in files and "model_shard1.pt" in files and "optimizer_shard1.pt" in files, files


def _run_and_save(rank, world, cfg, home):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    Trainer(cfg, rank, rank, world, device="cpu").train()


def _check_warm_start(rank, world, cfg, home, merged_path):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    tr = Trainer(cfg, rank, rank, world, device="cpu")
    merged = torch.load(merged_path)
    sd = tr.model.state_dict()
    q = merged["blocks.1.gqa.q_proj.weight"]
    per = q.shape[0] // world
    assert torch.equal(sd["blocks.1.gqa.q_proj.weight"], q[rank * per:(rank + 1) * per])
    d = merged["blocks.2.ffn.down_proj.weight"]
    perc = d.shape[1] // world
    assert torch.equal(sd["blocks.2.ffn.down_proj.weight"], d[:, rank * perc:(rank + 1) * perc])
    assert torch.equal(sd["token_emb.weight"], merged["token_emb.weight"])
    assert torch.equal(sd["norm.weight"], merged["norm.weight"])
    tr.train_n_step_test(1)


def test_sharded_checkpoints_merge_into_the_unsharded_layout(tmp_path):
    """Tensor-parallel, pipeline and expert-parallel runs write one model file per coordinate; merged, they must load
    (strictly) into the whole model and, for the dense model, equal what a single process trained on the same rows."""
    from torchure_b200.ckpt.merge import merge_model_shards
    from torchure_b200.models import build_model

    one = _single_process(tmp_path, 4, 0)
    for name, mesh in (("tp", {"dp": 1, "tp": 2}), ("pp", {"dp": 1, "pp": 2})):
        cfg = parity_config(world=1, steps=STEPS, accumulation=4, mesh=mesh, run_name=f"merge_{name}", save_steps=STEPS)
        run_distributed(_run_and_save, 2, cfg, str(tmp_path), timeout_s=240)
        root = str(tmp_path / "checkpoints" / f"merge_{name}")
        merged = merge_model_shards(root, STEPS)
        model = build_model(cfg["model"]["name"], cfg["model"]["config"])
        model.load_state_dict(merged)          # strict: every key, every shape
        got = {n: p.detach() for n, p in model.named_parameters()}
        _compare({"hist": one["hist"], "params": got}, one)
    # ... and the merged file of the pipeline run starts a tensor-parallel run (`init_from`): the ranks' slices must be
    # the slices of the merged tensors
    out = str(tmp_path / "merged_pp.pt")
    torch.save(merged, out)
    warm = parity_config(world=1, steps=STEPS, accumulation=4, mesh={"dp": 1, "tp": 2}, run_name="warm_tp")
    warm["init_from"] = out
    run_distributed(_check_warm_start, 2, warm, str(tmp_path), out, timeout_s=240)
    cfg = _moe_config(2, 1, mesh={"dp": 1, "ep": 2}, run_name="merge_ep", save_steps=STEPS)
    run_distributed(_run_and_save, 2, cfg, str(tmp_path), timeout_s=240)
    merged = merge_model_shards(str(tmp_path / "checkpoints" / "merge_ep"), STEPS)
    model = build_model(cfg["model"]["name"], cfg["model"]["config"])
    model.load_state_dict(merged)
    assert merged["blocks.0.ffn.w_gate"].shape[0] == 4
    ids = torch.randint(0, 4096, (1, 32), generator=torch.Generator().manual_seed(0))
    assert torch.isfinite(model(ids)).all()


def _run_fsdp_resume(rank, world, home, out):
    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    mesh = {"dp_shard": 2}
    straight = Trainer(parity_config(2, steps=5, run_name="fs_straight", accumulation=1, mesh=mesh), rank, rank, world,
                       device="cpu")
    straight.train()
    first = Trainer(parity_config(2, steps=5, run_name="fs_resumed", accumulation=1, save_steps=3, mesh=mesh), rank,
                    rank, world, device="cpu")
    first.num_train_steps = 3
    first.train()
    second = Trainer(parity_config(2, steps=5, run_name="fs_resumed", accumulation=1, resume="auto", save_steps=1000,
                                   mesh=mesh), rank, rank, world, device="cpu")
    assert second.start_step == 3
    second.train()
    a, b = _weights(straight), _weights(second)
    if rank == 0:
        torch.save({"a": a, "b": b}, out)


def test_fsdp_resume_is_exact(tmp_path):
    run_distributed(_run_fsdp_resume, 2, str(tmp_path), str(tmp_path / "r.pt"), timeout_s=240)
    got = torch.load(tmp_path / "r.pt")
    for n in got["a"]:
        assert torch.equal(got["a"][n], got["b"][n]), n
    files = sorted(os.listdir(tmp_path / "checkpoints" / "fs_resumed" / "3"))
    assert "model.pt" in files and "optimizer_shard0.pt" in files and "optimizer_shard1.pt" in files, files


def test_ddp_world2_matches_single_process(tmp_path):
    ddp_cfg = parity_config(world=2, steps=STEPS, accumulation=2)
    one_cfg = parity_config(world=1, steps=STEPS, accumulation=4)
    assert ddp_cfg["data"]["global_batch_size"] == one_cfg["data"]["global_batch_size"] == 8
    run_distributed(_run, 2, ddp_cfg, str(tmp_path), str(tmp_path / "ddp.pt"), 0, timeout_s=240)
    _compare(torch.load(tmp_path / "ddp.pt"), _single_process(tmp_path, 4, 2))  # Adam amplifies summation-order noise


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
