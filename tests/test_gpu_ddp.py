"""Fused DDP reducer on one GPU (world size 1: cast + fp32 accumulation + sum of squares, no communication)
and the trainer's fused clip path."""

import os

import pytest
import torch
import torch.distributed as dist

pytestmark = pytest.mark.gpu

CFG = dict(num_layers=2, num_heads=4, num_kv_heads=2, emb_dim=512, head_dim=128, vocab_size=4096, ffn_dim=1024)


@pytest.fixture(scope="module")
def pg():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1)
    yield
    dist.destroy_process_group()


def relerr(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def test_fused_reducer_world1_accumulates_in_fp32(pg):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.models import Qwen3
    from torchure_b200.objectives import ARObjective
    from torchure_b200.parallel.ddp import DDP

    torch.manual_seed(0)
    model = Qwen3(**CFG).cuda()
    model.init_weights()
    twin = Qwen3(**CFG).cuda()
    twin.load_state_dict(model.state_dict())
    ddp = DDP(model, Mesh({"dp": 1}), "dp", bucket_mb=1)
    assert ddp.fused and ddp.active
    obj = ARObjective(fused_linear_ce=True, ce_chunk_size=256)
    for cycle in range(2):
        ids = torch.randint(0, CFG["vocab_size"], (2, 2, 128), device="cuda")
        model.zero_grad()
        twin.zero_grad()
        for k in range(2):  # two micro-batches: the folded 1/2 scale is exact in bf16
            ddp.requires_sync = k == 1
            obj.compute_loss(model, {"input_ids": ids[k], "labels": ids[k]}, loss_scale=1 / 2).backward()
            (obj.compute_loss(twin, {"input_ids": ids[k], "labels": ids[k]}) / 2).backward()
        ddp.sync()
        total = 0.0
        for (n, p), (_, q) in zip(model.named_parameters(), twin.named_parameters()):
            assert p.grad.dtype == torch.float32
            assert relerr(p.grad, q.grad) < 1e-5, (n, cycle)
            total += q.grad.double().pow(2).sum().item()
        assert abs(ddp.sq_norm().item() - total) < 1e-3 * total
        flat = ddp.reducer.flat
        assert all(flat.data_ptr() <= p.grad.data_ptr() < flat.data_ptr() + flat.numel() * 4 for p in model.parameters())


def test_trainer_steps_gpu(pg, tmp_path):
    """Public Trainer API on one GPU: loss goes down over a few steps, clip coefficient applied on device."""
    os.environ["TORCHURE_B200_HOME"] = str(tmp_path)
    from torchure_b200.train.trainer import Trainer

    cfg = {
        "model": {"name": "qwen3_dense", "config": dict(CFG)},
        "mesh": {"dp": 1}, "seed": 1,
        "optimizer": {"name": "adamw", "config": {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "fused": True},
                      "max_norm": 1.0,
                      "scheduler": {"type": "wsd", "warmup_ratio": 0.1, "decay_ratio": 0.2, "total_steps": 20}},
        "objective": {"name": "AR", "config": {"ignore_index": -100, "fused_linear_ce": True, "ce_chunk_size": 256}},
        "data": {"name": "synthetic", "synthetic": True, "seed": 3, "mean_doc_len": 64, "eos_id": 0, "num_workers": 0,
                 "global_batch_size": 4, "micro_batch_size": 2, "seq_len": 256},
        "checkpointing": {"save_steps": 1000, "resume": None}, "run_name": "gpu_trainer",
    }
    tr = Trainer(cfg, 0, 0, 1, benchmark=True)
    hist = tr.train_n_step_test(8)
    assert all(torch.isfinite(torch.tensor(h["loss"])) for h in hist)
    assert hist[-1]["loss"] < hist[0]["loss"]
    assert hist[0]["grad_norm"] > 0


def test_trainer_cuda_graph_matches_eager(pg, tmp_path):
    """The captured-and-replayed device step follows the eager step: same losses, grad norms and weights over steps
    that cross the warm-up / capture / replay boundary and an lr schedule (lr and bias corrections are device-resident)."""
    os.environ["TORCHURE_B200_HOME"] = str(tmp_path)
    from torchure_b200.train.trainer import Trainer

    def cfg(graph):
        return {
            "model": {"name": "qwen3_dense", "config": dict(CFG)},
            "mesh": {"dp": 1}, "seed": 1, "cuda_graph": graph, "cuda_graph_warmup": 2,
            "optimizer": {"name": "adamw", "config": {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "fused": True},
                          "max_norm": 1.0,
                          "scheduler": {"type": "wsd", "warmup_ratio": 0.3, "decay_ratio": 0.3, "total_steps": 10}},
            "objective": {"name": "AR", "config": {"ignore_index": -100, "fused_linear_ce": True, "ce_chunk_size": 256}},
            "data": {"name": "synthetic", "synthetic": True, "seed": 3, "mean_doc_len": 64, "eos_id": 0, "num_workers": 0,
                     "global_batch_size": 4, "micro_batch_size": 2, "seq_len": 256},
            "checkpointing": {"save_steps": 1000, "resume": None}, "run_name": f"gpu_graph_{int(graph)}",
        }

    eager = Trainer(cfg(False), 0, 0, 1, benchmark=True)
    h_eager = eager.train_n_step_test(8)
    graphed = Trainer(cfg(True), 0, 0, 1, benchmark=True)
    h_graph = graphed.train_n_step_test(8)
    assert graphed._graph is not None, "the graph path must have been taken"
    for a, b in zip(h_eager, h_graph):
        assert abs(a["loss"] - b["loss"]) < 2e-3 * abs(a["loss"]), (a, b)
        assert abs(a["grad_norm"] - b["grad_norm"]) < 2e-2 * abs(a["grad_norm"]), (a, b)
    for (n, p), (_, q) in zip(eager.model.named_parameters(), graphed.model.named_parameters()):
        assert relerr(p, q) < 5e-3, n  # atomics order differs run to run and Adam amplifies it on tiny gradients
    # the optimizer's host bookkeeping advanced once per step, capture included
    st = graphed.optimizer.state[next(iter(graphed.model.parameters()))]
    assert int(st["step"].item()) == 8


def _gpu_cfg(run_name, graph=True, resume=None, save_steps=1000, steps=8):
    return {
        "model": {"name": "qwen3_dense", "config": dict(CFG)},
        "mesh": {"dp": 1}, "seed": 1, "cuda_graph": graph, "cuda_graph_warmup": 1,
        "optimizer": {"name": "adamw", "config": {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "fused": True},
                      "max_norm": 1.0,
                      "scheduler": {"type": "wsd", "warmup_ratio": 0.3, "decay_ratio": 0.3, "total_steps": steps}},
        "objective": {"name": "AR", "config": {"ignore_index": -100, "fused_linear_ce": True, "ce_chunk_size": 256}},
        "data": {"name": "synthetic", "synthetic": True, "seed": 3, "mean_doc_len": 64, "eos_id": 0, "num_workers": 0,
                 "global_batch_size": 4, "micro_batch_size": 2, "seq_len": 256},
        "checkpointing": {"save_steps": save_steps, "resume": resume}, "run_name": run_name,
    }


def test_trainer_resume_gpu_with_graph_replay(pg, tmp_path):
    """Checkpoint / resume through the GPU path: bf16 shadow weights, device-resident AdamW scalars and the captured
    step all restart from the files.  8 straight steps against 4 steps + checkpoint + 4 resumed steps (both replay
    the device step from a CUDA graph).  The gradient kernels use fp32 atomics, so the comparison is to rounding
    noise, not bitwise."""
    os.environ["TORCHURE_B200_HOME"] = str(tmp_path)
    from torchure_b200.train.trainer import Trainer

    straight = Trainer(_gpu_cfg("gpu_straight"), 0, 0, 1, benchmark=True)
    straight.train()
    first = Trainer(_gpu_cfg("gpu_resumed", save_steps=4), 0, 0, 1, benchmark=True)
    first.num_train_steps = 4
    first.train()
    assert first._graph is not None
    second = Trainer(_gpu_cfg("gpu_resumed", resume="auto"), 0, 0, 1, benchmark=True)
    assert second.start_step == 4
    second.train()
    assert second._graph is not None
    assert int(second.optimizer.state[next(iter(second.model.parameters()))]["step"].item()) == 8
    assert abs(second.scheduler.get_last_lr()[0] - straight.scheduler.get_last_lr()[0]) < 1e-12
    for (n, p), (_, q) in zip(straight.model.named_parameters(), second.model.named_parameters()):
        assert relerr(q, p) < 5e-3, n
    # the shadows the GEMMs read are the bf16 image of the resumed masters
    for p, shadow in second.model.engine().shadow_pairs():
        assert relerr(shadow, p.detach().bfloat16()) < 1e-6
