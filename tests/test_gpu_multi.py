"""Multi-GPU: NVLink collective kernels (peer loads/stores and multimem) against closed forms, and the fused DDP
reducer against a single-process run.  One process per GPU; skipped with fewer than 2 GPUs."""

import pytest
import torch

from tests.gpu_dist_utils import run_on_gpus

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

CFG = dict(num_layers=2, num_heads=4, num_kv_heads=2, emb_dim=512, head_dim=128, vocab_size=4096, ffn_dim=1024)


def _world():
    return min(torch.cuda.device_count(), 8)


def _collectives(rank, world):
    from torchure_b200.core import collective as C
    from torchure_b200.core.mesh import Mesh

    mesh = Mesh({"dp": world})
    comm = C.enable_sm100(mesh, "dp", 64 << 20)
    assert comm is not None
    tri = world * (world + 1) / 2
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 2e-2)):
        for n in (5, 1024, 70_000, 3_000_001):
            base = (torch.arange(n, device="cuda") % 251).float() / 251.0
            x = (base * (rank + 1)).to(dtype)
            C.all_reduce(x, mesh, "dp", "sum")
            torch.testing.assert_close(x.float(), (base.to(dtype).float() * tri), rtol=tol, atol=tol * tri)
            x = (base * (rank + 1)).to(dtype)
            C.all_reduce(x, mesh, "dp", "avg")
            torch.testing.assert_close(x.float(), base.to(dtype).float() * tri / world, rtol=tol, atol=tol)
            x = (base * (rank + 1)).to(dtype)
            C.all_reduce(x, mesh, "dp", "max")
            torch.testing.assert_close(x.float(), (base * world).to(dtype).float(), rtol=tol, atol=tol)
        # broadcast from coordinate 1
        x = torch.full((1000,), float(rank), device="cuda", dtype=dtype)
        C.broadcast(x, mesh, "dp", src=1)
        assert (x == 1).all()
        # all_gather / reduce_scatter / all_to_all
        x = torch.full((3, 5), float(rank), device="cuda", dtype=dtype)
        g = C.all_gather(x, mesh, "dp", 0)
        assert g.shape == (3 * world, 5)
        for r in range(world):
            assert (g[3 * r:3 * r + 3] == r).all()
        full = (torch.arange(world * 7, device="cuda").float() * (rank + 1)).to(dtype)
        rs = C.reduce_scatter(full, mesh, "dp", "sum")
        want = torch.arange(world * 7, device="cuda").float()[rank * 7:(rank + 1) * 7] * tri
        torch.testing.assert_close(rs.float(), want, rtol=2e-2, atol=1.0 if dtype == torch.bfloat16 else 1e-4)
        x = torch.tensor([[rank * 100.0 + j] * 4 for j in range(world)], device="cuda", dtype=dtype)
        a2a = C.all_to_all(x, mesh, "dp", 0, 0)
        want = torch.tensor([[s * 100.0 + rank] * 4 for s in range(world)], device="cuda", dtype=dtype)
        torch.testing.assert_close(a2a, want)
    comm.check()


def test_collectives_nvls():
    run_on_gpus(_collectives, _world())


def test_collectives_peer_loads_only():
    run_on_gpus(_collectives, _world(), env={"TORCHURE_B200_NVLS": "0"})


def _ddp_parity(rank, world):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.models import Qwen3
    from torchure_b200.objectives import ARObjective
    from torchure_b200.parallel.ddp import DDP

    mesh = Mesh({"dp": world})
    torch.manual_seed(100 + rank)  # different init per rank: the constructor must replicate rank 0
    model = Qwen3(**CFG).cuda()
    model.init_weights()
    # embed_tokens switches on the early reduction of the tied table's bucket plus the exchange of embedding rows
    ddp = DDP(model, mesh, "dp", bucket_mb=1, embed_tokens=2 * 128)
    assert ddp.fused and ddp.early_table is model.token_emb.weight
    torch.manual_seed(100)
    single = Qwen3(**CFG).cuda()
    single.init_weights()
    for (n, p), (_, q) in zip(model.named_parameters(), single.named_parameters()):
        assert torch.equal(p, q), n
    obj = ARObjective(fused_linear_ce=True, ce_chunk_size=256)
    K = 2
    for cycle in range(2):
        ids = torch.randint(0, CFG["vocab_size"], (K, world, 2, 128), device="cuda",
                            generator=torch.Generator("cuda").manual_seed(cycle))
        model.zero_grad()
        single.zero_grad()
        for k in range(K):
            ddp.requires_sync = k == K - 1
            obj.compute_loss(model, {"input_ids": ids[k, rank], "labels": ids[k, rank]}, loss_scale=1 / K).backward()
        ddp.sync()
        for k in range(K):
            flat = ids[k].reshape(world * 2, 128)
            (obj.compute_loss(single, {"input_ids": flat, "labels": flat}) / K).backward()
        total = 0.0
        for (n, p), (_, q) in zip(model.named_parameters(), single.named_parameters()):
            err = ((p.grad - q.grad).norm() / q.grad.norm().clamp_min(1e-12)).item()
            assert err < 2e-2, (n, cycle, err)
            total += p.grad.double().pow(2).sum().item()
        sq = ddp.sq_norm().item()
        assert abs(sq - total) < 1e-3 * total, (sq, total)
        # every rank holds bit-identical reduced gradients and the same norm
        check = torch.tensor([sq], device="cuda", dtype=torch.float64)
        lo, hi = check.clone(), check.clone()
        torch.distributed.all_reduce(lo, op=torch.distributed.ReduceOp.MIN)
        torch.distributed.all_reduce(hi, op=torch.distributed.ReduceOp.MAX)
        assert lo.item() == hi.item()
    ddp.reducer.comm.check()


def test_fused_ddp_matches_single_process():
    run_on_gpus(_ddp_parity, min(_world(), 4))


def test_fused_ddp_peer_loads_only():
    run_on_gpus(_ddp_parity, 2, env={"TORCHURE_B200_NVLS": "0"})


def _gemm_comm(rank, world):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.core.symm import SymmComm
    from torchure_b200.ops import kernels
    from torchure_b200.ops.gemm_comm import SymmetricOperand, ag_gemm, gemm_rs

    mesh = Mesh({"tp": world})
    comm = SymmComm(mesh.get_group("tp"), rank, world, staging_bytes=1 << 20, persistent_bytes=256 << 20)
    # all-gather -> GEMM: A row-sharded, B local; two shapes on one communicator (the arrival words are shared)
    for rows, K, N in ((256, 512, 512), (512, 1024, 768)):
        M = rows * world
        a_sh = SymmetricOperand(comm, (rows, K), torch.bfloat16)
        g = torch.Generator("cuda").manual_seed(7)
        a_full = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
        a_sh.tensor.copy_(a_full[rank * rows:(rank + 1) * rows])
        for _ in range(2):  # twice: the handshake flags must re-arm
            out, gathered = ag_gemm(comm, a_sh, b, return_gathered=True)
            ref = a_full.float() @ b.float().t()
            err = ((out.float() - ref).norm() / ref.norm()).item()
            assert err < 5e-3, ("ag_gemm", err)
            assert torch.equal(gathered, a_full)
        out = ag_gemm(comm, a_sh, b.t().contiguous(), b_mn=True)  # same product, B stored [K, N]
        err = ((out.float() - ref).norm() / ref.norm()).item()
        assert err < 5e-3, ("ag_gemm b_mn", err)
    # GEMM -> reduce-scatter: K split over ranks
    Kl = 512
    a_loc = torch.randn(M, Kl, device="cuda", generator=torch.Generator("cuda").manual_seed(100 + rank)).bfloat16()
    b_loc = torch.randn(N, Kl, device="cuda", generator=torch.Generator("cuda").manual_seed(200 + rank)).bfloat16()
    c_sh = SymmetricOperand(comm, (rows, N), torch.float32)
    partial = a_loc.float() @ b_loc.float().t()
    torch.distributed.all_reduce(partial)
    for _ in range(2):
        got = gemm_rs(comm, a_loc, b_loc, c_sh)
        torch.cuda.synchronize()
        want = partial[rank * rows:(rank + 1) * rows]
        err = ((got - want).norm() / want.norm()).item()
        assert err < 1e-3, ("gemm_rs", err)
        torch.distributed.barrier()
    got = gemm_rs(comm, a_loc, b_loc.t().contiguous(), c_sh, b_mn=True)
    torch.cuda.synchronize()
    err = ((got - want).norm() / want.norm()).item()
    assert err < 1e-3, ("gemm_rs b_mn", err)
    comm.check()
    kernels.check_error()


def test_fused_gemm_collectives():
    run_on_gpus(_gemm_comm, min(_world(), 4))


def _sp_fused_linears(rank, world):
    import torch.nn as nn

    from torchure_b200.core import collective
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.ops import kernels
    from torchure_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, _fused_comm

    mesh = Mesh({"tp": world})
    collective.enable_sm100(mesh, "tp", max_bytes=64 << 20, persistent_bytes=128 << 20)
    torch.manual_seed(3)
    D, F, S = 512, 1024, 256 * world
    up, down = nn.Linear(D, F, bias=False).cuda(), nn.Linear(F, D, bias=False).cuda()
    x_full = torch.randn(1, S, D, device="cuda")
    dy_full = torch.randn(1, S, D, device="cuda")
    rows = S // world
    # fp32 oracle on the full problem
    xr = x_full.clone().requires_grad_(True)
    yr = down(torch.nn.functional.silu(up(xr)))  # smooth: a sign flip under bf16 rounding would dominate the error
    yr.backward(dy_full)
    col = ColumnParallelLinear(up, mesh, "tp", sequence_parallel=True)
    row = RowParallelLinear(down, mesh, "tp", sequence_parallel=True)
    xs = x_full[:, rank * rows:(rank + 1) * rows].bfloat16().requires_grad_(True)
    assert _fused_comm(xs, mesh, "tp") is not None, "the fused path must be the one under test"
    ys = row(torch.nn.functional.silu(col(xs)))
    ys.backward(dy_full[:, rank * rows:(rank + 1) * rows].bfloat16())
    torch.cuda.synchronize()

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm()).item()

    per_f = F // world
    errs = {"y": rel(ys, yr[:, rank * rows:(rank + 1) * rows]),
            "dx": rel(xs.grad, xr.grad[:, rank * rows:(rank + 1) * rows]),
            "dw_col": rel(col.weight.grad, up.weight.grad[rank * per_f:(rank + 1) * per_f]),
            "dw_row": rel(row.weight.grad, down.weight.grad[:, rank * per_f:(rank + 1) * per_f])}
    assert max(errs.values()) < 2e-2, errs
    kernels.check_error()


def test_sequence_parallel_fused_linears():
    run_on_gpus(_sp_fused_linears, min(_world(), 4))


# ---- sharded training on the engine and the Trainer on several GPUs -------------------------------------------------
def _fsdp_parity(rank, world):
    """EngineFSDP against one unsharded model: reduce-scattered gradients, the published norm, two AdamW steps on
    the shards, the in-place all-gather of the bf16 weights."""
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.models import Qwen3
    from torchure_b200.objectives import ARObjective
    from torchure_b200.optim import build_optimizer
    from torchure_b200.parallel.fsdp_engine import EngineFSDP

    mesh = Mesh({"dp_shard": world})
    torch.manual_seed(100 + rank)
    model = Qwen3(**CFG).cuda()
    model.init_weights()
    torch.manual_seed(100)
    single = Qwen3(**CFG).cuda()
    single.init_weights()
    fsdp = EngineFSDP(model, mesh, "dp_shard")
    opt_cfg = {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "fused": True}
    opt = build_optimizer(None, "adamw", opt_cfg, params=fsdp.optimizer_params())
    fsdp.attach_shadows(opt)
    ref_opt = build_optimizer(single, "adamw", opt_cfg)
    for p, shadow in single.engine().shadow_pairs():
        ref_opt.attach_shadow(p, shadow)
    obj = ARObjective(fused_linear_ce=True, ce_chunk_size=256)
    K = 2
    ref_names = dict(single.named_parameters())
    for cycle in range(3):
        ids = torch.randint(0, CFG["vocab_size"], (K, world, 2, 128), device="cuda",
                            generator=torch.Generator("cuda").manual_seed(cycle))
        single.zero_grad()
        fsdp.begin_step()
        for k in range(K):
            fsdp.requires_sync = k == K - 1
            obj.compute_loss(model, {"input_ids": ids[k, rank], "labels": ids[k, rank]}, loss_scale=1 / K).backward()
        fsdp.sync()
        for k in range(K):
            flat = ids[k].reshape(world * 2, 128)
            (obj.compute_loss(single, {"input_ids": flat, "labels": flat}) / K).backward()
        total = 0.0
        for u in fsdp.units:
            for m in u.mats:
                want = torch.cat([ref_names[n].grad for n in m.names], dim=0)
                lo = rank * m.per
                err = ((m.shard.grad - want[lo:lo + m.per]).norm() / want[lo:lo + m.per].norm().clamp_min(1e-12)).item()
                # after the first optimizer step the two models differ by Adam's sign flips on noise-level gradients
                assert err < (4e-2 if cycle == 0 else 1e-1), (m.name, cycle, err)
                total += want.double().pow(2).sum().item()
        names = {p: n for n, p in model.named_parameters()}
        for p in fsdp.gains:
            want = ref_names[names[p]].grad
            err = ((p.grad - want).norm() / want.norm().clamp_min(1e-12)).item()
            assert err < (5e-2 if cycle == 0 else 1.5e-1), (names[p], cycle, err)
            total += want.double().pow(2).sum().item()
        sq = fsdp.sq_norm().item()
        if cycle == 0:
            assert abs(sq - total) < 2e-3 * total, (sq, total)
        mine = sum(m.shard.grad.double().pow(2).sum().item() for u in fsdp.units for m in u.mats)
        t = torch.tensor([mine], device="cuda", dtype=torch.float64)
        torch.distributed.all_reduce(t)
        gains = sum(p.grad.double().pow(2).sum().item() for p in fsdp.gains)
        assert abs(sq - (t.item() + gains)) < 1e-4 * sq, (sq, t.item() + gains)   # the published partials are exact
        opt.step()
        fsdp.mark_updated()
        opt.zero_grad()
        ref_opt.step()
        # the fused AdamW wrote this rank's rows of the bf16 copies; the in-place all-gather fills in the peers'
        fsdp.begin_step()
        for u in fsdp.units:
            fsdp.wait_gathered(u.index)
            for m in u.mats:
                whole = torch.empty(world * m.per, m.cols, device="cuda")
                torch.distributed.all_gather_into_tensor(whole, m.shard.detach().contiguous())
                assert torch.equal(m.full_w, whole.bfloat16()), (m.name, cycle)
    sd = fsdp.full_state_dict()
    for n, q in single.named_parameters():
        err = ((sd[n] - q).norm() / q.norm()).item()
        assert err < 5e-2, (n, err)
    fsdp.comm.check()


def test_engine_fsdp_matches_single_process():
    run_on_gpus(_fsdp_parity, min(_world(), 4))


def test_engine_fsdp_peer_loads_only():
    run_on_gpus(_fsdp_parity, 2, env={"TORCHURE_B200_NVLS": "0"})


def _trainer_cfg(mesh, run_name, global_batch, graph=True, steps=6):
    return {
        "model": {"name": "qwen3_dense", "config": dict(CFG)},
        "mesh": dict(mesh), "seed": 1, "cuda_graph": graph, "cuda_graph_warmup": 1,
        "optimizer": {"name": "adamw", "config": {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "fused": True},
                      "max_norm": 1.0,
                      "scheduler": {"type": "wsd", "warmup_ratio": 0.3, "decay_ratio": 0.3, "total_steps": steps}},
        "objective": {"name": "AR", "config": {"ignore_index": -100, "fused_linear_ce": True, "ce_chunk_size": 256}},
        "data": {"name": "synthetic", "synthetic": True, "seed": 3, "mean_doc_len": 64, "eos_id": 0, "num_workers": 0,
                 "global_batch_size": global_batch, "micro_batch_size": 2, "seq_len": 256},
        "ddp": {"bucket_mb": 1},
        "checkpointing": {"save_steps": 1000, "resume": None}, "run_name": run_name,
    }


def _trainer_strategies(rank, world, home, out):
    """Trainer end to end on `world` GPUs, CUDA-graph replay on: DDP and FSDP (selected by the mesh alone) must follow
    the same loss and gradient-norm trajectory, and an FSDP checkpoint must resume."""
    import os

    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    steps = 6
    ddp = Trainer(_trainer_cfg({"dp": world}, "t_ddp", 4 * world, steps=steps), rank, rank, world, benchmark=True)
    h_ddp = ddp.train_n_step_test(steps)
    assert ddp._graph is not None
    del ddp
    torch.cuda.empty_cache()
    cfg = _trainer_cfg({"dp_shard": world}, "t_fsdp", 4 * world, steps=steps)
    cfg["checkpointing"]["save_steps"] = 3
    fsdp = Trainer(cfg, rank, rank, world, benchmark=True)
    assert type(fsdp.ddp).__name__ == "EngineFSDP"
    fsdp.train()
    fsdp.check_device_errors()
    # the same run, resumed from its step-3 checkpoint (sharded optimizer files), must end where the straight run did
    cfg2 = _trainer_cfg({"dp_shard": world}, "t_fsdp", 4 * world, steps=steps)
    cfg2["checkpointing"]["resume"] = 3
    again = Trainer(cfg2, rank, rank, world, benchmark=True)
    assert again.start_step == 3
    again.train()
    a, b = fsdp.ddp.full_state_dict(), again.ddp.full_state_dict()
    for n in a:
        err = ((a[n] - b[n]).norm() / a[n].norm()).item()
        assert err < 5e-3, (n, err)
    del fsdp, again
    torch.cuda.empty_cache()
    f2 = Trainer(_trainer_cfg({"dp_shard": world}, "t_fsdp2", 4 * world, steps=steps), rank, rank, world, benchmark=True)
    h_fsdp = f2.train_n_step_test(steps)
    assert f2._graph is not None
    for x, y in zip(h_ddp, h_fsdp):
        assert abs(x["loss"] - y["loss"]) < 5e-3 * abs(x["loss"]), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 3e-2 * abs(x["grad_norm"]), (x, y)
    if rank == 0:
        torch.save({"ddp": h_ddp, "fsdp": h_fsdp}, out)


def test_trainer_ddp_and_fsdp_on_gpus(tmp_path):
    run_on_gpus(_trainer_strategies, min(_world(), 4), str(tmp_path), str(tmp_path / "h.pt"), timeout_s=240)
    got = torch.load(tmp_path / "h.pt")
    assert got["ddp"][-1]["loss"] < got["ddp"][0]["loss"]


def _trainer_vs_single(rank, world, home, out, emulate):
    import os

    os.environ["TORCHURE_B200_HOME"] = home
    from tests.test_trainer_parity import _Interleaved
    from torchure_b200.train.trainer import Trainer

    cfg = _trainer_cfg({"dp": world}, f"t_par_{world}", 4 * max(world, emulate), graph=True)
    tr = Trainer(cfg, rank, rank, world, benchmark=True)
    if emulate:
        from torchure_b200.data import CUDAPrefetcher

        tr.prefetcher = CUDAPrefetcher(_Interleaved(cfg, emulate), tr.device)
    hist = tr.train_n_step_test(6)
    if rank == 0:
        torch.save(hist, out)


def test_trainer_two_gpus_match_one(tmp_path):
    """2-GPU DDP through the Trainer (graph replay, fused reducer) against ONE GPU fed the same rows."""
    run_on_gpus(_trainer_vs_single, 2, str(tmp_path), str(tmp_path / "two.pt"), 0, timeout_s=240)
    run_on_gpus(_trainer_vs_single, 1, str(tmp_path), str(tmp_path / "one.pt"), 2, timeout_s=240)
    two, one = torch.load(tmp_path / "two.pt"), torch.load(tmp_path / "one.pt")
    for x, y in zip(two, one):
        assert abs(x["loss"] - y["loss"]) < 5e-3 * abs(y["loss"]), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 3e-2 * abs(y["grad_norm"]), (x, y)


# ---- long-context strategies on the attention kernels ----------------------------------------------------------------
def _dense_attention(q, k, v):
    """fp32 causal attention on (B, S, H, d) tensors."""
    rep = q.shape[2] // k.shape[2]
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    o = torch.nn.functional.scaled_dot_product_attention(qf, kf.repeat_interleave(rep, 1), vf.repeat_interleave(rep, 1),
                                                         is_causal=True)
    return o.transpose(1, 2)


def _ring_gpu(rank, world):
    """Ring attention over zigzag chunks with every block pair on the tcgen05 kernels: forward and all three
    gradients against dense attention over the whole sequence."""
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.ops import kernels
    from torchure_b200.parallel.context_parallel import ring_attention_tokens, zigzag_split

    mesh = Mesh({"cp": world})
    g = torch.Generator(device="cuda").manual_seed(0)
    B, Hq, Hkv, d = 1, 4, 2, 128
    S = 2 * world * 256
    q, k, v = (torch.randn(B, S, h, d, device="cuda", generator=g).bfloat16() for h in (Hq, Hkv, Hkv))
    do = torch.randn(B, S, Hq, d, device="cuda", generator=g).bfloat16()
    qf, kf, vf = (t.clone().float().requires_grad_() for t in (q, k, v))
    ref = _dense_attention(qf, kf, vf)
    ref.backward(do.float())
    ql, kl, vl = (zigzag_split(t, world, rank, 1).clone().requires_grad_() for t in (q, k, v))
    out = ring_attention_tokens(ql, kl, vl, mesh, "cp")
    assert out.grad_fn is not None and "RingAttentionSm100" in type(out.grad_fn).__name__, type(out.grad_fn)
    out.backward(zigzag_split(do, world, rank, 1))
    kernels.check_error()

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm()).item()

    assert rel(out, zigzag_split(ref.detach(), world, rank, 1)) < 1e-2
    for name, got, want in (("dq", ql.grad, qf.grad), ("dk", kl.grad, kf.grad), ("dv", vl.grad, vf.grad)):
        e = rel(got, zigzag_split(want, world, rank, 1))
        assert e < 2e-2, (name, e)


def test_ring_attention_on_kernels():
    run_on_gpus(_ring_gpu, min(_world(), 4))


def _ulysses_gpu(rank, world):
    from torchure_b200.core import collective as C
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.ops import kernels
    from torchure_b200.parallel.ulysses import ulysses_attention

    mesh = Mesh({"cp": world})
    C.enable_sm100(mesh, "cp", 64 << 20)     # the two all-to-alls run on the NVLink kernel
    g = torch.Generator(device="cuda").manual_seed(0)
    B, S, d = 1, 1024, 128
    Hq, Hkv = 4 * world, 2 * world
    q, k, v = (torch.randn(B, S, h, d, device="cuda", generator=g).bfloat16() for h in (Hq, Hkv, Hkv))
    do = torch.randn(B, S, Hq, d, device="cuda", generator=g).bfloat16()
    qf, kf, vf = (t.clone().float().requires_grad_() for t in (q, k, v))
    ref = _dense_attention(qf, kf, vf)
    ref.backward(do.float())
    ql, kl, vl = (t.chunk(world, dim=1)[rank].clone().requires_grad_() for t in (q, k, v))
    out = ulysses_attention(ql, kl, vl, mesh, "cp")      # default attention: the sm_100a flash_attention op
    out.backward(do.chunk(world, dim=1)[rank])
    kernels.check_error()

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm()).item()

    assert rel(out, ref.detach().chunk(world, dim=1)[rank]) < 1e-2
    for name, got, want in (("dq", ql.grad, qf.grad), ("dk", kl.grad, kf.grad), ("dv", vl.grad, vf.grad)):
        e = rel(got, want.chunk(world, dim=1)[rank])
        assert e < 2e-2, (name, e)


def test_ulysses_on_kernels():
    run_on_gpus(_ulysses_gpu, 2)


def _trainer_tp(rank, world, home, out):
    """Tensor parallelism on the sm_100a engine through the Trainer (mesh {dp: 1, tp: world}): the step's kernels are
    this repository's (no library GEMM or attention kernel in the profiler's census)."""
    import os

    os.environ["TORCHURE_B200_HOME"] = home
    import bench
    from torchure_b200.train.trainer import Trainer

    cfg = _trainer_cfg({"dp": 1, "tp": world}, "t_tp", 4, graph=False)
    tr = Trainer(cfg, rank, rank, world, benchmark=True)
    assert getattr(tr.model, "tp", None) is not None and tr.model.impl != "torch"
    hist = tr.train_n_step_test(6)
    census = bench.kernel_census(tr.train_step_untimed)
    library = [k["name"] for k in census["top"] if k["kind"] == "other" and any(
        w in k["name"].lower() for w in ("cutlass", "gemm", "fmha", "flash", "cudnn", "nvjet", "sdpa", "attention"))]
    assert not library, library
    assert census["own"]["launches"] > 50
    tr.check_device_errors()
    if rank == 0:
        torch.save(hist, out)


def test_trainer_tensor_parallel_on_engine(tmp_path):
    run_on_gpus(_trainer_tp, 2, str(tmp_path), str(tmp_path / "tp.pt"), timeout_s=240)
    run_on_gpus(_trainer_vs_single_cfg, 1, str(tmp_path), str(tmp_path / "one.pt"), timeout_s=240)
    tp, one = torch.load(tmp_path / "tp.pt"), torch.load(tmp_path / "one.pt")
    for x, y in zip(tp, one):
        assert abs(x["loss"] - y["loss"]) < 5e-3 * abs(y["loss"]), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 3e-2 * abs(y["grad_norm"]), (x, y)


def _trainer_cp(rank, world, home, out, kind="ring"):
    """Context parallelism on the sm_100a engine through the Trainer (mesh {dp: 1, cp: world}, or one GPU for the
    comparison): sequences of 512 tokens, so every zigzag chunk is one 128-token block of the pair kernels."""
    import os

    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    mesh = {"dp": 1, "cp": world} if world > 1 else {"dp": 1}
    cfg = _trainer_cfg(mesh, f"t_cp{world}{kind}", 4, graph=False)
    cfg["data"]["seq_len"] = 128 * 2 * 2
    cfg["cp"] = {"kind": kind}
    tr = Trainer(cfg, rank, rank, world, benchmark=True)
    if world > 1:
        assert tr.model.cp is not None
        if kind == "ring":
            assert tr.model.impl != "torch" and tr.model.engine().cp is not None
        seen = []
        tr.model.register_forward_pre_hook(lambda mod, args: seen.append(tuple(args[0].shape)))
    hist = tr.train_n_step_test(6)
    if world > 1:
        assert set(seen) == {(2, 512 // world)}, set(seen)
    tr.check_device_errors()
    if rank == 0:
        torch.save(hist, out)


def test_trainer_context_parallel_on_engine(tmp_path):
    """Ring attention inside the engine, and Ulysses (`cp.kind`) on the module path with the attention kernels
    between its all-to-alls, against one GPU."""
    run_on_gpus(_trainer_cp, 2, str(tmp_path), str(tmp_path / "cp.pt"), timeout_s=240)
    run_on_gpus(_trainer_cp, 2, str(tmp_path), str(tmp_path / "ul.pt"), "ulysses", timeout_s=240)
    run_on_gpus(_trainer_cp, 1, str(tmp_path), str(tmp_path / "one.pt"), timeout_s=240)
    one = torch.load(tmp_path / "one.pt")
    for got in (torch.load(tmp_path / "cp.pt"), torch.load(tmp_path / "ul.pt")):
        for x, y in zip(got, one):
            assert abs(x["loss"] - y["loss"]) < 5e-3 * abs(y["loss"]), (x, y)
            assert abs(x["grad_norm"] - y["grad_norm"]) < 3e-2 * abs(y["grad_norm"]), (x, y)


def _loss_parallel(rank, world, home, out):
    """The loss-parallel fused linear + CE on the kernels (each rank: V / world rows of the head, statistics ->
    two all-reduces -> gradient per chunk) against the unsharded kernel path on the same inputs, then through the
    Trainer (mesh {dp: 1, tp: world}, `tp.loss_parallel`)."""
    import os

    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.core import collective as C
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.loss import fused_linear_cross_entropy
    from torchure_b200.ops import kernels
    from torchure_b200.train.trainer import Trainer

    mesh = Mesh({"tp": world})
    C.enable_sm100(mesh, "tp", 64 << 20)
    g = torch.Generator(device="cuda").manual_seed(0)
    N, D, V = 700, 512, 4096
    h = torch.randn(N, D, device="cuda", generator=g).bfloat16()
    w = torch.randn(V, D, device="cuda", generator=g) * 0.05
    y = torch.randint(0, V, (N,), device="cuda", generator=g)
    y[::7] = -100
    h1, w1 = h.clone().requires_grad_(), w.clone().requires_grad_()
    want = fused_linear_cross_entropy(h1, w1, y, -100, 256)
    want.backward()
    h2, w2 = h.clone().requires_grad_(), w.clone().requires_grad_()
    got = fused_linear_cross_entropy(h2, w2, y, -100, 256, vocab_parallel=(mesh, "tp"))
    got.backward()
    kernels.check_error()

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm()).item()

    assert abs(got.item() - want.item()) < 1e-3 * abs(want.item()), (got.item(), want.item())
    assert rel(h2.grad, h1.grad) < 1e-2
    lo, hi = rank * V // world, (rank + 1) * V // world
    assert rel(w2.grad[lo:hi], w1.grad[lo:hi]) < 1e-2
    assert w2.grad[:lo].abs().sum() == 0 and w2.grad[hi:].abs().sum() == 0
    del mesh

    cfg = _trainer_cfg({"dp": 1, "tp": world}, "t_lp", 4, graph=False)
    cfg["tp"] = {"loss_parallel": True}
    tr = Trainer(cfg, rank, rank, world, benchmark=True)
    assert tr.model.vocab_parallel is not None and tr.model.impl != "torch"
    hist = tr.train_n_step_test(6)
    tr.check_device_errors()
    if rank == 0:
        torch.save(hist, out)


def test_loss_parallel_on_engine(tmp_path):
    run_on_gpus(_loss_parallel, 2, str(tmp_path), str(tmp_path / "lp.pt"), timeout_s=240)
    run_on_gpus(_trainer_vs_single_cfg, 1, str(tmp_path), str(tmp_path / "one.pt"), timeout_s=240)
    lp, one = torch.load(tmp_path / "lp.pt"), torch.load(tmp_path / "one.pt")
    for x, y in zip(lp, one):
        assert abs(x["loss"] - y["loss"]) < 5e-3 * abs(y["loss"]), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 3e-2 * abs(y["grad_norm"]), (x, y)


def _trainer_pp(rank, world, home, out):
    """Pipeline parallelism through the Trainer on GPUs (mesh {dp: 1, pp: world}): stages of PyTorch blocks under
    autocast, activations and their gradients over library p2p, two micro-batches per step through 1F1B."""
    import os

    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    cfg = _trainer_cfg({"dp": 1, "pp": world}, "t_pp", 4, graph=False)
    tr = Trainer(cfg, rank, rank, world, benchmark=True)
    assert type(tr.model).__name__ == "PipelineStage" and tr.microbatches_per_step == 2
    hist = tr.train_n_step_test(6)
    if rank == 0:
        torch.save(hist, out)


def test_trainer_pipeline_on_gpus(tmp_path):
    run_on_gpus(_trainer_pp, 2, str(tmp_path), str(tmp_path / "pp.pt"), timeout_s=240)
    run_on_gpus(_trainer_vs_single_cfg, 1, str(tmp_path), str(tmp_path / "one.pt"), timeout_s=240)
    pp, one = torch.load(tmp_path / "pp.pt"), torch.load(tmp_path / "one.pt")
    for x, y in zip(pp, one):
        assert abs(x["loss"] - y["loss"]) < 5e-3 * abs(y["loss"]), (x, y)
        assert abs(x["grad_norm"] - y["grad_norm"]) < 3e-2 * abs(y["grad_norm"]), (x, y)


def _trainer_vs_single_cfg(rank, world, home, out):
    import os

    os.environ["TORCHURE_B200_HOME"] = home
    from torchure_b200.train.trainer import Trainer

    tr = Trainer(_trainer_cfg({"dp": 1}, "t_tp_ref", 4, graph=False), rank, rank, world, benchmark=True)
    hist = tr.train_n_step_test(6)
    if rank == 0:
        torch.save(hist, out)


def _collective_stress(rank, world):
    """Race detection without a sanitizer: many collectives of random kind, size (odd sizes included), dtype and
    reduction, issued in a random order that is the same on every rank and alternating between two streams (ordered
    by events, as training orders its communication and compute streams), each checked against its closed form.
    The self-resetting flags must never let a late rank see an early rank's next handshake; the launchers run with
    their debug range checks on."""
    import random

    from torchure_b200.core import collective as C
    from torchure_b200.core.mesh import Mesh

    mesh = Mesh({"dp": world})
    comm = C.enable_sm100(mesh, "dp", 32 << 20)
    rng = random.Random(1234)
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    prev = torch.cuda.Event()
    prev.record()
    checks = []
    tri = world * (world + 1) / 2
    for it in range(150):
        kind = rng.choice(["all_reduce", "all_gather", "reduce_scatter", "all_to_all", "broadcast"])
        dtype = rng.choice([torch.float32, torch.bfloat16])
        n = rng.choice([1, 3, 17, 1000, 4097, 65536, 300_001, 1 << 20])
        st = streams[it % 2] if rng.random() < 0.7 else streams[rng.randrange(2)]
        with torch.cuda.stream(st):
            st.wait_event(prev)
            base = ((torch.arange(n, device="cuda") + it) % 13).float()
            if kind == "all_reduce":
                op = rng.choice(["sum", "avg", "max"])
                x = (base * (rank + 1)).to(dtype)
                C.all_reduce(x, mesh, "dp", op)
                want = base * {"sum": tri, "avg": tri / world, "max": world}[op]
                checks.append((kind, it, x.float(), want.to(dtype).float() if op == "max" else want, 2e-2 if dtype == torch.bfloat16 else 1e-5))
            elif kind == "all_gather":
                x = (base + rank).to(dtype)
                g = C.all_gather(x, mesh, "dp", 0)
                want = torch.cat([(base + r).to(dtype) for r in range(world)]).float()
                checks.append((kind, it, g.float(), want, 0.0))
            elif kind == "reduce_scatter":
                full = ((torch.arange(n * world, device="cuda") + it) % 13).float()
                x = (full * (rank + 1)).to(dtype)
                rs = C.reduce_scatter(x, mesh, "dp", "sum")
                checks.append((kind, it, rs.float(), full[rank * n:(rank + 1) * n] * tri, 2e-2 if dtype == torch.bfloat16 else 1e-5))
            elif kind == "all_to_all":
                m = max(1, n // world)
                x = torch.stack([torch.full((m,), rank * 100.0 + j, device="cuda") for j in range(world)]).to(dtype)
                a = C.all_to_all(x, mesh, "dp", 0, 0)
                want = torch.stack([torch.full((m,), s * 100.0 + rank, device="cuda") for s in range(world)]).to(dtype).float()
                checks.append((kind, it, a.float(), want, 0.0))
            else:
                src = rng.randrange(world)
                x = torch.full((n,), float(rank), device="cuda", dtype=dtype)
                C.broadcast(x, mesh, "dp", src=src)
                checks.append((kind, it, x.float(), torch.full((n,), float(src), device="cuda"), 0.0))
            prev = torch.cuda.Event()
            prev.record(st)
    torch.cuda.synchronize()
    for kind, it, got, want, tol in checks:
        if tol == 0.0:
            assert torch.equal(got, want), (kind, it)
        else:
            torch.testing.assert_close(got, want, rtol=tol, atol=tol * float(want.abs().max().item() + 1), msg=lambda m: f"{kind} #{it}: {m}")
    comm.check()


def test_collectives_random_order_stress():
    run_on_gpus(_collective_stress, _world(), env={"TORCHURE_B200_DEBUG": "1"})
