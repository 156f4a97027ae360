"""FSDP/HSDP, tensor + sequence parallel, vocab-parallel CE, Ulysses, ring attention, expert parallel, pipeline and
placement redistribution: each against a single-process computation, on gloo ranks."""

import pytest
import torch
import torch.nn.functional as F

from tests.dist_utils import run_distributed
from tests.tiny import TINY

CFG = dict(TINY, num_heads=4, num_kv_heads=2, emb_dim=32, head_dim=8)


def _model(seed=0, cfg=CFG):
    from torchure_b200.models import Qwen3

    torch.manual_seed(seed)
    m = Qwen3(**cfg, impl="torch")
    m.init_weights()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    return m


def _loss(m, ids):
    logits = m(ids)
    return F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), ids[:, 1:].reshape(-1))


def _fsdp(rank, world, hsdp):
    from torchure_b200.core.grad_helper import clip_grad_norm
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.fsdp import FSDP

    if hsdp:
        mesh = Mesh({"dp_replicate": 2, "dp_shard": world // 2})
        mesh.flatten(("dp_replicate", "dp_shard"), "dp")
        rep = "dp_replicate"
    else:
        mesh, rep = Mesh({"dp_shard": world}), None
    model, single = _model(1 + rank), _model(1)
    fsdp = FSDP(model, mesh, "dp_shard", rep)
    opt = torch.optim.AdamW(fsdp.parameters(), lr=1e-2)
    ref_opt = torch.optim.AdamW(single.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(0)
    for step in range(2):
        ids = torch.randint(0, CFG["vocab_size"], (world, 2, 16), generator=g)
        _loss(model, ids[rank]).backward()
        norm = clip_grad_norm(fsdp.parameters(), mesh, 1.0, shard_dims=("dp_shard",))
        opt.step()
        opt.zero_grad()
        sum(_loss(single, ids[r]) for r in range(world)).div(world).backward()
        ref_norm = torch.nn.utils.clip_grad_norm_(single.parameters(), 1.0)
        ref_opt.step()
        ref_opt.zero_grad()
        torch.testing.assert_close(norm, ref_norm, rtol=1e-4, atol=1e-6)
    full = fsdp.full_state_dict()
    for k, v in single.state_dict().items():
        torch.testing.assert_close(full[k], v, rtol=2e-3, atol=3e-5, msg=lambda m: f"{k}: {m}")
    # shard checkpoints round-trip
    sd = {k: v.clone() for k, v in fsdp.shard_state_dict().items()}
    fsdp.load_full_state_dict(single.state_dict())
    fsdp.load_shard_state_dict(sd)
    assert all(p.data.numel() == 0 for u in fsdp.units for p in u.params), "units must be resharded between steps"


def test_fsdp_matches_single_process():
    run_distributed(_fsdp, 2, False, timeout_s=120)


def test_hsdp_matches_single_process():
    run_distributed(_fsdp, 4, True, timeout_s=120)


def _tp(rank, world):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.tensor_parallel import parallelize_model, vocab_parallel_cross_entropy

    mesh = Mesh({"tp": world})
    single = _model(3)
    model = _model(3)
    parallelize_model(model, mesh, "tp")
    ids = torch.randint(0, CFG["vocab_size"], (2, 16), generator=torch.Generator().manual_seed(0))
    out, ref = model(ids), single(ids)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
    out.float().pow(2).mean().backward()
    ref.float().pow(2).mean().backward()
    torch.testing.assert_close(model.norm.weight.grad, single.norm.weight.grad, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(model.token_emb.weight.grad, single.token_emb.weight.grad, rtol=1e-4, atol=1e-6)
    per = single.blocks[0].gqa.q_proj.weight.shape[0] // world
    torch.testing.assert_close(model.blocks[0].gqa.q_proj.weight.grad,
                               single.blocks[0].gqa.q_proj.weight.grad[rank * per:(rank + 1) * per], rtol=1e-4, atol=1e-6)
    perc = single.blocks[1].ffn.down_proj.weight.shape[1] // world
    torch.testing.assert_close(model.blocks[1].ffn.down_proj.weight.grad,
                               single.blocks[1].ffn.down_proj.weight.grad[:, rank * perc:(rank + 1) * perc],
                               rtol=1e-4, atol=1e-6)
    # loss-parallel CE on vocabulary shards
    V = 64
    logits = torch.randn(10, V, generator=torch.Generator().manual_seed(1)).requires_grad_()
    labels = torch.randint(0, V, (10,), generator=torch.Generator().manual_seed(2))
    labels[3] = -100
    local = logits.detach()[:, rank * V // world:(rank + 1) * V // world].clone().requires_grad_()
    loss = vocab_parallel_cross_entropy(local, labels, mesh, "tp")
    loss.backward()
    want = F.cross_entropy(logits, labels, ignore_index=-100)
    want.backward()
    torch.testing.assert_close(loss, want.detach(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(local.grad, logits.grad[:, rank * V // world:(rank + 1) * V // world], rtol=1e-5, atol=1e-7)
    # the same inside the chunked fused linear + CE: every rank computes its V / tp rows of the head, two small
    # all-reduces per chunk; loss and dL/dhidden complete everywhere, dL/dweight complete in the rank's rows
    from torchure_b200.loss import fused_linear_cross_entropy

    g = torch.Generator().manual_seed(5)
    h = torch.randn(37, 16, generator=g)
    w = torch.randn(V, 16, generator=g) * 0.3
    y = torch.randint(0, V, (37,), generator=g)
    y[::5] = -100
    h1, w1 = h.clone().requires_grad_(), w.clone().requires_grad_()
    want = fused_linear_cross_entropy(h1, w1, y, -100, 8)
    want.backward()
    h2, w2 = h.clone().requires_grad_(), w.clone().requires_grad_()
    got = fused_linear_cross_entropy(h2, w2, y, -100, 8, vocab_parallel=(mesh, "tp"))
    got.backward()
    torch.testing.assert_close(got, want.detach(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(h2.grad, h1.grad, rtol=1e-5, atol=1e-7)
    lo, hi = rank * V // world, (rank + 1) * V // world
    torch.testing.assert_close(w2.grad[lo:hi], w1.grad[lo:hi], rtol=1e-5, atol=1e-7)
    assert w2.grad[:lo].abs().sum() == 0 and w2.grad[hi:].abs().sum() == 0


def test_tensor_parallel_and_vocab_parallel_ce():
    run_distributed(_tp, 2, timeout_s=120)


def _sp(rank, world):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear

    mesh = Mesh({"tp": world})
    torch.manual_seed(0)
    up, down = torch.nn.Linear(16, 32, bias=False), torch.nn.Linear(32, 16, bias=False)
    x = torch.randn(2, 8, 16)
    ref_in = x.clone().requires_grad_()
    ref = down(F.silu(up(ref_in)))
    ref.sum().backward()
    col, row = ColumnParallelLinear(up, mesh, "tp", True), RowParallelLinear(down, mesh, "tp", True)
    xs = x.chunk(world, dim=1)[rank].clone().requires_grad_()
    out = row(F.silu(col(xs)))
    torch.testing.assert_close(out, ref.detach().chunk(world, dim=1)[rank], rtol=1e-5, atol=1e-6)
    out.sum().backward()
    torch.testing.assert_close(xs.grad, ref_in.grad.chunk(world, dim=1)[rank], rtol=1e-5, atol=1e-6)


def test_sequence_parallel_linear_pair():
    run_distributed(_sp, 2, timeout_s=120)


def _attn_full(q, k, v):
    rep = q.shape[1] // k.shape[1]
    return F.scaled_dot_product_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1), is_causal=True)


def _ring(rank, world):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.context_parallel import ring_attention, zigzag_positions, zigzag_split

    mesh = Mesh({"cp": world})
    g = torch.Generator().manual_seed(0)
    B, Hq, Hkv, S, d = 2, 4, 2, 8 * world, 8
    q, k, v = (torch.randn(B, h, S, d, generator=g) for h in (Hq, Hkv, Hkv))
    do = torch.randn(B, Hq, S, d, generator=g)
    qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
    ref = _attn_full(qf, kf, vf)
    ref.backward(do)
    ql, kl, vl = (zigzag_split(t, world, rank, 2).clone().requires_grad_() for t in (q, k, v))
    out = ring_attention(ql, kl, vl, mesh, "cp")
    torch.testing.assert_close(out, zigzag_split(ref.detach(), world, rank, 2), rtol=1e-4, atol=1e-5)
    out.backward(zigzag_split(do, world, rank, 2))
    for got, want in ((ql.grad, qf.grad), (kl.grad, kf.grad), (vl.grad, vf.grad)):
        torch.testing.assert_close(got, zigzag_split(want, world, rank, 2), rtol=1e-4, atol=1e-5)
    pos = zigzag_positions(S, world, rank)
    assert pos[0].item() == rank * (S // (2 * world)) and pos[-1].item() == (2 * world - rank) * (S // (2 * world)) - 1


@pytest.mark.parametrize("world", [2, 4])
def test_ring_attention_zigzag(world):
    run_distributed(_ring, world, timeout_s=120)


def _ulysses(rank, world):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.ulysses import ulysses_attention

    mesh = Mesh({"sp": world})
    g = torch.Generator().manual_seed(0)
    B, Hq, Hkv, S, d = 2, 4, 2, 16, 8
    q, k, v = (torch.randn(B, S, h, d, generator=g) for h in (Hq, Hkv, Hkv))
    qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
    attn = lambda a, b, c: _attn_full(a.transpose(1, 2), b.transpose(1, 2), c.transpose(1, 2)).transpose(1, 2)
    ref = attn(qf, kf, vf)
    ref.sum().backward()
    ql, kl, vl = (t.chunk(world, dim=1)[rank].clone().requires_grad_() for t in (q, k, v))
    out = ulysses_attention(ql, kl, vl, mesh, "sp", attn)
    torch.testing.assert_close(out, ref.detach().chunk(world, dim=1)[rank], rtol=1e-4, atol=1e-5)
    out.sum().backward()
    torch.testing.assert_close(ql.grad, qf.grad.chunk(world, dim=1)[rank], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(kl.grad, kf.grad.chunk(world, dim=1)[rank], rtol=1e-4, atol=1e-5)


def test_ulysses_attention():
    run_distributed(_ulysses, 2, timeout_s=120)


def _moe(rank, world):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.expert_parallel import MoELayer

    mesh = Mesh({"ep": world})
    torch.manual_seed(0)
    full = MoELayer(16, 32, num_experts=4, top_k=2, capacity_factor=8.0)
    torch.manual_seed(0)
    ep = MoELayer(16, 32, num_experts=4, top_k=2, capacity_factor=8.0, mesh=mesh, dim="ep")
    ep.router.load_state_dict(full.router.state_dict())
    ep.load_full_experts(full.w_gate.detach(), full.w_up.detach(), full.w_down.detach())
    g = torch.Generator().manual_seed(1)
    xs = [torch.randn(6, 16, generator=g) for _ in range(world)]
    x = xs[rank].clone().requires_grad_()
    out = ep(x)
    xr = xs[rank].clone().requires_grad_()
    ref = full(xr)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
    out.sum().backward()
    ref.sum().backward()
    torch.testing.assert_close(x.grad, xr.grad, rtol=1e-4, atol=1e-5)


def test_expert_parallel_moe():
    run_distributed(_moe, 2, timeout_s=120)


def _cp_autocast(rank, world):
    """Context parallelism on the module path with mixed precision (CPU autocast stands in for the GPU's): bf16
    q / k / v through the PyTorch ring and through Ulysses, loss (averaged over the axis) against the fp32
    single-process value."""
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.models import Qwen3
    from torchure_b200.objectives import ARObjective

    mesh = Mesh({"cp": world})
    torch.manual_seed(0)
    m = Qwen3(**dict(CFG, num_layers=2), impl="torch")
    m.init_weights()
    ids = torch.randint(0, CFG["vocab_size"], (2, 64), generator=torch.Generator().manual_seed(1))
    obj = ARObjective(fused_linear_ce=True, ce_chunk_size=32)
    want = obj.compute_loss(m, {"input_ids": ids, "labels": ids}).item()
    for kind in ("ring", "ulysses"):
        m.cp, m.cp_kind = (mesh, "cp"), kind
        with torch.autocast("cpu", dtype=torch.bfloat16):
            loss = obj.compute_loss(m, {"input_ids": ids, "labels": ids})
        loss.backward()
        total = loss.detach().clone()
        torch.distributed.all_reduce(total)
        assert abs(total.item() / world - want) < 5e-3 * abs(want), (kind, total.item() / world, want)
        assert all(torch.isfinite(p.grad).all() for p in m.parameters())
        m.zero_grad()


def test_context_parallel_module_path_mixed_precision():
    run_distributed(_cp_autocast, 2, timeout_s=120)


def test_moe_load_balancing_term():
    """E * sum_e share_e * mean-probability_e: exactly 1 for a router that is indifferent, larger for one that
    over-subscribes an expert, differentiable through the router's probabilities; the model averages it over its
    layers and the objective adds `aux_loss_coef` times it."""
    from torchure_b200.models import build_model
    from torchure_b200.objectives import ARObjective
    from torchure_b200.parallel.expert_parallel import MoELayer

    torch.manual_seed(0)
    layer = MoELayer(16, 32, num_experts=4, top_k=2)
    x = torch.randn(64, 16)
    with torch.no_grad():
        layer.router.weight.zero_()
    layer(x)
    torch.testing.assert_close(layer.aux_loss, torch.tensor(1.0))
    with torch.no_grad():
        layer.router.weight[0] = 0.5 * x.mean(0).sign()      # favours expert 0 for most tokens
        layer.router.weight[0] += 0.3
    layer(x + 1.0)
    assert layer.aux_loss.item() > 1.05
    layer.aux_loss.backward()
    assert layer.router.weight.grad.abs().sum() > 0
    cfg = dict(CFG, num_layers=2, num_experts=4, top_k=2, moe_ffn_dim=32, aux_loss_coef=0.5)
    model = build_model("qwen3_moe", cfg)
    model.init_weights()
    ids = torch.randint(0, CFG["vocab_size"], (2, 16), generator=torch.Generator().manual_seed(0))
    obj = ARObjective(fused_linear_ce=True, ce_chunk_size=16)
    with_aux = obj.compute_loss(model, {"input_ids": ids, "labels": ids})
    aux = model.aux_loss().detach()
    model.aux_loss_coef = 0.0
    plain = obj.compute_loss(model, {"input_ids": ids, "labels": ids})
    torch.testing.assert_close(with_aux.detach(), plain.detach() + 0.5 * aux, rtol=1e-5, atol=1e-6)


def _moe_autocast(rank, world):
    """The dtype flow of a mixed-precision step (bf16 expert GEMMs and token exchange inside an fp32 residual stream),
    exercised with CPU autocast: the layer must run, return the stream's dtype and stay close to its fp32 result."""
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.expert_parallel import MoELayer

    mesh = Mesh({"ep": world})
    torch.manual_seed(0)
    layer = MoELayer(16, 32, num_experts=4, top_k=2, capacity_factor=8.0)
    layer.shard_(mesh, "ep")
    x = torch.randn(2, 6, 16, generator=torch.Generator().manual_seed(rank)).requires_grad_()
    want = layer(x)
    with torch.autocast("cpu", dtype=torch.bfloat16):
        got = layer(x)
    assert got.dtype == torch.float32
    torch.testing.assert_close(got, want, rtol=5e-2, atol=5e-3)
    got.sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()


def test_expert_parallel_moe_mixed_precision():
    run_distributed(_moe_autocast, 2, timeout_s=120)


def _pp(rank, world, schedule):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.pipeline import PipelineStage, run_schedule, split_layers

    assert [list(r) for r in split_layers(5, 2)] == [[0, 1, 2], [3, 4]]
    mesh = Mesh({"pp": world})
    cfg = dict(CFG, num_layers=4, tie_embeddings=False)
    model, single = _model(5, cfg), _model(5, cfg)
    stage = PipelineStage(model, mesh, "pp")
    g = torch.Generator().manual_seed(0)
    micro = [(torch.randint(0, cfg["vocab_size"], (2, 8), generator=g),) * 2 for _ in range(4)]
    loss_fn = lambda logits, ids: F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))
    loss = run_schedule(stage, micro, loss_fn, schedule)
    ref = sum(loss_fn(single(ids), ids) for ids, _ in micro) / len(micro)
    ref.backward()
    if stage.last:
        torch.testing.assert_close(loss, ref.detach(), rtol=1e-5, atol=1e-6)
    names = dict(single.named_parameters())
    for n, p in model.named_parameters():
        if p.grad is not None:
            torch.testing.assert_close(p.grad, names[n].grad, rtol=1e-4, atol=1e-6, msg=lambda m: f"{n}: {m}")
    owned = sum(1 for p in stage.parameters() if p.grad is not None)
    assert owned > 0


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
def test_pipeline_schedules(schedule):
    run_distributed(_pp, 2, schedule, timeout_s=120)


def _placement(rank, world):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.placement import Partial, Replicate, Shard, ShardedTensor

    mesh = Mesh({"tp": world})
    full = torch.arange(4 * world * 6, dtype=torch.float32).view(2 * world, 2, 6)
    s0 = ShardedTensor.from_full(full, mesh, "tp", Shard(0))
    assert torch.equal(s0.full(), full)
    s2 = s0.redistribute(Shard(2))
    assert s2.local.shape == (2 * world, 2, 6 // world) and torch.equal(s2.full(), full)
    assert torch.equal(ShardedTensor(full.clone(), mesh, "tp", Partial()).full(), full * world)
    ps = ShardedTensor(full.clone(), mesh, "tp", Partial()).redistribute(Shard(0))
    assert torch.equal(ps.local, full.chunk(world, 0)[rank] * world)
    assert torch.equal(ShardedTensor.from_full(full, mesh, "tp", Replicate()).redistribute(Shard(1)).full(), full)


def test_placement_redistribute():
    run_distributed(_placement, 2, timeout_s=120)
