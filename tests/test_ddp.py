"""DDP on gloo ranks: replication, gradient parity with one process, no_sync accumulation.

Coverage follows the reference's ``tests/data_parallel.py`` (tiny real Qwen3 so the tied embedding,
which receives two gradient contributions, is exercised; two cycles to catch re-arm bugs; swept over
bucket caps 25 MB / 8 KB / 0).
"""

import pytest
import torch

from tests.dist_utils import run_distributed
from tests.tiny import TINY

SEQ = 16


def _model(seed):
    from torchure_b200.models import Qwen3

    torch.manual_seed(seed)
    m = Qwen3(**TINY)
    m.init_weights()
    return m


def _loss(model, ids):
    from torchure_b200.objectives import ARObjective

    return ARObjective(fused_linear_ce=True, ce_chunk_size=8).compute_loss(model, {"input_ids": ids, "labels": ids})


def _batch(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, TINY["vocab_size"], (n, SEQ), generator=g)


def _replicate(rank, world, bucket_mb):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.ddp import DDP

    mesh = Mesh({"dp": world})
    model = _model(seed=100 + rank)
    DDP(model, mesh, "dp", bucket_mb)
    ref = _model(seed=100)
    for (n, a), (_, b) in zip(model.state_dict().items(), ref.state_dict().items()):
        assert torch.equal(a, b), n


def _grad_parity(rank, world, bucket_mb):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.ddp import DDP

    mesh = Mesh({"dp": world})
    model = _model(seed=5)
    ddp = DDP(model, mesh, "dp", bucket_mb)
    single = _model(seed=5)
    for cycle in range(2):
        ids = _batch(world, seed=cycle)
        model.zero_grad()
        _loss(model, ids[rank:rank + 1]).backward()
        ddp.sync()
        single.zero_grad()
        _loss(single, ids).backward()
        for (n, p), (_, q) in zip(model.named_parameters(), single.named_parameters()):
            torch.testing.assert_close(p.grad, q.grad, rtol=1e-4, atol=1e-6, msg=lambda m: f"{n} cycle {cycle}: {m}")


def _accumulation(rank, world, bucket_mb):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.ddp import DDP

    K = 3
    mesh = Mesh({"dp": world})
    model = _model(seed=9)
    ddp = DDP(model, mesh, "dp", bucket_mb)
    single = _model(seed=9)
    for cycle in range(2):
        ids = _batch(world * K, seed=10 + cycle).view(K, world, SEQ)
        model.zero_grad()
        for k in range(K):
            ddp.requires_sync = k == K - 1
            (_loss(model, ids[k, rank:rank + 1]) / K).backward()
            if k < K - 1:
                assert not ddp._works, "nothing may launch while requires_sync is False"
        ddp.sync()
        single.zero_grad()
        for k in range(K):
            (_loss(single, ids[k]) / K).backward()
        for (n, p), (_, q) in zip(model.named_parameters(), single.named_parameters()):
            torch.testing.assert_close(p.grad, q.grad, rtol=1e-4, atol=1e-6, msg=lambda m: f"{n}: {m}")


def _missed_sync(rank, world):
    from torchure_b200.core.mesh import Mesh
    from torchure_b200.parallel.ddp import DDP

    mesh = Mesh({"dp": world})
    model = _model(seed=1)
    ddp = DDP(model, mesh, "dp", 25)
    ddp.requires_sync = False
    _loss(model, _batch(1, 0)).backward()
    with pytest.raises(AssertionError):
        ddp.sync()


@pytest.mark.parametrize("bucket_mb", [25, 0.008, 0])
def test_replicate(bucket_mb):
    run_distributed(_replicate, 2, bucket_mb)


@pytest.mark.parametrize("bucket_mb", [25, 0.008, 0])
def test_grad_parity(bucket_mb):
    run_distributed(_grad_parity, 2, bucket_mb)


def test_grad_parity_world4():
    run_distributed(_grad_parity, 4, 0.008)


@pytest.mark.parametrize("bucket_mb", [25, 0.008])
def test_accumulation(bucket_mb):
    run_distributed(_accumulation, 2, bucket_mb)


def test_sync_catches_unlaunched_buckets():
    run_distributed(_missed_sync, 2)


def test_bucket_planner():
    from torchure_b200.models import Qwen3
    from torchure_b200.parallel.ddp import plan_buckets

    with torch.device("meta"):
        m = Qwen3(num_layers=28, num_heads=16, num_kv_heads=8, emb_dim=1024, head_dim=128, vocab_size=151936,
                  ffn_dim=3072)
    params = list(m.parameters())[::-1]
    assert len(params) == 310
    greedy = plan_buckets(params, 25 << 20, merge_small=False)
    assert len(greedy) == 71 and len(greedy[-1]) == 1 and greedy[-1][0].shape == (151936, 1024)
    merged = plan_buckets(params, 25 << 20)
    assert sum(len(b) for b in merged) == 310
    assert merged[-1][-1].shape == (151936, 1024)
    with torch.device("meta"):
        m4 = Qwen3(num_layers=36, num_heads=32, num_kv_heads=8, emb_dim=2560, head_dim=128, vocab_size=151936,
                   ffn_dim=9728)
    p4 = list(m4.parameters())[::-1]
    g4 = plan_buckets(p4, 25 << 20, merge_small=False)
    b4 = plan_buckets(p4, 25 << 20)
    assert len(g4) == 254
    assert len(b4) < len(g4)
    tiny = [b for b in b4 if sum(p.numel() * 4 for p in b) < (1 << 20)]
    assert not tiny, "no bucket under 1 MiB may remain"
