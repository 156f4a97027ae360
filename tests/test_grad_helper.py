"""Gradient clipping: agreement with torch.nn.utils.clip_grad_norm_, bitwise no-op below the
threshold, direction kept, measure-only, empty grads refused, sharded norm (coverage of the
reference's ``tests/grad_helper.py``)."""

import pytest
import torch

from tests.dist_utils import run_distributed
from tests.tiny import TINY


class OneRankMesh:
    def size(self, dim):
        return 1

    def coordinate(self, dim):
        return 0

    def get_group(self, dim):
        return None


def _model_with_grads(seed=0, scale=1.0):
    from torchure_b200.models import Qwen3

    torch.manual_seed(seed)
    m = Qwen3(**TINY)
    m.init_weights()
    ids = torch.randint(0, TINY["vocab_size"], (2, 16))
    out = m(ids)
    (out.float().pow(2).mean() * scale).backward()
    return m


@pytest.mark.parametrize("max_norm", [0.1, 1.0, 5.0])
def test_matches_torch(max_norm):
    from torchure_b200.core.grad_helper import clip_grad_norm

    a, b = _model_with_grads(3, 50.0), _model_with_grads(3, 50.0)
    ours = clip_grad_norm(list(a.parameters()), OneRankMesh(), max_norm)
    theirs = torch.nn.utils.clip_grad_norm_(b.parameters(), max_norm)
    torch.testing.assert_close(ours, theirs, rtol=1e-5, atol=1e-7)
    for p, q in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(p.grad, q.grad, rtol=1e-5, atol=1e-7)


def test_below_threshold_is_bitwise_noop():
    from torchure_b200.core.grad_helper import clip_grad_norm

    m = _model_with_grads(1, 1e-3)
    before = [p.grad.clone() for p in m.parameters()]
    norm = clip_grad_norm(list(m.parameters()), OneRankMesh(), 1e6)
    assert norm < 1e6
    for p, g in zip(m.parameters(), before):
        assert torch.equal(p.grad, g)


def test_clips_to_max_and_keeps_direction():
    from torchure_b200.core.grad_helper import clip_grad_norm

    m = _model_with_grads(2, 100.0)
    before = torch.cat([p.grad.flatten() for p in m.parameters()])
    pre = clip_grad_norm(list(m.parameters()), OneRankMesh(), 0.5)
    after = torch.cat([p.grad.flatten() for p in m.parameters()])
    torch.testing.assert_close(pre, before.norm())
    torch.testing.assert_close(after.norm(), torch.tensor(0.5), rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(after / after.norm(), before / before.norm())


def test_none_measures_only():
    from torchure_b200.core.grad_helper import clip_grad_norm

    m = _model_with_grads(4, 100.0)
    before = [p.grad.clone() for p in m.parameters()]
    norm = clip_grad_norm(list(m.parameters()), OneRankMesh(), None)
    torch.testing.assert_close(norm, torch.cat([g.flatten() for g in before]).norm())
    for p, g in zip(m.parameters(), before):
        assert torch.equal(p.grad, g)


def test_empty_grads_refused():
    from torchure_b200.core.grad_helper import clip_grad_norm
    from torchure_b200.models import Qwen3

    m = Qwen3(**TINY)
    with pytest.raises(AssertionError):
        clip_grad_norm(list(m.parameters()), OneRankMesh(), 1.0)


def test_coef_variant_leaves_grads():
    from torchure_b200.core.grad_helper import grad_norm_and_coef

    m = _model_with_grads(5, 100.0)
    before = [p.grad.clone() for p in m.parameters()]
    norm, coef = grad_norm_and_coef(list(m.parameters()), OneRankMesh(), 0.5)
    torch.testing.assert_close(coef, 0.5 / (norm + 1e-6))
    for p, g in zip(m.parameters(), before):
        assert torch.equal(p.grad, g)


def _sharded(rank, world):
    from torchure_b200.core.grad_helper import clip_grad_norm
    from torchure_b200.core.mesh import Mesh

    mesh = Mesh({"dp": world})
    full = torch.randn(world * 6, generator=torch.Generator().manual_seed(0)) * 10
    p = torch.nn.Parameter(torch.zeros(6))
    p.grad = full[rank * 6:(rank + 1) * 6].clone()
    norm = clip_grad_norm([p], mesh, 1.0, shard_dims=("dp",))
    torch.testing.assert_close(norm, full.norm())
    torch.testing.assert_close(p.grad, full[rank * 6:(rank + 1) * 6] * (1.0 / (full.norm() + 1e-6)))
    # replicated grads must not be reduced: shard_dims=() keeps the local norm
    q = torch.nn.Parameter(torch.zeros(6))
    q.grad = full[:6].clone()
    norm = clip_grad_norm([q], mesh, None, shard_dims=())
    torch.testing.assert_close(norm, full[:6].norm())


def test_sharded_norm_gloo():
    run_distributed(_sharded, 2)
