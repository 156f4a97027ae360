"""sm_100a engine against the PyTorch oracle path of the same model (fp32 weights, fp32 math)."""

import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = dict(num_layers=2, num_heads=4, num_kv_heads=2, emb_dim=512, head_dim=128, vocab_size=4096, ffn_dim=1024)


def relerr(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _pair(cfg=CFG, seed=0):
    from torchure_b200.models import Qwen3

    torch.manual_seed(seed)
    fast = Qwen3(**cfg).cuda()
    fast.init_weights()
    # a livelier test than init: non-unit norm gains
    with torch.no_grad():
        for n, p in fast.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    slow = Qwen3(**cfg, impl="torch").cuda()
    slow.load_state_dict(fast.state_dict())
    return fast, slow


@pytest.mark.parametrize("fused_ce", [True, False])
def test_forward_backward_matches_oracle(fused_ce):
    from torchure_b200 import ops
    from torchure_b200.objectives import ARObjective
    from torchure_b200.ops import kernels

    fast, slow = _pair()
    ids = torch.randint(0, CFG["vocab_size"], (2, 256), device="cuda")
    batch = {"input_ids": ids, "labels": ids}
    obj = ARObjective(fused_linear_ce=fused_ce, ce_chunk_size=200)
    before = ops.launches()
    loss = obj.compute_loss(fast, batch)
    loss.backward()
    assert ops.launches() - before > 50, "the sm_100a path must be the one that ran"
    ops.force_fallback(True)
    try:
        ref = ARObjective(fused_linear_ce=False).compute_loss(slow, batch)
        ref.backward()
    finally:
        ops.force_fallback(False)
    kernels.check_error()
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item())), (loss.item(), ref.item())
    for (n, p), (_, q) in zip(fast.named_parameters(), slow.named_parameters()):
        assert p.grad is not None, n
        assert p.grad.dtype == torch.float32 and p.grad.shape == p.shape
        assert relerr(p.grad, q.grad) < 3e-2, (n, relerr(p.grad, q.grad))


def test_hidden_matches_oracle():
    fast, slow = _pair(seed=1)
    ids = torch.randint(0, CFG["vocab_size"], (2, 128), device="cuda")
    with torch.no_grad():
        h = fast(ids, return_final_hidden=True)
        r = slow(ids, return_final_hidden=True)
        assert h.dtype == torch.bfloat16 and h.shape == r.shape
        assert relerr(h, r) < 1e-2
        assert relerr(fast(ids), slow(ids)) < 1e-2


def test_shadow_refresh_after_load_state_dict():
    fast, slow = _pair(seed=2)
    ids = torch.randint(0, CFG["vocab_size"], (1, 128), device="cuda")
    with torch.no_grad():
        a = fast(ids, return_final_hidden=True).clone()
        sd = {k: v * 1.5 if v.dim() == 2 else v for k, v in fast.state_dict().items()}
        fast.load_state_dict(sd)
        slow.load_state_dict(sd)
        b = fast(ids, return_final_hidden=True)
        assert relerr(b, slow(ids, return_final_hidden=True)) < 2e-2
        assert relerr(a, b) > 1e-2


def test_training_steps_track_oracle():
    """3 fused AdamW steps with clipping; shadows are rewritten by the optimizer kernel."""
    from torchure_b200 import ops
    from torchure_b200.core.grad_helper import clip_grad_norm
    from torchure_b200.objectives import ARObjective
    from torchure_b200.optim import build_optimizer

    fast, slow = _pair(seed=3)
    cfg = {"lr": 2e-4, "weight_decay": 0.1, "betas": [0.9, 0.95], "fused": True}
    of, os_ = build_optimizer(fast, "adamw", cfg), build_optimizer(slow, "adamw", dict(cfg, fused=False))
    for p, s in fast.engine().shadow_pairs():
        of.attach_shadow(p, s)
    obj = ARObjective(fused_linear_ce=True, ce_chunk_size=256)

    class M1:
        def size(self, d): return 1
        def coordinate(self, d): return 0
        def get_group(self, d): return None

    losses = []
    for step in range(3):
        ids = torch.randint(0, CFG["vocab_size"], (2, 256), device="cuda", generator=torch.Generator("cuda").manual_seed(step))
        batch = {"input_ids": ids, "labels": ids}
        lf = obj.compute_loss(fast, batch)
        lf.backward()
        clip_grad_norm(list(fast.parameters()), M1(), 1.0)
        of.step(); of.zero_grad()
        ops.force_fallback(True)
        try:
            ls = obj.compute_loss(slow, batch)
            ls.backward()
            clip_grad_norm(list(slow.parameters()), M1(), 1.0)
            os_.step(); os_.zero_grad()
        finally:
            ops.force_fallback(False)
        losses.append((lf.item(), ls.item()))
    for a, b in losses:
        assert abs(a - b) < 5e-3 * max(1.0, abs(b)), losses
    for (n, p), (_, q) in zip(fast.named_parameters(), slow.named_parameters()):
        assert relerr(p, q) < 1e-2, (n, relerr(p, q))


@pytest.mark.parametrize("shape", [(2, 128, 64, 1000, 64), (2, 256, 128, 5000, 512), (2, 1024, 1024, 151936, 1024)])
def test_fused_linear_ce_sm100(shape):
    """loss / dH / dW against hidden @ W^T -> F.cross_entropy in fp32 (tolerances of the reference's own test)."""
    from torchure_b200.loss import fused_linear_cross_entropy

    B, S, D, V, chunk = shape
    torch.manual_seed(0)
    h = torch.randn(B, S, D, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(V, D, device="cuda") * 0.02).requires_grad_()
    y = torch.randint(0, V, (B, S), device="cuda")
    y[torch.rand(B, S, device="cuda") < 0.05] = -100
    loss = fused_linear_cross_entropy(h, w, y, -100, chunk)
    loss.backward()
    h2 = h.detach().float().requires_grad_()
    w2 = w.detach().clone().requires_grad_()
    ref = torch.nn.functional.cross_entropy((h2 @ w2.t()).view(-1, V), y.view(-1), ignore_index=-100)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, ref.item())
    assert relerr(h.grad, h2.grad) < 3e-2
    assert relerr(w.grad, w2.grad) < 3e-2


def test_llama3_runs_on_the_engine_and_matches_oracle():
    """The Llama-3 variant (no QK-norm, theta 5e5, eps 1e-5) on the same kernels, at a head_dim they cover."""
    from torchure_b200 import ops
    from torchure_b200.models import Llama3
    from torchure_b200.objectives import ARObjective
    from torchure_b200.ops import kernels

    cfg = dict(num_layers=2, num_heads=4, num_kv_heads=2, emb_dim=512, vocab_size=4096, ffn_dim=1024)   # head_dim 128
    torch.manual_seed(5)
    fast = Llama3(**cfg).cuda()
    fast.init_weights()
    slow = Llama3(**cfg, impl="torch").cuda()
    slow.load_state_dict(fast.state_dict())
    ids = torch.randint(0, cfg["vocab_size"], (2, 256), device="cuda")
    batch = {"input_ids": ids, "labels": ids}
    before = ops.launches()
    loss = ARObjective(fused_linear_ce=True, ce_chunk_size=256).compute_loss(fast, batch)
    loss.backward()
    assert ops.launches() - before > 40
    ops.force_fallback(True)
    try:
        ref = ARObjective(fused_linear_ce=False).compute_loss(slow, batch)
        ref.backward()
    finally:
        ops.force_fallback(False)
    kernels.check_error()
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item()))
    for (n, p), (_, q) in zip(fast.named_parameters(), slow.named_parameters()):
        assert relerr(p.grad, q.grad) < 3e-2, (n, relerr(p.grad, q.grad))


def test_uncovered_shapes_are_loud():
    """A sequence length the attention kernels do not cover raises; a head_dim they do not cover runs the PyTorch
    path with a warning: never a silent library kernel on the hot path."""
    from torchure_b200.models import Qwen3

    m = Qwen3(**CFG).cuda()
    m.init_weights()
    with pytest.raises(RuntimeError, match="multiples of 128"):
        m(torch.randint(0, CFG["vocab_size"], (1, 100), device="cuda"))
    small = Qwen3(num_layers=1, num_heads=4, num_kv_heads=2, emb_dim=256, head_dim=64, vocab_size=512, ffn_dim=512).cuda()
    small.init_weights()
    with pytest.warns(UserWarning, match="PyTorch path"):
        out = small(torch.randint(0, 512, (1, 100), device="cuda"))
    assert out.shape == (1, 100, 512)
