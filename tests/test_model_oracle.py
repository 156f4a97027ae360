"""Model, loss and objective against independent oracles: F.cross_entropy for the fused CE, and
(when the reference tree is mounted) the reference's own Qwen3 on CPU fp32 with shared weights."""

import os
import sys

import pytest
import torch
import torch.nn.functional as F

from tests.tiny import PARITY, TINY

# the reference package: an explicit checkout (TORCHURE_REFERENCE_DIR) or the offline install under baseline/_ref
_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("TORCHURE_REFERENCE_DIR") or os.path.join(_HERE, "baseline", "_ref")


@pytest.mark.parametrize("shape", [(2, 128, 64, 1000, 64), (2, 256, 128, 5000, 512), (1, 100, 32, 300, 33)])
def test_fused_linear_ce_vs_cross_entropy(shape):
    from torchure_b200.loss import fused_linear_cross_entropy

    B, S, D, V, chunk = shape
    torch.manual_seed(0)
    h = torch.randn(B, S, D, requires_grad=True)
    w = (torch.randn(V, D) * 0.05).requires_grad_()
    y = torch.randint(0, V, (B, S))
    y[torch.rand(B, S) < 0.1] = -100
    loss = fused_linear_cross_entropy(h, w, y, -100, chunk)
    loss.backward()
    h2, w2 = h.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    ref = F.cross_entropy((h2 @ w2.t()).view(-1, V), y.view(-1), ignore_index=-100)
    ref.backward()
    torch.testing.assert_close(loss, ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(h.grad, h2.grad, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(w.grad, w2.grad, rtol=1e-4, atol=1e-6)
    with pytest.raises(RuntimeError):
        loss.backward()


def test_all_ignored_gives_zero():
    from torchure_b200.loss import fused_linear_cross_entropy

    h = torch.randn(4, 8, requires_grad=True)
    w = torch.randn(10, 8, requires_grad=True)
    loss = fused_linear_cross_entropy(h, w, torch.full((4,), -100), -100, 2)
    loss.backward()
    assert loss.item() == 0.0 and h.grad.abs().sum() == 0


def test_objective_fused_equals_plain():
    from torchure_b200.models import Qwen3
    from torchure_b200.objectives import ARObjective

    torch.manual_seed(0)
    m = Qwen3(**TINY)
    m.init_weights()
    ids = torch.randint(0, TINY["vocab_size"], (3, 16))
    batch = {"input_ids": ids, "labels": ids.clone()}
    a = ARObjective(fused_linear_ce=True, ce_chunk_size=7).compute_loss(m, batch)
    b = ARObjective(fused_linear_ce=False).compute_loss(m, batch)
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


def test_param_order_and_count():
    from torchure_b200.models import Qwen3

    with torch.device("meta"):
        m = Qwen3(num_layers=28, num_heads=16, num_kv_heads=8, emb_dim=1024, head_dim=128, vocab_size=151936)
    assert m.num_params() == 574_029_824  # default ffn 2816
    with torch.device("meta"):
        m = Qwen3(num_layers=28, num_heads=16, num_kv_heads=8, emb_dim=1024, head_dim=128, vocab_size=151936,
                  ffn_dim=3072)
    assert m.num_params() == 596_049_920
    names = [n for n, _ in m.named_parameters()]
    assert names[0] == "token_emb.weight" and names[-1] == "norm.weight" and len(names) == 310
    assert names[1:12] == [f"blocks.0.{s}.weight" for s in (
        "gqa.q_proj", "gqa.k_proj", "gqa.v_proj", "gqa.o_proj", "gqa.q_norm", "gqa.k_norm", "norm1", "norm2",
        "ffn.gate_proj", "ffn.up_proj", "ffn.down_proj")]


def test_init_statistics():
    from torchure_b200.models import Qwen3

    torch.manual_seed(0)
    m = Qwen3(**PARITY)
    m.init_weights()
    L = PARITY["num_layers"]
    assert abs(m.blocks[0].gqa.q_proj.weight.std().item() - 0.02) < 2e-3
    assert abs(m.blocks[0].gqa.o_proj.weight.std().item() - 0.02 * (2 * L) ** -0.5) < 1e-3
    assert torch.equal(m.norm.weight, torch.ones_like(m.norm.weight))
    assert m.lm_head.weight is m.token_emb.weight


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "torchure")), reason="reference package not available")
def test_matches_reference_model_cpu_fp32():
    sys.path.insert(0, REF)
    try:
        from torchure.models.qwen3.qwen3 import Qwen3 as RefQwen3
    finally:
        sys.path.remove(REF)
    from torchure_b200.models import Qwen3

    cfg = dict(TINY)
    torch.manual_seed(0)
    ref = RefQwen3(**cfg)
    ref.init_weights()
    # the reference's norms use eps=None (fp32 machine epsilon)
    ours = Qwen3(**cfg, norm_eps=torch.finfo(torch.float32).eps)
    missing = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    ids = torch.randint(0, cfg["vocab_size"], (2, 16))
    torch.testing.assert_close(ours(ids), ref(ids), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(ours(ids, return_final_hidden=True), ref(ids, return_final_hidden=True),
                               rtol=1e-4, atol=1e-5)
    mask = torch.ones(2, 16, dtype=torch.long)
    mask[0, :5] = 0
    a, b = ours(ids, attention_mask=mask), ref(ids, attention_mask=mask)
    torch.testing.assert_close(a[mask.bool()], b[mask.bool()], rtol=1e-4, atol=1e-5)
    ours(ids).sum().backward()
    ref(ids).sum().backward()
    for (n, p), (_, q) in zip(ours.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p.grad, q.grad, rtol=1e-3, atol=1e-5, msg=lambda m: f"{n}: {m}")
