"""tcgen05 flash attention against a plain fp32 softmax(QK^T)V."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def relerr(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _inputs(B, S, Hq, Hkv, seed=0, scale=1.0):
    torch.manual_seed(seed)
    hd = 128
    qk = (torch.randn(B * S, (Hq + Hkv) * hd, device="cuda") * scale).bfloat16()
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * hd, device="cuda").bfloat16()
    return qk, qkv


def _oracle(qk, qkv, B, S, Hq, Hkv):
    from torchure_b200.ops import oracle

    hd = 128
    q = qk[:, :Hq * hd].view(B, S, Hq, hd)
    k = qk[:, Hq * hd:].view(B, S, Hkv, hd)
    v = qkv[:, (Hq + Hkv) * hd:].view(B, S, Hkv, hd)
    o, lse = oracle.attention(q, k, v)
    return o.reshape(B * S, Hq * hd), lse


@pytest.mark.parametrize("B,S,Hq,Hkv,scale", [(1, 128, 2, 1, 1.0), (2, 512, 4, 2, 1.0), (1, 1024, 8, 2, 1.0),
                                              (1, 512, 2, 1, 4.0), (2, 2048, 4, 2, 0.3), (1, 4096, 16, 8, 1.0),
                                              (1, 4096, 32, 8, 1.0)])
def test_attn_fwd(B, S, Hq, Hkv, scale):
    from torchure_b200 import ops
    from torchure_b200.ops import kernels

    qk, qkv = _inputs(B, S, Hq, Hkv, scale=scale)
    o = torch.empty(B * S, Hq * 128, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    ops.ext().attn_fwd(qk, qkv, o, lse, B, S, Hq, Hkv)
    kernels.check_error()
    ro, rl = _oracle(qk, qkv, B, S, Hq, Hkv)
    assert relerr(o, ro) < 1e-2, relerr(o, ro)
    torch.testing.assert_close(lse, rl, rtol=2e-3, atol=2e-3)


def _grads_oracle(qk, qkv, d_o, B, S, Hq, Hkv):
    """fp32 reference gradients, one (batch, kv head) group at a time so the S x S scores of long sequences fit."""
    from torchure_b200.ops import oracle

    hd, r = 128, Hq // Hkv
    dq = torch.empty(B, S, Hq, hd, device="cuda")
    dk = torch.empty(B, S, Hkv, hd, device="cuda")
    dv = torch.empty(B, S, Hkv, hd, device="cuda")
    qa = qk[:, :Hq * hd].float().view(B, S, Hq, hd)
    ka = qk[:, Hq * hd:].float().view(B, S, Hkv, hd)
    va = qkv[:, (Hq + Hkv) * hd:].float().reshape(B, S, Hkv, hd)
    ga = d_o.float().view(B, S, Hq, hd)
    for b in range(B):
        for g in range(Hkv):
            q = qa[b:b + 1, :, g * r:(g + 1) * r].clone().requires_grad_()
            k = ka[b:b + 1, :, g:g + 1].clone().requires_grad_()
            v = va[b:b + 1, :, g:g + 1].clone().requires_grad_()
            o, _ = oracle.attention(q, k, v)
            o.backward(ga[b:b + 1, :, g * r:(g + 1) * r])
            dq[b, :, g * r:(g + 1) * r], dk[b, :, g], dv[b, :, g] = q.grad[0], k.grad[0, :, 0], v.grad[0, :, 0]
    return dq, dk, dv


@pytest.mark.parametrize("entry", ["attn_bwd_fused", "attn_bwd"])
@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 2, 1), (1, 256, 2, 1), (2, 512, 4, 2), (1, 1024, 8, 2), (1, 384, 2, 1),
                                        (1, 4096, 16, 8), (1, 4096, 32, 8)])
def test_attn_bwd(B, S, Hq, Hkv, entry):
    """Both backward implementations (single pass, two kernels) against fp32 autograd of the dense formula, up to
    the benchmark shapes (16/8 and 32/8 heads at 4096 tokens)."""
    from torchure_b200 import ops
    from torchure_b200.ops import kernels

    hd = 128
    qk, qkv = _inputs(B, S, Hq, Hkv, seed=1)
    o = torch.empty(B * S, Hq * hd, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    ops.ext().attn_fwd(qk, qkv, o, lse, B, S, Hq, Hkv)
    d_o = torch.randn(B * S, Hq * hd, device="cuda").bfloat16()
    dqkv = torch.zeros(B * S, (Hq + 2 * Hkv) * hd, dtype=torch.bfloat16, device="cuda")
    getattr(ops.ext(), entry)(d_o, qk, qkv, o, lse, dqkv, B, S, Hq, Hkv)
    kernels.check_error()
    rq, rk, rv = _grads_oracle(qk, qkv, d_o, B, S, Hq, Hkv)
    dq = dqkv[:, :Hq * hd].view(B, S, Hq, hd)
    dk = dqkv[:, Hq * hd:(Hq + Hkv) * hd].view(B, S, Hkv, hd)
    dv = dqkv[:, (Hq + Hkv) * hd:].view(B, S, Hkv, hd)
    assert relerr(dv, rv) < 1.5e-2, ("dv", relerr(dv, rv))
    assert relerr(dq, rq) < 1.5e-2, ("dq", relerr(dq, rq))
    assert relerr(dk, rk) < 1.5e-2, ("dk", relerr(dk, rk))


@pytest.mark.parametrize("B,Sq,Skv,Hq,Hkv,causal", [(2, 512, 512, 4, 2, True), (1, 256, 768, 4, 2, False),
                                                    (2, 384, 384, 8, 2, False)])
def test_flash_attention_block_pairs(B, Sq, Skv, Hq, Hkv, causal):
    """The block-pair entry points (separate q / k / v tensors, optional full visibility, Sq != Skv) through the
    differentiable ``flash_attention`` op, forward and backward, against the dense fp32 formula."""
    from torchure_b200.ops import kernels
    from torchure_b200.ops.attention import flash_attention, pair_supported

    torch.manual_seed(3)
    q = torch.randn(B, Sq, Hq, 128, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, Skv, Hkv, 128, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, Skv, Hkv, 128, device="cuda").bfloat16().requires_grad_()
    assert pair_supported(q, k, v)
    out = flash_attention(q, k, v, causal=causal)
    g = torch.randn_like(out)
    out.backward(g)
    kernels.check_error()
    rep = Hq // Hkv
    qf, kf, vf = (t.detach().float().transpose(1, 2).requires_grad_() for t in (q, k, v))
    s = qf @ kf.repeat_interleave(rep, 1).transpose(-1, -2) / 128 ** 0.5
    if causal:
        s = s.masked_fill(~torch.ones(Sq, Skv, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    ref = torch.softmax(s, -1) @ vf.repeat_interleave(rep, 1)
    ref.backward(g.float().transpose(1, 2))
    assert relerr(out, ref.transpose(1, 2)) < 1e-2
    for name, got, want in (("dq", q.grad, qf.grad), ("dk", k.grad, kf.grad), ("dv", v.grad, vf.grad)):
        assert relerr(got, want.transpose(1, 2)) < 1.5e-2, (name, relerr(got, want.transpose(1, 2)))
