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
                                              (1, 512, 2, 1, 4.0), (2, 2048, 4, 2, 0.3)])
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


@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 2, 1), (1, 256, 2, 1), (2, 512, 4, 2), (1, 1024, 8, 2)])
def test_attn_bwd(B, S, Hq, Hkv):
    from torchure_b200 import ops
    from torchure_b200.ops import kernels, oracle

    hd = 128
    qk, qkv = _inputs(B, S, Hq, Hkv, seed=1)
    o = torch.empty(B * S, Hq * hd, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    ops.ext().attn_fwd(qk, qkv, o, lse, B, S, Hq, Hkv)
    d_o = torch.randn(B * S, Hq * hd, device="cuda").bfloat16()
    dqkv = torch.zeros(B * S, (Hq + 2 * Hkv) * hd, dtype=torch.bfloat16, device="cuda")
    ops.ext().attn_bwd(d_o, qk, qkv, o, lse, dqkv, B, S, Hq, Hkv)
    kernels.check_error()
    q = qk[:, :Hq * hd].float().view(B, S, Hq, hd).requires_grad_()
    k = qk[:, Hq * hd:].float().view(B, S, Hkv, hd).requires_grad_()
    v = qkv[:, (Hq + Hkv) * hd:].float().reshape(B, S, Hkv, hd).requires_grad_()
    ro, _ = oracle.attention(q, k, v)
    ro.backward(d_o.float().view(B, S, Hq, hd))
    dq = dqkv[:, :Hq * hd].view(B, S, Hq, hd)
    dk = dqkv[:, Hq * hd:(Hq + Hkv) * hd].view(B, S, Hkv, hd)
    dv = dqkv[:, (Hq + Hkv) * hd:].view(B, S, Hkv, hd)
    assert relerr(dv, v.grad) < 1.5e-2, ("dv", relerr(dv, v.grad))
    assert relerr(dq, q.grad) < 1.5e-2, ("dq", relerr(dq, q.grad))
    assert relerr(dk, k.grad) < 1.5e-2, ("dk", relerr(dk, k.grad))
