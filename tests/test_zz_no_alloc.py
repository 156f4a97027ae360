"""Allocation-free attention backward, called through its exported C symbol.

The entry point exists for callers that may not touch the device allocator when they need this gradient (graph
replay inside another runtime, fixed-memory serving loops, plugins without an allocator of their own).  It must
give what the regular, allocating entry point gives, call after call, and it must say no to problems larger than
its built-in scratch.  Collected last on purpose: a failure here cannot hide any other test from an -x run.
"""

import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import torchure_b200

    path = os.path.join(os.path.dirname(torchure_b200.__file__), "_C.so")
    lib = ctypes.CDLL(path)
    fn = lib.tb_attn_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 4 + [ctypes.c_void_p, ctypes.c_void_p]
    return fn


def _case(B, S, Hq, Hkv, seed):
    from torchure_b200 import ops

    hd = 128
    torch.manual_seed(seed)
    qk = torch.randn(B * S, (Hq + Hkv) * hd, device="cuda").bfloat16()
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * hd, device="cuda").bfloat16()
    o = torch.empty(B * S, Hq * hd, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    ops.ext().attn_fwd(qk, qkv, o, lse, B, S, Hq, Hkv)
    d_o = torch.randn(B * S, Hq * hd, device="cuda").bfloat16()
    return qk, qkv, o, lse, d_o


def relerr(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def test_no_alloc_entry_matches_regular_entry_twice():
    from torchure_b200 import ops

    fn = _lib()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # two calls in a row on different problems: the second must not be disturbed by what the first left in the scratch
    for B, S, Hq, Hkv, seed in [(2, 512, 4, 2, 0), (1, 1024, 8, 2, 1)]:
        qk, qkv, o, lse, d_o = _case(B, S, Hq, Hkv, seed)
        want = torch.zeros(B * S, (Hq + 2 * Hkv) * 128, dtype=torch.bfloat16, device="cuda")
        ops.ext().attn_bwd(d_o, qk, qkv, o, lse, want, B, S, Hq, Hkv)
        got = torch.zeros_like(want)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(d_o.data_ptr(), qk.data_ptr(), qkv.data_ptr(), o.data_ptr(), lse.data_ptr(), got.data_ptr(), B, S, Hq, Hkv,
                status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before, "the entry point must not go through the allocator"
        assert int(status.item()) == 0
        # same kernels, same launch shapes, no atomics: the two entry points must agree bit for bit
        assert torch.equal(got, want), relerr(got, want)


def test_no_alloc_entry_rejects_oversized_problem():
    fn = _lib()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    dummy = torch.zeros(16, device="cuda")
    p = dummy.data_ptr()
    # 8 * 64 * 2048 rows is twice the built-in scratch: refused before anything is launched
    rc = fn(p, p, p, p, p, p, 8, 2048, 64, 8, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -30
    # an odd number of query heads per KV head is refused like the forward pass refuses it
    assert fn(p, p, p, p, p, p, 1, 128, 3, 1, status.data_ptr(), torch.cuda.current_stream().cuda_stream) == -2
