"""Mesh + collectives on 4 gloo ranks, mesh {"dp": 2, "tp": 2} so every axis is a true subgroup.

Mirrors the coverage of the reference's ``tests/collective.py`` (closed-form expectations from a
per-coordinate pattern, in-place identity, src as a coordinate, gather ordering, the
reduce_scatter/all_gather identity, all_to_all involution, ring hops, async==sync, subgroup
isolation, Mesh.flatten).
"""

import pytest
import torch

from tests.dist_utils import run_distributed

WORLD = 4


def pattern(coord: int, n: int = 8) -> torch.Tensor:
    return torch.arange(n, dtype=torch.float32) * (coord + 1)


def _mesh():
    from torchure_b200.core.mesh import Mesh

    return Mesh({"dp": WORLD // 2, "tp": 2})


def _suite(rank, world):
    from torchure_b200.core import collective as C
    from torchure_b200.core.mesh import Mesh

    mesh = _mesh()
    for dim in ("dp", "tp"):
        g, me = mesh.size(dim), mesh.coordinate(dim)
        tri = g * (g + 1) // 2
        base = torch.arange(8, dtype=torch.float32)
        # all_reduce sum / avg / max, in place
        t = pattern(me)
        out = C.all_reduce(t, mesh, dim, "sum")
        assert out is t
        torch.testing.assert_close(t, base * tri)
        t = pattern(me)
        C.all_reduce(t, mesh, dim, "avg")
        torch.testing.assert_close(t, base * tri / g)
        t = pattern(me)
        C.all_reduce(t, mesh, dim, "max")
        torch.testing.assert_close(t, base * g)
        t = pattern(me)
        C.all_reduce(t, mesh, dim, "min")
        torch.testing.assert_close(t, base)
        # async == sync
        t = pattern(me)
        t2, work = C.all_reduce(t, mesh, dim, "avg", async_op=True)
        work.wait()
        torch.testing.assert_close(t2, base * tri / g)
        # broadcast from coordinate 1 (not a global rank)
        t = pattern(me)
        C.broadcast(t, mesh, dim, src=1)
        torch.testing.assert_close(t, base * 2)
        # all_gather dim 0, dim -1, non-contiguous input, caller buffer
        x = pattern(me).view(2, 4)
        got = C.all_gather(x, mesh, dim, 0)
        want = torch.cat([pattern(c).view(2, 4) for c in range(g)], 0)
        torch.testing.assert_close(got, want)
        got = C.all_gather(x, mesh, dim, -1)
        torch.testing.assert_close(got, torch.cat([pattern(c).view(2, 4) for c in range(g)], -1))
        got = C.all_gather(x.t(), mesh, dim, 0)
        torch.testing.assert_close(got, torch.cat([pattern(c).view(2, 4).t() for c in range(g)], 0))
        buf = torch.empty(2 * g, 4)
        got = C.all_gather(x, mesh, dim, 0, output_tensor=buf)
        assert got.data_ptr() == buf.data_ptr()
        torch.testing.assert_close(buf, want)
        with pytest.raises(AssertionError):
            C.all_gather(x, mesh, dim, 1, output_tensor=torch.empty(2, 4 * g))
        # reduce_scatter sum / avg, indivisible raises
        full = torch.arange(4 * g, dtype=torch.float32) * (me + 1)
        got = C.reduce_scatter(full, mesh, dim, "sum")
        torch.testing.assert_close(got, torch.arange(4 * g, dtype=torch.float32)[me * 4:(me + 1) * 4] * tri)
        got = C.reduce_scatter(full, mesh, dim, "avg")
        torch.testing.assert_close(got, torch.arange(4 * g, dtype=torch.float32)[me * 4:(me + 1) * 4] * tri / g)
        with pytest.raises(AssertionError):
            C.reduce_scatter(torch.zeros(4 * g + 1), mesh, dim)
        # all_gather(reduce_scatter(x)) == all_reduce(x)
        x = torch.randn(4 * g, 3, generator=torch.Generator().manual_seed(rank))
        lhs = C.all_gather(C.reduce_scatter(x.clone(), mesh, dim, "sum"), mesh, dim, 0)
        rhs = C.all_reduce(x.clone(), mesh, dim, "sum")
        torch.testing.assert_close(lhs, rhs)
        # all_to_all: value-encoded (sender*100 + chunk), involution
        x = torch.tensor([[me * 100.0 + j] * 3 for j in range(g)])
        got = C.all_to_all(x, mesh, dim, 0, 0)
        torch.testing.assert_close(got, torch.tensor([[s * 100.0 + me] * 3 for s in range(g)]))
        torch.testing.assert_close(C.all_to_all(got, mesh, dim, 0, 0), x)
        y = torch.arange(2 * g * 3, dtype=torch.float32).view(2 * g, 3) + 1000 * me
        got = C.all_to_all(y, mesh, dim, split_dim=0, concat_dim=1)
        assert got.shape == (2, 3 * g)
        # ring: one hop, g hops home, new tensor
        x = pattern(me)
        r1 = C.ring_send_recv(x, mesh, dim)
        assert r1.data_ptr() != x.data_ptr()
        torch.testing.assert_close(r1, pattern((me - 1) % g))
        cur = x
        for _ in range(g):
            cur = C.ring_send_recv(cur, mesh, dim)
        torch.testing.assert_close(cur, x)
        C.barrier(mesh, dim)
    # subgroup isolation: power-of-two values make the members of a sum identifiable
    t = torch.tensor([float(1 << rank)])
    C.all_reduce(t, mesh, "tp", "sum")
    dp_c = mesh.coordinate("dp")
    assert t.item() == float((1 << (dp_c * 2)) + (1 << (dp_c * 2 + 1)))
    t = torch.tensor([float(1 << rank)])
    C.all_reduce(t, mesh, "dp", "sum")
    tp_c = mesh.coordinate("tp")
    assert t.item() == float(sum(1 << (d * 2 + tp_c) for d in range(2)))
    # flatten
    m3 = Mesh({"dp_replicate": 2, "dp_shard": 2})
    m3.flatten(("dp_replicate", "dp_shard"), "dp")
    assert m3.size("dp") == 4 and m3.coordinate("dp") == rank
    got = C.all_gather(torch.tensor([float(rank)]), m3, "dp", 0)
    torch.testing.assert_close(got, torch.arange(4, dtype=torch.float32))
    with pytest.raises(AssertionError):
        m3.flatten(("dp_shard", "dp_replicate"), "bad")
    with pytest.raises(AssertionError):
        m3.flatten(("dp_replicate",), "dp")
    C.barrier()


def test_collectives_and_mesh_gloo():
    run_distributed(_suite, WORLD)


def _bad_mesh(rank, world):
    from torchure_b200.core.mesh import Mesh

    with pytest.raises(AssertionError):
        Mesh({"dp": 3})


def test_mesh_product_mismatch():
    run_distributed(_bad_mesh, 2)
