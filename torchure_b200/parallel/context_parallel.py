"""Context parallelism: causal ring attention over a zigzag sequence layout.

The reference reserves ``torchure/parallelism/context_parallel.py`` (empty) and sketches the design in its roadmap:
zigzag chunks so causal work is balanced, K/V circulating around the ring (``ring_send_recv``, which stays on the
library p2p transport), partial results merged with their log-sum-exp, reverse accumulation of dK/dV in backward.

Layout: the sequence is cut into 2n chunks; rank r holds chunks (r, 2n-1-r) concatenated (``zigzag_split``).  At ring
step t a rank holds the K/V of rank (r - t) mod n.  Chunk-level causality decides which (query chunk, key chunk)
pairs are computed: full, diagonal (causal inside), or skipped.

Each pair is one call of a block attention that returns (out, lse); on GPUs that is the place to call the sm_100a
kernel (it already emits LSE); the reference implementation below is plain PyTorch so the algorithm is testable on CPU.
"""

from __future__ import annotations

import torch

from torchure_b200.core.collective import ring_send_recv


def zigzag_split(x: torch.Tensor, n: int, r: int, seq_dim: int = 1) -> torch.Tensor:
    chunks = x.chunk(2 * n, dim=seq_dim)
    return torch.cat([chunks[r], chunks[2 * n - 1 - r]], dim=seq_dim)


def zigzag_merge(parts: list[torch.Tensor], seq_dim: int = 1) -> torch.Tensor:
    """Inverse of zigzag_split given the per-rank tensors in rank order."""
    n = len(parts)
    chunks: list = [None] * (2 * n)
    for r, p in enumerate(parts):
        a, b = p.chunk(2, dim=seq_dim)
        chunks[r], chunks[2 * n - 1 - r] = a, b
    return torch.cat(chunks, dim=seq_dim)


def _block_attn(q, k, v, causal: bool):
    """q (B,H,Sq,d), k/v (B,H,Sk,d) -> out (B,H,Sq,d) fp32, lse (B,H,Sq)."""
    s = (q.float() @ k.float().transpose(-1, -2)) / q.shape[-1] ** 0.5
    if causal:
        mask = torch.ones(q.shape[-2], k.shape[-2], dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    return torch.exp(s - lse[..., None]) @ v.float(), lse


def _merge(out, lse, o2, l2):
    new = torch.logaddexp(lse, l2)
    return out * torch.exp(lse - new)[..., None] + o2 * torch.exp(l2 - new)[..., None], new


def _pairs(r: int, src: int, n: int):
    """(query half, key half, causal?) pairs to compute when rank r holds the K/V of rank src."""
    qc, kc = (r, 2 * n - 1 - r), (src, 2 * n - 1 - src)
    out = []
    for qi in range(2):
        for ki in range(2):
            if kc[ki] < qc[qi]:
                out.append((qi, ki, False))
            elif kc[ki] == qc[qi]:
                out.append((qi, ki, True))
    return out


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mesh, dim):
        n, r = mesh.size(dim), mesh.coordinate(dim)
        B, H, S2, d = q.shape
        half = S2 // 2
        rep = H // k.shape[1]
        out = torch.zeros(B, H, S2, d, dtype=torch.float32, device=q.device)
        lse = torch.full((B, H, S2), float("-inf"), dtype=torch.float32, device=q.device)
        kk, vv = k.contiguous(), v.contiguous()
        for t in range(n):
            src = (r - t) % n
            ke, ve = kk.repeat_interleave(rep, 1), vv.repeat_interleave(rep, 1)
            for qi, ki, causal in _pairs(r, src, n):
                qs, ks = slice(qi * half, (qi + 1) * half), slice(ki * half, (ki + 1) * half)
                o2, l2 = _block_attn(q[:, :, qs], ke[:, :, ks], ve[:, :, ks], causal)
                out[:, :, qs], lse[:, :, qs] = _merge(out[:, :, qs], lse[:, :, qs], o2, l2)
            if t + 1 < n:
                kk, vv = ring_send_recv(kk, mesh, dim), ring_send_recv(vv, mesh, dim)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.mesh, ctx.dim = mesh, dim
        return out.to(q.dtype)

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse = ctx.saved_tensors
        mesh, dim = ctx.mesh, ctx.dim
        n, r = mesh.size(dim), mesh.coordinate(dim)
        B, H, S2, d = q.shape
        half = S2 // 2
        Hkv = k.shape[1]
        rep = H // Hkv
        do = d_out.float()
        delta = (do * out).sum(-1)
        dq = torch.zeros_like(q, dtype=torch.float32)
        kk, vv = k.contiguous(), v.contiguous()
        dk_acc = torch.zeros(B, Hkv, S2, d, dtype=torch.float32, device=q.device)
        dv_acc = torch.zeros_like(dk_acc)
        scale = d ** -0.5
        for t in range(n):
            src = (r - t) % n
            ke, ve = kk.repeat_interleave(rep, 1).float(), vv.repeat_interleave(rep, 1).float()
            for qi, ki, causal in _pairs(r, src, n):
                qs, ks = slice(qi * half, (qi + 1) * half), slice(ki * half, (ki + 1) * half)
                s = (q[:, :, qs].float() @ ke[:, :, ks].transpose(-1, -2)) * scale
                if causal:
                    mask = torch.ones(half, half, dtype=torch.bool, device=q.device).tril()
                    s = s.masked_fill(~mask, float("-inf"))
                p = torch.exp(s - lse[:, :, qs][..., None])
                dp = do[:, :, qs] @ ve[:, :, ks].transpose(-1, -2)
                ds = p * (dp - delta[:, :, qs][..., None]) * scale
                dq[:, :, qs] += ds @ ke[:, :, ks]
                dk_acc[:, :, ks] += (ds.transpose(-1, -2) @ q[:, :, qs].float()).view(B, Hkv, rep, half, d).sum(2)
                dv_acc[:, :, ks] += (p.transpose(-1, -2) @ do[:, :, qs]).view(B, Hkv, rep, half, d).sum(2)
            # the gradient accumulators travel with their K/V block; after n hops they are home
            dk_acc, dv_acc = ring_send_recv(dk_acc, mesh, dim), ring_send_recv(dv_acc, mesh, dim)
            if t + 1 < n:
                kk, vv = ring_send_recv(kk, mesh, dim), ring_send_recv(vv, mesh, dim)
        return dq.to(q.dtype), dk_acc.to(k.dtype), dv_acc.to(v.dtype), None, None


def ring_attention(q, k, v, mesh, dim: str = "cp"):
    """Causal attention over a sequence sharded in zigzag order along `dim`.
    q (B, Hq, 2c, d), k/v (B, Hkv, 2c, d) are this rank's two chunks; returns (B, Hq, 2c, d)."""
    return _RingAttention.apply(q, k, v, mesh, dim)


def zigzag_positions(seq_len: int, n: int, r: int, device=None) -> torch.Tensor:
    """Global position ids of this rank's tokens (RoPE must use these, not 0..S/n)."""
    return zigzag_split(torch.arange(seq_len, device=device)[None], n, r, seq_dim=1)[0]
