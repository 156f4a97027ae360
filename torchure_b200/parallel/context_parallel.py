"""Context parallelism: causal ring attention over a zigzag sequence layout.

The reference reserves ``torchure/parallelism/context_parallel.py`` (empty) and sketches the design in its roadmap:
zigzag chunks so causal work is balanced, K/V circulating around the ring (``ring_send_recv``, which stays on the
library p2p transport), partial results merged with their log-sum-exp, reverse accumulation of dK/dV in backward.

Layout: the sequence is cut into 2n chunks; rank r holds chunks (r, 2n-1-r) concatenated (``zigzag_split``).  At ring
step t a rank holds the K/V of rank (r - t) mod n.  Chunk-level causality decides which (query chunk, key chunk)
pairs are computed: full, diagonal (causal inside), or skipped.

Each pair is one call of a block attention that returns (out, lse).  Two implementations of the same schedule:

``_RingAttention``       plain PyTorch on (B, H, S, d) tensors: the CPU / oracle path.
``_RingAttentionSm100``  (B, S, H, 128) bf16 tensors on Blackwell: every pair is one launch of the tcgen05 forward
                         kernel on the tensors where they lie (``attn_fwd_pair``: row offsets select the chunk, a flag
                         selects diagonal or full visibility) and one merge kernel; backward is one launch of the
                         single-pass backward kernel per pair, all pairs adding into one fp32 dQ accumulator, with
                         the dK / dV accumulators travelling around the ring.  The K/V exchange for step t+1 is issued
                         on a side stream before the pairs of step t are launched, so it runs under them.
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


def _ring_next(t: torch.Tensor, mesh, dim, side: torch.cuda.Stream) -> torch.Tensor:
    """Start sending `t` to the next rank of the ring on the side stream; the caller waits for `side` before use."""
    cur = torch.cuda.current_stream()
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        out = ring_send_recv(t, mesh, dim)
    t.record_stream(side)
    out.record_stream(cur)
    return out


def ring_fwd_sm100(q2, q_col0, k2, v2, B, S2, Hq, Hkv, mesh, dim):
    """Forward ring on the tcgen05 block-pair kernels.  q2: bf16 [B * S2, ld] whose head h sits at columns
    [q_col0 + 128 h, ...) (any row stride: the q columns of a fused projection are used where they lie); k2 / v2:
    contiguous bf16 [B * S2, Hkv * 128], this rank's chunks, which travel around the ring.  Returns the merged
    output (bf16 [B * S2, Hq * 128]) and its log-sum-exp (fp32 [B, Hq, S2])."""
    from torchure_b200 import ops

    ext = ops.ext()
    n, r = mesh.size(dim), mesh.coordinate(dim)
    half = S2 // 2
    dev = q2.device
    out = torch.zeros(B * S2, Hq * 128, dtype=torch.float32, device=dev)
    lse = torch.full((B, Hq, S2), float("-inf"), dtype=torch.float32, device=dev)
    o_p = torch.empty(B * half, Hq * 128, dtype=torch.bfloat16, device=dev)
    l_p = torch.empty(B, Hq, half, dtype=torch.float32, device=dev)
    side = torch.cuda.Stream(device=dev)
    kk, vv = k2, v2
    for t in range(n):
        src = (r - t) % n
        nk = nv = None
        if t + 1 < n:   # next step's K/V travel while this step's pairs run
            nk, nv = _ring_next(kk, mesh, dim, side), _ring_next(vv, mesh, dim, side)
        for qi, ki, causal in _pairs(r, src, n):
            ext.attn_fwd_pair(q2, q_col0, kk, 0, vv, 0, o_p, l_p, B, half, half, Hq, Hkv, S2, qi * half, S2, ki * half,
                              causal)
            ext.attn_merge(out, lse, o_p, l_p, B, half, Hq, S2, qi * half)
            ops.count_launch(2)
        if nk is not None:
            torch.cuda.current_stream().wait_stream(side)
            kk, vv = nk, nv
    return out.to(torch.bfloat16), lse


def ring_bwd_sm100(q2, q_col0, k2, v2, o16, lse, do2, B, S2, Hq, Hkv, mesh, dim):
    """Backward ring: one single-pass backward launch per block pair, all pairs adding into one head-major fp32 dQ
    accumulator; the fp32 dK / dV accumulators travel with their K/V block and are home after n hops.  Returns
    (dq_acc fp32 [B, Hq, S2, 128], dk fp32 [B, S2, Hkv * 128], dv likewise)."""
    from torchure_b200 import ops

    ext = ops.ext()
    n, r = mesh.size(dim), mesh.coordinate(dim)
    half = S2 // 2
    dev = q2.device
    nds = torch.empty(B, Hq, S2, dtype=torch.float32, device=dev)
    nlse2 = torch.empty_like(nds)
    dq_acc = torch.empty(B, Hq, S2, 128, dtype=torch.float32, device=dev)
    ext.attn_bwd_stats(do2, o16, lse, nds, nlse2, dq_acc, B, S2, Hq)   # statistics of the MERGED result; clears dq_acc
    ops.count_launch()
    dk_acc = torch.zeros(B, S2, Hkv * 128, dtype=torch.float32, device=dev)
    dv_acc = torch.zeros_like(dk_acc)
    dk_p = torch.empty(B * half, Hkv * 128, dtype=torch.bfloat16, device=dev)
    dv_p = torch.empty_like(dk_p)
    kk, vv = k2, v2
    side = torch.cuda.Stream(device=dev)
    for t in range(n):
        src = (r - t) % n
        nk = nv = None
        if t + 1 < n:
            nk, nv = _ring_next(kk, mesh, dim, side), _ring_next(vv, mesh, dim, side)
        for qi, ki, causal in _pairs(r, src, n):
            ext.attn_bwd_pair(q2, q_col0, kk, 0, vv, 0, do2, dq_acc, dk_p, dv_p, nds, nlse2, B, half, half, Hq, Hkv,
                              S2, qi * half, S2, ki * half, S2, qi * half, causal)
            ops.count_launch()
            ks = slice(ki * half, (ki + 1) * half)
            dk_acc[:, ks] += dk_p.view(B, half, Hkv * 128)
            dv_acc[:, ks] += dv_p.view(B, half, Hkv * 128)
        # the gradient accumulators travel with their K/V block; after n hops they are home
        dk_acc, dv_acc = ring_send_recv(dk_acc, mesh, dim), ring_send_recv(dv_acc, mesh, dim)
        if nk is not None:
            torch.cuda.current_stream().wait_stream(side)
            kk, vv = nk, nv
    return dq_acc, dk_acc, dv_acc


class _RingAttentionSm100(torch.autograd.Function):
    """q (B, S2, Hq, 128), k / v (B, S2, Hkv, 128) bf16: this rank's two zigzag chunks, token-major."""

    @staticmethod
    def forward(ctx, q, k, v, mesh, dim):
        B, S2, Hq, hd = q.shape
        Hkv = k.shape[2]
        q2 = q.contiguous().view(B * S2, Hq * hd)
        k2, v2 = k.contiguous().view(B * S2, Hkv * hd), v.contiguous().view(B * S2, Hkv * hd)
        o16, lse = ring_fwd_sm100(q2, 0, k2, v2, B, S2, Hq, Hkv, mesh, dim)
        ctx.save_for_backward(q2, k2, v2, o16, lse)
        ctx.mesh, ctx.dim, ctx.dims = mesh, dim, (B, S2, Hq, Hkv, hd)
        return o16.view(B, S2, Hq, hd)

    @staticmethod
    def backward(ctx, d_out):
        from torchure_b200 import ops

        q2, k2, v2, o16, lse = ctx.saved_tensors
        B, S2, Hq, Hkv, hd = ctx.dims
        do2 = d_out.to(torch.bfloat16).contiguous().view(B * S2, Hq * hd)
        dq_acc, dk_acc, dv_acc = ring_bwd_sm100(q2, 0, k2, v2, o16, lse, do2, B, S2, Hq, Hkv, ctx.mesh, ctx.dim)
        dq = torch.empty(B * S2, Hq * hd, dtype=torch.bfloat16, device=q2.device)
        ops.ext().attn_dq_convert(dq_acc, dq, B, S2, Hq)
        ops.count_launch()
        return (dq.view(B, S2, Hq, hd), dk_acc.to(torch.bfloat16).view(B, S2, Hkv, hd),
                dv_acc.to(torch.bfloat16).view(B, S2, Hkv, hd), None, None)


def ring_attention_tokens(q, k, v, mesh, dim: str = "cp"):
    """Token-major variant: q (B, 2c, Hq, d), k / v (B, 2c, Hkv, d) are this rank's two zigzag chunks; returns
    (B, 2c, Hq, d).  On Blackwell with bf16, d = 128 and c a multiple of 128 every block pair runs on the tcgen05
    attention kernels; anything else goes through the PyTorch implementation."""
    from torchure_b200.ops.attention import pair_supported

    half_ok = q.shape[1] % 256 == 0
    if half_ok and pair_supported(q, k, v):
        return _RingAttentionSm100.apply(q, k, v, mesh, dim)
    return _RingAttention.apply(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), mesh, dim).transpose(1, 2)


def ring_attention(q, k, v, mesh, dim: str = "cp"):
    """Causal attention over a sequence sharded in zigzag order along `dim`.
    q (B, Hq, 2c, d), k/v (B, Hkv, 2c, d) are this rank's two chunks; returns (B, Hq, 2c, d)."""
    from torchure_b200.ops.attention import pair_supported

    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if q.is_cuda and qt.shape[1] % 256 == 0 and pair_supported(qt, kt, vt):
        return _RingAttentionSm100.apply(qt, kt, vt, mesh, dim).transpose(1, 2)
    return _RingAttention.apply(q, k, v, mesh, dim)


def zigzag_positions(seq_len: int, n: int, r: int, device=None) -> torch.Tensor:
    """Global position ids of this rank's tokens (RoPE must use these, not 0..S/n)."""
    return zigzag_split(torch.arange(seq_len, device=device)[None], n, r, seq_dim=1)[0]
