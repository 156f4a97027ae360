"""Qwen3-style dense decoder (also the llama3 variant of the same block).

Module tree and ``state_dict`` keys match reference ``torchure/models/qwen3/qwen3.py``
(``token_emb``, ``blocks.{i}.gqa.{q,k,v,o}_proj``, ``blocks.{i}.gqa.{q,k}_norm``,
``blocks.{i}.norm{1,2}``, ``blocks.{i}.ffn.{gate,up,down}_proj``, ``norm``, ``lm_head``
tied to ``token_emb``; reference lines 86-353), so checkpoints interchange.

Two execution paths share the parameters:

``torch``  plain PyTorch ops under autograd: the fp32 oracle, the CPU path, and the path
           used when an attention mask (padding) is supplied.
``sm100``  one autograd node per transformer block whose forward and backward are
           sequences of hand-written sm_100a kernels (``torchure_b200/ops/block.py``):
           bf16 tcgen05 GEMMs on bf16 shadow weights, fused RMSNorm(+residual),
           fused QK-norm+RoPE, causal GQA flash attention with LSE, SwiGLU.  The residual
           stream stays fp32 as in the reference under autocast.

The path is picked per call: ``sm100`` when the input is on a CUDA device, the extension
is loaded and ``model.impl != "torch"``.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def default_ffn_dim(emb_dim: int) -> int:
    """8/3 * emb rounded up to a multiple of 256 (reference qwen3.py:247-249)."""
    return 256 * ((int(8 * emb_dim / 3) + 255) // 256)


class RMSNorm(nn.Module):
    """y = x * rsqrt(mean(x^2) + eps) * weight, statistics in fp32."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.dim = dim
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (y * self.weight.float()).to(x.dtype)


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin of shape positions.shape + (head_dim,), frequencies duplicated over both halves."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device).float() / head_dim))
    ang = positions.float()[..., None] * inv_freq
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotation: (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin). x: (B, H, S, hd)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    rot = torch.cat((-x2, x1), dim=-1)
    return x * cos.to(x.dtype) + rot * sin.to(x.dtype)


class RotaryEmbedding(nn.Module):
    def __init__(self, head_dim: int, base: float = 1_000_000.0):
        super().__init__()
        assert head_dim % 2 == 0, "RoPE needs an even head_dim"
        self.head_dim = head_dim
        self.base = float(base)
        inv_freq = 1.0 / (self.base ** (torch.arange(0, head_dim, 2).float() / head_dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self._cache: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}

    def tables(self, seq_len: int, device) -> tuple[torch.Tensor, torch.Tensor]:
        """(S, hd) fp32 cos/sin for positions 0..S-1, cached per (seq_len, device)."""
        key = (seq_len, torch.device(device))
        hit = self._cache.get(key)
        if hit is None:
            pos = torch.arange(seq_len, device=device)
            ang = pos.float()[:, None] * self.inv_freq.to(device)[None, :]
            ang = torch.cat([ang, ang], dim=-1)
            hit = (ang.cos().contiguous(), ang.sin().contiguous())
            self._cache[key] = hit
        return hit

    def zigzag_tables(self, local_len: int, n: int, r: int, device) -> tuple[torch.Tensor, torch.Tensor]:
        """(local_len, hd) fp32 cos/sin of the global positions that rank r of n holds under context parallelism:
        chunks r and 2n-1-r of a sequence of n * local_len tokens cut into 2n chunks."""
        key = ("zigzag", local_len, n, r, torch.device(device))
        hit = self._cache.get(key)
        if hit is None:
            cos, sin = self.tables(local_len * n, device)
            c = local_len // 2
            pos = torch.cat([torch.arange(r * c, (r + 1) * c, device=device),
                             torch.arange((2 * n - 1 - r) * c, (2 * n - r) * c, device=device)])
            hit = (cos[pos].contiguous(), sin[pos].contiguous())
            self._cache[key] = hit
        return hit

    def forward(self, position_ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """(B, 1, S, hd) fp32 cos/sin for arbitrary position ids (padded batches)."""
        ang = position_ids.float()[:, :, None] * self.inv_freq[None, None, :]
        ang = torch.cat([ang, ang], dim=-1)
        return ang.cos()[:, None], ang.sin()[:, None]


class GroupQueryAttention(nn.Module):
    def __init__(self, num_heads: int, emb_dim: int, num_kv_heads: int, head_dim: int | None,
                 qk_norm: bool = True, norm_eps: float = 1e-6):
        super().__init__()
        assert num_heads % num_kv_heads == 0, "num_heads must be a multiple of num_kv_heads"
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.emb_dim = emb_dim
        self.head_dim = head_dim if head_dim is not None else emb_dim // num_heads
        q_out, kv_out = num_heads * self.head_dim, num_kv_heads * self.head_dim
        self.q_proj = nn.Linear(emb_dim, q_out, bias=False)
        self.k_proj = nn.Linear(emb_dim, kv_out, bias=False)
        self.v_proj = nn.Linear(emb_dim, kv_out, bias=False)
        self.o_proj = nn.Linear(q_out, emb_dim, bias=False)
        self.qk_norm = qk_norm
        if qk_norm:
            self.q_norm = RMSNorm(self.head_dim, norm_eps)
            self.k_norm = RMSNorm(self.head_dim, norm_eps)

    def forward(self, x, cos, sin, attention_mask=None, batch_shape=None, cp=None, cp_kind="ring"):
        # `batch_shape` = (B, S) under sequence parallelism: x is then this rank's slice of the B * S tokens laid out
        # as one row sequence [1, B * S / n, D], which the column-parallel projections gather.
        # `cp` = (mesh, axis) under context parallelism: x holds this rank's part of every sequence and cos / sin its
        # global positions; attention runs as a ring over the axis (two zigzag chunks per rank), or, `cp_kind`
        # "ulysses", on whole sequences of 1/n of the heads between two all-to-alls (one contiguous chunk per rank).
        q = self.q_proj(x)
        B, S = batch_shape if batch_shape is not None else (x.shape[0], q.shape[1])
        q = q.view(B, S, self.num_heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(B, S, self.num_kv_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(B, S, self.num_kv_heads, self.head_dim).transpose(1, 2)
        if self.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        if cp is not None:
            from torchure_b200.parallel.context_parallel import ring_attention

            assert attention_mask is None, "context parallelism: causal path only"
            if cp_kind == "ulysses":
                from torchure_b200.parallel.ulysses import ulysses_attention

                o = ulysses_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), *cp).to(v.dtype)
                return self.o_proj(o.reshape(B, S, self.num_heads * self.head_dim))
            o = ring_attention(q, k, v, *cp).to(v.dtype)
            return self.o_proj(o.transpose(1, 2).reshape(B, S, self.num_heads * self.head_dim))
        rep = self.num_heads // self.num_kv_heads
        if rep > 1:
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
        if attention_mask is None:
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        else:
            causal = torch.ones(S, S, dtype=torch.bool, device=x.device).tril()
            mask = causal[None, None] & attention_mask[:, None, None, :].bool()
            # keep the diagonal so fully padded query rows do not produce NaN
            mask = mask | torch.eye(S, dtype=torch.bool, device=x.device)[None, None]
            o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        o = o.transpose(1, 2).reshape(B, S, self.num_heads * self.head_dim)
        if batch_shape is not None:
            o = o.reshape(1, B * S, -1)
        return self.o_proj(o)


class SwiGLU(nn.Module):
    def __init__(self, hidden_dim: int, ffn_dim: int):
        super().__init__()
        self.gate_proj = nn.Linear(hidden_dim, ffn_dim, bias=False)
        self.up_proj = nn.Linear(hidden_dim, ffn_dim, bias=False)
        self.down_proj = nn.Linear(ffn_dim, hidden_dim, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class TransformerBlock(nn.Module):
    def __init__(self, num_heads, emb_dim, num_kv_heads, head_dim=None, ffn_dim=None,
                 qk_norm=True, norm_eps=1e-6):
        super().__init__()
        self.gqa = GroupQueryAttention(num_heads, emb_dim, num_kv_heads, head_dim, qk_norm, norm_eps)
        self.norm1 = RMSNorm(emb_dim, norm_eps)
        self.norm2 = RMSNorm(emb_dim, norm_eps)
        self.ffn = SwiGLU(emb_dim, ffn_dim if ffn_dim is not None else default_ffn_dim(emb_dim))

    def forward(self, x, cos, sin, attention_mask=None, batch_shape=None, cp=None, cp_kind="ring"):
        x = x + self.gqa(self.norm1(x), cos, sin, attention_mask, batch_shape, cp, cp_kind)
        return x + self.ffn(self.norm2(x))


class Qwen3(nn.Module):
    """Dense decoder. ``impl``: "auto" (sm100 kernels on CUDA when built) or "torch"."""

    def __init__(self, num_layers: int, num_heads: int, num_kv_heads: int, emb_dim: int, head_dim: int | None,
                 vocab_size: int, ffn_dim: int | None = None, norm_eps: float = 1e-6,
                 rope_theta: float = 1_000_000.0, qk_norm: bool = True, tie_embeddings: bool = True,
                 impl: str = "auto"):
        super().__init__()
        self.cfg = dict(num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, emb_dim=emb_dim,
                        head_dim=head_dim if head_dim is not None else emb_dim // num_heads,
                        vocab_size=vocab_size, ffn_dim=ffn_dim if ffn_dim is not None else default_ffn_dim(emb_dim),
                        norm_eps=norm_eps, rope_theta=rope_theta, qk_norm=qk_norm, tie_embeddings=tie_embeddings)
        self.impl = impl
        hd = self.cfg["head_dim"]
        self.token_emb = nn.Embedding(vocab_size, emb_dim)
        self.rope = RotaryEmbedding(hd, rope_theta)
        self.blocks = nn.ModuleList(
            TransformerBlock(num_heads, emb_dim, num_kv_heads, hd, ffn_dim, qk_norm, norm_eps)
            for _ in range(num_layers)
        )
        self.norm = RMSNorm(emb_dim, norm_eps)
        self.lm_head = nn.Linear(emb_dim, vocab_size, bias=False)
        if tie_embeddings:
            self.lm_head.weight = self.token_emb.weight
        self._engine = None  # sm100 execution state (bf16 shadow weights), built lazily
        self._grad_sink = None  # object with grad_dest(p) / grad_written(p): where the engine writes weight grads

    # -- init ----------------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, std: float = 0.02) -> None:
        """N(0, std) for matrices and the embedding, ones for norms, then the two projections
        that write into the residual stream scaled by (2L)^-1/2 (reference qwen3.py:288-311)."""
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=std)
            elif isinstance(m, RMSNorm):
                nn.init.ones_(m.weight)
        scale = (2 * len(self.blocks)) ** -0.5
        for b in self.blocks:
            b.gqa.o_proj.weight.mul_(scale)
            b.ffn.down_proj.weight.mul_(scale)

    # -- execution path ------------------------------------------------------------------
    def _use_sm100(self, ids: torch.Tensor, attention_mask) -> bool:
        if self.impl == "torch" or attention_mask is not None or not ids.is_cuda:
            return False
        from torchure_b200 import ops

        if not ops.available():
            return False
        if self.cfg["head_dim"] != 128:
            if not getattr(self, "_warned_head_dim", False):
                import warnings

                warnings.warn(f"head_dim {self.cfg['head_dim']} is not covered by the sm_100a kernels (128 only): this "
                              "model runs on the PyTorch path", stacklevel=3)
                self._warned_head_dim = True
            return False
        return True

    def fused_param_groups(self):
        """Parameters whose gradients one fused GEMM produces (rows of Wqkv, rows of [Wgate; Wup]).  A gradient
        sink that lays each group out contiguously, in this order, receives them with a single wgrad launch."""
        groups = []
        for b in self.blocks:
            groups.append((b.gqa.q_proj.weight, b.gqa.k_proj.weight, b.gqa.v_proj.weight))
            groups.append((b.ffn.gate_proj.weight, b.ffn.up_proj.weight))
        return groups

    def set_grad_sink(self, sink) -> None:
        """Route weight gradients of the sm_100a path straight into `sink` (fused DDP buckets) instead of returning
        them through autograd.  With a sink installed the loss must be the root of backward (incoming gradient 1):
        fold any scaling into ``compute_loss(..., loss_scale=)``."""
        self._grad_sink = sink

    def engine(self):
        if self._engine is None:
            from torchure_b200.ops.block import Sm100Engine

            self._engine = Sm100Engine(self)
        return self._engine

    def forward(self, x: torch.Tensor, attention_mask: torch.Tensor | None = None,
                return_hidden_states: bool = False, return_final_hidden: bool = False):
        if self._use_sm100(x, attention_mask) and not return_hidden_states:
            h = self.engine().forward_hidden(x)  # post-final-norm hidden, bf16
            if return_final_hidden:
                return h
            return self.engine().lm_head(h)
        B, S = x.shape
        cp = getattr(self, "cp", None)      # (mesh, axis): x holds this rank's zigzag chunks of sequences n times longer
        if cp is not None:
            assert attention_mask is None and not return_hidden_states, "context parallelism: causal path only"
            n, r = cp[0].size(cp[1]), cp[0].coordinate(cp[1])
            if getattr(self, "cp_kind", "ring") == "ulysses":
                cos, sin = (t[r * S:(r + 1) * S] for t in self.rope.tables(S * n, x.device))
            else:
                cos, sin = self.rope.zigzag_tables(S, n, r, x.device)
            cos, sin = cos[None, None], sin[None, None]
        elif attention_mask is None:
            cos, sin = self.rope.tables(S, x.device)
            cos, sin = cos[None, None], sin[None, None]
        else:
            attention_mask = attention_mask.bool()
            pos = (attention_mask.long().cumsum(dim=1) - 1).masked_fill(~attention_mask, 0)
            cos, sin = self.rope(pos)
        h = self.token_emb(x)
        sp = getattr(self, "sp", None)      # (mesh, axis) under tensor parallelism with sequence parallelism
        if sp is not None:
            from torchure_b200.parallel.tensor_parallel import shard_sequence, unshard_sequence

            assert attention_mask is None and not return_hidden_states, "sequence parallelism: causal path only"
            # all B * S tokens as one row sequence, of which every rank of the axis keeps a contiguous slice
            h = shard_sequence(h.reshape(1, B * S, -1), *sp)
        hidden_states = [h] if return_hidden_states else []
        for block in self.blocks:
            if sp is not None:
                h = block(h, cos, sin, attention_mask, (B, S))
            elif cp is not None:
                h = block(h, cos, sin, None, None, cp, getattr(self, "cp_kind", "ring"))
            else:
                h = block(h, cos, sin, attention_mask)
            if return_hidden_states:
                hidden_states.append(h)
        if sp is not None:
            h = unshard_sequence(h, *sp).reshape(B, S, -1)
        h = self.norm(h)
        if return_final_hidden:
            return h
        logits = self.lm_head(h)
        return (logits, hidden_states) if return_hidden_states else logits

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())


def flops_per_token(cfg: dict, seq_len: int) -> float:
    """Training FLOPs per token: 6 x matmul params (head included) + causal attention."""
    D, L, F_, V = cfg["emb_dim"], cfg["num_layers"], cfg["ffn_dim"], cfg["vocab_size"]
    hd, Hq, Hkv = cfg["head_dim"], cfg["num_heads"], cfg["num_kv_heads"]
    per_block = D * (Hq + 2 * Hkv) * hd + Hq * hd * D + 3 * D * F_
    matmul = L * per_block + V * D
    attn = 3 * (2 * seq_len * Hq * hd) * L  # fwd 2*S*H*hd*2/2 (causal), bwd 2x
    return 6.0 * matmul + attn
