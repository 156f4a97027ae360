"""Llama-3 family on the shared decoder block.

The reference only reserves the name (``torchure/models/llama3/llama3.py:1-3`` is a
docstring and the registry maps ``llama3_2`` to ``None``, ``models/builder.py:5-12``).
Here it is the Qwen3 block without QK-norm, RoPE base 500000, ``head_dim = emb/heads``,
RMSNorm eps 1e-5 and (for the 1B/3B "3.2" sizes) tied embeddings, so every kernel and
parallelism path of the Qwen3 model applies unchanged.
"""

from __future__ import annotations

from torchure_b200.models.qwen3 import Qwen3


class Llama3(Qwen3):
    def __init__(self, num_layers: int, num_heads: int, num_kv_heads: int, emb_dim: int, vocab_size: int,
                 ffn_dim: int | None = None, head_dim: int | None = None, norm_eps: float = 1e-5,
                 rope_theta: float = 500_000.0, tie_embeddings: bool = True, impl: str = "auto"):
        super().__init__(num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, emb_dim=emb_dim,
                         head_dim=head_dim, vocab_size=vocab_size, ffn_dim=ffn_dim, norm_eps=norm_eps,
                         rope_theta=rope_theta, qk_norm=False, tie_embeddings=tie_embeddings, impl=impl)
