"""Qwen3-style decoder whose feed-forward layers are top-k routed mixtures of SwiGLU experts.

Not in the reference (its registry holds the dense model only; expert parallelism is an empty file there).  It exists
so that the expert-parallel layer (``parallel/expert_parallel.py``) has a model the config can select: every block
keeps the dense model's attention and norms and swaps the MLP for ``MoELayer``.  The blocks run the PyTorch path
(``impl`` is fixed to "torch"): the sm_100a engine has no grouped expert GEMM.

With ``mesh: {"dp": D, "ep": E}`` the Trainer calls ``shard_experts``: rank r of an ``ep`` group keeps experts
[r E_total / E, (r + 1) E_total / E) of every layer, tokens travel to their experts' owners and back through the
even-split all-to-all, and every rank of the group reads different rows (the axis is also a data axis).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from torchure_b200.models.qwen3 import Qwen3, RMSNorm
from torchure_b200.parallel.expert_parallel import MoELayer


class Qwen3MoE(Qwen3):
    def __init__(self, num_layers: int, num_heads: int, num_kv_heads: int, emb_dim: int, head_dim: int | None,
                 vocab_size: int, num_experts: int, top_k: int = 2, moe_ffn_dim: int | None = None,
                 capacity_factor: float = 2.0, aux_loss_coef: float = 0.01, ffn_dim: int | None = None,
                 norm_eps: float = 1e-6,
                 rope_theta: float = 1_000_000.0, qk_norm: bool = True, tie_embeddings: bool = True,
                 impl: str = "torch"):
        super().__init__(num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, emb_dim=emb_dim,
                         head_dim=head_dim, vocab_size=vocab_size, ffn_dim=ffn_dim, norm_eps=norm_eps,
                         rope_theta=rope_theta, qk_norm=qk_norm, tie_embeddings=tie_embeddings, impl="torch")
        width = moe_ffn_dim if moe_ffn_dim is not None else self.cfg["ffn_dim"]
        self.cfg.update(num_experts=num_experts, top_k=top_k, moe_ffn_dim=width, capacity_factor=capacity_factor,
                        aux_loss_coef=aux_loss_coef)
        self.aux_loss_coef = aux_loss_coef
        for block in self.blocks:
            block.ffn = MoELayer(emb_dim, width, num_experts, top_k, capacity_factor)

    @torch.no_grad()
    def init_weights(self, std: float = 0.02) -> None:
        """The dense model's scheme; the stacked expert matrices count as matrices, and every expert's down
        projection gets the residual-stream scaling (2L)^-1/2."""
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=std)
            elif isinstance(m, MoELayer):
                for w in (m.w_gate, m.w_up, m.w_down):
                    nn.init.normal_(w, mean=0.0, std=std)
            elif isinstance(m, RMSNorm):
                nn.init.ones_(m.weight)
        scale = (2 * len(self.blocks)) ** -0.5
        for b in self.blocks:
            b.gqa.o_proj.weight.mul_(scale)
            b.ffn.w_down.mul_(scale)

    def aux_loss(self) -> torch.Tensor:
        """Mean over the layers of the routers' load-balancing terms of the LAST forward pass; the objective adds
        ``aux_loss_coef`` times this to the language-model loss."""
        terms = [b.ffn.aux_loss for b in self.blocks]
        return torch.stack(terms).mean()

    def fused_param_groups(self):
        return [(b.gqa.q_proj.weight, b.gqa.k_proj.weight, b.gqa.v_proj.weight) for b in self.blocks]

    def shard_experts(self, mesh, dim: str = "ep") -> None:
        for b in self.blocks:
            b.ffn.shard_(mesh, dim)

    def expert_params(self) -> list[nn.Parameter]:
        return [w for b in self.blocks for w in (b.ffn.w_gate, b.ffn.w_up, b.ffn.w_down)]
