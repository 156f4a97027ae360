"""Expert parallelism: a top-k routed SwiGLU mixture-of-experts layer whose experts are spread over a mesh axis.

The reference reserves ``torchure/parallelism/expert_parallel.py`` (empty); the primitive it names for the token
shuffle is the even-split ``all_to_all``.  Here:

* ``MoELayer``  router (linear + softmax top-k), experts as stacked SwiGLU weights; with ``mesh`` given, rank r owns
  experts [r*E/n, (r+1)*E/n).
* dispatch: tokens are bucketed per expert with a fixed capacity (even splits: the all_to_all stays even), sent to the
  owning rank, processed, sent back (combine) and weighted by their gate values.  Overflowing tokens are dropped
  (contribute zero), as in capacity-factor routing.
* both exchanges are autograd functions (the backward of an all-to-all is the inverse all-to-all).
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from torchure_b200.core.collective import all_to_all


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mesh, dim):
        ctx.mesh, ctx.dim = mesh, dim
        return all_to_all(x.contiguous(), mesh, dim, 0, 0)

    @staticmethod
    def backward(ctx, g):
        return all_to_all(g.contiguous(), ctx.mesh, ctx.dim, 0, 0), None, None


class MoELayer(nn.Module):
    def __init__(self, hidden: int, ffn: int, num_experts: int, top_k: int = 2, capacity_factor: float = 2.0,
                 mesh=None, dim: str = "ep"):
        super().__init__()
        self.hidden, self.ffn, self.E, self.k, self.cf = hidden, ffn, num_experts, top_k, capacity_factor
        self.mesh, self.dim = mesh, dim
        self.n = mesh.size(dim) if mesh is not None else 1
        self.r = mesh.coordinate(dim) if mesh is not None else 0
        assert num_experts % self.n == 0, "experts must divide evenly over the ep axis"
        self.local_E = num_experts // self.n
        self.router = nn.Linear(hidden, num_experts, bias=False)
        self.aux_loss = None
        self.w_gate = nn.Parameter(torch.empty(self.local_E, ffn, hidden))
        self.w_up = nn.Parameter(torch.empty(self.local_E, ffn, hidden))
        self.w_down = nn.Parameter(torch.empty(self.local_E, hidden, ffn))
        for w in (self.w_gate, self.w_up, self.w_down):
            nn.init.normal_(w, std=0.02)

    def shard_(self, mesh, dim: str = "ep") -> None:
        """Turn a layer that holds all experts into rank r's part of an expert-parallel one: experts
        [r E / n, (r + 1) E / n) are kept (as new, smaller parameters), the router stays whole."""
        assert self.n == 1, "already sharded"
        n, r = mesh.size(dim), mesh.coordinate(dim)
        assert self.E % n == 0, "experts must divide evenly over the ep axis"
        local = self.E // n
        for name in ("w_gate", "w_up", "w_down"):
            full = getattr(self, name)
            setattr(self, name, nn.Parameter(full.detach()[r * local:(r + 1) * local].clone()))
        self.mesh, self.dim, self.n, self.r, self.local_E = mesh, dim, n, r, local

    def load_full_experts(self, w_gate, w_up, w_down) -> None:
        """Take this rank's slice of unsharded (E, ...) expert weights."""
        lo = self.r * self.local_E
        with torch.no_grad():
            self.w_gate.copy_(w_gate[lo:lo + self.local_E])
            self.w_up.copy_(w_up[lo:lo + self.local_E])
            self.w_down.copy_(w_down[lo:lo + self.local_E])

    def capacity(self, tokens: int) -> int:
        return max(1, int(self.cf * tokens * self.k / self.E + 0.999))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x = x.reshape(-1, self.hidden)
        T = x.shape[0]
        C = self.capacity(T)
        probs = F.softmax(self.router(x).float(), dim=-1)
        gate, expert = probs.topk(self.k, dim=-1)                 # (T, k)
        gate = gate / gate.sum(-1, keepdim=True)
        # load-balancing term (Switch Transformer): E * sum_e (share of the assignments that went to e) * (mean router
        # probability of e); 1 when routing is uniform, larger when experts are over-subscribed.  Over this rank's
        # tokens; the owner of the loss reads `aux_loss` after the forward pass
        share = F.one_hot(expert, self.E).sum(dim=(0, 1)).float() / (T * self.k)
        self.aux_loss = self.E * (share * probs.mean(0)).sum()
        # slot of every (token, choice) inside its expert's buffer; choices beyond the capacity are dropped
        flat_e = expert.reshape(-1)
        onehot = F.one_hot(flat_e, self.E)
        pos = (onehot.cumsum(0) - 1).gather(1, flat_e[:, None]).squeeze(1)
        keep = pos < C
        token = torch.arange(T, device=x.device).repeat_interleave(self.k)
        buf = x.new_zeros(self.E * C, self.hidden)
        slot = flat_e * C + pos
        buf = buf.index_add(0, slot[keep], x[token[keep]])
        # (E*C, hidden) is already grouped by owning rank: E = n * local_E
        if self.n > 1:
            buf = _AllToAll.apply(buf, self.mesh, self.dim)     # now: [source rank][local expert][C]
            work = buf.view(self.n, self.local_E, C, self.hidden).transpose(0, 1).reshape(self.local_E, self.n * C, -1)
        else:
            work = buf.view(self.local_E, C, self.hidden)
        h = F.silu(torch.bmm(work, self.w_gate.transpose(1, 2))) * torch.bmm(work, self.w_up.transpose(1, 2))
        y = torch.bmm(h, self.w_down.transpose(1, 2))
        if self.n > 1:
            y = y.view(self.local_E, self.n, C, self.hidden).transpose(0, 1).reshape(self.E * C, self.hidden)
            y = _AllToAll.apply(y, self.mesh, self.dim)
        else:
            y = y.reshape(self.E * C, self.hidden)
        out = x.new_zeros(T, self.hidden)
        contrib = y[slot[keep]].to(out.dtype) * gate.reshape(-1)[keep][:, None].to(out.dtype)
        out = out.index_add(0, token[keep], contrib)      # (under autocast y is bf16 while the residual stream is fp32)
        return out.view(shape)
