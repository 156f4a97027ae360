"""AdamW whose CUDA step is one hand-written multi-tensor kernel.

State layout (``state[p] = {step, exp_avg, exp_avg_sq}``, two param groups) is the one
``torch.optim.AdamW`` writes, so ``optimizer.pt`` interchanges with the reference
(``torchure/optimizer/builder.py:20-47``; config key ``fused`` selects the kernel).

The kernel (``torchure_b200/csrc/multi_tensor.cu``) reads fp32 or bf16 grads, multiplies
them by an optional device-resident clip coefficient, applies decoupled weight decay and
the bias-corrected Adam update to the fp32 master weights, and writes the bf16 shadow
copy that the GEMMs consume: one pass over 16 bytes/element read and 14 written, instead
of separate clip-scale, optimizer and autocast-cast passes.
"""

from __future__ import annotations

import torch


class AdamW(torch.optim.AdamW):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, fused=None, **kw):
        self._want_kernel = bool(fused)
        super().__init__(params, lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, **kw)
        self._grad_scale: torch.Tensor | None = None
        self._shadow: dict[torch.Tensor, torch.Tensor] = {}

    # -- hooks for the trainer -------------------------------------------------------------
    def set_grad_scale(self, coef: torch.Tensor | None) -> None:
        """Device scalar multiplied into every grad during the next step (fused grad clipping)."""
        self._grad_scale = coef

    def attach_shadow(self, param: torch.Tensor, shadow: torch.Tensor) -> None:
        """Register a bf16 tensor that receives the updated value of `param` at every step."""
        self._shadow[param] = shadow

    def _kernel_ok(self, group) -> bool:
        if not self._want_kernel:
            return False
        ps = [p for p in group["params"] if p.grad is not None]
        if not ps or not all(p.is_cuda and p.dtype == torch.float32 for p in ps):
            return False
        from torchure_b200.ops import multi_tensor

        return multi_tensor.available()

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        scale = self._grad_scale
        self._grad_scale = None
        if not any(self._kernel_ok(g) for g in self.param_groups):
            if scale is not None:
                grads = [p.grad for g in self.param_groups for p in g["params"] if p.grad is not None]
                torch._foreach_mul_(grads, scale)
            out = super().step()
            for p, s in self._shadow.items():
                s.copy_(p)
            return loss if closure is not None else out
        from torchure_b200.ops import multi_tensor

        for group in self.param_groups:
            ps = [p for p in group["params"] if p.grad is not None]
            if not ps:
                continue
            for p in ps:
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = torch.tensor(0.0, dtype=torch.float32)
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            # every tensor of a group steps together; read the count once on the host
            step0 = self.state[ps[0]]["step"]
            t = int(step0.item()) + 1
            for p in ps:
                self.state[p]["step"] = torch.tensor(float(t), dtype=torch.float32)
            b1, b2 = group["betas"]
            lr = group["lr"]
            lr = float(lr.item()) if torch.is_tensor(lr) else float(lr)
            multi_tensor.adamw_step(
                params=ps,
                grads=[p.grad for p in ps],
                exp_avgs=[self.state[p]["exp_avg"] for p in ps],
                exp_avg_sqs=[self.state[p]["exp_avg_sq"] for p in ps],
                shadows=[self._shadow.get(p) for p in ps],
                lr=lr, beta1=b1, beta2=b2, eps=group["eps"], weight_decay=group["weight_decay"],
                step=t, grad_scale=scale, maximize=group.get("maximize", False),
            )
        return loss
