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
        self._hyper: list[torch.Tensor] | None = None   # per group {lr, bias1, bias2} on the device
        self._hyper_cur: int | None = None
        self._graph_groups: dict[int, list[torch.Tensor]] = {}

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

        capturing = torch.cuda.is_current_stream_capturing()
        for gi, group in enumerate(self.param_groups):
            ps = [p for p in group["params"] if p.grad is not None]
            if not ps:
                continue
            t, lr = self._advance_group(group, ps)
            b1, b2 = group["betas"]
            hyper = None
            if self._hyper is not None:
                # lr and the bias corrections come from device memory, so the launch can be replayed from a graph
                if not capturing:
                    self._upload_hyper(gi, lr, 1.0 - b1 ** t, 1.0 - b2 ** t)
                hyper = self._hyper[gi]
            multi_tensor.adamw_step(
                params=ps,
                grads=[p.grad for p in ps],
                exp_avgs=[self.state[p]["exp_avg"] for p in ps],
                exp_avg_sqs=[self.state[p]["exp_avg_sq"] for p in ps],
                shadows=[self._shadow.get(p) for p in ps],
                lr=lr, beta1=b1, beta2=b2, eps=group["eps"], weight_decay=group["weight_decay"],
                step=t, grad_scale=scale, maximize=group.get("maximize", False), hyper=hyper,
            )
            self._graph_groups[gi] = ps
        return loss

    def _advance_group(self, group, ps) -> tuple[int, float]:
        """Host bookkeeping of one step for one group: state init, step count, current lr."""
        for p in ps:
            st = self.state[p]
            if len(st) == 0:
                st["step"] = torch.tensor(0.0, dtype=torch.float32)
                st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        # every tensor of a group steps together; read the count once on the host
        t = int(self.state[ps[0]]["step"].item()) + 1
        for p in ps:
            self.state[p]["step"] = torch.tensor(float(t), dtype=torch.float32)
        lr = group["lr"]
        return t, (float(lr.item()) if torch.is_tensor(lr) else float(lr))

    # -- CUDA-graph support -----------------------------------------------------------------------------
    def enable_device_hyper(self, ring: int = 8) -> None:
        """Keep {lr, 1-beta1^t, 1-beta2^t} of every group in device memory, refreshed from a ring of pinned host
        slots before each launch.  A captured step then never bakes a step-dependent scalar into a kernel node."""
        if self._hyper is not None:
            return
        dev = self.param_groups[0]["params"][0].device
        n = len(self.param_groups)
        self._hyper = [torch.zeros(3, dtype=torch.float32, device=dev) for _ in range(n)]
        self._hyper_host = torch.zeros(ring, n, 3, dtype=torch.float32).pin_memory()
        self._hyper_events = [None] * ring
        self._hyper_slot = 0

    def _upload_hyper(self, gi: int, lr: float, bias1: float, bias2: float) -> None:
        if gi == 0 or self._hyper_cur is None:
            slot = self._hyper_slot
            self._hyper_slot = (slot + 1) % self._hyper_host.shape[0]
            ev = self._hyper_events[slot]
            if ev is not None:
                ev.synchronize()  # the copy that last read this slot has run
            self._hyper_cur = slot
        slot = self._hyper_cur
        self._hyper_host[slot, gi, 0] = lr
        self._hyper_host[slot, gi, 1] = bias1
        self._hyper_host[slot, gi, 2] = bias2
        self._hyper[gi].copy_(self._hyper_host[slot, gi], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._hyper_events[slot] = ev

    def host_state(self) -> dict:
        """Step counters, for undoing the bookkeeping of a step that was only captured, not executed."""
        return {id(p): st["step"].clone() for p, st in self.state.items() if "step" in st}

    def restore_host_state(self, snap: dict) -> None:
        for p, st in self.state.items():
            if id(p) in snap:
                st["step"] = snap[id(p)].clone()

    def host_advance(self) -> None:
        """The host half of ``step()`` for a step whose kernels are replayed from a graph: advance the counters and
        refresh the device-resident scalars (stream-ordered before the replay)."""
        assert self._hyper is not None and self._graph_groups, "capture a step with enable_device_hyper() first"
        for gi, group in enumerate(self.param_groups):
            ps = self._graph_groups.get(gi)
            if not ps:
                continue
            t, lr = self._advance_group(group, ps)
            b1, b2 = group["betas"]
            self._upload_hyper(gi, lr, 1.0 - b1 ** t, 1.0 - b2 ** t)
