"""Fully sharded data parallelism (FSDP2-style units, optional HSDP replication).

The reference only reserves the file (``torchure/parallelism/fsdp2.py`` is empty) and describes the design in
``notes/FSDP2_SCOPE.md``: one unit per transformer block plus one unit for (embedding, head, final norm) because of
the weight tie; parameters sharded along the ``dp_shard`` axis, all-gathered for a unit's forward and again for its
backward, gradients reduce-scattered ("avg") to the owner shard; with HSDP the shard gradients are additionally
all-reduced along ``dp_replicate``.  This module implements that:

* every unit owns ONE flat fp32 shard (an ``nn.Parameter`` the optimizer sees) and, while it is unsharded, one flat
  buffer that all of its original parameters are views of (caller-owned ``all_gather(output_tensor=)`` buffers, so
  the views stay the same objects across steps);
* unshard in a forward pre-hook and in a backward pre-hook, reshard after forward and after the unit's last
  gradient arrived (post-accumulate-grad hooks count them down);
* gradient reduction: flat full gradient -> ``reduce_scatter("avg")`` along the shard axis (-> ``all_reduce("avg")``
  along the replicate axis) -> ``shard.grad``;
* ``clip_grad_norm(shards, mesh, max_norm, shard_dims=(shard_dim,))`` gives the global norm (the sharded path of
  ``core/grad_helper.py``);
* ``full_state_dict()`` / ``load_full_state_dict()`` gather to / scatter from the reference's unsharded key layout,
  ``shard_state_dict()`` is what per-shard checkpoint files hold.

All communication goes through ``core.collective`` and therefore uses the sm_100a NVLink kernels on GPUs (the
all-gather lands directly in the unit's persistent buffer) and gloo on CPU.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from torchure_b200.core.collective import MeshLike, all_gather, all_reduce, broadcast, reduce_scatter


class _Unit:
    def __init__(self, name: str, params: list[tuple[str, nn.Parameter]], mesh, shard_dim: str):
        self.name = name
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        self.shapes = [p.shape for p in self.params]
        self.numels = [p.numel() for p in self.params]
        self.world = mesh.size(shard_dim)
        self.rank = mesh.coordinate(shard_dim)
        total = sum(self.numels)
        self.padded = (total + self.world - 1) // self.world * self.world
        self.shard_numel = self.padded // self.world
        dev, dtype = self.params[0].device, self.params[0].dtype
        full = torch.zeros(self.padded, dtype=dtype, device=dev)
        at = 0
        for p, n in zip(self.params, self.numels):
            full[at:at + n].copy_(p.detach().reshape(-1))
            at += n
        lo = self.rank * self.shard_numel
        self.shard = nn.Parameter(full[lo:lo + self.shard_numel].clone())
        self.full: torch.Tensor | None = None
        self.pending = len(self.params)
        self.unsharded = False
        self._empty = torch.empty(0, dtype=dtype, device=dev)
        self._release()

    def _release(self) -> None:
        for p in self.params:
            p.data = self._empty
        self.full = None
        self.unsharded = False

    def unshard(self, mesh, shard_dim: str) -> None:
        if self.unsharded:
            return
        full = torch.empty(self.padded, dtype=self.shard.dtype, device=self.shard.device)
        all_gather(self.shard.detach(), mesh, shard_dim, 0, output_tensor=full)
        self.full = full
        at = 0
        for p, n, shape in zip(self.params, self.numels, self.shapes):
            p.data = full[at:at + n].view(shape)
            at += n
        self.unsharded = True

    def reshard(self) -> None:
        self._release()

    def reduce_grads(self, mesh, shard_dim: str, replicate_dim: str | None) -> None:
        flat = torch.zeros(self.padded, dtype=self.shard.dtype, device=self.shard.device)
        at = 0
        for p, n in zip(self.params, self.numels):
            if p.grad is not None:
                flat[at:at + n].copy_(p.grad.reshape(-1))
                p.grad = None
            at += n
        g = reduce_scatter(flat, mesh, shard_dim, "avg")
        if replicate_dim is not None and mesh.size(replicate_dim) > 1:
            all_reduce(g, mesh, replicate_dim, "avg")
        if self.shard.grad is None:
            self.shard.grad = g
        else:
            self.shard.grad.add_(g)


class FSDP:
    def __init__(self, model: nn.Module, mesh: MeshLike, shard_dim: str = "dp_shard", replicate_dim: str | None = None,
                 units: list[tuple[str, list[nn.Module]]] | None = None):
        self.model, self.mesh = model, mesh
        self.shard_dim, self.replicate_dim = shard_dim, replicate_dim
        self.requires_sync = True
        # identical start on every rank: broadcast from coordinate 0 of every data axis
        for t in [*model.parameters(), *model.buffers()]:
            broadcast(t.detach(), mesh, shard_dim, src=0)
            if replicate_dim is not None:
                broadcast(t.detach(), mesh, replicate_dim, src=0)
        if units is None:
            units = self.default_units(model)
        names = {p: n for n, p in model.named_parameters()}  # tied weights appear once
        seen: set[int] = set()
        self.units: list[_Unit] = []
        self._unit_of: dict[nn.Parameter, _Unit] = {}
        for uname, modules in units:
            plist = []
            for m in modules:
                for p in m.parameters():
                    if id(p) not in seen and p.requires_grad:
                        seen.add(id(p))
                        plist.append((names[p], p))
            if not plist:
                continue
            unit = _Unit(uname, plist, mesh, shard_dim)
            self.units.append(unit)
            for _, p in plist:
                self._unit_of[p] = unit
            for m in modules:
                m.register_forward_pre_hook(lambda mod, args, u=unit: self._pre_forward(u))
                m.register_forward_hook(lambda mod, args, out, u=unit: self._post_forward(u, out))
                m.register_full_backward_pre_hook(lambda mod, gout, u=unit: self._pre_backward(u))
            for _, p in plist:
                p.register_post_accumulate_grad_hook(self._on_grad)
        missing = [n for n, p in model.named_parameters() if p.requires_grad and id(p) not in seen]
        assert not missing, f"parameters outside every FSDP unit: {missing}"
        self._keep_unsharded: set[int] = set()

    @staticmethod
    def default_units(model) -> list[tuple[str, list[nn.Module]]]:
        """One unit per transformer block; embedding, head and final norm share a unit (tied weight)."""
        units = [(f"blocks.{i}", [b]) for i, b in enumerate(model.blocks)]
        rest = [m for m in (getattr(model, "token_emb", None), getattr(model, "norm", None),
                            getattr(model, "lm_head", None)) if m is not None]
        units.append(("root", rest))
        return units

    # -- hooks -------------------------------------------------------------------------------------
    def _pre_forward(self, u: _Unit) -> None:
        u.unshard(self.mesh, self.shard_dim)

    def _post_forward(self, u: _Unit, out) -> None:
        # the root unit's modules are used at both ends of the network: keep it until its gradients are reduced
        if u.name != "root":
            u.reshard()

    def _pre_backward(self, u: _Unit) -> None:
        u.unshard(self.mesh, self.shard_dim)

    def _on_grad(self, p: nn.Parameter) -> None:
        u = self._unit_of[p]
        u.pending -= 1
        if u.pending == 0:
            u.pending = len(u.params)
            u.reduce_grads(self.mesh, self.shard_dim, self.replicate_dim)
            u.reshard()

    # -- what the trainer needs ----------------------------------------------------------------------
    def parameters(self) -> list[nn.Parameter]:
        """The flat shards: hand these to the optimizer and to ``clip_grad_norm(..., shard_dims=(shard_dim,))``."""
        return [u.shard for u in self.units]

    # the strategy interface shared with DDP and the engine variant (``train/trainer.py``)
    fused = False

    def optimizer_params(self) -> list[nn.Parameter]:
        return self.parameters()

    @property
    def clip_shard_dims(self) -> tuple[str, ...]:
        return (self.shard_dim,)

    def sync(self) -> None:
        """Reductions are issued synchronously from the hooks: nothing to wait for."""

    def sq_norm(self):
        return None

    def unshard_all(self) -> None:
        for u in self.units:
            u.unshard(self.mesh, self.shard_dim)

    def reshard_all(self) -> None:
        for u in self.units:
            u.reshard()

    def full_state_dict(self) -> dict[str, torch.Tensor]:
        """Unsharded fp32 state under the model's own keys (collective: every rank must call it)."""
        self.unshard_all()
        sd = {k: v.detach().clone() for k, v in self.model.state_dict().items()}
        self.reshard_all()
        return sd

    def load_full_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        for u in self.units:
            full = torch.zeros(u.padded, dtype=u.shard.dtype, device=u.shard.device)
            at = 0
            for name, n in zip(u.names, u.numels):
                full[at:at + n].copy_(sd[name].reshape(-1))
                at += n
            lo = u.rank * u.shard_numel
            with torch.no_grad():
                u.shard.copy_(full[lo:lo + u.shard_numel])

    def shard_state_dict(self) -> dict[str, torch.Tensor]:
        return {f"{u.name}.flat_shard": u.shard.detach() for u in self.units}

    def load_shard_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            for u in self.units:
                u.shard.copy_(sd[f"{u.name}.flat_shard"])
