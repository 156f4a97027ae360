"""Sharded data parallelism on the sm_100a engine (FSDP2 units, optional HSDP replication).

Design scoped by the reference in ``notes/FSDP2_SCOPE.md:94-193`` (units per transformer block plus a root unit for
the tied embedding / head, parameters sharded along ``dp_shard``, gradients reduce-scattered with "avg", sharded
gradient-norm clip); the reference ships no code for it (``torchure/parallelism/fsdp2.py`` is empty).  Built for a
180 GB GPU and NVSwitch rather than translated from a memory-starved design:

* **What is sharded**: the fp32 master weights and both AdamW moments (12 of the 16 bytes/parameter of mixed
  precision AdamW), row-wise per fused matrix (``[Wq;Wk;Wv]``, ``Wo``, ``[Wgate;Wup]``, ``Wdown``, the embedding).
  Each rank owns rows ``[r N/W, (r+1) N/W)`` as one fp32 ``nn.Parameter`` the optimizer sees.
* **What stays whole**: the bf16 compute copies of every matrix (2 bytes/parameter) and one fp32 gradient buffer
  (4 bytes/parameter), both inside the symmetric allocation of the shard axis.  The engine's GEMMs read the bf16
  copies where they lie; the wgrad GEMM epilogues, the fused linear+CE and the norm kernels write fp32 gradients
  straight into the buffer (the engine's gradient-sink protocol), so cast, accumulation over micro-batches and
  packing cost no kernel.
* **Per step** (all on the communication stream, overlapped with compute):
  ``begin_step``   one in-place all-gather kernel per unit: the fused AdamW kernel has just rewritten this rank's
                   rows of the bf16 copies (they are the shards' shadow tensors), the kernel pushes them into every
                   peer's copy with ``multimem.st`` / peer stores; block i waits only for unit i.
  backward         when the last gradient of a unit has been written in the sync micro-batch, ONE kernel
                   reduce-scatters the unit: every rank reduces its own rows straight out of the peers' buffers
                   (``multimem.ld_reduce`` / peer loads), scales by 1/W, writes the fp32 shard gradient and
                   publishes the sum of squares for clipping.
  With a ``dp_replicate`` axis the shard gradients are then all-reduced ("avg") along it (HSDP).
* Norm gains (a few thousand floats per block) are replicated; their gradients share one small symmetric buffer
  that is all-reduced once per step.

Traffic per parameter and step: 2 bytes gathered + 4 bytes reduce-scattered, against 8 for DDP's fp32 all-reduce,
and AdamW touches 1/W of the parameters.  The all-gather -> GEMM kernel of ``ops/gemm_comm.py`` gathers the ROW
(token) operand of a GEMM, which is what sequence parallelism needs; gathering the weight operand that way would
produce the transposed product, so the weight gather is a separate, overlapped kernel here.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from torchure_b200 import ops
from torchure_b200.core.collective import all_gather, all_reduce, broadcast

BF16 = torch.bfloat16


class _Matrix:
    """One fused weight matrix: whole bf16 compute copy and whole fp32 gradient (symmetric), fp32 master rows of this
    rank."""

    def __init__(self, name: str, params: list[tuple[str, nn.Parameter]], comm, rank: int, world: int):
        self.name = name
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        self.rows = sum(p.shape[0] for p in self.params)
        self.cols = self.params[0].shape[1]
        assert all(p.shape[1] == self.cols for p in self.params)
        assert self.rows % world == 0 and (self.rows // world * self.cols) % 8 == 0, (
            f"{name}: {self.rows} rows x {self.cols} cannot be split evenly over {world} ranks in 16-byte units")
        self.per = self.rows // world
        self.full_w = comm.alloc(self.rows * self.cols, BF16).view(self.rows, self.cols)
        self.full_g = comm.alloc(self.rows * self.cols, torch.float32).view(self.rows, self.cols)
        self.full_g.zero_()
        lo = rank * self.per
        whole = torch.cat([p.detach().float() for p in self.params], dim=0)
        self.shard = nn.Parameter(whole[lo:lo + self.per].clone())      # fp32 master rows (optimizer parameter)
        self.shard_w = self.full_w[lo:lo + self.per]                     # this rank's rows of the bf16 copy
        self.shard_w.copy_(self.shard.detach())
        self.shard_grad = torch.zeros_like(self.shard.data)
        # views of the gradient buffer shaped like the original parameters, rows adjacent in fusion order
        self.grad_views = {}
        at = 0
        for p in self.params:
            self.grad_views[p] = self.full_g[at:at + p.shape[0]]
            at += p.shape[0]


class _Unit:
    def __init__(self, index: int, name: str, mats: list[_Matrix]):
        self.index, self.name, self.mats = index, name, mats
        self.params = [p for m in mats for p in m.params]
        self.pending = len(self.params)
        self.gathered = torch.cuda.Event()
        self.reduced: torch.cuda.Event | None = None


class EngineFSDP:
    fused = True

    def __init__(self, model, mesh, shard_dim: str = "dp_shard", replicate_dim: str | None = None, comm_sms: int = 16,
                 wait_limit_s: float = 30.0):
        from torchure_b200.core.symm import SymmComm

        assert ops.available(), "EngineFSDP needs the sm_100a extension and a Blackwell GPU"
        self.model, self.mesh = model, mesh
        self.shard_dim, self.replicate_dim = shard_dim, replicate_dim
        self.world, self.rank = mesh.size(shard_dim), mesh.coordinate(shard_dim)
        self.requires_sync = True
        self.comm_sms = comm_sms
        dev = model.token_emb.weight.device
        for t in [*model.parameters(), *model.buffers()]:   # identical start on every rank of the data axes
            broadcast(t.detach(), mesh, shard_dim, src=0)
            if replicate_dim is not None:
                broadcast(t.detach(), mesh, replicate_dim, src=0)
        eng = model.engine()
        self.engine = eng
        names = {p: n for n, p in model.named_parameters()}
        # ---- layout of the symmetric region -----------------------------------------------------------------
        specs: list[tuple[str, list[tuple[str, list[nn.Parameter]]]]] = []
        for i, b in enumerate(model.blocks):
            g, f = b.gqa, b.ffn
            specs.append((f"blocks.{i}", [
                ("wqkv", [g.q_proj.weight, g.k_proj.weight, g.v_proj.weight]), ("wo", [g.o_proj.weight]),
                ("wgu", [f.gate_proj.weight, f.up_proj.weight]), ("wd", [f.down_proj.weight])]))
        root = [("emb", [model.token_emb.weight])]
        if model.lm_head.weight is not model.token_emb.weight:
            root.append(("head", [model.lm_head.weight]))
        specs.append(("root", root))
        matrix_params = {p for _, mats in specs for _, ps in mats for p in ps}
        self.gains = [p for p in model.parameters() if p.requires_grad and p not in matrix_params]
        assert all(p.dim() == 1 for p in self.gains), "every parameter that is not a matrix must be a norm gain"
        n_gain = sum(p.numel() for p in self.gains)
        total = sum(p.numel() for p in matrix_params)
        need = total * 6 + (len(specs) * 8 + 4) * 256 + (n_gain + 64) * 4 + 4096
        self.comm = SymmComm(mesh.get_group(shard_dim), self.rank, self.world, staging_bytes=4096,
                             persistent_bytes=need, wait_limit_s=wait_limit_s)
        self.units: list[_Unit] = []
        for ui, (uname, mats) in enumerate(specs):
            ms = [_Matrix(f"{uname}.{mn}", [(names[p], p) for p in ps], self.comm, self.rank, self.world)
                  for mn, ps in mats]
            self.units.append(_Unit(ui, uname, ms))
        self.gain_flat = self.comm.alloc((n_gain + 63) // 64 * 64, torch.float32)
        self.gain_flat.zero_()
        self._gain_view: dict[torch.Tensor, torch.Tensor] = {}
        at = 0
        for p in self.gains:
            self._gain_view[p] = self.gain_flat[at:at + p.numel()].view_as(p)
            at += p.numel()
        self.gain_pending = len(self.gains)
        self.gain_reduced: torch.cuda.Event | None = None
        self.partials = self.comm.partials(len(self.units) + 1)
        self.partials.zero_()
        self._unit_of = {p: u for u in self.units for p in u.params}
        self._matrix_of = {p: m for u in self.units for m in u.mats for p in m.params}
        self._written: set[int] = set()
        self._launched = 0
        self.stream = torch.cuda.Stream(device=dev, priority=-1)
        # ---- hand the engine the whole bf16 copies; free the unsharded fp32 masters ---------------------------
        for layer, u in zip(eng.layers, self.units):
            layer.wqkv, layer.wo, layer.wgu, layer.wd = (m.full_w for m in u.mats)
        root_unit = self.units[-1]
        eng.emb_shadow = root_unit.mats[0].full_w
        eng.head_shadow = root_unit.mats[-1].full_w
        eng.external_shadows = True       # the shadows are maintained here (AdamW on the shards + all-gather)
        eng.bf16_embedding = True         # the fp32 table exists only in shards: look tokens up in the bf16 copy
        eng.pre_block = self.wait_gathered
        self._empty = torch.empty(0, device=dev)
        for p in matrix_params:
            p.data = self._empty
        model.set_grad_sink(self)
        self._stale = True                # the peers' rows of the bf16 copies are not filled in yet
        self._shadowed = False
        self._fresh: set[int] = set()

    # -- what the trainer needs -------------------------------------------------------------------------------
    def optimizer_params(self) -> list[nn.Parameter]:
        """fp32 master shards (2-D: weight decay applies) followed by the replicated gains (1-D)."""
        return [m.shard for u in self.units for m in u.mats] + list(self.gains)

    def attach_shadows(self, optimizer) -> None:
        """Let the fused AdamW kernel write this rank's rows of the bf16 compute copies while it updates the shards."""
        if hasattr(optimizer, "attach_shadow"):
            self._shadowed = True
            for u in self.units:
                for m in u.mats:
                    optimizer.attach_shadow(m.shard, m.shard_w)

    def mark_updated(self) -> None:
        """The shards changed (optimizer step, checkpoint load): the next forward must gather again."""
        self._stale = True

    def begin_step(self) -> None:
        """Launch the in-place all-gather of every unit on the communication stream, root first, then the blocks in
        forward order; the compute stream waits per unit (``wait_gathered``)."""
        if not self._stale:
            return
        cur = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(cur)
        order = [self.units[-1]] + self.units[:-1]
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            for u in order:
                if not self._shadowed:   # an optimizer without the shadow hook leaves the bf16 rows stale: recast
                    for m in u.mats:
                        m.shard_w.copy_(m.shard.detach())
                self.comm.all_gather_inplace_([m.full_w for m in u.mats], blocks=self.comm_sms)
                u.gathered.record(self.stream)
        self._stale = False
        self._fresh = {u.index for u in self.units}   # units whose gather the compute stream has not waited for yet

    def wait_gathered(self, block_index: int) -> None:
        """Called by the engine before block `block_index` (or -1: embedding / head) reads its weights."""
        u = self.units[block_index]
        if u.index in self._fresh:
            torch.cuda.current_stream().wait_event(u.gathered)
            self._fresh.discard(u.index)

    # -- gradient sink protocol of the engine -----------------------------------------------------------------
    def grad_dest(self, p: torch.Tensor) -> tuple[torch.Tensor, bool]:
        m = self._matrix_of.get(p)
        view = m.grad_views[p] if m is not None else self._gain_view[p]
        # no wait needed before the first write of a step: sync() made the compute stream wait for last step's
        # reduce-scatter, whose closing handshake means no peer reads this buffer any more
        return view, id(p) in self._written

    def grad_written(self, p: torch.Tensor) -> None:
        self._written.add(id(p))
        u = self._unit_of.get(p)
        if u is None:
            self.gain_pending -= 1
            if self.gain_pending == 0:
                self.gain_pending = len(self.gains)
                self._reduce_gains()
            return
        u.pending -= 1
        if u.pending == 0:
            u.pending = len(u.params)
            self._reduce_unit(u)

    def absorb(self, p) -> bool:   # DDP-hook compatibility: every gradient arrives through the sink here
        return False

    def _reduce_unit(self, u: _Unit) -> None:
        if not self.requires_sync:
            return
        ready = torch.cuda.Event()
        ready.record()
        last = u.index == len(self.units) - 1      # the root unit finishes last and has the GPU to itself
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            self.comm.reduce_scatter_symmetric([m.full_g for m in u.mats], [m.shard_grad for m in u.mats], "avg",
                                               sq_slot=u.index, blocks=self.comm.blocks if last else self.comm_sms)
            if self.replicate_dim is not None and self.mesh.size(self.replicate_dim) > 1:
                for m in u.mats:
                    all_reduce(m.shard_grad, self.mesh, self.replicate_dim, "avg")
            u.reduced = torch.cuda.Event()
            u.reduced.record(self.stream)
        for m in u.mats:
            m.shard.grad = m.shard_grad
        self._launched += 1

    def _reduce_gains(self) -> None:
        if not self.requires_sync:
            return
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            self.comm.all_reduce_symmetric_(self.gain_flat, "avg", sq_slot=len(self.units), blocks=4)
            if self.replicate_dim is not None and self.mesh.size(self.replicate_dim) > 1:
                all_reduce(self.gain_flat, self.mesh, self.replicate_dim, "avg")
            self.gain_reduced = torch.cuda.Event()
            self.gain_reduced.record(self.stream)
        for p in self.gains:
            p.grad = self._gain_view[p]
        self._launched += 1

    def sync(self) -> None:
        """Wait for every unit's reduce-scatter; fails loudly when a unit never filled."""
        want = len(self.units) + 1
        if self._launched != want:
            raise AssertionError(f"only {self._launched}/{want} gradient units were reduced: a parameter got no "
                                 "gradient in this backward, or requires_sync was still False on the last micro-batch")
        cur = torch.cuda.current_stream()
        for u in self.units:
            cur.wait_event(u.reduced)
        cur.wait_event(self.gain_reduced)
        self._launched = 0
        self._written.clear()

    def sq_norm(self) -> torch.Tensor:
        """Global sum of squares of the reduced gradients (every rank's shards plus the gains), bit-identical on all
        ranks of the shard axis.  With HSDP the replicate all-reduce comes after the partials were taken, so the sum is
        recomputed from the final shard gradients."""
        if self.replicate_dim is not None and self.mesh.size(self.replicate_dim) > 1:
            from torchure_b200.ops import multi_tensor

            sq = multi_tensor.sq_norm([m.shard_grad for u in self.units for m in u.mats])
            all_reduce(sq, self.mesh, self.shard_dim, "sum")
            return sq + multi_tensor.sq_norm([self.gain_flat])
        # every rank published the sum of squares of the rows (units) or of the slice (gains) IT reduced: the whole
        # table adds up to the global norm, in the same order on every rank
        return self.partials.sum()

    @property
    def clip_shard_dims(self) -> tuple[str, ...]:
        return (self.shard_dim,)

    # -- state ---------------------------------------------------------------------------------------------------
    def full_state_dict(self) -> dict[str, torch.Tensor]:
        """Unsharded fp32 state under the model's own keys (collective over the shard axis)."""
        sd = {}
        for u in self.units:
            for m in u.mats:
                whole = all_gather(m.shard.detach().contiguous(), self.mesh, self.shard_dim, gather_dim=0)
                at = 0
                for name, p_rows in zip(m.names, [v.shape[0] for v in m.grad_views.values()]):
                    sd[name] = whole[at:at + p_rows].clone()
                    at += p_rows
        names = {p: n for n, p in self.model.named_parameters()}
        for p in self.gains:
            sd[names[p]] = p.detach().clone()
        if self.model.lm_head.weight is self.model.token_emb.weight:
            sd["lm_head.weight"] = sd["token_emb.weight"]
        return sd

    def load_full_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        names = {p: n for n, p in self.model.named_parameters()}
        with torch.no_grad():
            for u in self.units:
                for m in u.mats:
                    whole = torch.cat([sd[n].to(m.shard.device, torch.float32) for n in m.names], dim=0)
                    lo = self.rank * m.per
                    m.shard.copy_(whole[lo:lo + m.per])
                    m.shard_w.copy_(m.shard)
            for p in self.gains:
                p.copy_(sd[names[p]].to(p.device))
        self.mark_updated()

    def shard_state_dict(self) -> dict[str, torch.Tensor]:
        return {m.name: m.shard.detach() for u in self.units for m in u.mats}

    def load_shard_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            for u in self.units:
                for m in u.mats:
                    m.shard.copy_(sd[m.name].to(m.shard.device))
                    m.shard_w.copy_(m.shard)
        self.mark_updated()
