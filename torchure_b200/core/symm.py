"""Symmetric memory communicator: the transport under the sm_100a collectives.

One ``SymmComm`` per mesh axis group.  It owns a symmetric allocation (every rank of the group maps
every other rank's copy, plus an NVSwitch multicast mapping when the fabric offers one), laid out as::

    [ flags 64 KiB | sum-of-squares partials 1 MiB | persistent region (DDP buckets) | staging area ]

The bootstrap (allocation, handle exchange, peer and multicast mapping) uses
``torch.distributed._symmetric_memory``; every byte moved afterwards is moved by the kernels of
``csrc/comm.cu`` (plain peer loads/stores or ``multimem`` instructions), never by NCCL.

Generic collectives on ordinary tensors stage through the staging area (one local copy in, one out).
Tensors allocated with ``alloc()`` live inside the symmetric region and are reduced in place.
Variant choice per call: one-shot reads for small all-reduces (<= 256 KiB), two-shot
(reduce-scatter + broadcast) above; ``multimem`` when a multicast mapping exists and the op is a sum/avg.

Set ``TORCHURE_B200_NVLS=0`` to keep every kernel on plain peer loads/stores.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from torchure_b200 import ops

_DEBUG = os.environ.get("TORCHURE_B200_DEBUG", "0") == "1"
_OPS = {"sum": 0, "avg": 1, "max": 2, "min": 3}
_DT = {torch.float32: 0, torch.bfloat16: 1}
ONESHOT_BYTES = 256 * 1024


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class SymmComm:
    def __init__(self, group, rank: int, world: int, staging_bytes: int = 64 << 20, persistent_bytes: int = 0,
                 wait_limit_s: float = 30.0, blocks: int = 128):
        import torch.distributed._symmetric_memory as symm_mem

        ext = ops.ext()
        self.ext = ext
        self.group, self.rank, self.world = group, rank, world
        self.blocks = min(blocks, ext.COMM_MAX_BLOCKS)
        self.header = ext.COMM_FLAG_BYTES + ext.COMM_PARTIAL_BYTES
        self.persistent_bytes = _align(persistent_bytes, 4096)
        self.staging_bytes = _align(staging_bytes, 4096)
        total = self.header + self.persistent_bytes + self.staging_bytes
        dev = torch.device("cuda", torch.cuda.current_device())
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.peers = [int(p) for p in self.handle.buffer_ptrs]
        assert self.peers[rank] == self.buf.data_ptr(), "symmetric allocation does not start at the tensor"
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)  # 0 when the fabric offers no multicast mapping
        if os.environ.get("TORCHURE_B200_NVLS", "1") == "0":
            mc = 0
        self.mc = mc
        self.limit_ns = int(wait_limit_s * 1e9)
        self._persist_at = 0
        self.staging_off = self.header + self.persistent_bytes
        torch.cuda.synchronize()
        dist.barrier(group=group)  # every rank's flags are zero before the first kernel touches them

    # -- helpers ---------------------------------------------------------------------------------
    def _ctx(self):
        return self.peers, self.mc, self.rank, self.world, self.limit_ns

    def _check_range(self, off: int, nbytes: int, what: str) -> None:
        """Debug build of the launchers (``TORCHURE_B200_DEBUG=1``): every byte range a kernel will touch in the
        symmetric allocation must lie inside it, past the flag and partial tables, and start on a 16-byte boundary.
        A bad range is refused here instead of becoming a stray store into a peer's memory."""
        if not _DEBUG:
            return
        total = self.buf.numel()
        if off % 16 != 0 or nbytes < 0 or off < self.header or off + nbytes > total:
            raise AssertionError(f"{what}: bytes [{off}, {off + nbytes}) outside the data area [{self.header}, {total}) "
                                 f"of the symmetric allocation, or misaligned (rank {self.rank})")

    def supports(self, t: torch.Tensor, copies: int = 1) -> bool:
        """True when `t` can go through the kernels; `copies` = staging bytes needed per byte of `t`."""
        ok = t.is_cuda and t.dtype in _DT and t.is_contiguous() and t.numel() > 0
        return ok and (copies == 1 or t.numel() * t.element_size() * copies + 4096 <= self.staging_bytes)

    def _pieces(self, t: torch.Tensor):
        """Flat views of `t` no larger than the staging area (elementwise collectives are chunkable)."""
        flat = t.view(-1)
        step = max(1, (self.staging_bytes - 256) // t.element_size() // 8 * 8)
        for lo in range(0, flat.numel(), step):
            yield flat[lo:lo + step]

    def _staging(self, nbytes: int, dtype, at: int = 0) -> torch.Tensor:
        lo = self.staging_off + at
        self._check_range(lo, nbytes, "staging area")
        assert at + nbytes <= self.staging_bytes, (
            f"message of {nbytes} bytes exceeds the {self.staging_bytes}-byte staging area of this communicator")
        return self.buf[lo:lo + nbytes].view(dtype)

    def offset_of(self, t: torch.Tensor) -> int | None:
        """Byte offset of `t` inside the symmetric allocation, or None if it lives elsewhere."""
        off = t.data_ptr() - self.buf.data_ptr()
        if 0 <= off and off + t.numel() * t.element_size() <= self.buf.numel():
            return off
        return None

    def alloc(self, numel: int, dtype=torch.float32) -> torch.Tensor:
        """Persistent tensor inside the symmetric region (same offset on every rank: call in the same order)."""
        nbytes = _align(numel * torch.empty((), dtype=dtype).element_size(), 256)
        assert self._persist_at + nbytes <= self.persistent_bytes, "persistent symmetric region exhausted"
        lo = self.header + self._persist_at
        self._persist_at += nbytes
        return self.buf[lo:lo + numel * torch.empty((), dtype=dtype).element_size()].view(dtype)

    def partials(self, n_slots: int) -> torch.Tensor:
        """(n_slots, MAX_RANKS * MAX_BLOCKS) fp32 view of the sum-of-squares table."""
        per = self.ext.COMM_MAX_RANKS * self.ext.COMM_MAX_BLOCKS
        lo = self.ext.COMM_FLAG_BYTES
        assert n_slots * per * 4 <= self.ext.COMM_PARTIAL_BYTES
        return self.buf[lo:lo + n_slots * per * 4].view(torch.float32).view(n_slots, per)

    def check(self) -> None:
        word = self.ext.comm_error_word()
        code = int(word[0].item())
        if code:
            word.zero_()
            raise RuntimeError(f"a collective gave up waiting for a peer flag (code {code}, rank {self.rank})")

    # -- collectives -----------------------------------------------------------------------------
    def all_reduce_symmetric_(self, t: torch.Tensor, op: str = "sum", sq_slot: int = -1, blocks: int | None = None):
        """In-place two-shot all-reduce of a tensor that lives in the symmetric region."""
        off = self.offset_of(t)
        assert off is not None and off % 16 == 0 and (t.numel() * t.element_size()) % 16 == 0
        self._check_range(off, t.numel() * t.element_size(), "all_reduce_symmetric_")
        use_mc = bool(self.mc) and op in ("sum", "avg")
        self.ext.comm_all_reduce(*self._ctx(), off, t.numel(), _DT[t.dtype], _OPS[op], use_mc, sq_slot,
                                 blocks or self.blocks)
        ops.count_launch()

    def all_gather_inplace_(self, fulls: list[torch.Tensor], blocks: int | None = None) -> None:
        """Each tensor of `fulls` lives in the symmetric region and is `world` equal row chunks; this rank's chunk
        (already written locally) is replicated into every peer's copy.  One kernel, no staging, no copy-out."""
        offs, sizes = [], []
        for t in fulls:
            off = self.offset_of(t)
            nbytes = t.numel() * t.element_size()
            assert off is not None and t.is_contiguous() and nbytes % (16 * self.world) == 0 and off % 16 == 0
            self._check_range(off, nbytes, "all_gather_inplace_")
            offs.append(off)
            sizes.append(nbytes // self.world)
        for lo in range(0, len(offs), self.ext.COMM_MAX_SEGMENTS):
            hi = lo + self.ext.COMM_MAX_SEGMENTS
            self.ext.comm_all_gather_inplace(*self._ctx(), offs[lo:hi], sizes[lo:hi], bool(self.mc) and self.world > 2,
                                             blocks or self.blocks)
            ops.count_launch()

    def reduce_scatter_symmetric(self, fulls: list[torch.Tensor], outs: list[torch.Tensor], op: str = "avg",
                                 sq_slot: int = -1, blocks: int | None = None) -> None:
        """outs[i] (local fp32, 1/world of fulls[i]) = op over ranks of this rank's row chunk of fulls[i], which lives
        in the symmetric region.  One kernel; the peers' copies are read in place."""
        assert len(fulls) == len(outs) <= self.ext.COMM_MAX_SEGMENTS
        offs = []
        for t, o in zip(fulls, outs):
            off = self.offset_of(t)
            assert off is not None and t.dtype == torch.float32 and t.numel() == o.numel() * self.world
            self._check_range(off, t.numel() * 4, "reduce_scatter_symmetric")
            offs.append(off)
        use_mc = bool(self.mc) and op in ("sum", "avg")
        self.ext.comm_reduce_scatter_symm(*self._ctx(), offs, outs, _OPS[op], use_mc, sq_slot, blocks or self.blocks)
        ops.count_launch()

    # generic collectives on ordinary tensors: ONE kernel each; the staging area is only the exchange medium
    def _aligned(self, *ts: torch.Tensor) -> bool:
        return all(t.data_ptr() % 16 == 0 and (t.numel() * t.element_size()) % 16 == 0 for t in ts)

    def _grid(self, nbytes: int) -> int:
        """CTAs for a message: one per 8 KiB (a 512-thread CTA moves 8 KiB per pass of 16-byte accesses), so that a
        64 KiB - 512 KiB one-shot all-reduce is spread over 8 - 64 CTAs instead of crawling through one."""
        return max(1, min(self.blocks, (nbytes + 8191) // 8192))

    def all_reduce_(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        nbytes = t.numel() * t.element_size()
        if self.offset_of(t) is not None and self._aligned(t):
            self.all_reduce_symmetric_(t, op)
            return t
        if nbytes > self.staging_bytes - 256:
            for piece in self._pieces(t):
                self.all_reduce_(piece, op)
            return t
        if not self._aligned(t):  # odd sizes: pad through a temporary
            pad = torch.zeros(_align(nbytes, 16) // t.element_size(), dtype=t.dtype, device=t.device)
            pad[: t.numel()].copy_(t.view(-1))
            self.all_reduce_(pad, op)
            t.view(-1).copy_(pad[: t.numel()])
            return t
        oneshot = nbytes <= ONESHOT_BYTES
        use_mc = bool(self.mc) and op in ("sum", "avg") and not oneshot
        self.ext.comm_all_reduce_fused(*self._ctx(), self.staging_off, t, t, t.numel(), _DT[t.dtype], _OPS[op], use_mc,
                                       oneshot, self._grid(nbytes))
        ops.count_launch()
        return t

    def broadcast_(self, t: torch.Tensor, src: int) -> torch.Tensor:
        nbytes = t.numel() * t.element_size()
        if nbytes > self.staging_bytes - 256:
            for piece in self._pieces(t):
                self.broadcast_(piece, src)
            return t
        if not self._aligned(t):
            pad = torch.zeros(_align(nbytes, 16) // t.element_size(), dtype=t.dtype, device=t.device)
            pad[: t.numel()].copy_(t.view(-1))
            self.broadcast_(pad, src)
            t.view(-1).copy_(pad[: t.numel()])
            return t
        self.ext.comm_broadcast(*self._ctx(), self.staging_off, t, t.numel(), _DT[t.dtype], src, bool(self.mc),
                                self._grid(nbytes))
        ops.count_launch()
        return t

    def _padded(self, t: torch.Tensor, rows: int):
        """(contiguous 16-byte-padded copy of t viewed (rows, n), n, padded n) for chunked collectives."""
        es = t.element_size()
        n = t.numel() // rows
        pn = _align(n * es, 16) // es
        if pn == n and t.data_ptr() % 16 == 0:
            return t.view(rows, n), n, pn
        buf = torch.zeros(rows, pn, dtype=t.dtype, device=t.device)
        buf[:, :n].copy_(t.view(rows, n))
        return buf, n, pn

    def all_gather(self, src: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        s2, n, pn = self._padded(src, 1)
        direct = pn == n and out.data_ptr() % 16 == 0
        dst = out.view(self.world, n) if direct else torch.empty(self.world, pn, dtype=src.dtype, device=src.device)
        self._staging(pn * self.world * src.element_size(), src.dtype)  # bounds check
        self.ext.comm_all_gather(*self._ctx(), self.staging_off, s2, dst, pn, _DT[src.dtype], bool(self.mc),
                                 self._grid(pn * src.element_size()))
        ops.count_launch()
        if not direct:
            out.view(self.world, n).copy_(dst[:, :n])
        return out

    def reduce_scatter(self, src: torch.Tensor, out: torch.Tensor, op: str = "sum") -> torch.Tensor:
        s2, n, pn = self._padded(src, self.world)
        direct = pn == n and out.data_ptr() % 16 == 0
        dst = out.view(-1) if direct else torch.empty(pn, dtype=src.dtype, device=src.device)
        self._staging(pn * self.world * src.element_size(), src.dtype)
        use_mc = bool(self.mc) and op in ("sum", "avg")
        self.ext.comm_reduce_scatter(*self._ctx(), self.staging_off, s2, dst, pn, _DT[src.dtype], _OPS[op], use_mc,
                                     self._grid(pn * src.element_size()))
        ops.count_launch()
        if not direct:
            out.view(-1).copy_(dst[:n])
        return out

    def all_to_all(self, src: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        s2, n, pn = self._padded(src, self.world)
        direct = pn == n and out.data_ptr() % 16 == 0
        dst = out.view(self.world, n) if direct else torch.empty(self.world, pn, dtype=src.dtype, device=src.device)
        self._staging(pn * self.world * src.element_size(), src.dtype)
        self.ext.comm_all_to_all(*self._ctx(), self.staging_off, s2, dst, pn, _DT[src.dtype],
                                 self._grid(pn * src.element_size()))
        ops.count_launch()
        if not direct:
            out.view(self.world, n).copy_(dst[:, :n])
        return out

    def barrier(self, pretend_world: int | None = None, phase: int = 0) -> None:
        """Cross-rank barrier on the current stream.  `phase` selects the flag row (0/1: collectives, 4/6: fused GEMMs;
        2/3 are for barriers that may overlap a collective running on another stream)."""
        self.ext.comm_barrier(*self._ctx(), pretend_world or self.world, phase)
        ops.count_launch()
