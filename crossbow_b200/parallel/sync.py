"""Model synchronisation back ends.

``FusedSynchroniser``     - the product: one persistent sm_100a kernel per GPU per clock (csrc/kernels/sync.cu) that
                            reduces the replicas, exchanges partial sums through peer-mapped memory over NVLink,
                            updates the central average model and corrects / overwrites the replicas.
``ReferenceSynchroniser`` - the bar: the reference's sequence restated step by step - per-replica difference / axpy
                            kernels, ``all_reduce`` (NCCL), central update, per-replica correction
                            (clib-multigpu/synch/sma.c:13-231, synch/common.c:3-57, synch/synchronoussgd.c:13-110).
Both implement ``synchronise(algo, ...)`` over the same flat device vectors and are interchangeable.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from ..ops import lib as L
from .peer import PeerBuffer

ALGO_SMA, ALGO_SSGD, ALGO_POLYAK = 0, 1, 2


class SyncTimeout(RuntimeError):
    """A bounded device-side wait on a peer expired (the peer is late, gone, or never joined)."""


class _PeerView:
    """A window of another PeerBuffer (same mapping, moved by `offset_bytes`); owns nothing."""

    def __init__(self, buf: PeerBuffer, offset_bytes: int):
        self.ptrs = [p + offset_bytes for p in buf.ptrs]
        self.local = buf.local + offset_bytes

    def close(self):
        pass


class _MulticastBuffer:
    """A buffer of ``numel`` floats on every rank that is ALSO bound to an NVLink multicast object, so kernels can address
    all copies at once with ``multimem`` instructions (``mc``) next to the ordinary peer pointers (``ptrs``).  Allocation,
    the exchange of handles between the processes and the multicast binding are torch's symmetric memory
    (``torch.distributed._symmetric_memory``); the kernels that use the addresses are this repository's."""

    def __init__(self, numel: int, rank: int, world: int, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.tensor = symm.empty(int(numel), dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
        self.tensor.zero_()
        self.handle = symm.rendezvous(self.tensor, group if group is not None else dist.group.WORLD)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.local = self.ptrs[rank]
        self.mc = int(self.handle.multicast_ptr or 0)
        torch.cuda.synchronize()
        dist.barrier(group)

    def as_tensor(self, numel: int, device=None) -> torch.Tensor:
        return self.tensor[:numel]

    def close(self):
        self.handle = None
        self.tensor = None


class FusedSynchroniser:
    def __init__(self, n: int, rank: int = 0, world: int = 1, two_shot: Optional[bool] = None, timeout_s: float = 5.0,
                 max_blocks: int = 0, group=None, parent: Optional["FusedSynchroniser"] = None, offset: int = 0, nvls: bool = False):
        """`nvls`: two-shot exchange through NVLink multicast (in-switch reduction with ``multimem.ld_reduce``, broadcast of
        the new central model with ``multimem.st``) instead of unicast peer stores.  Off by default; falls back to the
        peer-store path (with a warning) where the GPUs or the driver offer no multicast.
        `parent` / `offset`: this synchroniser covers elements [offset, offset + n) of the parent's vectors (a gradient
        bucket).  It has exchange buffers and flags of its own, so buckets of different sizes never share a flag slot or
        an inbox region, and it shares the parent's status word and central-model storage."""
        lib = L.load()
        self.lib, self.n, self.rank, self.world = lib, n, rank, world
        if n % 4:
            raise ValueError("flat vector length must be a multiple of 4")
        self.two_shot = bool(two_shot) if two_shot is not None else (n * 4 >= (8 << 20))
        self.timeout_s, self.max_blocks = timeout_s, max_blocks
        self.epoch = 0
        self.args_dev = lib.xb_device_alloc(lib.xb_sync_args_size())
        self.args_size = (lib.xb_sync_args_size() + 255) // 256 * 256
        self.args_pinned = lib.xb_pinned_alloc(8 * self.args_size)    # ring: an upload may still be pending when the next is built
        self.status = parent.status if parent is not None else torch.zeros(1, dtype=torch.int32, device="cuda")
        self.parent, self.offset, self.group = parent, offset, group
        self.children: List["FusedSynchroniser"] = []
        self.inbox = self.result = self.flags = self.zbuf = self.part = None
        self.nvls = False
        # release word + block counter, and the kernel's time line (see sync.cu): plain device memory of this rank
        self.release = torch.zeros(2, dtype=torch.int32, device="cuda")
        self.stamps = torch.zeros(lib.xb_sync_stamp_words(), dtype=torch.int64, device="cuda")
        if world > 1:
            self.inbox = PeerBuffer(4 * lib.xb_sync_inbox_floats(n, world, int(self.two_shot)), rank, world, group)
            self.result = PeerBuffer(4 * lib.xb_sync_result_floats(n) if self.two_shot else 256, rank, world, group)
            self.flags = PeerBuffer(4 * lib.xb_sync_flag_words(n, world), rank, world, group)
            if self.two_shot and parent is not None:
                self.zbuf = _PeerView(parent.zbuf, 4 * offset) if parent.zbuf is not None else None
            elif self.two_shot and nvls:
                try:
                    zb = _MulticastBuffer(n, rank, world, group)
                    pb = _MulticastBuffer(lib.xb_sync_part_floats(n), rank, world, group)
                    if not zb.mc or not pb.mc:
                        raise RuntimeError("no multicast address")
                    self.zbuf, self.part, self.nvls = zb, pb, True
                except Exception as e:           # no NVLink multicast here: the peer-store path does the same job
                    import warnings
                    warnings.warn(f"NVLS synchronisation is not available ({type(e).__name__}: {e}); using peer stores")
                    self.zbuf = PeerBuffer(4 * n, rank, world, group)
            elif self.two_shot:
                # peer-visible home for the central model: chunk owners then store the updated model straight into it
                self.zbuf = PeerBuffer(4 * n, rank, world, group)
        if world > 1 and parent is None:
            # every rank has mapped every peer's buffers before anyone launches a kernel that waits on a peer: mapping
            # can take seconds on one rank and milliseconds on another, more than a bounded device wait allows
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group)

    def make_buckets(self, ranges) -> List["FusedSynchroniser"]:
        """One child synchroniser per (offset, elements) range, in the given order (collective: every rank must pass the
        same ranges).  The children replace this synchroniser for the algorithm that is run bucket by bucket."""
        for c in self.children:
            c.close()
        self.children = [FusedSynchroniser(ln, self.rank, self.world, self.two_shot, self.timeout_s, self.max_blocks, self.group,
                                           parent=self, offset=off) for off, ln in ranges]
        return self.children

    def central_storage(self) -> Optional[torch.Tensor]:
        """Peer-visible tensor to keep the central model in (None when the exchange does not use one)."""
        return self.zbuf.as_tensor(self.n) if self.zbuf is not None else None

    @property
    def owner_apply(self) -> bool:
        return self.zbuf is not None

    def gather_momentum(self, zlast: torch.Tensor) -> torch.Tensor:
        """The central model's momentum vector in full.  With owner-apply every rank only maintains the chunks it owns
        (chunk c belongs to rank c mod world); this call is collective."""
        if not self.owner_apply:
            return zlast
        import torch.distributed as dist
        if self.children:                     # bucket by bucket: ownership follows each bucket's own chunking
            owner = torch.empty(self.n, dtype=torch.int64, device=zlast.device)
            for c in self.children:
                chunk = int(self.lib.xb_sync_chunk(c.n))
                owner[c.offset:c.offset + c.n] = (torch.arange(c.n, device=zlast.device) // chunk) % self.world
        else:
            chunk = int(self.lib.xb_sync_chunk(self.n))
            owner = (torch.arange(self.n, device=zlast.device) // chunk) % self.world
        full = torch.where(owner == self.rank, zlast, torch.zeros_like(zlast))
        dist.all_reduce(full)
        return full

    def descriptor(self, algo, replicas_w, replicas_prev, z, zlast, gacc, alpha, mu, scale, blend, copy, use_prev) -> L.XbSyncDesc:
        d = L.XbSyncDesc()
        d.rank, d.G, d.k, d.algo, d.n = self.rank, self.world, len(replicas_w), algo, self.n
        d.epoch = self.epoch
        d.two_shot, d.copy_to_replicas, d.use_prev = int(self.two_shot), int(copy), int(use_prev)
        d.alpha, d.mu, d.scale, d.blend = alpha, mu, scale, blend
        for i, w in enumerate(replicas_w):
            d.w[i] = w.data_ptr()
            d.prev[i] = replicas_prev[i].data_ptr() if replicas_prev is not None else w.data_ptr()
        d.z, d.zlast = z.data_ptr(), zlast.data_ptr()
        d.gacc = gacc.data_ptr() if gacc is not None else 0
        if self.world > 1:
            for g in range(self.world):
                d.inbox[g], d.result[g], d.flags[g] = self.inbox.ptrs[g], self.result.ptrs[g], self.flags.ptrs[g]
            if self.zbuf is not None and z.data_ptr() == self.zbuf.local:
                for g in range(self.world):
                    d.zpeer[g] = self.zbuf.ptrs[g]
                if self.nvls:
                    d.part_local, d.part_mc, d.z_mc = self.part.local, self.part.mc, self.zbuf.mc
        d.status = self.status.data_ptr()
        d.timeout_s = self.timeout_s
        d.release, d.stamps = self.release.data_ptr(), self.stamps.data_ptr()
        return d

    def releases_early(self, algo: int, copy: bool) -> bool:
        """True when the kernel publishes the release word BEFORE the exchange: model averaging that does not overwrite
        the replicas, on more than one GPU (a replica is then final once it has been corrected against the old central
        model; everything after that only touches the central model)."""
        return algo == ALGO_SMA and not copy and self.world > 1

    def wait_release(self, stream: int):
        """Make `stream` wait until the replicas of the last enqueued synchronisation have been released."""
        L.check(self.lib.xb_stream_wait_value32(stream, self.release.data_ptr(), self.epoch & 0xFFFFFFFF), "wait for the release word")

    def timeline(self, reset: bool = False) -> dict:
        """Device-side time line of this rank's synchronisations (call after the stream has been synchronised): number of
        launches, mean microseconds from kernel entry to the release of the replicas and from entry to the exit of the
        last block."""
        st = [int(v) for v in self.stamps.cpu().tolist()]
        entry, release, count, sum_rel, sum_tot = st[0], st[1], st[4], st[5], st[6]
        exit_ = st[2 + (self.epoch & 1)]
        if entry and exit_ >= entry:                      # the most recent launch has not been folded into the sums yet
            count, sum_rel, sum_tot = count + 1, sum_rel + ((release if release >= entry else exit_) - entry), sum_tot + (exit_ - entry)
        if reset:
            self.stamps.zero_()
        return {"launches": count, "release_us": sum_rel / max(1, count) / 1e3, "total_us": sum_tot / max(1, count) / 1e3}

    def synchronise(self, stream: int, algo: int, replicas_w: List[torch.Tensor], replicas_prev: Optional[List[torch.Tensor]],
                    z, zlast, gacc=None, alpha=0.0, mu=0.0, scale=1.0, blend=0.0, copy=False, use_prev=True):
        """Enqueue one synchronisation on ``stream`` (a raw cudaStream_t). Asynchronous; see ``check``."""
        self.epoch += 1
        d = self.descriptor(algo, replicas_w, replicas_prev, z, zlast, gacc, alpha, mu, scale, blend, copy, use_prev)
        self.launches = getattr(self, "launches", 0) + 1
        staging = self.args_pinned + (self.launches % 8) * self.args_size
        L.check(self.lib.xb_fused_sync(C.byref(d), self.args_dev, staging, self.max_blocks, stream), "fused sync")

    def check(self):
        """Host-side check of the device status word (call after the stream has been synchronised)."""
        s = int(self.status.item())
        if s != 0:
            self.status.zero_()
            raise SyncTimeout(f"fused synchronisation gave up waiting for a peer (status {s}, epoch {self.epoch})")

    def close(self):
        for c in self.children:
            c.close()
        self.children = []
        for b in (self.inbox, self.result, self.flags, self.zbuf, self.part):
            if b is not None:
                b.close()
        self.lib.xb_device_free(self.args_dev)
        self.lib.xb_pinned_free(self.args_pinned)


class ReferenceSynchroniser:
    """Reference-style synchronisation with separate element-wise kernels (torch ops on the flat vectors) and a
    library all-reduce.  Used as the measured baseline and as a second implementation in tests."""

    def __init__(self, n: int, rank: int = 0, world: int = 1, group=None):
        self.n, self.rank, self.world, self.group = n, rank, world, group
        self.D = torch.zeros(n, device="cuda")
        self.G = torch.zeros(n, device="cuda")

    def _allreduce(self, t):
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, group=self.group)

    def synchronise(self, stream, algo, replicas_w, replicas_prev, z, zlast, gacc=None, alpha=0.0, mu=0.0, scale=1.0,
                    blend=0.0, copy=False, use_prev=True):
        s = torch.cuda.ExternalStream(stream) if isinstance(stream, int) and stream else torch.cuda.current_stream()
        with torch.cuda.stream(s):
            if algo == ALGO_SMA:
                self.G.zero_()
                for i, w in enumerate(replicas_w):
                    src = replicas_prev[i] if use_prev else w
                    torch.sub(src, z, out=self.D)            # D = r.diff - z
                    w.add_(self.D, alpha=-alpha)             # r -= alpha*D
                    self.G.add_(self.D, alpha=alpha)         # G += alpha*D
                self._allreduce(self.G)
                tot = self.G
            elif algo == ALGO_SSGD:
                self._allreduce(gacc)
                tot = gacc.mul(scale)
                gacc.zero_()
            else:
                self.G.zero_()
                for w in replicas_w:
                    self.G.add_(w)
                self._allreduce(self.G)
                z.add_(self.G.mul(scale).sub_(z), alpha=blend)
                if alpha > 0:
                    for w in replicas_w:
                        w.sub_((w - z).mul_(alpha))
                return
            if mu > 0:
                tot = tot.add(zlast, alpha=mu)
                zlast.copy_(tot)
            z.add_(tot)
            if copy or algo == ALGO_SSGD:
                for w in replicas_w:
                    w.copy_(z)

    def check(self):
        pass

    def close(self):
        pass
