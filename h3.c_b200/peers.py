"""Peer-addressable buffers for sequence parallelism with the exchange fused into the kernels.

One process per GPU. Every rank allocates its exchange buffers with h3x_peer_alloc, the
64-byte CUDA IPC handles travel over any host-side all-gather the caller supplies (e.g.
torch.distributed.all_gather_object), and each rank maps the others' buffers. The result is
the h3x_ulysses_peers table the push kernels take. No reference counterpart (the reference is
single-device)."""
from __future__ import annotations

import ctypes as C

from .binding import BF16, Gpu, H3Error, Tensor, UlyssesPeers

FLAG_BYTES = 64   # 16 x uint32 barrier words


class PeerExchange:
    """Exchange object for `Dit`: owns the symmetric q/k/v, output and flag buffers.

    all_gather(obj) -> list of every rank's obj, in rank order (a host-side collective)."""

    def __init__(self, gpu: Gpu, world: int, rank: int, all_gather, loopback: bool = False):
        """loopback=True is a measurement aid: every peer entry points at this rank's own
        buffers and the barriers are skipped, so a step moves the same bytes with no NVLink
        traffic and no waiting (results are meaningless); step time minus the loopback step
        time is the exposed cost of the exchange."""
        self.gpu, self.world, self.rank, self.loopback = gpu, world, rank, loopback
        self._all_gather = all_gather
        self._blocks: list[int] = []
        self._mapped: list[int] = []
        self.peers = UlyssesPeers()
        self.peers.world, self.peers.rank = world, rank

    def share(self, nbytes: int) -> list[int]:
        """Allocate nbytes here, return every rank's block as mapped in this process."""
        lib, gpu = self.gpu.lib, self.gpu
        handle = (C.c_ubyte * 64)()
        block = lib.h3x_peer_alloc(gpu.handle, nbytes, handle)
        problem = None if block else f"h3x_peer_alloc failed: {gpu.error()}"
        if block:
            self._blocks.append(block)
        if self.loopback:
            if problem:
                raise H3Error(problem)
            return [block] * self.world
        # every rank takes part in both host collectives whatever happened locally, and all
        # ranks fail together: nobody is left waiting in a collective
        handles = self._all_gather(bytes(handle) if block else None)
        out = []
        if problem is None and all(h is not None for h in handles):
            for r, h in enumerate(handles):
                if r == self.rank:
                    out.append(block)
                    continue
                mapped = lib.h3x_peer_open(gpu.handle, (C.c_ubyte * 64).from_buffer_copy(h))
                if not mapped:
                    problem = f"h3x_peer_open failed: {gpu.error()}"
                    break
                self._mapped.append(mapped)
                out.append(mapped)
        elif problem is None:
            problem = "a peer could not allocate its buffer"
        problems = [p for p in self._all_gather(problem) if p]
        if problems:
            raise H3Error("peer-mapped buffers unavailable: " + problems[0])
        return out

    def setup(self, rows_local: int, heads: int, head_dim: int) -> dict[str, Tensor]:
        """Buffers for one Dit: gathered q/k/v [world*rows_local][heads/world][head_dim], output
        [rows_local][heads][head_dim], flag words. Returns the local tensors."""
        n = rows_local * heads * head_dim
        self.peers.rows_local = rows_local
        local = {}
        for name in ("q", "k", "v", "o"):
            ptrs = self.share(n * 2)
            for r, p in enumerate(ptrs):
                getattr(self.peers, name)[r] = p
            local[name] = self.gpu.wrap(ptrs[self.rank], n, BF16)
        for r, p in enumerate(self.share(FLAG_BYTES)):
            self.peers.flags[r] = p
        return local

    def barrier(self) -> None:
        if not self.loopback:
            self.gpu.op("h3x_peer_barrier", self.peers)

    def close(self) -> None:
        lib, gpu = self.gpu.lib, self.gpu
        for m in self._mapped:
            lib.h3x_peer_close(gpu.handle, m)
        self._all_gather(b"closed")      # nobody frees while a peer still maps the block
        for b in self._blocks:
            lib.h3x_peer_free(gpu.handle, b)
        self._mapped, self._blocks = [], []
