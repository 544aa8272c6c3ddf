"""Exchange buffers shared by the GPUs of one node, and the one-kernel attention-partial merge
that runs over them (NVLink peer loads and stores instead of NCCL calls).

Each rank allocates one buffer of a common layout; the 64-byte CUDA IPC handles travel through
the process group once at start-up and every rank maps every peer's buffer.  After that the data
path makes no library call: kernels read and write peer memory directly.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib
from .kernels import check, ptr, status_word, stream_ptr


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class _Span:
    """Device memory owned elsewhere, exposed to torch through the CUDA array interface."""

    def __init__(self, address: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False),
                                         "version": 3, "strides": None}


class PeerBuffers:
    """One zeroed device buffer of `nbytes` per rank, mapped into every rank of `group`.

    local            uint8 tensor over this rank's buffer
    addresses[r]     device address of rank r's buffer in THIS process
    With emulate_world=n (single process, tests) the n buffers are n local allocations.

    The constructor is collective (one all-gather of the handles).  It raises on every rank when an
    allocation failed anywhere, and on the ranks that could not map a peer; the group must agree on
    the outcome (as SparseDecodeStep does with an all-reduce) before any rank launches a kernel on
    the buffers, and must synchronise (host barrier) before close().
    """

    def __init__(self, nbytes: int, device: torch.device, group=None, emulate_world: Optional[int] = None):
        lib = _lib.load()
        self.device = torch.device(device)
        self.nbytes = _align(nbytes)
        self._owned: List[int] = []
        self._opened: List[int] = []
        with torch.cuda.device(self.device):
            if emulate_world is not None:
                self.rank, self.world = 0, emulate_world
                self.addresses = [self._alloc(lib)[0] for _ in range(emulate_world)]
            else:
                self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
                # Every rank takes part in the one collective below whether or not its allocation
                # worked (first byte = valid), so that a local failure cannot leave the others waiting.
                mine, handle, err = None, bytes(64), None
                try:
                    mine, handle = self._alloc(lib)
                except _lib.B200DSAError as e:
                    err = e
                h = torch.tensor([0 if mine is None else 1] + list(handle), dtype=torch.uint8, device=self.device)
                gathered = torch.empty(self.world, 65, dtype=torch.uint8, device=self.device)
                dist.all_gather_into_tensor(gathered.view(-1), h, group=group)
                gathered = gathered.cpu()
                if not bool(gathered[:, 0].all()):
                    self.close()
                    raise _lib.B200DSAError(f"exchange buffer allocation failed on a rank of the group ({err})")
                self.addresses = []
                try:
                    for r in range(self.world):
                        if r == self.rank:
                            self.addresses.append(mine)
                            continue
                        raw = (ctypes.c_ubyte * 64)(*gathered[r, 1:].tolist())
                        out = ctypes.c_void_p()
                        check(lib.b200dsa_peer_open(raw, ctypes.byref(out)), "b200dsa_peer_open")
                        self._opened.append(out.value)
                        self.addresses.append(out.value)
                except _lib.B200DSAError:
                    # ranks on another node, or IPC not permitted: unmap what was mapped; the buffer of
                    # this rank stays allocated until close(), peers may still have it mapped
                    for a in self._opened:
                        lib.b200dsa_peer_close(ctypes.c_void_p(a))
                    self._opened = []
                    raise
        self.views = [torch.as_tensor(_Span(a, self.nbytes), device=self.device) for a in self.addresses]
        self.local = self.views[self.rank]
        self._addr_array = (ctypes.c_void_p * self.world)(*self.addresses)

    def _alloc(self, lib):
        out = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        check(lib.b200dsa_peer_alloc(self.nbytes, ctypes.byref(out), handle), "b200dsa_peer_alloc")
        self._owned.append(out.value)
        return out.value, bytes(handle)

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's own (call on every rank, after a barrier)."""
        lib = _lib.load()
        self.views, self.local = [], None
        self.addresses = []
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for a in self._opened:
                lib.b200dsa_peer_close(ctypes.c_void_p(a))
            for a in self._owned:
                lib.b200dsa_peer_free(ctypes.c_void_p(a))
        self._opened, self._owned = [], []


class PeerLseCombine:
    """Merge of key-sharded attention partials in one kernel over peer memory; see
    b200dsa_peer_lse_combine.  The attention kernel writes straight into `ctx` / `lse` (views of
    this rank's exchange buffer); after run() `out` / `lse_out` hold the merged result on every rank."""

    def __init__(self, n_rows: int, device: torch.device, group=None, emulate_world: Optional[int] = None,
                 extra_bytes: int = 0):
        """extra_bytes: room after the flags for other data the ranks read from each other (`extra`)."""
        self.n_rows = n_rows
        self.off_ctx = 0
        self.off_lse = _align(n_rows * 512 * 2)
        self.off_out = self.off_lse + _align(n_rows * 4)
        self.off_lse_out = self.off_out + _align(n_rows * 512 * 2)
        self.off_flags = self.off_lse_out + _align(n_rows * 4)
        self.off_extra = self.off_flags + 256
        self.extra_bytes = extra_bytes
        self.buffers = PeerBuffers(self.off_extra + extra_bytes, device, group, emulate_world)
        self.barrier_state = torch.zeros(16, dtype=torch.int32, device=device)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=device)
        self._links = {}
        self.rank, self.world = self.buffers.rank, self.buffers.world
        self.state = [torch.zeros(2, dtype=torch.int32, device=device) for _ in range(emulate_world or 1)]
        v = self.views_of(self.rank)
        self.ctx, self.lse, self.out, self.lse_out = v

    def views_of(self, r: int):
        """(ctx bf16 [n,512], lse fp32 [n], out bf16 [n,512], lse_out fp32 [n]) inside rank r's buffer."""
        b, n = self.buffers.views[r], self.n_rows
        return (b[self.off_ctx:self.off_ctx + n * 1024].view(torch.bfloat16).view(n, 512),
                b[self.off_lse:self.off_lse + n * 4].view(torch.float32),
                b[self.off_out:self.off_out + n * 1024].view(torch.bfloat16).view(n, 512),
                b[self.off_lse_out:self.off_lse_out + n * 4].view(torch.float32))

    def extra_of(self, r: int) -> torch.Tensor:
        """uint8 view of the extra area of rank r's buffer."""
        return self.buffers.views[r][self.off_extra:self.off_extra + self.extra_bytes]

    def element_offsets(self, itemsize: int = 4) -> List[int]:
        """Offset of every rank's buffer from this rank's, in elements of `itemsize` bytes."""
        base = self.buffers.addresses[self.rank]
        return [(a - base) // itemsize for a in self.buffers.addresses]

    def link(self, slot: int):
        """b200dsa_peer_link for kernels that exchange through these buffers.  Slot 0 names the merge
        kernel's own "partial ready" flags and step counter (for the attention kernel that raises them);
        slots 1, 3..7 carry their own step counters."""
        if slot not in self._links:
            state = self.state[0] if slot == 0 else self.barrier_state[2 * slot - 2:2 * slot]
            self._links[slot] = _lib.PeerLink(ctypes.cast(self.buffers._addr_array, ctypes.c_void_p).value, self.rank,
                                              self.world, self.off_flags, slot, state.data_ptr())
        return self._links[slot]

    def barrier(self, slot: int = 1) -> None:
        """Node-wide barrier on the current stream (b200dsa_peer_barrier): what the peers wrote into
        their buffers before their call can be read from this rank afterwards."""
        rc = _lib.load().b200dsa_peer_barrier(
            self.buffers._addr_array, self.rank, self.world, self.off_flags, slot,
            ptr(self.barrier_state[2 * slot - 2:2 * slot - 1]), ptr(status_word(self.buffers.device)), stream_ptr())
        check(rc, "b200dsa_peer_barrier")

    def push_extra(self, nbytes: int, slot: int = 1) -> torch.Tensor:
        """All-gather by posted stores (b200dsa_peer_push): the first nbytes of this rank's extra area
        are stored into slot `rank` of the receive area that follows it in EVERY rank's extra area
        (extra_bytes >= nbytes * (1 + world)).  Returns the local receive area, uint8 [world, nbytes]."""
        if nbytes * (1 + self.world) > self.extra_bytes:
            raise _lib.B200DSAError("extra area too small for nbytes * (1 + world)")
        rc = _lib.load().b200dsa_peer_push(
            self.buffers._addr_array, self.rank, self.world, self.off_extra, nbytes, self.off_extra + nbytes,
            self.off_flags, slot, ptr(self.barrier_state[2 * slot - 2:2 * slot]),
            ptr(status_word(self.buffers.device)), stream_ptr())
        check(rc, "b200dsa_peer_push")
        return self.extra_of(self.rank)[nbytes:nbytes * (1 + self.world)].view(self.world, nbytes)

    def gather_extra(self, dst: torch.Tensor, slot: int = 1, nbytes: Optional[int] = None) -> torch.Tensor:
        """Barrier, then copy the first nbytes (default: all) of the extra area of every rank into dst
        (local, contiguous, world * nbytes bytes, rank-major) with peer loads; see b200dsa_peer_gather."""
        nbytes = self.extra_bytes if nbytes is None else nbytes
        if not dst.is_contiguous() or dst.numel() * dst.element_size() != self.world * nbytes:
            raise _lib.B200DSAError("dst must be contiguous with world * nbytes bytes")
        rc = _lib.load().b200dsa_peer_gather(
            self.buffers._addr_array, self.rank, self.world, self.off_extra, nbytes, ptr(dst),
            self.off_flags, slot, ptr(self.barrier_state[2 * slot - 2:2 * slot]),
            ptr(status_word(self.buffers.device)), stream_ptr())
        check(rc, "b200dsa_peer_gather")
        return dst

    def row_slice(self, r: Optional[int] = None):
        """(first, last+1) rows of the merged result that rank r computes (and, with local_only, keeps)."""
        r = self.rank if r is None else r
        per = (self.n_rows + self.world - 1) // self.world
        return min(r * per, self.n_rows), min((r + 1) * per, self.n_rows)

    def run(self, rank: Optional[int] = None, no_sync: bool = False, pre_signalled: bool = False,
            local_only: bool = False):
        """Launch on the current stream.  `rank` / no_sync are for single-GPU emulation only: there the
        ranks run one after another and must not wait for each other.  pre_signalled: the attention
        kernel already raised this rank's "partial ready" flags (sparse_mla_decode(signal=...)).
        local_only: reduce-scatter form, only rows row_slice() of `out` / `lse_out` are produced."""
        r = self.rank if rank is None else rank
        if self.buffers.world > 1 and rank is not None and not no_sync:
            raise _lib.B200DSAError("emulated ranks on one GPU must run with no_sync")
        state = self.state[r if len(self.state) > 1 else 0]
        rc = _lib.load().b200dsa_peer_lse_combine(
            self.buffers._addr_array, r, self.world, self.n_rows, self.off_ctx, self.off_lse, self.off_out,
            self.off_lse_out, self.off_flags, ptr(state), int(no_sync), int(pre_signalled), int(local_only),
            ptr(status_word(self.buffers.device)), stream_ptr())
        check(rc, "b200dsa_peer_lse_combine")
        return self.out, self.lse_out

    def close(self) -> None:
        self.ctx = self.lse = self.out = self.lse_out = None
        self.buffers.close()


class PeerAllGather:
    """All-gather of one byte range over NVLink by posted stores (b200dsa_peer_push): every rank
    contributes `chunk` bytes and ends with all `world * chunk` bytes in local memory.  Used to replicate
    a step's inputs inside the node when only 1/world of them crossed each rank's host link.

    Buffer of a rank: `n_send` send areas of `chunk` bytes (one per in-flight step), then the receive
    area [world, chunk], then 256 bytes of flags.  The constructor is collective."""

    def __init__(self, total_bytes: int, device: torch.device, group=None, n_send: int = 1,
                 emulate_world: Optional[int] = None):
        world = emulate_world if emulate_world is not None else dist.get_world_size(group)
        self.chunk = _align((total_bytes + world - 1) // world, 256)
        self.n_send = n_send
        self.off_recv = n_send * self.chunk
        self.off_flags = self.off_recv + world * self.chunk
        self.buffers = PeerBuffers(self.off_flags + 256, device, group, emulate_world)
        self.rank, self.world = self.buffers.rank, self.buffers.world
        self.state = torch.zeros(2, dtype=torch.int32, device=device)
        self.send = [self.buffers.local[i * self.chunk:(i + 1) * self.chunk] for i in range(n_send)]
        self.recv = self.buffers.local[self.off_recv:self.off_recv + world * self.chunk]

    def run(self, send_slot: int = 0) -> torch.Tensor:
        """Launch on the current stream; when the kernel ends every rank's chunk is in `recv`."""
        rc = _lib.load().b200dsa_peer_push(
            self.buffers._addr_array, self.rank, self.world, send_slot * self.chunk, self.chunk, self.off_recv,
            self.off_flags, 1, ptr(self.state), ptr(status_word(self.buffers.device)), stream_ptr())
        check(rc, "b200dsa_peer_push")
        return self.recv

    def close(self) -> None:
        self.send, self.recv = [], None
        self.buffers.close()
