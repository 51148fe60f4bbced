"""Result buffers that every rank of one machine can write: the storage behind the fused
product + all-gather (srtMatmulAllGather).

One process per GPU.  Each rank allocates one full-size result with srtPeerMemAlloc, the 64-byte
handles travel through torch.distributed, and each rank maps the others' buffers with
srtPeerMemOpen.  The reference's pmap gives every partition a view of one shared output
(Sources/SwiftRTCore/operators/pmap.swift:26-72); here "shared" is one buffer per GPU, all of
them holding all blocks once every rank has finished.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from . import _lib
from ._lib import lib
from .matmul import MatmulError


def _check(rc: int) -> None:
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())


class _RawDeviceMemory:
    """Just enough of the CUDA array interface for torch to wrap a device pointer."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2, "strides": None}


def _alloc_and_exchange(nbytes: int, device, rank: int, world: int, group):
    """(own device pointer, {rank: mapped pointer of that rank's buffer}) for a srtPeerMemAlloc'ed buffer of
    `nbytes` on every rank; the 64-byte handles travel through torch.distributed."""
    ptr = ctypes.c_void_p()
    handle = _lib.PeerMemHandle()
    with torch.cuda.device(device):
        _check(lib.srtPeerMemAlloc(nbytes, ctypes.byref(ptr), ctypes.byref(handle)))
    peers: dict[int, int] = {}
    if world > 1:
        handles: list = [None] * world
        dist.all_gather_object(handles, bytes(handle.bytes), group=group)
        with torch.cuda.device(device):
            for r, blob in enumerate(handles):
                if r == rank:
                    continue
                h = _lib.PeerMemHandle()
                ctypes.memmove(h.bytes, blob, 64)
                p = ctypes.c_void_p()
                _check(lib.srtPeerMemOpen(ctypes.byref(h), ctypes.byref(p)))
                peers[r] = p.value
    return ptr, peers


class PeerBuffer:
    """A dense tensor of `shape` on this rank's GPU plus the addresses of the same tensor on the
    other ranks' GPUs.

    tensor      this rank's buffer as a torch tensor (not owned by torch's allocator)
    peer_base   {rank: device address of that rank's buffer, mapped into this process}
    """

    def __init__(self, shape: Sequence[int], dtype: torch.dtype, group=None, device: Optional[torch.device] = None,
                 multicast: bool = False):
        """`multicast=True` allocates the buffers as torch symmetric memory instead, which also binds
        them to one NVLink multicast object: `multicast_base` is then the address of the multicast
        mapping (0 when the machine has none) and the peers' addresses come from the same handle."""
        self.group = group
        self.multicast_base = 0
        self._symm = None
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise ValueError("at most 8 ranks (7 peers)")
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype
        count = 1
        for s in self.shape:
            count *= s
        self.nbytes = max(count * torch.empty((), dtype=dtype).element_size(), 16)
        self._ptr = ctypes.c_void_p()
        self.peer_base: dict[int, int] = {}
        # flags for ranks_done(): one 64-bit slot per rank in every rank's array, zeroed before anybody signals
        self._epoch = 0
        self._flags_ptr, self._peer_flags = _alloc_and_exchange(256, self.device, self.rank, self.world, group)
        torch.as_tensor(_RawDeviceMemory(self._flags_ptr.value, 256), device=self.device).zero_()
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=group)
        if multicast and self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            with torch.cuda.device(self.device):
                self.tensor = symm_mem.empty(self.shape, dtype=dtype, device=self.device)
                self._symm = symm_mem.rendezvous(self.tensor, group if group is not None else dist.group.WORLD)
            self.multicast_base = int(self._symm.multicast_ptr or 0)
            self.peer_base = {r: int(p) for r, p in enumerate(self._symm.buffer_ptrs) if r != self.rank}
            self._token = None
            self._open = True
            return
        handle = _lib.PeerMemHandle()
        with torch.cuda.device(self.device):
            _check(lib.srtPeerMemAlloc(self.nbytes, ctypes.byref(self._ptr), ctypes.byref(handle)))
        raw = torch.as_tensor(_RawDeviceMemory(self._ptr.value, self.nbytes), device=self.device)
        self.tensor = raw[: count * raw.new_empty((), dtype=dtype).element_size()].view(dtype).reshape(self.shape)
        if self.world > 1:
            handles: list = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.bytes), group=group)
            with torch.cuda.device(self.device):
                for r, blob in enumerate(handles):
                    if r == self.rank:
                        continue
                    h = _lib.PeerMemHandle()
                    ctypes.memmove(h.bytes, blob, 64)
                    p = ctypes.c_void_p()
                    _check(lib.srtPeerMemOpen(ctypes.byref(h), ctypes.byref(p)))
                    self.peer_base[r] = p.value
        self._token = None
        self._open = True

    def peer_pointers(self, view: torch.Tensor) -> list[int]:
        """Addresses of `view` (a view of self.tensor) in every peer's buffer, by rank order."""
        offset = view.data_ptr() - self.tensor.data_ptr()
        if not 0 <= offset < self.nbytes:
            raise ValueError("not a view of this buffer")
        return [base + offset for _, base in sorted(self.peer_base.items())]

    def multicast_pointer(self, view: torch.Tensor) -> int:
        """Address of `view` in the multicast mapping (0 without one)."""
        if not self.multicast_base:
            return 0
        offset = view.data_ptr() - self.tensor.data_ptr()
        if not 0 <= offset < self.nbytes:
            raise ValueError("not a view of this buffer")
        return self.multicast_base + offset

    def ranks_done(self) -> None:
        """Orders everything the ranks enqueued so far before what follows on this rank's current
        stream: after it, blocks written by other ranks may be read."""
        if self.world > 1:
            # no collective: this rank's step number goes into its slot of every peer's flag array (behind the
            # kernels enqueued so far), then the stream waits -- bounded -- until all peers' numbers have arrived
            self._epoch += 1
            stream = torch.cuda.current_stream(self.device).cuda_stream
            ptrs = [p for _, p in sorted(self._peer_flags.items())]
            arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
            with torch.cuda.device(self.device):
                _check(lib.srtPeerSignal(arr, len(ptrs), self.rank, self._epoch, stream))
                _check(lib.srtPeerWait(self._flags_ptr, self.world, self.rank, self._epoch, 0, stream))

    def close(self) -> None:
        """Collective: unmaps the peers' buffers, then frees this rank's."""
        if not self._open:
            return
        self._open = False
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for p in self._peer_flags.values():
                _check(lib.srtPeerMemClose(p))
        self._peer_flags = {}
        if self.world > 1:
            dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            _check(lib.srtPeerMemFree(self._flags_ptr))
        if self._symm is not None:
            # symmetric memory is owned by torch: dropping the references releases the mappings
            self.peer_base = {}
            self.multicast_base = 0
            self._symm = None
            self.tensor = None
            return
        with torch.cuda.device(self.device):
            for p in self.peer_base.values():
                _check(lib.srtPeerMemClose(p))
        self.peer_base = {}
        if self.world > 1:
            dist.barrier(group=self.group)
            torch.cuda.synchronize(self.device)
        self.tensor = None
        with torch.cuda.device(self.device):
            _check(lib.srtPeerMemFree(self._ptr))
