"""Peer-memory groups: symmetric device regions every rank of an NVLink domain can store into.

``PeerGroup.allocate(nbytes)`` gives each rank a zero-filled region of the same size, exchanges the
CUDA IPC handles once over the bootstrap ``torch.distributed`` group (NCCL or gloo; objects only)
and maps every peer's region, so kernels get a table of base addresses indexed by rank.  After
that no library collective is needed to move rows: the dispatch and return kernels store straight
into the owner's buffers and publish an epoch flag.

``PeerGroup.local(world)`` builds the same structure for ``world`` simulated ranks inside one process
on one GPU (each "rank" gets its own region and every table simply points at the local regions); it
exists so that single-GPU tests can run the multi-rank data path kernel by kernel.

The reference has no counterpart (it calls ``dist.all_to_all_single``, ``moeflow/fixed.py:234,237``).
"""

from __future__ import annotations

import ctypes as C
import weakref

import torch
import torch.distributed as dist

from ..ops import _lib


class _RawDeviceMemory:
    """Owner of one cudaMalloc'd block; torch sees it through ``__cuda_array_interface__``."""

    def __init__(self, nbytes: int, ptr: int, owned: bool, opened: bool):
        self.nbytes, self.ptr, self._owned, self._opened = nbytes, ptr, owned, opened
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (ptr, False),
            "version": 3,
            "strides": None,
        }
        self._finalizer = weakref.finalize(self, _RawDeviceMemory._release, ptr, owned, opened)

    @staticmethod
    def _release(ptr: int, owned: bool, opened: bool) -> None:
        try:
            if owned:
                _lib.lib().mf_peer_free(C.c_void_p(ptr))
            elif opened:
                _lib.lib().mf_peer_close(C.c_void_p(ptr))
        except Exception:  # pragma: no cover - interpreter shutdown
            pass

    def release(self) -> None:
        self._finalizer()


class SymmetricRegion:
    """One rank's view of a symmetric allocation: the local block and every peer's base address."""

    def __init__(self, local: _RawDeviceMemory, peer_ptrs: list[int], rank: int, device: torch.device, keep=()):
        self.local, self.peer_ptrs, self.rank, self.device = local, list(peer_ptrs), rank, device
        self._keep = list(keep)  # mapped peer blocks (closed when this region goes away)
        self.bytes = torch.as_tensor(local, device=device)

    @property
    def world(self) -> int:
        return len(self.peer_ptrs)

    def view(self, offset: int, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """A tensor over ``[offset, offset + numel*itemsize)`` of the local block."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.bytes[offset : offset + nbytes].view(dtype).view(*shape)

    def table(self, offset: int = 0) -> torch.Tensor:
        """int64 device tensor ``[world]``: address of ``offset`` inside every rank's block."""
        return torch.tensor([p + offset for p in self.peer_ptrs], dtype=torch.int64, device=self.device)

    def close(self) -> None:
        for blk in self._keep:
            blk.release()
        self._keep.clear()
        self.local.release()


def check_exchange(gathered: list, world: int, nbytes: int) -> None:
    """Validate what the ranks exchanged at bootstrap: ``(rank, nbytes, 64-byte IPC handle)`` per rank.

    Every rank runs this on the same gathered list, so a rank that asked for a different size (for instance a
    different capacity) or sent a malformed handle makes all ranks raise the same error before any peer memory
    is mapped, instead of leaving some of them waiting.
    """
    if len(gathered) != world:
        raise RuntimeError(f"symmetric allocation: expected {world} bootstrap records, got {len(gathered)}")
    for r, record in enumerate(gathered):
        if not isinstance(record, tuple) or len(record) != 3:
            raise RuntimeError(f"symmetric allocation: malformed bootstrap record from rank {r}")
        peer_rank, peer_bytes, handle = record
        if peer_rank != r or peer_bytes != nbytes:
            raise RuntimeError(
                f"symmetric allocation mismatch: rank {r} reported rank {peer_rank}, {peer_bytes} bytes, "
                f"expected {nbytes}"
            )
        if not isinstance(handle, (bytes, bytearray)) or len(handle) != 64:
            raise RuntimeError(f"symmetric allocation: rank {r} sent a malformed IPC handle")


def _alloc(nbytes: int) -> _RawDeviceMemory:
    out = C.c_void_p()
    _lib.check(_lib.lib().mf_peer_alloc(C.byref(out), nbytes), "peer alloc")
    return _RawDeviceMemory(nbytes, out.value, owned=True, opened=False)


class PeerGroup:
    """The ranks that share symmetric regions (one process per GPU)."""

    def __init__(self, rank: int, world: int, group: dist.ProcessGroup | None = None, device=None):
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")

    @classmethod
    def from_dist(cls, group: dist.ProcessGroup | None = None, device=None) -> "PeerGroup":
        if dist.is_available() and dist.is_initialized():
            return cls(dist.get_rank(group), dist.get_world_size(group), group, device)
        return cls(0, 1, None, device)

    def allocate(self, nbytes: int) -> SymmetricRegion:
        nbytes = (nbytes + 255) // 256 * 256
        with torch.cuda.device(self.device):
            mine = _alloc(nbytes)
            if self.world == 1:
                return SymmetricRegion(mine, [mine.ptr], 0, self.device)
            handle = (C.c_ubyte * 64)()
            _lib.check(_lib.lib().mf_peer_export(C.c_void_p(mine.ptr), handle), "peer export")
            gathered: list = [None] * self.world
            dist.all_gather_object(gathered, (self.rank, nbytes, bytes(handle)), group=self.group)
            check_exchange(gathered, self.world, nbytes)
            ptrs, keep = [], []
            for r, (peer_rank, peer_bytes, peer_handle) in enumerate(gathered):
                if r == self.rank:
                    ptrs.append(mine.ptr)
                    continue
                out = C.c_void_p()
                buf = (C.c_ubyte * 64).from_buffer_copy(peer_handle)
                _lib.check(_lib.lib().mf_peer_open(buf, C.byref(out)), f"peer open (rank {r})")
                blk = _RawDeviceMemory(nbytes, out.value, owned=False, opened=True)
                keep.append(blk)
                ptrs.append(out.value)
            dist.barrier(group=self.group)
            return SymmetricRegion(mine, ptrs, self.rank, self.device, keep)

    @staticmethod
    def local(world: int, nbytes: int, device=None) -> list[SymmetricRegion]:
        """``world`` simulated ranks on one GPU in this process."""
        device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        nbytes = (nbytes + 255) // 256 * 256
        with torch.cuda.device(device):
            blocks = [_alloc(nbytes) for _ in range(world)]
        ptrs = [b.ptr for b in blocks]
        return [SymmetricRegion(b, ptrs, r, device) for r, b in enumerate(blocks)]


def ping(region: SymmetricRegion, offset: int, value: int, status: torch.Tensor, wait_ns: int = 1_000_000_000,
         skip_store: bool = False) -> None:
    """Store ``value`` into word ``[rank]`` at ``offset`` of every peer, then wait for all local words.

    With ``skip_store`` nothing is stored, so the bounded wait runs out and ``status`` gets the ping
    time-out code: the error path is exercised without hanging the GPU.
    """
    table = region.table(offset)
    local = region.view(offset, (region.world,), torch.int32)
    _lib.check(
        _lib.lib().mf_peer_ping(
            table.data_ptr(), local.data_ptr(), region.world, region.rank, value, int(skip_store),
            status.data_ptr(), wait_ns, _lib.stream_ptr(),
        ),
        "peer ping",
    )
    region._ping_table = table  # keep the table alive until the kernel has run
