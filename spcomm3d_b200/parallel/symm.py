"""Symmetric heaps: device memory that every rank of a node can address.

A `Fabric` hands out `SymmHeap`s.  A heap is one device allocation per rank,
of the same size on all ranks and laid out identically (named regions at
identical offsets), so the address of "row i of region R on rank p" is
`heap.peer_base[p] + offset(R) + i * row_bytes` and can be computed locally.
Kernels load and store through these addresses directly (NVLink / NVSwitch
peer access).

Two fabrics:

* `IpcFabric`   one process per GPU (torch.distributed world): allocations are
                exported with CUDA IPC handles, gathered over the process group
                and opened once.  This is the production path; it replaces the
                MPI communicators of the reference (miniapp/bench_spmm.cpp:
                137-149) underneath the fused kernels.
* `LocalFabric` all ranks of a (virtual) mesh inside one process on one GPU:
                "peer" memory is just another local allocation.  Used to run
                every rank of a mesh in lock step on a single device.

Region sizes may differ between ranks; the heap uses the maximum per region
(an all-reduce(MAX) of the size vector on the IPC fabric).
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from ..utils import native

ALIGN = 256


def _align(n: int) -> int:
    return (int(n) + ALIGN - 1) // ALIGN * ALIGN


class _RawCudaBuffer:
    """Minimal __cuda_array_interface__ carrier so torch can view raw device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _ck(rc: int, what: str):
    if rc != 0:
        msg = native.cuda().sp3_cuda_error_string(rc)
        raise RuntimeError(f"{what}: {msg.decode() if msg else rc}")


class SymmHeap:
    def __init__(self, rank: int, world: int, sizes: dict, base: int, peer_base, device, keep=None):
        self.rank, self.world, self.device = rank, world, device
        self.offsets, off = {}, 0
        for name, nbytes in sizes.items():
            self.offsets[name] = off
            off += _align(nbytes)
        self.nbytes = off
        self.sizes = dict(sizes)
        self.base = base
        self.peer_base = list(peer_base)  # address of every rank's heap as mapped here (self at [rank])
        self._keep = keep
        self.bytes = torch.as_tensor(_RawCudaBuffer(base, max(self.nbytes, 1)), device=device)

    @staticmethod
    def layout_bytes(sizes: dict) -> int:
        return sum(_align(v) for v in sizes.values())

    def addr(self, region: str, rank: int | None = None, byte_offset: int = 0) -> int:
        r = self.rank if rank is None else rank
        return self.peer_base[r] + self.offsets[region] + byte_offset

    def view(self, region: str, dtype, shape) -> torch.Tensor:
        """Tensor over my own copy of a region (shape may be smaller than the region)."""
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        if n > _align(self.sizes[region]):
            raise ValueError(f"view of {n} bytes exceeds region {region}")
        o = self.offsets[region]
        return self.bytes[o:o + n].view(dtype).view(*shape)


class LocalFabric:
    """All ranks in this process, one GPU: heaps are plain local allocations."""

    def __init__(self, world: int, device="cuda"):
        self.world, self.device = world, torch.device(device)
        self.kind = "local"

    def heaps(self, sizes_per_rank: list[dict]) -> list[SymmHeap]:
        """One heap per rank from every rank's region sizes."""
        names = list(sizes_per_rank[0].keys())
        sizes = {n: max(int(s[n]) for s in sizes_per_rank) for n in names}
        total = SymmHeap.layout_bytes(sizes)
        bufs = [torch.zeros(max(total, ALIGN) + ALIGN, dtype=torch.uint8, device=self.device)
                for _ in range(self.world)]
        bases = [(_b.data_ptr() + ALIGN - 1) // ALIGN * ALIGN for _b in bufs]
        return [SymmHeap(r, self.world, sizes, bases[r], bases, self.device, keep=bufs) for r in range(self.world)]


class IpcFabric:
    """One process per GPU; peers' heaps are mapped through CUDA IPC."""

    def __init__(self, group=None, device=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.kind = "ipc"
        self._allocs = []

    def heap(self, sizes: dict) -> SymmHeap:
        dist, lib = self.dist, native.cuda()
        names = list(sizes.keys())
        vec = torch.tensor([int(sizes[n]) for n in names], dtype=torch.int64, device=self.device)
        dist.all_reduce(vec, op=dist.ReduceOp.MAX, group=self.group)
        sizes = {n: int(v) for n, v in zip(names, vec.tolist())}
        total = max(SymmHeap.layout_bytes(sizes), ALIGN)
        base = ctypes.c_void_p()
        _ck(lib.sp3_symm_alloc(total, ctypes.byref(base)), "symmetric allocation")
        handle = (ctypes.c_ubyte * 64)()
        _ck(lib.sp3_ipc_get_handle(base, handle), "cudaIpcGetMemHandle")
        gathered = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle), group=self.group)
        peer_base = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                peer_base.append(base.value)
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            p = ctypes.c_void_p()
            _ck(lib.sp3_ipc_open(buf, ctypes.byref(p)), f"cudaIpcOpenMemHandle(rank {r})")
            peer_base.append(p.value)
        self._allocs.append((base.value, [p for r, p in enumerate(peer_base) if r != self.rank]))
        dist.barrier(group=self.group)
        return SymmHeap(self.rank, self.world, sizes, base.value, peer_base, self.device)

    def close(self):
        """Unmaps peers and frees own allocations (call between steps, with no kernel in flight)."""
        lib = native.cuda()
        torch.cuda.synchronize()
        self.dist.barrier(group=self.group)
        for base, peers in self._allocs:
            for p in peers:
                lib.sp3_ipc_close(ctypes.c_void_p(p))
        self.dist.barrier(group=self.group)
        for base, _ in self._allocs:
            lib.sp3_symm_free(ctypes.c_void_p(base))
        self._allocs = []
