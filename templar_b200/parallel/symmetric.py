"""Symmetric heap over CUDA IPC: every rank allocates the same buffers in the same order and
maps all peers' copies, so kernels can address ``peer_ptr(tensor, rank)`` directly over
NVLink (plain loads/stores; no TMA multicast anywhere).

Bootstrap rides on the existing ``torch.distributed`` process group (handles are exchanged
with ``all_gather_object``).  The flag barrier is a tiny kernel with a bounded wait: if a
peer never arrives, the kernel gives up after ``timeout_s``, sets the status word, and the
host raises on the next :meth:`SymmetricHeap.check` instead of the GPU spinning forever.

The reference has no counterpart: it moves everything through NCCL collectives
(src/tplr/distributed.py:35-549).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import native


GUARD, GUARD_BYTE = 256, 0xA5


class _DeviceBlock:
    """Exposes a raw device allocation through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmetricHeap:
    def __init__(self, device, rank: int, world_size: int, group=None, timeout_s: float = 30.0):
        self.device, self.rank, self.world_size, self.group = torch.device(device), rank, world_size, group
        self.timeout_ns = int(timeout_s * 1e9)
        self._allocs: list[tuple[int, int, list[int]]] = []   # (local_ptr, nbytes, [ptr per rank])
        self._blocks = []
        self._guards: list[torch.Tensor] = []
        self._epoch = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._flags = None

    @classmethod
    def create(cls, device, rank: int, world_size: int, group=None, timeout_s: float = 30.0) -> "SymmetricHeap":
        heap = cls(device, rank, world_size, group, timeout_s)
        heap._flags = heap.alloc(64, torch.int64)
        return heap

    # -- allocation -------------------------------------------------------------------------
    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Collective: every rank must call with the same arguments in the same order."""
        L = native.lib()
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = max(-(-numel * esz // 256) * 256, 256)
        out = ctypes.c_void_p()
        # GUARD bytes behind every block hold a fixed pattern: a store that runs past the end of a buffer (this
        # rank's or a peer's) lands there and is found by check_guards() instead of corrupting a neighbour
        native.check(L.tplr_heap_alloc(ctypes.c_ulonglong(nbytes + GUARD), ctypes.byref(out)), "heap_alloc")
        native.launch_count -= 1
        local = out.value
        hsz = L.tplr_ipc_handle_size()
        hbuf = ctypes.create_string_buffer(hsz)
        err = L.tplr_ipc_get(ctypes.c_void_p(local), hbuf)
        if err:
            raise native.NativeError(f"cudaIpcGetMemHandle failed: {err}")
        handles = [None] * self.world_size
        dist.all_gather_object(handles, bytes(hbuf.raw), group=self.group)
        ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs.append(local)
                continue
            p = ctypes.c_void_p()
            err = L.tplr_ipc_open(ctypes.create_string_buffer(h, hsz), ctypes.byref(p))
            if err:
                raise native.NativeError(f"cudaIpcOpenMemHandle(rank {r}) failed: {err}")
            ptrs.append(p.value)
        self._allocs.append((local, nbytes, ptrs))
        block = _DeviceBlock(local, nbytes + GUARD)
        self._blocks.append(block)
        t = torch.as_tensor(block, device=self.device)
        guard = t[nbytes:]
        guard.fill_(GUARD_BYTE)
        self._guards.append(guard)
        return t[:nbytes].view(dtype)[:numel]

    def check_guards(self) -> None:
        """Host sync; raises if the guard bytes behind any block of this rank were overwritten."""
        if not self._guards:
            return
        bad = torch.stack([(g != GUARD_BYTE).any() for g in self._guards])
        if bool(bad.any().item()):
            which = [i for i, b in enumerate(bad.tolist()) if b]
            raise MemoryError(f"symmetric heap: a store ran past the end of block(s) {which} on rank {self.rank}")

    def peer_ptr(self, tensor_or_ptr, rank: int) -> int:
        """Address, in this process, of ``tensor``'s memory inside rank ``rank``'s copy of the allocation."""
        p = tensor_or_ptr.data_ptr() if isinstance(tensor_or_ptr, torch.Tensor) else int(tensor_or_ptr)
        for local, nbytes, ptrs in self._allocs:
            if local <= p < local + nbytes:
                return ptrs[rank] + (p - local)
        raise ValueError("tensor is not part of the symmetric heap")

    # -- synchronisation ----------------------------------------------------------------------
    def barrier(self) -> None:
        """Stream-ordered barrier across all ranks (bounded device wait)."""
        self._epoch += 1
        ptrs = [self.peer_ptr(self._flags, r) for r in range(self.world_size)]
        native.check(native.lib().tplr_barrier(native.ptr_array(ptrs), self.world_size, self.rank,
                                               ctypes.c_ulonglong(self._epoch), ctypes.c_ulonglong(self.timeout_ns),
                                               self.status.data_ptr(), native.stream_ptr()), "barrier")

    def check(self) -> None:
        """Host sync; raises if any bounded wait expired since the last check."""
        v = int(self.status.item())
        if v:
            self.status.zero_()
            raise TimeoutError(f"symmetric-heap wait expired (status {v:#x}): a peer did not arrive")

    def close(self) -> None:
        L = native.lib()
        torch.cuda.synchronize(self.device)
        for local, _, ptrs in self._allocs:
            for r, p in enumerate(ptrs):
                if r != self.rank:
                    L.tplr_ipc_close(ctypes.c_void_p(p))
        # local blocks are released at process exit: tensors viewing them may still be alive
        self._allocs.clear()
