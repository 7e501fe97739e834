"""Peer memory between the GPUs of one NVLink node: shared buffers, a barrier and a small all-gather.

One process per GPU. A buffer is allocated with cudaMalloc on its own GPU and mapped by every other rank
through a CUDA IPC handle (the handles travel once, by `all_gather_object`); kernels then store into the
peers' buffers directly. The barrier is one small kernel per rank that stores a sequence number into every
peer's state block and waits, with a time limit, for the peers' numbers (include/nvfp4_capi.h:
gpu_kernels_nvfp4_peer_exchange): no collective library call and nothing for the host to wait on, so it can
sit in a CUDA graph between the kernels it orders. The reference keeps the equivalent signalling inside its
fused MoE kernel (kernels/moe/fused/sm90.cu:296-319, 532-541).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class DeviceView:
    """Lets torch wrap device memory this package allocated itself (CUDA array interface)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}


class SharedBuffer:
    """`nbytes` of zeroed device memory on every rank, each rank's mapped into all the others.

    ptrs[r] is rank r's buffer as seen from this process (ptrs[rank] = own). Collective: construct and
    close on every rank of the group, in the same order.
    """

    def __init__(self, nbytes: int, device, group=None):
        lib = _lib.load()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = torch.device(device)
        with torch.cuda.device(self.device):
            own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
            _lib.check(lib.gpu_kernels_nvfp4_ipc_alloc(nbytes, ctypes.byref(own), handle))
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            self.table = (ctypes.c_void_p * self.world)()          # host array, for the C ABI
            self._opened = []
            for r in range(self.world):
                if r == self.rank:
                    self.table[r] = own.value
                else:
                    ptr = ctypes.c_void_p()
                    _lib.check(lib.gpu_kernels_nvfp4_ipc_open(handles[r], ctypes.byref(ptr)))
                    self.table[r] = ptr.value
                    self._opened.append(ptr.value)
        self.own = own.value
        self.ptrs = [int(self.table[r]) for r in range(self.world)]
        self.device_table = torch.tensor(self.ptrs, dtype=torch.int64, device=self.device)

    def close(self) -> None:
        if self.own is None:
            return
        lib = _lib.load()
        torch.cuda.synchronize(self.device)
        for ptr in self._opened:
            lib.gpu_kernels_nvfp4_ipc_close(ptr)
        if dist.is_initialized():
            dist.barrier(group=self.group)                          # nobody still maps this rank's buffer
        lib.gpu_kernels_nvfp4_ipc_free(self.own)
        self.own = None


class PeerGroup:
    """Barrier and all-gather of a few integers between the ranks of one node, over peer memory."""

    def __init__(self, device, group=None, max_ints: int = 4096):
        self.max_ints = max_ints
        nbytes = ctypes.c_size_t()
        world = dist.get_world_size(group)
        _lib.check(_lib.load().gpu_kernels_nvfp4_peer_state_bytes(world, max_ints, ctypes.byref(nbytes)))
        self.state = SharedBuffer(nbytes.value, device, group)
        self.world, self.rank, self.device = self.state.world, self.state.rank, self.state.device

    def barrier(self) -> None:
        """Stream-ordered: completes on this rank after every rank's earlier stores into peer memory are visible."""
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_peer_exchange(
                self.state.own, self.state.device_table.data_ptr(), self.world, self.rank, None, 0, self.max_ints, None, _stream()))

    def all_gather_ints(self, payload: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """payload [n] int32 of every rank -> out [world, n] on every rank (also a barrier)."""
        n = payload.numel()
        if payload.dtype != torch.int32 or out.dtype != torch.int32 or out.numel() != self.world * n or n > self.max_ints:
            raise ValueError("all_gather_ints: int32 payload of at most max_ints values and a [world, n] int32 result")
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_peer_exchange(
                self.state.own, self.state.device_table.data_ptr(), self.world, self.rank, payload.data_ptr(), n,
                self.max_ints, out.data_ptr(), _stream()))
        return out

    def close(self) -> None:
        self.state.close()
