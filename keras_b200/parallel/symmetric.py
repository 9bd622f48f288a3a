"""Symmetric device buffers: the same allocation on every rank, mapped into every process with CUDA IPC.

``SymmetricBuffer(nbytes, group)`` allocates ``nbytes`` of device memory through the kernel library
(plain ``cudaMalloc`` memory, which IPC can export; the caching allocator's segments cannot be),
exchanges the IPC handles over the host group and opens the peers' handles.  ``ptrs[r]`` is rank
``r``'s buffer as mapped here (``ptrs[rank]`` is the local allocation).  Only the kernels of this
package dereference peer pointers; they are never handed to torch or another library.
"""

import ctypes

import torch
import torch.distributed as dist

from keras_b200.kernels import loader
from keras_b200.parallel import process_groups


class _RawCudaMemory:
    """Exposes a raw device pointer through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr, nbytes, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}
        self._owner = owner


def _lib():
    lib = loader.get()
    if lib is None:
        raise RuntimeError("Symmetric buffers need a CUDA device and the sm_100a kernel library.")
    return lib


def _err(lib):
    fn = lib.kb200_last_error
    fn.restype = ctypes.c_char_p
    return (fn() or b"").decode(errors="ignore")


class SymmetricBuffer:
    def __init__(self, nbytes, group=None, ranks=None):
        lib = _lib()
        self.nbytes = int(nbytes)
        self.group = group
        self.ranks = list(ranks) if ranks is not None else list(range(process_groups.world_size()))
        self.rank = self.ranks.index(process_groups.rank())
        self.world = len(self.ranks)
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        if lib.kb200_ipc_alloc(ctypes.c_longlong(self.nbytes), ctypes.byref(ptr), handle) != 0:
            raise RuntimeError("symmetric allocation failed: " + _err(lib))
        self.local_ptr = ptr.value
        handles = [None] * self.world
        host = process_groups.host_group()
        if self.world > 1:
            gathered = [None] * dist.get_world_size(host)
            dist.all_gather_object(gathered, (process_groups.rank(), bytes(handle.raw)), group=host)
            by_rank = dict(gathered)
            handles = [by_rank[r] for r in self.ranks]
        self.ptrs = []
        self._opened = []
        for i in range(self.world):
            if i == self.rank:
                self.ptrs.append(self.local_ptr)
                continue
            p = ctypes.c_void_p()
            if lib.kb200_ipc_open(ctypes.c_char_p(handles[i]), ctypes.byref(p)) != 0:
                raise RuntimeError(f"mapping the buffer of rank {self.ranks[i]} failed: " + _err(lib))
            self.ptrs.append(p.value)
            self._opened.append(p.value)
        self.ptr_array = (ctypes.c_void_p * self.world)(*self.ptrs)
        self._closed = False

    def tensor(self, dtype=torch.float32):
        """The local allocation as a torch tensor (no copy)."""
        raw = torch.as_tensor(_RawCudaMemory(self.local_ptr, self.nbytes, self), device=torch.device("cuda", torch.cuda.current_device()))
        return raw.view(dtype)

    def close(self):
        """Unmap the peers' buffers and free the local one.  Collective: every rank must have stopped using it."""
        if self._closed:
            return
        self._closed = True
        lib = _lib()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=process_groups.host_group())
        for p in self._opened:
            lib.kb200_ipc_close(ctypes.c_void_p(p))
        if self.world > 1:
            dist.barrier(group=process_groups.host_group())
        lib.kb200_ipc_free(ctypes.c_void_p(self.local_ptr))
