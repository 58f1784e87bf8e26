"""Host memory for transfers: DMA-able (page-locked) allocations, block pools for the weight
loader, and the model-tree -> buffer-tree mapping (zml/mem.zig of the reference).

The allocators and pools are native (libzb_cuda.so: host_mem.cu); blocks are exposed as
zero-copy `torch.uint8` / numpy views.  Without a usable CUDA device the same API hands out
page-aligned pageable memory (`pinned` is then False), so loaders behave the same on CPU.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional

import numpy as np
import torch

from . import meta
from .ops import _lib

_p, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
_lib.register_signature("zb_host_alloc", _i, [_sz, C.POINTER(_p), C.POINTER(_i)])
_lib.register_signature("zb_host_free", None, [_p, _i])
_lib.register_signature("zb_host_register", _i, [_p, _sz])
_lib.register_signature("zb_host_unregister", _i, [_p])
_lib.register_signature("zb_pool_create", _p, [_sz, _i, _i, _i])
_lib.register_signature("zb_pool_get", _p, [_p, _i])
_lib.register_signature("zb_pool_put", _i, [_p, _p])
_lib.register_signature("zb_pool_stats", None, [_p, C.POINTER(_i)])
_lib.register_signature("zb_pool_destroy", None, [_p])


class PoolTimeout(RuntimeError):
    pass


class HostBlock:
    """A range of host memory owned by an allocator or a pool."""

    def __init__(self, ptr: int, nbytes: int, pinned: bool, release: Optional[Callable[["HostBlock"], None]] = None):
        self.ptr, self.nbytes, self.pinned = ptr, nbytes, pinned
        self._release = release

    def numpy(self) -> np.ndarray:
        return np.ctypeslib.as_array((C.c_uint8 * self.nbytes).from_address(self.ptr))

    def torch(self) -> torch.Tensor:
        return torch.from_numpy(self.numpy())

    def free(self) -> None:
        if self._release is not None:
            rel, self._release = self._release, None
            rel(self)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.free()


class DmaAllocator:
    """Host allocations a GPU can DMA from directly (zml/mem.zig:17-36,121-180: host alloc +
    `dmaMap`).  `register` page-locks memory that was allocated elsewhere (an mmap, a numpy array)."""

    def alloc(self, nbytes: int) -> HostBlock:
        ptr, pinned = _p(), _i()
        if _lib.lib().zb_host_alloc(nbytes, C.byref(ptr), C.byref(pinned)) != 0:
            raise MemoryError(f"host allocation of {nbytes} bytes failed")
        return HostBlock(ptr.value, nbytes, bool(pinned.value),
                         lambda b: _lib.lib().zb_host_free(b.ptr, 1 if b.pinned else 0))

    def register(self, array: np.ndarray) -> bool:
        """True when the range is now page-locked (False on a machine without CUDA)."""
        rc = _lib.lib().zb_host_register(array.ctypes.data, array.nbytes)
        if rc < 0:
            raise RuntimeError(f"cudaHostRegister failed with error {-rc}")
        return rc == 0

    def unregister(self, array: np.ndarray) -> None:
        _lib.lib().zb_host_unregister(array.ctypes.data)


class _Pool:
    def __init__(self, block_bytes: int, blocks: int, pinned: bool, fixed: bool):
        self.block_bytes = block_bytes
        self._h = _lib.lib().zb_pool_create(block_bytes, blocks, 1 if pinned else 0, 1 if fixed else 0)
        if not self._h:
            raise MemoryError(f"cannot create a pool of {blocks} x {block_bytes} bytes")

    def get(self, timeout_s: Optional[float] = None) -> HostBlock:
        """Blocks while the pool is exhausted; raises PoolTimeout after `timeout_s`."""
        ptr = _lib.lib().zb_pool_get(self._h, -1 if timeout_s is None else int(timeout_s * 1000))
        if not ptr:
            raise PoolTimeout(f"no block became free within {timeout_s} s")
        return HostBlock(ptr, self.block_bytes, self.stats()["pinned"] > 0, self.put)

    def put(self, block: HostBlock) -> None:
        rc = _lib.lib().zb_pool_put(self._h, block.ptr)
        if rc != 0:
            raise ValueError("block does not belong to this pool" if rc == -1 else "pool has no block in flight")

    def stats(self) -> dict:
        a = (_i * 4)()
        _lib.lib().zb_pool_stats(self._h, a)
        return {"in_flight": a[0], "allocated": a[1], "pinned": a[2], "max_blocks": a[3]}

    def close(self) -> None:
        if self._h:
            _lib.lib().zb_pool_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class FixedBufferPool(_Pool):
    """`blocks` equal blocks carved out of one slab (zml/mem.zig:182-224)."""

    def __init__(self, block_bytes: int, blocks: int, pinned: bool = True):
        super().__init__(block_bytes, blocks, pinned, fixed=True)


class DynamicBufferPool(_Pool):
    """Blocks allocated on first use and recycled, with at most `max_blocks` in flight
    (zml/mem.zig:226-316)."""

    def __init__(self, max_blocks: int, block_bytes: int, pinned: bool = True):
        super().__init__(block_bytes, max_blocks, pinned, fixed=False)


def bufferize(model, to_buffer: Callable):
    """Model tree -> same tree with every Tensor replaced by `to_buffer(tensor)` and fields that
    hold no tensor dropped (`Bufferized(T)` of the reference, zml/mem.zig:321-381)."""
    return meta.bufferize(model, to_buffer)


Bufferized = bufferize
