"""Python handle on the page pool (include/sirius_pool.h)."""
from __future__ import annotations

import ctypes as C

from . import _lib, _runtime  # noqa: F401
from ._lib import call
from ._runtime import PoolConfig

TRAIN, INFER = 0, 1
STAT = {"infer_usage": 0, "train_usage": 1, "train_peak": 2, "train_all": 3, "free_pages": 4, "pool_nbytes": 5,
        "page_nbytes": 6, "num_map": 7, "num_unmap": 8, "infer_allocated": 9, "num_reuse": 10}


class PagePool:
    """One pool of physical pages on a GPU with a training and an inference allocator
    (colserve::sta::CUDAMemPool, common/cuda_allocator.h:61-150)."""

    def __init__(self, pool_gb: float, device: int = 0, page_mb: int = 32, host_backend: bool = False,
                 unmap_on_release: bool = False, shared_name: str | None = None):
        """shared_name: create the pool for other processes to attach to (PagePool.attach), as the reference's
        inference server does for its trainers."""
        cfg = PoolConfig(device, 1 if host_backend else 0, page_mb << 20, int(pool_gb * (1 << 30)), 0, 0,
                         int(unmap_on_release))
        self._h = C.c_void_p()
        if shared_name is None:
            call("srt_pool_create", C.byref(cfg), C.byref(self._h))
        else:
            call("srt_pool_create_shared", C.byref(cfg), shared_name.encode(), C.byref(self._h))

    @classmethod
    def attach(cls, shared_name: str, device: int = 0, timeout_ms: int = 10000) -> "PagePool":
        """Open a pool another process created with shared_name: same physical pages, this process's own
        allocators and virtual ranges."""
        self = cls.__new__(cls)
        self._h = C.c_void_p()
        call("srt_pool_attach", shared_name.encode(), device, timeout_ms, C.byref(self._h))
        return self

    @property
    def handle(self): return self._h

    def alloc(self, kind: int, nbytes: int) -> int:
        p = C.c_void_p()
        call("srt_pool_alloc", self._h, kind, nbytes, C.byref(p))
        return p.value

    def free(self, kind: int, ptr: int): call("srt_pool_free", self._h, kind, C.c_void_p(ptr))

    def empty_cache(self, kind: int = TRAIN) -> int:
        n = C.c_size_t()
        call("srt_pool_empty_cache", self._h, kind, C.byref(n))
        return n.value

    def stat(self, name: str) -> int: return _lib.lib().srt_pool_stat(self._h, STAT[name])

    def close(self):
        if self._h:
            call("srt_pool_destroy", self._h)
            self._h = C.c_void_p()
