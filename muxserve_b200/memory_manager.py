"""``KVStorage`` — block allocator of the unified KV pool (host C++ behind the C ABI).

Same methods, argument meaning and return encodings as the pybind class
``muxserve.memory_manager.KVStorage`` (csrc/memory_manager.cpp:159-165).
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from ._lib import MuxError, check, i32p, lib


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32).reshape(-1))


class KVStorage:
    def __init__(self, num_blocks: int):
        self._lib = lib()
        self._h = self._lib.mux_kv_storage_create(int(num_blocks))
        if not self._h:
            raise ValueError(f"KVStorage: invalid num_blocks {num_blocks}")
        self.num_blocks = int(num_blocks)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.mux_kv_storage_destroy(h)

    def allocate(self, size: int) -> np.ndarray:
        """Pops ``size`` block ids from the tail of the free list (memory_manager.cpp:12-23)."""
        out = np.empty(int(size), dtype=np.int32)
        check(self._lib.mux_kv_storage_allocate(self._h, int(size), i32p(out)), "KVStorage.allocate")
        return out

    def allocate_batch(self, batch_alloc_info, num_layers: int, num_heads: int) -> np.ndarray:
        """Rows ``[request id, logical blocks, has_blocks]`` -> ``[preempt_idx, block ids...]``.

        ``preempt_idx`` requests are served; the rest were preempted and lost
        their blocks (memory_manager.cpp:25-142).
        """
        info = _i32(batch_alloc_info)
        n = info.size // 3
        cap = 1 + int(np.maximum(info[1:3 * n:3], 0).astype(np.int64).sum()) * int(num_layers) * int(num_heads)
        out = np.empty(cap, dtype=np.int32)
        out_len = C.c_int64(0)
        check(self._lib.mux_kv_storage_allocate_batch(self._h, i32p(info), n, int(num_layers), int(num_heads),
                                                      i32p(out), cap, C.byref(out_len)),
              "KVStorage.allocate_batch")
        return out[:out_len.value].copy() if out_len.value < cap else out

    def free_batch(self, batch_request_ids: Sequence[int]) -> int:
        """Returns the blocks of the given requests to the free list; unknown ids are ignored."""
        ids = _i32(batch_request_ids)
        r = self._lib.mux_kv_storage_free_batch(self._h, i32p(ids), ids.size)
        if r < 0:
            raise MuxError(int(r), "KVStorage.free_batch")
        return int(r)

    def get_new_blocks_allocated(self) -> int:
        return int(self._lib.mux_kv_storage_new_blocks_allocated(self._h))

    # ---- introspection (not in the reference) ----
    def num_blocks_allocated(self) -> int:
        return int(self._lib.mux_kv_storage_num_blocks_allocated(self._h))

    def num_free(self) -> int:
        return int(self._lib.mux_kv_storage_num_free(self._h))

    def free_list(self) -> np.ndarray:
        out = np.empty(self.num_free(), dtype=np.int32)
        check(self._lib.mux_kv_storage_free_list(self._h, i32p(out), out.size), "KVStorage.free_list")
        return out

    def check_invariants(self) -> bool:
        """Every block id is in the free list or owned by exactly one request."""
        return self._lib.mux_kv_storage_check(self._h) == 0
