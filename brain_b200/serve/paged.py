"""Python faces of the native paged-KV bookkeeping (csrc/runtime/serving.cpp):
``BlockAllocator`` (free list + u16 refcounts), ``BlockTable`` (append / reserve / truncate /
release / fork / unshare_tail / adopt_prefix) and ``PrefixCache`` (full prompt blocks keyed by
(parent block, token ids), LRU eviction).  Reference: crates/model/src/paged.rs:20-328."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import numpy as np

from .. import _host

c = ctypes
_host.register({
    "bbh_alloc_new": (c.c_void_p, [c.c_uint32, c.c_uint32]),
    "bbh_alloc_free": (None, [c.c_void_p]),
    "bbh_alloc_free_blocks": (c.c_uint32, [c.c_void_p]),
    "bbh_alloc_refcount": (c.c_uint32, [c.c_void_p, c.c_uint32]),
    "bbh_alloc_alloc": (c.c_int64, [c.c_void_p]),
    "bbh_alloc_incref": (None, [c.c_void_p, c.c_uint32]),
    "bbh_alloc_decref": (c.c_int, [c.c_void_p, c.c_uint32]),
    "bbh_table_new": (c.c_void_p, []),
    "bbh_table_free": (None, [c.c_void_p]),
    "bbh_table_len": (c.c_uint32, [c.c_void_p]),
    "bbh_table_num_blocks": (c.c_uint32, [c.c_void_p]),
    "bbh_table_blocks": (None, [c.c_void_p, c.c_void_p]),
    "bbh_table_append": (c.c_int, [c.c_void_p, c.c_void_p, c.POINTER(c.c_uint32), c.POINTER(c.c_uint32)]),
    "bbh_table_reserve": (c.c_int64, [c.c_void_p, c.c_void_p, c.c_uint32]),
    "bbh_table_truncate": (None, [c.c_void_p, c.c_void_p, c.c_uint32]),
    "bbh_table_release": (None, [c.c_void_p, c.c_void_p]),
    "bbh_table_fork": (c.c_void_p, [c.c_void_p, c.c_void_p]),
    "bbh_table_unshare_tail": (c.c_int, [c.c_void_p, c.c_void_p, c.POINTER(c.c_uint32), c.POINTER(c.c_uint32)]),
    "bbh_table_adopt_prefix": (None, [c.c_void_p, c.c_void_p, c.c_void_p, c.c_uint32]),
    "bbh_prefix_new": (c.c_void_p, []),
    "bbh_prefix_free": (None, [c.c_void_p]),
    "bbh_prefix_len": (c.c_uint64, [c.c_void_p]),
    "bbh_prefix_lookup": (c.c_uint32, [c.c_void_p, c.c_void_p, c.c_uint64, c.c_uint32, c.c_uint64, c.c_void_p]),
    "bbh_prefix_insert_chain": (None, [c.c_void_p, c.c_void_p, c.c_void_p, c.c_uint64, c.c_void_p, c.c_uint32, c.c_uint32]),
    "bbh_prefix_evict": (c.c_uint32, [c.c_void_p, c.c_void_p, c.c_uint32]),
})


class BlockAllocator:
    def __init__(self, num_blocks: int, block_size: int):
        if num_blocks <= 0 or block_size <= 0:
            raise ValueError("num_blocks and block_size must be positive")
        self.block_size, self.num_blocks = block_size, num_blocks
        self._h = _host.lib().bbh_alloc_new(num_blocks, block_size)

    def __del__(self):
        if getattr(self, "_h", None):
            _host.lib().bbh_alloc_free(self._h)
            self._h = None

    def free_blocks(self) -> int:
        return int(_host.lib().bbh_alloc_free_blocks(self._h))

    def free_tokens(self) -> int:
        return self.free_blocks() * self.block_size

    def refcount(self, block: int) -> int:
        return int(_host.lib().bbh_alloc_refcount(self._h, block))

    def alloc(self) -> Optional[int]:
        b = int(_host.lib().bbh_alloc_alloc(self._h))
        return None if b < 0 else b

    def incref(self, block: int) -> None:
        _host.lib().bbh_alloc_incref(self._h, block)

    def decref(self, block: int) -> None:
        if _host.lib().bbh_alloc_decref(self._h, block) != 0:
            raise RuntimeError(f"double free of block {block}")


class BlockTable:
    def __init__(self, _h=None):
        self._h = _h if _h is not None else _host.lib().bbh_table_new()

    def __del__(self):
        if getattr(self, "_h", None):
            _host.lib().bbh_table_free(self._h)
            self._h = None

    def __len__(self) -> int:
        return int(_host.lib().bbh_table_len(self._h))

    def blocks(self) -> List[int]:
        n = int(_host.lib().bbh_table_num_blocks(self._h))
        out = np.empty(n, dtype=np.uint32)
        if n:
            _host.lib().bbh_table_blocks(self._h, out.ctypes.data)
        return out.tolist()

    def locate(self, tok: int, block_size: int) -> Tuple[int, int]:
        return self.blocks()[tok // block_size], tok % block_size

    def append(self, alloc: BlockAllocator) -> Tuple[int, int]:
        b, o = c.c_uint32(), c.c_uint32()
        if _host.lib().bbh_table_append(self._h, alloc._h, c.byref(b), c.byref(o)) != 0:
            raise MemoryError("paged KV pool exhausted")
        return b.value, o.value

    def reserve(self, n: int, alloc: BlockAllocator) -> int:
        start = int(_host.lib().bbh_table_reserve(self._h, alloc._h, n))
        if start < 0:
            raise MemoryError("paged KV pool exhausted")
        return start

    def truncate(self, new_len: int, alloc: BlockAllocator) -> None:
        if new_len > len(self):
            raise ValueError(f"truncate {new_len} > len {len(self)}")
        _host.lib().bbh_table_truncate(self._h, alloc._h, new_len)

    def release(self, alloc: BlockAllocator) -> None:
        _host.lib().bbh_table_release(self._h, alloc._h)

    def fork(self, alloc: BlockAllocator) -> "BlockTable":
        return BlockTable(_host.lib().bbh_table_fork(self._h, alloc._h))

    def unshare_tail(self, alloc: BlockAllocator) -> Optional[Tuple[int, int]]:
        o, n = c.c_uint32(), c.c_uint32()
        if _host.lib().bbh_table_unshare_tail(self._h, alloc._h, c.byref(o), c.byref(n)):
            return o.value, n.value
        return None

    def adopt_prefix(self, blocks, alloc: BlockAllocator) -> None:
        if len(self) != 0:
            raise ValueError("adopt_prefix expects a fresh sequence")
        arr = np.asarray(blocks, dtype=np.uint32)
        _host.lib().bbh_table_adopt_prefix(self._h, alloc._h, arr.ctypes.data, arr.size)


class PrefixCache:
    def __init__(self):
        self._h = _host.lib().bbh_prefix_new()

    def __del__(self):
        if getattr(self, "_h", None):
            _host.lib().bbh_prefix_free(self._h)
            self._h = None

    def __len__(self) -> int:
        return int(_host.lib().bbh_prefix_len(self._h))

    def lookup(self, prompt, block_size: int, max_tokens: int) -> List[int]:
        p = np.ascontiguousarray(np.asarray(prompt, dtype=np.uint32))
        out = np.empty(max(1, p.size // block_size), dtype=np.uint32)
        n = _host.lib().bbh_prefix_lookup(self._h, p.ctypes.data, p.size, block_size, max_tokens,
                                          out.ctypes.data)
        return out[:n].tolist()

    def insert_chain(self, prompt, blocks, start: int, alloc: BlockAllocator) -> None:
        self._alloc = alloc     # the native index is attached to this pool: keep the pool alive longer
        p = np.ascontiguousarray(np.asarray(prompt, dtype=np.uint32))
        b = np.ascontiguousarray(np.asarray(blocks, dtype=np.uint32))
        _host.lib().bbh_prefix_insert_chain(self._h, alloc._h, p.ctypes.data, p.size, b.ctypes.data,
                                            b.size, start)

    def evict(self, want: int, alloc: BlockAllocator) -> int:
        self._alloc = alloc
        return int(_host.lib().bbh_prefix_evict(self._h, alloc._h, want))
