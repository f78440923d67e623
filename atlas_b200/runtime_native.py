"""ctypes binding of the native host runtime (``csrc/runtime/*.cpp`` -> ``_C/libatlas_b200_runtime.so``): block pool,
radix tree, fault latch, direct-I/O reader.  :class:`NativeBlockPool` is a drop-in for ``kv.BlockPool`` (same method
names and exceptions); the engine uses it when ``ATLAS_NATIVE_RUNTIME=1``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Iterable, List, Optional, Sequence, Tuple

from .build import RUNTIME_LIB
from .kv.block_manager import OutOfBlocks

_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(RUNTIME_LIB):
            from . import build
            build.build_runtime()
        L = C.CDLL(RUNTIME_LIB)
        vp, i32p, u64p = C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_uint64)
        L.atlas_pool_create.restype = vp
        L.atlas_pool_create.argtypes = [C.c_int, C.c_int]
        L.atlas_pool_destroy.argtypes = [vp]
        for f in ("atlas_pool_num_free", "atlas_pool_check", "atlas_pool_block_size"):
            getattr(L, f).argtypes = [vp]
        L.atlas_pool_ref_count.argtypes = [vp, C.c_int]
        L.atlas_pool_alloc.argtypes = [vp, C.c_int, i32p]
        L.atlas_pool_inc_ref.argtypes = [vp, i32p, C.c_int]
        L.atlas_pool_free.argtypes = [vp, i32p, C.c_int]
        L.atlas_radix_create.restype = vp
        L.atlas_radix_create.argtypes = [vp]
        L.atlas_radix_destroy.argtypes = [vp]
        L.atlas_radix_match.argtypes = [vp, C.c_uint64, i32p, C.c_int, C.c_int, i32p, u64p, C.c_int]
        L.atlas_radix_release.argtypes = [vp, u64p, C.c_int]
        L.atlas_radix_insert.argtypes = [vp, C.c_uint64, i32p, C.c_int, i32p, C.c_int]
        L.atlas_radix_evict.argtypes = [vp, C.c_int]
        L.atlas_radix_num_nodes.argtypes = [vp]
        L.atlas_radix_evictable.argtypes = [vp]
        L.atlas_fault_trip.argtypes = [C.c_char_p]
        L.atlas_fault_reason.argtypes = [C.c_char_p, C.c_int]
        L.atlas_read_file.restype = C.c_longlong
        L.atlas_read_file.argtypes = [C.c_char_p, C.c_longlong, C.c_longlong, vp, C.c_int, C.c_longlong]
        L.atlas_uring_rw.restype = C.c_longlong
        L.atlas_uring_rw.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_longlong), C.POINTER(vp), C.c_longlong, C.c_int]
        _LIB = L
    return _LIB


def uring_available() -> bool:
    """True when the native runtime is built and this kernel / sandbox lets the process create an io_uring."""
    try:
        return bool(lib().atlas_uring_available())
    except (OSError, AttributeError):
        return False


def uring_rw(fd: int, write: bool, offsets: Sequence[int], addresses: Sequence[int], bytes_each: int, depth: int = 64) -> int:
    """``len(offsets)`` records of ``bytes_each`` between file offsets and host addresses, one batched submission."""
    n = len(offsets)
    if n == 0:
        return 0
    offs = (C.c_longlong * n)(*[int(o) for o in offsets])
    bufs = (C.c_void_p * n)(*[int(a) for a in addresses])
    r = lib().atlas_uring_rw(int(fd), 1 if write else 0, n, offs, bufs, int(bytes_each), int(depth))
    if r < 0:
        raise OSError(-r, os.strerror(-r))
    return int(r)


def _ints(xs: Sequence[int]):
    return (C.c_int * len(xs))(*xs)


class NativeBlockPool:
    def __init__(self, num_blocks: int, block_size: int):
        self.num_blocks, self.block_size = int(num_blocks), int(block_size)
        self._h = lib().atlas_pool_create(self.num_blocks, self.block_size)
        if not self._h:
            raise ValueError("bad pool geometry")
        self.high_water = 0

    def __del__(self):
        if getattr(self, "_h", None) and _LIB is not None:
            _LIB.atlas_pool_destroy(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return lib().atlas_pool_num_free(self._h)

    @property
    def num_used(self) -> int:
        return self.num_blocks - self.num_free

    def ref_count(self, block: int) -> int:
        return lib().atlas_pool_ref_count(self._h, block)

    def blocks_for_tokens(self, n_tokens: int) -> int:
        return (n_tokens + self.block_size - 1) // self.block_size

    def alloc(self, n: int = 1) -> List[int]:
        out = (C.c_int * max(1, n))()
        if lib().atlas_pool_alloc(self._h, n, out) != 0:
            raise OutOfBlocks(f"need {n} blocks, {self.num_free} free")
        self.high_water = max(self.high_water, self.num_used)
        return list(out[:n])

    def inc_ref(self, blocks: Iterable[int]) -> None:
        b = list(blocks)
        if b and lib().atlas_pool_inc_ref(self._h, _ints(b), len(b)) != 0:
            raise ValueError("inc_ref on a free block")

    def free(self, blocks: Iterable[int]) -> int:
        b = list(blocks)
        if not b:
            return 0
        r = lib().atlas_pool_free(self._h, _ints(b), len(b))
        if r < 0:
            raise ValueError("double free of a block")
        return r

    def check_invariants(self) -> None:
        rc = lib().atlas_pool_check(self._h)
        assert rc == 0, f"pool invariant broken ({rc})"


class NativeRadix:
    """Block-granular prefix index over a :class:`NativeBlockPool` (tokens in, block ids out)."""

    def __init__(self, pool: NativeBlockPool):
        self.pool = pool
        self._h = lib().atlas_radix_create(pool._h)

    def __del__(self):
        if getattr(self, "_h", None) and _LIB is not None:
            _LIB.atlas_radix_destroy(self._h)
            self._h = None

    def match(self, tokens: Sequence[int], namespace: int = 0, max_tokens: int = -1) -> Tuple[List[int], List[int]]:
        n = len(tokens)
        cap = max(1, n // self.pool.block_size)
        blocks, nodes = (C.c_int * cap)(), (C.c_uint64 * cap)()
        k = lib().atlas_radix_match(self._h, namespace, (C.c_int32 * max(1, n))(*tokens), n, max_tokens, blocks, nodes, cap)
        return list(blocks[:k]), list(nodes[:k])

    def release(self, nodes: Sequence[int]) -> None:
        if nodes:
            lib().atlas_radix_release(self._h, (C.c_uint64 * len(nodes))(*nodes), len(nodes))

    def insert(self, tokens: Sequence[int], blocks: Sequence[int], namespace: int = 0) -> int:
        return lib().atlas_radix_insert(self._h, namespace, (C.c_int32 * max(1, len(tokens)))(*tokens), len(tokens),
                                        _ints(list(blocks)) if blocks else (C.c_int * 1)(), len(blocks))

    def evict(self, want: int) -> int:
        return lib().atlas_radix_evict(self._h, want)

    @property
    def num_nodes(self) -> int:
        return lib().atlas_radix_num_nodes(self._h)

    def evictable_blocks(self) -> int:
        return lib().atlas_radix_evictable(self._h)


def fault_trip(reason: str) -> bool:
    return bool(lib().atlas_fault_trip(reason.encode()))


def fault_tripped() -> bool:
    return bool(lib().atlas_fault_tripped())


def fault_reason() -> Optional[str]:
    buf = C.create_string_buffer(1024)
    return buf.value.decode() if lib().atlas_fault_reason(buf, 1024) else None


def read_file_into(path: str, offset: int, length: int, dst_ptr: int, threads: int = 8, chunk: int = 8 << 20) -> int:
    """Direct-I/O read of ``[offset, offset+length)`` into the memory at ``dst_ptr``; returns the bytes read."""
    r = lib().atlas_read_file(path.encode(), offset, length, dst_ptr, threads, chunk)
    if r < 0:
        raise OSError(-r, os.strerror(-r), path)
    return int(r)
