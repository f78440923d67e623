"""Radix-tree prefix cache over block-sized token chunks, with recurrent-state snapshots.

Every tree edge is one full KV block keyed by its ``block_size`` token ids, so a lookup walks the
prompt block by block and returns the physical blocks that already hold that prefix.  The tree owns
one reference on each cached block; sequences that reuse a prefix take their own reference and pin
the nodes they use.  Unpinned leaves are evicted least-recently-used first.

Hybrid (Gated DeltaNet) models cannot resume from KV alone: a prefix is only reusable at depths where
a snapshot of the recurrent state was stored.  Snapshots live in a small slot pool that is decoupled
from the tree (a node holds at most a slot id); the pool has its own LRU.

Namespaces (LoRA adapter id, session / ``prompt_cache_key`` salt) get separate roots.

Reference parity: ``crates/spark-runtime/src/radix_tree.rs:1-70``, ``radix_tree/inner/{evict,lru_index}.rs``,
``radix_tree/snapshot*.rs`` (Marconi snapshot index), ``prefix_cache.rs:104-260``.
"""
from __future__ import annotations

import heapq
import itertools
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

from .block_manager import BlockPool, SlotPool


class RadixNode:
    __slots__ = ("key", "block", "parent", "children", "pins", "last_access", "snapshot", "depth")

    def __init__(self, key, block, parent, depth):
        self.key, self.block, self.parent, self.depth = key, block, parent, depth
        self.children: Dict[tuple, "RadixNode"] = {}
        self.pins = 0
        self.last_access = 0
        self.snapshot: Optional[int] = None


@dataclass
class PrefixMatch:
    blocks: List[int] = field(default_factory=list)
    nodes: List[RadixNode] = field(default_factory=list)
    num_tokens: int = 0
    snapshot_slot: Optional[int] = None


@dataclass
class PrefixCacheStats:
    lookups: int = 0
    hits: int = 0
    hit_tokens: int = 0
    lookup_tokens: int = 0
    inserted_blocks: int = 0
    evicted_blocks: int = 0
    snapshot_hits: int = 0
    snapshot_evictions: int = 0


class RadixCache:
    def __init__(self, pool: BlockPool, snapshot_slots: int = 0,
                 on_snapshot_free: Optional[Callable[[int], None]] = None):
        self.pool = pool
        self.bs = pool.block_size
        self.roots: Dict[Hashable, RadixNode] = {}
        self._clock = itertools.count(1)
        self.stats = PrefixCacheStats()
        self.num_nodes = 0
        self.snap_pool = SlotPool(snapshot_slots) if snapshot_slots > 0 else None
        self._snap_owner: Dict[int, RadixNode] = {}
        self._on_snapshot_free = on_snapshot_free

    # ------------------------------------------------------------------ lookup
    def _root(self, ns: Hashable) -> RadixNode:
        r = self.roots.get(ns)
        if r is None:
            r = self.roots[ns] = RadixNode((), -1, None, 0)
        return r

    def match(self, tokens: Sequence[int], namespace: Hashable = 0, need_snapshot: bool = False,
              max_tokens: Optional[int] = None) -> PrefixMatch:
        """Longest cached prefix of ``tokens`` in whole blocks, leaving at least one token to compute.

        The caller receives one pool reference per returned block and a pin on every returned node;
        give them back with :meth:`release` (pins) and ``pool.free`` (blocks).
        """
        self.stats.lookups += 1
        self.stats.lookup_tokens += len(tokens)
        limit = len(tokens) - 1 if max_tokens is None else min(max_tokens, len(tokens) - 1)
        node = self._root(namespace)
        path: List[RadixNode] = []
        now = next(self._clock)
        i = 0
        while i + self.bs <= limit:
            child = node.children.get(tuple(tokens[i:i + self.bs]))
            if child is None:
                break
            child.last_access = now
            path.append(child)
            node = child
            i += self.bs
        snap = None
        if need_snapshot:
            while path and path[-1].snapshot is None:
                path.pop()
            if path:
                snap = path[-1].snapshot
                self.stats.snapshot_hits += 1
        m = PrefixMatch([n.block for n in path], path, len(path) * self.bs, snap)
        if path:
            self.stats.hits += 1
            self.stats.hit_tokens += m.num_tokens
            self.pool.inc_ref(m.blocks)
            for n in path:
                n.pins += 1
        return m

    def release(self, nodes: Sequence[RadixNode]) -> None:
        for n in nodes:
            assert n.pins > 0
            n.pins -= 1

    # ------------------------------------------------------------------ insert
    def insert(self, tokens: Sequence[int], blocks: Sequence[int], namespace: Hashable = 0) -> List[RadixNode]:
        """Publish the full blocks of a sequence.  ``blocks[j]`` holds tokens ``[j*bs, (j+1)*bs)``.

        New nodes take their own reference on the block.  Where the tree already has the chunk, the
        existing block is kept (the caller's duplicate stays private to it).  Returns the node path.
        """
        node = self._root(namespace)
        now = next(self._clock)
        path = []
        nfull = min(len(tokens) // self.bs, len(blocks))
        for j in range(nfull):
            key = tuple(tokens[j * self.bs:(j + 1) * self.bs])
            child = node.children.get(key)
            if child is None:
                child = RadixNode(key, blocks[j], node, node.depth + 1)
                node.children[key] = child
                self.pool.inc_ref([blocks[j]])
                self.num_nodes += 1
                self.stats.inserted_blocks += 1
            child.last_access = now
            path.append(child)
            node = child
        return path

    # ------------------------------------------------------------------ snapshots
    def attach_snapshot(self, node: RadixNode) -> Optional[int]:
        """Reserve a snapshot slot for ``node`` (evicting the least-recently-used snapshot if the pool
        is full).  The caller copies the recurrent state into the returned slot."""
        if self.snap_pool is None:
            return None
        if node.snapshot is not None:
            return node.snapshot
        slot = self.snap_pool.alloc()
        if slot is None:
            victim = min((n for n in self._snap_owner.values() if n.pins == 0), key=lambda n: n.last_access, default=None)
            if victim is None:
                return None
            slot = victim.snapshot
            victim.snapshot = None
            del self._snap_owner[slot]
            self.stats.snapshot_evictions += 1
        node.snapshot = slot
        self._snap_owner[slot] = node
        return slot

    def _drop_snapshot(self, node: RadixNode) -> None:
        if node.snapshot is not None:
            slot = node.snapshot
            node.snapshot = None
            self._snap_owner.pop(slot, None)
            self.snap_pool.free(slot)
            if self._on_snapshot_free:
                self._on_snapshot_free(slot)

    # ------------------------------------------------------------------ eviction
    def evictable_blocks(self) -> int:
        """Blocks that eviction could return to the pool right now (unpinned subtrees whose blocks are
        referenced only by the tree)."""
        n = 0
        for root in self.roots.values():
            stack = list(root.children.values())
            while stack:
                x = stack.pop()
                if x.pins == 0 and self.pool.ref_count(x.block) == 1:
                    n += 1
                stack.extend(x.children.values())
        return n

    def evict(self, num_blocks: int) -> int:
        """Evict unpinned leaves, least recently used first, until ``num_blocks`` blocks were returned
        to the pool or nothing evictable is left.  Returns the number of blocks actually freed."""
        heap: List[Tuple[int, int, RadixNode]] = []
        tie = itertools.count()
        for root in self.roots.values():
            stack = list(root.children.values())
            while stack:
                x = stack.pop()
                if x.children:
                    stack.extend(x.children.values())
                elif x.pins == 0:
                    heapq.heappush(heap, (x.last_access, next(tie), x))
        freed = 0
        while heap and freed < num_blocks:
            _, _, leaf = heapq.heappop(heap)
            if leaf.children or leaf.pins:
                continue
            parent = leaf.parent
            del parent.children[leaf.key]
            self._drop_snapshot(leaf)
            freed += self.pool.free([leaf.block])
            self.num_nodes -= 1
            self.stats.evicted_blocks += 1
            if parent.parent is not None and not parent.children and parent.pins == 0:
                heapq.heappush(heap, (parent.last_access, next(tie), parent))
        return freed

    def clear(self) -> int:
        return self.evict(1 << 60)
