"""Stateful API stores: stored chat completions / responses (LRU + TTL), conversations, sessions.

Reference parity: ``crates/spark-server/src/{response_store,conversation_store,session_manager}.rs``.
"""
from __future__ import annotations

import threading
import time
import uuid
from collections import OrderedDict
from typing import Any, Dict, List, Optional


class LruTtlStore:
    def __init__(self, capacity: int = 1024, ttl_s: float = 3600.0):
        self.capacity, self.ttl_s = capacity, ttl_s
        self._d: "OrderedDict[str, tuple]" = OrderedDict()
        self._lock = threading.Lock()

    def put(self, key: str, value: Any) -> None:
        with self._lock:
            self._d[key] = (time.time(), value)
            self._d.move_to_end(key)
            while len(self._d) > self.capacity:
                self._d.popitem(last=False)

    def get(self, key: str) -> Optional[Any]:
        with self._lock:
            item = self._d.get(key)
            if item is None:
                return None
            if time.time() - item[0] > self.ttl_s:
                del self._d[key]
                return None
            self._d.move_to_end(key)
            return item[1]

    def delete(self, key: str) -> bool:
        with self._lock:
            return self._d.pop(key, None) is not None

    def __len__(self) -> int:
        return len(self._d)


class ConversationStore:
    def __init__(self, capacity: int = 1024):
        self._c = LruTtlStore(capacity, ttl_s=30 * 24 * 3600.0)

    def create(self, items: Optional[List[dict]] = None, metadata: Optional[dict] = None) -> dict:
        cid = "conv_" + uuid.uuid4().hex
        conv = {"id": cid, "object": "conversation", "created_at": int(time.time()), "metadata": metadata or {},
                "items": []}
        self._c.put(cid, conv)
        if items:
            self.add_items(cid, items)
        return conv

    def get(self, cid: str) -> Optional[dict]:
        return self._c.get(cid)

    def update(self, cid: str, metadata: dict) -> Optional[dict]:
        c = self._c.get(cid)
        if c is not None:
            c["metadata"] = metadata
        return c

    def delete(self, cid: str) -> bool:
        return self._c.delete(cid)

    def add_items(self, cid: str, items: List[dict]) -> Optional[List[dict]]:
        c = self._c.get(cid)
        if c is None:
            return None
        added = []
        for it in items:
            it = dict(it)
            it.setdefault("id", "msg_" + uuid.uuid4().hex[:24])
            it.setdefault("type", "message")
            c["items"].append(it)
            added.append(it)
        return added

    def delete_item(self, cid: str, item_id: str) -> bool:
        c = self._c.get(cid)
        if c is None:
            return False
        n = len(c["items"])
        c["items"] = [i for i in c["items"] if i.get("id") != item_id]
        return len(c["items"]) != n


class SessionManager:
    """Maps a client-supplied session / ``prompt_cache_key`` to a prefix-cache namespace salt."""

    def __init__(self):
        self._salts: Dict[str, int] = {}

    def namespace(self, key: Optional[str]) -> int:
        if not key:
            return 0
        if key not in self._salts:
            self._salts[key] = len(self._salts) + 1
        return self._salts[key]
