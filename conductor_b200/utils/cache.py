"""Compile cache: graph hash -> compiled artifact.

Counterpart of the reference's ``conductor/utils/cache.py:25-295`` (a pickle-on-disk cache of
``.so`` artifacts, LRU by last access, size cap).  Plans here are built in well under a
millisecond from the prebuilt kernel library, so the cache lives in memory only: it exists to
make recompiles of an already-seen graph free and to give ``GCUBackend`` the reference's
get / put / stats surface.  Keys must include dtypes, strides and device kind (the reference
hashes names and shapes only); ``ChoreoJITCompiler._generate_graph_hash`` does.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Optional


class CompilationCache:
    def __init__(self, max_entries: int = 256, enabled: bool = True):
        self.max_entries = max(1, int(max_entries))
        self.enabled = enabled
        self._entries: "OrderedDict[str, Any]" = OrderedDict()
        self.hits = 0
        self.misses = 0
        self.evictions = 0

    def get(self, key: str) -> Optional[Any]:
        if not self.enabled:
            return None
        item = self._entries.get(key)
        if item is None:
            self.misses += 1
            return None
        self._entries.move_to_end(key)          # LRU by last access, as the reference
        self.hits += 1
        return item

    def put(self, key: str, artifact: Any) -> None:
        if not self.enabled:
            return
        self._entries[key] = artifact
        self._entries.move_to_end(key)
        while len(self._entries) > self.max_entries:
            self._entries.popitem(last=False)
            self.evictions += 1

    def __contains__(self, key: str) -> bool:
        return self.enabled and key in self._entries

    def __len__(self) -> int:
        return len(self._entries)

    def clear(self) -> None:
        self._entries.clear()

    def get_stats(self) -> dict:
        total = self.hits + self.misses
        return {"entries": len(self._entries), "hits": self.hits, "misses": self.misses,
                "evictions": self.evictions, "hit_rate": (self.hits / total) if total else 0.0}
