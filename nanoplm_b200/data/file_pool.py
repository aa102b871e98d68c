"""Thread-safe LRU pool of open file handles (reference: src/nanoplm/data/file_pool.py:19-207).
Used by the pre-computed distillation dataset so DataLoader workers and prefetch threads share a
bounded number of open shard files. Handles are dropped on pickling."""
from __future__ import annotations

import resource
import threading
from collections import OrderedDict
from typing import Callable


def detect_file_limits(num_workers: int = 1, fraction: float = 0.7, minimum: int = 5) -> int:
    """Files each worker may keep open: fraction of RLIMIT_NOFILE split over workers, >= minimum."""
    try:
        soft, _ = resource.getrlimit(resource.RLIMIT_NOFILE)
    except (ValueError, OSError):
        soft = 1024
    if soft <= 0 or soft == resource.RLIM_INFINITY:
        soft = 4096
    return max(minimum, int(soft * fraction) // max(1, num_workers))


class ThreadSafeFileHandlePool:
    def __init__(self, max_open_files: int = 5, opener: Callable | None = None):
        if max_open_files < 1:
            raise ValueError("max_open_files must be >= 1")
        self.max_open_files = max_open_files
        self._opener = opener
        self._handles: "OrderedDict[str, object]" = OrderedDict()
        self._lock = threading.RLock()
        self.hits = self.misses = self.evictions = 0

    def _open(self, path: str):
        if self._opener is not None:
            return self._opener(path)
        import h5py
        return h5py.File(path, "r")

    def get(self, path: str):
        path = str(path)
        with self._lock:
            if path in self._handles:
                self.hits += 1
                self._handles.move_to_end(path)
                return self._handles[path]
            self.misses += 1
            while len(self._handles) >= self.max_open_files:
                _, old = self._handles.popitem(last=False)
                self.evictions += 1
                try:
                    old.close()
                except Exception:
                    pass
            h = self._open(path)
            self._handles[path] = h
            return h

    def close_all(self) -> None:
        with self._lock:
            for h in self._handles.values():
                try:
                    h.close()
                except Exception:
                    pass
            self._handles.clear()

    def stats(self) -> dict:
        total = self.hits + self.misses
        return {"hits": self.hits, "misses": self.misses, "evictions": self.evictions,
                "open": len(self._handles), "hit_rate": self.hits / total if total else 0.0}

    def __len__(self) -> int:
        return len(self._handles)

    def __getstate__(self):
        return {"max_open_files": self.max_open_files, "opener": self._opener}

    def __setstate__(self, state):
        self.__init__(state["max_open_files"], state["opener"])

    def __del__(self):
        try:
            self.close_all()
        except Exception:
            pass
