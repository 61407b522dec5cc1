"""Background page population for freshly created cache files.

A new file in memory-backed storage has no pages; the first store to each 4 KB page makes the kernel allocate and
zero it, and for ONE file that proceeds at a few GB/s however many threads write.  Different files populate in
parallel.  The cache writer therefore hands the mappings of all the files it has just created to a small pool of
threads that walk them round-robin with ``madvise(MADV_POPULATE_WRITE)`` while the caller is still encoding: by the
time the writer's cursor reaches a later shard its pages exist, and the row copies run at memory-copy speed.
Population never changes file contents (new pages are zero, existing pages are left alone).
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import List, Optional, Sequence, Tuple

_MADV_POPULATE_WRITE = 23
_CHUNK = 32 << 20
_MEMORY_FILESYSTEMS = ("tmpfs", "ramfs", "hugetlbfs", "devtmpfs")
MEM_FRACTION_FOR_PREFAULT = 0.5   # automatic mode populates ahead only when the new files fit this share of MemAvailable

_libc = None


def _madvise(addr: int, length: int) -> int:
    global _libc
    if _libc is None:
        _libc = ctypes.CDLL(None, use_errno=True)
        _libc.madvise.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        _libc.madvise.restype = ctypes.c_int
    return _libc.madvise(ctypes.c_void_p(addr), ctypes.c_size_t(length), _MADV_POPULATE_WRITE)


def filesystem_type(path: str) -> Optional[str]:
    """File-system type of the mount that holds ``path`` (longest mount-point prefix in /proc/mounts)."""
    try:
        real = os.path.realpath(path)
        best, kind = "", None
        with open("/proc/mounts", "r") as f:
            for line in f:
                parts = line.split()
                if len(parts) < 3:
                    continue
                mp = parts[1].replace("\\040", " ")
                if (real == mp or real.startswith(mp.rstrip("/") + "/")) and len(mp) > len(best):
                    best, kind = mp, parts[2]
        return kind
    except OSError:
        return None


def in_memory_filesystem(path: str) -> bool:
    return filesystem_type(path) in _MEMORY_FILESYSTEMS


def prefault_threads() -> int:
    """Half of this process's share of the cores, at most 8 (the row copies need the other half);
    ``TCB_PREFAULT_THREADS`` overrides it."""
    try:
        forced = int(os.environ.get("TCB_PREFAULT_THREADS", "0"))
    except ValueError:
        forced = 0
    if forced > 0:
        return min(forced, 64)
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        local_ranks = int(os.environ.get("LOCAL_WORLD_SIZE") or os.environ.get("WORLD_SIZE") or 1)
    except ValueError:
        local_ranks = 1
    return max(1, min(8, n // max(1, local_ranks) // 2))


class Prefaulter:
    """Populates ``(address, nbytes)`` ranges in the background, one chunk of each range in turn, so that the worker
    threads are spread over as many files as there are.  ``stop()`` must be called before the ranges are unmapped."""

    def __init__(self, ranges: Sequence[Tuple[int, int]], threads: Optional[int] = None):
        tasks: List[Tuple[int, int]] = []
        spans = [(a, n) for a, n in ranges if n > 0]
        most = max((n for _, n in spans), default=0)
        for off in range(0, most, _CHUNK):
            for a, n in spans:
                if off < n:
                    tasks.append((a + off, min(_CHUNK, n - off)))
        self._tasks = tasks
        self._next = 0
        self._lock = threading.Lock()
        self._stop = False
        self.failed = False
        self.populated = 0
        k = min(threads or prefault_threads(), max(1, len(tasks)))
        self._threads = [threading.Thread(target=self._run, name=f"tcb-prefault-{i}", daemon=True) for i in range(k)]
        for t in self._threads:
            t.start()

    def _run(self) -> None:
        while True:
            with self._lock:
                if self._stop or self._next >= len(self._tasks):
                    return
                addr, n = self._tasks[self._next]
                self._next += 1
            if _madvise(addr, n) != 0:
                self.failed = True      # an older kernel or a file system that refuses: the writer populates block by block
                with self._lock:
                    self._stop = True
                return
            with self._lock:
                self.populated += n

    def done(self) -> bool:
        return all(not t.is_alive() for t in self._threads)

    def stop(self) -> None:
        with self._lock:
            self._stop = True
        for t in self._threads:
            t.join()
