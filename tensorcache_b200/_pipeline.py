"""Shared host logic of the batch readers: cache manifests, shard maps, and the
Python handle of the native double-buffered pipeline (``tcb_streamer_*``)."""
from __future__ import annotations

import ctypes
import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import List, Optional

import numpy as np
import torch

from . import _lib


@dataclass
class ShardFiles:
    """One file set ``<prefix>_int8.bin / _scales.bin / _zp.bin`` opened read-only.  A cache of the
    symmetric codec (``amo_bq`` false) holds int8 codes and has no ``_zp.bin``; ``zp`` stays None."""
    prefix: str
    num_samples: int
    q: Optional[np.memmap] = None      # uint8 (AMO-BQ) or int8 (symmetric) [n, seq, dim]
    s: Optional[np.memmap] = None      # uint16 [n, groups] (bf16 bit patterns)
    zp: Optional[np.memmap] = None     # uint8 [n, groups]


@dataclass
class CacheLayout:
    """What a reader needs to know about a cache on disk (the file format written by
    src/tensorcache/feature_cache.py:85-127, 134-155, 446-540 of TensorCache)."""
    meta: dict
    seq_len: int
    dim: int
    group_size: int
    amo_bq: bool
    shards: List[ShardFiles] = field(default_factory=list)
    total_shards_on_disk: int = 1
    selected: Optional[List[int]] = None   # shard numbers opened, None = unsharded cache
    private: bool = False                   # mapped copy-on-write so that the mappings can be page-locked
    pinned_ranges: List[int] = field(default_factory=list)   # start addresses of the page-locked mappings
    pinned_device: Optional[object] = None

    @property
    def groups_per_sample(self) -> int:
        return (self.seq_len * self.dim + self.group_size - 1) // self.group_size

    @property
    def num_samples(self) -> int:
        return sum(s.num_samples for s in self.shards)

    @property
    def shard_sizes(self) -> List[int]:
        return [s.num_samples for s in self.shards]

    @property
    def shard_offsets(self) -> List[int]:
        off, out = 0, []
        for s in self.shards:
            out.append(off)
            off += s.num_samples
        return out

    def locate(self, idx: int):
        """global sample -> (position in self.shards, local row)"""
        if idx < 0:
            idx += self.num_samples
        if not 0 <= idx < self.num_samples:
            raise IndexError(f"idx {idx} out of range {self.num_samples}")
        for si, (off, sh) in enumerate(zip(self.shard_offsets, self.shards)):
            if off <= idx < off + sh.num_samples:
                return si, idx - off
        raise IndexError(idx)

    @property
    def nbytes(self) -> int:
        """Bytes of the opened shard files."""
        return sum(a.nbytes for sh in self.shards if sh.num_samples > 0 for a in (sh.q, sh.s, sh.zp) if a is not None)

    def pin(self, device) -> None:
        """Page-locks the mapped shard files (once; needs ``private`` mappings) so that the copy engine and the
        gather kernel read them in place.  Costs the shards' size in host memory and about 0.4 s per GB."""
        if self.pinned_ranges:
            return
        if not self.private:
            raise ValueError("page-locking needs a cache opened with private=True (copy-on-write mappings)")
        import torch
        with torch.cuda.device(device):
            try:
                for sh in self.shards:
                    if sh.num_samples == 0:
                        continue
                    for arr in (sh.q, sh.s, sh.zp):
                        if arr is None:
                            continue
                        nbytes = (arr.nbytes + 4095) // 4096 * 4096   # the mapping covers whole pages
                        _lib.check(_lib.lib().tcb_pin_host_range(ctypes.c_void_p(arr.ctypes.data), nbytes))
                        self.pinned_ranges.append(arr.ctypes.data)
            except Exception:
                self.unpin()
                raise
        self.pinned_device = device

    def unpin(self) -> None:
        if not self.pinned_ranges:
            return
        import torch
        ctx = torch.cuda.device(self.pinned_device) if self.pinned_device is not None and torch.cuda.is_available() else None
        if ctx is not None:
            ctx.__enter__()
        try:
            for addr in self.pinned_ranges:
                _lib.lib().tcb_unpin_host_range(ctypes.c_void_p(addr))
        finally:
            if ctx is not None:
                ctx.__exit__(None, None, None)
        self.pinned_ranges = []

    def close(self):
        self.unpin()
        for sh in self.shards:
            for name in ("q", "s", "zp"):
                mm = getattr(sh, name)
                if mm is not None and getattr(mm, "_mmap", None) is not None:
                    try:
                        mm._mmap.close()
                    except (BufferError, ValueError):
                        pass
                setattr(sh, name, None)


def _open_shard(prefix: str, n: int, seq_len: int, dim: int, groups: int, amo_bq: bool, private: bool = False) -> ShardFiles:
    sh = ShardFiles(prefix, n)
    if n > 0:
        expect = {"_int8.bin": n * seq_len * dim, "_scales.bin": n * groups * 2}
        if amo_bq:
            expect["_zp.bin"] = n * groups
        for suffix, nbytes in expect.items():
            path = prefix + suffix
            if not os.path.exists(path):
                raise FileNotFoundError(f"cache file {path!r} is missing")
            have = os.path.getsize(path)
            if have < nbytes:
                raise ValueError(f"cache file {path!r} is truncated: {have} bytes, {nbytes} needed for {n} samples")
        # "c" = private copy-on-write mapping: never written here, but the only kind of file mapping
        # the CUDA driver agrees to page-lock (resident-shard mode of the readers)
        mode = "c" if private else "r"
        sh.q = np.memmap(prefix + "_int8.bin", dtype=np.uint8 if amo_bq else np.int8, mode=mode, shape=(n, seq_len, dim))
        sh.s = np.memmap(prefix + "_scales.bin", dtype=np.uint16, mode=mode, shape=(n, groups))
        if amo_bq:
            sh.zp = np.memmap(prefix + "_zp.bin", dtype=np.uint8, mode=mode, shape=(n, groups))
    return sh


def resolve_shards(num_shards: int, shard_idx: Optional[int], rank: Optional[int], world_size: Optional[int],
                   all_rank_shards: bool) -> Optional[List[int]]:
    """Which shard numbers a reader opens.  None means "all of them, as one logical cache".

    rank / world_size follow ZeroCopyTensorStreamer (src/tensorcache/streamer.py:69-71):
    shard ``rank % num_shards``.  With ``all_rank_shards`` a rank instead takes every
    shard i with ``i % world_size == rank`` -- the two rules agree when
    ``world_size == num_shards``; the second leaves no shard unread when there are
    fewer ranks than shards.
    """
    if rank is not None and world_size is not None:
        if shard_idx is not None:
            raise ValueError("Specify either shard_idx or rank/world_size, not both")
        if world_size < 1 or not 0 <= rank < world_size:
            raise ValueError(f"rank {rank} outside world_size {world_size}")
        if all_rank_shards:
            return [i for i in range(num_shards) if i % world_size == rank]
        return [rank % num_shards]
    if shard_idx is not None:
        if not 0 <= shard_idx < num_shards:
            raise ValueError(f"shard_idx {shard_idx} out of range {num_shards}")
        return [shard_idx]
    return None


def open_cache(cache_prefix, shard_idx=None, rank=None, world_size=None, all_rank_shards=False, private=False) -> CacheLayout:
    """Parses ``<prefix>_shards.json`` or ``<prefix>_meta.json`` and maps the files."""
    prefix = str(cache_prefix)
    manifest_path = prefix + "_shards.json"
    if os.path.exists(manifest_path):
        with open(manifest_path, "r") as f:
            man = json.load(f)
        n_shards = man.get("num_shards", len(man.get("shard_prefixes", [])))
        prefixes = list(man.get("shard_prefixes") or [f"{prefix}_shard{i}" for i in range(n_shards)])
        # a cache that was moved after it was written: fall back to files beside the manifest
        for i, p in enumerate(prefixes):
            if not os.path.exists(p + "_meta.json") and not os.path.exists(p + "_int8.bin"):
                prefixes[i] = f"{prefix}_shard{i}"
        selected = resolve_shards(n_shards, shard_idx, rank, world_size, all_rank_shards)
        seq_len, dim, G = man["seq_len"], man["dim"], man["group_size"]
        amo = man.get("amo_bq", False)
        groups = (seq_len * dim + G - 1) // G
        sizes = list(man.get("shard_sizes") or [])
        lay = CacheLayout(man, seq_len, dim, G, amo, [], n_shards, selected if selected is not None else list(range(n_shards)),
                          private)
        for i in lay.selected:
            n = None
            mp = prefixes[i] + "_meta.json"
            if os.path.exists(mp):
                with open(mp, "r") as f:
                    sm = json.load(f)
                n = sm["num_samples"]
                if selected is not None and len(selected) == 1:
                    lay.meta = sm
            if n is None:
                n = sizes[i] if sizes else man["num_samples"] // n_shards
            lay.shards.append(_open_shard(prefixes[i], n, seq_len, dim, groups, amo, private))
        return lay
    # rank / world_size on an unsharded cache are ignored, as the reference's streamer does
    if shard_idx not in (None, 0):
        raise ValueError(f"shard_idx {shard_idx} out of range 1")
    meta_path = prefix + "_meta.json"
    with open(meta_path, "r") as f:
        meta = json.load(f)
    seq_len, dim, G = meta["seq_len"], meta["dim"], meta["group_size"]
    amo = meta.get("amo_bq", False)
    groups = (seq_len * dim + G - 1) // G
    lay = CacheLayout(meta, seq_len, dim, G, amo, [], 1, None, private)
    lay.shards.append(_open_shard(prefix, meta["num_samples"], seq_len, dim, groups, amo, private))
    return lay


def default_gather_threads() -> int:
    """Gather workers per reader: the cores this process may use, shared between the ranks of the
    node when a launcher says how many there are (LOCAL_WORLD_SIZE / WORLD_SIZE), at most 8."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        local_ranks = int(os.environ.get("LOCAL_WORLD_SIZE") or os.environ.get("WORLD_SIZE") or 1)
    except ValueError:
        local_ranks = 1
    return max(1, min(8, n // max(1, local_ranks) - 1))


def writer_threads() -> int:
    """Copy workers of the cache writer: this process's share of the cores, at most 16."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        local_ranks = int(os.environ.get("LOCAL_WORLD_SIZE") or os.environ.get("WORLD_SIZE") or 1)
    except ValueError:
        local_ranks = 1
    return max(1, min(16, n // max(1, local_ranks)))


MEM_FRACTION_FOR_RESIDENT_SHARDS = 0.25   # automatic mode page-locks shards only up to this share of MemAvailable


def _mem_available_bytes() -> Optional[int]:
    try:
        with open("/proc/meminfo", "r") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) * 1024
    except (OSError, ValueError, IndexError):
        pass
    return None


def try_make_resident(layout: CacheLayout, device: torch.device, wanted: Optional[bool]) -> bool:
    """Decides the reader mode.  ``wanted`` True: page-lock the opened shards or raise.  False: never.
    None (automatic): page-lock them when they fit ``MEM_FRACTION_FOR_RESIDENT_SHARDS`` of the host memory that is
    available right now and the driver agrees; otherwise say why in one warning and let the reader copy
    rows through page-locked staging as the reference does."""
    if wanted is False or layout.num_samples == 0:
        return False
    if layout.pinned_ranges:
        return True
    if wanted:
        layout.pin(device)
        return True
    import warnings
    avail = _mem_available_bytes()
    need = layout.nbytes
    if avail is not None and need > MEM_FRACTION_FOR_RESIDENT_SHARDS * avail:
        warnings.warn(f"tensorcache_b200: the opened shard(s) hold {need / 2**30:.1f} GiB, more than "
                      f"{MEM_FRACTION_FOR_RESIDENT_SHARDS:.0%} of the {avail / 2**30:.1f} GiB of host memory available; "
                      "reading through page-locked staging copies instead of keeping the shard page-locked", stacklevel=3)
        return False
    try:
        layout.pin(device)
        return True
    except Exception as e:   # the driver refused (memlock limit, unsupported mapping): the staging mode still works
        warnings.warn(f"tensorcache_b200: could not page-lock the shard files ({e}); reading through page-locked "
                      "staging copies instead", stacklevel=3)
        return False


class NativePipeline:
    """Owns the ring buffers (torch tensors) and the native streamer handle.  With ``pin_shards`` the shard
    files must already be page-locked (``CacheLayout.pin``); the copies then start from the mappings."""

    def __init__(self, layout: CacheLayout, batch_size: int, device: torch.device, n_slots: int,
                 n_threads: Optional[int] = None, pin_shards: bool = False):
        if device.type != "cuda":
            raise RuntimeError("the batch readers decode on a CUDA device only (no CPU decode path)")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device available for the batch reader")
        self.layout = layout
        self.device = device
        self.batch_size = int(batch_size)
        self.n_slots = int(n_slots)
        vps = layout.seq_len * layout.dim
        gps = layout.groups_per_sample
        B = self.batch_size
        self.pin_shards = bool(pin_shards)
        if self.pin_shards and not layout.pinned_ranges and layout.num_samples > 0:
            layout.pin(device)
        # One page-locked block and one device block per ring slot, laid out [codes | scales | zero points], so that a
        # full batch crosses PCIe as one copy.  The staging copy of the codes is not needed when the copy engine reads
        # the shard itself.
        amo = layout.amo_bq
        qdt = torch.uint8 if amo else torch.int8
        qb, sb, zb = B * vps, B * gps * 2, (B * gps if amo else 0)
        qb_pad, sb_pad = (qb + 255) // 256 * 256, (sb + 255) // 256 * 256
        contiguous = qb_pad == qb and sb_pad == sb     # otherwise the three arrays keep their own 256-byte alignment
        self._contiguous_slots = contiguous

        def carve(block, with_q):
            off = 0
            q = s = z = None
            if with_q:
                q = block[off:off + qb].view(qdt).view(B, layout.seq_len, layout.dim)
                off += qb_pad
            s = block[off:off + sb].view(torch.bfloat16).view(B, gps)
            off += sb_pad
            if amo:
                z = block[off:off + zb].view(B, gps)
            return q, s, z

        self._pinned_blocks, self._dev_blocks = [], []
        self.pinned_q, self.pinned_s, self.pinned_zp = [], [], ([] if amo else None)
        self.dev_q, self.dev_s, self.dev_zp = [], [], ([] if amo else None)
        for _ in range(n_slots):
            hb = torch.empty((0 if self.pin_shards else qb_pad) + sb_pad + zb, dtype=torch.uint8, pin_memory=True)
            db = torch.empty(qb_pad + sb_pad + zb, dtype=torch.uint8, device=device)
            self._pinned_blocks.append(hb)
            self._dev_blocks.append(db)
            hq, hs, hz = carve(hb, not self.pin_shards)
            dq, ds, dz = carve(db, True)
            if hq is not None:
                self.pinned_q.append(hq)
            self.pinned_s.append(hs)
            self.dev_q.append(dq)
            self.dev_s.append(ds)
            if amo:
                self.pinned_zp.append(hz)
                self.dev_zp.append(dz)
        self.dev_out = [torch.empty((B, layout.seq_len, layout.dim), dtype=torch.bfloat16, device=device) for _ in range(n_slots)]

        def table(tensors):
            if tensors is None:
                return None
            if not tensors:
                return (ctypes.c_void_p * n_slots)(*([None] * n_slots))
            return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])

        def base_table(name):
            return (ctypes.c_void_p * len(layout.shards))(
                *[(getattr(sh, name).ctypes.data if sh.num_samples > 0 else 0) for sh in layout.shards])

        self._tables = [table(t) for t in (self.pinned_q, self.pinned_s, self.pinned_zp, self.dev_q, self.dev_s, self.dev_zp, self.dev_out)]
        self._bases = [base_table("q"), base_table("s"), base_table("zp") if amo else None]
        self._sizes = (ctypes.c_int64 * len(layout.shards))(*layout.shard_sizes)
        d = _lib.StreamerDesc()
        d.n_shards = len(layout.shards)
        d.q_bases, d.s_bases, d.zp_bases = self._bases
        d.shard_sizes = self._sizes
        d.values_per_sample = vps
        d.groups_per_sample = gps
        d.group_size = layout.group_size
        d.batch_size = B
        d.n_slots = n_slots
        d.n_threads = n_threads or default_gather_threads()
        d.direct_dma = 1 if self.pin_shards else 0
        (d.pinned_q, d.pinned_s, d.pinned_zp, d.dev_q, d.dev_s, d.dev_zp, d.dev_out) = self._tables
        self._handle = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.check(_lib.lib().tcb_streamer_create(ctypes.byref(d), ctypes.byref(self._handle)))

    def begin(self, order: Optional[np.ndarray], n: int) -> None:
        if order is not None:
            order = np.ascontiguousarray(order, dtype=np.int64)
            _lib.check(_lib.lib().tcb_streamer_begin(self._handle, ctypes.c_void_p(order.ctypes.data), int(len(order))))
        else:
            _lib.check(_lib.lib().tcb_streamer_begin(self._handle, None, int(n)))

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def next_decoded(self):
        """(slot, rows); rows == 0 at the end of the pass."""
        slot, rows = ctypes.c_int(0), ctypes.c_int(0)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().tcb_streamer_next(self._handle, self._stream(), ctypes.byref(slot), ctypes.byref(rows)))
        return slot.value, rows.value

    def acquire(self):
        slot, rows = ctypes.c_int(0), ctypes.c_int(0)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().tcb_streamer_acquire(self._handle, self._stream(), ctypes.byref(slot), ctypes.byref(rows)))
        return slot.value, rows.value

    def release(self):
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().tcb_streamer_release(self._handle, self._stream()))

    def close(self):
        """Stops the native pipeline and drops the ring.  The shard files stay page-locked until the layout closes."""
        if getattr(self, "_handle", None) is not None and self._handle.value:
            _lib.lib().tcb_streamer_destroy(self._handle)
            self._handle = ctypes.c_void_p()
        for name in ("pinned_q", "pinned_s", "pinned_zp", "dev_q", "dev_s", "dev_zp", "dev_out", "_pinned_blocks", "_dev_blocks"):
            setattr(self, name, None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
