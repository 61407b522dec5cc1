"""Feature-cache files: ``FeatureCacheWriter`` and ``FeatureCacheDataset``.

File format and class surface follow src/tensorcache/feature_cache.py of
TensorCache (writer :21-540, dataset :543-1179): per shard three headerless
little-endian arrays ``<prefix>[_shard{i}]_int8.bin`` (uint8 ``[N, seq, dim]``),
``_scales.bin`` (uint16 = bf16 bits ``[N, groups]``), ``_zp.bin`` (uint8
``[N, groups]``), a ``_meta.json`` per file set and a ``<prefix>_shards.json``
manifest for sharded caches.  Caches written here are readable by the reference
and vice versa.  Caches of the symmetric codec (``amo_bq=False``, optionally
``adaptive=True``) hold int8 codes and have no ``_zp.bin``.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Optional, Union

import numpy as np
import torch

import ctypes

from . import _lib
from ._pipeline import NativePipeline, _mem_available_bytes, open_cache, try_make_resident, writer_threads
from ._prefault import MEM_FRACTION_FOR_PREFAULT, Prefaulter, in_memory_filesystem
from .codec import AMO_BQ_PRESETS, BlockwiseInt8Codec, dequantize_int8_amo_bq, dequantize_int8_g32


class FeatureCacheWriter:
    """Pre-allocates the cache files and fills them sample by sample.

    ``append`` takes ``[seq_len, dim]`` or ``[B, seq_len, dim]`` tensors (CPU or
    CUDA).  A whole call is quantised on the GPU in chunks, the codes come back
    through page-locked buffers, and rows are copied into the memory maps.  Each
    sample's codes equal ``compress(sample)`` because ``seq_len * dim`` must be a
    multiple of the group size (checked).

    ``prefault`` (not in the reference): populate the pages of the new files in the background while the first
    samples are still being encoded.  ``None`` = automatic: on when the files live in memory-backed storage and fit
    half of the available memory, which is where first-touch page allocation bounds the writer; ``False`` leaves
    the files sparse until rows land in them.
    """

    _CHUNK = 256  # samples per encode launch (the reference's CUDA path takes 64; every sample is encoded on
                  # its own, so the chunk size does not change a single code)

    def __init__(self, output_prefix: Union[str, Path], num_samples: int, seq_len: int, dim: int,
                 group_size: int = 32, adaptive: bool = False, amo_bq: bool = False, amo_lo: float = 0.95,
                 amo_hi: float = 1.05, amo_candidates: int = 32, amo_mode: Optional[str] = None,
                 num_shards: int = 1, quant_bits: int = 8, resume: bool = False, prefault: Optional[bool] = None):
        self._resolve_settings(output_prefix, num_samples, seq_len, dim, group_size, adaptive, amo_bq, amo_lo, amo_hi,
                               amo_candidates, amo_mode, num_shards, quant_bits, resume)
        self._open_maps(resume)
        self._prefaulter = None
        self._prefault_plan = None if (prefault is False or resume) else (prefault,)   # started by the first append()

    def _start_prefault(self, wanted: Optional[bool]) -> None:
        """Runs on the first append (a writer that never receives data allocates nothing).  Caches reopened for appending are
        left alone: they already have most of their pages."""
        spans = [(int(mm.ctypes.data), int(mm.nbytes)) for maps in self._maps if maps is not None for mm in maps]
        total = sum(n for _, n in spans)
        if wanted is None:
            avail = _mem_available_bytes()
            if not in_memory_filesystem(self.shard_prefixes[0] + "_int8.bin") or avail is None or \
                    total > MEM_FRACTION_FOR_PREFAULT * avail:
                return
        if total:
            self._prefaulter = Prefaulter(spans)

    def _resolve_settings(self, output_prefix, num_samples, seq_len, dim, group_size, adaptive, amo_bq, amo_lo, amo_hi,
                          amo_candidates, amo_mode, num_shards, quant_bits, resume):
        """Checks the settings and derives the file layout; touches no file."""
        self.output_prefix = Path(output_prefix)
        self.output_prefix.parent.mkdir(parents=True, exist_ok=True)
        if group_size <= 0:
            raise ValueError(f"group_size must be >0, got {group_size}")
        if amo_bq and amo_mode and amo_mode not in AMO_BQ_PRESETS:
            raise ValueError(f"amo_mode {amo_mode!r} unknown")
        if adaptive and amo_bq:
            raise ValueError("Pick one: adaptive or amo_bq")
        if quant_bits in (2, 3, 4):
            raise ValueError(f"Feature caches with {quant_bits}-bit are not supported")
        if quant_bits != 8:
            raise ValueError(f"quant_bits must be 8 for features, got {quant_bits}")
        if amo_mode is not None:
            if amo_mode not in AMO_BQ_PRESETS:
                raise ValueError(f"Unknown amo_mode {amo_mode!r}, choose from {list(AMO_BQ_PRESETS.keys())}")
            amo_candidates, amo_lo, amo_hi, _ = AMO_BQ_PRESETS[amo_mode]
        self.num_samples, self.seq_len, self.dim = num_samples, seq_len, dim
        self.group_size, self.adaptive, self.amo_bq = group_size, adaptive, amo_bq
        self.amo_mode, self.amo_lo, self.amo_hi, self.amo_candidates = amo_mode, amo_lo, amo_hi, amo_candidates
        self.quant_bits = quant_bits
        self.codec = BlockwiseInt8Codec(group_size=group_size, adaptive=adaptive, amo_bq=amo_bq, amo_lo=amo_lo, amo_hi=amo_hi,
                                        amo_candidates=amo_candidates, amo_mode=amo_mode if amo_bq else None)
        self.num_shards = max(1, int(num_shards))
        self.elements_per_sample = seq_len * dim
        self.scales_per_sample = (self.elements_per_sample + group_size - 1) // group_size
        if self.elements_per_sample % group_size:
            raise ValueError(f"seq_len * dim = {self.elements_per_sample} must be a multiple of group_size {group_size}")
        self.is_sharded = self.num_shards > 1
        if self.is_sharded and resume:
            raise NotImplementedError("open_append supports single-shard caches only (num_shards=1); rebuild sharded caches instead")
        if self.is_sharded:
            self.shard_prefixes = [f"{self.output_prefix}_shard{i}" for i in range(self.num_shards)]
            base, rem = divmod(num_samples, self.num_shards)
            self.shard_sizes = [base + (1 if i < rem else 0) for i in range(self.num_shards)]
            self.meta_path = str(self.output_prefix) + "_shards.json"
        else:
            self.shard_prefixes = [str(self.output_prefix)]
            self.shard_sizes = [num_samples]
            self.meta_path = str(self.output_prefix) + "_meta.json"
        self._shard_offsets = [int(v) for v in np.cumsum([0] + self.shard_sizes[:-1])]
        self._member_of = None   # (manifest prefix, shard number) when this writer fills one shard of a sharded cache
        self.current_idx = 0
        self._closed = False
        self._staging = None
        self._maps = []

    def _open_maps(self, resume: bool):
        seq_len, dim, amo_bq = self.seq_len, self.dim, self.amo_bq
        mode = "r+" if resume else "w+"
        self._maps = []
        for pref, sz in zip(self.shard_prefixes, self.shard_sizes):
            Path(pref).parent.mkdir(parents=True, exist_ok=True)
            paths = (pref + "_int8.bin", pref + "_scales.bin", pref + "_zp.bin")
            if sz == 0:
                self._maps.append(None)
                continue
            if resume:
                self._grow_file(paths[0], sz * seq_len * dim)
                self._grow_file(paths[1], sz * self.scales_per_sample * 2)
                if amo_bq:
                    self._grow_file(paths[2], sz * self.scales_per_sample)
            maps = [np.memmap(paths[0], dtype=np.uint8 if amo_bq else np.int8, mode=mode, shape=(sz, seq_len, dim)),
                    np.memmap(paths[1], dtype=np.uint16, mode=mode, shape=(sz, self.scales_per_sample))]
            if amo_bq:
                maps.append(np.memmap(paths[2], dtype=np.uint8, mode=mode, shape=(sz, self.scales_per_sample)))
            for mm in maps:   # ask for huge pages where the file system offers them (fewer faults while filling the file)
                try:
                    mm._mmap.madvise(14)   # MADV_HUGEPAGE; refused harmlessly elsewhere
                except (AttributeError, OSError, ValueError):
                    pass
            self._maps.append(tuple(maps))
        self.int8_path = self.shard_prefixes[0] + "_int8.bin"
        self.scales_path = self.shard_prefixes[0] + "_scales.bin"
        self.zp_path = self.shard_prefixes[0] + "_zp.bin" if amo_bq else None

    @classmethod
    def for_shard(cls, output_prefix: Union[str, Path], shard_idx: int, num_samples: int, seq_len: int, dim: int,
                  num_shards: int, **settings) -> "FeatureCacheWriter":
        """Writer for ONE shard of a ``num_shards``-way cache of ``num_samples`` samples, so that several
        processes (one per GPU) can fill a sharded cache together: shard ``i`` holds the global samples
        ``[offset_i, offset_i + size_i)`` of the sequential split (feature_cache.py:134-142 of the reference) and
        its writer takes exactly those, in order.  The files and the per-shard meta are byte-identical with what
        ``FeatureCacheWriter(..., num_shards=num_shards)`` writes for that shard; one process calls
        ``write_manifest`` with the same arguments to add ``<prefix>_shards.json``."""
        num_shards = int(num_shards)
        if not 0 <= shard_idx < num_shards:
            raise ValueError(f"shard_idx {shard_idx} out of range {num_shards}")
        if num_shards == 1:
            return cls(output_prefix, num_samples, seq_len, dim, **settings)
        base, rem = divmod(num_samples, num_shards)
        obj = cls(f"{output_prefix}_shard{shard_idx}", base + (1 if shard_idx < rem else 0), seq_len, dim, **settings)
        obj._member_of = (str(output_prefix), shard_idx)
        return obj

    @classmethod
    def write_manifest(cls, output_prefix: Union[str, Path], num_samples: int, seq_len: int, dim: int, num_shards: int,
                       **settings) -> str:
        """Writes ``<prefix>_shards.json`` for a cache whose shards were filled by ``for_shard`` writers."""
        obj = cls.__new__(cls)
        kw = dict(group_size=32, adaptive=False, amo_bq=False, amo_lo=0.95, amo_hi=1.05, amo_candidates=32, amo_mode=None,
                  quant_bits=8)
        settings.pop("prefault", None)    # a writer-only switch: accepted so that both calls can share one settings dict
        unknown = set(settings) - set(kw)
        if unknown:
            raise TypeError(f"unknown cache setting(s) {sorted(unknown)}")
        kw.update(settings)
        obj._resolve_settings(output_prefix, num_samples, seq_len, dim, kw["group_size"], kw["adaptive"], kw["amo_bq"],
                              kw["amo_lo"], kw["amo_hi"], kw["amo_candidates"], kw["amo_mode"], num_shards, kw["quant_bits"], False)
        obj._closed = True     # owns no file
        if not obj.is_sharded:
            raise ValueError("a manifest belongs to a cache of at least two shards")
        obj._write_manifest(num_samples)
        return obj.meta_path

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _grow_file(path, nbytes: int) -> None:
        if path is None or not os.path.exists(path):
            raise FileNotFoundError(f"cannot append: missing cache file {path!r}")
        with open(path, "r+b") as f:
            if f.seek(0, os.SEEK_END) < nbytes:
                f.truncate(nbytes)

    @classmethod
    def open_append(cls, output_prefix, extra_samples: int, **expected_settings) -> "FeatureCacheWriter":
        """Reopens a single-shard cache to add ``extra_samples`` rows after the existing ones."""
        prefix = str(output_prefix)
        extra_samples = int(extra_samples)
        if extra_samples <= 0:
            raise ValueError(f"extra_samples must be > 0, got {extra_samples}")
        if os.path.exists(prefix + "_shards.json"):
            raise NotImplementedError("open_append supports single-shard caches only (num_shards=1); rebuild sharded caches instead")
        meta_path = prefix + "_meta.json"
        if not os.path.exists(meta_path):
            raise FileNotFoundError(f"cannot append: missing cache meta {meta_path!r}")
        with open(meta_path, "r") as f:
            meta = json.load(f)
        known = ("seq_len", "dim", "group_size", "adaptive", "amo_bq", "amo_mode", "amo_lo", "amo_hi", "amo_candidates", "quant_bits")
        for key, want in expected_settings.items():
            if key not in known:
                raise TypeError(f"unknown cache setting {key!r}")
            have = meta.get(key, 8 if key == "quant_bits" else None)
            if want is not None and have is not None and want != have:
                raise ValueError(f"append settings mismatch for {key!r}: cache has {have!r}, got {want!r} "
                                 "— refusing to append to a differently-encoded cache")
        kw = dict(seq_len=meta["seq_len"], dim=meta["dim"], group_size=meta["group_size"],
                  adaptive=meta.get("adaptive", False), amo_bq=meta.get("amo_bq", False), quant_bits=meta.get("quant_bits", 8))
        if kw["amo_bq"]:
            if meta.get("amo_mode"):
                kw["amo_mode"] = meta["amo_mode"]
            else:
                kw.update(amo_lo=meta.get("amo_lo", 0.95), amo_hi=meta.get("amo_hi", 1.05), amo_candidates=meta.get("amo_candidates", 32))
        old_total = int(meta["num_samples"])
        obj = cls(output_prefix, old_total + extra_samples, resume=True, **kw)
        obj.current_idx = old_total
        return obj

    def _shard_for_global(self, gidx: int):
        for si, off in enumerate(self._shard_offsets):
            if off <= gidx < off + self.shard_sizes[si]:
                return si, gidx - off
        raise IndexError(f"global_idx {gidx} out of range {self.num_samples}")

    def _host_staging(self, which: int):
        """Two sets of page-locked landing buffers for chunks of codes (allocated once), so that the
        encode + device-to-host copy of one chunk overlaps the file writes of the previous one."""
        if self._staging is None:
            pin = torch.cuda.is_available()
            n = self._CHUNK
            self._staging = [(
                torch.empty((n, self.seq_len, self.dim), dtype=torch.uint8 if self.amo_bq else torch.int8, pin_memory=pin),
                torch.empty((n, self.scales_per_sample), dtype=torch.int16, pin_memory=pin),
                torch.empty((n, self.scales_per_sample), dtype=torch.uint8, pin_memory=pin) if self.amo_bq else None,
            ) for _ in range(2)]
        return self._staging[which]

    def _flush_chunk(self, pending):
        """Waits for a chunk's device-to-host copies and moves its rows into the shard files
        (multi-threaded, cache-bypassing copy; a chunk may straddle shards)."""
        event, which, cur, start = pending
        event.synchronize()
        hq, hs, hz = self._host_staging(which)
        L = _lib.lib()
        threads = writer_threads()
        pos = 0
        while pos < cur:
            si, li = self._shard_for_global(start + pos)
            li = int(li)
            take = int(min(cur - pos, self.shard_sizes[si] - li))
            for mm, host in zip(self._maps[si], (hq, hs, hz)):
                row_bytes = int(mm[0].nbytes)   # consecutive samples are contiguous in the file and in the landing buffer
                _lib.check(L.tcb_write_block(ctypes.c_void_p(mm.ctypes.data + li * row_bytes),
                                             ctypes.c_void_p(int(host.data_ptr()) + int(pos) * row_bytes), take * row_bytes, threads))
            pos += take

    def append(self, tensor_bf16: torch.Tensor):
        if tensor_bf16.ndim == 2:
            tensor_bf16 = tensor_bf16.unsqueeze(0)
        B = tensor_bf16.shape[0]
        if tuple(tensor_bf16.shape[1:]) != (self.seq_len, self.dim):
            raise ValueError(f"expected [..., {self.seq_len}, {self.dim}], got {tuple(tensor_bf16.shape)}")
        if self.current_idx + B > self.num_samples:
            raise ValueError(f"Exceeds pre-allocated {self.num_samples}: have {self.current_idx}, adding {B}")
        if getattr(self, "_prefault_plan", None) is not None:
            plan, self._prefault_plan = self._prefault_plan, None
            self._start_prefault(plan[0])
        done, k, pending = 0, 0, None
        while done < B:
            cur = min(self._CHUNK, B - done)
            sub = tensor_bf16[done:done + cur]
            if not sub.is_cuda:
                sub = sub.cuda(non_blocking=True)
            enc = self.codec.quantize(sub)      # (q, s, zp, shape) for AMO-BQ, (q, s, shape) for the symmetric codec
            q, s = enc[0], enc[1]
            hq, hs, hz = self._host_staging(k & 1)
            hq[:cur].copy_(q.view(cur, self.seq_len, self.dim), non_blocking=True)
            hs[:cur].copy_(s.view(torch.int16).view(cur, self.scales_per_sample), non_blocking=True)
            if self.amo_bq:
                hz[:cur].copy_(enc[2].view(cur, self.scales_per_sample), non_blocking=True)
            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream(q.device))
            if pending is not None:
                self._flush_chunk(pending)      # overlaps the encode / copy just enqueued
            pending = (event, k & 1, cur, self.current_idx + done)
            done += cur
            k += 1
        if pending is not None:
            self._flush_chunk(pending)
        self.current_idx += B

    def _meta(self, num_samples: int, prefix: str, with_bits: bool) -> dict:
        meta = {
            "num_samples": num_samples, "seq_len": self.seq_len, "dim": self.dim, "group_size": self.group_size,
            "adaptive": self.adaptive, "amo_bq": self.amo_bq, "amo_mode": self.amo_mode if self.amo_bq else None,
            "amo_lo": self.amo_lo if self.amo_bq else None, "amo_hi": self.amo_hi if self.amo_bq else None,
            "amo_candidates": self.amo_candidates if self.amo_bq else None,
        }
        if with_bits:
            meta["quant_bits"] = self.quant_bits
        meta.update(int8_file=os.path.basename(prefix + "_int8.bin"), scales_file=os.path.basename(prefix + "_scales.bin"),
                    zp_file=os.path.basename(prefix + "_zp.bin") if self.amo_bq else None)
        return meta

    def close(self):
        if getattr(self, "_closed", True):
            return
        self._closed = True
        if getattr(self, "_prefaulter", None) is not None:
            self._prefaulter.stop()     # no thread may touch a mapping that is about to go away
            self._prefaulter = None
        for maps in self._maps:
            if maps is None:
                continue
            for mm in maps:
                mm.flush()
                if getattr(mm, "_mmap", None) is not None:
                    mm._mmap.close()
        self._maps = []
        self._staging = None
        if self.is_sharded:
            for i, pref in enumerate(self.shard_prefixes):
                actual = max(0, min(self.shard_sizes[i], self.current_idx - int(self._shard_offsets[i])))
                with open(pref + "_meta.json", "w") as f:
                    json.dump(self._meta(actual, pref, with_bits=False), f, indent=2)
            self._write_manifest(self.current_idx)
        else:
            # one shard of a sharded cache carries the per-shard form of the meta (no "quant_bits" key)
            with open(self.meta_path, "w") as f:
                json.dump(self._meta(self.current_idx, str(self.output_prefix), with_bits=self._member_of is None), f, indent=2)

    def _write_manifest(self, total_written: int):
        manifest = self._meta(total_written, str(self.output_prefix), with_bits=False)
        for k in ("int8_file", "scales_file", "zp_file"):
            manifest.pop(k)
        manifest.update(num_shards=self.num_shards, shard_sizes=self.shard_sizes, shard_prefixes=self.shard_prefixes,
                        shard_metas=[pref + "_meta.json" for pref in self.shard_prefixes])
        with open(self.meta_path, "w") as f:
            json.dump(manifest, f, indent=2)


class FeatureCacheDataset(torch.utils.data.Dataset):
    """Memory-mapped reader: ``ds[i]`` returns copies ``(q, scales, zp)`` -- ``(q, scales)`` for a
    cache of the symmetric codec -- or the decoded bf16 sample on ``auto_dequant_device``;
    ``iter_batches`` streams decoded batches through the native pipeline.

    ``rank`` / ``world_size`` select shard ``rank % num_shards`` like
    ``ZeroCopyTensorStreamer`` does.  (The reference class computes that mapping
    before it has read the manifest and therefore always opens shard 0,
    feature_cache.py:569-578; that defect is not reproduced.)
    """

    def __init__(self, cache_prefix: Union[str, Path], auto_dequant_device: Optional[str] = None,
                 shard_idx: Optional[int] = None, rank: Optional[int] = None, world_size: Optional[int] = None,
                 all_rank_shards: bool = False, pin_shard: Optional[bool] = None):
        self.cache_prefix = Path(cache_prefix)
        self._pin_wanted = pin_shard     # as for ZeroCopyTensorStreamer: True / False / None (automatic, decided at the
        self.pin_shard = False           # first iter_batches call); copy-on-write mappings can be page-locked later
        self._layout = open_cache(cache_prefix, shard_idx, rank, world_size, all_rank_shards, private=pin_shard is not False)
        lay = self._layout
        self.meta = lay.meta
        self.is_sharded = lay.selected is not None
        self.num_shards = len(lay.shards)
        self.shard_prefixes = [s.prefix for s in lay.shards]
        self.shard_sizes = lay.shard_sizes
        self.shard_offsets = lay.shard_offsets
        self.num_samples = lay.num_samples
        self.seq_len, self.dim, self.group_size, self.amo_bq = lay.seq_len, lay.dim, lay.group_size, lay.amo_bq
        self.scales_count = lay.groups_per_sample
        self.auto_dequant_device = auto_dequant_device
        self._pipes = []
        self._idle_pipes = {}
        self._closed = False

    def __len__(self) -> int:
        return self.num_samples

    def __getitem__(self, idx: int):
        si, li = self._layout.locate(int(idx))
        sh = self._layout.shards[si]
        q = torch.from_numpy(np.array(sh.q[li]))
        s = torch.from_numpy(np.array(sh.s[li]).view(np.int16)).view(torch.bfloat16)
        if not self.amo_bq:
            if self.auto_dequant_device is not None:
                dev = self.auto_dequant_device
                return dequantize_int8_g32(q.to(dev, non_blocking=True), s.to(dev, non_blocking=True),
                                           (self.seq_len, self.dim), group_size=self.group_size)
            return q, s
        zp = torch.from_numpy(np.array(sh.zp[li]))
        if self.auto_dequant_device is not None:
            dev = self.auto_dequant_device
            return dequantize_int8_amo_bq(q.to(dev, non_blocking=True), s.to(dev, non_blocking=True),
                                          zp.to(dev, non_blocking=True), (self.seq_len, self.dim), group_size=self.group_size)
        return q, s, zp

    def iter_batches(self, batch_size: int = 128, shuffle: bool = True, device: str = "cuda:0", dequantize: bool = True):
        """Yields bf16 ``[rows, seq_len, dim]`` views of a two-slot output ring
        (valid until two more batches have been requested), or cloned
        ``(q, scales, zp)`` device tensors (``(q, scales)`` for a symmetric cache) when
        ``dequantize=False``.

        The first call decides the reader mode (``pin_shard`` of the constructor): with the shard(s)
        page-locked in host memory the rows go to the GPU without a CPU copy, exactly as in
        ``ZeroCopyTensorStreamer``; the page-locking is paid once and kept until ``close()``.  The ring of
        a pass is kept for the next pass with the same batch size and device."""
        dev = torch.device(device)
        self.pin_shard = try_make_resident(self._layout, dev, self._pin_wanted)
        key = (int(batch_size), str(dev), self.pin_shard)
        pipe = self._idle_pipes.pop(key, None)
        if pipe is None:
            pipe = NativePipeline(self._layout, batch_size, dev, n_slots=2, pin_shards=self.pin_shard)
        self._pipes.append(pipe)
        reusable = False
        try:
            if shuffle:
                order = np.arange(self.num_samples)
                np.random.shuffle(order)
                pipe.begin(order, self.num_samples)
            else:
                pipe.begin(None, self.num_samples)
            while True:
                if dequantize:
                    slot, rows = pipe.next_decoded()
                    if rows == 0:
                        break
                    yield pipe.dev_out[slot][:rows]
                else:
                    slot, rows = pipe.acquire()
                    if rows == 0:
                        break
                    out = (pipe.dev_q[slot][:rows].clone(), pipe.dev_s[slot][:rows].clone())
                    if self.amo_bq:
                        out += (pipe.dev_zp[slot][:rows].clone(),)
                    pipe.release()
                    yield out
            reusable = True
        except GeneratorExit:
            reusable = True       # an abandoned pass: no batch is held at a yield, and the next begin() drops what is in flight
            raise
        finally:
            torch.cuda.synchronize(pipe.device)
            self._pipes.remove(pipe)
            if reusable and key not in self._idle_pipes and not self._closed:
                self._idle_pipes[key] = pipe      # reused by the next pass
            else:
                pipe.close()

    def close(self):
        self._closed = True
        for p in list(getattr(self, "_pipes", [])) + list(getattr(self, "_idle_pipes", {}).values()):
            p.close()
        self._pipes = []
        self._idle_pipes = {}
        if getattr(self, "_layout", None) is not None:
            self._layout.close()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
