"""``ZeroCopyTensorStreamer``: ring-buffered batch reader over an AMO-BQ feature cache.

Same constructor, iteration protocol and public attributes as the reference class
(src/tensorcache/streamer.py:19-587).  The work happens in the native pipeline
(``tcb_streamer_*``): gather threads copy rows from the memory-mapped shard into
page-locked staging, a copy stream moves them to the GPU, and the decode kernel
runs on the caller's current stream, all overlapped across ring slots.

Differences from the reference, on purpose:
* the ring is ordered by events in both directions (the reference lets the host
  and the copy stream overwrite buffers that may still be in use);
* the decode device must be CUDA (the reference's ``device="cpu"`` branch is a
  CPU implementation, which this package does not have); the host-side parts
  (manifest, rank -> shard mapping, ``len``) work without a GPU;
* ``all_rank_shards=True`` lets a rank read every shard ``i`` with
  ``i % world_size == rank`` instead of the single shard ``rank % num_shards``;
* ``pin_shard`` chooses how rows reach the GPU.  ``True`` keeps the opened shard(s) resident and
  page-locked in host memory (a private mapping of the files, pinned once at about 0.4 s per GB,
  costing as much RAM as the shard) so that the copy engine reads the rows itself and no CPU copy
  remains.  ``False`` is the reference's small-footprint behaviour (worker threads copy rows into
  page-locked staging).  The default ``None`` picks the first when the shard(s) fit a quarter of the
  host memory available at that moment and the driver agrees to page-lock them, and the second,
  with a one-line warning, otherwise;
* the ring has three slots by default (``ring_slots``; the reference has two), which
  costs one more batch of staging and output memory and hides the host gather.
"""
from __future__ import annotations

from pathlib import Path
from typing import Iterator, Optional, Union

import numpy as np
import torch

from ._pipeline import NativePipeline, open_cache, try_make_resident


class ZeroCopyTensorStreamer:
    def __init__(
        self,
        cache_prefix: Union[str, Path],
        batch_size: int = 128,
        device: str = "cuda:0",
        shuffle: bool = True,
        low_vram: bool = False,
        shard_idx: Optional[int] = None,
        rank: Optional[int] = None,
        world_size: Optional[int] = None,
        all_rank_shards: bool = False,
        gather_threads: Optional[int] = None,
        ring_slots: Optional[int] = None,
        pin_shard: Optional[bool] = None,
    ):
        self.cache_prefix = Path(cache_prefix)
        self.batch_size = int(batch_size)
        self.device = torch.device(device)
        self.shuffle = shuffle
        self.low_vram = low_vram
        self.rank = rank
        self.world_size = world_size
        self._pin_wanted = pin_shard            # True / False / None (automatic)
        self.pin_shard = False                  # what the reader ended up doing; set when the pipeline is built
        self._layout = open_cache(cache_prefix, shard_idx, rank, world_size, all_rank_shards, private=pin_shard is not False)
        lay = self._layout
        self.meta = lay.meta
        self.is_sharded = lay.selected is not None and len(lay.shards) > 1
        self.num_shards = len(lay.shards)
        self.shard_idx = lay.selected[0] if lay.selected is not None and len(lay.selected) == 1 and (
            shard_idx is not None or rank is not None) else shard_idx
        self.shard_prefixes = [s.prefix for s in lay.shards]
        self.shard_sizes = lay.shard_sizes
        self.shard_offsets = lay.shard_offsets
        self.num_samples = lay.num_samples
        self.seq_len = lay.seq_len
        self.dim = lay.dim
        self.group_size = lay.group_size
        self.amo_bq = lay.amo_bq
        self.scales_per_sample = lay.groups_per_sample
        # ring depth: 1 = serial (low_vram); the default of 3 keeps the gather, the H2D copy and the decode of
        # three different batches in flight (the reference's ring has 2); a yielded view stays valid until
        # n_bufs further batches have been requested
        self.n_bufs = 1 if low_vram else int(ring_slots or 3)
        if not 1 <= self.n_bufs <= 8:
            raise ValueError(f"ring_slots {self.n_bufs} outside 1..8")
        self.indices = np.arange(self.num_samples)
        self._gather_threads = gather_threads
        self._pipe: Optional[NativePipeline] = None
        self._closed = False
        self.out_bf16 = None
        self.out_bf16_0 = self.out_bf16_1 = None
        if self.device.type == "cuda" and torch.cuda.is_available():
            self._ensure_pipeline()

    # -- host-side helpers -------------------------------------------------
    def __len__(self) -> int:
        return (self.num_samples + self.batch_size - 1) // self.batch_size

    def __enter__(self) -> "ZeroCopyTensorStreamer":
        return self

    def __exit__(self, exc_type, exc_val, exc_tb) -> None:
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ensure_pipeline(self) -> NativePipeline:
        if self._closed:
            raise RuntimeError("streamer is closed")
        if self._pipe is None:
            self.pin_shard = try_make_resident(self._layout, self.device, self._pin_wanted)
            self._pipe = NativePipeline(self._layout, self.batch_size, self.device, self.n_bufs, self._gather_threads,
                                        pin_shards=self.pin_shard)
            self.out_bf16 = self._pipe.dev_out
            self.out_bf16_0 = self.out_bf16[0]
            self.out_bf16_1 = self.out_bf16[1] if len(self.out_bf16) > 1 else self.out_bf16[0]
            none = [None] * self.n_bufs   # a cache of the symmetric codec has no zero points
            self.gpu_int8, self.gpu_scales, self.gpu_zp = self._pipe.dev_q, self._pipe.dev_s, self._pipe.dev_zp or none
            self.pinned_int8, self.pinned_scales, self.pinned_zp = self._pipe.pinned_q, self._pipe.pinned_s, self._pipe.pinned_zp or none
        return self._pipe

    # -- iteration -----------------------------------------------------------
    def __iter__(self) -> Iterator[torch.Tensor]:
        """Yields bf16 ``[rows, seq_len, dim]`` views into the output ring.  A view
        stays valid until ``n_bufs`` further batches have been requested; clone it
        to keep it longer.  Shuffling uses numpy's global RNG, like the reference."""
        pipe = self._ensure_pipeline()
        if self.shuffle:
            np.random.shuffle(self.indices)
            pipe.begin(self.indices, self.num_samples)
        else:
            pipe.begin(None, self.num_samples)
        while True:
            slot, rows = pipe.next_decoded()
            if rows == 0:
                return
            yield pipe.dev_out[slot][:rows]

    def close(self):
        if getattr(self, "_closed", True):
            return
        self._closed = True
        if self._pipe is not None:
            if torch.cuda.is_available():
                torch.cuda.synchronize(self.device)
            self._pipe.close()
            self._pipe = None
        self.out_bf16 = self.out_bf16_0 = self.out_bf16_1 = None
        self.gpu_int8 = self.gpu_scales = self.gpu_zp = None
        self.pinned_int8 = self.pinned_scales = self.pinned_zp = None
        self._layout.close()
