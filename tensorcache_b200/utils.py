"""One-line helpers with the reference's signatures (src/tensorcache/utils.py:22-44, 125-152)."""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch

from .codec import AMO_BQ_PRESETS, dequantize_int8_amo_bq, quantize_int8_amo_bq


def estimate_compression(shape: Tuple[int, ...], group_size: int = 32, amo_bq: bool = True) -> Dict[str, Any]:
    """Storage arithmetic without quantising anything."""
    numel = math.prod(shape)
    bpe = 1 + (3 if amo_bq else 2) / group_size
    return {
        "numel": numel,
        "num_blocks": (numel + group_size - 1) // group_size,
        "bytes_per_elem": bpe,
        "total_bytes": int(numel * bpe),
        "total_MB": numel * bpe / 1024 / 1024,
        "ratio_vs_bf16": 2.0 / bpe,
        "ratio_vs_fp32": 4.0 / bpe,
        "group_size": group_size,
        "amo_bq": amo_bq,
    }


def compress(x: torch.Tensor, mode: str = "balanced", group_size: int = 32):
    """AMO-BQ compress -> ``(q, scales, zero_points, shape)``."""
    if mode in AMO_BQ_PRESETS:
        return quantize_int8_amo_bq(x, group_size, mode=mode)
    if mode in ("sym", "adaptive"):
        raise NotImplementedError(f"mode {mode!r} (symmetric codec) is outside the B200 AMO-BQ path")
    raise ValueError(f"mode {mode!r} unknown, choose from {list(AMO_BQ_PRESETS.keys()) + ['sym', 'adaptive']}")


def decompress(q: torch.Tensor, scales: torch.Tensor, shape: Tuple[int, ...],
               zero_points: Optional[torch.Tensor] = None, group_size: int = 32) -> torch.Tensor:
    """Decompress AMO-BQ codes to bf16 of ``shape``."""
    if zero_points is None:
        raise NotImplementedError("symmetric decode (zero_points=None) is outside the B200 AMO-BQ path")
    return dequantize_int8_amo_bq(q, scales, zero_points, shape, group_size)
