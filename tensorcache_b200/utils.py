"""One-line helpers with the reference's signatures (src/tensorcache/utils.py:22-44, 125-152)."""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch

from .codec import (AMO_BQ_PRESETS, dequantize_int8_amo_bq, dequantize_int8_g32, quantize_int8_adaptive,
                    quantize_int8_amo_bq, quantize_int8_g32)


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
    """AMO-BQ compress -> ``(q, scales, zero_points, shape)``; modes ``"sym"`` / ``"adaptive"`` return the
    symmetric codec's ``(q, scales, shape)`` as the reference does (utils.py:125-139)."""
    if mode in AMO_BQ_PRESETS:
        return quantize_int8_amo_bq(x, group_size, mode=mode)
    if mode == "sym":
        return quantize_int8_g32(x, group_size)
    if mode == "adaptive":
        return quantize_int8_adaptive(x, group_size)
    raise ValueError(f"mode {mode!r} unknown, choose from {list(AMO_BQ_PRESETS.keys()) + ['sym', 'adaptive']}")


def decompress(q: torch.Tensor, scales: torch.Tensor, shape: Tuple[int, ...],
               zero_points: Optional[torch.Tensor] = None, group_size: int = 32) -> torch.Tensor:
    """Decompress to bf16 of ``shape``: AMO-BQ codes when ``zero_points`` is given, else symmetric codes."""
    if zero_points is None:
        return dequantize_int8_g32(q, scales, shape, group_size)
    return dequantize_int8_amo_bq(q, scales, zero_points, shape, group_size)
