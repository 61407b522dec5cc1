"""One-line helpers with the reference's signatures (src/tensorcache/utils.py:22-152)."""
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


def _rel_error_percent(x: torch.Tensor, rec: torch.Tensor) -> float:
    xf = x.float()
    return (torch.norm(xf - rec.float().to(xf.device)) / torch.norm(xf)).item() * 100


def benchmark_tensor(x: torch.Tensor, group_size: int = 32, device: Optional[str] = None, verbose: bool = True,
                     include_quality: bool = False) -> Dict[str, Any]:
    """Relative error (percent) and encode latency of every codec mode on ``x``; the result dictionary has the
    reference's keys (utils.py:46-103): ``sym_g32``, ``adaptive``, ``amo_<mode>`` -> ``{"rel_rmse%", "ms", ...}``.
    ``quality`` is only tried when ``include_quality`` is set.  Latency is measured with CUDA events."""
    if device:
        x = x.to(device)

    def timed(fn):
        if not torch.cuda.is_available():
            raise RuntimeError("tensorcache_b200 computes on a CUDA device only (no CPU fallback) and none is available")
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = fn()
        stop.record()
        stop.synchronize()
        return out, start.elapsed_time(stop)

    results: Dict[str, Any] = {}
    for name, fn in (("sym_g32", quantize_int8_g32), ("adaptive", quantize_int8_adaptive)):
        (q, s, shape), ms = timed(lambda: fn(x, group_size))
        results[name] = {"rel_rmse%": _rel_error_percent(x, dequantize_int8_g32(q, s, shape, group_size)), "ms": ms}
    modes = ["fast", "balanced", "accurate", "max"] + (["quality"] if include_quality else [])
    for mode in modes:
        (q, s, zp, shape), ms = timed(lambda: quantize_int8_amo_bq(x, group_size, mode=mode))
        n, lo, hi = AMO_BQ_PRESETS[mode][:3]
        results[f"amo_{mode}"] = {"rel_rmse%": _rel_error_percent(x, dequantize_int8_amo_bq(q, s, zp, shape, group_size)),
                                  "ms": ms, "N": n, "lo": lo, "hi": hi}
    if verbose:
        print(f"tensorcache_b200 bench {tuple(x.shape)} {x.dtype} {x.device}")
        for key, v in results.items():
            label = f"sym_g{group_size}" if key == "sym_g32" else key
            bpe = 1 + (3 if key.startswith("amo") else 2) / group_size
            print(f"{label:14s} rel={v['rel_rmse%']:.4f}% ms={v['ms']:.3f} B/elem={bpe:.4f}")
    return results


def auto_select_mode(x: torch.Tensor, target_rmse: float = 0.5, group_size: int = 32, include_quality: bool = False) -> str:
    """Cheapest AMO-BQ preset whose relative error (percent) meets ``target_rmse``; falls back to the same search at
    G16 (returned as ``"G16_<mode>"``), then to the strongest preset -- the reference's policy (utils.py:106-122)."""
    res = benchmark_tensor(x, group_size, verbose=False, include_quality=include_quality)
    modes = ["fast", "balanced", "accurate", "max"] + (["quality"] if include_quality else [])
    for mode in modes:
        if res[f"amo_{mode}"]["rel_rmse%"] <= target_rmse:
            return mode
    if group_size > 16:
        return f"G16_{auto_select_mode(x, target_rmse, 16, include_quality)}"
    return "quality" if include_quality else "max"


def selftest_sum_order(rows_per_group_size: int = 4000, seed: int = 9) -> None:
    """Checks on THIS host that ``torch.sum(dim=-1)`` over a group's fp32 terms (what the reference's scale
    search compares, src/tensorcache/codec.py:877) adds in the order the encode kernels assume.  The order
    belongs to the torch build and the CPU's vector ISA; if it differs here, encoded scales can differ from
    what this host's own reference run would produce, and the call raises ``RuntimeError`` saying so.  Needs
    no GPU."""
    import ctypes

    from . import _lib

    L = _lib.lib()
    g = torch.Generator().manual_seed(seed)
    for G in (8, 16, 24, 32, 48, 64, 128):
        e = (torch.rand(rows_per_group_size, G, generator=g) * torch.exp(4 * torch.randn(rows_per_group_size, 1, generator=g))).contiguous()
        sums = e.sum(dim=-1).contiguous()
        rc = L.tcb_selftest_sum_order(ctypes.c_void_p(e.data_ptr()), rows_per_group_size, G, ctypes.c_void_p(sums.data_ptr()))
        if rc == _lib.ERR_SUM_ORDER:
            raise RuntimeError(L.tcb_last_error().decode("utf-8", "replace"))
        _lib.check(rc)
