"""AMO-BQ codec on the B200 kernels, with the reference's Python signatures.

Mirrors ``src/tensorcache/codec.py:700-1041`` of TensorCache (``AMO_BQ_PRESETS``,
``quantize_int8_amo_bq``, ``dequantize_int8_amo_bq``, ``BlockwiseInt8Codec``) and the
symmetric codec next to it (``quantize_int8_g32``, ``quantize_int8_adaptive``,
``dequantize_int8_g32``, ``codec.py:530-697``).
All arithmetic runs in the CUDA library; CPU tensors are accepted for drop-in
compatibility by staging them through the current CUDA device (the results are
bit-identical to the reference's CPU path, so callers cannot tell), and the
outputs come back on the input's device as the reference returns them.  Without
a CUDA device every compute call raises -- there is no CPU implementation here.
"""
from __future__ import annotations

import ctypes
from functools import lru_cache
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib

AMO_BQ_PRESETS = {
    # (num_candidates, lo, hi, description) -- same registry as the reference
    "fast": (16, 0.95, 1.05, "16 multipliers in 0.95-1.05"),
    "balanced": (32, 0.95, 1.05, "32 multipliers in 0.95-1.05 (default)"),
    "accurate": (48, 0.95, 1.10, "48 multipliers in 0.95-1.10"),
    "max": (64, 0.85, 1.10, "64 multipliers in 0.85-1.10"),
    "quality": (64, 0.85, 1.10, "bf16-grid search scored on decoded values"),
}

SUPPORTED_GROUP_SIZES = (8, 16, 24, 32, 48, 64, 128)
_DTYPES = {torch.bfloat16: _lib.DT_BF16, torch.float16: _lib.DT_F16, torch.float32: _lib.DT_F32}


def _resolve_amo_preset(mode, num_candidates, lo, hi):
    if mode is None:
        return num_candidates, lo, hi
    if mode not in AMO_BQ_PRESETS:
        raise ValueError(f"Unknown amo_mode {mode!r}, choose from {list(AMO_BQ_PRESETS.keys())}")
    n, plo, phi, _ = AMO_BQ_PRESETS[mode]
    return (n if num_candidates is None else num_candidates,
            plo if lo is None else lo,
            phi if hi is None else hi)


@lru_cache(maxsize=64)
def _multipliers(lo: float, hi: float, n: int) -> np.ndarray:
    """Candidate multipliers exactly as the reference builds them: torch.linspace
    evaluated on the CPU in fp32 (codec.py:852).  Cached per (lo, hi, n)."""
    return torch.linspace(lo, hi, n, dtype=torch.float32, device="cpu").numpy().copy()


def _compute_device(t: torch.Tensor) -> torch.device:
    if t.is_cuda:
        return t.device
    if not torch.cuda.is_available():
        raise RuntimeError("tensorcache_b200 computes on a CUDA device only (no CPU fallback) and none is available")
    return torch.device("cuda", torch.cuda.current_device())


def _check_group_size(group_size: int) -> None:
    if group_size not in SUPPORTED_GROUP_SIZES:
        raise ValueError(f"group_size {group_size} is not supported by the B200 kernels, choose from {SUPPORTED_GROUP_SIZES}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr() if t is not None and t.numel() else 0)


def quantize_int8_amo_bq(
    x: torch.Tensor,
    group_size: int = 32,
    num_candidates: int = 32,
    lo: float = 0.95,
    hi: float = 1.05,
    mode: Optional[str] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Tuple[int, ...]]:
    """AMO-BQ encode; same contract as the reference (codec.py:774-893).

    Returns ``(q uint8 [numel], scales bf16 [ceil(numel/G)], zero_points uint8
    [ceil(numel/G)], orig_shape)`` on ``x.device``.  ``mode`` overrides
    ``num_candidates / lo / hi``.  The codes equal the reference's CPU result bit
    for bit.  Nothing here synchronises with the host for CUDA inputs, so the call
    can be captured in a CUDA graph.
    """
    if mode is not None:
        num_candidates, lo, hi = _resolve_amo_preset(mode, None, None, None)
    _check_group_size(group_size)
    if x.dtype not in _DTYPES:
        x = x.float()
    dev = _compute_device(x)
    orig_shape = x.shape
    numel = x.numel()
    ngroups = (numel + group_size - 1) // group_size
    with torch.cuda.device(dev):
        xd = x.reshape(-1).contiguous() if x.is_cuda else x.reshape(-1).contiguous().to(dev)
        q = torch.empty(numel, dtype=torch.uint8, device=dev)
        s = torch.empty(ngroups, dtype=torch.bfloat16, device=dev)
        zp = torch.empty(ngroups, dtype=torch.uint8, device=dev)
        if numel:
            stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            L = _lib.lib()
            if mode == "quality":
                rc = L.tcb_compress_amo_quality(_ptr(xd), _DTYPES[xd.dtype], numel, group_size, _ptr(q), _ptr(s), _ptr(zp), stream)
            else:
                if not 1 <= int(num_candidates) <= 64:
                    raise ValueError(f"num_candidates {num_candidates} outside 1..64")
                m = _multipliers(float(lo), float(hi), int(num_candidates))
                rc = L.tcb_compress_amo(_ptr(xd), _DTYPES[xd.dtype], numel, group_size, ctypes.c_void_p(m.ctypes.data),
                                        int(num_candidates), _ptr(q), _ptr(s), _ptr(zp), stream)
            _lib.check(rc)
    if not x.is_cuda:
        q, s, zp = q.cpu(), s.cpu(), zp.cpu()
    return q, s, zp, orig_shape


def dequantize_int8_amo_bq(
    q_uint8: torch.Tensor,
    scales: torch.Tensor,
    zero_points: torch.Tensor,
    orig_shape: Tuple[int, ...],
    group_size: int = 32,
    out_buffer: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """AMO-BQ decode ``rec = (q - zp) * scale`` -> bf16; contract of codec.py:896-966.

    ``q_uint8`` may have any shape (its flattened order is what counts);
    ``scales`` / ``zero_points`` need ``ceil(numel / group_size)`` elements.  If
    ``out_buffer`` is given it is written in place and returned (the same object).
    """
    _check_group_size(group_size)
    numel = q_uint8.numel()
    ngroups = (numel + group_size - 1) // group_size
    if scales.numel() < ngroups or zero_points.numel() < ngroups:
        raise ValueError(f"need {ngroups} scales / zero points for {numel} values at G={group_size}, "
                         f"got {scales.numel()} / {zero_points.numel()}")
    if q_uint8.dtype != torch.uint8 or zero_points.dtype != torch.uint8 or scales.dtype != torch.bfloat16:
        raise ValueError("AMO-BQ decode takes uint8 codes, bf16 scales and uint8 zero points")
    dev = _compute_device(q_uint8)
    if out_buffer is None:
        out_buffer = torch.empty(orig_shape, dtype=torch.bfloat16, device=q_uint8.device)
    if out_buffer.numel() != numel or out_buffer.dtype != torch.bfloat16:
        raise ValueError("out_buffer must be a bf16 tensor with as many elements as q")
    if numel == 0:
        return out_buffer
    with torch.cuda.device(dev):
        qd = q_uint8.contiguous().to(dev)
        sd = scales.contiguous().to(dev)
        zd = zero_points.contiguous().to(dev)
        direct = out_buffer.is_cuda and out_buffer.device == dev and out_buffer.is_contiguous()
        od = out_buffer if direct else torch.empty(numel, dtype=torch.bfloat16, device=dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(_lib.lib().tcb_decompress_amo(_ptr(qd), _ptr(sd), _ptr(zd), _ptr(od), numel, group_size, stream))
        if not direct:
            out_buffer.copy_(od.view(out_buffer.shape))
    return out_buffer


def _quantize_sym(x: torch.Tensor, group_size: int, num_candidates: int):
    _check_group_size(group_size)
    if x.dtype not in _DTYPES:
        x = x.float()
    dev = _compute_device(x)
    orig_shape = x.shape
    numel = x.numel()
    ngroups = (numel + group_size - 1) // group_size
    with torch.cuda.device(dev):
        xd = x.reshape(-1).contiguous() if x.is_cuda else x.reshape(-1).contiguous().to(dev)
        q = torch.empty(numel, dtype=torch.int8, device=dev)
        s = torch.empty(ngroups, dtype=torch.bfloat16, device=dev)
        if numel:
            stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            if num_candidates:
                if not 1 <= int(num_candidates) <= 64:
                    raise ValueError(f"num_candidates {num_candidates} outside 1..64")
                m = _multipliers(0.90, 1.05, int(num_candidates))
                mp = ctypes.c_void_p(m.ctypes.data)
            else:
                mp = ctypes.c_void_p(0)
            _lib.check(_lib.lib().tcb_compress_sym(_ptr(xd), _DTYPES[xd.dtype], numel, group_size, mp, int(num_candidates),
                                                   _ptr(q), _ptr(s), stream))
    if not x.is_cuda:
        q, s = q.cpu(), s.cpu()
    return q, s, orig_shape


def quantize_int8_g32(x: torch.Tensor, group_size: int = 32):
    """Symmetric block-wise int8: ``(q int8 [numel], scales bf16 [ceil(numel/G)], orig_shape)``.

    Contract and bits of the reference's CPU path (codec.py:530-565): scale = bf16(max|x| / 127),
    q = clamp(round(x / scale), -128, 127), non-finite values become 0.
    """
    return _quantize_sym(x, group_size, 0)


def quantize_int8_adaptive(x: torch.Tensor, group_size: int = 32, num_candidates: int = 31):
    """Symmetric int8 with the reference's least-squares scale search over 0.90-1.05 (codec.py:568-620)."""
    return _quantize_sym(x, group_size, num_candidates)


def dequantize_int8_g32(q_int8: torch.Tensor, scales: torch.Tensor, orig_shape: Tuple[int, ...], group_size: int = 32,
                        out_buffer: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Symmetric decode ``rec = q * scale`` -> bf16; contract of codec.py:623-697."""
    _check_group_size(group_size)
    numel = q_int8.numel()
    ngroups = (numel + group_size - 1) // group_size
    if scales.numel() < ngroups:
        raise ValueError(f"need {ngroups} scales for {numel} values at G={group_size}, got {scales.numel()}")
    if q_int8.dtype != torch.int8 or scales.dtype != torch.bfloat16:
        raise ValueError("symmetric decode takes int8 codes and bf16 scales")
    dev = _compute_device(q_int8)
    if out_buffer is None:
        out_buffer = torch.empty(orig_shape, dtype=torch.bfloat16, device=q_int8.device)
    if out_buffer.numel() != numel or out_buffer.dtype != torch.bfloat16:
        raise ValueError("out_buffer must be a bf16 tensor with as many elements as q")
    if numel == 0:
        return out_buffer
    with torch.cuda.device(dev):
        qd = q_int8.contiguous().to(dev)
        sd = scales.contiguous().to(dev)
        direct = out_buffer.is_cuda and out_buffer.device == dev and out_buffer.is_contiguous()
        od = out_buffer if direct else torch.empty(numel, dtype=torch.bfloat16, device=dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(_lib.lib().tcb_decompress_sym(_ptr(qd), _ptr(sd), _ptr(od), numel, group_size, stream))
        if not direct:
            out_buffer.copy_(od.view(out_buffer.shape))
    return out_buffer


class BlockwiseInt8Codec:
    """Configuration holder with ``quantize`` / ``dequantize``; mirrors codec.py:969-1041.

    Default is the symmetric codec, ``adaptive=True`` its scale search, ``amo_bq=True`` AMO-BQ.
    """

    def __init__(self, group_size: int = 32, adaptive: bool = False, amo_bq: bool = False,
                 amo_lo: float = 0.95, amo_hi: float = 1.05, amo_candidates: int = 32,
                 amo_mode: Optional[str] = None):
        if amo_bq and amo_mode and amo_mode not in AMO_BQ_PRESETS:
            raise ValueError(f"amo_mode {amo_mode!r} unknown, choose {list(AMO_BQ_PRESETS.keys())}")
        if adaptive and amo_bq:
            raise ValueError("Choose one: adaptive or amo_bq, not both")
        self.group_size = group_size
        self.adaptive = adaptive
        self.amo_bq = amo_bq
        self.amo_mode = amo_mode
        if amo_mode is not None:
            self.amo_candidates, self.amo_lo, self.amo_hi = _resolve_amo_preset(amo_mode, None, None, None)
        else:
            self.amo_lo, self.amo_hi, self.amo_candidates = amo_lo, amo_hi, amo_candidates

    def __repr__(self):
        if self.amo_bq:
            bpe = 1 + 3 / self.group_size
            tag = self.amo_mode or f"{self.amo_candidates},{self.amo_lo}-{self.amo_hi}"
            return f"BlockwiseInt8Codec(G={self.group_size}, amo_bq={tag} {bpe:.4f}B 1:{2 / bpe:.2f}x)"
        if self.adaptive:
            return f"BlockwiseInt8Codec(G={self.group_size}, adaptive 0.90-1.05 1:{2 / (1 + 2 / self.group_size):.2f}x)"
        return f"BlockwiseInt8Codec(G={self.group_size}, sym 1:{2 / (1 + 2 / self.group_size):.2f}x)"

    def quantize(self, x: torch.Tensor):
        if self.amo_bq:
            return quantize_int8_amo_bq(x, group_size=self.group_size, num_candidates=self.amo_candidates,
                                        lo=self.amo_lo, hi=self.amo_hi, mode=self.amo_mode)
        if self.adaptive:
            return quantize_int8_adaptive(x, group_size=self.group_size)
        return quantize_int8_g32(x, group_size=self.group_size)

    def dequantize(self, q_int8, scales, orig_shape, zero_points=None, out_buffer=None):
        if zero_points is None:
            return dequantize_int8_g32(q_int8, scales, orig_shape, group_size=self.group_size, out_buffer=out_buffer)
        return dequantize_int8_amo_bq(q_int8, scales, zero_points, orig_shape, group_size=self.group_size, out_buffer=out_buffer)
