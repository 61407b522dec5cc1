"""ctypes front end of the C oracle (``amo_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the tests, the smoke check and the
benchmark's CPU-baseline leg.  The product package never imports this module.

All functions take and return numpy arrays (bf16 travels as uint16 bit
patterns).  ``linspace_multipliers`` reproduces the candidate table of the
reference (``torch.linspace`` on the CPU, codec.py:852 of TensorCache).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libamo_oracle.so"
_lib = None

DT_BF16, DT_F16, DT_F32 = 0, 1, 2

# (num_candidates, lo, hi) of the reference presets, codec.py:700-706
PRESETS = {
    "fast": (16, 0.95, 1.05),
    "balanced": (32, 0.95, 1.05),
    "accurate": (48, 0.95, 1.10),
    "max": (64, 0.85, 1.10),
    "quality": (64, 0.85, 1.10),
}


def build(force: bool = False) -> Path:
    """Compile the oracle with gcc if the shared object is missing or stale."""
    src = _HERE / "amo_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libamo_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        L.tcb_oracle_decompress.argtypes = [vp, vp, vp, vp, i64, i32, i32]
        L.tcb_oracle_decompress.restype = None
        L.tcb_oracle_compress.argtypes = [vp, i32, i64, i32, vp, i32, vp, vp, vp, i32]
        L.tcb_oracle_compress.restype = i32
        L.tcb_oracle_compress_quality.argtypes = [vp, i32, i64, i32, vp, vp, vp, i32]
        L.tcb_oracle_compress_quality.restype = i32
        L.tcb_oracle_dequant_matmul.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i32, i32]
        L.tcb_oracle_dequant_matmul.restype = None
        L.tcb_oracle_compress_sym.argtypes = [vp, i32, i64, i32, vp, i32, vp, vp, i32]
        L.tcb_oracle_compress_sym.restype = i32
        L.tcb_oracle_decompress_sym.argtypes = [vp, vp, vp, i64, i32, i32]
        L.tcb_oracle_decompress_sym.restype = None
        L.tcb_oracle_sum_group.argtypes = [vp, i32]
        L.tcb_oracle_sum_group.restype = ctypes.c_float
        _lib = L
    return _lib


def default_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data) if a is not None else ctypes.c_void_p(0)


def linspace_multipliers(lo: float, hi: float, n: int) -> np.ndarray:
    """The fp32 candidate multipliers exactly as the reference computes them."""
    import torch

    return torch.linspace(lo, hi, n, dtype=torch.float32, device="cpu").numpy().copy()


def _as_input(x: np.ndarray):
    x = np.ascontiguousarray(x)
    if x.dtype == np.uint16:
        return x, DT_BF16
    if x.dtype == np.float16:
        return x.view(np.uint16), DT_F16
    if x.dtype == np.float32:
        return x, DT_F32
    raise TypeError(f"oracle input must be uint16 (bf16 bits), float16 or float32, got {x.dtype}")


def compress(x: np.ndarray, group_size: int = 32, mode: str | None = "balanced",
             num_candidates: int = 32, lo: float = 0.95, hi: float = 1.05, nthreads: int = 1):
    """(q uint8 [numel], scales uint16 [ceil(numel/G)], zp uint8 [...]) of a flat tensor.

    ``x``: uint16 array holding bf16 bit patterns, or float16 / float32 array.
    """
    xin, dt = _as_input(x)
    numel = xin.size
    ngroups = (numel + group_size - 1) // group_size
    q = np.empty(numel, np.uint8)
    s = np.empty(ngroups, np.uint16)
    zp = np.empty(ngroups, np.uint8)
    if mode is not None:
        num_candidates, lo, hi = PRESETS[mode]
    if mode == "quality":
        rc = lib().tcb_oracle_compress_quality(_ptr(xin), dt, numel, group_size, _ptr(q), _ptr(s), _ptr(zp), nthreads)
    else:
        m = linspace_multipliers(lo, hi, num_candidates)
        rc = lib().tcb_oracle_compress(_ptr(xin), dt, numel, group_size, _ptr(m), num_candidates,
                                       _ptr(q), _ptr(s), _ptr(zp), nthreads)
    if rc != 0:
        raise ValueError("oracle: unsupported group size / candidate count")
    return q, s, zp


def decompress(q: np.ndarray, scales: np.ndarray, zp: np.ndarray, group_size: int = 32,
               nthreads: int = 1, out: np.ndarray | None = None) -> np.ndarray:
    """bf16 bit patterns (uint16) of (q - zp) * scale, flat."""
    q = np.ascontiguousarray(q).reshape(-1)
    scales = np.ascontiguousarray(scales).reshape(-1)
    zp = np.ascontiguousarray(zp).reshape(-1)
    assert q.dtype == np.uint8 and scales.dtype == np.uint16 and zp.dtype == np.uint8
    if out is None:
        out = np.empty(q.size, np.uint16)
    lib().tcb_oracle_decompress(_ptr(q), _ptr(scales), _ptr(zp), _ptr(out), q.size, group_size, nthreads)
    return out


def compress_sym(x: np.ndarray, group_size: int = 32, adaptive: bool = False, num_candidates: int = 31,
                 nthreads: int = 1):
    """(q int8 [numel], scales uint16 [ceil(numel/G)]) of the symmetric codec; ``adaptive`` runs the
    reference's scale search over torch.linspace(0.90, 1.05, num_candidates)."""
    xin, dt = _as_input(x)
    numel = xin.size
    q = np.empty(numel, np.int8)
    s = np.empty((numel + group_size - 1) // group_size, np.uint16)
    m = linspace_multipliers(0.90, 1.05, num_candidates) if adaptive else None
    rc = lib().tcb_oracle_compress_sym(_ptr(xin), dt, numel, group_size, _ptr(m), num_candidates if adaptive else 0,
                                       _ptr(q), _ptr(s), nthreads)
    if rc != 0:
        raise ValueError("oracle: unsupported group size / candidate count")
    return q, s


def decompress_sym(q: np.ndarray, scales: np.ndarray, group_size: int = 32, nthreads: int = 1) -> np.ndarray:
    """bf16 bit patterns (uint16) of int8 q * scale, flat."""
    q = np.ascontiguousarray(q).reshape(-1)
    scales = np.ascontiguousarray(scales).reshape(-1)
    assert q.dtype == np.int8 and scales.dtype == np.uint16
    out = np.empty(q.size, np.uint16)
    lib().tcb_oracle_decompress_sym(_ptr(q), _ptr(scales), _ptr(out), q.size, group_size, nthreads)
    return out


def dequant_matmul(dense_bf16: np.ndarray, q: np.ndarray, scales: np.ndarray, zp: np.ndarray | None,
                   bias_bf16: np.ndarray | None, group_size: int = 32, nthreads: int = 1) -> np.ndarray:
    """fp32 [R_d, R_q] = dense [R_d, K] @ dequant(q [R_q, K])^T (+ bias), double accumulation."""
    R_d, K = dense_bf16.shape
    R_q = q.shape[0]
    out = np.empty((R_d, R_q), np.float32)
    dense_bf16 = np.ascontiguousarray(dense_bf16)
    q = np.ascontiguousarray(q).view(np.uint8)
    scales = np.ascontiguousarray(scales).reshape(-1)
    zpc = None if zp is None else np.ascontiguousarray(zp).reshape(-1)
    bc = None if bias_bf16 is None else np.ascontiguousarray(bias_bf16)
    lib().tcb_oracle_dequant_matmul(_ptr(dense_bf16), _ptr(q), _ptr(scales), _ptr(zpc), _ptr(bc), _ptr(out),
                                    R_d, R_q, K, group_size, nthreads)
    return out


def sum_group(e: np.ndarray) -> float:
    e = np.ascontiguousarray(e, np.float32)
    return float(lib().tcb_oracle_sum_group(_ptr(e), e.size))
