"""ctypes binding of ``libtcb200.so`` (the C ABI declared in ``include/tcb200.h``).

There is no fallback: if the shared object is missing the import of any compute
entry point raises with the build command, and a failing call raises with the
library's own message.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libtcb200.so"

TCB_OK = 0
ERR_BAD_ARG, ERR_GROUP_SIZE, ERR_CUDA, ERR_TIMEOUT, ERR_ALIGNMENT, ERR_TOO_LARGE, ERR_IO, ERR_SUM_ORDER = 1, 2, 3, 4, 5, 6, 7, 8
DT_BF16, DT_F16, DT_F32 = 0, 1, 2
NOALLOC_MAX_VALUES = 4 * 1024 * 1024  # TCB_NOALLOC_MAX_VALUES

_vp, _i64, _i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
_pp = ctypes.POINTER(ctypes.c_void_p)


class StreamerDesc(ctypes.Structure):
    """Mirror of ``tcb_streamer_desc``."""

    _fields_ = [
        ("n_shards", _i32),
        ("q_bases", _pp),
        ("s_bases", _pp),
        ("zp_bases", _pp),
        ("shard_sizes", ctypes.POINTER(_i64)),
        ("values_per_sample", _i64),
        ("groups_per_sample", _i64),
        ("group_size", _i32),
        ("batch_size", _i32),
        ("n_slots", _i32),
        ("n_threads", _i32),
        ("pinned_q", _pp),
        ("pinned_s", _pp),
        ("pinned_zp", _pp),
        ("dev_q", _pp),
        ("dev_s", _pp),
        ("dev_zp", _pp),
        ("dev_out", _pp),
        ("direct_dma", _i32),
    ]


# name -> (restype, argtypes); every symbol include/tcb200.h declares
SIGNATURES = {
    "tcb_version": (_i32, []),
    "tcb_last_error": (ctypes.c_char_p, []),
    "tcb_selftest_sum_order": (_i32, [_vp, _i64, _i32, _vp]),
    "tcb_decompress_amo": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _vp]),
    "tcb_decompress_amo_host_noalloc": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _vp]),
    "tcb_compress_amo": (_i32, [_vp, _i32, _i64, _i32, _vp, _i32, _vp, _vp, _vp, _vp]),
    "tcb_compress_amo_quality": (_i32, [_vp, _i32, _i64, _i32, _vp, _vp, _vp, _vp]),
    "tcb_compress_sym": (_i32, [_vp, _i32, _i64, _i32, _vp, _i32, _vp, _vp, _vp]),
    "tcb_decompress_sym": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "tcb_fused_dequant_linear": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "tcb_fused_dequant_linear_check": (_i32, [_vp]),
    "tcb_selftest_bounded_wait": (_i32, [_i32, _vp]),
    "tcb_gather_rows": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _i32]),
    "tcb_write_block": (_i32, [_vp, _vp, _i64, _i32]),
    "tcb_pin_host_range": (_i32, [_vp, _i64]),
    "tcb_unpin_host_range": (_i32, [_vp]),
    "tcb_streamer_create": (_i32, [ctypes.POINTER(StreamerDesc), ctypes.POINTER(_vp)]),
    "tcb_streamer_num_samples": (_i32, [_vp, ctypes.POINTER(_i64)]),
    "tcb_streamer_begin": (_i32, [_vp, _vp, _i64]),
    "tcb_streamer_next": (_i32, [_vp, _vp, ctypes.POINTER(_i32), ctypes.POINTER(_i32)]),
    "tcb_streamer_acquire": (_i32, [_vp, _vp, ctypes.POINTER(_i32), ctypes.POINTER(_i32)]),
    "tcb_streamer_release": (_i32, [_vp, _vp]),
    "tcb_streamer_destroy": (_i32, [_vp]),
}

_lib = None


class TcbError(RuntimeError):
    """A call into libtcb200 returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libtcb200 error {code}: {message}")
        self.code = code


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA library with `python -m tensorcache_b200.build` "
                "(needs nvcc; there is no CPU or PyTorch fallback for this path)")
        L = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError here means a stale build
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int) -> None:
    """Maps a status to the reference's error convention: bad arguments are
    ValueError, everything else RuntimeError (the reference silently falls back
    on kernel failure; this library has nothing to fall back to)."""
    if rc == TCB_OK:
        return
    msg = lib().tcb_last_error().decode("utf-8", "replace")
    if rc in (ERR_BAD_ARG, ERR_GROUP_SIZE, ERR_ALIGNMENT, ERR_TOO_LARGE):
        raise ValueError(f"libtcb200: {msg}")
    raise TcbError(rc, msg)
