"""C-ABI checks that need no GPU: the library loads, exports every symbol the
header declares, validates arguments before touching the device, and its
host-side row gather works."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "tcb200.h").read_text()
    return sorted(set(re.findall(r"TCB_API\s+[\w\s\*]+?\b(tcb_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ("tcb_decompress_amo", "tcb_compress_amo", "tcb_compress_amo_quality", "tcb_fused_dequant_linear", "tcb_gather_rows",
                 "tcb_streamer_create", "tcb_streamer_next", "tcb_last_error", "tcb_version"):
        assert must in names


def test_library_exports_every_declared_symbol(built_lib):
    from tensorcache_b200 import _lib

    for name in declared_symbols():
        assert hasattr(built_lib, name), f"{name} declared in include/tcb200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature in tensorcache_b200/_lib.py"
    assert built_lib.tcb_version() == 100


def test_argument_validation_happens_before_any_device_work(built_lib):
    from tensorcache_b200 import _lib

    L = built_lib
    assert L.tcb_decompress_amo(None, None, None, None, 0, 32, None) == _lib.TCB_OK            # empty is fine
    assert L.tcb_decompress_amo(None, None, None, None, 10, 20, None) == _lib.ERR_GROUP_SIZE
    assert b"group_size 20" in L.tcb_last_error()
    assert L.tcb_decompress_amo(None, None, None, None, 10, 24, None) == _lib.ERR_BAD_ARG       # 24 is a group size; nulls
    assert L.tcb_decompress_amo(None, None, None, None, -1, 32, None) == _lib.ERR_BAD_ARG
    assert L.tcb_decompress_amo(None, None, None, None, 10, 32, None) == _lib.ERR_BAD_ARG       # null pointers
    m = (ctypes.c_float * 4)(1, 1, 1, 1)
    assert L.tcb_compress_amo(None, 0, 10, 32, m, 0, None, None, None, None) == _lib.ERR_TOO_LARGE
    assert L.tcb_compress_amo(None, 0, 10, 32, m, 65, None, None, None, None) == _lib.ERR_TOO_LARGE
    assert L.tcb_compress_amo(None, 0, 10, 32, None, 4, None, None, None, None) == _lib.ERR_BAD_ARG
    assert L.tcb_compress_amo(None, 7, 10, 32, m, 4, None, None, None, None) == _lib.ERR_BAD_ARG  # dtype
    assert L.tcb_compress_amo_quality(None, 0, 10, 40, None, None, None, None) == _lib.ERR_GROUP_SIZE
    assert L.tcb_compress_sym(None, 0, 10, 32, m, 65, None, None, None) == _lib.ERR_TOO_LARGE
    assert L.tcb_compress_sym(None, 0, 10, 32, None, 4, None, None, None) == _lib.ERR_BAD_ARG     # table missing
    assert L.tcb_compress_sym(None, 0, 10, 12, None, 0, None, None, None) == _lib.ERR_GROUP_SIZE
    assert L.tcb_compress_sym(None, 0, 0, 32, None, 0, None, None, None) == _lib.TCB_OK
    assert L.tcb_decompress_sym(None, None, None, 0, 32, None) == _lib.TCB_OK
    assert L.tcb_decompress_sym(None, None, None, 10, 32, None) == _lib.ERR_BAD_ARG
    assert L.tcb_decompress_sym(None, None, None, 10, 7, None) == _lib.ERR_GROUP_SIZE
    assert L.tcb_fused_dequant_linear(None, None, None, None, None, None, 8, 8, 128, 24, 1, None) == _lib.ERR_GROUP_SIZE
    assert L.tcb_compress_amo_quality(None, 0, 0, 16, None, None, None, None) == _lib.TCB_OK
    assert L.tcb_fused_dequant_linear(None, None, None, None, None, None, 8, 8, 100, 32, 1, None) == _lib.ERR_BAD_ARG  # K % 64
    assert L.tcb_fused_dequant_linear(None, None, None, None, None, None, 8, 8, 128, 32, 1, None) == _lib.ERR_BAD_ARG  # nulls
    with pytest.raises(ValueError):
        _lib.check(_lib.ERR_GROUP_SIZE)


@pytest.mark.parametrize("nthreads", [1, 3, 8])
def test_gather_rows(built_lib, nthreads):
    rng = np.random.default_rng(0)
    src = rng.integers(0, 256, (50, 1000), dtype=np.uint8)
    idx = rng.permutation(50)[:17].astype(np.int64)
    dst = np.zeros((17, 1000), np.uint8)
    assert built_lib.tcb_gather_rows(dst.ctypes.data, src.ctypes.data, 1000, idx.ctypes.data, 0, 17, nthreads) == 0
    assert np.array_equal(dst, src[idx])
    dst2 = np.zeros((20, 1000), np.uint8)
    assert built_lib.tcb_gather_rows(dst2.ctypes.data, src.ctypes.data, 1000, None, 30, 20, nthreads) == 0
    assert np.array_equal(dst2, src[30:50])
    assert built_lib.tcb_gather_rows(dst2.ctypes.data, src.ctypes.data, 1000, None, 0, 0, nthreads) == 0
    assert built_lib.tcb_gather_rows(None, src.ctypes.data, 1000, None, 0, 5, nthreads) != 0


def test_gather_large_rows_take_the_streaming_copy_path(built_lib):
    """Rows of >= 4 KB are copied with cache-bypassing stores; odd sizes and unaligned
    destinations exercise its head / tail handling."""
    rng = np.random.default_rng(1)
    for row_bytes, off in ((4096, 0), (5003, 0), (342528, 0), (21408, 7), (10704, 1)):
        src = rng.integers(0, 256, (40, row_bytes), dtype=np.uint8)
        idx = rng.permutation(40)[:23].astype(np.int64)
        buf = np.full(23 * row_bytes + 64, 0xAB, np.uint8)
        dst = buf[off:off + 23 * row_bytes]
        assert built_lib.tcb_gather_rows(dst.ctypes.data, src.ctypes.data, row_bytes, idx.ctypes.data, 0, 23, 4) == 0
        assert np.array_equal(dst.reshape(23, row_bytes), src[idx]), (row_bytes, off)
        assert np.all(buf[:off] == 0xAB) and np.all(buf[off + 23 * row_bytes:] == 0xAB)


def test_product_package_does_not_touch_the_oracle():
    """The oracle is test infrastructure; nothing under tensorcache_b200/ may import it."""
    for p in (ROOT / "tensorcache_b200").rglob("*.py"):
        text = p.read_text()
        assert "oracle" not in text.replace("oracle/", ""), f"{p} mentions the oracle"
        assert "import triton" not in text and "torch.compile" not in text


def test_sum_order_selftest_passes_here_and_detects_another_order(built_lib):
    """tcb_selftest_sum_order (host only): this host's torch.sum(dim=-1) matches the order the encoders use,
    and a sum taken in plain left-to-right order is reported with its own status."""
    import ctypes

    import numpy as np
    import torch

    import tensorcache_b200 as tc
    from tensorcache_b200 import _lib

    tc.selftest_sum_order(rows_per_group_size=500)
    g = torch.Generator().manual_seed(1)
    e = (torch.rand(2000, 32, generator=g) * torch.exp(4 * torch.randn(2000, 1, generator=g))).contiguous()
    seq = np.zeros(2000, np.float32)
    for k in range(32):                       # strict left-to-right accumulation: another order
        seq = (seq + e[:, k].numpy()).astype(np.float32)
    assert not np.array_equal(seq.view(np.uint32), e.sum(-1).numpy().view(np.uint32))
    rc = built_lib.tcb_selftest_sum_order(ctypes.c_void_p(e.data_ptr()), 2000, 32, seq.ctypes.data)
    assert rc == _lib.ERR_SUM_ORDER and b"order" in built_lib.tcb_last_error()
    assert built_lib.tcb_selftest_sum_order(None, 0, 32, None) == 0
    assert built_lib.tcb_selftest_sum_order(ctypes.c_void_p(e.data_ptr()), 10, 20, seq.ctypes.data) == _lib.ERR_GROUP_SIZE
