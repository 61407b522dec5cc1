"""The allocation-free decode entry point (host codes -> device bf16 through the library's
built-in staging array) against the regular entry point and the CPU oracle, through the C ABI.

This file is named so that pytest collects it last: if it fails under ``-x`` every other
test has already run.  It also passes when run alone in a fresh process."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(L, dev, q, s, zp, G):
    qd, sd, zd = (torch.from_numpy(a).to(dev) for a in (q, s.view(np.int16), zp))
    out = torch.empty(q.size, dtype=torch.int16, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    assert L.tcb_decompress_amo(qd.data_ptr(), sd.data_ptr(), zd.data_ptr(), out.data_ptr(), q.size, G, st) == 0, L.tcb_last_error()
    torch.cuda.synchronize(dev)
    return out.cpu().numpy()


def _noalloc(L, dev, q, s, zp, G):
    out = torch.full((q.size + 16,), 0x7B7B, dtype=torch.int16, device=dev)   # canary behind the output
    st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    rc = L.tcb_decompress_amo_host_noalloc(q.ctypes.data, s.ctypes.data, zp.ctypes.data, out.data_ptr(), q.size, G, st)
    assert rc == 0, L.tcb_last_error()
    torch.cuda.synchronize(dev)
    o = out.cpu().numpy()
    assert np.all(o[q.size:] == 0x7B7B)
    return o[:q.size]


def test_noalloc_decode_matches_regular_entry_point_on_consecutive_calls(built_lib):
    from oracle import amo_oracle as orc
    from tensorcache_b200 import _lib

    L = built_lib
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    rng = np.random.default_rng(17)
    # two calls in a row on the shared staging array: a large one, then a smaller one with other
    # data and another group size (stale bytes of the first call are still behind it), then a ragged one
    for numel, G in ((_lib.NOALLOC_MAX_VALUES, 32), (1_000_000, 16), (65 * 64 + 13, 64)):
        ng = (numel + G - 1) // G
        q = rng.integers(0, 256, numel, dtype=np.uint8)
        zp = rng.integers(0, 256, ng, dtype=np.uint8)
        s = torch.exp(torch.rand(ng) * 10 - 8).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).copy()
        want = _regular(L, dev, q, s, zp, G)
        got = _noalloc(L, dev, q, s, zp, G)
        assert np.array_equal(got, want), (numel, G)          # bit-exact, as every decode test
        got2 = _noalloc(L, dev, q, s, zp, G)                  # same call again
        assert np.array_equal(got2, want), (numel, G)
        assert np.array_equal(got.view(np.uint16), orc.decompress(q, s, zp, G)), (numel, G)   # and directly against the CPU oracle
    # a call after the set-up call takes no device memory: the free-memory figure of the driver does not move
    numel, G = 1 << 20, 32
    q = rng.integers(0, 256, numel, dtype=np.uint8)
    zp = rng.integers(0, 256, numel // G, dtype=np.uint8)
    s = np.full(numel // G, 0x3C00, np.uint16)
    out = torch.empty(numel, dtype=torch.int16, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize(dev)
    free_before = torch.cuda.mem_get_info(dev)[0]
    for _ in range(3):
        assert L.tcb_decompress_amo_host_noalloc(q.ctypes.data, s.ctypes.data, zp.ctypes.data, out.data_ptr(), numel, G, st) == 0
    torch.cuda.synchronize(dev)
    assert torch.cuda.mem_get_info(dev)[0] == free_before
    # sizes beyond the built-in staging area are refused before anything is enqueued
    big = np.zeros(8, np.uint8)
    rc = L.tcb_decompress_amo_host_noalloc(big.ctypes.data, big.ctypes.data, big.ctypes.data, 16, _lib.NOALLOC_MAX_VALUES + 1, 32, None)
    assert rc == _lib.ERR_TOO_LARGE and b"at most" in L.tcb_last_error()
    assert L.tcb_decompress_amo_host_noalloc(None, None, None, None, 0, 32, None) == 0
