"""Pins the C oracle to the reference's own CPU implementation, bit for bit.

Needs the TensorCache sources on disk (``--reference <dir containing src/>``), so
it only runs where the reference is mounted; the committed fixtures under
``tests/golden/`` carry its outputs everywhere else.

    python oracle/check_against_reference.py --reference /path/to/TensorCache [--full]

Compares q / scale bits / zero points of ``tc.compress`` (CPU tensors) and the
bf16 bits of ``tc.decompress`` with the oracle, over the BASELINE-style synthetic
tensors, the edge cases of the reference tests (empty, 1, 31, 32, 33, 65, 1024,
1027 values; NaN / Inf; constant groups) and random group sizes; likewise the
symmetric codec (``quantize_int8_g32`` / ``quantize_int8_adaptive`` / ``dequantize_int8_g32``).
"""
from __future__ import annotations

import argparse
import sys
import time
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from oracle import amo_oracle as orc  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)


def config0_style(seed: int, shape):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    ch = torch.exp(0.5 * torch.randn(shape[-1], generator=g))
    x = x * ch
    mask = torch.rand(shape, generator=g) < 0.001
    x = torch.where(mask, 20 * x, x)
    return x.to(torch.bfloat16)


def student_t_style(seed: int, shape):
    g = torch.Generator().manual_seed(seed)
    ch = torch.exp(1.0 * torch.randn(shape[-1], generator=g))
    out = []
    for _ in range(shape[0]):
        z = torch.randn(shape[1:], generator=g)
        w = torch.randn((4,) + tuple(shape[1:]), generator=g)
        out.append((z / torch.sqrt((w * w).sum(0) / 4) * ch).to(torch.bfloat16))
    return torch.stack(out)


def to_oracle_input(x: torch.Tensor) -> np.ndarray:
    if x.dtype == torch.bfloat16:
        return bits(x)
    return x.contiguous().numpy().reshape(-1)


def compare(tc, x: torch.Tensor, mode, G, label, nthreads, **kw):
    t0 = time.time()
    if mode is None:
        q, s, zp, _ = tc.quantize_int8_amo_bq(x, G, **kw)
    else:
        q, s, zp, _ = tc.compress(x, mode, G)
    t1 = time.time()
    oq, os_, ozp = orc.compress(to_oracle_input(x), G, mode, nthreads=nthreads,
                                **({"num_candidates": kw.get("num_candidates", 32), "lo": kw.get("lo", 0.95),
                                    "hi": kw.get("hi", 1.05)} if mode is None else {}))
    t2 = time.time()
    dq = int((q.numpy().reshape(-1) != oq).sum())
    ds = int((bits(s) != os_).sum()) if s.numel() else 0
    dz = int((zp.numpy().reshape(-1) != ozp).sum())
    ok = dq == 0 and ds == 0 and dz == 0
    # decode parity on the same codes
    if q.numel():
        rec = tc.decompress(q, s, tuple(x.shape), zp, G)
        orec = orc.decompress(oq, os_, ozp, G, nthreads=nthreads)
        dr = int((bits(rec) != orec).sum())
    else:
        dr = 0
    ok = ok and dr == 0
    print(f"{'OK  ' if ok else 'FAIL'} {label:46s} numel={x.numel():>10d} q!={dq} s!={ds} zp!={dz} rec!={dr}"
          f"  ref {t1 - t0:6.2f}s oracle {t2 - t1:6.2f}s", flush=True)
    return ok


def compare_sym(tc, x: torch.Tensor, adaptive: bool, G, label, nthreads):
    """quantize_int8_g32 / quantize_int8_adaptive and dequantize_int8_g32 against the oracle."""
    from tensorcache.codec import dequantize_int8_g32, quantize_int8_adaptive, quantize_int8_g32

    t0 = time.time()
    q, s, _ = (quantize_int8_adaptive if adaptive else quantize_int8_g32)(x, G)
    t1 = time.time()
    oq, os_ = orc.compress_sym(to_oracle_input(x), G, adaptive, nthreads=nthreads)
    t2 = time.time()
    dq = int((q.numpy().reshape(-1) != oq).sum())
    ds = int((bits(s) != os_).sum()) if s.numel() else 0
    dr = 0
    if q.numel():
        rec = dequantize_int8_g32(q, s, tuple(x.shape), G)
        dr = int((bits(rec) != orc.decompress_sym(oq, os_, G, nthreads=nthreads)).sum())
    ok = dq == 0 and ds == 0 and dr == 0
    print(f"{'OK  ' if ok else 'FAIL'} {label:46s} numel={x.numel():>10d} q!={dq} s!={ds} rec!={dr}"
          f"  ref {t1 - t0:6.2f}s oracle {t2 - t1:6.2f}s", flush=True)
    return ok


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="directory of the TensorCache checkout (contains src/)")
    ap.add_argument("--full", action="store_true", help="also run the multi-million-value configurations")
    ap.add_argument("--threads", type=int, default=orc.default_threads())
    a = ap.parse_args()
    sys.path.insert(0, str(Path(a.reference) / "src"))
    import tensorcache as tc

    print("reference", tc.__version__, "torch", torch.__version__, torch.backends.cpu.get_cpu_capability())
    ok = True
    nt = a.threads

    # sum order, directly against torch on this host
    g = torch.Generator().manual_seed(123)
    for G in (8, 16, 24, 32, 48, 64, 128):
        e = torch.rand(20000, G, generator=g) * torch.exp(4 * torch.randn(20000, 1, generator=g))
        ref = e.sum(-1).numpy()
        mine = np.array([orc.sum_group(r) for r in e.numpy()], np.float32)
        bad = int((ref.view(np.uint32) != mine.view(np.uint32)).sum())
        print(f"{'OK  ' if bad == 0 else 'FAIL'} sum order G={G}: {bad} of {len(ref)} rows differ")
        ok &= bad == 0

    # edge sizes x modes x group sizes
    g = torch.Generator().manual_seed(7)
    for numel in (0, 1, 31, 32, 33, 65, 1024, 1027):
        x = (torch.randn(numel, generator=g) * 3).to(torch.bfloat16)
        for mode in ("fast", "balanced", "accurate", "max", "quality"):
            for G in (16, 32, 64):
                ok &= compare(tc, x, mode, G, f"edge numel={numel} {mode} G{G}", 1)
    # non-finite and constant groups (tests/test_fused_ops.py:89-107, tests/test_amo_quality.py:41-50)
    x = torch.randn(4096, generator=g)
    x[5] = float("nan"); x[40] = float("inf"); x[41] = float("-inf"); x[64:96] = float("nan")
    x[128:160] = 3.0; x[160:192] = -3.0; x[192:224] = 0.0; x[224:256] = 1e30; x[300] = -1e38; x[301] = 3e38
    for dt in (torch.bfloat16, torch.float32, torch.float16):
        xx = x.to(dt)
        for mode in ("fast", "balanced", "accurate", "max", "quality"):
            for G in (16, 32, 64):
                ok &= compare(tc, xx, mode, G, f"nonfinite/const {str(dt)[6:]} {mode} G{G}", 1)
    # other group sizes and custom candidate tables
    x = config0_style(11, (8, 96, 96))
    for G in (8, 24, 48, 128):
        for mode in ("balanced", "quality"):
            ok &= compare(tc, x, mode, G, f"odd G {mode} G{G}", nt)
    for n, lo, hi in ((1, 1.0, 1.0), (7, 0.9, 1.2), (64, 0.5, 1.5)):
        ok &= compare(tc, x, None, 32, f"custom N={n} {lo}-{hi}", nt, num_candidates=n, lo=lo, hi=hi)
    # tiny-magnitude and huge-magnitude data (denormal quotients, overflowing ranges)
    for scale in (1e-30, 1e-38, 1e-41, 1e30, 1e37):
        xx = (torch.randn(32 * 2000, generator=g) * scale).to(torch.float32)
        for mode in ("balanced", "quality"):
            ok &= compare(tc, xx, mode, 32, f"magnitude {scale:g} {mode}", nt)

    # symmetric codec (plain and with the adaptive scale search)
    g = torch.Generator().manual_seed(9)
    for numel in (0, 1, 31, 32, 33, 65, 1027):
        xx = (torch.randn(numel, generator=g) * 3).to(torch.bfloat16)
        for adaptive in (False, True):
            for G in (16, 32, 64):
                ok &= compare_sym(tc, xx, adaptive, G, f"sym edge numel={numel} adaptive={adaptive} G{G}", 1)
    xn = torch.randn(4096, generator=g)
    xn[5] = float("nan"); xn[40] = float("inf"); xn[41] = float("-inf"); xn[64:96] = float("nan")
    xn[128:160] = 3.0; xn[160:192] = -3.0; xn[192:224] = 0.0; xn[224:256] = 1e30; xn[300] = -1e38; xn[301] = 3e38
    for dt in (torch.bfloat16, torch.float32, torch.float16):
        for adaptive in (False, True):
            for G in (16, 32, 64):
                ok &= compare_sym(tc, xn.to(dt), adaptive, G, f"sym nonfinite/const {str(dt)[6:]} adaptive={adaptive} G{G}", 1)
    for G in (8, 24, 48, 128):
        for adaptive in (False, True):
            ok &= compare_sym(tc, x, adaptive, G, f"sym odd G adaptive={adaptive} G{G}", nt)
    for scale in (1e-30, 1e-38, 1e-41, 1e30, 1e37):
        xx = (torch.randn(32 * 2000, generator=g) * scale).to(torch.float32)
        for adaptive in (False, True):
            ok &= compare_sym(tc, xx, adaptive, 32, f"sym magnitude {scale:g} adaptive={adaptive}", nt)
    for adaptive in (False, True):
        ok &= compare_sym(tc, config0_style(0, (4, 446, 768)), adaptive, 32, f"sym config0[:4] adaptive={adaptive}", nt)
        ok &= compare_sym(tc, student_t_style(2, (2, 1024, 1024)), adaptive, 32, f"sym config2-slice adaptive={adaptive}", nt)

    # BASELINE-style tensors
    x0 = config0_style(0, (16, 446, 768))
    for mode, G in (("balanced", 32), ("fast", 32), ("balanced", 16), ("balanced", 64), ("quality", 32)):
        xs = x0 if a.full or mode == "balanced" and G == 32 else x0[:2]
        ok &= compare(tc, xs, mode, G, f"config0 {mode} G{G}", nt)
    x2 = student_t_style(2, (2, 1024, 1024))
    for mode, G in (("fast", 32), ("balanced", 16), ("balanced", 32), ("quality", 16), ("quality", 32)):
        ok &= compare(tc, x2, mode, G, f"config2-slice {mode} G{G}", nt)
    if a.full:
        x1 = config0_style(1, (128, 446, 768))
        for G in (32, 16):
            ok &= compare(tc, x1, "balanced", G, f"config1 balanced G{G}", nt)
        x2 = student_t_style(2, (16, 1024, 1024))
        for mode in ("accurate", "max", "quality"):
            ok &= compare(tc, x2, mode, 32, f"config2-16 {mode} G32", nt)
    print("ALL OK" if ok else "MISMATCHES FOUND")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
