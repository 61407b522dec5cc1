"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE.

    cd tests/golden && python make_golden.py --reference /path/to/TensorCache

It imports TensorCache (v0.7.3) from ``<reference>/src`` and records what its CPU
PyTorch path produces:

* ``amo_small.npz``   inputs (bf16 / fp16 / fp32) and the full outputs
  (q, scale bits, zero points, decoded bf16 bits) for every AMO mode at
  G16/G32/G64, plus ragged sizes, non-finite values and constant groups.
* ``codec_extra.npz``  the same for the symmetric codec (``quantize_int8_g32``,
  ``quantize_int8_adaptive``, ``dequantize_int8_g32``) at G 8..128, and AMO-BQ at G8 / G128.
* ``cache_sym_single/``, ``cache_sym_sharded/``, ``cache_sym_rows.npz``  tiny caches of the
  symmetric codec (plain; adaptive with 3 shards) and the rows the reference's readers return.
* ``config_digests.json``  SHA-256 digests of the reference outputs on the
  full-size seeded synthetic tensors of the benchmark configurations (the
  inputs are regenerated from the seed by ``tests/synth.py``; their digests are
  recorded too so a different RNG stream is detected instead of mis-reported).
* ``cache_single/``, ``cache_sharded/``  tiny caches written by the reference's
  ``FeatureCacheWriter`` (single file set; 3 shards), and ``cache_rows.npz`` with
  the rows the reference's readers return for them.

Nothing here is read from the reference at test time; only these outputs are.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from tests import synth  # noqa: E402

MODES = ("fast", "balanced", "accurate", "max", "quality")


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1).copy()


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def make_codec_extra(tc):
    from tensorcache.codec import dequantize_int8_g32, quantize_int8_adaptive, quantize_int8_g32

    out = {}

    def record_sym(name, x, adaptive, G):
        q, s, _ = (quantize_int8_adaptive if adaptive else quantize_int8_g32)(x, G)
        out[f"{name}/q"] = q.numpy().reshape(-1).copy()
        out[f"{name}/s"] = bits(s)
        out[f"{name}/rec"] = bits(dequantize_int8_g32(q, s, tuple(x.shape), G)) if q.numel() else np.zeros(0, np.uint16)

    x = synth.config0_style(100, (6, 16, 96))  # the block of amo_small.npz
    out["x_main"] = bits(x)
    for G in (8, 16, 24, 32, 48, 64, 128):
        for adaptive in (False, True):
            record_sym(f"main/{'adaptive' if adaptive else 'sym'}/G{G}", x, adaptive, G)
    for G in (8, 128):
        for mode in ("balanced", "quality"):
            q, s, zp, _ = tc.compress(x, mode, G)
            out[f"main/{mode}/G{G}/q"] = q.numpy().reshape(-1).copy()
            out[f"main/{mode}/G{G}/s"] = bits(s)
            out[f"main/{mode}/G{G}/zp"] = zp.numpy().reshape(-1).copy()
            out[f"main/{mode}/G{G}/rec"] = bits(tc.decompress(q, s, tuple(x.shape), zp, G))
    g = torch.Generator().manual_seed(101)
    for numel in synth.EDGE_NUMELS:
        xr = (torch.randn(numel, generator=g) * 2.5).to(torch.bfloat16)
        out[f"x_ragged{numel}"] = bits(xr)
        for adaptive in (False, True):
            for G in (16, 32, 24):
                record_sym(f"ragged{numel}/{'adaptive' if adaptive else 'sym'}/G{G}", xr, adaptive, G)
    xe = synth.edge_values()
    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "f16"), (torch.float32, "f32")):
        for adaptive in (False, True):
            for G in (16, 32, 64):
                record_sym(f"edge_{tag}/{'adaptive' if adaptive else 'sym'}/G{G}", xe.to(dt), adaptive, G)
    out["mult/adaptive"] = torch.linspace(0.90, 1.05, 31).numpy().copy()
    np.savez_compressed("codec_extra.npz", **out)
    print("codec_extra.npz", os.path.getsize("codec_extra.npz"), "bytes,", len(out), "arrays")


def make_sym_caches(tc):
    """Caches of the symmetric codec written by the reference's writer, and what its readers return."""
    from tensorcache.codec import dequantize_int8_g32

    rows = {}
    for sub in ("cache_sym_single", "cache_sym_sharded"):
        shutil.rmtree(sub, ignore_errors=True)
        os.makedirs(sub)
    feats = synth.config0_style(102, (7, 6, 64))  # the samples of cache_single / cache_sharded
    rows["features"] = bits(feats)
    w = tc.FeatureCacheWriter("cache_sym_single/feat", 7, 6, 64, group_size=32)
    w.append(feats[:3]); w.append(feats[3]); w.append(feats[4:]); w.close()
    w = tc.FeatureCacheWriter("cache_sym_sharded/feat", 7, 6, 64, group_size=16, adaptive=True, num_shards=3)
    w.append(feats); w.close()
    for sub in ("cache_sym_single", "cache_sym_sharded"):
        ds = tc.FeatureCacheDataset(f"{sub}/feat")
        for i in range(len(ds)):
            q, s = ds[i]
            rows[f"{sub}/{i}/q"] = q.numpy().copy()
            rows[f"{sub}/{i}/s"] = bits(s)
            rows[f"{sub}/{i}/rec"] = bits(dequantize_int8_g32(q, s, (6, 64), ds.group_size))
        ds.close()
    st = tc.ZeroCopyTensorStreamer("cache_sym_sharded/feat", batch_size=2, device="cpu", shuffle=False, rank=1, world_size=3)
    rows["cache_sym_sharded/rank1_of_3/num_samples"] = np.array([st.num_samples])
    rows["cache_sym_sharded/rank1_of_3/rec"] = np.concatenate([bits(b) for b in st])
    st.close()
    np.savez_compressed("cache_sym_rows.npz", **rows)
    print("cache_sym_rows.npz", len(rows), "arrays")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--skip-large", action="store_true")
    ap.add_argument("--only-codec-extra", action="store_true",
                    help="regenerate codec_extra.npz and the symmetric-codec caches, nothing else")
    a = ap.parse_args()
    sys.path.insert(0, str(Path(a.reference) / "src"))
    import tensorcache as tc

    os.chdir(HERE)
    make_codec_extra(tc)
    make_sym_caches(tc)
    if a.only_codec_extra:
        return
    small = {}

    def record(name, x, mode, G, **kw):
        if mode is None:
            q, s, zp, _ = tc.quantize_int8_amo_bq(x, G, **kw)
        else:
            q, s, zp, _ = tc.compress(x, mode, G)
        small[f"{name}/q"] = q.numpy().reshape(-1).copy()
        small[f"{name}/s"] = bits(s)
        small[f"{name}/zp"] = zp.numpy().reshape(-1).copy()
        if q.numel():
            small[f"{name}/rec"] = bits(tc.decompress(q, s, tuple(x.shape), zp, G))
        else:
            small[f"{name}/rec"] = np.zeros(0, np.uint16)

    # 1. a config-0 style block, every mode and group size
    x = synth.config0_style(100, (6, 16, 96))  # 9216 values
    small["x_main"] = bits(x)
    for mode in MODES:
        for G in (16, 32, 64):
            record(f"main/{mode}/G{G}", x, mode, G)
    # 2. ragged sizes
    g = torch.Generator().manual_seed(101)
    for numel in synth.EDGE_NUMELS:
        xr = (torch.randn(numel, generator=g) * 2.5).to(torch.bfloat16)
        small[f"x_ragged{numel}"] = bits(xr)
        for mode in ("balanced", "quality"):
            for G in (16, 32, 64):
                record(f"ragged{numel}/{mode}/G{G}", xr, mode, G)
    # 3. non-finite values and constant groups, three input dtypes
    xe = synth.edge_values()
    small["x_edge_f32"] = xe.numpy().copy()
    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "f16"), (torch.float32, "f32")):
        xx = xe.to(dt)
        for mode in MODES:
            for G in (16, 32, 64):
                record(f"edge_{tag}/{mode}/G{G}", xx, mode, G)
    # 4. custom candidate tables (tests/test_fused_ops.py:74-86) and other group sizes
    for n, lo, hi in ((1, 1.0, 1.0), (7, 0.9, 1.2)):
        record(f"custom/N{n}", x, None, 32, num_candidates=n, lo=lo, hi=hi)
        small[f"custom/N{n}/mult"] = torch.linspace(lo, hi, n, dtype=torch.float32).numpy().copy()
    for G in (24, 48):
        for mode in ("balanced", "quality"):
            record(f"main/{mode}/G{G}", x, mode, G)
    # candidate tables of the presets, as the reference's torch.linspace gives them
    for mode, (n, lo, hi, _) in tc.AMO_BQ_PRESETS.items():
        small[f"mult/{mode}"] = torch.linspace(lo, hi, n, dtype=torch.float32).numpy().copy()
    np.savez_compressed("amo_small.npz", **small)
    print("amo_small.npz", os.path.getsize("amo_small.npz"), "bytes,", len(small), "arrays")

    # 5. digests at benchmark sizes
    dig = {"torch": torch.__version__, "reference": tc.__version__, "cases": {}}

    def digest_case(name, x, mode, G):
        q, s, zp, _ = tc.compress(x, mode, G)
        rec = tc.decompress(q, s, tuple(x.shape), zp, G)
        dig["cases"][name] = {
            "x": sha(bits(x)), "numel": x.numel(), "mode": mode, "group_size": G,
            "q": sha(q.numpy()), "s": sha(bits(s)), "zp": sha(zp.numpy()), "rec": sha(bits(rec)),
        }
        print(name, "done", flush=True)

    x0 = synth.config0_style(0, (16, 446, 768))
    for mode, G in (("balanced", 32), ("fast", 32), ("quality", 32), ("balanced", 16), ("balanced", 64),
                    ("quality", 16), ("accurate", 32), ("max", 32)):
        digest_case(f"config0/{mode}/G{G}", x0, mode, G)
    if not a.skip_large:
        x1 = synth.config0_style(1, (128, 446, 768))
        for G in (32, 16):
            digest_case(f"config1/balanced/G{G}", x1, "balanced", G)
        x2 = synth.config2_slices(16)
        for mode in ("fast", "balanced", "quality"):
            for G in (16, 32):
                digest_case(f"config2_first16/{mode}/G{G}", x2, mode, G)
        _, W = synth.config3_tensors(rows_x=8)
        digest_case("config3_weight/balanced/G32", W, "balanced", 32)
    with open("config_digests.json", "w") as f:
        json.dump(dig, f, indent=1, sort_keys=True)

    # 6. caches written by the reference writer, rows as the reference readers return them
    rows = {}
    for sub in ("cache_single", "cache_sharded"):
        shutil.rmtree(sub, ignore_errors=True)
        os.makedirs(sub)
    feats = synth.config0_style(102, (7, 6, 64))  # 7 samples of [6, 64]
    rows["features"] = bits(feats)
    w = tc.FeatureCacheWriter("cache_single/feat", 7, 6, 64, group_size=32, amo_bq=True, amo_mode="balanced")
    w.append(feats[:3]); w.append(feats[3]); w.append(feats[4:]); w.close()
    w = tc.FeatureCacheWriter("cache_sharded/feat", 7, 6, 64, group_size=16, amo_bq=True, amo_mode="quality",
                              num_shards=3)
    w.append(feats); w.close()
    for sub in ("cache_single", "cache_sharded"):
        ds = tc.FeatureCacheDataset(f"{sub}/feat")
        G = ds.group_size
        for i in range(len(ds)):
            q, s, zp = ds[i]
            rows[f"{sub}/{i}/q"] = q.numpy().copy()
            rows[f"{sub}/{i}/s"] = bits(s)
            rows[f"{sub}/{i}/zp"] = zp.numpy().copy()
            rows[f"{sub}/{i}/rec"] = bits(tc.decompress(q, s, (6, 64), zp, G))
        ds.close()
    st = tc.ZeroCopyTensorStreamer("cache_sharded/feat", batch_size=2, device="cpu", shuffle=False, rank=1, world_size=3)
    rows["cache_sharded/rank1_of_3/num_samples"] = np.array([st.num_samples])
    rows["cache_sharded/rank1_of_3/rec"] = np.concatenate([bits(b) for b in st])
    st.close()
    np.savez_compressed("cache_rows.npz", **rows)
    print("done")


if __name__ == "__main__":
    main()
