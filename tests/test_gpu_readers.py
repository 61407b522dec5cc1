"""Writer / reader parity on the GPU: files byte-identical with the reference
writer's, batches bit-identical with decompress of the same codes."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import tensorcache_b200 as tc
from tests import synth
from tests.util import bits, from_bits

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
DEV = "cuda:0"


def _features(golden_rows):
    return from_bits(golden_rows["features"]).view(7, 6, 64)


@pytest.mark.parametrize("sub,kw", [("cache_single", dict(group_size=32, amo_mode="balanced")),
                                    ("cache_sharded", dict(group_size=16, amo_mode="quality", num_shards=3))])
def test_writer_output_is_byte_identical_with_the_reference_writer(tmp_path, golden_rows, sub, kw):
    feats = _features(golden_rows)
    w = tc.FeatureCacheWriter(tmp_path / "feat", 7, 6, 64, amo_bq=True, **kw)
    w.append(feats[:3].to(DEV))       # CUDA batch
    w.append(feats[3])                # single CPU sample
    w.append(feats[4:])               # CPU batch
    with pytest.raises(ValueError):
        w.append(feats[0])            # past capacity
    w.close()
    w.close()                          # idempotent
    for ref_file in sorted((GOLDEN / sub).iterdir()):
        mine = tmp_path / ref_file.name
        assert mine.exists(), ref_file.name
        if ref_file.suffix == ".bin":
            assert mine.read_bytes() == ref_file.read_bytes(), ref_file.name
        else:
            a, b = json.loads(mine.read_text()), json.loads(ref_file.read_text())
            for k in ("shard_prefixes", "shard_metas"):   # path strings differ by construction
                a.pop(k, None), b.pop(k, None)
            assert a == b, ref_file.name


def test_open_append_continues_a_cache(tmp_path, golden_rows):
    feats = _features(golden_rows)
    w = tc.FeatureCacheWriter(tmp_path / "feat", 4, 6, 64, group_size=32, amo_bq=True, amo_mode="balanced")
    w.append(feats[:4]); w.close()
    with pytest.raises(ValueError):
        tc.FeatureCacheWriter.open_append(tmp_path / "feat", 3, group_size=16)
    w = tc.FeatureCacheWriter.open_append(tmp_path / "feat", 3, group_size=32)
    w.append(feats[4:].to(DEV)); w.close()
    for name in ("feat_int8.bin", "feat_scales.bin", "feat_zp.bin"):
        assert (tmp_path / name).read_bytes() == (GOLDEN / "cache_single" / name).read_bytes()
    assert json.loads((tmp_path / "feat_meta.json").read_text())["num_samples"] == 7


@pytest.mark.parametrize("sub", ["cache_single", "cache_sharded"])
def test_readers_on_reference_written_caches(golden_rows, sub):
    want = np.concatenate([golden_rows[f"{sub}/{i}/rec"] for i in range(7)])
    prefix = GOLDEN / sub / "feat"
    # ring streamer, contiguous, B=2 -> partial last batch
    with tc.ZeroCopyTensorStreamer(prefix, batch_size=2, device=DEV, shuffle=False) as st:
        assert len(st) == 4 and st.out_bf16_0 is not None
        for _ in range(2):            # re-iterable
            got = [b.clone() for b in st]
            assert [g.shape[0] for g in got] == [2, 2, 2, 1]
            assert np.array_equal(bits(torch.cat(got)), want)
    # low_vram (single slot) and a batch larger than the cache
    with tc.ZeroCopyTensorStreamer(prefix, batch_size=16, device=DEV, shuffle=False, low_vram=True) as st:
        got = [b.clone() for b in st]
        assert len(got) == 1 and np.array_equal(bits(got[0]), want)
    # shuffled: every sample exactly once
    np.random.seed(3)
    with tc.ZeroCopyTensorStreamer(prefix, batch_size=3, device=DEV, shuffle=True) as st:
        got = torch.cat([b.clone() for b in st])
        order = st.indices.copy()
    per = want.reshape(7, -1)
    assert sorted(order.tolist()) == list(range(7))
    assert np.array_equal(bits(got).reshape(7, -1), per[order])
    # dataset: iter_batches (decoded and raw), auto_dequant_device
    ds = tc.FeatureCacheDataset(prefix, auto_dequant_device=DEV)
    assert np.array_equal(bits(ds[2]), golden_rows[f"{sub}/2/rec"])
    got = torch.cat([b.clone() for b in ds.iter_batches(batch_size=4, shuffle=False, device=DEV)])
    assert np.array_equal(bits(got), want)
    raw = list(ds.iter_batches(batch_size=4, shuffle=False, device=DEV, dequantize=False))
    assert len(raw) == 2 and raw[0][0].shape == (4, 6, 64) and raw[1][0].shape == (3, 6, 64)
    q = torch.cat([r[0] for r in raw]).cpu().numpy().reshape(7, -1)
    assert np.array_equal(q, np.stack([golden_rows[f"{sub}/{i}/q"].reshape(-1) for i in range(7)]))
    rec = tc.decompress(torch.cat([r[0] for r in raw]), torch.cat([r[1] for r in raw]), (7, 6, 64),
                        torch.cat([r[2] for r in raw]), ds.group_size)
    assert np.array_equal(bits(rec), want)
    ds.close()


def test_rank_sharding_on_the_gpu(golden_rows):
    prefix = GOLDEN / "cache_sharded" / "feat"
    with tc.ZeroCopyTensorStreamer(prefix, batch_size=2, device=DEV, shuffle=False, rank=1, world_size=3) as st:
        got = torch.cat([b.clone() for b in st])
    assert np.array_equal(bits(got), golden_rows["cache_sharded/rank1_of_3/rec"])
    seen = []
    for r in range(2):   # two ranks over three shards, every shard read once
        with tc.ZeroCopyTensorStreamer(prefix, batch_size=4, device=DEV, shuffle=False, rank=r, world_size=2, all_rank_shards=True) as st:
            seen.append(bits(torch.cat([b.clone() for b in st])).reshape(st.num_samples, -1))
    rows = {i: golden_rows[f"cache_sharded/{i}/rec"] for i in range(7)}
    assert np.array_equal(seen[0], np.stack([rows[i] for i in (0, 1, 2, 5, 6)]))
    assert np.array_equal(seen[1], np.stack([rows[i] for i in (3, 4)]))


def test_larger_cache_round_trip_and_early_exit(tmp_path):
    """2 shards x 160 samples of [32, 256]; contiguous and shuffled passes, abandoning a pass midway."""
    x = synth.config0_style(40, (320, 32, 256))
    w = tc.FeatureCacheWriter(tmp_path / "feat", 320, 32, 256, group_size=32, amo_bq=True, amo_mode="fast", num_shards=2)
    for i in range(0, 320, 100):
        w.append(x[i:i + 100].to(DEV))
    w.close()
    q, s, zp, _ = tc.compress(x.to(DEV), "fast", 32)
    want = bits(tc.decompress(q, s, (320, 32, 256), zp, 32)).reshape(320, -1)
    with tc.ZeroCopyTensorStreamer(tmp_path / "feat", batch_size=48, device=DEV, shuffle=False, gather_threads=4) as st:
        assert st.num_samples == 320 and len(st) == 7
        it = iter(st)
        next(it); next(it)            # leave the pass after two batches
        del it
        got = bits(torch.cat([b.clone() for b in st])).reshape(320, -1)
        assert np.array_equal(got, want)
        st.shuffle = True
        np.random.seed(11)
        got = bits(torch.cat([b.clone() for b in st])).reshape(320, -1)
        assert np.array_equal(got, want[st.indices])
    with tc.ZeroCopyTensorStreamer(tmp_path / "feat", batch_size=64, device=DEV, shuffle=False, shard_idx=1) as st:
        got = bits(torch.cat([b.clone() for b in st])).reshape(160, -1)
        assert np.array_equal(got, want[160:])


def test_resident_shard_mode_reads_the_same_batches(tmp_path, golden_rows):
    """pin_shard=True: the shard mappings are page-locked and the copy engine reads rows directly.
    Same bits as the staging path, contiguous (few long runs) and shuffled (one copy per row)."""
    want7 = np.concatenate([golden_rows[f"cache_sharded/{i}/rec"] for i in range(7)])
    with tc.ZeroCopyTensorStreamer(GOLDEN / "cache_sharded" / "feat", batch_size=3, device=DEV, shuffle=False, pin_shard=True) as st:
        for _ in range(2):
            assert np.array_equal(bits(torch.cat([b.clone() for b in st])), want7)
    x = synth.config0_style(41, (300, 32, 256))
    w = tc.FeatureCacheWriter(tmp_path / "feat", 300, 32, 256, group_size=32, amo_bq=True, amo_mode="fast", num_shards=3)
    w.append(x.to(DEV)); w.close()
    q, s, zp, _ = tc.compress(x.to(DEV), "fast", 32)
    want = bits(tc.decompress(q, s, (300, 32, 256), zp, 32)).reshape(300, -1)
    with tc.ZeroCopyTensorStreamer(tmp_path / "feat", batch_size=64, device=DEV, shuffle=False, pin_shard=True) as st:
        assert st.pin_shard and len(st) == 5
        assert np.array_equal(bits(torch.cat([b.clone() for b in st])).reshape(300, -1), want)
        st.shuffle = True
        np.random.seed(5)
        got = bits(torch.cat([b.clone() for b in st])).reshape(300, -1)
        assert np.array_equal(got, want[st.indices])
    with tc.ZeroCopyTensorStreamer(tmp_path / "feat", batch_size=50, device=DEV, shuffle=True, pin_shard=True, rank=2, world_size=3) as st:
        np.random.seed(6)
        got = bits(torch.cat([b.clone() for b in st])).reshape(100, -1)
        assert np.array_equal(got, want[200:][st.indices])


# ---------------------------------------------------------- caches of the symmetric codec

@pytest.mark.parametrize("sub,kw", [("cache_sym_single", dict(group_size=32)),
                                    ("cache_sym_sharded", dict(group_size=16, adaptive=True, num_shards=3))])
def test_symmetric_writer_output_is_byte_identical_with_the_reference_writer(tmp_path, golden_sym_rows, sub, kw):
    feats = from_bits(golden_sym_rows["features"]).view(7, 6, 64)
    w = tc.FeatureCacheWriter(tmp_path / "feat", 7, 6, 64, **kw)
    w.append(feats[:3].to(DEV)); w.append(feats[3]); w.append(feats[4:])
    w.close()
    assert not list(tmp_path.glob("*_zp.bin"))
    for ref_file in sorted((GOLDEN / sub).iterdir()):
        mine = tmp_path / ref_file.name
        assert mine.exists(), ref_file.name
        if ref_file.suffix == ".bin":
            assert mine.read_bytes() == ref_file.read_bytes(), ref_file.name
        else:
            a, b = json.loads(mine.read_text()), json.loads(ref_file.read_text())
            for k in ("shard_prefixes", "shard_metas"):
                a.pop(k, None), b.pop(k, None)
            assert a == b, ref_file.name


@pytest.mark.parametrize("sub", ["cache_sym_single", "cache_sym_sharded"])
def test_readers_on_reference_written_symmetric_caches(golden_sym_rows, sub):
    want = np.concatenate([golden_sym_rows[f"{sub}/{i}/rec"] for i in range(7)])
    prefix = GOLDEN / sub / "feat"
    for kw in (dict(), dict(pin_shard=False), dict(low_vram=True), dict(pin_shard=True)):
        with tc.ZeroCopyTensorStreamer(prefix, batch_size=2, device=DEV, shuffle=False, **kw) as st:
            assert not st.amo_bq
            for _ in range(2):
                assert np.array_equal(bits(torch.cat([b.clone() for b in st])), want), kw
    np.random.seed(4)
    with tc.ZeroCopyTensorStreamer(prefix, batch_size=3, device=DEV, shuffle=True) as st:
        got = torch.cat([b.clone() for b in st])
        assert np.array_equal(bits(got).reshape(7, -1), want.reshape(7, -1)[st.indices])
    ds = tc.FeatureCacheDataset(prefix, auto_dequant_device=DEV)
    assert np.array_equal(bits(ds[2]), golden_sym_rows[f"{sub}/2/rec"])
    got = torch.cat([b.clone() for b in ds.iter_batches(batch_size=4, shuffle=False, device=DEV)])
    assert np.array_equal(bits(got), want)
    raw = list(ds.iter_batches(batch_size=4, shuffle=False, device=DEV, dequantize=False))
    assert len(raw) == 2 and len(raw[0]) == 2 and raw[0][0].dtype == torch.int8
    rec = tc.decompress(torch.cat([r[0] for r in raw]), torch.cat([r[1] for r in raw]), (7, 6, 64), None, ds.group_size)
    assert np.array_equal(bits(rec), want)
    ds.close()
    if sub == "cache_sym_sharded":
        with tc.ZeroCopyTensorStreamer(prefix, batch_size=2, device=DEV, shuffle=False, rank=1, world_size=3) as st:
            assert np.array_equal(bits(torch.cat([b.clone() for b in st])), golden_sym_rows["cache_sym_sharded/rank1_of_3/rec"])


def test_larger_symmetric_cache_round_trip(tmp_path):
    """2 shards x 150 samples of [32, 256], adaptive codec: staging and resident paths, contiguous and shuffled."""
    x = synth.config0_style(42, (300, 32, 256))
    w = tc.FeatureCacheWriter(tmp_path / "feat", 300, 32, 256, group_size=32, adaptive=True, num_shards=2)
    w.append(x[:170].to(DEV)); w.append(x[170:]); w.close()
    q, s, _ = tc.compress(x.to(DEV), "adaptive", 32)
    want = bits(tc.decompress(q, s, (300, 32, 256), None, 32)).reshape(300, -1)
    for pin in (False, True):
        with tc.ZeroCopyTensorStreamer(tmp_path / "feat", batch_size=64, device=DEV, shuffle=False, pin_shard=pin) as st:
            assert np.array_equal(bits(torch.cat([b.clone() for b in st])).reshape(300, -1), want)
            st.shuffle = True
            np.random.seed(8)
            got = bits(torch.cat([b.clone() for b in st])).reshape(300, -1)
            assert np.array_equal(got, want[st.indices])


def test_benchmark_shape_cache_round_trip(tmp_path):
    """The benchmark's sample shape [446, 768], B = 128, two shards of 160 samples: every reader mode returns the
    bits of decompress(compress(rows)), contiguous and shuffled, with a partial last batch."""
    x = synth.config0_style(4, (320, 446, 768))
    w = tc.FeatureCacheWriter(tmp_path / "feat", 320, 446, 768, group_size=32, amo_bq=True, amo_mode="balanced", num_shards=2)
    w.append(x[:200].to(DEV)); w.append(x[200:]); w.close()
    q, s, zp, _ = tc.compress(x.to(DEV), "balanced", 32)
    want = tc.decompress(q, s, (320, 446, 768), zp, 32)
    for kw in (dict(), dict(pin_shard=False), dict(pin_shard=True)):
        with tc.ZeroCopyTensorStreamer(tmp_path / "feat", batch_size=128, device=DEV, shuffle=False, **kw) as st:
            assert len(st) == 3 and st.pin_shard == kw.get("pin_shard", True)   # automatic mode: resident, the shards are small
            got = torch.cat([b.clone() for b in st])
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), kw
            st.shuffle = True
            np.random.seed(12)
            got = torch.cat([b.clone() for b in st])
            idx = torch.from_numpy(st.indices.copy()).to(DEV)
            assert torch.equal(got.view(torch.int16), want[idx].view(torch.int16)), kw
    for r in range(2):
        with tc.FeatureCacheDataset(tmp_path / "feat", rank=r, world_size=2) as ds:
            got = torch.cat([b.clone() for b in ds.iter_batches(batch_size=128, shuffle=False, device=DEV)])
            assert torch.equal(got.view(torch.int16), want[160 * r:160 * (r + 1)].view(torch.int16))


def test_automatic_reader_mode_and_its_fallback(tmp_path, monkeypatch):
    """pin_shard=None (the default) page-locks the shard when it fits the memory budget and otherwise reads through
    staging copies with a warning; both return the same bits.  FeatureCacheDataset.iter_batches follows the same
    rule, pays the page-locking once, and reuses its ring for the next pass."""
    from tensorcache_b200 import _pipeline

    x = synth.config0_style(43, (150, 32, 256))
    w = tc.FeatureCacheWriter(tmp_path / "feat", 150, 32, 256, group_size=32, amo_bq=True, amo_mode="fast")
    w.append(x.to(DEV)); w.close()
    q, s, zp, _ = tc.compress(x.to(DEV), "fast", 32)
    want = bits(tc.decompress(q, s, (150, 32, 256), zp, 32)).reshape(150, -1)
    with tc.ZeroCopyTensorStreamer(tmp_path / "feat", batch_size=64, device=DEV, shuffle=False) as st:
        assert st.pin_shard is True
        assert np.array_equal(bits(torch.cat([b.clone() for b in st])).reshape(150, -1), want)
    with tc.FeatureCacheDataset(tmp_path / "feat") as ds:
        for _ in range(2):
            got = torch.cat([b.clone() for b in ds.iter_batches(batch_size=64, shuffle=False, device=DEV)])
            assert ds.pin_shard is True and np.array_equal(bits(got).reshape(150, -1), want)
        assert len(ds._idle_pipes) == 1 and not ds._pipes          # one ring, kept between the passes
        it = ds.iter_batches(batch_size=64, shuffle=False, device=DEV)
        first = next(it).clone()
        it.close()                                                  # an abandoned pass gives its ring back for reuse
        assert np.array_equal(bits(first).reshape(64, -1), want[:64]) and not ds._pipes and len(ds._idle_pipes) == 1
        got = torch.cat([b.clone() for b in ds.iter_batches(batch_size=64, shuffle=False, device=DEV)])
        assert np.array_equal(bits(got).reshape(150, -1), want)    # and the next pass starts from the beginning
        np.random.seed(3)
        raw = list(ds.iter_batches(batch_size=50, shuffle=False, device=DEV, dequantize=False))
        assert len(raw) == 3 and torch.equal(torch.cat([r[0] for r in raw]).view(-1), q)
    monkeypatch.setattr(_pipeline, "MEM_FRACTION_FOR_RESIDENT_SHARDS", 0.0)
    with pytest.warns(UserWarning, match="staging"):
        st = tc.ZeroCopyTensorStreamer(tmp_path / "feat", batch_size=64, device=DEV, shuffle=False)
    with st:
        assert st.pin_shard is False
        assert np.array_equal(bits(torch.cat([b.clone() for b in st])).reshape(150, -1), want)
    with pytest.raises(Exception):   # an explicit request is not silently downgraded: a read-only mapping cannot be page-locked
        lay = _pipeline.open_cache(tmp_path / "feat", private=False)
        try:
            _pipeline.try_make_resident(lay, torch.device(DEV), True)
        finally:
            lay.close()


def test_per_shard_writers_fill_the_same_cache_as_one_sharded_writer(tmp_path):
    """FeatureCacheWriter.for_shard + write_manifest (one process per shard) against FeatureCacheWriter(num_shards=3):
    every file byte-identical, manifests equal up to the path strings, and the readers take it by rank / world_size."""
    x = synth.config0_style(44, (100, 16, 128))
    kw = dict(group_size=16, amo_bq=True, amo_mode="balanced")
    one = tc.FeatureCacheWriter(tmp_path / "a" / "feat", 100, 16, 128, num_shards=3, **kw)
    one.append(x.to(DEV)); one.close()
    sizes, off = [34, 33, 33], 0
    for i, n in enumerate(sizes):
        w = tc.FeatureCacheWriter.for_shard(tmp_path / "b" / "feat", i, 100, 16, 128, 3, **kw)
        assert w.num_samples == n
        w.append(x[off:off + n].to(DEV)); w.close()
        off += n
    tc.FeatureCacheWriter.write_manifest(tmp_path / "b" / "feat", 100, 16, 128, 3, **kw)
    names = sorted(f.name for f in (tmp_path / "a").iterdir())
    assert names == sorted(f.name for f in (tmp_path / "b").iterdir()) and len(names) == 3 * 4 + 1
    for name in names:
        fa, fb = tmp_path / "a" / name, tmp_path / "b" / name
        if name.endswith(".bin"):
            assert fa.read_bytes() == fb.read_bytes(), name
        else:
            a, b = json.loads(fa.read_text()), json.loads(fb.read_text())
            for k in ("shard_prefixes", "shard_metas"):
                a.pop(k, None), b.pop(k, None)
            assert a == b, name
    q, s, zp, _ = tc.compress(x.to(DEV), "balanced", 16)
    want = bits(tc.decompress(q, s, (100, 16, 128), zp, 16)).reshape(100, -1)
    with tc.ZeroCopyTensorStreamer(tmp_path / "b" / "feat", batch_size=32, device=DEV, shuffle=False, rank=1, world_size=3) as st:
        assert st.num_samples == 33
        assert np.array_equal(bits(torch.cat([b.clone() for b in st])).reshape(33, -1), want[34:67])
    with pytest.raises(ValueError):
        tc.FeatureCacheWriter.for_shard(tmp_path / "c" / "feat", 3, 100, 16, 128, 3, **kw)


@pytest.mark.parametrize("prefault", [True, None])
def test_background_page_population_changes_no_byte(tmp_path, prefault):
    """A writer that populates its new files in the background (forced, and the automatic rule on memory-backed
    storage) writes the same bytes as one that leaves the files sparse, also when it is closed before it is full."""
    import os, shutil
    x = synth.config0_style(45, (300, 16, 128))
    kw = dict(group_size=32, amo_bq=True, amo_mode="balanced", num_shards=3)
    shm = Path("/dev/shm") / f"tcb_prefault_cache_{os.getpid()}"
    root = shm if (prefault is None and os.access("/dev/shm", os.W_OK)) else tmp_path / "p"
    try:
        plain = tc.FeatureCacheWriter(tmp_path / "a" / "feat", 400, 16, 128, prefault=False, **kw)
        assert plain._prefaulter is None
        plain.append(x.to(DEV)); plain.close()
        w = tc.FeatureCacheWriter(root / "feat", 400, 16, 128, prefault=prefault, **kw)
        assert w._prefaulter is None                                  # nothing is populated before data arrives
        w.append(x[:100].to(DEV))
        assert (w._prefaulter is not None) == (prefault is True or root == shm)
        w.append(x[100:]); w.close()                                  # 300 of 400 samples: the last shard stays partly empty
        assert w._prefaulter is None
        for f in sorted((tmp_path / "a").iterdir()):
            if f.suffix == ".bin":
                assert (root / f.name).read_bytes() == f.read_bytes(), f.name
    finally:
        shutil.rmtree(shm, ignore_errors=True)
