"""Host-side logic that needs no GPU: the Python API surface, cache files written
by the reference, rank -> shard mapping, and a world_size-2 gloo run."""
import json
import os
import shutil
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import tensorcache_b200 as tc
from tensorcache_b200._pipeline import open_cache, resolve_shards
from tests.util import bits

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_api_surface_and_errors():
    assert set(tc.AMO_BQ_PRESETS) == {"fast", "balanced", "accurate", "max", "quality"}
    assert tc.AMO_BQ_PRESETS["accurate"][:3] == (48, 0.95, 1.10)
    c = tc.BlockwiseInt8Codec(group_size=16, amo_bq=True, amo_mode="quality")
    assert (c.amo_candidates, c.amo_lo, c.amo_hi) == (64, 0.85, 1.10)
    assert repr(tc.BlockwiseInt8Codec(32, amo_bq=True, amo_mode="balanced")) == \
        "BlockwiseInt8Codec(G=32, amo_bq=balanced 1.0938B 1:1.83x)"
    with pytest.raises(ValueError):
        tc.BlockwiseInt8Codec(amo_bq=True, amo_mode="nope")
    with pytest.raises(ValueError):
        tc.BlockwiseInt8Codec(adaptive=True, amo_bq=True)
    with pytest.raises(ValueError, match="unknown"):
        tc.compress(torch.zeros(4), mode="nope")
    with pytest.raises(ValueError):
        tc.quantize_int8_amo_bq(torch.zeros(64), group_size=20)
    with pytest.raises(ValueError):
        tc.quantize_int8_g32(torch.zeros(64), group_size=12)
    assert repr(tc.BlockwiseInt8Codec(32)) == "BlockwiseInt8Codec(G=32, sym 1:1.88x)"
    assert repr(tc.BlockwiseInt8Codec(32, adaptive=True)) == "BlockwiseInt8Codec(G=32, adaptive 0.90-1.05 1:1.88x)"
    e = tc.estimate_compression((16, 446, 768), 32)
    assert e["bytes_per_elem"] == 1.09375 and e["num_blocks"] == 171264


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_compute_calls_fail_loudly_without_a_gpu():
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        tc.compress(torch.zeros(64))
    with pytest.raises(RuntimeError):
        tc.decompress(torch.zeros(64, dtype=torch.uint8), torch.ones(2, dtype=torch.bfloat16), (64,),
                      torch.zeros(2, dtype=torch.uint8))


def test_rank_to_shard_rules():
    assert resolve_shards(8, None, 3, 8, False) == [3]
    assert resolve_shards(8, None, 9, 16, False) == [1]            # rank % num_shards, as the reference streamer
    assert resolve_shards(8, None, 1, 2, True) == [1, 3, 5, 7]
    assert resolve_shards(8, None, 5, 8, True) == [5]
    assert resolve_shards(8, 2, None, None, False) == [2]
    assert resolve_shards(8, None, None, None, False) is None
    with pytest.raises(ValueError):
        resolve_shards(8, 1, 0, 8, False)
    with pytest.raises(ValueError):
        resolve_shards(8, 8, None, None, False)
    covered = sorted(i for r in range(4) for i in resolve_shards(8, None, r, 4, True))
    assert covered == list(range(8))


@pytest.mark.parametrize("sub", ["cache_single", "cache_sharded"])
def test_reads_caches_written_by_the_reference(golden_rows, sub):
    ds = tc.FeatureCacheDataset(GOLDEN / sub / "feat")
    assert len(ds) == 7 and (ds.seq_len, ds.dim) == (6, 64)
    assert ds.group_size == (32 if sub == "cache_single" else 16)
    for i in range(7):
        q, s, zp = ds[i]
        assert q.dtype == torch.uint8 and s.dtype == torch.bfloat16 and zp.dtype == torch.uint8
        assert np.array_equal(q.numpy(), golden_rows[f"{sub}/{i}/q"])
        assert np.array_equal(bits(s), golden_rows[f"{sub}/{i}/s"])
        assert np.array_equal(zp.numpy(), golden_rows[f"{sub}/{i}/zp"])
    assert np.array_equal(ds[-1][0].numpy(), golden_rows[f"{sub}/6/q"])
    with pytest.raises(IndexError):
        ds[7]
    ds.close()


@pytest.mark.parametrize("sub", ["cache_sym_single", "cache_sym_sharded"])
def test_reads_symmetric_caches_written_by_the_reference(golden_sym_rows, sub):
    ds = tc.FeatureCacheDataset(GOLDEN / sub / "feat")
    assert len(ds) == 7 and not ds.amo_bq and ds.group_size == (32 if sub == "cache_sym_single" else 16)
    for i in range(7):
        row = ds[i]
        assert len(row) == 2 and row[0].dtype == torch.int8 and row[1].dtype == torch.bfloat16
        assert np.array_equal(row[0].numpy(), golden_sym_rows[f"{sub}/{i}/q"])
        assert np.array_equal(bits(row[1]), golden_sym_rows[f"{sub}/{i}/s"])
    ds.close()
    st = tc.ZeroCopyTensorStreamer(GOLDEN / "cache_sym_sharded" / "feat", batch_size=2, device="cpu", shuffle=False,
                                   rank=1, world_size=3)
    assert st.num_samples == int(golden_sym_rows["cache_sym_sharded/rank1_of_3/num_samples"][0]) and not st.amo_bq
    st.close()


def test_streamer_host_side_matches_reference_mapping(golden_rows):
    st = tc.ZeroCopyTensorStreamer(GOLDEN / "cache_sharded" / "feat", batch_size=2, device="cpu", shuffle=False,
                                   rank=1, world_size=3)
    assert st.num_samples == int(golden_rows["cache_sharded/rank1_of_3/num_samples"][0]) == 2
    assert st.shard_idx == 1 and len(st) == 1 and st.group_size == 16 and st.amo_bq
    st.close()
    whole = tc.ZeroCopyTensorStreamer(GOLDEN / "cache_sharded" / "feat", batch_size=4, device="cpu")
    assert whole.num_samples == 7 and len(whole) == 2 and whole.shard_sizes == [3, 2, 2]
    whole.close()
    with pytest.raises(ValueError):
        tc.ZeroCopyTensorStreamer(GOLDEN / "cache_sharded" / "feat", shard_idx=3, device="cpu")
    with pytest.raises(ValueError):
        tc.FeatureCacheDataset(GOLDEN / "cache_sharded" / "feat", shard_idx=0, rank=0, world_size=3)
    # the reference's dataset class opens shard 0 for every rank; this one follows the streamer rule
    ds = tc.FeatureCacheDataset(GOLDEN / "cache_sharded" / "feat", rank=2, world_size=3)
    assert len(ds) == 2 and np.array_equal(ds[0][0].numpy(), golden_rows["cache_sharded/5/q"])
    ds.close()


def test_truncated_and_missing_files_are_reported(tmp_path):
    for f in (GOLDEN / "cache_single").iterdir():
        shutil.copy(f, tmp_path / f.name)
    with open(tmp_path / "feat_int8.bin", "r+b") as f:
        f.truncate(100)
    with pytest.raises(ValueError, match="truncated"):
        tc.FeatureCacheDataset(tmp_path / "feat")
    os.remove(tmp_path / "feat_zp.bin")
    with pytest.raises((FileNotFoundError, ValueError)):
        tc.FeatureCacheDataset(tmp_path / "feat")


def test_writer_argument_checks(tmp_path):
    with pytest.raises(ValueError):
        tc.FeatureCacheWriter(tmp_path / "a", 4, 6, 64, group_size=0, amo_bq=True)
    with pytest.raises(ValueError):
        tc.FeatureCacheWriter(tmp_path / "a", 4, 6, 64, amo_bq=True, quant_bits=4)
    with pytest.raises(ValueError):
        tc.FeatureCacheWriter(tmp_path / "a", 4, 6, 64, amo_bq=True, amo_mode="nope")
    with pytest.raises(ValueError):
        tc.FeatureCacheWriter(tmp_path / "a", 4, 6, 64, adaptive=True, amo_bq=True)
    with pytest.raises(FileNotFoundError):
        tc.FeatureCacheWriter.open_append(tmp_path / "missing", 3)


def _gloo_worker(rank, world, port, prefix, q):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tensorcache_b200 import _lib

    lay = open_cache(prefix, None, rank, world, True)   # shards i with i % world == rank
    L = _lib.lib()
    sums = []
    for sh in lay.shards:
        dst = np.zeros((sh.num_samples, lay.seq_len * lay.dim), np.uint8)
        assert L.tcb_gather_rows(dst.ctypes.data, sh.q.ctypes.data, lay.seq_len * lay.dim, None, 0, sh.num_samples, 2) == 0
        sums.extend(int(r.astype(np.int64).sum()) for r in dst)
    mine = torch.zeros(8, dtype=torch.int64)
    mine[:len(sums)] = torch.tensor(sums)
    count = torch.tensor([len(sums)])
    gathered = [torch.zeros(8, dtype=torch.int64) for _ in range(world)]
    counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gathered, mine)
    dist.all_gather(counts, count)
    if rank == 0:
        q.put(([int(c) for c in counts], [g[:int(c)].tolist() for g, c in zip(gathered, counts)], lay.selected))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_cover_a_three_shard_cache_exactly_once(golden_rows):
    """world_size = 2 on CPU (gloo): every sample is read by exactly one rank, no exchange of data."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, str(GOLDEN / "cache_sharded" / "feat"), q)) for r in range(2)]
    for p in procs:
        p.start()
    counts, sums, selected0 = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert counts == [5, 2] and selected0 == [0, 2]     # rank 0: shards 0 and 2 (3 + 2 samples); rank 1: shard 1
    want = {i: int(golden_rows[f"cache_sharded/{i}/q"].astype(np.int64).sum()) for i in range(7)}
    assert sums[0] == [want[0], want[1], want[2], want[5], want[6]]
    assert sums[1] == [want[3], want[4]]


def test_manifest_written_for_per_shard_writers_equals_the_reference_manifest(tmp_path):
    """FeatureCacheWriter.write_manifest (the piece one rank adds when every rank filled its own shard) produces the
    manifest the reference's sharded writer wrote for the same cache, path strings aside.  Needs no GPU."""
    import json

    import tensorcache_b200 as tc

    ref = json.loads((GOLDEN / "cache_sharded" / "feat_shards.json").read_text())
    path = tc.FeatureCacheWriter.write_manifest(tmp_path / "feat", ref["num_samples"], ref["seq_len"], ref["dim"], ref["num_shards"],
                                                group_size=ref["group_size"], amo_bq=True, amo_mode=ref["amo_mode"])
    mine = json.loads(open(path).read())
    assert [os.path.basename(p) for p in mine["shard_prefixes"]] == [f"feat_shard{i}" for i in range(ref["num_shards"])]
    for k in ("shard_prefixes", "shard_metas"):
        mine.pop(k), ref.pop(k)
    assert mine == ref
    assert not list(tmp_path.glob("*.bin"))          # touches no data file
    with pytest.raises(ValueError):
        tc.FeatureCacheWriter.write_manifest(tmp_path / "single", 7, 6, 64, 1)
    with pytest.raises(TypeError):
        tc.FeatureCacheWriter.write_manifest(tmp_path / "bad", 7, 6, 64, 3, colour="red")


def test_prefaulter_populates_new_files_in_the_background_without_changing_them(tmp_path):
    """The writer's page population (madvise on the mappings of freshly created files): every page of every range ends
    up allocated, existing bytes stay, a stopped populator leaves its threads joined."""
    from tensorcache_b200._prefault import Prefaulter, filesystem_type, in_memory_filesystem
    base = Path("/dev/shm") if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else tmp_path
    folder = base / f"tcb_prefault_test_{os.getpid()}"
    folder.mkdir()
    try:
        assert filesystem_type(str(folder)) is not None
        if base != tmp_path:
            assert in_memory_filesystem(str(folder / "a.bin"))
        sizes = [5 << 20, (33 << 20) + 123, 4096]
        maps = [np.memmap(folder / f"f{i}.bin", dtype=np.uint8, mode="w+", shape=(n,)) for i, n in enumerate(sizes)]
        maps[0][:16] = np.arange(16, dtype=np.uint8)          # data that is already there survives
        pf = Prefaulter([(int(m.ctypes.data), int(m.nbytes)) for m in maps], threads=3)
        pf.stop()                                              # joins; whatever was not started stays unpopulated
        assert pf.done()
        pf = Prefaulter([(int(m.ctypes.data), int(m.nbytes)) for m in maps], threads=3)
        for t in pf._threads:
            t.join()
        assert pf.done()
        if not pf.failed:                                      # kernels before 5.14 refuse the advice; the writer then runs without
            assert pf.populated == sum(sizes)
            for i, n in enumerate(sizes):
                assert os.stat(folder / f"f{i}.bin").st_blocks * 512 >= n
        assert maps[0][:16].tolist() == list(range(16)) and int(maps[0][16:].max()) == 0 and int(maps[1].max()) == 0
        pf.stop()
        del maps
    finally:
        shutil.rmtree(folder, ignore_errors=True)
