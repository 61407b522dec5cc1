"""The scenarios of the reference's own tests for this path, run against tensorcache_b200 with the
same shapes, seeds and assertions (tests/test_codec.py:48-106, :570-650 and tests/test_amo_quality.py:53-135,
:165-200 of TensorCache).  Where the reference compares two of its own code paths, the comparison here
is between the writer / readers and `compress` / `decompress` of the same rows."""
import json

import pytest
import torch

import tensorcache_b200 as tc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel_rmse_percent(x, rec):
    return (torch.norm(x.float() - rec.float().cpu()) / torch.norm(x.float())).item() * 100.0


def test_quantize_dequantize_roundtrip():
    torch.manual_seed(42)
    x = torch.randn(16, 446, 768, dtype=torch.bfloat16)
    q, s, shape = tc.quantize_int8_g32(x, group_size=32)
    rec = tc.dequantize_int8_g32(q, s, shape, group_size=32)
    assert rec.shape == x.shape and rec.dtype == torch.bfloat16
    assert rel_rmse_percent(x, rec) < 1.0


def test_adaptive_quantize_roundtrip():
    torch.manual_seed(42)
    x = torch.randn(8, 128, 768, dtype=torch.bfloat16)
    q, s, shape = tc.quantize_int8_adaptive(x, group_size=32)
    rec = tc.dequantize_int8_g32(q, s, shape, group_size=32)
    assert rec.shape == x.shape
    assert rel_rmse_percent(x, rec) < 1.0


def test_feature_cache_disk_io(tmp_path):
    prefix = tmp_path / "test_feat_cache"
    num_samples, seq_len, dim = 20, 100, 256
    writer = tc.FeatureCacheWriter(prefix, num_samples=num_samples, seq_len=seq_len, dim=dim, group_size=32)
    writer.append(torch.randn(num_samples, seq_len, dim, dtype=torch.bfloat16))
    writer.close()
    dataset = tc.FeatureCacheDataset(prefix)
    assert len(dataset) == num_samples
    q_int8, scales = dataset[0]
    rec = tc.dequantize_int8_g32(q_int8, scales, (seq_len, dim), group_size=32)
    assert rec.shape == (seq_len, dim) and rec.dtype == torch.bfloat16
    dataset.close()
    writer.close()


def test_feature_cache_append_mode(tmp_path):
    prefix, ref_prefix = tmp_path / "append_feat", tmp_path / "ref_feat"
    N, M, seq_len, dim = 12, 7, 64, 128
    torch.manual_seed(0)
    feats_old = torch.randn(N, seq_len, dim, dtype=torch.bfloat16)
    feats_new = torch.randn(M, seq_len, dim, dtype=torch.bfloat16)
    writer = tc.FeatureCacheWriter(prefix, num_samples=N, seq_len=seq_len, dim=dim, group_size=32)
    writer.append(feats_old)
    writer.close()
    for bad in (dict(dim=999), dict(group_size=16), dict(amo_bq=True)):
        with pytest.raises(ValueError):
            tc.FeatureCacheWriter.open_append(prefix, M, **bad)
    with pytest.raises(FileNotFoundError):
        tc.FeatureCacheWriter.open_append(tmp_path / "nope", M)
    writer2 = tc.FeatureCacheWriter.open_append(prefix, extra_samples=M, group_size=32)
    assert writer2.current_idx == N
    writer2.append(feats_new)
    writer2.close()
    assert json.loads((tmp_path / "append_feat_meta.json").read_text())["num_samples"] == N + M
    ref = tc.FeatureCacheWriter(ref_prefix, num_samples=N + M, seq_len=seq_len, dim=dim, group_size=32)
    ref.append(torch.cat([feats_old, feats_new], dim=0))
    ref.close()
    ds, ref_ds = tc.FeatureCacheDataset(prefix), tc.FeatureCacheDataset(ref_prefix)
    assert len(ds) == N + M
    for i in range(N + M):
        (q, s), (rq, rs) = ds[i], ref_ds[i]
        assert torch.equal(q, rq) and torch.equal(s, rs), i
    ds.close()
    ref_ds.close()
    writer3 = tc.FeatureCacheWriter.open_append(prefix, extra_samples=1)
    with pytest.raises(ValueError):
        writer3.append(torch.randn(2, seq_len, dim, dtype=torch.bfloat16))
    writer3.close()
    assert json.loads((tmp_path / "append_feat_meta.json").read_text())["num_samples"] == N + M
    sharded = tmp_path / "sharded_feat"
    wsh = tc.FeatureCacheWriter(sharded, num_samples=4, seq_len=seq_len, dim=dim, group_size=32, num_shards=2)
    wsh.append(torch.randn(4, seq_len, dim, dtype=torch.bfloat16))
    wsh.close()
    with pytest.raises(NotImplementedError):
        tc.FeatureCacheWriter.open_append(sharded, 1)


def test_quality_grid_bound_covers_bf16_mantissas():
    scales = torch.arange(128, 256).float() / 128
    for exponent in (-90, -10, 0, 30, 90):
        scale0 = scales * 2.0 ** exponent
        lo = (scale0 * .85).bfloat16().view(torch.int16).int()
        hi = (scale0 * 1.10).bfloat16().view(torch.int16).int()
        assert ((hi - lo) < 64).all()      # the kernels' 64-candidate loop covers every bf16 scale in the window


def test_quality_cache_append_preserves_settings_and_rows(tmp_path):
    torch.manual_seed(42)
    x = torch.randn(3, 2, 32, dtype=torch.bfloat16)
    prefix = tmp_path / "quality"
    with tc.FeatureCacheWriter(prefix, 2, 2, 32, amo_bq=True, amo_mode="quality", group_size=16) as writer:
        writer.append(x[:2])
    old_bytes = (tmp_path / "quality_int8.bin").read_bytes()
    meta = json.loads((tmp_path / "quality_meta.json").read_text())
    assert meta["amo_mode"] == "quality" and meta["group_size"] == 16 and meta["amo_candidates"] == 64
    for settings in ({"amo_mode": "balanced"}, {"group_size": 32}):
        with pytest.raises(ValueError, match="mismatch"):
            tc.FeatureCacheWriter.open_append(prefix, 1, **settings)
        assert (tmp_path / "quality_int8.bin").read_bytes() == old_bytes
    with tc.FeatureCacheWriter.open_append(prefix, 1, amo_mode="quality", group_size=16) as writer:
        writer.append(x[2])
    assert (tmp_path / "quality_int8.bin").read_bytes().startswith(old_bytes)
    with tc.FeatureCacheDataset(prefix) as ds:
        assert len(ds) == 3
        for i in range(3):
            q, s, z = ds[i]
            expected = tc.compress(x[i], mode="quality", group_size=16)
            for actual, wanted in zip((q.flatten(), s, z), expected[:3]):
                assert torch.equal(actual, wanted)


def test_quality_sharded_cache_roundtrip(tmp_path):
    x = torch.randn(4, 2, 32, dtype=torch.bfloat16)
    prefix = tmp_path / "shards"
    with tc.FeatureCacheWriter(prefix, 4, 2, 32, amo_bq=True, amo_mode="quality", group_size=16, num_shards=2) as writer:
        writer.append(x)
    with tc.FeatureCacheDataset(prefix) as ds:
        assert ds.group_size == 16 and len(ds) == 4
        for i in range(4):
            q, s, z = ds[i]
            expected = tc.compress(x[i], mode="quality", group_size=16)
            assert torch.equal(q.flatten(), expected[0]) and torch.equal(s, expected[1]) and torch.equal(z, expected[2])


def test_quality_helpers_require_opt_in():
    x = torch.randn(64, dtype=torch.bfloat16)
    assert "amo_quality" not in tc.benchmark_tensor(x, verbose=False)
    assert "amo_quality" in tc.benchmark_tensor(x, verbose=False, include_quality=True)
    assert tc.auto_select_mode(x, target_rmse=0, group_size=16) == "max"
    assert tc.auto_select_mode(x, target_rmse=0, group_size=16, include_quality=True) == "quality"
    default, balanced = tc.compress(x), tc.compress(x, mode="balanced")
    assert all(torch.equal(a, b) for a, b in zip(default[:3], balanced[:3]))


@pytest.mark.parametrize("num_shards", [1, 2])
def test_quality_gpu_cache_batches_and_ring_streamer(tmp_path, num_shards):
    torch.manual_seed(53)
    x = torch.randn(5, 2, 32, dtype=torch.bfloat16, device=DEV)
    encoded = tc.compress(x, mode="quality", group_size=16)
    expected = tc.decompress(encoded[0], encoded[1], encoded[3], encoded[2], group_size=16)
    prefix = tmp_path / "gpu_quality"
    with tc.FeatureCacheWriter(prefix, 5, 2, 32, amo_bq=True, amo_mode="quality", group_size=16, num_shards=num_shards) as writer:
        writer.append(x)
    with tc.FeatureCacheDataset(prefix) as ds:
        batches = [batch.clone() for batch in ds.iter_batches(batch_size=2, shuffle=False, device=DEV)]
        assert torch.equal(torch.cat(batches), expected)
    with tc.ZeroCopyTensorStreamer(prefix, batch_size=2, device=DEV, shuffle=False) as streamer:
        batches = [batch.clone() for batch in streamer]
        assert torch.equal(torch.cat(batches), expected)


def test_fused_dequant_linear_reference_shapes():
    """tests/test_fused_ops.py:255-281: M, K, N = 128, 768, 512 with the symmetric codec's own codes."""
    torch.manual_seed(0)
    M, K, N = 128, 768, 512
    x = torch.randn(M, K, dtype=torch.bfloat16, device=DEV)
    q_int8, scales, shape = tc.quantize_int8_g32(x, group_size=32)
    layer = tc.FusedDequantLinear(K, N, bias=True, group_size=32).to(DEV)
    y = layer(q_int8.view(M, K), scales)
    x_rec = tc.dequantize_int8_g32(q_int8, scales, shape, group_size=32)
    y_ref = torch.nn.functional.linear(x_rec.float(), layer.weight.float(), layer.bias.float())
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert (torch.norm(y.float() - y_ref) / torch.norm(y_ref)).item() < 1e-2   # rel. Frobenius, the benchmark's tolerance
