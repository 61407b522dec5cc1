"""Mode "quality" against an independent brute-force search (the property the reference pins in
tests/test_amo_quality.py:13-38): the decoded squared error of the chosen (scale, zero point, codes)
must equal the best achievable over every bf16 scale of the search window and all 256 codes.
Also the reference's exact-reconstruction cases (:41-50) and the window-size bound (:53-59)."""
import numpy as np
import pytest
import torch

from tests.util import bits, from_bits


def _bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()


def brute_force_error(x: np.ndarray, G: int) -> float:
    pad = (-x.size) % G
    blocks = np.concatenate([x.astype(np.float32), np.zeros(pad, np.float32)]).reshape(-1, G)
    total = 0.0
    f32 = np.float32
    for blk in blocks:
        lower, upper = min(f32(blk.min()), f32(0)), max(f32(blk.max()), f32(0))
        scale0 = max(f32(upper / f32(255)) - f32(lower / f32(255)), f32(1e-8 / 255.0))
        lo = int(bits(torch.tensor([scale0 * f32(0.85)]).to(torch.bfloat16))[0])
        hi = int(bits(torch.tensor([scale0 * f32(1.10)]).to(torch.bfloat16))[0])
        assert 0 <= hi - lo < 64
        scales = from_bits(np.arange(lo, hi + 1, dtype=np.uint16)).float().numpy()
        zps = np.clip(np.rint((-lower / scales).astype(np.float32)), 0, 255)
        levels = _bf16_round((np.arange(256, dtype=np.float32)[None, :] - zps[:, None]) * scales[:, None])   # [S, 256]
        err = ((blk[None, :, None] - levels[:, None, :]) ** 2).min(axis=2).sum(axis=1)                      # [S]
        total += float(err.min())
    return total


def _case(G, dtype):
    g = torch.Generator().manual_seed(41 + G)
    return torch.randn(5 * G + 3, generator=g).to(dtype)


@pytest.mark.parametrize("G", [16, 24, 32, 48, 64])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_oracle_quality_reaches_the_brute_force_optimum(G, dtype):
    from oracle import amo_oracle as orc

    x = _case(G, dtype)
    xin = bits(x) if dtype == torch.bfloat16 else x.numpy()
    q, s, zp = orc.compress(xin, G, "quality")
    rec = from_bits(orc.decompress(q, s, zp, G)).float().numpy()
    got = float(((x.float().numpy() - rec) ** 2).sum())
    assert got == pytest.approx(brute_force_error(x.float().numpy(), G), rel=1e-5, abs=1e-9)


def test_search_window_never_needs_more_than_64_scales():
    m = (torch.arange(128, 256).float() / 128)
    for e in (-90, -10, 0, 30, 90):
        s0 = m * 2.0 ** e
        lo = (s0 * 0.85).to(torch.bfloat16).view(torch.int16).int()
        hi = (s0 * 1.10).to(torch.bfloat16).view(torch.int16).int()
        assert bool(((hi - lo) < 64).all())


@pytest.mark.gpu
@pytest.mark.parametrize("G", [16, 32, 64])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gpu_quality_reaches_the_brute_force_optimum(G, dtype):
    import tensorcache_b200 as tc

    x = _case(G, dtype)
    q, s, zp, shape = tc.compress(x.cuda(), "quality", G)
    assert q.dtype == torch.uint8 and zp.dtype == torch.uint8 and s.dtype == torch.bfloat16 and tuple(shape) == tuple(x.shape)
    rec = tc.decompress(q, s, shape, zp, G).float().cpu().numpy()
    got = float(((x.float().numpy() - rec) ** 2).sum())
    assert got == pytest.approx(brute_force_error(x.float().numpy(), G), rel=1e-5, abs=1e-9)


@pytest.mark.gpu
@pytest.mark.parametrize("G", [16, 32])
def test_gpu_quality_reconstructs_special_blocks_exactly(G):
    """empty input; NaN / +-Inf -> exactly 0; constant +3 / -3 / 0 blocks exactly."""
    import tensorcache_b200 as tc

    for x in (torch.empty(0), torch.tensor([float("nan"), float("inf"), -float("inf")]),
              torch.full((G,), 3.0), torch.full((G,), -3.0), torch.zeros(G)):
        q, s, zp, shape = tc.compress(x.cuda(), "quality", G)
        rec = tc.decompress(q, s, shape, zp, G)
        assert bool(torch.isfinite(s.float()).all()) and bool(torch.isfinite(rec.float()).all())
        want = torch.where(torch.isfinite(x), x, torch.zeros_like(x)).to(torch.bfloat16)
        assert torch.equal(rec.cpu(), want)
