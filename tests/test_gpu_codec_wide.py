"""Parity of the widened codec surface with the reference, through the C ABI: the symmetric
codec (quantize_int8_g32 / quantize_int8_adaptive / dequantize_int8_g32) and the AMO-BQ codec
at the group sizes beyond 16 / 32 / 64.  Bit-exact bar against the golden fixtures (outputs
of the reference's CPU path) and the C oracle pinned to them."""
import ctypes

import numpy as np
import pytest
import torch

from tests import synth
from tests.test_gpu_codec import DT, _stream, abi_compress, abi_decompress
from tests.util import bits, from_bits

pytestmark = pytest.mark.gpu

ALL_G = (8, 16, 24, 32, 48, 64, 128)


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def L(built_lib):
    return built_lib


def abi_compress_sym(L, dev, x_np, dtype_tag, G, mult=None, x_off=0):
    """tcb_compress_sym on a device copy of x_np (uint16 bits for bf16 / f16, or float32)."""
    n = x_np.size
    ng = (n + G - 1) // G
    tdt = torch.float32 if dtype_tag == "f32" else torch.int16
    esz = 4 if dtype_tag == "f32" else 2
    xd = torch.zeros(n + x_off + 8, dtype=tdt, device=dev)
    xd[x_off:x_off + n] = torch.from_numpy(x_np.view(np.int16) if esz == 2 else x_np).to(dev)
    q = torch.full((n + 64,), 0x5A, dtype=torch.int8, device=dev)
    s = torch.full((ng + 8,), 0x5A5A, dtype=torch.int16, device=dev)
    if mult is None:
        mp, nc = None, 0
    else:
        m = np.ascontiguousarray(mult, np.float32)
        mp, nc = m.ctypes.data, len(m)
    rc = L.tcb_compress_sym(xd.data_ptr() + esz * x_off, DT[dtype_tag], n, G, mp, nc, q.data_ptr(), s.data_ptr(), _stream(dev))
    assert rc == 0, L.tcb_last_error()
    torch.cuda.synchronize(dev)
    qh, sh = q.cpu().numpy(), s.cpu().numpy().view(np.uint16)
    assert np.all(qh[n:] == 0x5A) and np.all(sh[ng:] == 0x5A5A), "encode wrote outside its outputs"
    return qh[:n].copy(), sh[:ng].copy()


def abi_decompress_sym(L, dev, q, s, G, q_off=0, out_off=0):
    n = q.size
    qd = torch.zeros(n + q_off + 64, dtype=torch.int8, device=dev)
    qd[q_off:q_off + n] = torch.from_numpy(q).to(dev)
    sd = from_bits(s).to(dev)
    canary = 0x7B7B
    od = torch.full((n + out_off + 64,), canary, dtype=torch.int16, device=dev)
    rc = L.tcb_decompress_sym(qd.data_ptr() + q_off, sd.data_ptr(), od.data_ptr() + 2 * out_off, n, G, _stream(dev))
    assert rc == 0, L.tcb_last_error()
    torch.cuda.synchronize(dev)
    o = od.cpu().numpy().view(np.uint16)
    assert np.all(o[:out_off] == canary) and np.all(o[out_off + n:] == canary), "decode wrote outside its output"
    return o[out_off:out_off + n].copy()


def check_sym_case(L, dev, g, name, x_np, tag, G, adaptive):
    q, s = abi_compress_sym(L, dev, x_np, tag, G, g["mult/adaptive"] if adaptive else None)
    assert np.array_equal(q, g[f"{name}/q"]), f"{name}: codes differ at {np.flatnonzero(q != g[f'{name}/q'])[:8]}"
    assert np.array_equal(s, g[f"{name}/s"]), f"{name}: scales"
    rec = abi_decompress_sym(L, dev, g[f"{name}/q"], g[f"{name}/s"], G)
    assert np.array_equal(rec, g[f"{name}/rec"]), f"{name}: decode"


# ------------------------------------------------------------------ golden vectors

@pytest.mark.parametrize("kind", ["sym", "adaptive"])
@pytest.mark.parametrize("G", ALL_G)
def test_golden_symmetric_main_block(L, dev, golden_extra, kind, G):
    check_sym_case(L, dev, golden_extra, f"main/{kind}/G{G}", golden_extra["x_main"], "bf16", G, kind == "adaptive")


@pytest.mark.parametrize("kind", ["sym", "adaptive"])
def test_golden_symmetric_ragged_and_nonfinite(L, dev, golden_extra, kind):
    for numel in synth.EDGE_NUMELS:
        for G in (16, 32, 24):
            if numel == 0:
                assert L.tcb_compress_sym(None, 0, 0, G, None, 0, None, None, None) == 0
                assert L.tcb_decompress_sym(None, None, None, 0, G, None) == 0
                continue
            check_sym_case(L, dev, golden_extra, f"ragged{numel}/{kind}/G{G}", golden_extra[f"x_ragged{numel}"], "bf16", G,
                           kind == "adaptive")
    xe = synth.edge_values()
    for tag, arr in (("bf16", bits(xe.to(torch.bfloat16))), ("f16", bits(xe.to(torch.float16))), ("f32", xe.numpy())):
        for G in (16, 32, 64):
            check_sym_case(L, dev, golden_extra, f"edge_{tag}/{kind}/G{G}", arr, tag, G, kind == "adaptive")


@pytest.mark.parametrize("mode", ["balanced", "quality"])
@pytest.mark.parametrize("G", [8, 24, 48, 128])
def test_golden_amo_other_group_sizes(L, dev, golden_small, golden_extra, mode, G):
    g = golden_small if G in (24, 48) else golden_extra
    name = f"main/{mode}/G{G}"
    q, s, zp = abi_compress(L, dev, g["x_main"], "bf16", G, mode, golden_small[f"mult/{mode}"])
    assert np.array_equal(q, g[f"{name}/q"]) and np.array_equal(s, g[f"{name}/s"]) and np.array_equal(zp, g[f"{name}/zp"])
    assert np.array_equal(abi_decompress(L, dev, g[f"{name}/q"], g[f"{name}/s"], g[f"{name}/zp"], G), g[f"{name}/rec"])


# --------------------------------------------------------------- against the oracle

def test_decode_all_group_sizes_and_alignments_against_oracle(L, dev):
    from oracle import amo_oracle as orc

    rng = np.random.default_rng(15)
    for G in ALL_G:
        for n in (1, 7, 8, 9, 47, 48, 49, 4096 + 5, 100_003):
            ng = (n + G - 1) // G
            q = rng.integers(0, 256, n, dtype=np.uint8)
            zp = rng.integers(0, 256, ng, dtype=np.uint8)
            s = bits(torch.exp(torch.rand(ng) * 12 - 9).to(torch.bfloat16))
            want = orc.decompress(q, s, zp, G)
            want_sym = orc.decompress_sym(q.view(np.int8), s, G)
            for q_off, out_off in ((0, 0), (0, 8), (8, 0), (16, 16), (1, 0), (0, 1), (3, 5)):
                assert np.array_equal(abi_decompress(L, dev, q, s, zp, G, q_off, out_off), want), (G, n, q_off, out_off)
                assert np.array_equal(abi_decompress_sym(L, dev, q.view(np.int8), s, G, q_off, out_off), want_sym), \
                    ("sym", G, n, q_off, out_off)


def test_decode_with_scales_and_zero_points_at_odd_addresses(L, dev):
    """The G = 8 / 24 / 48 kernels fetch several scales / zero points per load when the arrays allow it; views that start
    one element into a larger tensor (2-byte aligned scales, 1-byte aligned zero points) take the scalar loads instead.
    Same bits either way, codes and output on the 32-byte aligned fast path."""
    from oracle import amo_oracle as orc

    rng = np.random.default_rng(16)
    for G in (8, 24, 48, 16, 32):
        n = 96 * 4099       # a multiple of every group size in the loop
        ng = n // G
        q = rng.integers(0, 256, n, dtype=np.uint8)
        zp = rng.integers(0, 256, ng, dtype=np.uint8)
        s = bits(torch.exp(torch.rand(ng) * 12 - 9).to(torch.bfloat16))
        want, want_sym = orc.decompress(q, s, zp, G), orc.decompress_sym(q.view(np.int8), s, G)
        qd = torch.from_numpy(q).to(dev)
        for s_off, z_off in ((0, 0), (1, 1), (3, 2), (2, 3)):
            sd = torch.zeros(ng + 8, dtype=torch.int16, device=dev)
            sd[s_off:s_off + ng] = torch.from_numpy(s.view(np.int16)).to(dev)
            zd = torch.zeros(ng + 8, dtype=torch.uint8, device=dev)
            zd[z_off:z_off + ng] = torch.from_numpy(zp).to(dev)
            od = torch.empty(n, dtype=torch.int16, device=dev)
            rc = L.tcb_decompress_amo(qd.data_ptr(), sd.data_ptr() + 2 * s_off, zd.data_ptr() + z_off, od.data_ptr(), n, G, _stream(dev))
            assert rc == 0, L.tcb_last_error()
            assert np.array_equal(od.cpu().numpy().view(np.uint16), want), (G, s_off, z_off)
            rc = L.tcb_decompress_sym(qd.data_ptr(), sd.data_ptr() + 2 * s_off, od.data_ptr(), n, G, _stream(dev))
            assert rc == 0, L.tcb_last_error()
            assert np.array_equal(od.cpu().numpy().view(np.uint16), want_sym), ("sym", G, s_off)


def test_symmetric_decode_every_code_is_exact(L, dev):
    from oracle import amo_oracle as orc

    q = np.tile(np.arange(-128, 128, dtype=np.int8), 64)
    for sbits in (0x3C00, 0x3C7F, 0x0080, 0x0001, 0x7F7F, 0x3F80, 0x2A55, 0xBF80):
        s = np.full(q.size // 16, sbits, np.uint16)
        assert np.array_equal(abi_decompress_sym(L, dev, q, s, 16), orc.decompress_sym(q, s, 16)), hex(sbits)


def test_encode_every_group_size_against_oracle(L, dev):
    """Config-0 style values and magnitude extremes, all coders, every group size, ragged length."""
    from oracle import amo_oracle as orc

    g = torch.Generator().manual_seed(33)
    x0 = synth.config0_style(35, (3, 64, 96)).reshape(-1)[:-11]
    cases = [("bf16", bits(x0)), ("f32", x0.float().numpy()), ("f16", bits(x0.to(torch.float16)))]
    for scale in (1e-38, 1e-41, 1e30, 3e37):
        cases.append(("f32", (torch.randn(48 * 300 + 5, generator=g) * scale).numpy()))
    adaptive_m = orc.linspace_multipliers(0.90, 1.05, 31)
    for tag, arr in cases:
        for G in ALL_G:
            oarr = arr.view(np.float16) if tag == "f16" else arr
            for mode in ("fast", "quality"):
                want = orc.compress(oarr, G, mode, nthreads=4)
                m = orc.linspace_multipliers(*orc.PRESETS[mode][1:], orc.PRESETS[mode][0])
                got = abi_compress(L, dev, arr, tag, G, mode, m, x_off=1 if G == 24 else 0)
                for a, b, what in zip(got, want, ("codes", "scales", "zero points")):
                    assert np.array_equal(a, b), (tag, G, mode, what, np.flatnonzero(a != b)[:5])
            for adaptive in (False, True):
                want = orc.compress_sym(oarr, G, adaptive, nthreads=4)
                # offsets: 0 and 16 elements keep the streaming kernel's alignment, 1 and 8 force the general kernel
                for x_off in ((0, 1, 8, 16) if not adaptive else (1 if G == 48 else 0,)):
                    got = abi_compress_sym(L, dev, arr, tag, G, adaptive_m if adaptive else None, x_off=x_off)
                    for a, b, what in zip(got, want, ("codes", "scales")):
                        assert np.array_equal(a, b), (tag, G, "adaptive" if adaptive else "sym", x_off, what, np.flatnonzero(a != b)[:5])


def test_symmetric_streaming_encoder_boundary_cases(L, dev):
    """Values placed on and next to the rounding boundaries k + 0.5 of x / scale, where the reciprocal
    shortcut must hand over to the exact division, and groups whose maximum makes the bf16 scale round
    up or down."""
    from oracle import amo_oracle as orc

    rng = np.random.default_rng(77)
    n_groups = 16384
    for G in (16, 32, 64, 128):
        amax = np.exp(rng.uniform(-60, 60, n_groups)).astype(np.float32)
        sf = torch.from_numpy(amax / np.float32(127.0)).to(torch.bfloat16).float().numpy()
        k = rng.integers(-127, 127, (n_groups, G)).astype(np.float32) + 0.5
        x = k * sf[:, None]                                   # x / sf is a half-integer up to rounding
        ulps = rng.integers(-2, 3, x.shape)
        x = (x.view(np.int32) + ulps).view(np.float32)        # ... and its neighbours
        x[:, 0] = amax                                        # pin the group maximum
        x = np.clip(x, -amax[:, None], amax[:, None]).astype(np.float32).reshape(-1)
        xb = bits(torch.from_numpy(x).to(torch.bfloat16))     # bf16 values over a bf16 scale: exact ties are common
        for tag, arr in (("f32", x), ("bf16", xb)):
            want = orc.compress_sym(arr, G, False, nthreads=4)
            got = abi_compress_sym(L, dev, arr, tag, G)
            assert np.array_equal(got[1], want[1]), (G, tag, "scales")
            assert np.array_equal(got[0], want[0]), (G, tag, np.flatnonzero(got[0] != want[0])[:8])


def test_symmetric_benchmark_size_against_oracle(dev):
    """[16, 446, 768] config-0 tensor and two heavy-tailed [1024, 1024] slices through the Python API."""
    import tensorcache_b200 as tc
    from oracle import amo_oracle as orc

    for x in (synth.config0_style(0, (16, 446, 768)), synth.config2_slices(2)):
        xb = bits(x)
        for mode, adaptive in (("sym", False), ("adaptive", True)):
            q, s, shape = tc.compress(x.to(dev), mode, 32)
            oq, os_ = orc.compress_sym(xb, 32, adaptive, nthreads=orc.default_threads())
            assert tuple(shape) == tuple(x.shape) and q.dtype == torch.int8 and s.dtype == torch.bfloat16
            assert np.array_equal(q.cpu().numpy(), oq) and np.array_equal(bits(s.cpu()), os_)
            rec = tc.decompress(q, s, shape, None, 32)
            assert rec.shape == x.shape and np.array_equal(bits(rec.cpu()), orc.decompress_sym(oq, os_, 32))


def test_symmetric_python_api_contract(dev, golden_extra):
    import tensorcache_b200 as tc

    x = from_bits(golden_extra["x_main"]).reshape(6, 16, 96)
    # CPU tensors in, CPU tensors out (staged through the GPU), same bits as the reference
    q, s, shape = tc.quantize_int8_g32(x, 32)
    assert not q.is_cuda and np.array_equal(q.numpy(), golden_extra["main/sym/G32/q"]) and tuple(shape) == (6, 16, 96)
    q2, s2, _ = tc.quantize_int8_adaptive(x.to(dev), 32)
    assert q2.is_cuda and np.array_equal(q2.cpu().numpy(), golden_extra["main/adaptive/G32/q"])
    assert np.array_equal(bits(s2.cpu()), golden_extra["main/adaptive/G32/s"])
    buf = torch.empty(6, 16, 96, dtype=torch.bfloat16, device=dev)
    out = tc.dequantize_int8_g32(q2, s2, shape, 32, out_buffer=buf)
    assert out is buf and np.array_equal(bits(buf.cpu()), golden_extra["main/adaptive/G32/rec"])
    codec = tc.BlockwiseInt8Codec(group_size=64, adaptive=True)
    cq, cs, cshape = codec.quantize(x.to(dev))
    assert np.array_equal(cq.cpu().numpy(), golden_extra["main/adaptive/G64/q"])
    assert np.array_equal(bits(codec.dequantize(cq, cs, cshape).cpu()), golden_extra["main/adaptive/G64/rec"])
    with pytest.raises(ValueError):
        tc.dequantize_int8_g32(q2.view(torch.uint8), s2, shape, 32)
    # the symmetric codes are what FusedDequantLinear takes without zero points
    lin = tc.FusedDequantLinear(128, 256, bias=False, group_size=32).to(dev)
    a = torch.randn(64, 128, device=dev, dtype=torch.bfloat16)
    aq, as_, _ = tc.quantize_int8_g32(a, 32)
    y = lin(aq.view(64, 128), as_)
    ref = tc.dequantize_int8_g32(aq, as_, (64, 128), 32).float() @ lin.weight.float().t()
    assert (y.float() - ref).norm() / ref.norm() < 1e-2  # tolerance of the fused GEMM: rel. Frobenius <= 1e-2


def test_benchmark_tensor_and_auto_select_mode(dev, golden_small, golden_extra):
    import tensorcache_b200 as tc

    x = from_bits(golden_small["x_main"]).reshape(6, 16, 96)
    res = tc.benchmark_tensor(x.to(dev), 32, verbose=False, include_quality=True)
    assert set(res) == {"sym_g32", "adaptive", "amo_fast", "amo_balanced", "amo_accurate", "amo_max", "amo_quality"}
    xf = x.float().reshape(-1)
    for key, g, name in (("amo_balanced", golden_small, "main/balanced/G32"), ("amo_quality", golden_small, "main/quality/G32"),
                         ("sym_g32", golden_extra, "main/sym/G32"), ("adaptive", golden_extra, "main/adaptive/G32")):
        rec = from_bits(g[f"{name}/rec"]).float()
        want = (torch.norm(xf - rec) / torch.norm(xf)).item() * 100      # error of the reference's own output
        assert abs(res[key]["rel_rmse%"] - want) <= 1e-4 * want, key
        assert res[key]["ms"] > 0
    assert res["amo_max"]["N"] == 64 and res["amo_fast"]["lo"] == 0.95
    assert tc.auto_select_mode(x.to(dev), target_rmse=100.0) == "fast"
    assert tc.auto_select_mode(x.to(dev), target_rmse=0.0) == "G16_max"
    assert tc.auto_select_mode(x.to(dev), target_rmse=0.0, group_size=16, include_quality=True) == "quality"


def test_encoders_with_unaligned_output_pointers(L, dev):
    """Codes written to a byte pointer that is not 8-byte aligned (the lane kernels' byte-wise store path)."""
    from oracle import amo_oracle as orc

    x = bits(synth.config0_style(51, (2, 48, 96)).reshape(-1))
    n = x.size
    xd = torch.from_numpy(x.view(np.int16)).to(dev)
    for G in (8, 16, 24, 32, 64):
        ng = n // G
        for mode in ("balanced", "quality", "adaptive"):
            q = torch.full((n + 16,), 0x5A, dtype=torch.uint8, device=dev)
            s = torch.zeros(ng, dtype=torch.int16, device=dev)
            zp = torch.zeros(ng, dtype=torch.uint8, device=dev)
            off = 3
            if mode == "adaptive":
                m = orc.linspace_multipliers(0.90, 1.05, 31)
                rc = L.tcb_compress_sym(xd.data_ptr(), 0, n, G, m.ctypes.data, 31, q.data_ptr() + off, s.data_ptr(), _stream(dev))
                want_q, want_s = orc.compress_sym(x, G, True, nthreads=4)
                want_q = want_q.view(np.uint8)
            elif mode == "quality":
                rc = L.tcb_compress_amo_quality(xd.data_ptr(), 0, n, G, q.data_ptr() + off, s.data_ptr(), zp.data_ptr(), _stream(dev))
                want_q, want_s, _ = orc.compress(x, G, "quality", nthreads=4)
            else:
                m = orc.linspace_multipliers(0.95, 1.05, 32)
                rc = L.tcb_compress_amo(xd.data_ptr(), 0, n, G, m.ctypes.data, 32, q.data_ptr() + off, s.data_ptr(), zp.data_ptr(), _stream(dev))
                want_q, want_s, _ = orc.compress(x, G, "balanced", nthreads=4)
            assert rc == 0, L.tcb_last_error()
            torch.cuda.synchronize(dev)
            qh = q.cpu().numpy()
            assert np.all(qh[:off] == 0x5A) and np.all(qh[off + n:] == 0x5A), (G, mode, "wrote outside")
            assert np.array_equal(qh[off:off + n], want_q), (G, mode)
            assert np.array_equal(s.cpu().numpy().view(np.uint16), want_s), (G, mode)


def test_more_than_two_to_the_31_values(dev):
    """Index arithmetic past 2^31: encode (fast preset and plain symmetric) and decode 2^31 + 4096 + 5 values,
    checked against the oracle on windows at the start, across the 2^31 boundary and at the ragged end."""
    import tensorcache_b200 as tc
    from oracle import amo_oracle as orc

    n = (1 << 31) + 4096 + 5
    G = 32
    gen = torch.Generator(device=dev).manual_seed(99)
    tile = (torch.randn(1 << 20, generator=gen, device=dev) * 3).to(torch.bfloat16)
    x = tile.repeat((n + tile.numel() - 1) // tile.numel())[:n].contiguous()
    x[(1 << 31) - 7:(1 << 31) + 9] = torch.arange(16, device=dev, dtype=torch.float32).to(torch.bfloat16) - 4   # distinct values at the boundary
    windows = [(0, 1 << 16), ((1 << 31) - (1 << 15), (1 << 31) + (1 << 15)), (n - (1 << 15) - 5, n)]
    windows = [(a // G * G, b) for a, b in windows]
    q, s, zp, _ = tc.compress(x, "fast", G)
    rec = tc.decompress(q, s, (n,), zp, G)
    sq, ss, _ = tc.compress(x, "sym", G)
    srec = tc.decompress(sq, ss, (n,), None, G)
    torch.cuda.synchronize(dev)
    for a, b in windows:
        xw = bits(x[a:b].cpu())
        oq, os_, ozp = orc.compress(xw, G, "fast", nthreads=4)
        ga, gb = a // G, (b + G - 1) // G
        assert np.array_equal(q[a:b].cpu().numpy(), oq), (a, b)
        assert np.array_equal(bits(s[ga:gb].cpu()), os_) and np.array_equal(zp[ga:gb].cpu().numpy(), ozp), (a, b)
        assert np.array_equal(bits(rec[a:b].cpu()), orc.decompress(oq, os_, ozp, G)), (a, b)
        osq, oss = orc.compress_sym(xw, G, False, nthreads=4)
        assert np.array_equal(sq[a:b].cpu().numpy(), osq) and np.array_equal(bits(ss[ga:gb].cpu()), oss), ("sym", a, b)
        assert np.array_equal(bits(srec[a:b].cpu()), orc.decompress_sym(osq, oss, G)), ("sym", a, b)
