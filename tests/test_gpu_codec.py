"""Parity of the CUDA encode / decode kernels with the reference, through the C ABI.

Bit-exact bar: codes, scale bits, zero points and decoded bf16 bits must equal the
reference's CPU results (golden fixtures, and the C oracle pinned to them)."""
import ctypes

import numpy as np
import pytest
import torch

from tests import synth
from tests.util import MODES, bits, from_bits, input_stream_mismatch, sha

pytestmark = pytest.mark.gpu

DT = {"bf16": 0, "f16": 1, "f32": 2}


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def L(built_lib):
    return built_lib


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def abi_decompress(L, dev, q, s, zp, G, q_off=0, out_off=0):
    """Calls tcb_decompress_amo on device copies of numpy inputs; offsets (in elements)
    shift the q / out pointers to exercise unaligned addresses.  Checks canaries."""
    n = q.size
    pad = 64
    qd = torch.zeros(n + q_off + pad, dtype=torch.uint8, device=dev)
    qd[q_off:q_off + n] = torch.from_numpy(q).to(dev)
    sd = from_bits(s).to(dev)
    zd = torch.from_numpy(zp).to(dev)
    canary = 0x7B7B
    od = torch.full((n + out_off + pad,), canary, dtype=torch.int16, device=dev)
    rc = L.tcb_decompress_amo(qd.data_ptr() + q_off, sd.data_ptr(), zd.data_ptr(), od.data_ptr() + 2 * out_off, n, G, _stream(dev))
    assert rc == 0, L.tcb_last_error()
    torch.cuda.synchronize(dev)
    o = od.cpu().numpy().view(np.uint16)
    assert np.all(o[:out_off] == canary) and np.all(o[out_off + n:] == canary), "decode wrote outside its output"
    return o[out_off:out_off + n].copy()


def abi_compress(L, dev, x_np, dtype_tag, G, mode, mult=None, x_off=0):
    """Calls tcb_compress_amo / _quality.  x_np: uint16 bits (bf16/f16) or float32."""
    n = x_np.size
    ng = (n + G - 1) // G
    tdt = {"bf16": torch.int16, "f16": torch.int16, "f32": torch.float32}[dtype_tag]
    esz = 2 if tdt == torch.int16 else 4
    xd = torch.zeros(n + x_off + 8, dtype=tdt, device=dev)
    src = torch.from_numpy(x_np.view(np.int16) if esz == 2 else x_np).to(dev)
    xd[x_off:x_off + n] = src
    canary = 0x5A
    q = torch.full((n + 64,), canary, dtype=torch.uint8, device=dev)
    s = torch.full((ng + 8,), 0x5A5A, dtype=torch.int16, device=dev)
    zp = torch.full((ng + 8,), canary, dtype=torch.uint8, device=dev)
    xp = xd.data_ptr() + esz * x_off
    if mode == "quality":
        rc = L.tcb_compress_amo_quality(xp, DT[dtype_tag], n, G, q.data_ptr(), s.data_ptr(), zp.data_ptr(), _stream(dev))
    else:
        m = np.ascontiguousarray(mult, np.float32)
        rc = L.tcb_compress_amo(xp, DT[dtype_tag], n, G, m.ctypes.data, len(m), q.data_ptr(), s.data_ptr(), zp.data_ptr(), _stream(dev))
    assert rc == 0, L.tcb_last_error()
    torch.cuda.synchronize(dev)
    qh, sh, zh = q.cpu().numpy(), s.cpu().numpy().view(np.uint16), zp.cpu().numpy()
    assert np.all(qh[n:] == canary) and np.all(sh[ng:] == 0x5A5A) and np.all(zh[ng:] == canary), "encode wrote outside its outputs"
    return qh[:n].copy(), sh[:ng].copy(), zh[:ng].copy()


def check_case(L, dev, g, name, x_np, tag, G, mode, mult=None):
    q, s, zp = abi_compress(L, dev, x_np, tag, G, mode, mult)
    assert np.array_equal(q, g[f"{name}/q"]), f"{name}: codes differ at {np.flatnonzero(q != g[f'{name}/q'])[:8]}"
    assert np.array_equal(s, g[f"{name}/s"]), f"{name}: scales"
    assert np.array_equal(zp, g[f"{name}/zp"]), f"{name}: zero points"
    rec = abi_decompress(L, dev, g[f"{name}/q"], g[f"{name}/s"], g[f"{name}/zp"], G)
    assert np.array_equal(rec, g[f"{name}/rec"]), f"{name}: decode"


# ------------------------------------------------------------------ golden vectors

@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("G", [16, 32, 64])
def test_golden_main_block(L, dev, golden_small, mode, G):
    check_case(L, dev, golden_small, f"main/{mode}/G{G}", golden_small["x_main"], "bf16", G, mode, golden_small[f"mult/{mode}"])


@pytest.mark.parametrize("numel", synth.EDGE_NUMELS)
def test_golden_ragged_sizes(L, dev, golden_small, numel):
    for mode in ("balanced", "quality"):
        for G in (16, 32, 64):
            name = f"ragged{numel}/{mode}/G{G}"
            if numel == 0:
                m = (ctypes.c_float * 32)(*golden_small["mult/balanced"])
                assert L.tcb_compress_amo(None, 0, 0, G, m, 32, None, None, None, None) == 0
                assert L.tcb_decompress_amo(None, None, None, None, 0, G, None) == 0
                continue
            check_case(L, dev, golden_small, name, golden_small[f"x_ragged{numel}"], "bf16", G, mode, golden_small[f"mult/{mode}"])


@pytest.mark.parametrize("tag", ["bf16", "f16", "f32"])
def test_golden_nonfinite_and_constant_groups(L, dev, golden_small, tag):
    xe = torch.from_numpy(golden_small["x_edge_f32"])
    x = {"bf16": lambda: bits(xe.to(torch.bfloat16)), "f16": lambda: bits(xe.to(torch.float16)), "f32": lambda: xe.numpy()}[tag]()
    for mode in MODES:
        for G in (16, 32, 64):
            check_case(L, dev, golden_small, f"edge_{tag}/{mode}/G{G}", x, tag, G, mode, golden_small[f"mult/{mode}"])


@pytest.mark.parametrize("n", [1, 7])
def test_golden_custom_candidate_tables(L, dev, golden_small, n):
    check_case(L, dev, golden_small, f"custom/N{n}", golden_small["x_main"], "bf16", 32, None, golden_small[f"custom/N{n}/mult"])


# --------------------------------------------------------------- against the oracle

def test_decode_all_alignments_against_oracle(L, dev):
    from oracle import amo_oracle as orc

    rng = np.random.default_rng(5)
    for G in (16, 32, 64):
        for n in (1, 15, 16, 17, 4096 + 5, 100_003):
            ng = (n + G - 1) // G
            q = rng.integers(0, 256, n, dtype=np.uint8)
            zp = rng.integers(0, 256, ng, dtype=np.uint8)
            s = bits(torch.exp(torch.rand(ng) * 12 - 9).to(torch.bfloat16))
            want = orc.decompress(q, s, zp, G)
            for q_off, out_off in ((0, 0), (0, 8), (16, 0), (1, 0), (0, 1), (3, 5)):
                got = abi_decompress(L, dev, q, s, zp, G, q_off, out_off)
                assert np.array_equal(got, want), (G, n, q_off, out_off)


def test_decode_every_code_zero_point_pair_is_exact(L, dev):
    """All 65536 (q, zp) pairs against several scales: the exact-product argument, tested."""
    from oracle import amo_oracle as orc

    q = np.tile(np.arange(256, dtype=np.uint8), 256)                # group g holds q = 0..255 ...
    q = np.repeat(q.reshape(256, 256), 1, axis=0).reshape(-1)
    zp = np.repeat(np.arange(256, dtype=np.uint8), 256 // 16)        # ... with zp = g // 16 at G = 16
    for sbits in (0x3C00, 0x3C7F, 0x0080, 0x0001, 0x7F7F, 0x3F80, 0x2A55):
        s = np.full(q.size // 16, sbits, np.uint16)
        want = orc.decompress(q, s, zp, 16)
        got = abi_decompress(L, dev, q, s, zp, 16)
        assert np.array_equal(got, want), hex(sbits)


def test_encode_unaligned_input_and_magnitudes(L, dev):
    from oracle import amo_oracle as orc

    g = torch.Generator().manual_seed(21)
    for scale in (1.0, 1e-30, 1e-38, 1e-41, 1e30, 1e37):
        x = (torch.randn(32 * 700 + 13, generator=g) * scale)
        for tag, arr in (("f32", x.numpy()), ("bf16", bits(x.to(torch.bfloat16)))):
            for mode, G in (("balanced", 32), ("quality", 16), ("max", 64)):
                want = orc.compress(arr, G, mode, nthreads=4)
                for off in (0, 1):
                    got = abi_compress(L, dev, arr, tag, G, mode, orc.linspace_multipliers(*orc.PRESETS[mode][1:], orc.PRESETS[mode][0]), x_off=off)
                    for a, b, what in zip(got, want, ("codes", "scales", "zero points")):
                        assert np.array_equal(a, b), (scale, tag, mode, G, off, what)


# ----------------------------------------------------------- benchmark-size digests

def _digest_case(tc, dev, digests, name, x):
    case = digests["cases"][name]
    if sha(bits(x)) != case["x"]:
        input_stream_mismatch(digests)
    q, s, zp, shape = tc.compress(x.to(dev), case["mode"], case["group_size"])
    assert sha(q) == case["q"], f"{name}: codes"
    assert sha(s) == case["s"], f"{name}: scales"
    assert sha(zp) == case["zp"], f"{name}: zero points"
    out = torch.empty(shape, dtype=torch.bfloat16, device=dev)
    ret = tc.dequantize_int8_amo_bq(q, s, zp, shape, case["group_size"], out_buffer=out)
    assert ret is out
    assert sha(out) == case["rec"], f"{name}: decode"


def test_config0_digests(dev, digests):
    import tensorcache_b200 as tc

    x = synth.config0_style(0, (16, 446, 768))
    for name in [n for n in digests["cases"] if n.startswith("config0/")]:
        _digest_case(tc, dev, digests, name, x)


def test_config1_digests(dev, digests):
    import tensorcache_b200 as tc

    x = synth.config0_style(1, (128, 446, 768))
    for name in ("config1/balanced/G32", "config1/balanced/G16"):
        _digest_case(tc, dev, digests, name, x)


def test_config2_first_slices_digests(dev, digests):
    import tensorcache_b200 as tc

    x = synth.config2_slices(16)
    for name in [n for n in digests["cases"] if n.startswith("config2_first16/")]:
        _digest_case(tc, dev, digests, name, x)


def test_config3_weight_digest(dev, digests):
    import tensorcache_b200 as tc

    _, W = synth.config3_tensors(rows_x=8)
    _digest_case(tc, dev, digests, "config3_weight/balanced/G32", W)


def test_config2_full_size_against_oracle(dev):
    """[256,1024,1024] Student-t tensor drawn on the GPU; codes compared with the C oracle."""
    import tensorcache_b200 as tc
    from oracle import amo_oracle as orc

    gen = torch.Generator(device=dev).manual_seed(2)
    ch = torch.exp(torch.randn(1024, generator=gen, device=dev))
    x = torch.empty((256, 1024, 1024), dtype=torch.bfloat16, device=dev)
    for b in range(0, 256, 32):
        z = torch.randn((32, 1024, 1024), generator=gen, device=dev)
        w = torch.randn((4, 32, 1024, 1024), generator=gen, device=dev)
        x[b:b + 32] = (z / torch.sqrt((w * w).sum(0) / 4) * ch).to(torch.bfloat16)
        del z, w
    q, s, zp, _ = tc.compress(x, "balanced", 32)
    xh = bits(x)
    oq, os_, ozp = orc.compress(xh, 32, "balanced", nthreads=orc.default_threads())
    assert np.array_equal(q.cpu().numpy(), oq)
    assert np.array_equal(bits(s), os_) and np.array_equal(zp.cpu().numpy(), ozp)
    # size-independent property on the remaining modes: for groups whose range spans zero,
    # decode(encode(x)) stays within half a step, plus what a candidate scale below 1.0 may
    # clip off the ends of the range ((1 - 0.85) * 255 steps at most), plus half a bf16 ulp
    # of the largest value (the decoder rounds to bf16).  One-sided groups are excluded: the
    # preset modes do not force the range to include zero and clamp the zero point instead.
    for mode, G in (("fast", 16), ("quality", 32)):
        sub = x[:64]
        q, s, zp, shape = tc.compress(sub, mode, G)
        rec = tc.decompress(q, s, shape, zp, G)
        xs = sub.float().view(-1, G)
        err = (rec.float().view(-1, G) - xs).abs()
        bound = s.float().view(-1, 1) * (0.51 + 0.16 * 255) + xs.abs().amax(1, keepdim=True) * 2.0 ** -8
        spans_zero = (xs.amin(1) <= 0) & (xs.amax(1) >= 0)
        assert bool((err <= bound)[spans_zero].all()), mode
        assert int(spans_zero.sum()) > 0.9 * spans_zero.numel()
        sl = slice(0, 8 * 1024 * 1024)
        oq, os_, ozp = orc.compress(xh[sl], G, mode, nthreads=orc.default_threads())
        assert np.array_equal(q.cpu().numpy()[sl], oq) and np.array_equal(bits(s)[: oq.size // G], os_)


# ------------------------------------------------------------------- Python API

def test_python_api_contract(dev, golden_small):
    import tensorcache_b200 as tc

    x = from_bits(golden_small["x_main"]).view(6, 16, 96)
    q, s, zp, shape = tc.compress(x.to(dev))                      # default = balanced G32
    assert q.dtype == torch.uint8 and q.shape == (x.numel(),) and q.device.type == "cuda"
    assert s.dtype == torch.bfloat16 and zp.dtype == torch.uint8 and tuple(shape) == (6, 16, 96)
    assert np.array_equal(q.cpu().numpy(), golden_small["main/balanced/G32/q"])
    # CPU tensors are staged through the GPU and come back on the CPU
    qc, sc, zc, _ = tc.compress(x, "quality", 16)
    assert qc.device.type == "cpu" and np.array_equal(qc.numpy(), golden_small["main/quality/G16/q"])
    rc = tc.decompress(qc, sc, (6, 16, 96), zc, 16)
    assert rc.device.type == "cpu" and np.array_equal(bits(rc), golden_small["main/quality/G16/rec"])
    # non-contiguous input (tests/test_fused_ops.py:74-86 of the reference)
    xt = x.view(96, 96).t().to(dev)
    qa = tc.compress(xt, "fast", 32)[0]
    qb = tc.compress(xt.contiguous(), "fast", 32)[0]
    assert torch.equal(qa, qb)
    # codec object, out_buffer identity, [B, groups] shaped scales
    codec = tc.BlockwiseInt8Codec(group_size=32, amo_bq=True, amo_mode="balanced")
    q2, s2, z2, _ = codec.quantize(x.to(dev))
    out = torch.empty((6, 16, 96), dtype=torch.bfloat16, device=dev)
    assert codec.dequantize(q2.view(6, 16, 96), s2.view(6, -1), (6, 16, 96), zero_points=z2.view(6, -1), out_buffer=out) is out
    assert np.array_equal(bits(out), golden_small["main/balanced/G32/rec"])
    with pytest.raises(ValueError):
        tc.dequantize_int8_amo_bq(q2, s2[:3], z2, (6, 16, 96), 32)


def test_encoder_is_cuda_graph_capturable(dev):
    """tests/test_fused_ops.py:110-130 of the reference: no host sync inside the encoder."""
    import tensorcache_b200 as tc

    x = synth.config0_style(31, (4, 32, 64)).to(dev)
    static_x = x.clone()
    for mode, G in (("balanced", 32), ("quality", 16)):
        tc.compress(static_x, mode, G)  # warm-up outside capture
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            q, s, zp, _ = tc.compress(static_x, mode, G)
        y = synth.config0_style(32, (4, 32, 64)).to(dev)
        static_x.copy_(y)
        graph.replay()
        torch.cuda.synchronize(dev)
        q2, s2, zp2, _ = tc.compress(y, mode, G)
        assert torch.equal(q, q2) and torch.equal(s.view(torch.int16), s2.view(torch.int16)) and torch.equal(zp, zp2)


def test_decoder_is_cuda_graph_capturable(dev):
    """The decode launch carries a programmatic-dependent-launch attribute; it must still capture and replay."""
    import tensorcache_b200 as tc

    x = synth.config0_style(33, (8, 64, 128)).to(dev)
    q, s, zp, shape = tc.compress(x, "balanced", 32)
    want = tc.decompress(q, s, shape, zp, 32)
    out = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(3):
            tc.dequantize_int8_amo_bq(q, s, zp, shape, 32, out_buffer=out)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize(dev)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("G", [16, 32, 64])
def test_unpadded_low_precision_input_equals_zero_padded_fp32_input(dev, dtype, G):
    """tests/test_fused_ops.py:57-71 of the reference: the encoder reads bf16 / fp16 directly and pads
    ragged tails itself; the result must equal encoding the zero-padded fp32 copy."""
    import tensorcache_b200 as tc

    g = torch.Generator().manual_seed(77)
    for numel in (0, 1, 31, 32, 65, 1024):
        x = (torch.randn(numel, generator=g) * 4).to(dtype).to(dev)
        padded = torch.nn.functional.pad(x.float(), (0, (-numel) % G))
        for mode in ("balanced", "quality"):
            q1, s1, z1, _ = tc.compress(x, mode, G)
            q2, s2, z2, _ = tc.compress(padded, mode, G)
            assert torch.equal(q1, q2[:numel]) and torch.equal(z1, z2)
            assert torch.equal(s1.view(torch.int16), s2.view(torch.int16))


@pytest.mark.parametrize("mode", MODES)
def test_nonfinite_values_reconstruct_as_zero_in_every_mode(dev, mode):
    """tests/test_fused_ops.py:89-107 of the reference."""
    import tensorcache_b200 as tc

    g = torch.Generator().manual_seed(78)
    x = torch.randn(4, 96, generator=g)
    x[0, 3] = float("nan"); x[1, 40] = float("inf"); x[2, 41] = float("-inf"); x[3, :32] = float("nan")
    for G in (16, 32):
        q, s, zp, shape = tc.compress(x.to(torch.bfloat16).to(dev), mode, G)
        rec = tc.decompress(q, s, shape, zp, G).float().cpu()
        assert bool(torch.isfinite(s.float()).all()) and bool(torch.isfinite(rec).all())
        assert bool((rec[~torch.isfinite(x)] == 0).all())
        fin = torch.isfinite(x)
        assert float((rec[fin] - x[fin]).abs().max()) < 0.2
