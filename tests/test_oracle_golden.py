"""The C oracle against what the reference itself produced (tests/golden/, made by
make_golden.py with the reference imported).  CPU only."""
import numpy as np
import pytest
import torch

from oracle import amo_oracle as orc
from tests import synth
from tests.util import MODES, bits, input_stream_mismatch, sha

NT = orc.default_threads()


def _check(g, name, x, mode, G, **kw):
    q, s, zp = orc.compress(x, G, mode, **kw)
    assert np.array_equal(q, g[f"{name}/q"]), f"{name}: codes"
    assert np.array_equal(s, g[f"{name}/s"]), f"{name}: scales"
    assert np.array_equal(zp, g[f"{name}/zp"]), f"{name}: zero points"
    rec = orc.decompress(q, s, zp, G)
    assert np.array_equal(rec, g[f"{name}/rec"]), f"{name}: decode"


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("G", [16, 32, 64])
def test_main_block(golden_small, mode, G):
    _check(golden_small, f"main/{mode}/G{G}", golden_small["x_main"], mode, G)


@pytest.mark.parametrize("G", [24, 48])
@pytest.mark.parametrize("mode", ["balanced", "quality"])
def test_other_group_sizes(golden_small, mode, G):
    _check(golden_small, f"main/{mode}/G{G}", golden_small["x_main"], mode, G)


@pytest.mark.parametrize("G", [8, 128])
@pytest.mark.parametrize("mode", ["balanced", "quality"])
def test_smallest_and_largest_group_size(golden_extra, mode, G):
    _check(golden_extra, f"main/{mode}/G{G}", golden_extra["x_main"], mode, G)


def _check_sym(g, name, x, adaptive, G):
    q, s = orc.compress_sym(x, G, adaptive)
    assert np.array_equal(q, g[f"{name}/q"]), f"{name}: codes"
    assert np.array_equal(s, g[f"{name}/s"]), f"{name}: scales"
    assert np.array_equal(orc.decompress_sym(q, s, G), g[f"{name}/rec"]), f"{name}: decode"


@pytest.mark.parametrize("kind", ["sym", "adaptive"])
@pytest.mark.parametrize("G", [8, 16, 24, 32, 48, 64, 128])
def test_symmetric_codec_main_block(golden_extra, kind, G):
    _check_sym(golden_extra, f"main/{kind}/G{G}", golden_extra["x_main"], kind == "adaptive", G)


@pytest.mark.parametrize("kind", ["sym", "adaptive"])
def test_symmetric_codec_ragged_and_nonfinite(golden_extra, kind):
    for numel in synth.EDGE_NUMELS:
        for G in (16, 32, 24):
            _check_sym(golden_extra, f"ragged{numel}/{kind}/G{G}", golden_extra[f"x_ragged{numel}"], kind == "adaptive", G)
    xe = synth.edge_values()
    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "f16"), (torch.float32, "f32")):
        xx = xe.to(dt)
        xin = bits(xx) if dt == torch.bfloat16 else xx.numpy()
        for G in (16, 32, 64):
            _check_sym(golden_extra, f"edge_{tag}/{kind}/G{G}", xin, kind == "adaptive", G)
    assert np.array_equal(orc.linspace_multipliers(0.90, 1.05, 31), golden_extra["mult/adaptive"])


@pytest.mark.parametrize("numel", synth.EDGE_NUMELS)
def test_ragged_sizes(golden_small, numel):
    for mode in ("balanced", "quality"):
        for G in (16, 32, 64):
            _check(golden_small, f"ragged{numel}/{mode}/G{G}", golden_small[f"x_ragged{numel}"], mode, G)


@pytest.mark.parametrize("tag", ["bf16", "f16", "f32"])
def test_nonfinite_and_constant_groups(golden_small, tag):
    xe = torch.from_numpy(golden_small["x_edge_f32"])
    x = {"bf16": lambda: bits(xe.to(torch.bfloat16)), "f16": lambda: xe.to(torch.float16).numpy(),
         "f32": lambda: xe.numpy()}[tag]()
    for mode in MODES:
        for G in (16, 32, 64):
            _check(golden_small, f"edge_{tag}/{mode}/G{G}", x, mode, G)


def test_edge_values_reconstruct_as_the_reference_tests_demand(golden_small):
    """tests/test_amo_quality.py:41-50 of the reference: non-finite -> exactly 0,
    constant +-3 and 0 groups exactly."""
    xe = torch.from_numpy(golden_small["x_edge_f32"])
    q, s, zp = orc.compress(xe.numpy(), 32, "quality")
    rec = torch.from_numpy(orc.decompress(q, s, zp, 32).view(np.int16)).view(torch.bfloat16).float()
    assert torch.all(rec[~torch.isfinite(xe)] == 0)
    assert torch.all(rec[128:160] == 3.0) and torch.all(rec[160:192] == -3.0) and torch.all(rec[192:224] == 0.0)


@pytest.mark.parametrize("n", [1, 7])
def test_custom_candidate_tables(golden_small, n):
    lo, hi = {1: (1.0, 1.0), 7: (0.9, 1.2)}[n]
    assert np.array_equal(orc.linspace_multipliers(lo, hi, n), golden_small[f"custom/N{n}/mult"])
    _check(golden_small, f"custom/N{n}", golden_small["x_main"], None, 32, num_candidates=n, lo=lo, hi=hi)


def test_preset_multiplier_tables_match_this_torch(golden_small):
    for mode, (n, lo, hi) in orc.PRESETS.items():
        assert np.array_equal(orc.linspace_multipliers(lo, hi, n), golden_small[f"mult/{mode}"]), mode


def test_sum_order_matches_torch_on_this_host():
    g = torch.Generator().manual_seed(9)
    for G in (16, 32, 64):
        e = torch.rand(4000, G, generator=g) * torch.exp(4 * torch.randn(4000, 1, generator=g))
        ref = e.sum(-1).numpy()
        mine = np.array([orc.sum_group(r) for r in e.numpy()], np.float32)
        assert np.array_equal(ref.view(np.uint32), mine.view(np.uint32)), f"G={G}"


DIGEST_CASES = [
    ("config0/balanced/G32", lambda: synth.config0_style(0, (16, 446, 768))),
    ("config0/quality/G16", lambda: synth.config0_style(0, (16, 446, 768))),
    ("config0/max/G32", lambda: synth.config0_style(0, (16, 446, 768))),
    ("config0/balanced/G64", lambda: synth.config0_style(0, (16, 446, 768))),
    ("config2_first16/balanced/G32", lambda: synth.config2_slices(16)),
]


@pytest.mark.parametrize("name,make", DIGEST_CASES, ids=[c[0] for c in DIGEST_CASES])
def test_benchmark_size_digests(digests, name, make):
    case = digests["cases"][name]
    x = make()
    if sha(bits(x)) != case["x"]:
        input_stream_mismatch(digests)
    q, s, zp = orc.compress(bits(x), case["group_size"], case["mode"], nthreads=NT)
    assert sha(q) == case["q"] and sha(s) == case["s"] and sha(zp) == case["zp"]
    assert sha(orc.decompress(q, s, zp, case["group_size"], nthreads=NT)) == case["rec"]


def test_dequant_matmul_oracle_against_torch():
    g = torch.Generator().manual_seed(3)
    X = torch.randn(24, 128, generator=g).to(torch.bfloat16)
    W = (0.02 * torch.randn(40, 128, generator=g)).to(torch.bfloat16)
    q, s, zp = orc.compress(bits(W), 32, "balanced")
    Wd = torch.from_numpy(orc.decompress(q, s, zp, 32).view(np.int16)).view(torch.bfloat16).view(40, 128)
    # the oracle multiplies the un-rounded fp32 dequantised weight
    qf = torch.from_numpy(q).float().view(40, 4, 32)
    sf = torch.from_numpy(s.view(np.int16)).view(torch.bfloat16).float().view(40, 4, 1)
    zf = torch.from_numpy(zp).float().view(40, 4, 1)
    Wf = ((qf - zf) * sf).view(40, 128)
    ref = X.double() @ Wf.double().T
    got = orc.dequant_matmul(bits(X).reshape(24, 128), q.reshape(40, 128), s, zp, None, 32, nthreads=2)
    assert np.allclose(got, ref.float().numpy(), rtol=1e-6, atol=1e-7)
    assert (Wd.float() - Wf).abs().max() <= Wf.abs().max() * 2 ** -8
