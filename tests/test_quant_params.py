"""QuantParam math: oracle restatement and the library's host implementation against the
reference's known-answer tests.

Golden values are the ones asserted in the reference's own unit tests:
  src/Nncase.Tests/Core/UnitTestQuantUtility.cs:19-36
  src/Nncase.Tests/Quant/UnitTestQuantAlgorithm.cs:36-65
"""
import numpy as np
import pytest

from oracle import quant_params as QP

GOLDEN_QP = [
    # (min, max, bits, mode, zero_point, scale)
    (-1.0, 1.0, 8, QP.SIGNED_SYMMETRIC, 0, 0.007874016),
    (-1.0, 1.0, 8, QP.SIGNED_ASYMMETRIC, 0, 0.007843138),
    (-1.234, 2.345, 8, QP.UNSIGNED, 88, 0.014035294),
]
GOLDEN_FIXUP = [
    # (min, max, symmetric, out_min, out_max)
    (0.0, 0.0, False, 0.0, 0.1),
    (0.0, 0.0, True, -0.01, 0.01),
    (0.0, 0.005, False, 0.0, 0.01),
]


@pytest.mark.parametrize("mn,mx,bits,mode,zp,scale", GOLDEN_QP)
def test_oracle_get_quant_param(mn, mx, bits, mode, zp, scale):
    z, s = QP.get_quant_param(mn, mx, bits, mode)
    assert z == zp
    assert s == np.float32(scale)


@pytest.mark.parametrize("mn,mx,sym,omn,omx", GOLDEN_FIXUP)
def test_oracle_fixup_range(mn, mx, sym, omn, omx):
    a, b = QP.fixup_range(mn, mx, sym)
    assert a == np.float32(omn) and b == np.float32(omx)


def test_oracle_weights_ranges_by_channel():
    w = np.ones(16 * 3 * 3 * 3, np.float32)
    r = QP.weights_ranges_by_channel(w, 16)
    assert all(a == 0.0 and b == 1.0 for a, b in r)


@pytest.mark.parametrize("mn,mx,bits,mode,zp,scale", GOLDEN_QP)
def test_library_get_quant_param(mn, mx, bits, mode, zp, scale):
    from nncase_b200 import kernels as K
    qp = K.get_quant_param(mn, mx, bits, mode)
    assert qp.zero_point == zp
    assert np.float32(qp.scale) == np.float32(scale)


@pytest.mark.parametrize("mn,mx,sym,omn,omx", GOLDEN_FIXUP)
def test_library_fixup_range(mn, mx, sym, omn, omx):
    from nncase_b200 import kernels as K
    a, b = K.fixup_range(mn, mx, sym)
    assert np.float32(a) == np.float32(omn) and np.float32(b) == np.float32(omx)


def test_library_matches_oracle_on_random_ranges():
    from nncase_b200 import kernels as K
    rng = np.random.default_rng(7)
    for _ in range(500):
        a, b = np.sort(rng.normal(0, 3, 2)).astype(np.float32)
        for mode in (QP.UNSIGNED, QP.SIGNED_SYMMETRIC, QP.SIGNED_ASYMMETRIC):
            z, s = QP.get_quant_param(a, b, 8, mode)
            qp = K.get_quant_param(a, b, 8, mode)
            assert (qp.zero_point, np.float32(qp.scale)) == (z, s)


def test_invalid_mode_is_rejected():
    from nncase_b200 import kernels as K
    from nncase_b200.lib import NncbError
    with pytest.raises(NncbError) as e:
        K.get_quant_param(-1, 1, 8, 7)
    assert e.value.code == -22


# ---- calibration (Quantizer.GetRangesAsync / FixUpRange / per-channel weight params) -------------
def test_builder_calib_fixup_range_matches_oracle():
    """builder.calib_fixup_range against the restatement of Quantizer.FixUpRange (Quantizer.cs:358-387),
    including its edge cases: all-positive, all-negative, degenerate and sub-threshold ranges."""
    from nncase_b200 import builder
    cases = [(0.5, 2.0), (-3.0, -1.0), (0.0, 0.0), (0.0, 5e-7), (-1e-7, 1e-7), (-1.234, 2.345), (1e-6, 2e-6),
             (-7.5, 0.0), (3.0, 3.0)]
    rng = np.random.default_rng(15)
    cases += [tuple(np.sort(rng.normal(0, 2, 2))) for _ in range(200)]
    for mn, mx in cases:
        a, b = builder.calib_fixup_range(mn, mx)
        oa, ob = QP.calib_fixup_range(mn, mx)
        assert (np.float32(a), np.float32(b)) == (oa, ob), (mn, mx)


def test_builder_calibrate_is_the_union_of_finite_min_max():
    """builder.calibrate against Quantizer.GetRangesAsync (Quantizer.cs:389-409): per tensor, the union over
    the samples of GetMinMax (finite values only, Quantizer.Algorithms.cs:14-30), computed here with the
    oracle's get_min_max on the float tensors of an independent forward."""
    import torch

    from nncase_b200 import builder, networks
    g = networks.single_conv(seed=77, c=8, oc=8, hw=6)
    rng = np.random.default_rng(5)
    samples = [rng.uniform(-1, 1, (1, 8, 6, 6)).astype(np.float32) for _ in range(5)]
    samples[2][0, 0, 0, 0] = np.inf       # non-finite values do not enter a range
    samples[3][0, 1, 2, 3] = np.nan
    got = builder.calibrate(g, samples)
    want = {}
    for s in samples:
        _, tens = builder.float_forward(g, torch.from_numpy(s))
        for name, v in tens.items():
            mn, mx = QP.get_min_max(v.numpy())
            if name in want:
                want[name] = (min(want[name][0], mn), max(want[name][1], mx))
            else:
                want[name] = (mn, mx)
    assert set(want) <= set(got)
    assert np.float32(got["x"][0]) == want["x"][0] and np.float32(got["x"][1]) == want["x"][1]
    # the input range ignores the inf that was planted
    assert np.isfinite(got["x"][1]) and got["x"][1] <= 1.0
    # tensors downstream of the planted inf / nan are partly non-finite; only their finite part counts
    assert all(np.isfinite(v[0]) and np.isfinite(v[1]) for v in got.values())
    assert np.float32(got["y"][0]) == want["y"][0] and np.float32(got["y"][1]) == want["y"][1]


def test_builder_activation_and_weight_params_match_oracle():
    """activation_qp = GetQuantParam(FixUpRange(range), 8, Unsigned); quantize_weights = per-output-channel
    GetQuantParam of the raw channel min/max (Quantizer.cs:620-661) and q = clamp(rint(w / s + zp))."""
    from nncase_b200 import builder
    rng = np.random.default_rng(16)
    for _ in range(100):
        mn, mx = np.sort(rng.normal(0, 2, 2)).astype(np.float32)
        qp = builder.activation_qp((mn, mx))
        z, s = QP.get_quant_param(*QP.calib_fixup_range(mn, mx), 8, QP.UNSIGNED)
        assert (qp.zero_point, np.float32(qp.scale)) == (z, s)
    w = rng.normal(0, 0.05, (12, 6, 3, 3)).astype(np.float32)
    for wq_type, mode, lo, hi in (("uint8", QP.UNSIGNED, 0, 255), ("int8", QP.SIGNED_SYMMETRIC, -128, 127)):
        q, zps, scales = builder.quantize_weights(w, wq_type)
        oz, osc = QP.weights_quant_params(w, 12, 8, mode)
        assert np.array_equal(zps, oz) and np.array_equal(scales, osc)
        want = np.clip(np.rint(w / osc[:, None, None, None] + oz[:, None, None, None].astype(np.float32)), lo, hi)
        assert np.array_equal(q.astype(np.int32), want.transpose(0, 2, 3, 1).astype(np.int32))
