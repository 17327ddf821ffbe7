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
