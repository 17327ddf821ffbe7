"""QuantParam and range math of the reference, restated in numpy.

TEST INFRASTRUCTURE ONLY. Follows
  src/Nncase.Core/Utilities/QuantUtility.cs:41-67   GetQuantParam
  src/Nncase.Core/Utilities/QuantUtility.cs:72-97   FixupRange
  src/Nncase.Core/Utilities/QuantUtility.cs:106-151 GetWeightsRangesByChannel
  src/Nncase.Quantization/Quantization/Quantizer.Algorithms.cs:14-30  GetMinMax (finite only)
  src/Nncase.Quantization/Quantization/Quantizer.cs:358-387           calibration FixUpRange
Pinned by the reference's known-answer tests (tests/test_quant_params.py lists them).

Arithmetic notes: ranges are C# ``float``; ``range.Max - range.Min`` is a float subtraction,
the divisions run in double, ``Math.Round`` rounds half to even, the scale is cast to float.
"""
import numpy as np

UNSIGNED, SIGNED_SYMMETRIC, SIGNED_ASYMMETRIC = 0, 1, 2
f32 = np.float32


def fixup_range(rmin, rmax, symmetric=False):
    """QuantUtility.FixupRange (QuantUtility.cs:72-97)."""
    rmin, rmax = f32(rmin), f32(rmax)
    if symmetric:
        r = max(max(abs(rmin), abs(rmax)), f32(0.01))
        return f32(-r), f32(r)
    rmax = max(f32(0), rmax)
    rmin = min(f32(0), rmin)
    r = f32(rmax - rmin)
    if r == 0:
        r = f32(0.1)
    elif r < f32(0.01):
        r = f32(0.01)
    return rmin, f32(rmin + r)


def calib_fixup_range(rmin, rmax, symmetric=False):
    """Quantizer.FixUpRange used on calibrated activation ranges (Quantizer.cs:358-387)."""
    rmin, rmax = f32(rmin), f32(rmax)
    if symmetric:
        r = max(f32(0.01), max(abs(rmin), abs(rmax)))
        return f32(-r), f32(r)
    if rmax < 0:
        rmax = f32(0)
    if rmin > 0:
        rmin = f32(0)
    r = f32(rmax - rmin)
    if r < f32(1e-6):
        r = f32(0.1)
    return rmin, f32(rmin + r)


def _qrange(bits, mode):
    if mode == UNSIGNED:
        return 0.0, float((1 << bits) - 1)
    if mode == SIGNED_SYMMETRIC:
        return float(-(1 << (bits - 1)) + 1), float((1 << (bits - 1)) - 1)
    if mode == SIGNED_ASYMMETRIC:
        return float(-(1 << (bits - 1))), float((1 << (bits - 1)) - 1)
    raise ValueError("Invalid QuantMode")


def get_quant_param(rmin, rmax, bits=8, mode=UNSIGNED):
    """QuantUtility.GetQuantParam (QuantUtility.cs:41-67) -> (zero_point:int, scale:float32)."""
    rmin, rmax = fixup_range(rmin, rmax, mode == SIGNED_SYMMETRIC)
    qmin, qmax = _qrange(bits, mode)
    span = float(f32(rmax - rmin))  # float subtraction, then widened
    scale = span / (qmax - qmin)
    bias = np.round(float(rmin) * (qmin - qmax) / span) + qmin  # np.round: half to even
    return int(bias), f32(scale)


def get_min_max(t):
    """Quantizer.GetMinMax: min/max over finite values (Quantizer.Algorithms.cs:14-30)."""
    t = np.asarray(t, dtype=np.float32).ravel()
    t = t[np.isfinite(t)]
    if t.size == 0:
        return f32(np.finfo(np.float32).max), f32(np.finfo(np.float32).min)
    return f32(t.min()), f32(t.max())


def weights_ranges_by_channel(w, channels):
    """QuantUtility.GetWeightsRangesByChannel (QuantUtility.cs:106-151): [(min,max)] per
    output channel with the non-symmetric fix-up applied."""
    w = np.asarray(w, dtype=np.float32).reshape(channels, -1)
    out = []
    for ch in range(channels):
        out.append(fixup_range(w[ch].min(), w[ch].max(), False))
    return out


def weights_quant_params(w, channels, bits=8, mode=UNSIGNED):
    """Per-output-channel QuantParams as Quantizer.AssignQuantParameters derives them
    (Quantizer.cs:620-661): raw per-channel min/max -> GetQuantParam."""
    w = np.asarray(w, dtype=np.float32).reshape(channels, -1)
    zps = np.empty(channels, np.int32)
    scales = np.empty(channels, np.float32)
    for ch in range(channels):
        zps[ch], scales[ch] = get_quant_param(w[ch].min(), w[ch].max(), bits, mode)
    return zps, scales
