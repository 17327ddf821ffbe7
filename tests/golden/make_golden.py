"""Generates the golden fixtures in this directory from the reference's own CPU kernels.

Run where the reference checkout is available:  python tests/golden/make_golden.py
It needs oracle/_ref/libnncase_ref.so (``make -C oracle ref``). The fixtures let the oracle be
checked on machines that have neither the checkout nor the prebuilt library.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import qoracle as Q  # noqa: E402
from oracle import quant_params as QP  # noqa: E402
from oracle import ref as R  # noqa: E402


def main():
    rng = np.random.default_rng(20240)
    scale, zp = 0.014035294, 88
    x = rng.normal(0, 1.2, 4096).astype(np.float32)
    k = np.arange(-40, 300, dtype=np.float32)
    ties = (k + np.float32(0.5) - np.float32(zp)) * np.float32(scale)
    x = np.concatenate([x, ties]).astype(np.float32)
    q = R.quantize_u8(x, scale, zp)
    np.savez_compressed(os.path.join(HERE, "quantize_dequantize.npz"), x=x, scale=np.float32(scale), zp=np.int32(zp),
                        q_u8=q, deq_f32=R.dequantize_u8(q, scale, zp))

    # a slice of config 1 (3x3, stride 1, pad 1, ReLU6, 64 -> 64 channels) on a 12x12 image
    x = rng.uniform(-1, 1, (1, 12, 12, 64)).astype(np.float32)
    w = rng.normal(0, 0.05, (64, 3, 3, 64)).astype(np.float32)
    b = rng.normal(0, 0.01, 64).astype(np.float32)
    zx, sx = QP.get_quant_param(*QP.get_min_max(x))
    zw, sw = QP.weights_quant_params(w, 64)
    xq = R.quantize_u8(x, sx, zx)
    wq = np.stack([R.quantize_u8(w[i], sw[i], zw[i]) for i in range(64)])
    yf = R.conv2d_f32(x.transpose(0, 3, 1, 2), w.transpose(0, 3, 1, 2), b, pad=(1, 1, 1, 1), clamp=(0, 6))
    zo, so = QP.get_quant_param(*QP.get_min_max(yf))
    mult = (np.float32(sx) * sw).astype(np.float32)
    y_ref = R.qconv2d_composite_u8(xq, wq, zw, sw, b, sx, zx, so, zo, pad=(1, 1, 1, 1), clamp=(0, 6))
    y_int = Q.qconv2d_u8(xq, wq, zw, mult, b, zx, so, zo, pad=(1, 1, 1, 1), clamp=(0, 6))
    mism = int((y_ref != y_int).sum())
    np.savez_compressed(os.path.join(HERE, "conv_config1_slice.npz"), xq=xq, wq=wq, zw=zw, mult=mult, bias=b,
                        zx=np.int32(zx), so=np.float32(so), zo=np.int32(zo), y_ref_composite=y_ref, y_integer=y_int,
                        allowed_mismatches=np.int32(mism))
    print("conv slice: integer vs reference composite mismatches:", mism, "of", y_int.size)


if __name__ == "__main__":
    main()
