"""The `cuda` runtime plugin, loaded through the REFERENCE's own module loader.

oracle/_ref/libnncase_ref.so is the reference's native runtime compiled in simulator mode; the
harness asks its runtime_module::collect / create for the module kind "cuda", which dlopens
libnncase.simulator.cuda.so (the plugin built in nncase_b200/plugin) exactly as the interpreter
would for a kmodel that contains a cuda module. The custom calls are then invoked with host tensors
like the StackVM's CUSCALL opcode does, and checked against the C oracle.
"""
import ctypes as C
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libnncase_ref.so")
PLUGIN = os.path.join(ROOT, "tests", "plugin_harness", "libnncase.simulator.cuda.so")
PRODUCT_PLUGIN = os.path.join(ROOT, "nncase_b200", "plugin", "libnncase.simulator.cuda.so")
HARNESS = os.path.join(ROOT, "tests", "plugin_harness", "libplugin_harness.so")


@pytest.fixture(scope="module")
def harness():
    for p in (REF, PLUGIN, HARNESS):
        if not os.path.exists(p):
            pytest.skip(f"{os.path.relpath(p, ROOT)} not built (needs the reference checkout at build time)")
    # The plugin (the product's source linked against the stand-in runtime, as a maintainer links
    # it against Nncase.Runtime.Native) is loaded by path first; the reference's loader then finds
    # it by its soname when it dlopens "libnncase.simulator.cuda.so". Everything stays RTLD_LOCAL.
    C.CDLL(PLUGIN)
    return C.CDLL(HARNESS)


def test_product_plugin_exports_the_plugin_contract():
    if not os.path.exists(PRODUCT_PLUGIN):
        pytest.skip("plugin not built (needs the reference checkout at build time)")
    import subprocess
    syms = subprocess.check_output(["nm", "-D", "--defined-only", PRODUCT_PLUGIN], text=True)
    assert " T create_runtime_module" in syms and " T collect_custom_call" in syms


def test_reference_loader_finds_the_plugin_and_its_custom_calls(harness):
    buf = C.create_string_buffer(1024)
    n = harness.harness_list_custom_calls(buf, C.c_size_t(1024))
    assert n == 3
    assert buf.value.decode().split() == ["cuda.quantize", "cuda.dequantize", "cuda.qconv2d"]
    assert harness.harness_create_module() == 0


def test_custom_call_without_a_gpu_reports_an_error(harness):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    x = np.zeros(16, np.float32)
    out = np.zeros(16, np.uint8)
    rc = harness.harness_quantize(x.ctypes.data_as(C.c_void_p), C.c_size_t(16), C.c_float(0.1), 0, 6,
                                  out.ctypes.data_as(C.c_void_p), C.c_size_t(1))
    assert rc < 0  # -EIO from the CUDA library, carried through result<> as an error, no fallback


@pytest.mark.gpu
def test_quantize_dequantize_custom_calls(harness, qo):
    rng = np.random.default_rng(3)
    x = rng.normal(0, 1, 10007).astype(np.float32)
    out = np.zeros(x.size, np.uint8)
    assert harness.harness_quantize(x.ctypes.data_as(C.c_void_p), C.c_size_t(x.size), C.c_float(0.02), 117, 6,
                                    out.ctypes.data_as(C.c_void_p), C.c_size_t(1)) == 0
    assert np.array_equal(out, qo.quantize_u8(x, 0.02, 117))
    back = np.zeros(x.size, np.float32)
    assert harness.harness_dequantize(out.ctypes.data_as(C.c_void_p), C.c_size_t(x.size), C.c_float(0.02), 117,
                                      back.ctypes.data_as(C.c_void_p)) == 0
    assert np.array_equal(back, qo.dequantize_u8(out, 0.02, 117))


@pytest.mark.gpu
def test_qconv2d_custom_call(harness, qo):
    from nncase_b200.lib import Conv2dDesc
    rng = np.random.default_rng(4)
    n, h, w, c, oc = 2, 14, 14, 64, 64
    x = rng.integers(0, 256, (n, h, w, c), dtype=np.uint8)
    wq = rng.integers(0, 256, (oc, 3, 3, c), dtype=np.uint8)
    zw = rng.integers(110, 140, oc).astype(np.int32)
    mult = rng.uniform(2e-5, 6e-5, oc).astype(np.float32)
    bias = rng.normal(0, 0.2, oc).astype(np.float32)
    d = Conv2dDesc()
    d.stride_h = d.stride_w = d.dil_h = d.dil_w = d.groups = 1
    d.pad_t = d.pad_b = d.pad_l = d.pad_r = 1
    d.x_zp, d.out_scale, d.out_zp = 121, 0.05, 3
    d.clamp_lo, d.clamp_hi = 0.0, 6.0
    want = qo.qconv2d_u8(x, wq, zw, mult, bias, 121, 0.05, 3, pad=(1, 1, 1, 1), clamp=(0, 6))
    out = np.zeros(want.shape, np.uint8)
    xs = (C.c_size_t * 4)(*x.shape)
    ws = (C.c_size_t * 4)(*wq.shape)
    rc = harness.harness_qconv2d(C.byref(d), C.c_size_t(C.sizeof(d)), x.ctypes.data_as(C.c_void_p), xs,
                                 wq.ctypes.data_as(C.c_void_p), ws, 0, zw.ctypes.data_as(C.c_void_p),
                                 mult.ctypes.data_as(C.c_void_p), bias.ctypes.data_as(C.c_void_p), None,
                                 out.ctypes.data_as(C.c_void_p), C.c_size_t(out.size))
    assert rc == 0
    assert np.array_equal(out, want)


def test_qconv2d_custom_call_validates_its_tensors(harness):
    """Tensors reach a custom call from a kmodel: shapes that do not fit the descriptor are refused with
    invalid_argument before any byte is read through them (host-only checks, no GPU needed)."""
    from nncase_b200.lib import Conv2dDesc
    n, h, w, c, oc = 1, 6, 6, 32, 16
    x = np.zeros((n, h, w, c), np.uint8)
    zw = np.zeros(oc, np.int32)
    mult = np.ones(oc, np.float32)
    bias = np.zeros(oc, np.float32)

    def call(wshape, kdesc=None, res_bytes=None, out_elems=None):
        d = Conv2dDesc()
        d.stride_h = d.stride_w = d.dil_h = d.dil_w = d.groups = 1
        d.out_scale = 0.05
        for k, v in (kdesc or {}).items():
            setattr(d, k, v)
        wq = np.zeros(wshape, np.uint8)
        out_elems = out_elems or n * h * w * oc
        out = np.zeros(out_elems, np.uint8)
        res = np.zeros(res_bytes, np.uint8) if res_bytes else None
        return harness.harness_qconv2d(C.byref(d), C.c_size_t(C.sizeof(d)), x.ctypes.data_as(C.c_void_p),
                                       (C.c_size_t * 4)(*x.shape), wq.ctypes.data_as(C.c_void_p),
                                       (C.c_size_t * 4)(*wshape), 0, zw.ctypes.data_as(C.c_void_p),
                                       mult.ctypes.data_as(C.c_void_p), bias.ctypes.data_as(C.c_void_p),
                                       res.ctypes.data_as(C.c_void_p) if res is not None else None,
                                       out.ctypes.data_as(C.c_void_p), C.c_size_t(res_bytes or out_elems))

    EINVAL = -22
    assert call((oc, 1, 1, c + 1)) == EINVAL                     # weights' channel count is not c / groups
    assert call((oc, 9, 9, c)) == EINVAL                         # kernel larger than the (unpadded) input
    assert call((oc, 1, 1, c), dict(stride_h=0)) == EINVAL       # non-positive stride
    assert call((oc, 1, 1, c), dict(pad_t=-1)) == EINVAL         # negative padding
    assert call((oc, 1, 1, c), dict(groups=3)) == EINVAL         # channels not divisible by groups
    assert call((oc, 1, 1, c), res_bytes=17) == EINVAL           # residual that does not have the output's size
