"""ctypes binding of libnncase_b200.so (the C ABI in include/nncase_b200.h)."""
import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnncase_b200.so")
_LIB = None

# element types (nncb_dtype)
I8, I16, U8, F16, F32 = 2, 3, 6, 10, 11
# nncb_quant_mode
UNSIGNED, SIGNED_SYMMETRIC, SIGNED_ASYMMETRIC = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TC = 0, 1, 2
ACT_RELU, ACT_SIGMOID, ACT_SWISH, ACT_HARD_SWISH = 0, 1, 2, 3


class NncbError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"nncase_b200 error {code}: {msg}")
        self.code = code


class Conv2dDesc(C.Structure):
    """nncb_conv2d_desc"""
    _fields_ = [
        ("n", C.c_int32), ("h", C.c_int32), ("w", C.c_int32), ("c", C.c_int32),
        ("oc", C.c_int32), ("kh", C.c_int32), ("kw", C.c_int32),
        ("stride_h", C.c_int32), ("stride_w", C.c_int32),
        ("pad_t", C.c_int32), ("pad_b", C.c_int32), ("pad_l", C.c_int32), ("pad_r", C.c_int32),
        ("dil_h", C.c_int32), ("dil_w", C.c_int32),
        ("groups", C.c_int32), ("w_signed", C.c_int32), ("x_zp", C.c_int32),
        ("out_scale", C.c_float), ("out_zp", C.c_int32),
        ("clamp_lo", C.c_float), ("clamp_hi", C.c_float),
        ("has_residual", C.c_int32), ("res_scale", C.c_float), ("res_zp", C.c_int32),
        ("add_out_scale", C.c_float), ("add_out_zp", C.c_int32),
        ("has_y2", C.c_int32), ("y2_scale", C.c_float), ("y2_zp", C.c_int32),
        ("y2_lo", C.c_float), ("y2_hi", C.c_float),
        ("f32_out", C.c_int32), ("force_path", C.c_int32),
    ]


def build():
    """Compile the library in-tree for sm_100a (needs nvcc, no GPU)."""
    subprocess.check_call(["make", "-s", "-j8", "-C", os.path.join(_HERE, "csrc")])


_VP, _SZ, _I, _F = C.c_void_p, C.c_size_t, C.c_int, C.c_float
_I32 = C.c_int32
# name -> (restype, argtypes); every symbol declared in include/nncase_b200.h
SIGNATURES = {
    "nncb_context_create": (_I, [_I, _VP, C.POINTER(_VP)]),
    "nncb_context_destroy": (_I, [_VP]),
    "nncb_context_set_stream": (_I, [_VP, _VP]),
    "nncb_context_stream": (_VP, [_VP]),
    "nncb_synchronize": (_I, [_VP]),
    "nncb_launch_count": (C.c_uint64, [_VP]),
    "nncb_check_device_status": (_I, [_VP]),
    "nncb_last_error": (C.c_char_p, []),
    "nncb_version": (C.c_char_p, []),
    "nncb_malloc": (_I, [_VP, _SZ, C.POINTER(_VP)]),
    "nncb_free": (_I, [_VP, _VP]),
    "nncb_memcpy_h2d": (_I, [_VP, _VP, _VP, _SZ]),
    "nncb_memcpy_d2h": (_I, [_VP, _VP, _VP, _SZ]),
    "nncb_memset": (_I, [_VP, _VP, _I, _SZ]),
    "nncb_fixup_range": (_I, [C.POINTER(_F), C.POINTER(_F), _I]),
    "nncb_get_quant_param": (_I, [_F, _F, _I, _I, C.POINTER(_I32), C.POINTER(_F)]),
    "nncb_quantize": (_I, [_VP, _VP, _VP, _SZ, _F, _I32, _I]),
    "nncb_dequantize": (_I, [_VP, _VP, _VP, _SZ, _F, _I32, _I]),
    "nncb_quantize_host": (_I, [_VP, _VP, _VP, _SZ, _F, _I32, _I]),
    "nncb_dequantize_host": (_I, [_VP, _VP, _VP, _SZ, _F, _I32, _I]),
    "nncb_quantize_nchw_to_nhwc_u8": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _F, _I32]),
    "nncb_quantize_nchw_to_s2d_u8": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _F, _I32]),
    "nncb_dequantize_nhwc_to_nchw_f32": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _F, _I32]),
    "nncb_nchw_to_nhwc_u8": (_I, [_VP, _VP, _VP, _I, _I, _I, _I]),
    "nncb_nhwc_to_nchw_u8": (_I, [_VP, _VP, _VP, _I, _I, _I, _I]),
    "nncb_qadd_u8": (_I, [_VP, _VP, _VP, _VP, _SZ, _F, _I32, _F, _I32, _F, _I32]),
    "nncb_requant_u8": (_I, [_VP, _VP, _VP, _SZ, _F, _I32, _F, _I32, _F, _F]),
    "nncb_activation_u8": (_I, [_VP, _I, _VP, _VP, _SZ, _F, _I32, _F, _I32]),
    "nncb_make_activation_table": (_I, [_I, _F, _I32, _F, _I32, _VP]),
    "nncb_make_requant_table": (_I, [_F, _I32, _F, _I32, _F, _F, _VP]),
    "nncb_softmax_f32": (_I, [_VP, _VP, _VP, _SZ, _I, _F]),
    "nncb_quantize_nhwc_to_s2d_u8": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _F, _I32]),
    "nncb_quantize_to_s2d_padded_u8": (_I, [_VP, _VP, _I, _VP, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I32]),
    "nncb_copy_channels_u8": (_I, [_VP, _VP, _I, _I, _VP, _I, _I, _I, _SZ, _VP]),
    "nncb_resize_nearest_u8": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _I, _I]),
    "nncb_lut_u8": (_I, [_VP, _VP, _VP, _SZ, _VP]),
    "nncb_maxpool_u8": (_I, [_VP, _VP, _VP] + [_I] * 12 + [_I32]),
    "nncb_reduce_window2d_u8": (_I, [_VP, _I, _VP, _VP] + [_I] * 13 + [_F, _I32, _F, _I32]),
    "nncb_qbinary_u8": (_I, [_VP, _I, _VP, _VP, _VP, _SZ, _F, _I32, _F, _I32, _F, _I32]),
    "nncb_global_avgpool_u8": (_I, [_VP, _VP, _VP, _I, _I, _I, _I, _F, _I32, _F, _I32]),
    "nncb_qconv2d_create": (_I, [_VP, C.POINTER(Conv2dDesc), _VP, _VP, _VP, _VP, _VP, C.POINTER(_VP)]),
    "nncb_qconv2d_destroy": (_I, [_VP]),
    "nncb_qconv2d_path": (_I, [_VP]),
    "nncb_qconv2d_out_shape": (_I, [_VP, C.POINTER(_I), C.POINTER(_I)]),
    "nncb_qconv2d_run": (_I, [_VP, _VP, _VP, _VP, _VP, _VP]),
    "nncb_gemv_w8a16": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I]),
    "nncb_gemv_w8a16_swiglu": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I]),
    "nncb_add_rmsnorm_f16": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _I, _F]),
    "nncb_rope_kv_append_f16": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _I]),
    "nncb_swiglu_f16": (_I, [_VP, _VP, _VP, _I, _I]),
    "nncb_ipc_export": (_I, [_VP, _VP, _VP, _SZ]),
    "nncb_ipc_import": (_I, [_VP, _VP, _SZ, C.POINTER(_VP)]),
    "nncb_ipc_close": (_I, [_VP, _VP]),
    "nncb_peer_allreduce_add_rmsnorm_f16": (_I, [_VP, _VP, C.POINTER(_VP), C.POINTER(_VP), _I, _I, _I, _VP, _VP, _I, _I, _F]),
    "nncb_embedding_f16": (_I, [_VP, _VP, _VP, _VP, _I, _I, _I]),
    "nncb_paged_attention_workspace_size": (_I, [_VP, _I, _I, _I, _I, _I, _I, C.POINTER(_SZ)]),
    "nncb_paged_attention_decode": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _F, _VP, _SZ]),
    "nncb_paged_attention_decode_rope": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _I, _F, _VP,
                                              _SZ]),
    "nncb_paged_attention_decode_noalloc": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _I, _F]),
    "nncb_context_set_option": (_I, [_VP, C.c_char_p, C.c_int64]),
    "nncb_context_get_option": (_I, [_VP, C.c_char_p, C.POINTER(C.c_int64)]),
    "nncb_selftest_reciprocal_division": (_I, [_VP, _F, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64)]),
    "nncb_conv2d_f32": (_I, [_VP, _VP, _VP, _VP, _VP] + [_I] * 16 + [_F, _F]),
    "nncb_clamp_f32": (_I, [_VP, _VP, _VP, _SZ, _F, _F]),
    "nncb_swish_f32": (_I, [_VP, _VP, _VP, _SZ]),
    "nncb_add_f32": (_I, [_VP, _VP, _VP, _VP, _SZ]),
    "nncb_maxpool_f32": (_I, [_VP, _VP, _VP] + [_I] * 12),
    "nncb_global_mean_f32": (_I, [_VP, _VP, _VP, _SZ, _I]),
    "nncb_minmax_f32": (_I, [_VP, _VP, _SZ, C.POINTER(_F), C.POINTER(_F)]),
    "nncb_program_create": (_I, [_VP, _VP, _SZ, _VP, _SZ, C.POINTER(_VP)]),
    "nncb_program_destroy": (_I, [_VP]),
    "nncb_program_run": (_I, [_VP, _VP, _VP]),
    "nncb_program_run_host": (_I, [_VP, _VP, _VP, C.POINTER(_VP), _I32]),
    "nncb_program_info": (_I, [_VP, C.POINTER(_I32), C.POINTER(_I32), C.POINTER(_I32 * 3), C.POINTER(_I32), C.POINTER(_I32),
                               C.POINTER(_I32)]),
    "nncb_program_output": (_I, [_VP, _I32, C.POINTER(_I32)]),
    "nncb_program_tensor": (_I, [_VP, _I32, C.POINTER(_VP), C.POINTER(_I32 * 3), C.POINTER(_I32), C.POINTER(_F),
                                 C.POINTER(_I32), C.POINTER(_SZ)]),
    "nncb_program_set_profiling": (_I, [_VP, _I]),
    "nncb_program_launches_per_call": (C.c_uint64, [_VP]),
    "nncb_program_profile_text": (_I, [_VP, C.c_char_p, _SZ]),
    "nncb_program_profile_ms": (_I, [_VP, C.POINTER(_F), _I32]),
    "nncb_selftest_int8_peak": (_I, [_VP, C.c_uint32, _I, _I, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "nncb_selftest_mma_issue": (_I, [_VP, _I, _I, C.c_uint32, C.POINTER(C.c_double)]),
    "nncb_qconv2d_host": (_I, [_VP, C.POINTER(Conv2dDesc), _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP]),
}


def load():
    """Load the shared library; raises if it has not been built (no fallback exists)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise NncbError(-2, f"{LIB_PATH} is missing: build it with nncase_b200.lib.build() "
                                "(make -C nncase_b200/csrc); there is no CPU fallback")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = lib
    return _LIB


def check(rc):
    if rc < 0:
        raise NncbError(rc, load().nncb_last_error().decode())
    return rc
