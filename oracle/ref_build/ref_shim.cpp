// C entry points over the nncase reference CPU kernels, for use as a parity checker
// and as the timed CPU baseline.
//
// TEST INFRASTRUCTURE ONLY: nothing in the shipped library links or loads this.
// It is compiled together with the reference's own translation units, taken from
// the reference checkout where they lie (see oracle/Makefile), into
// oracle/_ref/libnncase_ref.so. Each wrapper only adapts flat C arguments to the
// reference's C++ signatures declared in
//   src/Native/src/kernels/stackvm/reference/ref_ops.h
//   src/Native/src/kernels/stackvm/optimized/opt_ops.h
#include <cstdint>
#include <cstring>
#include <nncase/kernels/kernel_context.h>
#include "opt_ops.h"
#include "ref_ops.h"
#include <nncase/runtime/datatypes.h>
#include <nncase/kernels/stackvm/tensor_ops.h>
#include <nncase/runtime/runtime_tensor.h>
#include <nncase/runtime/util.h>

using namespace nncase;
using nncase::kernels::default_kernel_context;
using nncase::kernels::kernel_context;
using nncase::runtime::stackvm::binary_op_t;
using nncase::runtime::stackvm::reduce_op_t;
namespace kref = nncase::kernels::stackvm::reference;
namespace kopt = nncase::kernels::stackvm::optimized;
namespace kdetail = nncase::kernels::detail;

// Defined (non-static, global scope) in reference/reduce_window.cpp:124-144.
result<void> reduce_window2d_impl(
    reduce_op_t op, const float *input, float init_value, float *output,
    gsl::span<const size_t> in_shape, gsl::span<const size_t> in_strides,
    gsl::span<const size_t> out_strides, const padding &padding_h,
    const padding &padding_w, int32_t filter_h, int32_t filter_w,
    int32_t stride_h, int32_t stride_w, int32_t dilation_h, int32_t dilation_w,
    value_range<float> fused_activation, bool count_include_pad,
    kernel_context &context) noexcept;

namespace {
dims_t contiguous_strides(const dims_t &shape) {
    dims_t s(shape.size());
    size_t acc = 1;
    for (size_t i = shape.size(); i-- > 0;) {
        s[i] = acc;
        acc *= shape[i];
    }
    return s;
}
int rc(const result<void> &r) { return r.is_ok() ? 0 : -1; }
} // namespace

extern "C" {

// optimized::quantize f32 -> u8 (the path kernels::stackvm::quantize takes for
// contiguous tensors, tensor_ops.cpp:681-695; optimized/quantize.cpp:59-92).
int nncase_ref_quantize_u8(const float *in, uint8_t *out, size_t n, float scale,
                           int32_t zero_point, int use_optimized) {
    dims_t shape{n}, strides{1};
    auto &ctx = default_kernel_context();
    if (use_optimized)
        return rc(kopt::quantize(dt_float32, dt_uint8, (const gsl::byte *)in,
                                      (gsl::byte *)out, shape, strides, strides, scale,
                                      (float)zero_point, ctx));
    return rc(kref::quantize(dt_float32, dt_uint8, (const gsl::byte *)in,
                                  (gsl::byte *)out, shape, strides, strides, scale,
                                  (float)zero_point, ctx));
}

int nncase_ref_quantize_i8(const float *in, int8_t *out, size_t n, float scale,
                           int32_t zero_point, int use_optimized) {
    dims_t shape{n}, strides{1};
    auto &ctx = default_kernel_context();
    if (use_optimized)
        return rc(kopt::quantize(dt_float32, dt_int8, (const gsl::byte *)in,
                                      (gsl::byte *)out, shape, strides, strides, scale,
                                      (float)zero_point, ctx));
    return rc(kref::quantize(dt_float32, dt_int8, (const gsl::byte *)in,
                                  (gsl::byte *)out, shape, strides, strides, scale,
                                  (float)zero_point, ctx));
}

int nncase_ref_dequantize_u8(const uint8_t *in, float *out, size_t n, float scale,
                             int32_t zero_point, int use_optimized) {
    dims_t shape{n}, strides{1};
    auto &ctx = default_kernel_context();
    if (use_optimized)
        return rc(kopt::dequantize(dt_uint8, dt_float32, (const gsl::byte *)in,
                                        (gsl::byte *)out, shape, strides, strides, scale,
                                        (float)zero_point, ctx));
    return rc(kref::dequantize(dt_uint8, dt_float32, (const gsl::byte *)in,
                                    (gsl::byte *)out, shape, strides, strides, scale,
                                    (float)zero_point, ctx));
}

int nncase_ref_dequantize_i8(const int8_t *in, float *out, size_t n, float scale,
                             int32_t zero_point, int use_optimized) {
    dims_t shape{n}, strides{1};
    auto &ctx = default_kernel_context();
    if (use_optimized)
        return rc(kopt::dequantize(dt_int8, dt_float32, (const gsl::byte *)in,
                                        (gsl::byte *)out, shape, strides, strides, scale,
                                        (float)zero_point, ctx));
    return rc(kref::dequantize(dt_int8, dt_float32, (const gsl::byte *)in,
                                    (gsl::byte *)out, shape, strides, strides, scale,
                                    (float)zero_point, ctx));
}

// reference::conv2d, f32 NCHW / OIHW (reference/convolution.cpp:118-143).
int nncase_ref_conv2d_f32(const float *in, const float *w, const float *bias, float *out,
                          size_t n, size_t c, size_t h, size_t wd, size_t oc, size_t kh,
                          size_t kw, int groups, int stride_h, int stride_w, int pad_t,
                          int pad_b, int pad_l, int pad_r, int dil_h, int dil_w,
                          float clamp_lo, float clamp_hi) {
    dims_t in_shape{n, c, h, wd};
    dims_t w_shape{oc, c / (size_t)groups, kh, kw};
    padding ph{pad_t, pad_b}, pw{pad_l, pad_r};
    size_t oh = kdetail::get_windowed_output_size(h, (int32_t)kh, stride_h, dil_h, ph);
    size_t ow = kdetail::get_windowed_output_size(wd, (int32_t)kw, stride_w, dil_w, pw);
    dims_t out_shape{n, oc, oh, ow};
    dims_t bias_strides{1};
    return rc(kref::conv2d(dt_float32, (const gsl::byte *)in, (const gsl::byte *)w,
                                (const gsl::byte *)bias, (gsl::byte *)out, in_shape,
                                contiguous_strides(in_shape), w_shape,
                                contiguous_strides(w_shape), bias_strides,
                                contiguous_strides(out_shape), ph, pw, groups, stride_h,
                                stride_w, dil_h, dil_w, {clamp_lo, clamp_hi}));
}

// reference::matmul, f32, A[b0,b1,M,K] x B[b0',b1',K,N] (reference/matmul.cpp:92-110).
int nncase_ref_matmul_f32(const float *a, const float *b, float *out, const size_t *a_shape,
                          size_t a_rank, const size_t *b_shape, size_t b_rank) {
    dims_t as(a_shape, a_shape + a_rank), bs(b_shape, b_shape + b_rank);
    return rc(kref::matmul(dt_float32, (const gsl::byte *)a, (const gsl::byte *)b,
                                (gsl::byte *)out, as, bs));
}

// reference::softmax on the given axis, f32 (reference/softmax.cpp:30-128).
int nncase_ref_softmax_f32(const float *in, float *out, const size_t *shape, size_t rank,
                           int64_t axis, float beta) {
    dims_t s(shape, shape + rank);
    auto st = contiguous_strides(s);
    return rc(kref::softmax(dt_float32, (const gsl::byte *)in, (gsl::byte *)out, s, st,
                                 st, axis, beta, false));
}

// reference::binary add/mul on equal-shaped f32 tensors (reference/binary.cpp:28-123).
int nncase_ref_binary_f32(int op, const float *a, const float *b, float *out, size_t n) {
    dims_t s{n}, st{1};
    return rc(kref::binary(dt_float32, (binary_op_t)op, (const gsl::byte *)a,
                                (const gsl::byte *)b, (gsl::byte *)out, s, st, s, st, s, st));
}

// reduce_window2d f32 NCHW; op: 0 mean, 1 min, 2 max, 3 sum (reduce_op_t order).
int nncase_ref_reduce_window2d_f32(int op, const float *in, float init_value, float *out,
                                   size_t n, size_t c, size_t h, size_t w, int fh, int fw,
                                   int stride_h, int stride_w, int pad_t, int pad_b, int pad_l,
                                   int pad_r, int count_include_pad) {
    dims_t in_shape{n, c, h, w};
    padding ph{pad_t, pad_b}, pw{pad_l, pad_r};
    size_t oh = kdetail::get_windowed_output_size(h, fh, stride_h, 1, ph);
    size_t ow = kdetail::get_windowed_output_size(w, fw, stride_w, 1, pw);
    dims_t out_shape{n, c, oh, ow};
    return rc(reduce_window2d_impl((reduce_op_t)op, in, init_value, out, in_shape,
                                   contiguous_strides(in_shape), contiguous_strides(out_shape),
                                   ph, pw, fh, fw, stride_h, stride_w, 1, 1,
                                   value_range<float>::full(), count_include_pad != 0,
                                   default_kernel_context()));
}

// kernels::stackvm::{relu, sigmoid, swish, hard_swish}(value_t) on a flat f32 tensor
// (reference/activation.cpp:32-38 through the value_t dispatch of kernel_template.h:52-65).
// kind: 0 relu, 1 sigmoid, 2 swish, 3 hard_swish.
int nncase_ref_unary_f32(int kind, const float *in, float *out, size_t n) {
    using namespace nncase::runtime;
    auto run = [&]() -> result<void> {
        try_var(t, hrt::create(dt_float32, dims_t{n}, {(gsl::byte *)in, n * 4}, true, hrt::pool_cpu_only));
        value_t x = t.impl(), y;
        switch (kind) {
        case 0: { try_set(y, nncase::kernels::stackvm::relu(x)); break; }
        case 1: { try_set(y, nncase::kernels::stackvm::sigmoid(x)); break; }
        case 2: { try_set(y, nncase::kernels::stackvm::swish(x)); break; }
        case 3: { try_set(y, nncase::kernels::stackvm::hard_swish(x)); break; }
        default: return err(std::errc::invalid_argument);
        }
        try_var(yt, y.as<tensor>());
        try_var(src, get_input_data(yt));
        std::memcpy(out, src, n * 4);
        return ok();
    };
    return rc(run());
}

int nncase_ref_binary_op_add(void) { return (int)binary_op_t::add; }
int nncase_ref_binary_op_mul(void) { return (int)binary_op_t::mul; }
int nncase_ref_reduce_op_max(void) { return (int)reduce_op_t::max; }
int nncase_ref_reduce_op_mean(void) { return (int)reduce_op_t::mean; }

} // extern "C"
