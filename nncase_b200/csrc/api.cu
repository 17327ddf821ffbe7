// extern "C" entry points declared in include/nncase_b200.h, the context object and the
// host-side QuantParam math.
#include "qconv.cuh"
#include <algorithm>
#include <cmath>
#include <vector>

namespace nncb {

std::string &last_error() {
    static thread_local std::string e;
    return e;
}

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error() = buf;
    return code;
}

int after_launch(nncb_context *ctx, const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(-EIO, "launch of %s failed: %s", what, cudaGetErrorString(e));
    ctx->launches++;
    return 0;
}

// ---- host float arithmetic: one IEEE rounding per operation, like the device intrinsics ----
// (host code of this library is compiled with floating-point contraction off)
static inline int32_t host_quant_impl(float x, float scale, float zp, int32_t lo, int32_t hi) {
    volatile float q = x / scale;
    volatile float v = q + zp;
    float r = nearbyintf(v);
    // saturating conversion like the device's cvt.rni.s32.f32
    int32_t i = r >= 2147483648.f ? INT32_MAX : (r <= -2147483648.f ? INT32_MIN : (std::isnan(r) ? 0 : (int32_t)r));
    return i < lo ? lo : (i > hi ? hi : i);
}

void make_requant_table(float si, int32_t zi, float so, int32_t zo, float lo, float hi, uint8_t table[256]) {
    for (int q = 0; q < 256; q++) {
        volatile float d = (float)q - (float)zi;
        volatile float f = d * si;
        float t = f < hi ? f : hi;
        float c = t > lo ? t : lo;
        table[q] = (uint8_t)host_quant_impl(c, so, (float)zo, 0, 255);
    }
}

// Unary activations of the reference are evaluated in double and cast back to float
// (UNARY_TEMPLATE, src/Native/src/kernels/stackvm/reference/kernel_template.h:19-50 with the formulas
// of reference/activation.cpp:32-38). On a u8 tensor the op is a function of 256 values:
//   table[q] = quantize((float)f((double)dequantize(q)), out)
int make_activation_table(int kind, float si, int32_t zi, float so, int32_t zo, uint8_t table[256]) {
    for (int q = 0; q < 256; q++) {
        volatile float d = (float)q - (float)zi;
        volatile float xf = d * si;
        const double x = (double)xf;
        double y;
        switch (kind) {
        case NNCB_ACT_RELU:
            y = std::max((double)0, x);
            break;
        case NNCB_ACT_SIGMOID:
            y = 1 / (1 + std::exp(-x));
            break;
        case NNCB_ACT_SWISH:
            y = x / (1 + std::exp(-x));
            break;
        case NNCB_ACT_HARD_SWISH:
            y = x * std::max((double)0.f, std::min((double)1.f, (double)(1.f / 6 * x + 0.5)));
            break;
        default:
            return fail(-EINVAL, "unknown activation kind %d", kind);
        }
        table[q] = (uint8_t)host_quant_impl((float)y, so, (float)zo, 0, 255);
    }
    return 0;
}

EpiParams make_epi(const nncb_qconv2d *cv) {
    const nncb_conv2d_desc &d = cv->d;
    EpiParams p;
    p.mult = cv->d_mult;
    p.bias = cv->d_bias;
    p.lut = cv->d_lut;
    p.y2_lut = cv->d_y2lut;
    p.out_scale = d.out_scale;
    p.out_zp = (float)d.out_zp;
    p.clamp_lo = d.clamp_lo;
    p.clamp_hi = d.clamp_hi;
    p.has_res = d.has_residual;
    p.res_scale = d.res_scale;
    p.res_zp = (float)d.res_zp;
    p.add_scale = d.add_out_scale;
    p.add_zp = (float)d.add_out_zp;
    return p;
}

int quantize(nncb_context *, const float *, void *, size_t, float, int32_t, int);
int dequantize(nncb_context *, const void *, float *, size_t, float, int32_t, int);
int quantize_nchw_to_nhwc_u8(nncb_context *, const float *, uint8_t *, int, int, int, int, int, float, int32_t);
int quantize_nchw_to_s2d_u8(nncb_context *, const float *, uint8_t *, int, int, int, int, int, float, int32_t, bool, int, int,
                            int, int);
int copy_channels_u8(nncb_context *, const uint8_t *, int, int, uint8_t *, int, int, int, size_t, const uint8_t *);
int resize_nearest_u8(nncb_context *, const uint8_t *, uint8_t *, int, int, int, int, int, int);
int dequantize_nhwc_to_nchw_f32(nncb_context *, const uint8_t *, float *, int, int, int, int, float, int32_t);
int nchw_to_nhwc_u8(nncb_context *, const uint8_t *, uint8_t *, int, int, int, int);
int nhwc_to_nchw_u8(nncb_context *, const uint8_t *, uint8_t *, int, int, int, int);
int qadd_u8(nncb_context *, const uint8_t *, const uint8_t *, uint8_t *, size_t, float, int32_t, float, int32_t, float, int32_t);
int lut_u8(nncb_context *, const uint8_t *, uint8_t *, size_t, const uint8_t *);
int maxpool_u8(nncb_context *, const uint8_t *, uint8_t *, int, int, int, int, int, int, int, int, int, int, int, int, int32_t);
int global_avgpool_u8(nncb_context *, const uint8_t *, uint8_t *, int, int, int, int, float, int32_t, float, int32_t);
int reduce_window2d_u8(nncb_context *, int, const uint8_t *, uint8_t *, int, int, int, int, int, int, int, int, int, int, int, int,
                       int, float, int32_t, float, int32_t);
int qbinary_u8(nncb_context *, int, const uint8_t *, const uint8_t *, uint8_t *, size_t, float, int32_t, float, int32_t, float,
               int32_t);
int softmax_f32(nncb_context *, const float *, float *, size_t, int, float);

size_t paged_attention_scratch_bytes(int B, int Hq, int splits);
int paged_attention_pick_splits(const nncb_context *ctx, int B, int Hkv, int max_ctx);
int paged_attention_check(int B, int Hq, int Hkv, int head_dim, int page_size, int max_pages);
int paged_attention_launch(nncb_context *ctx, const void *q, const void *k_pool, const void *v_pool,
                           const int32_t *block_table, const int32_t *ctx_lens, void *out, int B, int Hq, int Hkv,
                           int max_pages, int num_pages, float scale, int splits, void *scratch, const PaRope *rope = nullptr);

int gemv_w8a16(nncb_context *, const void *, const int8_t *, const void *, const void *, const void *, void *, int, int, int);
int gemv_w8a16_swiglu(nncb_context *, const void *, const int8_t *, const void *, const void *, void *, int, int, int);
int add_rmsnorm_f16(nncb_context *, void *, const void *, const void *, void *, int, int, float);
int rope_kv_append_f16(nncb_context *, const void *, void *, const float *, const float *, const int32_t *,
                       const int32_t *, void *, void *, int, int, int, int, int, int, int, int);
int swiglu_f16(nncb_context *, const void *, void *, int, int);
int peer_allreduce_add_rmsnorm_f16(nncb_context *, void *, const void *const *, void *const *, int, int, int, const void *, void *, int,
                                   int, float);
int embedding_f16(nncb_context *, const void *, const int32_t *, void *, int, int, int);
int int8_peak_selftest(nncb_context *ctx, uint32_t mmas_per_sm, int repeats, int w_signed, double *best_tops, double *mean_tops);
int mma_issue_selftest(nncb_context *ctx, int n_cols, int issuers, uint32_t mmas_per_issuer, double *cycles_per_mma);
size_t paged_attention_static_capacity();
int paged_attention_static_scratch(int device, void **ptr);

static size_t qtype_size(int qtype) { return qtype == NNCB_I16 ? 2 : 1; }

} // namespace nncb

using namespace nncb;

#define CHECK_CTX(ctx)                                                                          \
    do {                                                                                        \
        if (!(ctx))                                                                             \
            return fail(-EINVAL, "null context");                                               \
        cudaError_t e__ = cudaSetDevice((ctx)->device);                                         \
        if (e__ != cudaSuccess)                                                                 \
            return fail(-EIO, "cudaSetDevice(%d) failed: %s", (ctx)->device, cudaGetErrorString(e__)); \
    } while (0)

extern "C" {

const char *nncb_version(void) { return "nncase_b200 0.1 (sm_100a)"; }
const char *nncb_last_error(void) { return last_error().c_str(); }

int nncb_context_create(int device, void *stream, nncb_context **out) {
    if (!out)
        return fail(-EINVAL, "nncb_context_create: null out");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(-EIO, "no CUDA device available: %s", e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    if (device < 0 || device >= count)
        return fail(-EINVAL, "device %d out of range (0..%d)", device, count - 1);
    NNCB_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    NNCB_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(-ENOSYS, "device %d is sm_%d%d; this library contains sm_100a code only", device, prop.major, prop.minor);
    // kernels that need more than 48 KB of dynamic shared memory: the limit is a per-device attribute
    NNCB_TRY(paged_attention_set_attributes());
    NNCB_TRY(gemv_set_attributes());
    NNCB_TRY(nncb::gemm_w8a16_tc_set_attributes());
    nncb_context *ctx = new nncb_context();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->stream = (cudaStream_t)stream; // NULL is the CUDA default stream
    const size_t ws_bytes = (size_t)nncb::GEMV_SPLIT_SLOTS * (16 * 64 * sizeof(float) + sizeof(int));
    cudaError_t ce = cudaMalloc(&ctx->d_status, sizeof(int));
    if (ce == cudaSuccess)
        ce = cudaMemset(ctx->d_status, 0, sizeof(int));
    if (ce == cudaSuccess)
        ce = cudaMalloc(&ctx->d_gemv_ws, ws_bytes);
    if (ce == cudaSuccess)
        ce = cudaMemset(ctx->d_gemv_ws, 0, ws_bytes);
    if (ce != cudaSuccess) {
        cudaFree(ctx->d_status);
        cudaFree(ctx->d_gemv_ws);
        delete ctx;
        cudaGetLastError();
        return fail(ce == cudaErrorMemoryAllocation ? -ENOMEM : -EIO, "nncb_context_create: %s", cudaGetErrorString(ce));
    }
    *out = ctx;
    return 0;
}

// name -> field of nncb_options
static int *option_slot(nncb_context *ctx, const char *name) {
    struct { const char *name; int *slot; } table[] = {
        {"conv.tile_n", &ctx->opt.conv_tile_n},
        {"conv.mma_issuers", &ctx->opt.conv_mma_issuers},
        {"conv.load_warps", &ctx->opt.conv_load_warps},
        {"conv.wide_patch", &ctx->opt.conv_wide_patch},
        {"conv.add_table", &ctx->opt.conv_add_table},
        {"depthwise.dot_product", &ctx->opt.depthwise_dot},
        {"attention.warps", &ctx->opt.attention_warps},
        {"attention.splits", &ctx->opt.attention_splits},
        {"launch.overlap", &ctx->opt.launch_overlap},
        {"matmul.tensor_core", &ctx->opt.matmul_tensor_core},
        {"wait_limit_us", reinterpret_cast<int *>(&ctx->opt.wait_limit_us)},
        {"peer_wait_limit_us", reinterpret_cast<int *>(&ctx->opt.peer_wait_limit_us)},
        {"debug.withhold_load", &ctx->opt.debug_withhold_load},
    };
    for (auto &e : table)
        if (name && strcmp(name, e.name) == 0)
            return e.slot;
    return nullptr;
}

int nncb_context_set_option(nncb_context *ctx, const char *name, int64_t value) {
    if (!ctx)
        return fail(-EINVAL, "null context");
    int *slot = option_slot(ctx, name);
    if (!slot)
        return fail(-EINVAL, "unknown option '%s'", name ? name : "(null)");
    if (value < 0 || value > 0x7fffffff || (slot == reinterpret_cast<int *>(&ctx->opt.wait_limit_us) && value == 0))
        return fail(-EINVAL, "option '%s': value %lld out of range", name, (long long)value);
    *slot = (int)value;
    return 0;
}

int nncb_context_get_option(nncb_context *ctx, const char *name, int64_t *value) {
    if (!ctx || !value)
        return fail(-EINVAL, "null argument");
    int *slot = option_slot(ctx, name);
    if (!slot)
        return fail(-EINVAL, "unknown option '%s'", name ? name : "(null)");
    *value = *slot;
    return 0;
}

int nncb_context_destroy(nncb_context *ctx) {
    if (!ctx)
        return 0;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(ctx->d_status);
    cudaFree(ctx->d_gemv_ws);
    delete ctx;
    return 0;
}

int nncb_context_set_stream(nncb_context *ctx, void *stream) {
    CHECK_CTX(ctx);
    ctx->stream = (cudaStream_t)stream;
    return 0;
}

void *nncb_context_stream(nncb_context *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int nncb_synchronize(nncb_context *ctx) {
    CHECK_CTX(ctx);
    NNCB_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return 0;
}

uint64_t nncb_launch_count(nncb_context *ctx) { return ctx ? ctx->launches : 0; }

int nncb_check_device_status(nncb_context *ctx) {
    CHECK_CTX(ctx);
    int st = 0;
    NNCB_CUDA_TRY(cudaMemcpyAsync(&st, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    NNCB_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    if (st != 0) {
        NNCB_CUDA_TRY(cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream));
        if (st >= 200 && st < 300)
            return fail(-ERANGE, "a kernel refused an out-of-range index read from device memory (code %d)", st);
        return fail(-ETIMEDOUT, "a kernel gave up waiting (role code %d) and returned early", st);
    }
    return 0;
}

int nncb_malloc(nncb_context *ctx, size_t bytes, void **dptr) {
    CHECK_CTX(ctx);
    if (!dptr)
        return fail(-EINVAL, "nncb_malloc: null out");
    *dptr = nullptr;
    if (bytes == 0)
        return 0;
    cudaError_t e = cudaMalloc(dptr, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(-ENOMEM, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    }
    return 0;
}

int nncb_free(nncb_context *ctx, void *dptr) {
    CHECK_CTX(ctx);
    if (dptr)
        NNCB_CUDA_TRY(cudaFree(dptr));
    return 0;
}

int nncb_memcpy_h2d(nncb_context *ctx, void *dst, const void *src, size_t bytes) {
    CHECK_CTX(ctx);
    if (bytes)
        NNCB_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return 0;
}

int nncb_memcpy_d2h(nncb_context *ctx, void *dst, const void *src, size_t bytes) {
    CHECK_CTX(ctx);
    if (bytes) {
        NNCB_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        NNCB_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    }
    return 0;
}

int nncb_memset(nncb_context *ctx, void *dst, int value, size_t bytes) {
    CHECK_CTX(ctx);
    if (bytes)
        NNCB_CUDA_TRY(cudaMemsetAsync(dst, value, bytes, ctx->stream));
    return 0;
}

// ---- QuantParam math -----------------------------------------------------------------------
int nncb_fixup_range(float *rmin, float *rmax, int symmetric) {
    if (!rmin || !rmax)
        return fail(-EINVAL, "nncb_fixup_range: null pointer");
    if (symmetric) {
        float r = std::fmax(std::fmax(std::fabs(*rmin), std::fabs(*rmax)), 0.01f);
        *rmin = -r;
        *rmax = r;
        return 0;
    }
    float mx = std::fmax(0.f, *rmax), mn = std::fmin(0.f, *rmin);
    volatile float r = mx - mn;
    float rr = r;
    if (rr == 0)
        rr = 0.1f;
    else if (rr < 0.01f)
        rr = 0.01f;
    volatile float nm = mn + rr;
    *rmin = mn;
    *rmax = nm;
    return 0;
}

int nncb_get_quant_param(float rmin, float rmax, int bits, int mode, int32_t *zero_point, float *scale) {
    if (!zero_point || !scale || bits < 2 || bits > 16)
        return fail(-EINVAL, "nncb_get_quant_param: bad argument");
    nncb_fixup_range(&rmin, &rmax, mode == NNCB_SIGNED_SYMMETRIC);
    double qmin, qmax;
    switch (mode) {
    case NNCB_UNSIGNED:
        qmin = 0, qmax = (double)((1 << bits) - 1);
        break;
    case NNCB_SIGNED_SYMMETRIC:
        qmin = (double)(-(1 << (bits - 1)) + 1), qmax = (double)((1 << (bits - 1)) - 1);
        break;
    case NNCB_SIGNED_ASYMMETRIC:
        qmin = (double)(-(1 << (bits - 1))), qmax = (double)((1 << (bits - 1)) - 1);
        break;
    default:
        return fail(-EINVAL, "Invalid QuantMode");
    }
    volatile float spanf = rmax - rmin; // the reference subtracts in float, then divides in double
    double span = (double)spanf;
    double sc = span / (qmax - qmin);
    double bias = std::nearbyint((double)rmin * (qmin - qmax) / span) + qmin; // banker's rounding
    *zero_point = (int32_t)bias;
    *scale = (float)sc;
    return 0;
}

// ---- streaming ops -------------------------------------------------------------------------
int nncb_quantize(nncb_context *ctx, const float *in, void *out, size_t n, float scale, int32_t zp, int qtype) {
    CHECK_CTX(ctx);
    return quantize(ctx, in, out, n, scale, zp, qtype);
}
int nncb_dequantize(nncb_context *ctx, const void *in, float *out, size_t n, float scale, int32_t zp, int qtype) {
    CHECK_CTX(ctx);
    return dequantize(ctx, in, out, n, scale, zp, qtype);
}

int nncb_quantize_host(nncb_context *ctx, const float *in, void *out, size_t n, float scale, int32_t zp, int qtype) {
    CHECK_CTX(ctx);
    if (n == 0)
        return 0;
    if (qtype != NNCB_U8 && qtype != NNCB_I8 && qtype != NNCB_I16)
        return fail(-ENOSYS, "quantize: unsupported target type %d", qtype);
    void *din = nullptr, *dout = nullptr;
    NNCB_TRY(nncb_malloc(ctx, n * 4, &din));
    int rc = nncb_malloc(ctx, n * qtype_size(qtype), &dout);
    if (rc == 0)
        rc = nncb_memcpy_h2d(ctx, din, in, n * 4);
    if (rc == 0)
        rc = quantize(ctx, (const float *)din, dout, n, scale, zp, qtype);
    if (rc == 0)
        rc = nncb_memcpy_d2h(ctx, out, dout, n * qtype_size(qtype));
    cudaFree(din);
    cudaFree(dout);
    return rc;
}

int nncb_dequantize_host(nncb_context *ctx, const void *in, float *out, size_t n, float scale, int32_t zp, int qtype) {
    CHECK_CTX(ctx);
    if (n == 0)
        return 0;
    if (qtype != NNCB_U8 && qtype != NNCB_I8 && qtype != NNCB_I16)
        return fail(-ENOSYS, "dequantize: unsupported source type %d", qtype);
    void *din = nullptr, *dout = nullptr;
    NNCB_TRY(nncb_malloc(ctx, n * qtype_size(qtype), &din));
    int rc = nncb_malloc(ctx, n * 4, &dout);
    if (rc == 0)
        rc = nncb_memcpy_h2d(ctx, din, in, n * qtype_size(qtype));
    if (rc == 0)
        rc = dequantize(ctx, din, (float *)dout, n, scale, zp, qtype);
    if (rc == 0)
        rc = nncb_memcpy_d2h(ctx, out, dout, n * 4);
    cudaFree(din);
    cudaFree(dout);
    return rc;
}

int nncb_quantize_nchw_to_nhwc_u8(nncb_context *ctx, const float *in, uint8_t *out, int n, int c, int h, int w, int c_pad, float scale, int32_t zp) {
    CHECK_CTX(ctx);
    return quantize_nchw_to_nhwc_u8(ctx, in, out, n, c, h, w, c_pad, scale, zp);
}
int nncb_quantize_nchw_to_s2d_u8(nncb_context *ctx, const float *in, uint8_t *out, int n, int c, int h, int w, int c_pad, float scale, int32_t zp) {
    CHECK_CTX(ctx);
    return quantize_nchw_to_s2d_u8(ctx, in, out, n, c, h, w, c_pad, scale, zp, false, 0, 0, 0, 0);
}
int nncb_quantize_nhwc_to_s2d_u8(nncb_context *ctx, const float *in, uint8_t *out, int n, int h, int w, int c, int c_pad, float scale, int32_t zp) {
    CHECK_CTX(ctx);
    return quantize_nchw_to_s2d_u8(ctx, in, out, n, c, h, w, c_pad, scale, zp, true, 0, 0, 0, 0);
}
int nncb_quantize_to_s2d_padded_u8(nncb_context *ctx, const float *in, int in_nhwc, uint8_t *out, int n, int c, int h, int w,
                                   int c_pad, int pad_t, int pad_b, int pad_l, int pad_r, float scale, int32_t zp) {
    CHECK_CTX(ctx);
    return quantize_nchw_to_s2d_u8(ctx, in, out, n, c, h, w, c_pad, scale, zp, in_nhwc != 0, pad_t, pad_b, pad_l, pad_r);
}
int nncb_copy_channels_u8(nncb_context *ctx, const uint8_t *src, int src_c, int src_off, uint8_t *dst, int dst_c, int dst_off, int len, size_t pixels, const uint8_t *host_table) {
    CHECK_CTX(ctx);
    return copy_channels_u8(ctx, src, src_c, src_off, dst, dst_c, dst_off, len, pixels, host_table);
}
int nncb_resize_nearest_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int fy, int fx) {
    CHECK_CTX(ctx);
    return resize_nearest_u8(ctx, x, y, n, h, w, c, fy, fx);
}
int nncb_dequantize_nhwc_to_nchw_f32(nncb_context *ctx, const uint8_t *in, float *out, int n, int h, int w, int c, float scale, int32_t zp) {
    CHECK_CTX(ctx);
    return dequantize_nhwc_to_nchw_f32(ctx, in, out, n, h, w, c, scale, zp);
}
int nncb_nchw_to_nhwc_u8(nncb_context *ctx, const uint8_t *in, uint8_t *out, int n, int c, int h, int w) {
    CHECK_CTX(ctx);
    return nchw_to_nhwc_u8(ctx, in, out, n, c, h, w);
}
int nncb_nhwc_to_nchw_u8(nncb_context *ctx, const uint8_t *in, uint8_t *out, int n, int h, int w, int c) {
    CHECK_CTX(ctx);
    return nhwc_to_nchw_u8(ctx, in, out, n, h, w, c);
}
int nncb_qadd_u8(nncb_context *ctx, const uint8_t *a, const uint8_t *b, uint8_t *y, size_t n, float sa, int32_t za, float sb, int32_t zb, float so, int32_t zo) {
    CHECK_CTX(ctx);
    return qadd_u8(ctx, a, b, y, n, sa, za, sb, zb, so, zo);
}
int nncb_requant_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, size_t n, float si, int32_t zi, float so, int32_t zo, float lo, float hi) {
    CHECK_CTX(ctx);
    uint8_t table[256];
    make_requant_table(si, zi, so, zo, lo, hi, table);
    return lut_u8(ctx, x, y, n, table);
}
int nncb_make_activation_table(int kind, float si, int32_t zi, float so, int32_t zo, uint8_t *table) {
    if (!table)
        return fail(-EINVAL, "nncb_make_activation_table: null table");
    return make_activation_table(kind, si, zi, so, zo, table);
}
int nncb_make_requant_table(float si, int32_t zi, float so, int32_t zo, float lo, float hi, uint8_t *table) {
    if (!table)
        return fail(-EINVAL, "nncb_make_requant_table: null table");
    make_requant_table(si, zi, so, zo, lo, hi, table);
    return 0;
}
int nncb_activation_u8(nncb_context *ctx, int kind, const uint8_t *x, uint8_t *y, size_t n, float si, int32_t zi, float so, int32_t zo) {
    CHECK_CTX(ctx);
    uint8_t table[256];
    NNCB_TRY(make_activation_table(kind, si, zi, so, zo, table));
    return lut_u8(ctx, x, y, n, table);
}
int nncb_softmax_f32(nncb_context *ctx, const float *in, float *out, size_t rows, int cols, float beta) {
    CHECK_CTX(ctx);
    return softmax_f32(ctx, in, out, rows, cols, beta);
}
int nncb_lut_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, size_t n, const uint8_t *host_table) {
    CHECK_CTX(ctx);
    return lut_u8(ctx, x, y, n, host_table);
}
int nncb_maxpool_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int kh, int kw, int sh, int sw, int pt, int pb, int pl, int pr, int32_t zp) {
    CHECK_CTX(ctx);
    return maxpool_u8(ctx, x, y, n, h, w, c, kh, kw, sh, sw, pt, pb, pl, pr, zp);
}
int nncb_global_avgpool_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, float si, int32_t zi, float so, int32_t zo) {
    CHECK_CTX(ctx);
    return global_avgpool_u8(ctx, x, y, n, h, w, c, si, zi, so, zo);
}

int nncb_reduce_window2d_u8(nncb_context *ctx, int op, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int kh, int kw,
                            int stride_h, int stride_w, int pad_t, int pad_b, int pad_l, int pad_r, int count_include_pad,
                            float si, int32_t zi, float so, int32_t zo) {
    CHECK_CTX(ctx);
    if (!x || !y)
        return fail(-EINVAL, "nncb_reduce_window2d_u8: null pointer");
    return reduce_window2d_u8(ctx, op, x, y, n, h, w, c, kh, kw, stride_h, stride_w, pad_t, pad_b, pad_l, pad_r,
                              count_include_pad, si, zi, so, zo);
}
int nncb_qbinary_u8(nncb_context *ctx, int op, const uint8_t *a, const uint8_t *b, uint8_t *y, size_t n, float sa, int32_t za,
                    float sb, int32_t zb, float so, int32_t zo) {
    CHECK_CTX(ctx);
    return qbinary_u8(ctx, op, a, b, y, n, sa, za, sb, zb, so, zo);
}

// ---- decode-step operators -----------------------------------------------------------------
int nncb_gemv_w8a16(nncb_context *ctx, const void *x, const int8_t *w, const void *scale, const void *bias,
                    const void *residual, void *y, int m, int n, int k) {
    CHECK_CTX(ctx);
    if (!x || !w || !scale || !y)
        return fail(-EINVAL, "nncb_gemv_w8a16: null pointer");
    return gemv_w8a16(ctx, x, w, scale, bias, residual, y, m, n, k);
}
int nncb_gemv_w8a16_swiglu(nncb_context *ctx, const void *x, const int8_t *w, const void *scale, const void *bias, void *y,
                           int m, int n, int k) {
    CHECK_CTX(ctx);
    if (!x || !w || !scale || !y)
        return fail(-EINVAL, "nncb_gemv_w8a16_swiglu: null pointer");
    return gemv_w8a16_swiglu(ctx, x, w, scale, bias, y, m, n, k);
}
int nncb_add_rmsnorm_f16(nncb_context *ctx, void *x, const void *delta, const void *weight, void *h, int rows, int cols, float eps) {
    CHECK_CTX(ctx);
    if (!x || !weight || !h)
        return fail(-EINVAL, "nncb_add_rmsnorm_f16: null pointer");
    return add_rmsnorm_f16(ctx, x, delta, weight, h, rows, cols, eps);
}
int nncb_rope_kv_append_f16(nncb_context *ctx, const void *qkv, void *q_out, const float *cos_table, const float *sin_table,
                            const int32_t *positions, const int32_t *block_table, void *k_pool, void *v_pool, int batch,
                            int q_heads, int kv_heads, int head_dim, int page_size, int max_pages, int max_pos,
                            int num_pages) {
    CHECK_CTX(ctx);
    if (!qkv || !q_out || !cos_table || !sin_table || !positions || !block_table || !k_pool || !v_pool)
        return fail(-EINVAL, "nncb_rope_kv_append_f16: null pointer");
    return rope_kv_append_f16(ctx, qkv, q_out, cos_table, sin_table, positions, block_table, k_pool, v_pool, batch, q_heads,
                              kv_heads, head_dim, page_size, max_pages, max_pos, num_pages);
}
int nncb_swiglu_f16(nncb_context *ctx, const void *gate_up, void *out, int rows, int inter) {
    CHECK_CTX(ctx);
    if (!gate_up || !out)
        return fail(-EINVAL, "nncb_swiglu_f16: null pointer");
    return swiglu_f16(ctx, gate_up, out, rows, inter);
}
int nncb_embedding_f16(nncb_context *ctx, const void *table, const int32_t *ids, void *out, int rows, int cols, int vocab) {
    CHECK_CTX(ctx);
    if (!table || !ids || !out)
        return fail(-EINVAL, "nncb_embedding_f16: null pointer");
    return embedding_f16(ctx, table, ids, out, rows, cols, vocab);
}

// ---- paged attention -----------------------------------------------------------------------
int nncb_paged_attention_workspace_size(nncb_context *ctx, int batch, int q_heads, int kv_heads, int head_dim,
                                        int page_size, int max_pages, size_t *bytes) {
    CHECK_CTX(ctx);
    if (!bytes)
        return fail(-EINVAL, "nncb_paged_attention_workspace_size: null out");
    NNCB_TRY(paged_attention_check(batch, q_heads, kv_heads, head_dim, page_size, max_pages));
    const int splits = paged_attention_pick_splits(ctx, batch, kv_heads, max_pages * page_size);
    *bytes = paged_attention_scratch_bytes(batch, q_heads, splits);
    return 0;
}

int nncb_paged_attention_decode(nncb_context *ctx, const void *q, const void *k_pool, const void *v_pool,
                                const int32_t *block_table, const int32_t *context_lens, void *out, int batch,
                                int q_heads, int kv_heads, int head_dim, int page_size, int max_pages, int num_pages,
                                float scale, void *workspace, size_t workspace_bytes) {
    CHECK_CTX(ctx);
    if (!q || !k_pool || !v_pool || !block_table || !context_lens || !out)
        return fail(-EINVAL, "nncb_paged_attention_decode: null pointer");
    NNCB_TRY(paged_attention_check(batch, q_heads, kv_heads, head_dim, page_size, max_pages));
    if ((reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool) | reinterpret_cast<uintptr_t>(q) |
         reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(workspace)) & 15)
        return fail(-EINVAL, "nncb_paged_attention_decode: pointers must be 16-byte aligned");
    const int splits = paged_attention_pick_splits(ctx, batch, kv_heads, max_pages * page_size);
    const size_t need = paged_attention_scratch_bytes(batch, q_heads, splits);
    if (need > 0 && (!workspace || workspace_bytes < need))
        return fail(-EINVAL, "nncb_paged_attention_decode: workspace of %zu bytes required, %zu given", need,
                    workspace ? workspace_bytes : (size_t)0);
    return paged_attention_launch(ctx, q, k_pool, v_pool, block_table, context_lens, out, batch, q_heads, kv_heads,
                                  max_pages, num_pages, scale, splits, workspace);
}

int nncb_paged_attention_decode_rope(nncb_context *ctx, const void *qkv, const float *cos_table, const float *sin_table,
                                     const int32_t *positions, void *k_pool, void *v_pool, const int32_t *block_table,
                                     const int32_t *context_lens, void *out, int batch, int q_heads, int kv_heads,
                                     int head_dim, int page_size, int max_pages, int max_pos, int num_pages, float scale,
                                     void *workspace, size_t workspace_bytes) {
    CHECK_CTX(ctx);
    if (!qkv || !cos_table || !sin_table || !positions || !k_pool || !v_pool || !block_table || !context_lens || !out)
        return fail(-EINVAL, "nncb_paged_attention_decode_rope: null pointer");
    if (max_pos <= 0)
        return fail(-EINVAL, "nncb_paged_attention_decode_rope: max_pos must be positive");
    NNCB_TRY(paged_attention_check(batch, q_heads, kv_heads, head_dim, page_size, max_pages));
    if ((reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool) | reinterpret_cast<uintptr_t>(qkv) |
         reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(workspace) | reinterpret_cast<uintptr_t>(cos_table) |
         reinterpret_cast<uintptr_t>(sin_table)) & 15)
        return fail(-EINVAL, "nncb_paged_attention_decode_rope: pointers must be 16-byte aligned");
    const int splits = paged_attention_pick_splits(ctx, batch, kv_heads, max_pages * page_size);
    const size_t need = paged_attention_scratch_bytes(batch, q_heads, splits);
    if (need > 0 && (!workspace || workspace_bytes < need))
        return fail(-EINVAL, "nncb_paged_attention_decode_rope: workspace of %zu bytes required, %zu given", need,
                    workspace ? workspace_bytes : (size_t)0);
    PaRope rope = {qkv, cos_table, sin_table, positions, max_pos};
    return paged_attention_launch(ctx, nullptr, k_pool, v_pool, block_table, context_lens, out, batch, q_heads, kv_heads,
                                  max_pages, num_pages, scale, splits, workspace, &rope);
}

int nncb_paged_attention_decode_noalloc(nncb_context *ctx, const void *q, const void *k_pool, const void *v_pool,
                                        const int32_t *block_table, const int32_t *context_lens, void *out, int batch,
                                        int q_heads, int kv_heads, int head_dim, int page_size, int max_pages,
                                        int num_pages, float scale) {
    CHECK_CTX(ctx);
    if (!q || !k_pool || !v_pool || !block_table || !context_lens || !out)
        return fail(-EINVAL, "nncb_paged_attention_decode_noalloc: null pointer");
    NNCB_TRY(paged_attention_check(batch, q_heads, kv_heads, head_dim, page_size, max_pages));
    if ((reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool) | reinterpret_cast<uintptr_t>(q) |
         reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(-EINVAL, "nncb_paged_attention_decode_noalloc: pointers must be 16-byte aligned");
    const int splits = paged_attention_pick_splits(ctx, batch, kv_heads, max_pages * page_size);
    const size_t need = paged_attention_scratch_bytes(batch, q_heads, splits);
    if (need > paged_attention_static_capacity())
        return fail(-E2BIG,
                    "nncb_paged_attention_decode_noalloc: batch %d x %d heads x %d context splits needs %zu bytes of "
                    "scratch, the built-in array holds %zu; use nncb_paged_attention_decode with a workspace",
                    batch, q_heads, splits, need, paged_attention_static_capacity());
    void *scratch = nullptr;
    NNCB_TRY(paged_attention_static_scratch(ctx->device, &scratch));
    return paged_attention_launch(ctx, q, k_pool, v_pool, block_table, context_lens, out, batch, q_heads, kv_heads,
                                  max_pages, num_pages, scale, splits, scratch);
}

int nncb_ipc_export(nncb_context *ctx, const void *dptr, void *handle, size_t handle_bytes) {
    CHECK_CTX(ctx);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!dptr || !handle || handle_bytes < sizeof(cudaIpcMemHandle_t))
        return fail(-EINVAL, "nncb_ipc_export: needs a device pointer and 64 bytes for the handle");
    cudaIpcMemHandle_t hd;
    NNCB_CUDA_TRY(cudaIpcGetMemHandle(&hd, const_cast<void *>(dptr)));
    memcpy(handle, &hd, sizeof(hd));
    return 0;
}

int nncb_ipc_import(nncb_context *ctx, const void *handle, size_t handle_bytes, void **dptr) {
    CHECK_CTX(ctx);
    if (!handle || handle_bytes < sizeof(cudaIpcMemHandle_t) || !dptr)
        return fail(-EINVAL, "nncb_ipc_import: needs a 64-byte handle and an out pointer");
    cudaIpcMemHandle_t hd;
    memcpy(&hd, handle, sizeof(hd));
    NNCB_CUDA_TRY(cudaIpcOpenMemHandle(dptr, hd, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}

int nncb_ipc_close(nncb_context *ctx, void *dptr) {
    CHECK_CTX(ctx);
    if (!dptr)
        return 0;
    NNCB_CUDA_TRY(cudaIpcCloseMemHandle(dptr));
    return 0;
}

int nncb_peer_allreduce_add_rmsnorm_f16(nncb_context *ctx, void *x, const void *const *partials, void *const *flags, int world,
                                        int rank, int slot, const void *weight, void *h, int rows, int cols, float eps) {
    CHECK_CTX(ctx);
    if (!x || !partials || !flags || !weight || !h)
        return fail(-EINVAL, "nncb_peer_allreduce_add_rmsnorm_f16: null pointer");
    return peer_allreduce_add_rmsnorm_f16(ctx, x, partials, flags, world, rank, slot, weight, h, rows, cols, eps);
}

int nncb_selftest_int8_peak(nncb_context *ctx, uint32_t mmas_per_sm, int repeats, int w_signed, double *best_tops,
                            double *mean_tops) {
    CHECK_CTX(ctx);
    if (!best_tops || !mean_tops)
        return fail(-EINVAL, "nncb_selftest_int8_peak: null out");
    return int8_peak_selftest(ctx, mmas_per_sm, repeats, w_signed, best_tops, mean_tops);
}

int nncb_selftest_mma_issue(nncb_context *ctx, int n_cols, int issuers, uint32_t mmas_per_issuer, double *cycles_per_mma) {
    CHECK_CTX(ctx);
    if (!cycles_per_mma)
        return fail(-EINVAL, "nncb_selftest_mma_issue: null out");
    return mma_issue_selftest(ctx, n_cols, issuers, mmas_per_issuer, cycles_per_mma);
}

// ---- quantized conv ------------------------------------------------------------------------
int nncb_qconv2d_destroy(nncb_qconv2d *cv) {
    if (!cv)
        return 0;
    cudaSetDevice(cv->device);
    tc_conv_destroy(cv);
    cudaFree(cv->d_w);
    cudaFree(cv->d_wdw);
    cudaFree(cv->d_wdp);
    cudaFree(cv->d_cdp);
    cudaFree(cv->d_wzp);
    cudaFree(cv->d_mult);
    cudaFree(cv->d_bias);
    cudaFree(cv->d_lut);
    cudaFree(cv->d_y2lut);
    delete cv;
    return 0;
}

static int upload(nncb_context *ctx, void **dst, const void *src, size_t bytes) {
    NNCB_CUDA_TRY(cudaMalloc(dst, bytes));
    NNCB_CUDA_TRY(cudaMemcpyAsync(*dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return 0;
}

int nncb_qconv2d_create(nncb_context *ctx, const nncb_conv2d_desc *desc, const void *weights, const int32_t *w_zp,
                        const float *mult, const float *bias, const uint8_t *lut, nncb_qconv2d **out) {
    CHECK_CTX(ctx);
    if (!desc || !weights || !mult || !bias || !out)
        return fail(-EINVAL, "nncb_qconv2d_create: null argument");
    const nncb_conv2d_desc &d = *desc;
    if (d.n <= 0 || d.h <= 0 || d.w <= 0 || d.c <= 0 || d.oc <= 0 || d.kh <= 0 || d.kw <= 0 || d.stride_h <= 0 ||
        d.stride_w <= 0 || d.dil_h <= 0 || d.dil_w <= 0 || d.groups <= 0 || d.pad_t < 0 || d.pad_b < 0 || d.pad_l < 0 ||
        d.pad_r < 0)
        return fail(-EINVAL, "nncb_qconv2d_create: non-positive dimension");
    if (d.c % d.groups != 0 || d.oc % d.groups != 0)
        return fail(-EINVAL, "nncb_qconv2d_create: channels not divisible by groups");
    const int oh = conv_out_size(d.h, d.kh, d.stride_h, d.dil_h, d.pad_t, d.pad_b);
    const int ow = conv_out_size(d.w, d.kw, d.stride_w, d.dil_w, d.pad_l, d.pad_r);
    if (oh <= 0 || ow <= 0)
        return fail(-EINVAL, "nncb_qconv2d_create: empty output");
    if (!(d.out_scale > 0) && !d.f32_out)
        return fail(-EINVAL, "nncb_qconv2d_create: output scale must be positive");
    if (lut && (d.has_residual || d.f32_out))
        return fail(-ENOSYS, "nncb_qconv2d_create: activation table cannot be combined with residual add or f32 output");
    if (d.f32_out && (d.has_residual || d.has_y2))
        return fail(-ENOSYS, "nncb_qconv2d_create: f32 output cannot be combined with residual add or a second output");

    nncb_qconv2d *cv = new nncb_qconv2d();
    cv->d = d;
    cv->device = ctx->device;
    cv->oh = oh;
    cv->ow = ow;
    const size_t wbytes = (size_t)d.oc * d.kh * d.kw * (d.c / d.groups);
    std::vector<int32_t> wz(d.oc, 0);
    if (w_zp)
        memcpy(wz.data(), w_zp, sizeof(int32_t) * d.oc);
    int rc = upload(ctx, &cv->d_w, weights, wbytes);
    if (rc == 0)
        rc = upload(ctx, (void **)&cv->d_wzp, wz.data(), sizeof(int32_t) * d.oc);
    if (rc == 0)
        rc = upload(ctx, (void **)&cv->d_mult, mult, sizeof(float) * d.oc);
    if (rc == 0)
        rc = upload(ctx, (void **)&cv->d_bias, bias, sizeof(float) * d.oc);
    if (rc == 0 && lut)
        rc = upload(ctx, (void **)&cv->d_lut, lut, 256);
    uint8_t y2t[256];
    if (rc == 0 && d.has_y2) {
        const float fs = d.has_residual ? d.add_out_scale : d.out_scale;
        const int32_t fz = d.has_residual ? d.add_out_zp : d.out_zp;
        make_requant_table(fs, fz, d.y2_scale, d.y2_zp, d.y2_lo, d.y2_hi, y2t);
        rc = upload(ctx, (void **)&cv->d_y2lut, y2t, 256);
    }
    if (rc == 0) {
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess)
            rc = fail(-EIO, "upload failed: %s", cudaGetErrorString(e));
    }
    if (rc == 0) {
        std::string why;
        const bool tc_ok = tc_conv_supported(d, &why);
        if (d.force_path == PATH_TC && !tc_ok)
            rc = fail(-ENOSYS, "tcgen05 path not available for this convolution: %s", why.c_str());
        else if (d.force_path == PATH_SIMT || !tc_ok)
            cv->path = PATH_SIMT;
        else
            cv->path = PATH_TC;
    }
    if (rc == 0 && cv->path == PATH_TC)
        rc = tc_conv_create(ctx, cv, weights, w_zp);
    if (rc == 0 && cv->path == PATH_SIMT)
        rc = simt_conv_prepare(ctx, cv, weights, w_zp);
    if (rc != 0) {
        nncb_qconv2d_destroy(cv);
        return rc;
    }
    *out = cv;
    return 0;
}

int nncb_selftest_reciprocal_division(nncb_context *ctx, float scale, uint64_t count, uint64_t seed, uint64_t *mismatches) {
    CHECK_CTX(ctx);
    if (!mismatches)
        return fail(-EINVAL, "nncb_selftest_reciprocal_division: null out");
    unsigned long long m = 0;
    int rc = reciprocal_division_selftest(ctx, scale, count, seed, &m);
    *mismatches = m;
    return rc;
}

int nncb_qconv2d_path(const nncb_qconv2d *cv) { return cv ? cv->path : -EINVAL; }

int nncb_qconv2d_out_shape(const nncb_qconv2d *cv, int *oh, int *ow) {
    if (!cv || !oh || !ow)
        return fail(-EINVAL, "nncb_qconv2d_out_shape: null argument");
    *oh = cv->oh;
    *ow = cv->ow;
    return 0;
}

int nncb_qconv2d_run(nncb_context *ctx, nncb_qconv2d *cv, const uint8_t *x, const uint8_t *res, void *y, uint8_t *y2) {
    CHECK_CTX(ctx);
    if (!cv || !x || !y)
        return fail(-EINVAL, "nncb_qconv2d_run: null argument");
    if (cv->device != ctx->device)
        return fail(-EINVAL, "nncb_qconv2d_run: plan belongs to device %d, context to %d", cv->device, ctx->device);
    if (cv->d.has_residual && !res)
        return fail(-EINVAL, "nncb_qconv2d_run: residual input missing");
    if (cv->d.has_y2 && !y2)
        return fail(-EINVAL, "nncb_qconv2d_run: second output missing");
    if (!cv->d.has_residual)
        res = nullptr;
    if (!cv->d.has_y2)
        y2 = nullptr;
    if (cv->path == PATH_TC)
        return tc_conv_run(ctx, cv, x, res, y, y2);
    return simt_conv_run(ctx, cv, x, res, y, y2);
}

int nncb_qconv2d_host(nncb_context *ctx, const nncb_conv2d_desc *desc, const void *weights, const int32_t *w_zp,
                      const float *mult, const float *bias, const uint8_t *lut, const uint8_t *x, const uint8_t *res,
                      void *y, uint8_t *y2) {
    CHECK_CTX(ctx);
    nncb_qconv2d *cv = nullptr;
    NNCB_TRY(nncb_qconv2d_create(ctx, desc, weights, w_zp, mult, bias, lut, &cv));
    const size_t in_bytes = (size_t)desc->n * desc->h * desc->w * desc->c;
    const size_t out_elems = (size_t)desc->n * cv->oh * cv->ow * desc->oc;
    const size_t out_bytes = out_elems * (desc->f32_out ? 4 : 1);
    void *dx = nullptr, *dr = nullptr, *dy = nullptr, *dy2 = nullptr;
    int rc = nncb_malloc(ctx, in_bytes, &dx);
    if (rc == 0)
        rc = nncb_malloc(ctx, out_bytes, &dy);
    if (rc == 0 && desc->has_residual)
        rc = nncb_malloc(ctx, out_elems, &dr);
    if (rc == 0 && desc->has_y2)
        rc = nncb_malloc(ctx, out_elems, &dy2);
    if (rc == 0)
        rc = nncb_memcpy_h2d(ctx, dx, x, in_bytes);
    if (rc == 0 && desc->has_residual)
        rc = res ? nncb_memcpy_h2d(ctx, dr, res, out_elems) : fail(-EINVAL, "residual input missing");
    if (rc == 0)
        rc = nncb_qconv2d_run(ctx, cv, (const uint8_t *)dx, (const uint8_t *)dr, dy, (uint8_t *)dy2);
    if (rc == 0)
        rc = nncb_memcpy_d2h(ctx, y, dy, out_bytes);
    if (rc == 0 && desc->has_y2)
        rc = y2 ? nncb_memcpy_d2h(ctx, y2, dy2, out_elems) : fail(-EINVAL, "second output missing");
    if (rc == 0)
        rc = nncb_check_device_status(ctx);
    cudaFree(dx);
    cudaFree(dr);
    cudaFree(dy);
    cudaFree(dy2);
    nncb_qconv2d_destroy(cv);
    return rc;
}

} // extern "C"
