// Float kernels for calibration: the forward pass the reference's Quantizer runs once per calibration
// sample to collect activation ranges (Quantizer.GetRangesAsync, src/Nncase.Quantization/Quantization/
// Quantizer.cs:389-409, evaluating every RangeOf node through CalibrationEvaluator.cs:34-71), and the range
// reduction itself (GetMinMax over finite values, Quantizer.Algorithms.cs:14-30).
//
// Semantics are those of the reference's float kernels: conv2d = bias + sum over in-image taps, then the fused
// clamp (reference/convolution.cpp:50-106); reduce_window2d max with padded taps contributing the value 0
// (reference/reduce_window.cpp:86-90); swish evaluated in double and cast (kernel_template.h:33-47). Layout NCHW
// f32, weights OIHW, like the reference's tensors. This is compile-time work, not the inference hot path: the
// kernels are plain shared-memory-tiled CUDA-core code.
#include "internal.cuh"
#include <cfloat>
#include <vector>

namespace nncb {

struct ConvF32 {
    int n, c, h, w, oc, kh, kw, sh, sw, pt, pl, dh, dw, groups, oh, ow;
    float lo, hi;
};

// Implicit GEMM per group: M = n*oh*ow pixels, N = oc/groups channels, K = (c/groups)*kh*kw.
// 64 x 64 outputs per block of 256 threads (4 x 4 per thread), K in slices of 16 through shared memory.
__global__ void __launch_bounds__(256)
conv2d_f32_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
                  float *__restrict__ y, const ConvF32 g) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float As[BK][BM + 4], Bs[BK][BN + 4];
    const int grp = blockIdx.z, cg = g.c / g.groups, ng = g.oc / g.groups;
    const int K = cg * g.kh * g.kw, taps = g.kh * g.kw;
    const long long M = (long long)g.n * g.oh * g.ow;
    const long long m0 = (long long)blockIdx.x * BM;
    const int n0 = blockIdx.y * BN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    // operand loads: every thread fetches 4 elements of A (fixed pixel, 4 k's) and 4 of B (fixed channel, 4 k's)
    const int lm = tid & 63, lk = tid >> 6; // lk in 0..3, elements k = lk + 4*i
    const long long am = m0 + lm;
    int a_img = 0, a_oy = 0, a_ox = 0;
    const bool a_ok = am < M;
    if (a_ok) {
        a_ox = (int)(am % g.ow);
        a_oy = (int)((am / g.ow) % g.oh);
        a_img = (int)(am / ((long long)g.ow * g.oh));
    }
    const int bn = n0 + lm;
    const bool b_ok = bn < ng;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int kk = lk + 4 * i, k = k0 + kk;
            float av = 0.f, bv = 0.f;
            if (k < K) {
                const int ci = k / taps, r = k - ci * taps, ky = r / g.kw, kx = r - ky * g.kw;
                if (a_ok) {
                    const int iy = a_oy * g.sh - g.pt + ky * g.dh, ix = a_ox * g.sw - g.pl + kx * g.dw;
                    if (iy >= 0 && iy < g.h && ix >= 0 && ix < g.w)
                        av = x[(((size_t)a_img * g.c + grp * cg + ci) * g.h + iy) * g.w + ix];
                }
                if (b_ok)
                    bv = w[((size_t)(grp * ng + bn)) * K + k];
            }
            As[kk][lm] = av;
            Bs[kk][lm] = bv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++)
                a[i] = As[kk][ty * 4 + i], b[i] = Bs[kk][tx * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const long long m = m0 + ty * 4 + i;
        if (m >= M)
            continue;
        const int ox = (int)(m % g.ow), oy = (int)((m / g.ow) % g.oh), img = (int)(m / ((long long)g.ow * g.oh));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int nn = n0 + tx * 4 + j;
            if (nn >= ng)
                continue;
            const int oc = grp * ng + nn;
            float v = acc[i][j] + (bias ? bias[oc] : 0.f);
            v = fminf(fmaxf(v, g.lo), g.hi);
            y[(((size_t)img * g.oc + oc) * g.oh + oy) * g.ow + ox] = v;
        }
    }
}

// depthwise (groups == c == oc): one thread per output
__global__ void __launch_bounds__(256)
dwconv2d_f32_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
                    float *__restrict__ y, const ConvF32 g) {
    const size_t total = (size_t)g.n * g.oc * g.oh * g.ow;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int ox = (int)(i % g.ow), oy = (int)((i / g.ow) % g.oh);
        const int ch = (int)((i / ((size_t)g.ow * g.oh)) % g.oc), img = (int)(i / ((size_t)g.ow * g.oh * g.oc));
        float acc = bias ? bias[ch] : 0.f;
        for (int ky = 0; ky < g.kh; ky++) {
            const int iy = oy * g.sh - g.pt + ky * g.dh;
            if (iy < 0 || iy >= g.h)
                continue;
            for (int kx = 0; kx < g.kw; kx++) {
                const int ix = ox * g.sw - g.pl + kx * g.dw;
                if (ix < 0 || ix >= g.w)
                    continue;
                acc = fmaf(x[(((size_t)img * g.c + ch) * g.h + iy) * g.w + ix], w[((size_t)ch * g.kh + ky) * g.kw + kx], acc);
            }
        }
        y[i] = fminf(fmaxf(acc, g.lo), g.hi);
    }
}

// kind: 0 clamp(lo, hi), 1 swish (x / (1 + exp(-x)) in double, cast), 2 add (x + other)
__global__ void __launch_bounds__(256)
elementwise_f32_kernel(int kind, const float *__restrict__ x, const float *__restrict__ other, float *__restrict__ y, size_t n,
                       float lo, float hi) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        float r;
        if (kind == 0)
            r = fminf(fmaxf(v, lo), hi);
        else if (kind == 1)
            r = (float)((double)v / (1.0 + exp(-(double)v)));
        else
            r = v + other[i];
        y[i] = r;
    }
}

// reduce_window2d max over NCHW f32; a tap outside the image contributes the value 0
__global__ void __launch_bounds__(256)
maxpool_f32_kernel(const float *__restrict__ x, float *__restrict__ y, int n, int c, int h, int w, int oh, int ow, int kh,
                   int kw, int sh, int sw, int pt, int pl) {
    const size_t total = (size_t)n * c * oh * ow;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int ox = (int)(i % ow), oy = (int)((i / ow) % oh);
        const size_t plane = i / ((size_t)ow * oh);
        float m = -FLT_MAX;
        int cnt = 0;
        for (int ky = 0; ky < kh; ky++) {
            const int iy = oy * sh - pt + ky;
            if (iy < 0 || iy >= h)
                continue;
            for (int kx = 0; kx < kw; kx++) {
                const int ix = ox * sw - pl + kx;
                if (ix < 0 || ix >= w)
                    continue;
                m = fmaxf(m, x[(plane * h + iy) * w + ix]);
                cnt++;
            }
        }
        if (cnt < kh * kw)
            m = fmaxf(m, 0.f);
        y[i] = m;
    }
}

// mean over H x W of every (image, channel) plane: one warp per plane
__global__ void __launch_bounds__(256)
global_mean_f32_kernel(const float *__restrict__ x, float *__restrict__ y, size_t planes, int hw) {
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= planes)
        return;
    float s = 0.f;
    for (int i = lane; i < hw; i += 32)
        s += x[warp * hw + i];
    for (int o = 16; o; o >>= 1)
        s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0)
        y[warp] = s / (float)hw;
}

// min and max over the finite values of x: per-block partials (out[2*block], out[2*block+1])
__global__ void __launch_bounds__(256)
minmax_f32_kernel(const float *__restrict__ x, size_t n, float *__restrict__ out) {
    float mn = FLT_MAX, mx = -FLT_MAX;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        if (isfinite(v))
            mn = fminf(mn, v), mx = fmaxf(mx, v);
    }
    for (int o = 16; o; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    __shared__ float smn[8], smx[8];
    if ((threadIdx.x & 31) == 0)
        smn[threadIdx.x >> 5] = mn, smx[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; i++)
            mn = fminf(mn, smn[i]), mx = fmaxf(mx, smx[i]);
        out[2 * blockIdx.x] = fminf(mn, smn[0]);
        out[2 * blockIdx.x + 1] = fmaxf(mx, smx[0]);
    }
}

static int grid_for(const nncb_context *ctx, size_t items) {
    size_t b = (items + 255) / 256, cap = (size_t)ctx->sm_count * 16;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

} // namespace nncb

using namespace nncb;

extern "C" {

int nncb_conv2d_f32(nncb_context *ctx, const float *x, const float *w, const float *bias, float *y, int n, int c, int h, int wd,
                    int oc, int kh, int kw, int stride_h, int stride_w, int pad_t, int pad_b, int pad_l, int pad_r, int dil_h,
                    int dil_w, int groups, float clamp_lo, float clamp_hi) {
    if (!ctx)
        return fail(-EINVAL, "null context");
    NNCB_CUDA_TRY(cudaSetDevice(ctx->device));
    if (!x || !w || !y)
        return fail(-EINVAL, "nncb_conv2d_f32: null pointer");
    if (n <= 0 || c <= 0 || h <= 0 || wd <= 0 || oc <= 0 || kh <= 0 || kw <= 0 || stride_h <= 0 || stride_w <= 0 || dil_h <= 0 ||
        dil_w <= 0 || groups <= 0 || pad_t < 0 || pad_b < 0 || pad_l < 0 || pad_r < 0 || c % groups || oc % groups)
        return fail(-EINVAL, "nncb_conv2d_f32: bad geometry");
    ConvF32 g{n, c, h, wd, oc, kh, kw, stride_h, stride_w, pad_t, pad_l, dil_h, dil_w, groups,
              conv_out_size(h, kh, stride_h, dil_h, pad_t, pad_b), conv_out_size(wd, kw, stride_w, dil_w, pad_l, pad_r), clamp_lo,
              clamp_hi};
    if (g.oh <= 0 || g.ow <= 0)
        return fail(-EINVAL, "nncb_conv2d_f32: empty output");
    if (groups == c && groups == oc && groups > 1) {
        dwconv2d_f32_kernel<<<grid_for(ctx, (size_t)n * oc * g.oh * g.ow), 256, 0, ctx->stream>>>(x, w, bias, y, g);
        return after_launch(ctx, "dwconv2d_f32");
    }
    const long long M = (long long)n * g.oh * g.ow;
    const dim3 grid((unsigned)((M + 63) / 64), (unsigned)((oc / groups + 63) / 64), (unsigned)groups);
    if (grid.y > 65535 || grid.z > 65535)
        return fail(-ENOSYS, "nncb_conv2d_f32: too many channel tiles or groups");
    conv2d_f32_kernel<<<grid, 256, 0, ctx->stream>>>(x, w, bias, y, g);
    return after_launch(ctx, "conv2d_f32");
}

static int elementwise(nncb_context *ctx, int kind, const float *x, const float *other, float *y, size_t n, float lo, float hi) {
    if (!ctx)
        return fail(-EINVAL, "null context");
    NNCB_CUDA_TRY(cudaSetDevice(ctx->device));
    if (n == 0)
        return 0;
    if (!x || !y || (kind == 2 && !other))
        return fail(-EINVAL, "float element-wise kernel: null pointer");
    elementwise_f32_kernel<<<grid_for(ctx, n), 256, 0, ctx->stream>>>(kind, x, other, y, n, lo, hi);
    return after_launch(ctx, "elementwise_f32");
}
int nncb_clamp_f32(nncb_context *ctx, const float *x, float *y, size_t n, float lo, float hi) { return elementwise(ctx, 0, x, nullptr, y, n, lo, hi); }
int nncb_swish_f32(nncb_context *ctx, const float *x, float *y, size_t n) { return elementwise(ctx, 1, x, nullptr, y, n, 0, 0); }
int nncb_add_f32(nncb_context *ctx, const float *a, const float *b, float *y, size_t n) { return elementwise(ctx, 2, a, b, y, n, 0, 0); }

int nncb_maxpool_f32(nncb_context *ctx, const float *x, float *y, int n, int c, int h, int w, int kh, int kw, int stride_h,
                     int stride_w, int pad_t, int pad_b, int pad_l, int pad_r) {
    if (!ctx)
        return fail(-EINVAL, "null context");
    NNCB_CUDA_TRY(cudaSetDevice(ctx->device));
    if (!x || !y || n <= 0 || c <= 0 || h <= 0 || w <= 0 || kh <= 0 || kw <= 0 || stride_h <= 0 || stride_w <= 0)
        return fail(-EINVAL, "nncb_maxpool_f32: bad argument");
    const int oh = conv_out_size(h, kh, stride_h, 1, pad_t, pad_b), ow = conv_out_size(w, kw, stride_w, 1, pad_l, pad_r);
    if (oh <= 0 || ow <= 0)
        return fail(-EINVAL, "nncb_maxpool_f32: empty output");
    maxpool_f32_kernel<<<grid_for(ctx, (size_t)n * c * oh * ow), 256, 0, ctx->stream>>>(x, y, n, c, h, w, oh, ow, kh, kw, stride_h,
                                                                                        stride_w, pad_t, pad_l);
    return after_launch(ctx, "maxpool_f32");
}

int nncb_global_mean_f32(nncb_context *ctx, const float *x, float *y, size_t planes, int hw) {
    if (!ctx)
        return fail(-EINVAL, "null context");
    NNCB_CUDA_TRY(cudaSetDevice(ctx->device));
    if (!x || !y || planes == 0 || hw <= 0)
        return fail(-EINVAL, "nncb_global_mean_f32: bad argument");
    global_mean_f32_kernel<<<(unsigned)((planes * 32 + 255) / 256), 256, 0, ctx->stream>>>(x, y, planes, hw);
    return after_launch(ctx, "global_mean_f32");
}

// min / max over the finite values (HOST results; synchronises). Empty or all non-finite input gives
// (FLT_MAX, -FLT_MAX) like the reference's GetMinMax.
int nncb_minmax_f32(nncb_context *ctx, const float *x, size_t n, float *min_out, float *max_out) {
    if (!ctx)
        return fail(-EINVAL, "null context");
    NNCB_CUDA_TRY(cudaSetDevice(ctx->device));
    if (!min_out || !max_out || (n && !x))
        return fail(-EINVAL, "nncb_minmax_f32: null pointer");
    *min_out = FLT_MAX, *max_out = -FLT_MAX;
    if (n == 0)
        return 0;
    const int grid = grid_for(ctx, n);
    float *d = nullptr;
    NNCB_CUDA_TRY(cudaMalloc(&d, sizeof(float) * 2 * grid));
    minmax_f32_kernel<<<grid, 256, 0, ctx->stream>>>(x, n, d);
    int rc = after_launch(ctx, "minmax_f32");
    std::vector<float> hst(2 * (size_t)grid);
    if (rc == 0) {
        cudaError_t e = cudaMemcpyAsync(hst.data(), d, sizeof(float) * hst.size(), cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess)
            e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess)
            rc = fail(-EIO, "nncb_minmax_f32: %s", cudaGetErrorString(e));
    }
    cudaFree(d);
    if (rc == 0)
        for (int i = 0; i < grid; i++) {
            *min_out = hst[2 * i] < *min_out ? hst[2 * i] : *min_out;
            *max_out = hst[2 * i + 1] > *max_out ? hst[2 * i + 1] : *max_out;
        }
    return rc;
}

} // extern "C"
