// HBM-streaming kernels: Quantize / Dequantize, layout changes, element-wise add, table
// look-up, pooling. All are bandwidth-bound: 128-bit loads and stores, grid sized as a
// multiple of the SM count with a grid-stride loop.
#include "internal.cuh"
#include "qconv.cuh"
#include <type_traits>

namespace nncb {

static inline int stream_grid(const nncb_context *ctx, size_t work_items, int threads) {
    size_t blocks = (work_items + threads - 1) / threads;
    size_t cap = (size_t)ctx->sm_count * 16;
    if (blocks > cap)
        blocks = cap;
    if (blocks < 1)
        blocks = 1;
    return (int)blocks;
}

// ---- quantize -----------------------------------------------------------------------------
template <typename Q> struct qlimits;
template <> struct qlimits<uint8_t> { static constexpr int lo = 0, hi = 255; };
template <> struct qlimits<int8_t> { static constexpr int lo = -128, hi = 127; };
template <> struct qlimits<int16_t> { static constexpr int lo = -32768, hi = 32767; };

// 16 elements per thread per iteration: four float4 loads, one 16-byte (8-bit types) or two
// 16-byte (16-bit type) stores. `vec_ok` is false when a pointer is not 16-byte aligned.
template <typename Q>
__global__ void __launch_bounds__(256) quantize_kernel(const float *__restrict__ in, Q *__restrict__ out,
                                                       size_t n, float scale, float zp, bool vec_ok) {
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    const size_t nvec = vec_ok ? n / 16 : 0;
    for (size_t v = tid; v < nvec; v += nthreads) {
        const float4 *p = reinterpret_cast<const float4 *>(in) + v * 4;
        float4 f[4];
#pragma unroll
        for (int i = 0; i < 4; i++)
            f[i] = __ldcs(p + i);
        alignas(16) Q q[16];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            q[i * 4 + 0] = (Q)quant_dev(f[i].x, scale, zp, qlimits<Q>::lo, qlimits<Q>::hi);
            q[i * 4 + 1] = (Q)quant_dev(f[i].y, scale, zp, qlimits<Q>::lo, qlimits<Q>::hi);
            q[i * 4 + 2] = (Q)quant_dev(f[i].z, scale, zp, qlimits<Q>::lo, qlimits<Q>::hi);
            q[i * 4 + 3] = (Q)quant_dev(f[i].w, scale, zp, qlimits<Q>::lo, qlimits<Q>::hi);
        }
        uint4 *o = reinterpret_cast<uint4 *>(out + v * 16);
        const uint4 *qs = reinterpret_cast<const uint4 *>(q);
#pragma unroll
        for (int i = 0; i < (int)(sizeof(Q) * 16 / 16); i++)
            __stcs(o + i, qs[i]);
    }
    for (size_t i = nvec * 16 + tid; i < n; i += nthreads)
        out[i] = (Q)quant_dev(in[i], scale, zp, qlimits<Q>::lo, qlimits<Q>::hi);
}

// Four elements per thread per step: consecutive lanes read consecutive 4-byte (8-byte for int16) words and write
// consecutive float4 -- a warp's store instruction covers 512 contiguous bytes -- with four independent
// steps in flight per thread (the stream is 80 % writes; the loads of the next steps overlap them).
template <typename Q>
__global__ void __launch_bounds__(256) dequantize_kernel(const Q *__restrict__ in, float *__restrict__ out,
                                                         size_t n, float scale, float zp, bool vec_ok) {
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    const size_t nvec = vec_ok ? n / 4 : 0; // groups of four elements
    constexpr int UN = 4;
    using W = typename std::conditional<sizeof(Q) == 1, uint32_t, uint2>::type;
    auto deq4 = [&](const W &w) {
        alignas(8) Q q[4];
        *reinterpret_cast<W *>(q) = w;
        float4 f;
        f.x = dequant_dev((float)q[0], zp, scale);
        f.y = dequant_dev((float)q[1], zp, scale);
        f.z = dequant_dev((float)q[2], zp, scale);
        f.w = dequant_dev((float)q[3], zp, scale);
        return f;
    };
    size_t v = tid;
    for (; v + (UN - 1) * nthreads < nvec; v += UN * nthreads) {
        W w[UN];
#pragma unroll
        for (int u = 0; u < UN; u++)
            w[u] = __ldcs(reinterpret_cast<const W *>(in) + v + u * nthreads);
#pragma unroll
        for (int u = 0; u < UN; u++)
            __stcs(reinterpret_cast<float4 *>(out) + v + u * nthreads, deq4(w[u]));
    }
    for (; v < nvec; v += nthreads)
        __stcs(reinterpret_cast<float4 *>(out) + v, deq4(__ldcs(reinterpret_cast<const W *>(in) + v)));
    for (size_t i = nvec * 4 + tid; i < n; i += nthreads)
        out[i] = dequant_dev((float)in[i], zp, scale);
}

static inline bool aligned16(const void *a, const void *b) {
    return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
}

int quantize(nncb_context *ctx, const float *in, void *out, size_t n, float scale, int32_t zp, int qtype) {
    if (n == 0)
        return 0;
    if (!in || !out)
        return fail(-EINVAL, "quantize: null pointer");
    const int threads = 256;
    const int grid = stream_grid(ctx, (n + 15) / 16, threads);
    const bool v = aligned16(in, out);
    switch (qtype) {
    case NNCB_U8:
        quantize_kernel<uint8_t><<<grid, threads, 0, ctx->stream>>>(in, (uint8_t *)out, n, scale, (float)zp, v);
        break;
    case NNCB_I8:
        quantize_kernel<int8_t><<<grid, threads, 0, ctx->stream>>>(in, (int8_t *)out, n, scale, (float)zp, v);
        break;
    case NNCB_I16:
        quantize_kernel<int16_t><<<grid, threads, 0, ctx->stream>>>(in, (int16_t *)out, n, scale, (float)zp, v);
        break;
    default:
        return fail(-ENOSYS, "quantize: unsupported target type %d", qtype);
    }
    return after_launch(ctx, "quantize");
}

int dequantize(nncb_context *ctx, const void *in, float *out, size_t n, float scale, int32_t zp, int qtype) {
    if (n == 0)
        return 0;
    if (!in || !out)
        return fail(-EINVAL, "dequantize: null pointer");
    const int threads = 256;
    const bool v = aligned16(in, out);
    const int grid = stream_grid(ctx, (n + 15) / 16, threads);
    switch (qtype) {
    case NNCB_U8:
        dequantize_kernel<uint8_t><<<grid, threads, 0, ctx->stream>>>((const uint8_t *)in, out, n, scale, (float)zp, v);
        break;
    case NNCB_I8:
        dequantize_kernel<int8_t><<<grid, threads, 0, ctx->stream>>>((const int8_t *)in, out, n, scale, (float)zp, v);
        break;
    case NNCB_I16:
        dequantize_kernel<int16_t><<<grid, threads, 0, ctx->stream>>>((const int16_t *)in, out, n, scale, (float)zp, v);
        break;
    default:
        return fail(-ENOSYS, "dequantize: unsupported source type %d", qtype);
    }
    return after_launch(ctx, "dequantize");
}

// ---- NCHW f32 -> NHWC u8 (quantize + transpose) ----------------------------------------------
// Tile of 32 channels x 64 pixels through shared memory: global reads run along pixels
// (contiguous in NCHW), global writes along channels (contiguous in NHWC).
template <bool QUANT>
__global__ void __launch_bounds__(256)
nchw_to_nhwc_kernel(const void *__restrict__ in_, uint8_t *__restrict__ out, int c, int hw, int c_pad,
                    float scale, float zp) {
    __shared__ uint8_t tile[64][33];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 64, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6; // 64 x 4
    const uint8_t zq = (uint8_t)min(max(__float2int_rn(zp), 0), 255);
    for (int cc = ty; cc < 32; cc += 4) {
        int ch = c0 + cc, p = p0 + tx;
        uint8_t q = zq;
        if (ch < c && p < hw) {
            size_t idx = ((size_t)n * c + ch) * hw + p;
            if (QUANT)
                q = (uint8_t)quant_dev(__ldcs(reinterpret_cast<const float *>(in_) + idx), scale, zp, 0, 255);
            else
                q = reinterpret_cast<const uint8_t *>(in_)[idx];
        }
        tile[tx][cc] = q;
    }
    __syncthreads();
    const int wc = threadIdx.x & 31, wp = threadIdx.x >> 5; // 32 channels x 8 pixels
    for (int pp = wp; pp < 64; pp += 8) {
        int ch = c0 + wc, p = p0 + pp;
        if (ch < c_pad && p < hw)
            out[((size_t)n * hw + p) * c_pad + ch] = tile[pp][wc];
    }
}

// Few channels (c_pad == 4, c <= 4): one thread per pixel, one 32-bit store.
__global__ void __launch_bounds__(256)
quantize_nchw_to_nhwc4_kernel(const float *__restrict__ in, uint32_t *__restrict__ out, int c, size_t hw,
                              size_t total_pix, float scale, float zp) {
    grid_dependency_release(); // a tensor-core convolution that follows sets itself up meanwhile
    const uint32_t zq = (uint32_t)min(max(__float2int_rn(zp), 0), 255);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_pix;
         i += (size_t)gridDim.x * blockDim.x) {
        size_t n = i / hw, p = i % hw;
        uint32_t word = 0;
#pragma unroll
        for (int ch = 0; ch < 4; ch++) {
            uint32_t q = zq;
            if (ch < c)
                q = (uint32_t)quant_dev(__ldcs(in + (n * c + ch) * hw + p), scale, zp, 0, 255);
            word |= q << (8 * ch);
        }
        out[i] = word;
    }
}

int quantize_nchw_to_nhwc_u8(nncb_context *ctx, const float *in, uint8_t *out, int n, int c, int h, int w,
                             int c_pad, float scale, int32_t zp) {
    if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || c_pad < c)
        return fail(-EINVAL, "quantize_nchw_to_nhwc_u8: bad shape");
    const int hw = h * w;
    if (c_pad == 4 && (reinterpret_cast<uintptr_t>(out) & 3) == 0) {
        size_t total = (size_t)n * hw;
        quantize_nchw_to_nhwc4_kernel<<<stream_grid(ctx, total, 256), 256, 0, ctx->stream>>>(
            in, reinterpret_cast<uint32_t *>(out), c, (size_t)hw, total, scale, (float)zp);
        return after_launch(ctx, "quantize_nchw_to_nhwc4");
    }
    dim3 grid((hw + 63) / 64, (c_pad + 31) / 32, n);
    nchw_to_nhwc_kernel<true><<<grid, 256, 0, ctx->stream>>>(in, out, c, hw, c_pad, scale, (float)zp);
    return after_launch(ctx, "quantize_nchw_to_nhwc");
}

// ---- NCHW f32 -> space-to-depth(2) NHWC u8 ---------------------------------------------------
// out[n][Y][X][(dy*2+dx)*c + ch] = quantize(in[n][ch][2Y+dy][2X+dx]); channels 4c..c_pad-1 hold the
// zero point. Turns a stride-2 convolution over few channels (an image stem) into a stride-1
// convolution over c_pad channels that the tensor-core kernel can take. One thread per cell.
// quantize with the division as q0 = RN(x r), q = RN(q0 + RN(x - q0 s) r) (r = RN(1/s), verified on the host: the
// correctly rounded quotient) and rint + clamp as one saturating conversion; quotients too large for the
// sequence to be proven (they saturate anyway, but x r may overflow) and NaN take the division.
__device__ __forceinline__ uint32_t quant_u8_fast(float x, float s, float r, float zp) {
    const float q0 = __fmul_rn(x, r);
    if (!(fabsf(q0) < 1e30f))
        return (uint32_t)quant_dev(x, s, zp, 0, 255);
    const float q = __fmaf_rn(__fmaf_rn(-q0, s, x), r, q0);
    uint32_t o;
    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(o) : "f"(__fadd_rn(q, zp)));
    return o;
}

// CT: the channel count when it is known at compile time (3: images), else 0 and `c` is used. With CT the
// twelve loads of a cell are independent and every byte lands in a fixed place of the cell's words.
constexpr uint32_t S2D_ROWS = 1, POOL_ROWS = 1; // cell / output rows per block (more rows per block measured slower)
template <int CPAD, bool IN_NHWC, int CT>
__global__ void __launch_bounds__(256)
quantize_nchw_to_s2d_kernel(const float *__restrict__ in, uint8_t *__restrict__ out, int c_rt, int h, int w,
                            float scale, float rscale, float zp, int pad_t, int pad_b, int pad_l, int pad_r,
                            uint32_t total_rows) {
    grid_dependency_release(); // a tensor-core convolution that follows sets itself up meanwhile
    // output cells include a border of pad_* cells that hold the zero point in every channel;
    // blockIdx.x = (image, cell row), blockIdx.y * blockDim.x + thread = cell in the row
    const int c = CT ? CT : c_rt;
    const int hc = h / 2 + pad_t + pad_b, wc = w / 2 + pad_l + pad_r;
    const uint32_t zq = (uint32_t)min(max(__float2int_rn(zp), 0), 255);
    const int xc = (int)(blockIdx.y * blockDim.x + threadIdx.x);
    // a block walks S2D_ROWS consecutive cell rows: fewer, longer-lived blocks than one per row
    for (uint32_t row = blockIdx.x * S2D_ROWS; row < min((blockIdx.x + 1) * S2D_ROWS, total_rows); row++)
    if (xc < wc) {
        const int X = xc - pad_l;
        const int Y = (int)(row % (uint32_t)hc) - pad_t;
        const size_t n = row / (uint32_t)hc;
        const size_t i = (size_t)row * wc + xc;
        uint32_t words[CPAD / 4];
#pragma unroll
        for (int k = 0; k < CPAD / 4; k++)
            words[k] = zq * 0x01010101u;
        const bool inside = X >= 0 && Y >= 0 && X < w / 2 && Y < h / 2;
        auto one = [&](int ch, int dy) {
            float2 v;
            if (IN_NHWC) {
                const float *px = in + ((n * h + (2 * Y + dy)) * (size_t)w + 2 * X) * c + ch;
                v = make_float2(__ldcs(px), __ldcs(px + c));
            } else {
                v = __ldcs(reinterpret_cast<const float2 *>(in + ((n * c + ch) * h + (2 * Y + dy)) * (size_t)w + 2 * X));
            }
            uint32_t q0, q1;
            if (rscale != 0.f) {
                q0 = quant_u8_fast(v.x, scale, rscale, zp), q1 = quant_u8_fast(v.y, scale, rscale, zp);
            } else {
                q0 = (uint32_t)quant_dev(v.x, scale, zp, 0, 255), q1 = (uint32_t)quant_dev(v.y, scale, zp, 0, 255);
            }
            const int i0 = (dy * 2 + 0) * c + ch, i1 = (dy * 2 + 1) * c + ch;
#pragma unroll
            for (int k = 0; k < CPAD / 4; k++) {
                // constant-indexed update keeps `words` in registers
                if ((i0 >> 2) == k)
                    words[k] = (words[k] & ~(0xFFu << (8 * (i0 & 3)))) | (q0 << (8 * (i0 & 3)));
                if ((i1 >> 2) == k)
                    words[k] = (words[k] & ~(0xFFu << (8 * (i1 & 3)))) | (q1 << (8 * (i1 & 3)));
            }
        };
        if (inside && CT && !IN_NHWC && rscale != 0.f) {
            // Straight-line form for a known channel count: all loads first (independent), then the division-free
            // quantization two values at a time on packed f32x2 operations, bytes assembled with byte permutes.
            // Inputs are clamped to [xlo, xhi] first: beyond them the result is 0 or 255 either way (the bounds sit
            // two quantization steps outside the u8 range), NaN takes xlo like the reference's conversion gives 0,
            // and no product can overflow.
            const float xlo = scale * (-zp - 2.f), xhi = scale * (257.f - zp);
            const uint64_t r2 = pack2(rscale, rscale), ns2 = pack2(-scale, -scale), z2 = pack2(zp, zp);
            const float *base = in + ((n * CT) * h + 2 * Y) * (size_t)w + 2 * X;
            const uint32_t plane = (uint32_t)h * (uint32_t)w;
            float2 v[CT ? CT : 1][2];
#pragma unroll
            for (int ch = 0; ch < (CT ? CT : 1); ch++)
#pragma unroll
                for (int dy = 0; dy < 2; dy++)
                    v[ch][dy] = __ldcs(reinterpret_cast<const float2 *>(base + ch * plane + dy * (uint32_t)w));
            uint32_t q[4 * (CT ? CT : 1)]; // byte (dy*2 + dx)*c + ch
#pragma unroll
            for (int ch = 0; ch < (CT ? CT : 1); ch++)
#pragma unroll
                for (int dy = 0; dy < 2; dy++) {
                    const float a = fminf(fmaxf(v[ch][dy].x, xlo), xhi), b = fminf(fmaxf(v[ch][dy].y, xlo), xhi);
                    const uint64_t x2 = pack2(a, b);
                    const uint64_t q0 = mul2(x2, r2);
                    float u0, u1;
                    unpack2(add2(fma2(fma2(q0, ns2, x2), r2, q0), z2), u0, u1);
                    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q[(dy * 2 + 0) * CT + ch]) : "f"(u0));
                    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q[(dy * 2 + 1) * CT + ch]) : "f"(u1));
                }
#pragma unroll
            for (int k = 0; k < CPAD / 4; k++) {
                uint32_t b[4];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    b[j] = (4 * k + j) < 4 * CT ? q[(4 * k + j) < 4 * CT ? 4 * k + j : 0] : zq;
                words[k] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
            }
        } else if (inside) {
            if (CT) {
#pragma unroll
                for (int ch = 0; ch < (CT ? CT : 1); ch++) {
                    one(ch, 0);
                    one(ch, 1);
                }
            } else {
                for (int ch = 0; ch < c; ch++) {
                    one(ch, 0);
                    one(ch, 1);
                }
            }
        }
        uint4 *o = reinterpret_cast<uint4 *>(out + i * CPAD);
#pragma unroll
        for (int k = 0; k < CPAD / 16; k++)
            o[k] = make_uint4(words[4 * k], words[4 * k + 1], words[4 * k + 2], words[4 * k + 3]);
    }
}

int quantize_nchw_to_s2d_u8(nncb_context *ctx, const float *in, uint8_t *out, int n, int c, int h, int w, int c_pad,
                            float scale, int32_t zp, bool in_nhwc, int pad_t, int pad_b, int pad_l, int pad_r) {
    if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || (h & 1) || (w & 1))
        return fail(-EINVAL, "quantize_nchw_to_s2d_u8: height and width must be positive and even");
    if (pad_t < 0 || pad_b < 0 || pad_l < 0 || pad_r < 0)
        return fail(-EINVAL, "quantize_nchw_to_s2d_u8: negative padding");
    if (4 * c > c_pad || (c_pad != 16 && c_pad != 32))
        return fail(-EINVAL, "quantize_nchw_to_s2d_u8: c_pad must be 16 or 32 and hold 4*c channels");
    if ((reinterpret_cast<uintptr_t>(in) & 7) || (reinterpret_cast<uintptr_t>(out) & 15))
        return fail(-EINVAL, "quantize_nchw_to_s2d_u8: pointers must be 8-byte (in) and 16-byte (out) aligned");
    const int hc = h / 2 + pad_t + pad_b, wc = w / 2 + pad_l + pad_r;
    const int bt = wc >= 256 ? 256 : (wc + 31) / 32 * 32;
    if ((size_t)n * hc > 0x7fffffffull)
        return fail(-EINVAL, "quantize_nchw_to_s2d_u8: too many rows");
    const uint32_t total_rows = (uint32_t)((size_t)n * hc);
    const dim3 grid((total_rows + S2D_ROWS - 1) / S2D_ROWS, (unsigned)((wc + bt - 1) / bt));
    // the reciprocal of the scale, when it is one the division-free sequence is proven for (else 0: divide)
    bool r_ok = true;
    float rscale = rn_reciprocal(scale, &r_ok);
    if (!r_ok)
        rscale = 0.f;
#define NNCB_S2D(CP, NH, CT_)                                                                                          \
    quantize_nchw_to_s2d_kernel<CP, NH, CT_><<<grid, bt, 0, ctx->stream>>>(in, out, c, h, w, scale, rscale, (float)zp, pad_t, \
                                                                           pad_b, pad_l, pad_r, total_rows)
    if (c == 3) {
        if (c_pad == 32 && in_nhwc)
            NNCB_S2D(32, true, 3);
        else if (c_pad == 32)
            NNCB_S2D(32, false, 3);
        else if (in_nhwc)
            NNCB_S2D(16, true, 3);
        else
            NNCB_S2D(16, false, 3);
    } else {
        if (c_pad == 32 && in_nhwc)
            NNCB_S2D(32, true, 0);
        else if (c_pad == 32)
            NNCB_S2D(32, false, 0);
        else if (in_nhwc)
            NNCB_S2D(16, true, 0);
        else
            NNCB_S2D(16, false, 0);
    }
#undef NNCB_S2D
    return after_launch(ctx, "quantize_nchw_to_s2d");
}

int nchw_to_nhwc_u8(nncb_context *ctx, const uint8_t *in, uint8_t *out, int n, int c, int h, int w) {
    if (n <= 0 || c <= 0 || h <= 0 || w <= 0)
        return fail(-EINVAL, "nchw_to_nhwc_u8: bad shape");
    const int hw = h * w;
    dim3 grid((hw + 63) / 64, (c + 31) / 32, n);
    nchw_to_nhwc_kernel<false><<<grid, 256, 0, ctx->stream>>>(in, out, c, hw, c, 1.f, 0.f);
    return after_launch(ctx, "nchw_to_nhwc_u8");
}

// ---- NHWC u8 -> NCHW (f32 dequantized, or u8) ---------------------------------------------------
template <bool DEQUANT>
__global__ void __launch_bounds__(256)
nhwc_to_nchw_kernel(const uint8_t *__restrict__ in, void *__restrict__ out_, int c, int hw, float scale, float zp) {
    __shared__ uint8_t tile[64][33];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 64, c0 = blockIdx.y * 32;
    const int wc = threadIdx.x & 31, wp = threadIdx.x >> 5;
    for (int pp = wp; pp < 64; pp += 8) {
        int ch = c0 + wc, p = p0 + pp;
        tile[pp][wc] = (ch < c && p < hw) ? in[((size_t)n * hw + p) * c + ch] : 0;
    }
    __syncthreads();
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    for (int cc = ty; cc < 32; cc += 4) {
        int ch = c0 + cc, p = p0 + tx;
        if (ch < c && p < hw) {
            size_t idx = ((size_t)n * c + ch) * hw + p;
            if (DEQUANT)
                __stcs(reinterpret_cast<float *>(out_) + idx, dequant_dev((float)tile[tx][cc], zp, scale));
            else
                reinterpret_cast<uint8_t *>(out_)[idx] = tile[tx][cc];
        }
    }
}

int dequantize_nhwc_to_nchw_f32(nncb_context *ctx, const uint8_t *in, float *out, int n, int h, int w, int c,
                                float scale, int32_t zp) {
    if (n <= 0 || c <= 0 || h <= 0 || w <= 0)
        return fail(-EINVAL, "dequantize_nhwc_to_nchw_f32: bad shape");
    const int hw = h * w;
    dim3 grid((hw + 63) / 64, (c + 31) / 32, n);
    nhwc_to_nchw_kernel<true><<<grid, 256, 0, ctx->stream>>>(in, out, c, hw, scale, (float)zp);
    return after_launch(ctx, "dequantize_nhwc_to_nchw");
}

int nhwc_to_nchw_u8(nncb_context *ctx, const uint8_t *in, uint8_t *out, int n, int h, int w, int c) {
    if (n <= 0 || c <= 0 || h <= 0 || w <= 0)
        return fail(-EINVAL, "nhwc_to_nchw_u8: bad shape");
    const int hw = h * w;
    dim3 grid((hw + 63) / 64, (c + 31) / 32, n);
    nhwc_to_nchw_kernel<false><<<grid, 256, 0, ctx->stream>>>(in, out, c, hw, 1.f, 0.f);
    return after_launch(ctx, "nhwc_to_nchw_u8");
}

// ---- element-wise add between quantized tensors ------------------------------------------------
// rso != 0: the division-free form. byte -> float and the zero-point subtraction are one PRMT and one exact add
// (the bits 0x4B0000qq are the float 2^23 + qq, and (2^23 + qq) - (2^23 + z) = qq - z exactly), the output division
// is the verified-reciprocal sequence, rint + clamp one saturating conversion.
__device__ __forceinline__ uint32_t qadd4(uint32_t a, uint32_t b, float sa, float za, float sb, float zb,
                                          float so, float zo, float rso) {
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if (rso != 0.f) {
            const float qa = __uint_as_float(__byte_perm(a, 0x4B000000u, 0x7440 | i)); // 2^23 + byte i of a
            const float qb = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7440 | i));
            const float fa = __fmul_rn(__fsub_rn(qa, __fadd_rn(8388608.0f, za)), sa);
            const float fb = __fmul_rn(__fsub_rn(qb, __fadd_rn(8388608.0f, zb)), sb);
            r |= quant_u8_fast(__fadd_rn(fa, fb), so, rso, zo) << (8 * i);
        } else {
            float fa = dequant_dev((float)((a >> (8 * i)) & 255), za, sa);
            float fb = dequant_dev((float)((b >> (8 * i)) & 255), zb, sb);
            r |= (uint32_t)quant_dev(__fadd_rn(fa, fb), so, zo, 0, 255) << (8 * i);
        }
    }
    return r;
}

// The division-free form on two elements per instruction (f32x2: each half rounds like the scalar operation).
// Bytes i and i + 1 of a and b -> two output bytes in the low half of the result.
__device__ __forceinline__ uint32_t qadd2(uint32_t a, uint32_t b, int i, uint64_t nza2, uint64_t sa2, uint64_t nzb2,
                                          uint64_t sb2, uint64_t rso2, uint64_t nso2, uint64_t zo2) {
    // 2^23 + byte as float bits; nza2 = -(2^23 + za): the sum is byte - za exactly
    const uint64_t qa = pack2(__uint_as_float(__byte_perm(a, 0x4B000000u, 0x7440 | i)),
                              __uint_as_float(__byte_perm(a, 0x4B000000u, 0x7440 | (i + 1))));
    const uint64_t qb = pack2(__uint_as_float(__byte_perm(b, 0x4B000000u, 0x7440 | i)),
                              __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7440 | (i + 1))));
    // fa and fb must each round before they are added: a packed add fed by a packed multiply would be contracted
    // into one fused multiply-add, so the sum runs as two scalar adds
    const uint64_t fa = mul2(add2(qa, nza2), sa2), fb = mul2(add2(qb, nzb2), sb2);
    float fa0, fa1, fb0, fb1;
    unpack2(fa, fa0, fa1);
    unpack2(fb, fb0, fb1);
    const uint64_t x2 = pack2(__fadd_rn(fa0, fb0), __fadd_rn(fa1, fb1));
    const uint64_t q0 = mul2(x2, rso2);
    const uint64_t q2 = fma2(fma2(q0, nso2, x2), rso2, q0);
    float u0, u1;
    unpack2(add2(q2, zo2), u0, u1);
    uint32_t r0, r1;
    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(r0) : "f"(u0));
    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(r1) : "f"(u1));
    return r0 | (r1 << 8);
}
__device__ __forceinline__ uint32_t qadd4p(uint32_t a, uint32_t b, uint64_t nza2, uint64_t sa2, uint64_t nzb2, uint64_t sb2,
                                           uint64_t rso2, uint64_t nso2, uint64_t zo2) {
    return qadd2(a, b, 0, nza2, sa2, nzb2, sb2, rso2, nso2, zo2) | (qadd2(a, b, 2, nza2, sa2, nzb2, sb2, rso2, nso2, zo2) << 16);
}

__global__ void __launch_bounds__(256)
qadd_kernel(const uint8_t *__restrict__ a, const uint8_t *__restrict__ b, uint8_t *__restrict__ y, size_t n,
            float sa, float za, float sb, float zb, float so, float zo, float rso, bool vec_ok) {
    grid_dependency_release(); // a tensor-core convolution that follows sets itself up meanwhile
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    const size_t nvec = vec_ok ? n / 16 : 0;
    if (rso != 0.f) {
        const float mza = -__fadd_rn(8388608.0f, za), mzb = -__fadd_rn(8388608.0f, zb);
        const uint64_t nza2 = pack2(mza, mza), nzb2 = pack2(mzb, mzb), sa2 = pack2(sa, sa), sb2 = pack2(sb, sb);
        const uint64_t rso2 = pack2(rso, rso), nso2 = pack2(-so, -so), zo2 = pack2(zo, zo);
        auto one = [&](const uint4 &va, const uint4 &vb) {
            uint4 r;
            r.x = qadd4p(va.x, vb.x, nza2, sa2, nzb2, sb2, rso2, nso2, zo2);
            r.y = qadd4p(va.y, vb.y, nza2, sa2, nzb2, sb2, rso2, nso2, zo2);
            r.z = qadd4p(va.z, vb.z, nza2, sa2, nzb2, sb2, rso2, nso2, zo2);
            r.w = qadd4p(va.w, vb.w, nza2, sa2, nzb2, sb2, rso2, nso2, zo2);
            return r;
        };
        size_t v = tid;
        for (; v + nthreads < nvec; v += 2 * nthreads) { // two independent vectors in flight
            const uint4 a0 = __ldcs(reinterpret_cast<const uint4 *>(a) + v), b0 = __ldcs(reinterpret_cast<const uint4 *>(b) + v);
            const uint4 a1 = __ldcs(reinterpret_cast<const uint4 *>(a) + v + nthreads);
            const uint4 b1 = __ldcs(reinterpret_cast<const uint4 *>(b) + v + nthreads);
            __stcs(reinterpret_cast<uint4 *>(y) + v, one(a0, b0));
            __stcs(reinterpret_cast<uint4 *>(y) + v + nthreads, one(a1, b1));
        }
        for (; v < nvec; v += nthreads)
            __stcs(reinterpret_cast<uint4 *>(y) + v,
                   one(__ldcs(reinterpret_cast<const uint4 *>(a) + v), __ldcs(reinterpret_cast<const uint4 *>(b) + v)));
    } else {
        for (size_t v = tid; v < nvec; v += nthreads) {
            uint4 va = __ldcs(reinterpret_cast<const uint4 *>(a) + v);
            uint4 vb = __ldcs(reinterpret_cast<const uint4 *>(b) + v);
            uint4 r;
            r.x = qadd4(va.x, vb.x, sa, za, sb, zb, so, zo, rso);
            r.y = qadd4(va.y, vb.y, sa, za, sb, zb, so, zo, rso);
            r.z = qadd4(va.z, vb.z, sa, za, sb, zb, so, zo, rso);
            r.w = qadd4(va.w, vb.w, sa, za, sb, zb, so, zo, rso);
            __stcs(reinterpret_cast<uint4 *>(y) + v, r);
        }
    }
    for (size_t i = nvec * 16 + tid; i < n; i += nthreads) {
        float fa = dequant_dev((float)a[i], za, sa), fb = dequant_dev((float)b[i], zb, sb);
        y[i] = (uint8_t)quant_dev(__fadd_rn(fa, fb), so, zo, 0, 255);
    }
}

int qadd_u8(nncb_context *ctx, const uint8_t *a, const uint8_t *b, uint8_t *y, size_t n, float sa, int32_t za,
            float sb, int32_t zb, float so, int32_t zo) {
    if (n == 0)
        return 0;
    if (!a || !b || !y)
        return fail(-EINVAL, "qadd_u8: null pointer");
    bool v = aligned16(a, b) && aligned16(y, y);
    // zero points within a byte keep 2^23 + z exact; the reciprocal must be one the sequence is proven for
    bool r_ok = za >= 0 && za <= 255 && zb >= 0 && zb <= 255;
    float rso = rn_reciprocal(so, &r_ok);
    if (!r_ok)
        rso = 0.f;
    qadd_kernel<<<stream_grid(ctx, (n + 15) / 16, 256), 256, 0, ctx->stream>>>(a, b, y, n, sa, (float)za, sb,
                                                                                  (float)zb, so, (float)zo, rso, v);
    return after_launch(ctx, "qadd_u8");
}

// ---- table look-up -------------------------------------------------------------------------------
struct lut256 {
    uint8_t t[256];
};

__global__ void __launch_bounds__(256)
lut_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, size_t n, const lut256 table, bool vec_ok) {
    __shared__ uint8_t s[256];
    s[threadIdx.x] = table.t[threadIdx.x];
    __syncthreads();
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    const size_t nvec = vec_ok ? n / 16 : 0;
    for (size_t v = tid; v < nvec; v += nthreads) {
        uint4 in = __ldcs(reinterpret_cast<const uint4 *>(x) + v);
        uint32_t w[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            uint32_t r = 0;
#pragma unroll
            for (int i = 0; i < 4; i++)
                r |= (uint32_t)s[(w[k] >> (8 * i)) & 255] << (8 * i);
            w[k] = r;
        }
        __stcs(reinterpret_cast<uint4 *>(y) + v, make_uint4(w[0], w[1], w[2], w[3]));
    }
    for (size_t i = nvec * 16 + tid; i < n; i += nthreads)
        y[i] = s[x[i]];
}

int lut_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, size_t n, const uint8_t *host_table) {
    if (n == 0)
        return 0;
    if (!x || !y || !host_table)
        return fail(-EINVAL, "lut_u8: null pointer");
    lut256 t;
    memcpy(t.t, host_table, 256);
    lut_kernel<<<stream_grid(ctx, (n + 15) / 16, 256), 256, 0, ctx->stream>>>(x, y, n, t, aligned16(x, y));
    return after_launch(ctx, "lut_u8");
}

// ---- max pooling on u8 NHWC ----------------------------------------------------------------------
// One thread per (output pixel, 16-channel group) when c % 16 == 0 (128-bit accesses, byte-wise
// max via __vmaxu4), else one thread per element.
__global__ void __launch_bounds__(256)
maxpool_vec_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int n, int h, int w, int c, int oh,
                   int ow, int kh, int kw, int sh, int sw, int pt, int pl, uint32_t zp4) {
    grid_dependency_release(); // a tensor-core convolution that follows sets itself up meanwhile
    // blockIdx.x = (image, output row); blockIdx.y * blockDim.x + thread = (output column, channel group)
    const uint32_t cg = (uint32_t)c / 16u;
    const uint32_t j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j < (uint32_t)ow * cg) {
        const int g = (int)(j % cg), ox = (int)(j / cg);
        const int oy = (int)(blockIdx.x % (uint32_t)oh), b = (int)(blockIdx.x / (uint32_t)oh);
        const size_t p = (size_t)blockIdx.x * ow + ox;
        uint4 m = make_uint4(0, 0, 0, 0);
        int cnt = 0;
        for (int ky = 0; ky < kh; ky++) {
            int iy = oy * sh - pt + ky;
            if (iy < 0 || iy >= h)
                continue;
            for (int kx = 0; kx < kw; kx++) {
                int ix = ox * sw - pl + kx;
                if (ix < 0 || ix >= w)
                    continue;
                uint4 v = __ldg(reinterpret_cast<const uint4 *>(x + (((size_t)b * h + iy) * w + ix) * c) + g);
                m.x = __vmaxu4(m.x, v.x);
                m.y = __vmaxu4(m.y, v.y);
                m.z = __vmaxu4(m.z, v.z);
                m.w = __vmaxu4(m.w, v.w);
                cnt++;
            }
        }
        if (cnt < kh * kw) {
            m.x = __vmaxu4(m.x, zp4);
            m.y = __vmaxu4(m.y, zp4);
            m.z = __vmaxu4(m.z, zp4);
            m.w = __vmaxu4(m.w, zp4);
        }
        reinterpret_cast<uint4 *>(y + p * c)[g] = m;
    }
}

// The same with the window size known at compile time: the window's loads are independent and all in flight
// before the first maximum (the general kernel's loops issue one load at a time).
template <int KH, int KW>
__global__ void __launch_bounds__(256)
maxpool_vec_fixed_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int n, int h, int w, int c, int oh, int ow,
                         int sh, int sw, int pt, int pl, uint32_t zp4, uint32_t total_rows) {
    grid_dependency_release(); // a tensor-core convolution that follows sets itself up meanwhile
    const uint32_t cg = (uint32_t)c / 16u;
    const uint32_t j = blockIdx.y * blockDim.x + threadIdx.x;
    // a block walks POOL_ROWS consecutive output rows: fewer, longer-lived blocks than one per row
    for (uint32_t row = blockIdx.x * POOL_ROWS; row < min((blockIdx.x + 1) * POOL_ROWS, total_rows); row++)
    if (j < (uint32_t)ow * cg) {
        const int g = (int)(j % cg), ox = (int)(j / cg);
        const int oy = (int)(row % (uint32_t)oh), b = (int)(row / (uint32_t)oh);
        const size_t p = (size_t)row * ow + ox;
        uint4 v[KH * KW];
        bool all = true;
#pragma unroll
        for (int ky = 0; ky < KH; ky++)
#pragma unroll
            for (int kx = 0; kx < KW; kx++) {
                const int iy = oy * sh - pt + ky, ix = ox * sw - pl + kx;
                const bool valid = iy >= 0 && iy < h && ix >= 0 && ix < w;
                all = all && valid;
                v[ky * KW + kx] = valid ? __ldg(reinterpret_cast<const uint4 *>(x + (((size_t)b * h + iy) * w + ix) * c) + g)
                                        : make_uint4(0, 0, 0, 0);
            }
        // Byte-wise maximum on the three-input 16-bit-pair maximum of the hardware: every word is split into its
        // even and its odd bytes (one byte permute each), the taps are reduced three at a time, and the two halves
        // are interleaved again. The byte-wise __vmaxu4 is a multi-instruction sequence, and with nine taps it made
        // the kernel issue-bound.
        const uint32_t zlo = all ? 0u : (zp4 & 0x00FF00FFu); // a padded tap holds the zero point
        uint32_t mw[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            uint32_t lo = zlo, hi = zlo;
            auto word = [&](int t) { return k == 0 ? v[t].x : (k == 1 ? v[t].y : (k == 2 ? v[t].z : v[t].w)); };
            int t = 0;
#pragma unroll
            for (; t + 1 < KH * KW; t += 2) {
                const uint32_t a = word(t), b = word(t + 1);
                lo = __vimax3_u16x2(lo, __byte_perm(a, 0u, 0x4240), __byte_perm(b, 0u, 0x4240));
                hi = __vimax3_u16x2(hi, __byte_perm(a, 0u, 0x4341), __byte_perm(b, 0u, 0x4341));
            }
            if (t < KH * KW) {
                const uint32_t a = word(t);
                lo = __vimax3_u16x2(lo, __byte_perm(a, 0u, 0x4240), 0u);
                hi = __vimax3_u16x2(hi, __byte_perm(a, 0u, 0x4341), 0u);
            }
            mw[k] = __byte_perm(lo, hi, 0x6240);
        }
        reinterpret_cast<uint4 *>(y + p * c)[g] = make_uint4(mw[0], mw[1], mw[2], mw[3]);
    }
}

__global__ void __launch_bounds__(256)
maxpool_scalar_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int n, int h, int w, int c,
                      int oh, int ow, int kh, int kw, int sh, int sw, int pt, int pl, int zp) {
    const size_t total = (size_t)n * oh * ow * c;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        int ch = (int)(i % c);
        size_t p = i / c;
        int ox = (int)(p % ow);
        int oy = (int)((p / ow) % oh);
        int b = (int)(p / ((size_t)ow * oh));
        int m = 0, cnt = 0;
        for (int ky = 0; ky < kh; ky++) {
            int iy = oy * sh - pt + ky;
            if (iy < 0 || iy >= h)
                continue;
            for (int kx = 0; kx < kw; kx++) {
                int ix = ox * sw - pl + kx;
                if (ix < 0 || ix >= w)
                    continue;
                m = max(m, (int)x[(((size_t)b * h + iy) * w + ix) * c + ch]);
                cnt++;
            }
        }
        if (cnt < kh * kw)
            m = max(m, zp);
        y[i] = (uint8_t)m;
    }
}

int maxpool_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int kh, int kw,
               int sh, int sw, int pt, int pb, int pl, int pr, int32_t zp) {
    if (n <= 0 || h <= 0 || w <= 0 || c <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0)
        return fail(-EINVAL, "maxpool_u8: bad shape");
    const int oh = conv_out_size(h, kh, sh, 1, pt, pb), ow = conv_out_size(w, kw, sw, 1, pl, pr);
    if (oh <= 0 || ow <= 0)
        return fail(-EINVAL, "maxpool_u8: empty output");
    const int z = zp < 0 ? 0 : (zp > 255 ? 255 : zp);
    if (c % 16 == 0 && aligned16(x, y)) {
        const int row_items = ow * (c / 16);
        const int bt = row_items >= 256 ? 256 : (row_items + 31) / 32 * 32;
        if ((size_t)n * oh > 0x7fffffffull)
            return fail(-EINVAL, "maxpool_u8: too many rows");
        const dim3 grid((unsigned)((size_t)n * oh), (unsigned)((row_items + bt - 1) / bt));
        const uint32_t z4 = (uint32_t)z * 0x01010101u;
        const uint32_t rows = (uint32_t)((size_t)n * oh);
        const dim3 gridf((rows + POOL_ROWS - 1) / POOL_ROWS, grid.y);
        if (kh == 3 && kw == 3) {
            maxpool_vec_fixed_kernel<3, 3><<<gridf, bt, 0, ctx->stream>>>(x, y, n, h, w, c, oh, ow, sh, sw, pt, pl, z4, rows);
            return after_launch(ctx, "maxpool_u8");
        }
        if (kh == 2 && kw == 2) {
            maxpool_vec_fixed_kernel<2, 2><<<gridf, bt, 0, ctx->stream>>>(x, y, n, h, w, c, oh, ow, sh, sw, pt, pl, z4, rows);
            return after_launch(ctx, "maxpool_u8");
        }
        if (kh == 5 && kw == 5) {
            maxpool_vec_fixed_kernel<5, 5><<<gridf, bt, 0, ctx->stream>>>(x, y, n, h, w, c, oh, ow, sh, sw, pt, pl, z4, rows);
            return after_launch(ctx, "maxpool_u8");
        }
        maxpool_vec_kernel<<<grid, bt, 0, ctx->stream>>>(
            x, y, n, h, w, c, oh, ow, kh, kw, sh, sw, pt, pl, (uint32_t)z * 0x01010101u);
    } else {
        size_t total = (size_t)n * oh * ow * c;
        maxpool_scalar_kernel<<<stream_grid(ctx, total, 256), 256, 0, ctx->stream>>>(x, y, n, h, w, c, oh, ow, kh,
                                                                                      kw, sh, sw, pt, pl, z);
    }
    return after_launch(ctx, "maxpool_u8");
}

// ---- global mean over H x W ----------------------------------------------------------------------
// One thread per (image, channel); consecutive threads read consecutive channels.
__global__ void __launch_bounds__(256)
global_avgpool_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int n, int hw, int c, float si,
                      int zi, float so, float zo) {
    const size_t total = (size_t)n * c;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        int ch = (int)(i % c);
        size_t b = i / c;
        const uint8_t *p = x + b * hw * c + ch;
        int s = 0;
        for (int k = 0; k < hw; k++)
            s += p[(size_t)k * c];
        s -= hw * zi;
        float m = __fdiv_rn(__fmul_rn((float)s, si), (float)hw);
        y[i] = (uint8_t)quant_dev(m, so, zo, 0, 255);
    }
}

int global_avgpool_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, float si,
                      int32_t zi, float so, int32_t zo) {
    if (n <= 0 || h <= 0 || w <= 0 || c <= 0)
        return fail(-EINVAL, "global_avgpool_u8: bad shape");
    size_t total = (size_t)n * c;
    global_avgpool_kernel<<<stream_grid(ctx, total, 256), 256, 0, ctx->stream>>>(x, y, n, h * w, c, si, zi, so,
                                                                                 (float)zo);
    return after_launch(ctx, "global_avgpool_u8");
}

// i / d and i % d; 32-bit arithmetic when i fits (a 64-bit division costs some seventy instructions).
__device__ __forceinline__ void divmod_fast(size_t i, uint32_t d, size_t &q, uint32_t &r) {
    if (i <= 0xffffffffull) {
        const uint32_t ii = (uint32_t)i;
        q = ii / d, r = ii % d;
    } else {
        q = i / d, r = (uint32_t)(i % d);
    }
}

// ---- channel-block copy with optional table (concat / split of NHWC tensors) ---------------------
// dst[p][dst_off + j] = table ? table[src[p][src_off + j]] : src[p][src_off + j],  j < len, p < pixels.
// Concat requantises every input into the output's quant param (a 256-entry table per input); a
// split is the same copy without a table. 16-byte accesses when offsets and widths allow.
__global__ void __launch_bounds__(256)
copy_channels_kernel(const uint8_t *__restrict__ src, int src_c, int src_off, uint8_t *__restrict__ dst, int dst_c,
                     int dst_off, int len, size_t pixels, const lut256 table, bool use_table, bool vec_ok) {
    __shared__ uint8_t s[256];
    s[threadIdx.x] = table.t[threadIdx.x];
    __syncthreads();
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    if (vec_ok) {
        const int vpp = len / 16; // 16-byte vectors per pixel
        const size_t total = pixels * vpp;
        for (size_t i = tid; i < total; i += nth) {
            size_t p;
            uint32_t v;
            divmod_fast(i, (uint32_t)vpp, p, v);
            uint4 in = __ldg(reinterpret_cast<const uint4 *>(src + p * src_c + src_off) + v);
            if (use_table) {
                uint32_t w[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
                for (int k = 0; k < 4; k++)
                    w[k] = (uint32_t)s[w[k] & 255] | ((uint32_t)s[(w[k] >> 8) & 255] << 8) |
                           ((uint32_t)s[(w[k] >> 16) & 255] << 16) | ((uint32_t)s[w[k] >> 24] << 24);
                in = make_uint4(w[0], w[1], w[2], w[3]);
            }
            reinterpret_cast<uint4 *>(dst + p * dst_c + dst_off)[v] = in;
        }
    } else {
        const size_t total = pixels * len;
        for (size_t i = tid; i < total; i += nth) {
            const size_t p = i / len;
            const int j = (int)(i % len);
            const uint8_t q = src[p * src_c + src_off + j];
            dst[p * dst_c + dst_off + j] = use_table ? s[q] : q;
        }
    }
}

int copy_channels_u8(nncb_context *ctx, const uint8_t *src, int src_c, int src_off, uint8_t *dst, int dst_c, int dst_off,
                     int len, size_t pixels, const uint8_t *host_table) {
    if (pixels == 0 || len == 0)
        return 0;
    if (!src || !dst || src_c <= 0 || dst_c <= 0 || src_off < 0 || dst_off < 0 || len < 0 || src_off + len > src_c ||
        dst_off + len > dst_c)
        return fail(-EINVAL, "copy_channels_u8: channel block out of range");
    lut256 t;
    if (host_table)
        memcpy(t.t, host_table, 256);
    else
        memset(t.t, 0, 256);
    const bool vec = aligned16(src, dst) && ((src_c | src_off | dst_c | dst_off | len) % 16 == 0);
    const size_t items = vec ? pixels * (len / 16) : pixels * len;
    copy_channels_kernel<<<stream_grid(ctx, items, 256), 256, 0, ctx->stream>>>(src, src_c, src_off, dst, dst_c, dst_off,
                                                                                len, pixels, t, host_table != nullptr, vec);
    return after_launch(ctx, "copy_channels_u8");
}

// ---- nearest-neighbour resize by an integer factor (NHWC u8) --------------------------------------
// out[n][y][x][:] = in[n][y / fy][x / fx][:]  (resize_image nearest with asymmetric coordinates and
// floor rounding, reference/resize_image.cpp, for integer scale factors).
__global__ void __launch_bounds__(256)
resize_nearest_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int n, int h, int w, int c, int fy, int fx,
                      bool vec_ok) {
    const int oh = h * fy, ow = w * fx;
    const int per = vec_ok ? c / 16 : c;
    const size_t total = (size_t)n * oh * ow * per;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t p, row, b;
        uint32_t j, ox, oy;
        divmod_fast(i, (uint32_t)per, p, j);
        divmod_fast(p, (uint32_t)ow, row, ox);
        divmod_fast(row, (uint32_t)oh, b, oy);
        const size_t sp = (b * h + oy / fy) * w + ox / fx;
        if (vec_ok)
            reinterpret_cast<uint4 *>(y + p * c)[j] = __ldg(reinterpret_cast<const uint4 *>(x + sp * c) + j);
        else
            y[p * c + j] = x[sp * c + j];
    }
}

int resize_nearest_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int fy, int fx) {
    if (n <= 0 || h <= 0 || w <= 0 || c <= 0 || fy <= 0 || fx <= 0)
        return fail(-EINVAL, "resize_nearest_u8: bad shape");
    const bool vec = c % 16 == 0 && aligned16(x, y);
    const size_t total = (size_t)n * h * fy * w * fx * (vec ? c / 16 : c);
    resize_nearest_kernel<<<stream_grid(ctx, total, 256), 256, 0, ctx->stream>>>(x, y, n, h, w, c, fy, fx, vec);
    return after_launch(ctx, "resize_nearest_u8");
}

// ---- softmax over the last axis (f32) -----------------------------------------------------------
// reference::softmax (src/Native/src/kernels/stackvm/reference/softmax.cpp:30-80): subtract the
// row maximum, scale by beta, expf, sum, multiply by 1/sum. One warp per row, shuffle reductions.
__global__ void __launch_bounds__(256)
softmax_rows_kernel(const float *__restrict__ in, float *__restrict__ out, size_t rows, int cols, float beta) {
    const int lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t r = warp; r < rows; r += nwarps) {
        const float *x = in + r * cols;
        float *y = out + r * cols;
        float mx = -INFINITY;
        for (int j = lane; j < cols; j += 32)
            mx = fmaxf(mx, x[j]);
        for (int o = 16; o > 0; o >>= 1)
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
        for (int j = lane; j < cols; j += 32) {
            const float e = expf(__fmul_rn(__fsub_rn(x[j], mx), beta));
            y[j] = e;
            sum += e;
        }
        for (int o = 16; o > 0; o >>= 1)
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = __fdiv_rn(1.0f, sum);
        for (int j = lane; j < cols; j += 32)
            y[j] = __fmul_rn(y[j], inv);
    }
}

int softmax_f32(nncb_context *ctx, const float *in, float *out, size_t rows, int cols, float beta) {
    if (rows == 0)
        return 0;
    if (!in || !out || cols <= 0)
        return fail(-EINVAL, "softmax_f32: bad argument");
    const int grid = stream_grid(ctx, rows * 32, 256);
    softmax_rows_kernel<<<grid, 256, 0, ctx->stream>>>(in, out, rows, cols, beta);
    return after_launch(ctx, "softmax_f32");
}


// ---- reduce_window2d with any of the reference's four reducers, and the other binary operators -------------
// General forms (one thread per output element, channels fastest so that a warp's accesses are contiguous); the
// shapes the benchmark networks use have the specialised kernels above. Arithmetic as stated with the entry
// points in the public header; the output division is the IEEE one.
// OP: 0 mean, 1 min, 2 max, 3 sum (reduce_op_t).
template <int OP>
__global__ void __launch_bounds__(256)
reduce_window2d_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int n, int h, int w, int c, int oh, int ow,
                       int kh, int kw, int sh, int sw, int pt, int pl, int count_include_pad, float si, int zi, float so,
                       float zo) {
    const size_t total = (size_t)n * oh * ow * c;
    const int zq = min(max(zi, 0), 255);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int ch = (int)(i % c);
        const size_t p = i / c;
        const int ox = (int)(p % ow), oy = (int)((p / ow) % oh), b = (int)(p / ((size_t)ow * oh));
        int mx = -1, mn = 256, cnt = 0, sum = 0;
        for (int ky = 0; ky < kh; ky++) {
            const int iy = oy * sh - pt + ky;
            if (iy < 0 || iy >= h)
                continue;
            for (int kx = 0; kx < kw; kx++) {
                const int ix = ox * sw - pl + kx;
                if (ix < 0 || ix >= w)
                    continue;
                const int v = x[(((size_t)b * h + iy) * w + ix) * c + ch];
                mx = max(mx, v), mn = min(mn, v), sum += v, cnt++;
            }
        }
        float r;
        if (OP == 1 || OP == 2) {
            int q = OP == 2 ? mx : mn;
            if (cnt < kh * kw)
                q = OP == 2 ? max(q, zq) : min(q, zq); // a tap outside the image holds the real value 0
            r = dequant_dev((float)q, (float)zi, si);
        } else {
            r = __fmul_rn((float)(sum - cnt * zi), si);
            if (OP == 0)
                r = __fdiv_rn(r, (float)(count_include_pad ? kh * kw : cnt));
        }
        y[i] = (uint8_t)quant_dev(r, so, zo, 0, 255);
    }
}

int reduce_window2d_u8(nncb_context *ctx, int op, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int kh, int kw,
                       int sh, int sw, int pt, int pb, int pl, int pr, int count_include_pad, float si, int32_t zi, float so,
                       int32_t zo) {
    if (n <= 0 || h <= 0 || w <= 0 || c <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || pt < 0 || pb < 0 || pl < 0 ||
        pr < 0)
        return fail(-EINVAL, "reduce_window2d_u8: bad shape");
    if (!(si > 0) || !(so > 0))
        return fail(-EINVAL, "reduce_window2d_u8: scales must be positive");
    if (pt >= kh || pb >= kh || pl >= kw || pr >= kw)
        return fail(-EINVAL, "reduce_window2d_u8: padding as large as the window leaves windows without a tap");
    const int oh = conv_out_size(h, kh, sh, 1, pt, pb), ow = conv_out_size(w, kw, sw, 1, pl, pr);
    if (oh <= 0 || ow <= 0)
        return fail(-EINVAL, "reduce_window2d_u8: empty output");
    const size_t total = (size_t)n * oh * ow * c;
    const int grid = stream_grid(ctx, total, 256);
#define NNCB_RW(OP_)                                                                                                  \
    reduce_window2d_kernel<OP_><<<grid, 256, 0, ctx->stream>>>(x, y, n, h, w, c, oh, ow, kh, kw, sh, sw, pt, pl,      \
                                                               count_include_pad, si, zi, so, (float)zo)
    switch (op) {
    case 0: NNCB_RW(0); break;
    case 1: NNCB_RW(1); break;
    case 2: NNCB_RW(2); break;
    case 3: NNCB_RW(3); break;
    default: return fail(-ENOSYS, "reduce_window2d_u8: reducer %d (0 mean, 1 min, 2 max, 3 sum)", op);
    }
#undef NNCB_RW
    return after_launch(ctx, "reduce_window2d_u8");
}

// OP: 1 sub, 2 mul, 5 min, 6 max (binary_op_t; add has its own kernel)
template <int OP>
__global__ void __launch_bounds__(256)
qbinary_kernel(const uint8_t *__restrict__ a, const uint8_t *__restrict__ b, uint8_t *__restrict__ y, size_t n, float sa,
               float za, float sb, float zb, float so, float zo) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float fa = dequant_dev((float)a[i], za, sa), fb = dequant_dev((float)b[i], zb, sb);
        float r;
        if (OP == 1)
            r = __fsub_rn(fa, fb);
        else if (OP == 2)
            r = __fmul_rn(fa, fb);
        else if (OP == 5)
            r = fa < fb ? fa : fb;
        else
            r = fa > fb ? fa : fb;
        y[i] = (uint8_t)quant_dev(r, so, zo, 0, 255);
    }
}

int qbinary_u8(nncb_context *ctx, int op, const uint8_t *a, const uint8_t *b, uint8_t *y, size_t n, float sa, int32_t za,
               float sb, int32_t zb, float so, int32_t zo) {
    if (op == 0)
        return qadd_u8(ctx, a, b, y, n, sa, za, sb, zb, so, zo);
    if (n == 0)
        return 0;
    if (!a || !b || !y)
        return fail(-EINVAL, "qbinary_u8: null pointer");
    const int grid = stream_grid(ctx, n, 256);
#define NNCB_QB(OP_) qbinary_kernel<OP_><<<grid, 256, 0, ctx->stream>>>(a, b, y, n, sa, (float)za, sb, (float)zb, so, (float)zo)
    switch (op) {
    case 1: NNCB_QB(1); break;
    case 2: NNCB_QB(2); break;
    case 5: NNCB_QB(5); break;
    case 6: NNCB_QB(6); break;
    default: return fail(-ENOSYS, "qbinary_u8: operator %d (0 add, 1 sub, 2 mul, 5 min, 6 max)", op);
    }
#undef NNCB_QB
    return after_launch(ctx, "qbinary_u8");
}

} // namespace nncb
