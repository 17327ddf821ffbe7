// Decode-step kernels of a Qwen2-shaped transformer with i8 weights and f16 activations:
// small-M weight-only-quantized MatMul, RMSNorm (optionally fused with the residual add), rotary
// embedding + KV-page append, SwiGLU, embedding gather. The reference has none of these
// operators (its op list is src/Native/include/nncase/kernels/stackvm/tensor_ops.h:29-479);
// arithmetic follows its mat_mul convention (f32 accumulation, reference/matmul.cpp:28-51) with
// f16 storage between operators.
//
// At batch 64 every one of these is tiny next to the KV-cache read of the attention kernel: a
// layer's weights are 15 MB (2.3 us of HBM time), so the design goal here is few launches that keep
// many loads in flight and capture into one CUDA graph, not peak tensor throughput.
#include "internal.cuh"
#include <cuda_fp16.h>

namespace nncb {

// ---- y[m][n] = (sum_k x[m][k] * w[n][k]) * scale[n] (+ bias[n]) (+ residual[m][n]) ---------------
// x f16 [M<=64][K], w i8 [N][K] (per-output-channel symmetric), scale f16 [N], y f16 [M][N].
// Weight-bandwidth bound: every weight byte is read once, the activations (at most 64 x K f16) are
// staged in shared memory once per CTA and reused for all the output channels the CTA walks
// (persistent loop over channel blocks; K beyond the shared-memory chunk is streamed chunk by chunk).
// Tensor-core math: mma.sync m16n8k16 f16 with the weights as A (converted i8 -> f16 in registers) and
// x^T as B. Inside a 64-wide K chunk the k index is permuted (lane t of a row owns bytes 16t..16t+15)
// so that every lane fetches its weights with one 16-byte load per row and its activations with
// 8-byte shared-memory loads (row pitch = 8 mod 128 bytes: conflict-free); a dot product does not
// care about the order of k. The next chunk's weights are in flight while the current one is
// multiplied. Two warp arrangements: G = 8, every warp owns 16 channels of a 128-channel block and
// walks all of K (no reduction; layers with many output channels); G = 1, the eight warps share 16
// channels and split K, reducing through shared memory (few output channels: more CTAs, more loads
// in flight).
constexpr int GEMV_WARPS = 8;

__device__ __forceinline__ void mma16816_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// two signed bytes (byte 2i, 2i+1 of w, i = 0 or 1) -> half2, exactly
__device__ __forceinline__ uint32_t i8x2_to_half2(uint32_t w, int pair) {
    // (b ^ 0x80) | 0x6400 is the half 1024 + (b + 128); subtracting 1152 gives b
    const uint32_t sel = pair == 0 ? 0x4140u : 0x4342u; // bytes {b0, 0x64, b1, 0x64} / {b2, 0x64, b3, 0x64}
    const uint32_t h = __byte_perm(w ^ 0x80808080u, 0x64646464u, sel);
    const __half2 v = __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<const uint32_t *>(&v);
}

// SwiGLU folded into the MatMul's epilogue (swiglu != 0): the weight rows come in blocks of 16 = the gate
// rows of 8 outputs followed by their up rows, y has n / 2 columns and
// y[m][8 * block + r] = f16(silu(f16(gate)) * f16(up)) -- the gate/up activations never go to memory.
struct GemvFusion {
    int swiglu;
};

constexpr int GEMV_KC_MAX = 1280; // largest K chunk of activations held in shared memory (64 x 1280 f16 = 160 KB)

template <int MT, int G> // MT token tiles of 8; G channel groups per CTA (8 or 1)
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_w8a16_kernel(const __half *__restrict__ x, const int8_t *__restrict__ w, const __half *__restrict__ scale,
                  const __half *__restrict__ bias, const __half *__restrict__ residual, __half *__restrict__ y, int M,
                  int N, int K, int KC, float *__restrict__ split_ws, int *__restrict__ split_cnt, const GemvFusion fu) {
    // split_ws != null (G == 1 only): gridDim.y CTAs share a channel block, each taking one K chunk of KC;
    // partial sums meet in split_ws ([block][K chunk][16][64] f32) and the CTA that arrives last (split_cnt,
    // zero between launches) adds them in chunk order, finishes the block and clears the counter.
    extern __shared__ __align__(16) uint8_t gemv_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int pitch = KC * 2 + 8; // bytes per token row
    float(*red)[16][MT * 8 + 1] = reinterpret_cast<float(*)[16][MT * 8 + 1]>(gemv_smem + (size_t)MT * 8 * pitch);
    const int nblk = (N + 16 * G - 1) / (16 * G);
    const bool split = G == 1 && split_ws != nullptr;
    const int k_begin = split ? (int)blockIdx.y * KC : 0, k_end = split ? min(K, k_begin + KC) : K;
    const bool resident = split || K <= KC;

    auto stage_x = [&](int kc0, int len) {
        const int per_row = len / 8; // 16-byte pieces
        for (int idx = threadIdx.x; idx < MT * 8 * per_row; idx += GEMV_WARPS * 32) {
            const int tok = idx / per_row, c8 = idx % per_row;
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)min(tok, M - 1) * K + kc0) + c8);
            uint2 *dst = reinterpret_cast<uint2 *>(gemv_smem + (size_t)tok * pitch + c8 * 16);
            dst[0] = make_uint2(v.x, v.y);
            dst[1] = make_uint2(v.z, v.w);
        }
    };
    if (resident) {
        stage_x(k_begin, k_end - k_begin);
        __syncthreads();
    }
    for (int blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
        float acc[MT][4];
#pragma unroll
        for (int i = 0; i < MT; i++)
            acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        const int n0 = blk * 16 * G + (G == 1 ? 0 : warp * 16);
        const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1); // clamped rows of a partial last block
        const int8_t *w0 = w + (size_t)r0 * K + 16 * t, *w1 = w + (size_t)r1 * K + 16 * t;
        for (int kc0 = k_begin; kc0 < k_end; kc0 += KC) {
            const int len = min(KC, k_end - kc0);
            if (!resident) {
                __syncthreads(); // the previous chunk has been consumed
                stage_x(kc0, len);
                __syncthreads();
            }
            const int chunks = len / 64;
            const int c_first = G == 1 ? warp : 0, c_step = G == 1 ? GEMV_WARPS : 1;
            // PF chunks of weights are in flight per warp (1 KB each): the loop is a stream of dependent
            // loads otherwise, one memory latency per chunk
            constexpr int PF = 4;
            uint4 pa[PF], pb[PF];
#pragma unroll
            for (int p = 0; p < PF; p++) {
                const int c = c_first + p * c_step;
                pa[p] = pb[p] = make_uint4(0, 0, 0, 0);
                if (c < chunks) {
                    pa[p] = __ldg(reinterpret_cast<const uint4 *>(w0 + kc0 + c * 64));
                    pb[p] = __ldg(reinterpret_cast<const uint4 *>(w1 + kc0 + c * 64));
                }
            }
            for (int ch0 = c_first; ch0 < chunks; ch0 += PF * c_step) {
#pragma unroll
                for (int p = 0; p < PF; p++) {
                    const int ch = ch0 + p * c_step;
                    if (ch >= chunks)
                        break;
                    const uint4 wa = pa[p], wb = pb[p];
                    const int nxt = ch + PF * c_step;
                    if (nxt < chunks) {
                        pa[p] = __ldg(reinterpret_cast<const uint4 *>(w0 + kc0 + nxt * 64));
                        pb[p] = __ldg(reinterpret_cast<const uint4 *>(w1 + kc0 + nxt * 64));
                    }
                    const uint32_t wav[4] = {wa.x, wa.y, wa.z, wa.w}, wbv[4] = {wb.x, wb.y, wb.z, wb.w};
                    const uint8_t *xrow = gemv_smem + (size_t)g * pitch + (ch * 64 + 16 * t) * 2;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint32_t a0 = i8x2_to_half2(wav[j], 0), a2 = i8x2_to_half2(wav[j], 1);
                        const uint32_t a1 = i8x2_to_half2(wbv[j], 0), a3 = i8x2_to_half2(wbv[j], 1);
#pragma unroll
                        for (int i = 0; i < MT; i++) {
                            const uint2 bfrag = *reinterpret_cast<const uint2 *>(xrow + (size_t)(8 * i) * pitch + 8 * j);
                            mma16816_f16(acc[i], a0, a1, a2, a3, bfrag.x, bfrag.y);
                        }
                    }
                }
            }
        }
        if (G == 1) {
#pragma unroll
            for (int i = 0; i < MT; i++) {
                red[warp][g][8 * i + 2 * t] = acc[i][0];
                red[warp][g][8 * i + 2 * t + 1] = acc[i][1];
                red[warp][g + 8][8 * i + 2 * t] = acc[i][2];
                red[warp][g + 8][8 * i + 2 * t + 1] = acc[i][3];
            }
            __syncthreads();
            bool finish = true;
            if (split) {
                // publish this CTA's K slice in its own slot, then see whether every slice of the block has
                // arrived (slots instead of atomic adds: the sum below has a fixed order)
                float *ws = split_ws + ((size_t)blk * gridDim.y + blockIdx.y) * 16 * 64;
                for (int idx = threadIdx.x; idx < MT * 8 * 16; idx += GEMV_WARPS * 32) {
                    const int tok = idx / 16, r = idx % 16;
                    float s = 0.f;
#pragma unroll
                    for (int wv = 0; wv < GEMV_WARPS; wv++)
                        s += red[wv][r][tok];
                    ws[r * 64 + tok] = s;
                }
                __shared__ int s_last;
                __threadfence();
                __syncthreads();
                if (threadIdx.x == 0)
                    s_last = atomicAdd(split_cnt + blk, 1) == (int)gridDim.y - 1;
                __syncthreads();
                finish = s_last != 0;
                if (finish)
                    __threadfence();
            }
            // thread -> (token, channel)
            for (int idx = threadIdx.x; finish && idx < MT * 8 * 16; idx += GEMV_WARPS * 32) {
                const int tok = idx / 16, r = idx % 16;
                const int n = n0 + r;
                float s = 0.f;
                if (split) {
                    const float *cell = split_ws + (size_t)blk * gridDim.y * 16 * 64 + r * 64 + tok;
                    for (int ks = 0; ks < (int)gridDim.y; ks++)
                        s += __ldcg(cell + (size_t)ks * 16 * 64);
                } else {
#pragma unroll
                    for (int wv = 0; wv < GEMV_WARPS; wv++)
                        s += red[wv][r][tok];
                }
                if (tok >= M || n >= N)
                    continue;
                float v = s * __half2float(scale[n]);
                if (bias)
                    v += __half2float(bias[n]);
                if (fu.swiglu) {
                    // rows 0..7 of the block are gates, 8..15 the matching ups: pair them through shared memory
                    red[0][r][tok] = __half2float(__float2half_rn(v));
                    continue;
                }
                if (residual)
                    v += __half2float(residual[(size_t)tok * N + n]);
                y[(size_t)tok * N + n] = __float2half_rn(v);
            }
            if (fu.swiglu && finish) {
                __syncthreads();
                for (int idx = threadIdx.x; idx < MT * 8 * 8; idx += GEMV_WARPS * 32) {
                    const int tok = idx / 8, r = idx % 8;
                    if (tok >= M || n0 + r + 8 >= N)
                        continue;
                    const float gt = red[0][r][tok], up = red[0][r + 8][tok];
                    y[(size_t)tok * (N / 2) + blk * 8 + r] = __float2half_rn(gt / (1.0f + expf(-gt)) * up);
                }
            }
            if (split && finish && threadIdx.x == 0)
                split_cnt[blk] = 0;
            __syncthreads(); // red is reused by the next block
        } else {
            // this warp's 16 channels x all tokens: accumulator (row = channel g / g + 8, column = token 2t, 2t + 1)
            if (fu.swiglu) {
                // accumulator rows g (gate) and g + 8 (up) of this warp's 16-row block belong to one output
                const int ng = n0 + g, nu = n0 + g + 8;
                if (nu < N) {
                    const float sg_ = __half2float(scale[ng]), su = __half2float(scale[nu]);
                    const float bg = bias ? __half2float(bias[ng]) : 0.f, bu = bias ? __half2float(bias[nu]) : 0.f;
#pragma unroll
                    for (int i = 0; i < MT; i++)
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const int tok = 8 * i + 2 * t + e;
                            if (tok >= M)
                                continue;
                            const float gt = __half2float(__float2half_rn(acc[i][e] * sg_ + bg));
                            const float up = __half2float(__float2half_rn(acc[i][2 + e] * su + bu));
                            y[(size_t)tok * (N / 2) + (n0 >> 1) + g] = __float2half_rn(gt / (1.0f + expf(-gt)) * up);
                        }
                }
                continue;
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int n = n0 + g + 8 * h;
                if (n >= N)
                    continue;
                const float sc = __half2float(scale[n]), bi = bias ? __half2float(bias[n]) : 0.f;
#pragma unroll
                for (int i = 0; i < MT; i++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int tok = 8 * i + 2 * t + e;
                        if (tok >= M)
                            continue;
                        float v = acc[i][2 * h + e] * sc + bi;
                        if (residual)
                            v += __half2float(residual[(size_t)tok * N + n]);
                        y[(size_t)tok * N + n] = __float2half_rn(v);
                    }
            }
        }
    }
}

static int gemv_w8a16_fused(nncb_context *ctx, const void *x, const int8_t *w, const void *scale, const void *bias,
                            const void *residual, void *y, int M, int N, int K, const GemvFusion &fu);

int gemv_w8a16(nncb_context *ctx, const void *x, const int8_t *w, const void *scale, const void *bias,
               const void *residual, void *y, int M, int N, int K) {
    GemvFusion fu = {0};
    return gemv_w8a16_fused(ctx, x, w, scale, bias, residual, y, M, N, K, fu);
}

int gemv_w8a16_swiglu(nncb_context *ctx, const void *x, const int8_t *w, const void *scale, const void *bias, void *y,
                      int M, int N, int K) {
    if (N % 16 != 0)
        return fail(-EINVAL, "gemv_w8a16_swiglu: gate/up rows come in blocks of 16");
    GemvFusion fu = {1};
    return gemv_w8a16_fused(ctx, x, w, scale, bias, nullptr, y, M, N, K, fu);
}

static int gemv_w8a16_fused(nncb_context *ctx, const void *x, const int8_t *w, const void *scale, const void *bias,
                            const void *residual, void *y, int M, int N, int K, const GemvFusion &fu) {
    if (M <= 0 || N <= 0 || K <= 0)
        return fail(-EINVAL, "gemv_w8a16: non-positive dimension");
    if (M > 64)
        return fail(-ENOSYS, "gemv_w8a16: built for at most 64 rows of activations (decode batches)");
    if (K % 64 != 0)
        return fail(-ENOSYS, "gemv_w8a16: K must be a multiple of 64");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15)
        return fail(-EINVAL, "gemv_w8a16: x and w must be 16-byte aligned");
    if (ctx->opt.matmul_tensor_core && gemm_w8a16_tc_applies(ctx, M, N, K))
        return gemm_w8a16_tc(ctx, x, w, scale, bias, residual, y, M, N, K, fu.swiglu);
    const __half *xs = (const __half *)x, *sc = (const __half *)scale, *bi = (const __half *)bias,
                 *re = (const __half *)residual;
    __half *ys = (__half *)y;
    const int mt = (M + 7) / 8, mtt = mt <= 1 ? 1 : (mt <= 2 ? 2 : (mt <= 4 ? 4 : 8));
    const int KC = K <= GEMV_KC_MAX ? K : 1024;
    // many output channels: each warp owns 16 of them; few: the warps split K so that more CTAs carry loads
    const bool wide = N >= 2048;
    const int nblk = (N + (wide ? 127 : 15)) / (wide ? 128 : 16);
    size_t smem = (size_t)mtt * 8 * (KC * 2 + 8);
    if (!wide)
        smem += sizeof(float) * GEMV_WARPS * 16 * (mtt * 8 + 1);
    const int per_sm = (int)((227u * 1024u) / (smem + 1024));
    const int slots = (per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm)) * ctx->sm_count;
    // A long K with few output channels (the down projection): the K chunks go to different CTAs, which
    // meet in the context's f32 workspace; otherwise one CTA per channel block walks K itself.
    const int k_splits = (K + KC - 1) / KC;
    const bool split = !wide && k_splits > 1 && nblk * k_splits <= GEMV_SPLIT_SLOTS && ctx->d_gemv_ws != nullptr;
    dim3 grid(nblk < slots ? nblk : slots, 1, 1);
    float *ws = nullptr;
    int *cnt = nullptr;
    if (split) {
        grid = dim3(nblk, k_splits, 1);
        ws = ctx->d_gemv_ws;
        cnt = reinterpret_cast<int *>(ctx->d_gemv_ws + (size_t)GEMV_SPLIT_SLOTS * 16 * 64);
    }
#define NNCB_GEMV(MT_, G_)                                                                                            \
    do {                                                                                                              \
        gemv_w8a16_kernel<MT_, G_><<<grid, GEMV_WARPS * 32, smem, ctx->stream>>>(xs, w, sc, bi, re, ys, M, N, K, KC, ws, cnt, fu);  \
    } while (0)
    switch (mtt * 2 + (wide ? 1 : 0)) {
    case 2: NNCB_GEMV(1, 1); break;
    case 3: NNCB_GEMV(1, 8); break;
    case 4: NNCB_GEMV(2, 1); break;
    case 5: NNCB_GEMV(2, 8); break;
    case 8: NNCB_GEMV(4, 1); break;
    case 9: NNCB_GEMV(4, 8); break;
    case 16: NNCB_GEMV(8, 1); break;
    default: NNCB_GEMV(8, 8); break;
    }
#undef NNCB_GEMV
    return after_launch(ctx, "gemv_w8a16");
}

int gemv_set_attributes() {
#define NNCB_GEMV_ATTR(MT_, G_)                                                                                       \
    NNCB_CUDA_TRY(cudaFuncSetAttribute(gemv_w8a16_kernel<MT_, G_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024))
    NNCB_GEMV_ATTR(1, 1);
    NNCB_GEMV_ATTR(1, 8);
    NNCB_GEMV_ATTR(2, 1);
    NNCB_GEMV_ATTR(2, 8);
    NNCB_GEMV_ATTR(4, 1);
    NNCB_GEMV_ATTR(4, 8);
    NNCB_GEMV_ATTR(8, 1);
    NNCB_GEMV_ATTR(8, 8);
#undef NNCB_GEMV_ATTR
    return 0;
}

// ---- RMSNorm, optionally fused with the residual add ---------------------------------------------
//   if delta: x <- f16(x + delta)  (written back);  h = f16( x * rsqrt(mean(x^2) + eps) * w )
// one CTA of 128 threads per row; f32 statistics.
// The row stays in registers between the statistics and the scaling (one read of x and delta); rows longer
// than 128 x 16 elements take the general kernel below.
__global__ void __launch_bounds__(128)
add_rmsnorm_row_kernel(__half *__restrict__ x, const __half *__restrict__ delta, const __half *__restrict__ w,
                       __half *__restrict__ h, int cols, float eps) {
    __shared__ float part[4];
    grid_dependency_wait();    // launched as a programmatic dependent: x and delta are earlier kernels' output
    grid_dependency_release(); // a MatMul that follows sets itself up and fetches its weights meanwhile
    const size_t row = blockIdx.x;
    uint2 *xr = reinterpret_cast<uint2 *>(x + row * cols);
    const uint2 *dr = reinterpret_cast<const uint2 *>(delta + row * cols);
    const int pieces = cols / 4; // 8-byte pieces, at most 4 per thread
    uint2 v[4];
    float ss = 0.f;
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const int pc = threadIdx.x + 128 * q;
        v[q] = make_uint2(0, 0);
        if (pc < pieces) {
            v[q] = xr[pc];
            __half2 *hv = reinterpret_cast<__half2 *>(&v[q]);
            if (delta) {
                const uint2 d = __ldg(dr + pc);
                const __half2 *dv = reinterpret_cast<const __half2 *>(&d);
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const float2 a = __half22float2(hv[e]), b2 = __half22float2(dv[e]);
                    hv[e] = __floats2half2_rn(a.x + b2.x, a.y + b2.y);
                }
                xr[pc] = v[q];
            }
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float2 a = __half22float2(hv[e]);
                ss += a.x * a.x + a.y * a.y;
            }
        }
    }
    for (int o = 16; o > 0; o >>= 1)
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0)
        part[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float inv = rsqrtf((part[0] + part[1] + part[2] + part[3]) / (float)cols + eps);
    uint2 *hr = reinterpret_cast<uint2 *>(h + row * cols);
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const int pc = threadIdx.x + 128 * q;
        if (pc < pieces) {
            const uint2 gm = __ldg(reinterpret_cast<const uint2 *>(w) + pc);
            const __half2 *hv = reinterpret_cast<const __half2 *>(&v[q]), *gv = reinterpret_cast<const __half2 *>(&gm);
            uint2 o2;
            __half2 *ov = reinterpret_cast<__half2 *>(&o2);
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float2 a = __half22float2(hv[e]), gg = __half22float2(gv[e]);
                ov[e] = __floats2half2_rn(a.x * inv * gg.x, a.y * inv * gg.y);
            }
            hr[pc] = o2;
        }
    }
}

__global__ void __launch_bounds__(128)
add_rmsnorm_kernel(__half *__restrict__ x, const __half *__restrict__ delta, const __half *__restrict__ w,
                   __half *__restrict__ h, int cols, float eps) {
    __shared__ float part[4];
    grid_dependency_release();
    const size_t row = blockIdx.x;
    __half *xr = x + row * cols;
    float ss = 0.f;
    for (int j = threadIdx.x; j < cols; j += 128) {
        float v = __half2float(xr[j]);
        if (delta) {
            v = __half2float(__float2half_rn(v + __half2float(delta[row * cols + j])));
            xr[j] = __float2half_rn(v);
        }
        ss += v * v;
    }
    for (int o = 16; o > 0; o >>= 1)
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0)
        part[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float tot = part[0] + part[1] + part[2] + part[3];
    const float inv = rsqrtf(tot / (float)cols + eps);
    for (int j = threadIdx.x; j < cols; j += 128)
        h[row * cols + j] = __float2half_rn(__half2float(xr[j]) * inv * __half2float(w[j]));
}

int add_rmsnorm_f16(nncb_context *ctx, void *x, const void *delta, const void *w, void *h, int rows, int cols, float eps) {
    if (rows <= 0 || cols <= 0)
        return fail(-EINVAL, "rmsnorm: non-positive dimension");
    const bool al8 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(w) |
                       reinterpret_cast<uintptr_t>(h)) & 7) == 0;
    if (cols % 4 == 0 && cols <= 2048 && al8)
        NNCB_CUDA_TRY(launch_dependent(ctx, add_rmsnorm_row_kernel, dim3(rows), dim3(128), 0, (__half *)x, (const __half *)delta,
                                       (const __half *)w, (__half *)h, cols, eps));
    else
        add_rmsnorm_kernel<<<rows, 128, 0, ctx->stream>>>((__half *)x, (const __half *)delta, (const __half *)w, (__half *)h,
                                                           cols, eps);
    return after_launch(ctx, "add_rmsnorm");
}

// ---- all-reduce over peer memory, fused with the residual add and RMSNorm -------------------------
// Tensor-parallel ranks (one process per GPU) each hold a partial [rows][cols] f16 of a row-split projection in a
// buffer the other ranks have mapped (CUDA IPC). This kernel is the whole exchange:
//   delta = f16( sum over ranks, in rank order, of the partials in f32 )      -- every rank adds in the same order
//   x <- f16(x + delta);  h = f16( x * rsqrt(mean(x^2) + eps) * w )            -- as add_rmsnorm_row_kernel
// It starts after this rank's MatMul (stream order), so block 0 first tells every peer that this rank's partial of
// sequence number `seq` is complete (a release store into the peer's flag block); every block then waits -- bounded --
// until its own flag block shows `seq` from every peer, and reads the peers' rows with L2-coherent loads over NVLink.
// Flag block of a rank (32 unsigned, zeroed once): flag[slot][source rank] at 8 * slot + source, the sequence number
// of the rank's last finished launch per slot at 16 + slot, its count of finished blocks at 18 + slot. Two slots
// alternate (o projection, down projection): a rank can reach its next write of a slot only after every peer has
// finished reading the previous contents (the peers' flags for the launch in between are sent after those reads).
enum { ERR_PEER_WAIT = 401 };
struct PeerArgs {
    const __half *part[8]; // rank r's partial (own: local memory; others: peer mappings)
    unsigned *flags[8];    // rank r's flag block
    int world, rank, slot;
    unsigned limit_us;
};
__global__ void __launch_bounds__(128)
peer_allreduce_add_rmsnorm_kernel(__half *__restrict__ x, const PeerArgs pa, const __half *__restrict__ w, __half *__restrict__ h,
                                  int cols, float eps, int *status) {
    __shared__ float part[4];
    __shared__ int s_ok;
    grid_dependency_wait();    // launched as a programmatic dependent of the MatMul that writes this rank's partial
    grid_dependency_release();
    unsigned *mine = pa.flags[pa.rank];
    if (threadIdx.x == 0) {
        const unsigned seq = *reinterpret_cast<volatile unsigned *>(mine + 16 + pa.slot) + 1u;
        if (blockIdx.x == 0) {
            __threadfence_system();
            for (int p = 0; p < pa.world; p++)
                if (p != pa.rank)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pa.flags[p] + 8 * pa.slot + pa.rank), "r"(seq) : "memory");
        }
        // an earlier give-up on this context is not waited for again
        bool ok = *reinterpret_cast<volatile int *>(status) == 0;
        unsigned long long t0 = 0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (int p = 0; p < pa.world && ok; p++) {
            if (p == pa.rank)
                continue;
            const unsigned *f = mine + 8 * pa.slot + p;
            for (unsigned spin = 0;; spin++) {
                unsigned v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                if ((int)(v - seq) >= 0)
                    break;
                if ((spin & 63u) == 63u) {
                    unsigned long long t1;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                    if (t1 - t0 > (unsigned long long)pa.limit_us * 1000ull) {
                        atomicCAS(status, 0, (int)ERR_PEER_WAIT);
                        ok = false;
                        break;
                    }
                }
            }
        }
        s_ok = ok ? 1 : 0;
        part[0] = __uint_as_float(seq);
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    const unsigned seq = __float_as_uint(part[0]);
    __syncthreads();
    const size_t row = blockIdx.x;
    uint2 *xr = reinterpret_cast<uint2 *>(x + row * cols);
    const int pieces = cols / 4; // 8-byte pieces, at most 4 per thread
    uint2 v[4];
    float ss = 0.f;
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const int pc = threadIdx.x + 128 * q;
        v[q] = make_uint2(0, 0);
        if (pc < pieces) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int p = 0; p < pa.world; p++) {
                if (!ok && p != pa.rank)
                    continue; // a peer that never answered is not read
                const uint2 d = __ldcg(reinterpret_cast<const uint2 *>(pa.part[p] + row * cols) + pc);
                const __half2 *dv = reinterpret_cast<const __half2 *>(&d);
                const float2 a0 = __half22float2(dv[0]), a1 = __half22float2(dv[1]);
                acc[0] += a0.x, acc[1] += a0.y, acc[2] += a1.x, acc[3] += a1.y;
            }
            v[q] = xr[pc];
            __half2 *hv = reinterpret_cast<__half2 *>(&v[q]);
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float2 a = __half22float2(hv[e]);
                const float2 b2 = __half22float2(__floats2half2_rn(acc[2 * e], acc[2 * e + 1])); // the all-reduced f16 value
                hv[e] = __floats2half2_rn(a.x + b2.x, a.y + b2.y);
            }
            xr[pc] = v[q];
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float2 a = __half22float2(hv[e]);
                ss += a.x * a.x + a.y * a.y;
            }
        }
    }
    for (int o = 16; o > 0; o >>= 1)
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0)
        part[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float inv = rsqrtf((part[0] + part[1] + part[2] + part[3]) / (float)cols + eps);
    uint2 *hr = reinterpret_cast<uint2 *>(h + row * cols);
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const int pc = threadIdx.x + 128 * q;
        if (pc < pieces) {
            const uint2 gm = __ldg(reinterpret_cast<const uint2 *>(w) + pc);
            const __half2 *hv = reinterpret_cast<const __half2 *>(&v[q]), *gv = reinterpret_cast<const __half2 *>(&gm);
            uint2 o2;
            __half2 *ov = reinterpret_cast<__half2 *>(&o2);
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float2 a = __half22float2(hv[e]), gg = __half22float2(gv[e]);
                ov[e] = __floats2half2_rn(a.x * inv * gg.x, a.y * inv * gg.y);
            }
            hr[pc] = o2;
        }
    }
    // the last block to finish publishes the sequence number for the next launch on this slot
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(mine + 18 + pa.slot, 1u) == gridDim.x - 1) {
            mine[18 + pa.slot] = 0u;
            *reinterpret_cast<volatile unsigned *>(mine + 16 + pa.slot) = seq;
        }
    }
}

int peer_allreduce_add_rmsnorm_f16(nncb_context *ctx, void *x, const void *const *partials, void *const *flags, int world, int rank,
                                   int slot, const void *w, void *h, int rows, int cols, float eps) {
    if (rows <= 0 || cols <= 0)
        return fail(-EINVAL, "peer_allreduce_add_rmsnorm: non-positive dimension");
    if (world < 2 || world > 8 || rank < 0 || rank >= world || slot < 0 || slot > 1)
        return fail(-EINVAL, "peer_allreduce_add_rmsnorm: world must be 2..8, rank inside it, slot 0 or 1");
    if (cols % 4 != 0 || cols > 2048)
        return fail(-ENOSYS, "peer_allreduce_add_rmsnorm: rows of up to 2048 elements, a multiple of 4, are built");
    PeerArgs pa;
    uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(h);
    for (int p = 0; p < 8; p++) {
        pa.part[p] = p < world ? (const __half *)partials[p] : nullptr;
        pa.flags[p] = p < world ? (unsigned *)flags[p] : nullptr;
        if (p < world && (!partials[p] || !flags[p]))
            return fail(-EINVAL, "peer_allreduce_add_rmsnorm: null buffer for rank %d", p);
        bits |= reinterpret_cast<uintptr_t>(pa.part[p]);
    }
    if (bits & 7)
        return fail(-EINVAL, "peer_allreduce_add_rmsnorm: pointers must be 8-byte aligned");
    pa.world = world, pa.rank = rank, pa.slot = slot, pa.limit_us = ctx->opt.peer_wait_limit_us;
    NNCB_CUDA_TRY(launch_dependent(ctx, peer_allreduce_add_rmsnorm_kernel, dim3(rows), dim3(128), 0, (__half *)x, pa, (const __half *)w,
                                   (__half *)h, cols, eps, ctx->d_status));
    return after_launch(ctx, "peer_allreduce_add_rmsnorm");
}

// ---- rotary embedding of q and k, and append of k, v to the paged cache --------------------------
// qkv [B][(Hq + 2 Hkv) * 64] f16 (q heads, then k heads, then v heads). Rotation pairs dimension i
// with i + 32 ("rotate half"): out[i] = x[i] cos - x[i+32] sin, out[i+32] = x[i+32] cos + x[i] sin,
// cos/sin from a host table [max_pos][32] f32. Rotated q goes to q_out [B][Hq][64] (dense, the layout
// the attention kernel reads); k (rotated) and v go to page block_table[b][pos / 16], slot pos % 16.
// Positions and page ids come from device memory the caller filled: a position outside [0, max_pos) or
// beyond the block-table row, or a page id outside [0, num_pages), stores nothing for that sequence and
// records ERR_BAD_INDEX in the context's status word (nncb_check_device_status reports it).
enum { ERR_BAD_INDEX = 201 };
__global__ void __launch_bounds__(64)
rope_kv_append_kernel(const __half *__restrict__ qkv, __half *__restrict__ q_out, const float *__restrict__ cos_t,
                      const float *__restrict__ sin_t,
                      const int *__restrict__ positions, const int *__restrict__ block_table, __half *__restrict__ k_pool,
                      __half *__restrict__ v_pool, int Hq, int Hkv, int max_pages, int max_pos, int num_pages, int *status) {
    const int b = blockIdx.y, head = blockIdx.x; // heads 0..Hq-1: q; Hq..Hq+Hkv-1: k; then v
    const int d = threadIdx.x;                   // 0..63
    const int pos = positions[b];
    if (pos < 0 || pos >= max_pos || pos / 16 >= max_pages) {
        if (d == 0)
            atomicCAS(status, 0, ERR_BAD_INDEX);
        return;
    }
    const __half *row = qkv + (size_t)b * (Hq + 2 * Hkv) * 64 + (size_t)head * 64;
    const bool is_v = head >= Hq + Hkv;
    float out;
    const float xv = __half2float(row[d]);
    if (is_v) {
        out = xv;
    } else {
        const int i = d & 31;
        const float c = cos_t[(size_t)pos * 32 + i], s = sin_t[(size_t)pos * 32 + i];
        const float other = __half2float(row[d < 32 ? d + 32 : d - 32]);
        out = d < 32 ? xv * c - other * s : xv * c + other * s;
    }
    const __half ho = __float2half_rn(out);
    if (head < Hq) {
        q_out[((size_t)b * Hq + head) * 64 + d] = ho;
    } else {
        const int kvh = is_v ? head - Hq - Hkv : head - Hq;
        const int page = block_table[(size_t)b * max_pages + pos / 16];
        if (page < 0 || page >= num_pages) {
            if (d == 0)
                atomicCAS(status, 0, ERR_BAD_INDEX);
            return;
        }
        __half *dst = (is_v ? v_pool : k_pool) + (((size_t)page * Hkv + kvh) * 16 + (pos % 16)) * 64;
        dst[d] = ho;
    }
}

int rope_kv_append_f16(nncb_context *ctx, const void *qkv, void *q_out, const float *cos_t, const float *sin_t, const int32_t *positions,
                       const int32_t *block_table, void *k_pool, void *v_pool, int B, int Hq, int Hkv, int head_dim,
                       int page_size, int max_pages, int max_pos, int num_pages) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || max_pages <= 0 || max_pos <= 0 || num_pages <= 0)
        return fail(-EINVAL, "rope_kv_append: non-positive dimension");
    if (head_dim != 64 || page_size != 16)
        return fail(-ENOSYS, "rope_kv_append: only head_dim 64 and 16-token pages are built");
    dim3 grid(Hq + 2 * Hkv, B);
    rope_kv_append_kernel<<<grid, 64, 0, ctx->stream>>>((const __half *)qkv, (__half *)q_out, cos_t, sin_t, positions, block_table,
                                                       (__half *)k_pool, (__half *)v_pool, Hq, Hkv, max_pages, max_pos,
                                                       num_pages, ctx->d_status);
    return after_launch(ctx, "rope_kv_append");
}

// ---- SwiGLU: out[m][j] = silu(gu[m][j]) * gu[m][inter + j], f32 math -------------------------------
__global__ void __launch_bounds__(256)
swiglu_kernel(const __half *__restrict__ gu, __half *__restrict__ out, size_t rows, int inter) {
    const size_t total = rows * inter;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / inter, j = i % inter;
        const float g = __half2float(gu[r * 2 * inter + j]), u = __half2float(gu[r * 2 * inter + inter + j]);
        out[i] = __float2half_rn(g / (1.0f + expf(-g)) * u);
    }
}

int swiglu_f16(nncb_context *ctx, const void *gu, void *out, int rows, int inter) {
    if (rows <= 0 || inter <= 0)
        return fail(-EINVAL, "swiglu: non-positive dimension");
    const size_t total = (size_t)rows * inter;
    int grid = (int)((total + 255) / 256);
    if (grid > ctx->sm_count * 8)
        grid = ctx->sm_count * 8;
    swiglu_kernel<<<grid, 256, 0, ctx->stream>>>((const __half *)gu, (__half *)out, (size_t)rows, inter);
    return after_launch(ctx, "swiglu");
}

// ---- embedding gather: out[m][:] = table[ids[m]][:] -----------------------------------------------
__global__ void __launch_bounds__(128)
embedding_kernel(const __half *__restrict__ table, const int *__restrict__ ids, __half *__restrict__ out, int cols,
                 int vocab) {
    const int id = min(max(ids[blockIdx.x], 0), vocab - 1);
    const uint32_t *src = reinterpret_cast<const uint32_t *>(table + (size_t)id * cols);
    uint32_t *dst = reinterpret_cast<uint32_t *>(out + (size_t)blockIdx.x * cols);
    for (int j = threadIdx.x; j < cols / 2; j += 128)
        dst[j] = src[j];
}

int embedding_f16(nncb_context *ctx, const void *table, const int32_t *ids, void *out, int rows, int cols, int vocab) {
    if (rows <= 0 || cols <= 0 || vocab <= 0 || (cols & 1))
        return fail(-EINVAL, "embedding: bad dimension");
    embedding_kernel<<<rows, 128, 0, ctx->stream>>>((const __half *)table, ids, (__half *)out, cols, vocab);
    return after_launch(ctx, "embedding");
}

} // namespace nncb
