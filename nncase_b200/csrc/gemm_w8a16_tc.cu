// Small-M weight-only-quantized MatMul on the tensor cores of sm_100a:
//   y[m][n] = (sum_k x[m][k] * w[n][k]) * scale[n] (+ bias[n]) (+ residual[m][n]),   m < M <= 64 tokens
// x f16 [M][K], w i8 [N][K] (per-output-channel symmetric), scale / bias f16 [N], y f16 [M][N]; with swiglu the weight
// rows come in blocks of 16 (the gate rows of 8 outputs, then their up rows) and y has N / 2 columns. Same arithmetic
// as gemv_w8a16 (csrc/decoder_ops.cu: f32 accumulation, then acc * scale + bias in f32, f16 between operators); the
// reference has no such operator (its MatMul is reference/matmul.cpp:28-51 on floats).
//
// At 64 tokens these MatMuls are real GEMMs; the CUDA-core-fed mma.sync form spends its time converting weights and
// fetching activation fragments. Here the 128 output channels of a CTA are the M of a tcgen05.mma kind::f16
// (M 128, N 64 tokens, K 16), the accumulator lives in TMEM, and per 64-wide K block
//   * the load warp brings the i8 weight tile [128][64] (8 KB) and the f16 activation tile [64][64] (8 KB, 128-byte
//     swizzle: it is the MMA's B operand as it lands) with two TMA loads into a ring of stages;
//   * eight warps turn the weight bytes into the f16 A operand [128][64] in 128-byte-swizzled shared memory
//     (exact: (b ^ 0x80) | 0x6400 is the half 1152 + b), one such tile per ring slot;
//   * one thread issues the four MMAs of the block and commits once, which frees the slot.
// After the last block the eight warps read the accumulator (lane = channel, 32 token columns each) and finish.
// Few output channels (qkv, o, down projections: 7 to 9 channel tiles) leave most SMs idle, so K is split over
// CTAs; their f32 partials meet in a per-context workspace and the CTA that arrives last at a tile adds them in
// split order (deterministic) and finishes. Every wait is bounded; no multicast.
// Measured at 64 tokens against the mma.sync form: down projection (896 x 4864) 19.2 -> 14.5 us, LM head
// (151936 x 896) 73 -> 56 us, gate/up with SwiGLU (9728 x 896) 14.3 -> 15 us. What-if builds of the LM head: no
// conversion 53 us, no MMAs 52 us, neither 46 us, and without the epilogue's 2-byte stores 36 us: the tile-per-CTA
// form re-reads the 112 KB of activations once per channel tile (as many bytes as the weights) and stores its
// output in 64-byte pieces; a persistent CTA with resident activations and a staged, 16-byte-per-thread store is
// the next step. Also measured and not kept: a load ring of six slots with two converted tiles, one CTA per SM
// (gate/up 13 us, LM head 82 us: nothing hides a CTA's fill and drain any more), and two MMA-issuing threads with an
// accumulator each, added in the epilogue (no change: the issuing thread is not what paces a K block here).
#include "tc_dev.cuh"
#include <cuda_fp16.h>

namespace nncb {

namespace {

constexpr int GT_STAGES = 3;                   // ring slots: i8 weights 8 KB + f16 activations 8 KB (TMA) and the converted
                                               // f16 weight tile 16 KB of the same K block; two CTAs fit an SM
constexpr int GT_CONV_WARPS = 8;               // conversion warps = epilogue warps (two per TMEM lane quarter: 32 token columns each)
constexpr int GT_THREADS = 32 * (2 + GT_CONV_WARPS);
constexpr uint32_t GT_W8_BYTES = 128 * 64, GT_X_BYTES = 64 * 128, GT_A16_BYTES = 128 * 128;
constexpr uint32_t GT_STAGE_BYTES = GT_W8_BYTES + GT_X_BYTES;
constexpr size_t GT_SMEM = GT_STAGES * (GT_STAGE_BYTES + GT_A16_BYTES) + 1024;
constexpr int GT_MAX_SLOTS = 256;              // (channel tile, K split) pairs with a partial in the workspace
enum { GT_ERR_LOAD = 301, GT_ERR_CONVERT = 302, GT_ERR_MMA = 303, GT_ERR_EPILOGUE = 304 };

struct GtShared {
    uint64_t full[GT_STAGES], a_full[GT_STAGES], freed[GT_STAGES], acc_full;
    uint32_t tmem_slot;
    int last;                // split K: this CTA is the last to arrive at its channel tile
    volatile int abort_flag;
    unsigned wait_limit_us;  // must follow abort_flag (mbar_wait_slow reads it through the flag's address)
};

struct GtArgs {
    const __half *scale, *bias, *residual;
    __half *y;
    float *ws;               // [slots][64][128] f32 partials
    int *cnt;                // [channel tiles], zero between launches
    int *status;
    int M, N, K, k_blocks, kb_per_split, splits, swiglu;
    uint32_t idesc;
    unsigned limit_us;
};

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, dev::Desc a, dev::Desc b, uint32_t idesc, uint32_t accum) {
    asm volatile("{\n.reg .pred p;\n.reg .b64 da, db;\nsetp.ne.b32 p, %6, 0;\n"
                 "mov.b64 da, {%1, %2};\nmov.b64 db, {%3, %4};\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}"
                 ::"r"(tmem_d), "r"(a.lo), "r"(a.hi), "r"(b.lo), "r"(b.hi), "r"(idesc), "r"(accum)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&r)[32]) {
    uint32_t *u = reinterpret_cast<uint32_t *>(r);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 "tcgen05.wait::ld.sync.aligned;"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
                   "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
                   "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
                   "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
                 : "r"(taddr)
                 : "memory");
}
// two signed bytes (byte 2i, 2i + 1 of w) -> half2, exactly
__device__ __forceinline__ uint32_t i8x2_to_half2(uint32_t w, int pair) {
    const uint32_t sel = pair == 0 ? 0x4140u : 0x4342u;
    const uint32_t h = __byte_perm(w ^ 0x80808080u, 0x64646464u, sel);
    const __half2 v = __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ void conv_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * GT_CONV_WARPS) : "memory"); }

__global__ void __launch_bounds__(GT_THREADS, 2)
gemm_w8a16_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const GtArgs a) {
    using namespace dev;
    extern __shared__ uint8_t gt_smem[];
    __shared__ __align__(8) GtShared sh;
    const uint32_t base = (smem_u32(gt_smem) + 1023u) & ~1023u;
    const uint32_t a16_base = base + GT_STAGES * GT_STAGE_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int kb0 = split * a.kb_per_split;
    const int kb1 = min(a.k_blocks, kb0 + a.kb_per_split);
    const int n_blocks = kb1 - kb0; // >= 1 by construction of the grid
    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        sh.wait_limit_us = a.limit_us;
        sh.last = 0;
        for (int s = 0; s < GT_STAGES; s++) {
            mbar_init(smem_u32(&sh.full[s]), 1);
            mbar_init(smem_u32(&sh.a_full[s]), GT_CONV_WARPS);
            mbar_init(smem_u32(&sh.freed[s]), 1); // one commit frees the slot for the load warp and the conversion warps
        }
        mbar_init(smem_u32(&sh.acc_full), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_slot)), "r"(64u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = sh.tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < n_blocks; i++) {
                const int s = i % GT_STAGES;
                if (!mbar_wait(smem_u32(&sh.freed[s]), ((i / GT_STAGES) & 1) ^ 1, &sh.abort_flag, a.status, GT_ERR_LOAD))
                    break;
                const uint32_t full = smem_u32(&sh.full[s]), dst = base + s * GT_STAGE_BYTES;
                mbar_expect_tx(full, GT_STAGE_BYTES);
                tma_load_2d(dst, &tmap_w, full, (kb0 + i) * 64, tile * 128);           // weights [128 channels][64 k] i8
                tma_load_2d(dst + GT_W8_BYTES, &tmap_x, full, (kb0 + i) * 64, 0);      // activations [64 tokens][64 k] f16
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int i = 0; i < n_blocks && ok; i++) {
                const int s = i % GT_STAGES;
                ok = mbar_wait(smem_u32(&sh.a_full[s]), (i / GT_STAGES) & 1, &sh.abort_flag, a.status, GT_ERR_MMA) &&
                     mbar_wait(smem_u32(&sh.full[s]), (i / GT_STAGES) & 1, &sh.abort_flag, a.status, GT_ERR_MMA);
                if (!ok)
                    break;
                fence_after_sync();
                const Desc da = make_desc(smem_desc(a16_base + s * GT_A16_BYTES, 128));
                const Desc db = make_desc(smem_desc(base + s * GT_STAGE_BYTES + GT_W8_BYTES, 128));
                mma_f16(tmem, da, db, a.idesc, i != 0);
                mma_f16(tmem, da + 2, db + 2, a.idesc, 1);
                mma_f16(tmem, da + 4, db + 4, a.idesc, 1);
                mma_f16(tmem, da + 6, db + 6, a.idesc, 1);
                mma_commit(smem_u32(&sh.freed[s])); // the activations, the weight bytes and the converted tile of this slot
            }
            if (ok)
                mma_commit(smem_u32(&sh.acc_full));
        }
    } else {
        // ---- conversion, then the epilogue ----
        const int ct = threadIdx.x - 64; // 0 .. 255
        bool ok = true;
        for (int i = 0; i < n_blocks && ok; i++) {
            const int s = i % GT_STAGES;
            ok = mbar_wait(smem_u32(&sh.full[s]), (i / GT_STAGES) & 1, &sh.abort_flag, a.status, GT_ERR_CONVERT) &&
                 mbar_wait(smem_u32(&sh.freed[s]), ((i / GT_STAGES) & 1) ^ 1, &sh.abort_flag, a.status, GT_ERR_CONVERT);
            if (!ok)
                break;
            const uint32_t src = base + s * GT_STAGE_BYTES, dst = a16_base + s * GT_A16_BYTES;
#pragma unroll
            for (int q0 = 0; q0 < 512 / (32 * GT_CONV_WARPS); q0++) {
                const int q = ct + q0 * 32 * GT_CONV_WARPS; // 16-byte chunk of the i8 tile: row q / 4, bytes 16 (q % 4) ..
                const int row = q >> 2, c16 = q & 3;
                uint32_t w0, w1, w2, w3;
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(src + q * 16));
                const uint32_t d0 = dst + row * 128 + (((2 * c16) ^ (row & 7)) << 4);
                const uint32_t d1 = dst + row * 128 + (((2 * c16 + 1) ^ (row & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(d0), "r"(i8x2_to_half2(w0, 0)), "r"(i8x2_to_half2(w0, 1)),
                             "r"(i8x2_to_half2(w1, 0)), "r"(i8x2_to_half2(w1, 1))
                             : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(d1), "r"(i8x2_to_half2(w2, 0)), "r"(i8x2_to_half2(w2, 1)),
                             "r"(i8x2_to_half2(w3, 0)), "r"(i8x2_to_half2(w3, 1))
                             : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the MMA reads this tile through the async proxy
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&sh.a_full[s]));
        }
        if (ok)
            ok = mbar_wait(smem_u32(&sh.acc_full), 0, &sh.abort_flag, a.status, GT_ERR_EPILOGUE);
        if (ok) {
            fence_after_sync();
            const int quarter = warp & 3;                 // TMEM lanes 32 quarter .. + 31 are this warp's
            const int t0 = ((warp - 2) >> 2) * 32;        // ... and token columns t0 .. t0 + 31
            const int ch = quarter * 32 + lane;           // channel within the tile
            const int n = tile * 128 + ch;
            float v[32];
            tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + t0, v);
            bool finish = true;
            if (a.splits > 1) {
                // partial sums meet in the workspace; the CTA that arrives last at this tile adds them in split order
                float *mine = a.ws + ((size_t)(tile * a.splits + split) * 64 + t0) * 128;
#pragma unroll
                for (int t = 0; t < 32; t++)
                    mine[t * 128 + ch] = v[t];
                __threadfence();
                conv_bar_sync();
                if (ct == 0)
                    sh.last = atomicAdd(&a.cnt[tile], 1) == a.splits - 1;
                conv_bar_sync();
                finish = sh.last != 0;
                if (finish) {
                    __threadfence();
#pragma unroll
                    for (int t = 0; t < 32; t++)
                        v[t] = 0.f;
                    for (int sp = 0; sp < a.splits; sp++) {
                        const float *p = a.ws + ((size_t)(tile * a.splits + sp) * 64 + t0) * 128 + ch;
                        float u[32];
#pragma unroll
                        for (int t = 0; t < 32; t++)
                            u[t] = __ldcg(p + t * 128);
#pragma unroll
                        for (int t = 0; t < 32; t++)
                            v[t] += u[t];
                    }
                    if (ct == 0)
                        a.cnt[tile] = 0;
                }
            }
            if (finish && !a.swiglu && n < a.N) {
                const float sc = __half2float(a.scale[n]), bi = a.bias ? __half2float(a.bias[n]) : 0.f;
#pragma unroll
                for (int t = 0; t < 32; t++) {
                    if (t0 + t >= a.M)
                        break;
                    float r = v[t] * sc + bi;
                    if (a.residual)
                        r += __half2float(a.residual[(size_t)(t0 + t) * a.N + n]);
                    a.y[(size_t)(t0 + t) * a.N + n] = __float2half_rn(r);
                }
            }
            if (finish && a.swiglu) {
                // lanes 0-7 / 16-23 hold gate rows, lanes 8-15 / 24-31 the matching up rows (blocks of 16 rows)
                const bool valid = n < a.N;
                const float sc = valid ? __half2float(a.scale[n]) : 0.f, bi = (valid && a.bias) ? __half2float(a.bias[n]) : 0.f;
                const int out_col = (n >> 4) * 8 + (lane & 7);
#pragma unroll
                for (int t = 0; t < 32; t++) {
                    if (t0 + t >= a.M)
                        break;
                    const float mineh = __half2float(__float2half_rn(v[t] * sc + bi));
                    const float up = __shfl_down_sync(0xffffffffu, mineh, 8);
                    if (valid && (lane & 8) == 0 && n + 8 < a.N)
                        a.y[(size_t)(t0 + t) * (a.N / 2) + out_col] = __float2half_rn(mineh / (1.0f + expf(-mineh)) * up);
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(64u) : "memory");
}

} // namespace

// Matrices of less than 2 M weights (the qkv and o projections of a 0.5 B model) stay on the mma.sync form: a
// launch's fixed costs (set-up, first loads, the partials' round trip) outweigh what the tensor pipe saves there
// (measured at 64 tokens: 6.9 us against 10.8 us). Option matmul.tensor_core = 2 takes every shape that fits.
bool gemm_w8a16_tc_applies(const nncb_context *ctx, int M, int N, int K) {
    if (ctx->d_gemm_ws == nullptr || M < 1 || M > 64 || K % 64 != 0 || K < 64 || N < 16)
        return false;
    return ctx->opt.matmul_tensor_core >= 2 || (long long)N * K >= (1ll << 21);
}

// Launches the tensor-core form (the caller has checked gemm_w8a16_tc_applies and the pointer alignment).
int gemm_w8a16_tc(nncb_context *ctx, const void *x, const int8_t *w, const void *scale, const void *bias, const void *residual,
                  void *y, int M, int N, int K, int swiglu) {
    NNCB_TRY(load_driver_entry_points());
    CUtensorMap tw, tx;
    {
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
        cuuint64_t strides[1] = {(cuuint64_t)K};
        cuuint32_t box[2] = {64, 128}, estr[2] = {1, 1};
        CUresult r = g_encode_tiled(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(w), dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(-EIO, "gemm_w8a16: encoding the weight tensor map failed (CUresult %d)", (int)r);
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
        cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        cuuint32_t box[2] = {64, 64}, estr[2] = {1, 1};
        CUresult r = g_encode_tiled(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x), dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(-EIO, "gemm_w8a16: encoding the activation tensor map failed (CUresult %d)", (int)r);
    }
    GtArgs a;
    a.scale = (const __half *)scale, a.bias = (const __half *)bias, a.residual = (const __half *)residual, a.y = (__half *)y;
    a.ws = ctx->d_gemm_ws;
    a.cnt = reinterpret_cast<int *>(ctx->d_gemm_ws + (size_t)GT_MAX_SLOTS * 64 * 128);
    a.status = ctx->d_status;
    a.M = M, a.N = N, a.K = K, a.k_blocks = K / 64, a.swiglu = swiglu;
    const int tiles = (N + 127) / 128;
    // K split: only where the channel tiles alone leave most SMs idle, and never more partials than the workspace holds
    int splits = 1;
    if (tiles < ctx->sm_count) {
        splits = (2 * ctx->sm_count) / tiles; // two CTAs fit an SM
        if (splits > 4)
            splits = 4; // the last CTA of a tile reads every partial: 32 KB each
        if (splits > a.k_blocks)
            splits = a.k_blocks;
        while (splits > 1 && tiles * splits > GT_MAX_SLOTS)
            splits--;
    }
    a.kb_per_split = (a.k_blocks + splits - 1) / splits;
    a.splits = (a.k_blocks + a.kb_per_split - 1) / a.kb_per_split; // no empty split
    if (tiles > GT_MAX_SLOTS && a.splits > 1)
        a.splits = 1, a.kb_per_split = a.k_blocks;
    a.idesc = (1u << 4) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24); // f16 x f16 -> f32, N 64, M 128
    a.limit_us = ctx->opt.wait_limit_us;
    dim3 grid(tiles, a.splits, 1);
    gemm_w8a16_tc_kernel<<<grid, GT_THREADS, GT_SMEM, ctx->stream>>>(tw, tx, a);
    return after_launch(ctx, "gemm_w8a16_tc");
}

// The dynamic shared-memory limit is a per-device attribute of the kernel: set for the current device when a context
// is created on it.
int gemm_w8a16_tc_set_attributes() {
    NNCB_CUDA_TRY(cudaFuncSetAttribute(gemm_w8a16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM));
    return 0;
}

size_t gemm_w8a16_tc_workspace_bytes() { return (size_t)GT_MAX_SLOTS * 64 * 128 * sizeof(float) + 4096 * sizeof(int); }

} // namespace nncb
