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
// A ring stage holds one or two such K blocks; the two groups of four conversion warps take the stages in turn.
// After the last stage the eight warps read the accumulator (lane = channel, 32 token columns each) and finish.
// Two shapes of launch:
//   * many channel tiles (an LM head): two CTAs per SM, four one-block load stages and two stages of converted
//     tiles each (three and three: LM head 54 -> 52 us), the whole K in one CTA, the result finished from registers;
//   * few channel tiles (the projections of a layer: 7 to 76): K is split over the 2, 4 or 8 CTAs of a thread-block
//     cluster. Every CTA leaves its f32 partial [64 tokens][128 channels] in its own shared memory (the ring is idle
//     by then); after a cluster barrier CTA r finishes token rows 64 r / S .. of the tile, adding the S partials in
//     rank order (deterministic) through distributed shared memory; a second barrier keeps every partial alive
//     until its readers are done. With at most 74 tiles one CTA per SM runs five two-block stages (all the loads
//     of a split in flight at once), otherwise the two-CTA form.
// The load thread sends the first ring-full of loads before the block's first barrier. Every wait is bounded (the
// cluster barriers wait for CTAs whose own waits are bounded); no multicast.
// Measured at 64 tokens, back to back with L2-resident weights (CUDA-core form -> this kernel): qkv projection
// (1152 x 896) 6.9 -> 5.7 us, o (896 x 896) 6.9 -> 5.7, down (896 x 4864) 19.2 -> 9.0, gate/up with SwiGLU
// (9728 x 896) 14.3 -> 10.1, LM head (151936 x 896) 73 -> 55.6 us. An earlier form met the K splits in a global
// workspace, the last CTA of a tile adding the partials: that CTA's serial finish took 3 us (6 us with SwiGLU) of a
// 15 us launch, which is what the cluster form removes. What-if builds of the LM head: no conversion 53 us, no
// MMAs 52 us, neither 46 us, without the epilogue's stores 36 us. Also measured and not kept: a persistent CTA per
// SM with the activations resident and a staged, 16-byte-per-thread store (LM head 58 us, gate/up 15 us: no
// change), the K-split partials pushed into the finishing CTA's shared memory with remote stores so that one
// cluster barrier is enough (qkv 5.5 us, down 7.8 us: no change), the first activation loads sent by the MMA thread
// and the peers' partials fetched in one batch of 16 (no change; the LM head loses 4 us when its first loads wait
// for the block's first barrier), gate/up on three CTAs per SM with two load stages and K split four ways (11.0
// against 9.2 us), the unsplit form's tile stored through shared memory, 16 bytes per thread (LM head 56 against
// 51 us), a load ring of six slots with one CTA per SM for the LM head (82 us: nothing hides a CTA's fill and
// drain), and two MMA-issuing threads with an accumulator each (no change).
#include "tc_dev.cuh"
#include <cuda_fp16.h>

namespace nncb {

namespace {

constexpr int GT_CONV_WARPS = 8;               // conversion warps = epilogue warps (two per TMEM lane quarter: 32 token columns each)
constexpr int GT_THREADS = 32 * (2 + GT_CONV_WARPS);
// One K block of 64: i8 weights [128][64] 8 KB + f16 activations [64][64] 8 KB (TMA) and the converted f16 weight tile 16 KB.
constexpr uint32_t GT_W8_BYTES = 128 * 64, GT_X_BYTES = 64 * 128, GT_A16_BYTES = 128 * 128;
constexpr uint32_t GT_BLOCK_BYTES = GT_W8_BYTES + GT_X_BYTES;
constexpr int GT_MAX_LS = 8;
// A ring stage holds KS K blocks; LS load stages and AS stages of converted tiles.
constexpr size_t gt_smem_bytes(int ks, int ls, int as) { return (size_t)ks * (ls * GT_BLOCK_BYTES + as * GT_A16_BYTES) + 1024; }
enum { GT_ERR_LOAD = 301, GT_ERR_CONVERT = 302, GT_ERR_MMA = 303, GT_ERR_EPILOGUE = 304 };

struct GtShared {
    uint64_t full[GT_MAX_LS], a_full[GT_MAX_LS], freed[GT_MAX_LS], acc_full;
    uint32_t tmem_slot;
    volatile int abort_flag;
    unsigned wait_limit_us;  // must follow abort_flag (mbar_wait_slow reads it through the flag's address)
};

struct GtArgs {
    const __half *scale, *bias, *residual;
    __half *y;
    int *status;
    int M, N, K, k_blocks, kb_per_split, swiglu;
    int cluster;             // > 1: K is split over the CTAs of a cluster (2, 4 or 8), one channel tile per cluster
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
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// the address, in the cluster's shared window, of this CTA's shared-memory location `addr` in CTA `rank`
__device__ __forceinline__ uint32_t peer_smem(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float2 ld_cluster_f32x2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
    return v;
}

template <int KS, int LS, int AS, int CTAS>
__global__ void __launch_bounds__(GT_THREADS, CTAS)
gemm_w8a16_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const GtArgs a) {
    using namespace dev;
    static_assert(LS <= GT_MAX_LS && AS <= LS, "ring sizes");
    constexpr uint32_t STAGE_BYTES = KS * GT_BLOCK_BYTES, A16_STAGE_BYTES = KS * GT_A16_BYTES;
    extern __shared__ uint8_t gt_smem[];
    __shared__ __align__(8) GtShared sh;
    const uint32_t base = (smem_u32(gt_smem) + 1023u) & ~1023u;
    const uint32_t a16_base = base + LS * STAGE_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y; // with a cluster, blockIdx.y is the rank in it (cluster 1 x S x 1, grid y = S)
    const int kb0 = split * a.kb_per_split;
    const int n_blocks = max(min(a.k_blocks, kb0 + a.kb_per_split) - kb0, 0); // 0: a cluster rank past the last K block adds zeros
    const int n_stages = (n_blocks + KS - 1) / KS;
    // the load thread: K blocks of stage st into ring slot s (part 1: the weights, 2: the activations, 3: both)
    auto load_stage = [&](int st, int s, int part) {
        const int nsub = min(KS, n_blocks - st * KS);
        const uint32_t full = smem_u32(&sh.full[s]), dst = base + s * STAGE_BYTES;
        if (part & 1)
            mbar_expect_tx(full, nsub * GT_BLOCK_BYTES);
        for (int u = 0; u < nsub; u++) {
            const int kx = (kb0 + st * KS + u) * 64;
            if (part & 1)
                tma_load_2d(dst + u * GT_BLOCK_BYTES, &tmap_w, full, kx, tile * 128);           // weights [128 channels][64 k] i8
            if (part & 2)
                tma_load_2d(dst + u * GT_BLOCK_BYTES + GT_W8_BYTES, &tmap_x, full, kx, 0);      // activations [64 tokens][64 k] f16
        }
    };
    grid_dependency_release(); // the next kernel of the stream may set itself up while this one runs
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
        sh.abort_flag = 0;
        sh.wait_limit_us = a.limit_us;
        for (int s = 0; s < LS; s++) {
            mbar_init(smem_u32(&sh.full[s]), 1);
            mbar_init(smem_u32(&sh.freed[s]), 1); // one commit frees a stage's load slot and its converted tiles
        }
        for (int s = 0; s < AS; s++)
            mbar_init(smem_u32(&sh.a_full[s]), GT_CONV_WARPS / 2);
        mbar_init(smem_u32(&sh.acc_full), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the weights of the first ring-full leave at once: nothing else has touched these slots, and the weights
        // are nobody's output
        for (int st = 0; st < LS && st < n_stages; st++)
            load_stage(st, st, 1);
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
    // Launched as a programmatic dependent, the kernel has come this far beside the kernel before it in the stream;
    // its activations and residual are that kernel's (or an earlier one's) output, and every bounded wait below
    // starts its clock here.
    grid_dependency_wait();
    if (threadIdx.x == 0)
        for (int st = 0; st < LS && st < n_stages; st++)
            load_stage(st, st, 2);

    const int ct = threadIdx.x - 64; // 0 .. 255 among the conversion / epilogue threads
    bool ok = true;
    if (warp == 0) {
        if (lane == 0) {
            for (int st = LS; st < n_stages; st++) {
                const int s = st % LS;
                if (!mbar_wait(smem_u32(&sh.freed[s]), ((st / LS) & 1) ^ 1, &sh.abort_flag, a.status, GT_ERR_LOAD))
                    break;
                load_stage(st, s, 3);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int st = 0; st < n_stages && ok; st++) {
                const int s = st % LS, sa = st % AS;
                ok = mbar_wait(smem_u32(&sh.a_full[sa]), (st / AS) & 1, &sh.abort_flag, a.status, GT_ERR_MMA) &&
                     mbar_wait(smem_u32(&sh.full[s]), (st / LS) & 1, &sh.abort_flag, a.status, GT_ERR_MMA);
                if (!ok)
                    break;
                fence_after_sync();
                const int nsub = min(KS, n_blocks - st * KS);
                for (int u = 0; u < nsub; u++) {
                    const Desc da = make_desc(smem_desc(a16_base + sa * A16_STAGE_BYTES + u * GT_A16_BYTES, 128));
                    const Desc db = make_desc(smem_desc(base + s * STAGE_BYTES + u * GT_BLOCK_BYTES + GT_W8_BYTES, 128));
                    mma_f16(tmem, da, db, a.idesc, (st | u) != 0);
                    mma_f16(tmem, da + 2, db + 2, a.idesc, 1);
                    mma_f16(tmem, da + 4, db + 4, a.idesc, 1);
                    mma_f16(tmem, da + 6, db + 6, a.idesc, 1);
                }
                mma_commit(smem_u32(&sh.freed[s])); // the activations, the weight bytes and the converted tiles of this stage
            }
            if (ok && n_stages > 0)
                mma_commit(smem_u32(&sh.acc_full));
        }
    } else {
        // ---- conversion: the two groups of four warps take the stages in turn, so that one group's waits and
        // fences overlap the other's loads and stores ----
        const int cgrp = (warp - 2) >> 2, cgt = ct & 127;
        for (int st = cgrp; st < n_stages && ok; st += 2) {
            const int s = st % LS, sa = st % AS;
            ok = mbar_wait(smem_u32(&sh.full[s]), (st / LS) & 1, &sh.abort_flag, a.status, GT_ERR_CONVERT);
            // the slot of the converted tiles is free once the MMAs of stage st - AS have completed: that stage's
            // commit on its load slot. That barrier is at most one phase ahead: the MMAs go in stage order, so no
            // later stage of the slot completes before stage st has been converted.
            if (ok && st >= AS)
                ok = mbar_wait(smem_u32(&sh.freed[(st - AS) % LS]), ((st - AS) / LS) & 1, &sh.abort_flag, a.status, GT_ERR_CONVERT);
            if (!ok)
                break;
            const int nsub = min(KS, n_blocks - st * KS);
            for (int u = 0; u < nsub; u++) {
                const uint32_t src = base + s * STAGE_BYTES + u * GT_BLOCK_BYTES, dst = a16_base + sa * A16_STAGE_BYTES + u * GT_A16_BYTES;
#pragma unroll
                for (int q0 = 0; q0 < 4; q0++) {
                    const int q = cgt + q0 * 128; // 16-byte chunk of the i8 tile: row q / 4, bytes 16 (q % 4) ..
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
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the MMA reads these tiles through the async proxy
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_u32(&sh.a_full[sa]));
        }
        // ---- the accumulator: lane = channel of the tile, 32 token columns per warp ----
        const int quarter = warp & 3;          // TMEM lanes 32 quarter .. + 31 are this warp's
        const int t0 = ((warp - 2) >> 2) * 32; // ... and token columns t0 .. t0 + 31
        const int ch = quarter * 32 + lane;
        const int n = tile * 128 + ch;
        if (a.cluster == 1) {
            // the whole K in this CTA: finish from registers
            const bool valid = n < a.N;
            const float sc = valid ? __half2float(a.scale[n]) : 0.f, bi = (valid && a.bias) ? __half2float(a.bias[n]) : 0.f;
            if (ok)
                ok = mbar_wait(smem_u32(&sh.acc_full), 0, &sh.abort_flag, a.status, GT_ERR_EPILOGUE);
            if (ok) {
                fence_after_sync();
                float v[32];
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + t0, v);
                if (!a.swiglu && valid) {
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
                if (a.swiglu) {
                    // lanes 0-7 / 16-23 hold gate rows, lanes 8-15 / 24-31 the matching up rows (blocks of 16 rows)
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
        } else {
            // K split over the cluster: this CTA's f32 partial [64 tokens][128 channels] goes to its own shared
            // memory (the ring is idle once the accumulator is complete) and is added up after the cluster barrier
            if (ok && n_stages > 0)
                ok = mbar_wait(smem_u32(&sh.acc_full), 0, &sh.abort_flag, a.status, GT_ERR_EPILOGUE);
            float v[32];
            if (ok && n_stages > 0) {
                fence_after_sync();
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + t0, v);
            } else {
#pragma unroll
                for (int t = 0; t < 32; t++)
                    v[t] = 0.f;
            }
#pragma unroll
            for (int t = 0; t < 32; t++)
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(base + (uint32_t)((t0 + t) * 128 + ch) * 4u), "f"(v[t]) : "memory");
        }
    }
    if (a.cluster > 1) {
        __syncwarp(); // the role threads rejoin their warps before the warp-aligned cluster barrier
        cluster_arrive();
        // Token rows 64 / S * rank .. of the tile are this CTA's to finish: the S partials are added in rank order.
        // A thread fetches eight (row, rank) pairs at a time from the peers' shared memory, then finishes those rows.
        const int S = a.cluster, lg = 31 - __clz(S), rows = 64 >> lg, row0 = split * rows;
        const int RB = 8 >> lg; // rows per batch of eight fetches
        if (warp >= 2 && !a.swiglu) {
            // a thread owns two neighbouring channels, 64 threads a token row
            const int c2 = ct & 63, n = tile * 128 + 2 * c2;
            const bool v0 = n < a.N, v1 = n + 1 < a.N, pair = v1 && (a.N & 1) == 0;
            const float sc0 = v0 ? __half2float(a.scale[n]) : 0.f, sc1 = v1 ? __half2float(a.scale[n + 1]) : 0.f;
            const float bi0 = (v0 && a.bias) ? __half2float(a.bias[n]) : 0.f, bi1 = (v1 && a.bias) ? __half2float(a.bias[n + 1]) : 0.f;
            const uint32_t own = base + (uint32_t)(2 * c2) * 4u;
            cluster_wait(); // every partial of the cluster is written
            for (int k0 = 0; k0 < (16 >> lg); k0 += RB) { // this thread's rows: row0 + (ct >> 6) + 4 k
                float2 res[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int t = row0 + (ct >> 6) + 4 * (k0 + j);
                    res[j] = make_float2(0.f, 0.f);
                    if (a.residual && j < RB && t < a.M) {
                        const size_t o = (size_t)t * a.N + n;
                        if (pair)
                            res[j] = __half22float2(*reinterpret_cast<const __half2 *>(a.residual + o));
                        else {
                            res[j].x = v0 ? __half2float(a.residual[o]) : 0.f;
                            res[j].y = v1 ? __half2float(a.residual[o + 1]) : 0.f;
                        }
                    }
                }
                float2 u[8];
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const int t = row0 + (ct >> 6) + 4 * (k0 + (q >> lg));
                    u[q] = ld_cluster_f32x2(peer_smem(own, (uint32_t)(q & (S - 1))) + (uint32_t)t * 512u);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int t = row0 + (ct >> 6) + 4 * (k0 + j);
                    if (j >= RB || t >= a.M)
                        continue;
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        if ((q >> lg) == j)
                            s0 += u[q].x, s1 += u[q].y;
                    float r0 = s0 * sc0 + bi0, r1 = s1 * sc1 + bi1;
                    if (a.residual)
                        r0 += res[j].x, r1 += res[j].y;
                    const size_t o = (size_t)t * a.N + n;
                    if (pair)
                        *reinterpret_cast<__half2 *>(a.y + o) = __halves2half2(__float2half_rn(r0), __float2half_rn(r1));
                    else {
                        if (v0)
                            a.y[o] = __float2half_rn(r0);
                        if (v1)
                            a.y[o + 1] = __float2half_rn(r1);
                    }
                }
            }
        } else if (warp >= 2) {
            // a thread owns outputs 2 o2, 2 o2 + 1 of the tile's 64 (gate rows at channel 16 b + j, their up rows 8
            // further), 32 threads a token row; its rows are row0 + (ct >> 5) + 8 j
            const int o2 = ct & 31, cg = ((2 * o2) >> 3) * 16 + ((2 * o2) & 7), n = tile * 128 + cg;
            const bool valid = n + 9 < a.N;
            float sc[4], bi[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int nn = n + (q & 1) + (q >> 1) * 8;
                sc[q] = valid ? __half2float(a.scale[nn]) : 0.f;
                bi[q] = (valid && a.bias) ? __half2float(a.bias[nn]) : 0.f;
            }
            const uint32_t own = base + (uint32_t)cg * 4u;
            cluster_wait();
            float2 ug[8], uu[8];
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const int t = row0 + (ct >> 5) + 8 * (q >> lg);
                const uint32_t src = peer_smem(own, (uint32_t)(q & (S - 1))) + (uint32_t)t * 512u;
                ug[q] = ld_cluster_f32x2(src), uu[q] = ld_cluster_f32x2(src + 32u);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int t = row0 + (ct >> 5) + 8 * j;
                if (j >= RB || t >= a.M)
                    continue;
                float g0 = 0.f, g1 = 0.f, u0 = 0.f, u1 = 0.f;
#pragma unroll
                for (int q = 0; q < 8; q++)
                    if ((q >> lg) == j)
                        g0 += ug[q].x, g1 += ug[q].y, u0 += uu[q].x, u1 += uu[q].y;
                const float gh0 = __half2float(__float2half_rn(g0 * sc[0] + bi[0])), gh1 = __half2float(__float2half_rn(g1 * sc[1] + bi[1]));
                const float uh0 = __half2float(__float2half_rn(u0 * sc[2] + bi[2])), uh1 = __half2float(__float2half_rn(u1 * sc[3] + bi[3]));
                if (valid)
                    *reinterpret_cast<__half2 *>(a.y + (size_t)t * (a.N / 2) + tile * 64 + 2 * o2) =
                        __halves2half2(__float2half_rn(gh0 / (1.0f + expf(-gh0)) * uh0), __float2half_rn(gh1 / (1.0f + expf(-gh1)) * uh1));
            }
        } else {
            cluster_wait();
        }
        // no CTA leaves while a peer may still read its partial
        __syncwarp();
        cluster_arrive();
        cluster_wait();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(64u) : "memory");
}

} // namespace

#define GT_WIDE 1, 4, 2, 2
#define GT_DEEP 2, 5, 2, 1
constexpr size_t GT_SMEM_WIDE = gt_smem_bytes(1, 4, 2), GT_SMEM_DEEP = gt_smem_bytes(2, 5, 2);

// Where this form is the faster one (measured on the projections of a 0.5 B model and its LM head): more than 32
// tokens -- below that the CUDA-core form streams the weights in 3 to 6 us a projection, less than this kernel's
// set-up, first loads and cluster barriers cost (5 us) -- and at least 128 K weights (measured down to 896 x 256,
// the per-rank projections of eight-way tensor parallelism: 4.6 against 4.7 us; 576 x 896: 4.8 against 6.9 us).
// Option matmul.tensor_core = 2 takes every shape that fits.
bool gemm_w8a16_tc_applies(const nncb_context *ctx, int M, int N, int K) {
    if (M < 1 || M > 64 || K % 64 != 0 || K < 64 || N < 16)
        return false;
    return ctx->opt.matmul_tensor_core >= 2 || (M > 32 && (long long)N * K >= (1ll << 17));
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
    a.status = ctx->d_status;
    a.M = M, a.N = N, a.K = K, a.k_blocks = K / 64, a.swiglu = swiglu;
    const int tiles = (N + 127) / 128;
    // Many channel tiles (an LM head): two CTAs per SM, a short ring each, the whole K in one CTA. Few (the
    // projections of a layer): one CTA per SM with a long ring of two-block stages, and K split over the CTAs of a
    // cluster of 2, 4 or 8 as far as the SMs go.
    const bool deep = 2 * tiles <= ctx->sm_count;
    int cluster = 1;
    for (int c = 8; c > 1; c >>= 1)
        if (tiles * c <= (deep ? 1 : 2) * ctx->sm_count && c <= a.k_blocks) {
            cluster = c;
            break;
        }
    a.cluster = cluster;
    a.kb_per_split = (a.k_blocks + cluster - 1) / cluster;
    a.idesc = (1u << 4) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24); // f16 x f16 -> f32, N 64, M 128
    a.limit_us = ctx->opt.wait_limit_us;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, cluster, 1);
    cfg.blockDim = dim3(GT_THREADS, 1, 1);
    cfg.dynamicSmemBytes = deep ? GT_SMEM_DEEP : GT_SMEM_WIDE;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1, attr[0].val.clusterDim.y = cluster, attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = ctx->opt.launch_overlap ? 2 : 1;
    if (deep)
        NNCB_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_w8a16_tc_kernel<GT_DEEP>, tw, tx, a));
    else
        NNCB_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_w8a16_tc_kernel<GT_WIDE>, tw, tx, a));
    return after_launch(ctx, "gemm_w8a16_tc");
}

// The dynamic shared-memory limit is a per-device attribute of the kernel: set for the current device when a context
// is created on it.
int gemm_w8a16_tc_set_attributes() {
    NNCB_CUDA_TRY(cudaFuncSetAttribute(gemm_w8a16_tc_kernel<GT_WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM_WIDE));
    NNCB_CUDA_TRY(cudaFuncSetAttribute(gemm_w8a16_tc_kernel<GT_DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM_DEEP));
    return 0;
}

} // namespace nncb
