// Paged-attention decode: one query token per sequence against a paged f16 KV cache.
//
// The reference has no attention op; layout and semantics are defined here (the tests restate
// them on the CPU in numpy):
//   q            [B][Hq][64]                      f16
//   k_pool/v_pool [num_pages][Hkv][16][64]         f16, 16-token pages
//   block_table  [B][max_pages]                   int32 page ids, context_lens [B] int32
//   out          [B][Hq][64]                      f16
//   out[b,h] = softmax_t( scale * q[b,h] . K[b, h/(Hq/Hkv), t] ) . V[...]   over t < context_lens[b]
// scores, softmax (max-subtract, exp, sum, multiply by 1/sum as reference/softmax.cpp:30-80) and the
// value sum run in f32.
//
// The kernel is bound by HBM: every K and V byte is read exactly once. One CTA handles one
// (sequence, kv head, split of the context); the Hq/Hkv query heads that share a kv head are
// processed together, so the pages are fetched once for all of them. Each of the four warps owns
// its own pages and its own three-stage cp.async ring (no block barrier in the loop): 32 tokens
// per stage, 16-byte chunks XOR-swizzled so that ldmatrix is conflict-free. The arithmetic
// (0.5 flop per KV byte per head) is done with mma.sync m16n8k16 f16 -> f32 so that instruction
// issue stays far below the memory time: S^T = Q K^T with the heads as M (7 of 16 rows used), the
// softmax row statistics reduced with two warp shuffles across the four lanes that share a head,
// and O += P V with P taken straight from the S accumulator registers, split into a high and a
// low f16 part so that P carries 22 bits.
// With `splits` > 1 partial (max, sum, unnormalised output) triples go to a scratch buffer and a
// second small kernel merges them.
// The ROPE form of the kernel takes the step's unrotated qkv rows instead of q: it rotates the q heads it reads and
// the new token's k ("rotate half", the arithmetic of rope_kv_append_kernel), writes k and v to their page, and --
// when the tile that holds the new token has landed in shared memory -- puts them into the token's row of the tile,
// so the pool write needs no ordering against the loads of the same launch. Its arguments travel in a kernel
// parameter of their own: with them inside PaArgs the compiler gave the plain form 103 registers instead of 128
// and the plain kernel lost 5 % (4.27 against 4.51 TB/s).
#include "internal.cuh"
#include <cuda_fp16.h>

namespace nncb {

constexpr int PA_D = 64, PA_PAGE = 16, PA_STAGES = 3, PA_TOK = 32; // tokens per stage
constexpr int PA_STAGE_BYTES = PA_TOK * PA_D * 2;                                  // K or V of one stage

struct PaArgs {
    const __half *q, *k_pool, *v_pool;
    const int *block_table, *ctx_lens;
    __half *out;
    float *part_o;  // [B][Hq][splits][64]
    float *part_ml; // [B][Hq][splits][2]
    int B, Hq, Hkv, max_pages, splits;
    int num_pages;    // pages in the pools: page ids outside [0, num_pages) are never dereferenced
    int *status;      // the context's status word
    float scale_log2; // scale * log2(e)
};
// Fused rotary embedding and append (the ROPE form of the kernel; PaArgs::q is then unused): qkv
// [B][(Hq + 2 Hkv) * 64] holds this step's unrotated q heads, k heads, v heads; cos_t / sin_t [max_pos][32] f32;
// positions [B].
struct PaRopeArgs {
    const __half *qkv;
    const float *cos_t, *sin_t;
    const int *positions;
    __half *k_pool_w, *v_pool_w;
    int max_pos;
};
enum { PA_ERR_BAD_INDEX = 202 };

__device__ __forceinline__ uint32_t pa_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    const int sz = valid ? 16 : 0; // zero-fill when the row lies beyond the context
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

// byte offset of 16-byte chunk `c` (0..7) of token row `r` (0..31) inside a stage tile
__device__ __forceinline__ uint32_t pa_off(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

// PA_WARPS warps per CTA (4: two CTAs per SM, context splits fill the machine; 8: one CTA per SM takes a
// whole context -- no partials, no merge launch -- when there are enough (sequence, kv head) pairs).
template <int PA_WARPS, bool ROPE>
__global__ void __launch_bounds__(PA_WARPS * 32)
paged_attention_decode_kernel(const PaArgs a, const PaRopeArgs ra) {
    extern __shared__ __align__(128) uint8_t pa_smem_raw[];
    grid_dependency_release(); // the output projection that follows sets itself up and fetches its weights meanwhile
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = a.Hq / a.Hkv;
    // Lengths and page ids come from device memory the caller filled. A length is clamped to what the
    // block-table row can describe; a page id outside the pools reads as zeros (the zero-fill path of
    // rows beyond the context); both record PA_ERR_BAD_INDEX in the context's status word.
    int ctx = a.ctx_lens[b];
    if (ctx < 0 || ctx > a.max_pages * PA_PAGE) {
        if (threadIdx.x == 0)
            atomicCAS(a.status, 0, (int)PA_ERR_BAD_INDEX);
        ctx = ctx < 0 ? 0 : a.max_pages * PA_PAGE;
    }
    const int n_pages = (ctx + PA_PAGE - 1) / PA_PAGE;
    const int pages_per_split = (n_pages + a.splits - 1) / a.splits;
    const int p_begin = split * pages_per_split;
    const int p_end = min(n_pages, p_begin + pages_per_split);
    const int *table = a.block_table + (size_t)b * a.max_pages;

    // stage ring of this warp: [stage][K | V]
    uint8_t *ring = pa_smem_raw + (size_t)warp * PA_STAGES * 2 * PA_STAGE_BYTES;
    const uint32_t ring_s = pa_smem(ring);

    // Q as the A operand (rows = heads of the group, rows >= group are zero)
    uint32_t qa[4][2];
    if (!ROPE) {
        const bool hv = g < group;
        const __half *qrow = a.q + ((size_t)b * a.Hq + kvh * group + (hv ? g : 0)) * PA_D;
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            qa[ks][0] = hv ? *reinterpret_cast<const uint32_t *>(qrow + ks * 16 + 2 * t) : 0u;
            qa[ks][1] = hv ? *reinterpret_cast<const uint32_t *>(qrow + ks * 16 + 8 + 2 * t) : 0u;
        }
    }

    // 32-token units of this split, dealt round-robin to the warps
    const int n_units = (p_end > p_begin) ? (p_end - p_begin + 1) / 2 : 0;
    const int my_units = (n_units > warp) ? (n_units - warp + PA_WARPS - 1) / PA_WARPS : 0;

    auto issue = [&](int u, int stage) {
        // unit u of this warp -> pages p_begin + 2*(warp + 4u) and the next one
        const int page0 = p_begin + 2 * (warp + PA_WARPS * u);
        const uint32_t ks = ring_s + stage * 2 * PA_STAGE_BYTES, vs = ks + PA_STAGE_BYTES;
        const int c = lane & 7;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int r = (lane >> 3) + 4 * j; // token row 0..31
            const int page = page0 + (r >> 4);
            bool valid = page < p_end && page * PA_PAGE + (r & 15) < ctx;
            int pid = valid ? table[page] : 0;
            if (pid < 0 || pid >= a.num_pages) {
                atomicCAS(a.status, 0, (int)PA_ERR_BAD_INDEX);
                valid = false, pid = 0;
            }
            const size_t off = (((size_t)pid * a.Hkv + kvh) * PA_PAGE + (r & 15)) * PA_D + c * 8;
            cp_async16(ks + pa_off(r, c), a.k_pool + off, valid);
            cp_async16(vs + pa_off(r, c), a.v_pool + off, valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float m_run = -INFINITY, l_run = 0.f; // head g: running max (log2 domain) and this lane's partial sum
    float o[8][4];
#pragma unroll
    for (int n = 0; n < 8; n++)
        o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    for (int u = 0; u < PA_STAGES - 1; u++) {
        if (u < my_units)
            issue(u, u);
        else
            asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // Fused rotary embedding and append: this step's q, k, v arrive unrotated. Rotation pairs dimension i with
    // i + 32 ("rotate half"): out[i] = x[i] cos - x[i+32] sin, out[i+32] = x[i+32] cos + x[i] sin, rounded to f16 --
    // the same arithmetic, in the same order, as rope_kv_append_kernel (csrc/decoder_ops.cu). It runs here, behind
    // the first page loads, so that its chain of dependent reads hides in their flight.
    int new_u = -1, new_row = 0;  // the warp's unit that holds the new token, and the token's row in it
    uint32_t new_k = 0u, new_v = 0u; // dims 2 lane, 2 lane + 1 of the new token's rotated k and its v
    if (ROPE) {
        // Launched as a programmatic dependent of the qkv MatMul: the page loads above read nothing that kernel
        // writes and are in flight while it finishes; its output is first touched here.
        grid_dependency_wait();
        int pos = ra.positions[b];
        const bool pos_ok = pos >= 0 && pos < ra.max_pos && pos / PA_PAGE < a.max_pages;
        if (!pos_ok) {
            if (threadIdx.x == 0)
                atomicCAS(a.status, 0, (int)PA_ERR_BAD_INDEX);
            pos = 0;
        }
        const size_t row_stride = (size_t)(a.Hq + 2 * a.Hkv) * PA_D;
        const float *cs = ra.cos_t + (size_t)pos * 32, *sn = ra.sin_t + (size_t)pos * 32;
        {
            const bool hv = g < group;
            const __half *qrow = ra.qkv + (size_t)b * row_stride + (size_t)(kvh * group + (hv ? g : 0)) * PA_D;
            // this lane's dims: 16 ks + 8 j + 2 t + e; the partner of ks < 2 is ks + 2 of the same (j, e)
#pragma unroll
            for (int kl = 0; kl < 2; kl++) {
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int i = kl * 16 + 8 * j + 2 * t; // index into the cos / sin row (even)
                    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(qrow + i));
                    const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(qrow + i + 32));
                    const float2 c = *reinterpret_cast<const float2 *>(cs + i), sv = *reinterpret_cast<const float2 *>(sn + i);
                    const float l0 = lo.x * c.x - hi.x * sv.x, l1 = lo.y * c.y - hi.y * sv.y;
                    const float h0 = hi.x * c.x + lo.x * sv.x, h1 = hi.y * c.y + lo.y * sv.y;
                    qa[kl][j] = hv ? pack_half2(l0, l1) : 0u;
                    qa[kl + 2][j] = hv ? pack_half2(h0, h1) : 0u;
                }
            }
        }
        // The new token's k (rotated) and v belong in page block_table[b][pos / 16], slot pos % 16. The warp whose
        // unit holds that page writes them to the pool and keeps them: when the unit's tile has landed it puts them
        // into the token's row of the tile itself, so the pool write needs no ordering against this launch's loads.
        const int new_page = pos / PA_PAGE;
        if (pos_ok && new_page >= p_begin && new_page < p_end) {
            const int uu = (new_page - p_begin) >> 1;
            if (uu % PA_WARPS == warp) {
                const int d = 2 * lane, i = d & 31;
                const __half *krow = ra.qkv + (size_t)b * row_stride + (size_t)(a.Hq + kvh) * PA_D;
                const __half *vrow = krow + (size_t)a.Hkv * PA_D;
                const float2 x = __half22float2(*reinterpret_cast<const __half2 *>(krow + d));
                const float2 other = __half22float2(*reinterpret_cast<const __half2 *>(krow + (d < 32 ? d + 32 : d - 32)));
                const float2 c = *reinterpret_cast<const float2 *>(cs + i), sv = *reinterpret_cast<const float2 *>(sn + i);
                const float o0 = d < 32 ? x.x * c.x - other.x * sv.x : x.x * c.x + other.x * sv.x;
                const float o1 = d < 32 ? x.y * c.y - other.y * sv.y : x.y * c.y + other.y * sv.y;
                new_k = pack_half2(o0, o1);
                new_v = *reinterpret_cast<const uint32_t *>(vrow + d);
                const int pid = table[new_page];
                if (pid < 0 || pid >= a.num_pages) {
                    atomicCAS(a.status, 0, (int)PA_ERR_BAD_INDEX); // reads as zeros below, like any bad page
                } else {
                    const size_t off = (((size_t)pid * a.Hkv + kvh) * PA_PAGE + (pos % PA_PAGE)) * PA_D + d;
                    *reinterpret_cast<uint32_t *>(ra.k_pool_w + off) = new_k;
                    *reinterpret_cast<uint32_t *>(ra.v_pool_w + off) = new_v;
                    new_u = uu / PA_WARPS;
                    new_row = pos - (p_begin + 2 * uu) * PA_PAGE;
                }
            }
        } else if (pos_ok && split == 0 && threadIdx.x == 0 && new_page >= n_pages) {
            atomicCAS(a.status, 0, (int)PA_ERR_BAD_INDEX); // the context length does not cover the new token
        }
    }
    for (int u = 0; u < my_units; u++) {
        if (u + PA_STAGES - 1 < my_units)
            issue(u + PA_STAGES - 1, (u + PA_STAGES - 1) % PA_STAGES);
        else
            asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(PA_STAGES - 1) : "memory");
        __syncwarp();
        const int stage = u % PA_STAGES;
        const uint32_t ks = ring_s + stage * 2 * PA_STAGE_BYTES, vs = ks + PA_STAGE_BYTES;
        const int tok0 = (p_begin + 2 * (warp + PA_WARPS * u)) * PA_PAGE; // first token of this unit
        if (ROPE && u == new_u) {
            // the new token's row of the tile: what the pool holds from now on, whatever the load saw
            const uint32_t off = pa_off(new_row, lane >> 2) + (uint32_t)(lane & 3) * 4u;
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(ks + off), "r"(new_k) : "memory");
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(vs + off), "r"(new_v) : "memory");
            __syncwarp();
        }
        const int tok_end = min(ctx, p_end * PA_PAGE);                    // tokens beyond belong to nobody or to the next split

        // ---- S^T = Q K^T : 4 n-tiles of 8 tokens, 4 k-steps of 16 dims ----
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kp = 0; kp < 2; kp++) {
                // matrices: dims chunk 4kp+0 .. 4kp+3 of tokens 8j..8j+7 -> (b0,b1) of k-steps 2kp, 2kp+1
                uint32_t b0, b1, b2, b3;
                const int r = 8 * j + (lane & 7), c = 4 * kp + (lane >> 3);
                ldsm_x4(ks + pa_off(r, c), b0, b1, b2, b3);
                mma16816(s[j], qa[2 * kp][0], 0u, qa[2 * kp][1], 0u, b0, b1);
                mma16816(s[j], qa[2 * kp + 1][0], 0u, qa[2 * kp + 1][1], 0u, b2, b3);
            }
        }
        // ---- online softmax for head g (values s[j][0], s[j][1] = tokens 8j+2t, 8j+2t+1) ----
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int tok = tok0 + 8 * j + 2 * t + e;
                s[j][e] = tok < tok_end ? s[j][e] * a.scale_log2 : -INFINITY;
                mx = fmaxf(mx, s[j][e]);
            }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        // every unit holds at least one token of the context, so m_new is finite
        const float alpha = exp2f(m_run - m_new);
        m_run = m_new;
        float psum = 0.f;
        uint32_t ph[4], pl[4]; // P as f16 high and low parts, A-operand order
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float p0 = exp2f(s[j][0] - m_new), p1 = exp2f(s[j][1] - m_new);
            psum += p0 + p1;
            const __half2 hi = __floats2half2_rn(p0, p1);
            const float2 hif = __half22float2(hi);
            ph[j] = *reinterpret_cast<const uint32_t *>(&hi);
            pl[j] = pack_half2(p0 - hif.x, p1 - hif.y);
        }
        l_run = l_run * alpha + psum;
#pragma unroll
        for (int n = 0; n < 8; n++) {
            o[n][0] *= alpha;
            o[n][1] *= alpha;
        }
        // ---- O += P V : 2 k-steps of 16 tokens, 8 n-tiles of 8 dims ----
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
#pragma unroll
            for (int np = 0; np < 4; np++) {
                // matrices: (tokens 16kk..+7, dims chunk 2np), (tokens +8.., 2np), (tokens .., 2np+1), (tokens +8, 2np+1)
                uint32_t b0, b1, b2, b3;
                const int r = 16 * kk + ((lane >> 3) & 1) * 8 + (lane & 7), c = 2 * np + (lane >> 4);
                ldsm_x4_t(vs + pa_off(r, c), b0, b1, b2, b3);
                mma16816(o[2 * np], ph[2 * kk], 0u, ph[2 * kk + 1], 0u, b0, b1);
                mma16816(o[2 * np], pl[2 * kk], 0u, pl[2 * kk + 1], 0u, b0, b1);
                mma16816(o[2 * np + 1], ph[2 * kk], 0u, ph[2 * kk + 1], 0u, b2, b3);
                mma16816(o[2 * np + 1], pl[2 * kk], 0u, pl[2 * kk + 1], 0u, b2, b3);
            }
        }
        __syncwarp();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

    // ---- merge the four warps through shared memory (reusing the rings) ----
    __syncthreads();
    float *mrg_m = reinterpret_cast<float *>(pa_smem_raw);       // [warp][8]
    float *mrg_l = mrg_m + PA_WARPS * 8;                         // [warp][8]
    float *mrg_o = mrg_l + PA_WARPS * 8;                         // [warp][8][64]
    if (t == 0) {
        mrg_m[warp * 8 + g] = m_run;
        mrg_l[warp * 8 + g] = l_run;
    }
#pragma unroll
    for (int n = 0; n < 8; n++) {
        mrg_o[(warp * 8 + g) * PA_D + 8 * n + 2 * t] = o[n][0];
        mrg_o[(warp * 8 + g) * PA_D + 8 * n + 2 * t + 1] = o[n][1];
    }
    __syncthreads();
    // item = (head, four dims): head = item / 16, dims 4 * (item % 16) ..
    for (int item = threadIdx.x; item < 8 * 16; item += PA_WARPS * 32) {
        const int h = item >> 4, d0 = (item & 15) * 4;
        if (h >= group)
            continue;
        float M = -INFINITY;
        for (int w = 0; w < PA_WARPS; w++)
            M = fmaxf(M, mrg_m[w * 8 + h]);
        float L = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int w = 0; w < PA_WARPS; w++) {
            const float mw = mrg_m[w * 8 + h];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
            L += mrg_l[w * 8 + h] * f;
            for (int i = 0; i < 4; i++)
                acc[i] += mrg_o[(w * 8 + h) * PA_D + d0 + i] * f;
        }
        const int hq = kvh * group + h;
        if (a.splits == 1) {
            const float inv = L > 0.f ? 1.0f / L : 0.f; // empty context -> zeros
            __half2 *dst = reinterpret_cast<__half2 *>(a.out + ((size_t)b * a.Hq + hq) * PA_D + d0);
            dst[0] = __floats2half2_rn(acc[0] * inv, acc[1] * inv);
            dst[1] = __floats2half2_rn(acc[2] * inv, acc[3] * inv);
        } else {
            const size_t pi = ((size_t)b * a.Hq + hq) * a.splits + split;
            *reinterpret_cast<float4 *>(a.part_o + pi * PA_D + d0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            if ((item & 15) == 0) {
                a.part_ml[pi * 2] = M;
                a.part_ml[pi * 2 + 1] = L;
            }
        }
    }
}

// merges the per-split partial results: one block of 64 threads per (sequence, head)
__global__ void __launch_bounds__(64)
paged_attention_merge_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml, __half *__restrict__ out,
                             int splits) {
    grid_dependency_release();
    const size_t bh = blockIdx.x;
    const int d = threadIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < splits; s++)
        M = fmaxf(M, part_ml[(bh * splits + s) * 2]);
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < splits; s++) {
        const float ms = part_ml[(bh * splits + s) * 2];
        const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
        L += part_ml[(bh * splits + s) * 2 + 1] * f;
        acc += part_o[(bh * splits + s) * PA_D + d] * f;
    }
    out[bh * PA_D + d] = __float2half_rn(L > 0.f ? acc * (1.0f / L) : 0.f);
}

size_t paged_attention_scratch_bytes(int B, int Hq, int splits) {
    return splits <= 1 ? 0 : (size_t)B * Hq * splits * (PA_D + 2) * sizeof(float);
}

// Eight-warp CTAs (one per SM) once the (sequence, kv head) pairs alone fill half the SMs; four-warp CTAs
// (two per SM) with context splits below that.
static int paged_attention_pick_warps(const nncb_context *ctx, int B, int Hkv) {
    if (ctx->opt.attention_warps) // tuning override: force the CTA width (4 or 8)
        return ctx->opt.attention_warps == 8 ? 8 : 4;
    return 2 * B * Hkv >= ctx->sm_count ? 8 : 4;
}

int paged_attention_pick_splits(const nncb_context *ctx, int B, int Hkv, int max_ctx) {
    // Split the context so that the grid fills the CTA slots in ONE wave -- a second, partly filled wave
    // costs a full pass -- but keep at least 8 pages (4 units) per CTA.
    const int warps = paged_attention_pick_warps(ctx, B, Hkv);
    const int per_sm = (int)((227u * 1024u) / ((size_t)warps * PA_STAGES * 2 * PA_STAGE_BYTES + 1024));
    const int ctas = B * Hkv, slots = (per_sm > 16 ? 16 : per_sm) * ctx->sm_count;
    int s = slots / ctas;
    const int pages = (max_ctx + PA_PAGE - 1) / PA_PAGE;
    const int cap = pages / 8 > 1 ? pages / 8 : 1;
    if (s > cap)
        s = cap;
    if (s > 16)
        s = 16;
    if (ctx->opt.attention_splits) // tuning override: force the split count
        s = ctx->opt.attention_splits;
    return s < 1 ? 1 : s;
}

int paged_attention_check(int B, int Hq, int Hkv, int head_dim, int page_size, int max_pages) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || max_pages <= 0)
        return fail(-EINVAL, "paged_attention: non-positive dimension");
    if (head_dim != PA_D || page_size != PA_PAGE)
        return fail(-ENOSYS, "paged_attention: only head_dim 64 and 16-token pages are built");
    if (Hq % Hkv != 0 || Hq / Hkv > 8)
        return fail(-ENOSYS, "paged_attention: query heads per kv head must divide evenly and be at most 8");
    return 0;
}

int paged_attention_set_attributes() {
    NNCB_CUDA_TRY(cudaFuncSetAttribute(paged_attention_decode_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       4 * PA_STAGES * 2 * PA_STAGE_BYTES));
    NNCB_CUDA_TRY(cudaFuncSetAttribute(paged_attention_decode_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       8 * PA_STAGES * 2 * PA_STAGE_BYTES));
    NNCB_CUDA_TRY(cudaFuncSetAttribute(paged_attention_decode_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       4 * PA_STAGES * 2 * PA_STAGE_BYTES));
    NNCB_CUDA_TRY(cudaFuncSetAttribute(paged_attention_decode_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       8 * PA_STAGES * 2 * PA_STAGE_BYTES));
    return 0;
}

// Launches on ctx->stream. scratch: at least paged_attention_scratch_bytes(B, Hq, splits) bytes when splits > 1.
int paged_attention_launch(nncb_context *ctx, const void *q, const void *k_pool, const void *v_pool,
                           const int32_t *block_table, const int32_t *ctx_lens, void *out, int B, int Hq, int Hkv,
                           int max_pages, int num_pages, float scale, int splits, void *scratch, const PaRope *rope) {
    if (num_pages <= 0)
        return fail(-EINVAL, "paged_attention: num_pages must be positive");
    PaArgs a;
    PaRopeArgs ra = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0};
    if (rope) {
        ra.qkv = (const __half *)rope->qkv, ra.cos_t = rope->cos_t, ra.sin_t = rope->sin_t, ra.positions = rope->positions;
        ra.k_pool_w = (__half *)const_cast<void *>(k_pool), ra.v_pool_w = (__half *)const_cast<void *>(v_pool);
        ra.max_pos = rope->max_pos;
    }
    a.num_pages = num_pages, a.status = ctx->d_status;
    a.q = (const __half *)q, a.k_pool = (const __half *)k_pool, a.v_pool = (const __half *)v_pool;
    a.block_table = block_table, a.ctx_lens = ctx_lens, a.out = (__half *)out;
    a.B = B, a.Hq = Hq, a.Hkv = Hkv, a.max_pages = max_pages, a.splits = splits;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.part_o = (float *)scratch;
    a.part_ml = a.part_o ? a.part_o + (size_t)B * Hq * splits * PA_D : nullptr;
    const int warps = paged_attention_pick_warps(ctx, B, Hkv);
    const size_t smem = (size_t)warps * PA_STAGES * 2 * PA_STAGE_BYTES; // 96 KB or 192 KB
    dim3 grid(splits, Hkv, B);
    if (warps == 8 && rope)
        NNCB_CUDA_TRY(launch_dependent(ctx, paged_attention_decode_kernel<8, true>, grid, dim3(8 * 32), smem, a, ra));
    else if (warps == 8)
        paged_attention_decode_kernel<8, false><<<grid, 8 * 32, smem, ctx->stream>>>(a, ra);
    else if (rope)
        NNCB_CUDA_TRY(launch_dependent(ctx, paged_attention_decode_kernel<4, true>, grid, dim3(4 * 32), smem, a, ra));
    else
        paged_attention_decode_kernel<4, false><<<grid, 4 * 32, smem, ctx->stream>>>(a, ra);
    NNCB_TRY(after_launch(ctx, "paged_attention_decode"));
    if (splits > 1) {
        paged_attention_merge_kernel<<<B * Hq, 64, 0, ctx->stream>>>(a.part_o, a.part_ml, a.out, splits);
        NNCB_TRY(after_launch(ctx, "paged_attention_merge"));
    }
    return 0;
}

// ---- variant that allocates nothing -----------------------------------------------------------
// Scratch for the split partials lives in this fixed device array instead of caller memory. Every
// GPU that loads the library holds it until the process exits.
constexpr size_t PA_STATIC_SCRATCH_BYTES = 768u << 10; // 768 KiB
static __device__ __align__(256) unsigned char pa_static_scratch[PA_STATIC_SCRATCH_BYTES];

size_t paged_attention_static_capacity() { return PA_STATIC_SCRATCH_BYTES; }

// Device address of the array on `device`. In host code the array's name is only a handle, not
// a device pointer, so the address is asked from the runtime once per device, with that device
// current, and remembered.
int paged_attention_static_scratch(int device, void **ptr) {
    constexpr int MAX_DEV = 64;
    static void *cached[MAX_DEV] = {nullptr};
    if (device < 0 || device >= MAX_DEV)
        return fail(-EINVAL, "paged_attention (static scratch): device %d out of range", device);
    if (!cached[device]) {
        int cur = -1;
        NNCB_CUDA_TRY(cudaGetDevice(&cur));
        if (cur != device)
            return fail(-EINVAL, "paged_attention (static scratch): device %d is not current", device);
        void *p = nullptr;
        NNCB_CUDA_TRY(cudaGetSymbolAddress(&p, pa_static_scratch));
        cached[device] = p;
    }
    *ptr = cached[device];
    return 0;
}

} // namespace nncb
