// Shared declarations of the nncase_b200 CUDA library (host side + small device helpers).
#pragma once
#include <cerrno>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cuda_runtime.h>
#include <string>

#include "../../include/nncase_b200.h"

// Per-context options (nncb_context_set_option). They stand in for the reference's interpreter
// options_dict (src/Native/src/runtime/interpreter.cpp:29-31): tuning overrides and the limit of
// kernel-internal waits. 0 = let the library choose.
struct nncb_options {
    int conv_tile_n = 0;        // force the N tile of the tensor-core convolution (128, 96, 64, 48 or 32)
    int conv_mma_issuers = 0;   // force the number of MMA-issuing warps of the tensor-core convolution (1 or 2)
    int conv_load_warps = 0;    // force its load warps (1; 2: activations and weights apart; 3: two, stages in turn)
    int conv_wide_patch = 1;    // 0: keep 64-/128-channel stride-1 layers on the im2col form
    int conv_add_table = 0;     // fused residual add of the tensor-core convolution: 2: the float chain on packed arithmetic instead of the byte-pair table (same bits, measured slower)
    int depthwise_dot = 1;      // 0: the multiply-add form of the 3x3 depthwise kernel
    int attention_warps = 0;    // force the CTA width of paged attention (4 or 8)
    int attention_splits = 0;   // force its number of context splits
    unsigned wait_limit_us = 1000000; // kernel-internal waits give up after this long
    unsigned peer_wait_limit_us = 30000000; // ... and waits for another rank's flag (ranks start their steps at different times) after this long
    int matmul_tensor_core = 1; // w8a16 MatMul on tcgen05: 0 never, 1 for matrices of 2 M weights or more, 2 wherever it fits
    int launch_overlap = 1;     // tensor-core convolutions are launched as programmatic dependents of their predecessor
    int debug_withhold_load = 0; // self-test of the give-up path: the convolution's producer leaves out one load
};

struct nncb_context {
    nncb_options opt;
    int device = 0;
    cudaStream_t stream = nullptr;
    uint64_t launches = 0;
    int sm_count = 148;
    int *d_status = nullptr;  // device word: 0 ok, else code of the first bounded wait that gave up
    float *d_gemv_ws = nullptr; // split-K meeting place of gemv_w8a16: GEMV_SPLIT_SLOTS x 16 x 64 f32 + one counter per slot, counters zero between launches
};

namespace nncb {

constexpr int GEMV_SPLIT_SLOTS = 512; // (channel block, K chunk) slots of 16 x 64 f32 in a context's split-K workspace

std::string &last_error();
int fail(int code, const char *fmt, ...);

#define NNCB_CUDA_TRY(expr)                                                                     \
    do {                                                                                        \
        cudaError_t e__ = (expr);                                                               \
        if (e__ != cudaSuccess)                                                                 \
            return nncb::fail(-EIO, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__),    \
                              __FILE__, __LINE__);                                              \
    } while (0)

#define NNCB_TRY(expr)                                                                          \
    do {                                                                                        \
        int r__ = (expr);                                                                       \
        if (r__ < 0)                                                                            \
            return r__;                                                                         \
    } while (0)

// Checks the launch that was just enqueued and counts it.
int after_launch(nncb_context *ctx, const char *what);
bool gemm_w8a16_tc_applies(const nncb_context *ctx, int M, int N, int K);
int gemm_w8a16_tc(nncb_context *ctx, const void *x, const int8_t *w, const void *scale, const void *bias, const void *residual,
                  void *y, int M, int N, int K, int swiglu);
int gemm_w8a16_tc_set_attributes();

// ---- programmatic dependent launch ------------------------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may become resident while its predecessor in
// the stream still runs (on SMs the predecessor has left): its set-up -- barriers, TMEM allocation, tables and
// constants that no kernel writes -- overlaps the predecessor's last tiles and the launch latency. It must call
// grid_dependency_wait() before it touches memory that an earlier kernel wrote or reads; the wait returns when
// the predecessor grid has completed and its writes are visible (launched without the attribute, at once). A
// kernel lets its own dependent in with grid_dependency_release(); without that call the dependent starts when
// the kernel ends, as in a plain launch.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_dependent(nncb_context *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->opt.launch_overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Raise the dynamic shared-memory limit of this file's kernels on the CURRENT device (the attribute is per
// device; called for every context that is created).
int paged_attention_set_attributes();
// This step's unrotated qkv rows with the rotary tables and positions: the attention kernel then rotates q, and
// rotates and appends the new token's k / v, itself.
struct PaRope {
    const void *qkv;
    const float *cos_t, *sin_t;
    const int32_t *positions;
    int max_pos;
};
int gemv_set_attributes();

inline int conv_out_size(int in, int k, int stride, int dil, int pad_before, int pad_after) {
    return (in + pad_before + pad_after - ((k - 1) * dil + 1)) / stride + 1;
}

// Host float arithmetic identical to the device's IEEE operations (this file is compiled
// with contraction off for host code): the quantize formula of the reference.
inline int32_t host_quant(float x, float scale, float zp, int32_t lo, int32_t hi);

// ---- device helpers -----------------------------------------------------------------------
// q = clamp(rint(x / scale + zp), lo, hi): IEEE division, addition and round-half-even, the
// same three roundings as `nearbyintf(x / scale + bias)` in the reference's quantize.
__device__ __forceinline__ int quant_dev(float x, float scale, float zp, int lo, int hi) {
    float v = __fadd_rn(__fdiv_rn(x, scale), zp);
    int q = __float2int_rn(v);
    return min(max(q, lo), hi);
}
// y = (q - zp) * scale with one rounding per operation.
__device__ __forceinline__ float dequant_dev(float q, float zp, float scale) {
    return __fmul_rn(__fsub_rn(q, zp), scale);
}
// kernels::detail::clamp = max(min(v, hi), lo)
// Two IEEE single-precision operations per instruction (sm_100 f32x2 forms): each half rounds exactly like
// the scalar operation, and the epilogue, which is bound by instruction issue, spends one slot instead of two.
// Never feed mul2 straight into add2 (or an fma2 with a factor of one or an addend of -0) where the product has to
// round on its own: the assembler turns all of these into one fused multiply-add.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t p;
    asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "f"(lo), "f"(hi));
    return p;
}
__device__ __forceinline__ void unpack2(uint64_t p, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p)); }
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ float clamp_dev(float v, float lo, float hi) {
    float t = v < hi ? v : hi;
    return t > lo ? t : lo;
}

} // namespace nncb
