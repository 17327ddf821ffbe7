// Device helpers of the tcgen05 / TMA kernels (mbarriers with bounded waits, TMA loads, shared-memory operand
// descriptors, MMA issue and commit, TMEM loads) and the host's way to the tensor-map encoders of the driver.
#pragma once
#include <cuda.h>

#include "internal.cuh"

namespace nncb {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);
typedef CUresult (*PFN_encodeIm2col)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                     const cuuint64_t *, const int *, const int *, cuuint32_t, cuuint32_t,
                                     const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled g_encode_tiled = nullptr;
static PFN_encodeIm2col g_encode_im2col = nullptr;

// The driver API is reached through the runtime so that the library has no link-time
// dependency on libcuda and loads on machines without a driver.
static int load_driver_entry_points() {
    if (g_encode_tiled && g_encode_im2col)
        return 0;
    cudaDriverEntryPointQueryResult qres;
    void *fn = nullptr;
    NNCB_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (!fn || qres != cudaDriverEntryPointSuccess)
        return fail(-EIO, "cuTensorMapEncodeTiled is not available from this driver");
    g_encode_tiled = (PFN_encodeTiled)fn;
    fn = nullptr;
    NNCB_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres));
    if (!fn || qres != cudaDriverEntryPointSuccess)
        return fail(-EIO, "cuTensorMapEncodeIm2col is not available from this driver");
    g_encode_im2col = (PFN_encodeIm2col)fn;
    return 0;
}


namespace dev {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait. Returns false when the block is aborting or the wait ran out (the context's
// "wait_limit_us", 1 s unless changed; the limit is the word that follows the abort flag in shared
// memory); in the latter case it records `code` in the status word and raises the abort flag.
// The first probe is inlined at the call site: the one-thread producer and MMA loops run one
// dependent instruction at a time, so a call and a timer read per K block would cost more than
// the K block's loads and MMAs.
// try_wait with a suspend-time hint: the thread sleeps in hardware until the phase completes or `ns`
// nanoseconds have passed, instead of coming back to spend issue slots on another probe
__device__ __forceinline__ bool mbar_try_suspend(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity), "r"(ns)
                 : "memory");
    return ok != 0;
}
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
    const uint64_t t0 = globaltimer_ns();
    const uint64_t limit_ns = 1000ull * reinterpret_cast<volatile const unsigned *>(abort_flag)[1];
    for (uint32_t it = 1;; it++) {
        // a role that is ahead of the others sleeps on the barrier instead of spending issue slots on probes
        if (mbar_try_suspend(bar, parity, 20000u))
            return true;
        if (*abort_flag)
            return false;
        if (globaltimer_ns() - t0 > limit_ns) {
            atomicCAS(status, 0, code);
            *abort_flag = 1;
            __threadfence_block();
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
    if (mbar_try(bar, parity))
        return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, code);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c, int w,
                                                   int h, int n, uint16_t off_w, uint16_t off_h) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
                 : "memory");
}

// Swizzled K-major descriptor with an explicit stride offset (bytes from one 8-row group to the next)
__device__ __forceinline__ uint64_t smem_desc_sbo(uint32_t addr, int kb, uint32_t sbo) {
    const uint64_t layout = kb == 128 ? 2 : (kb == 64 ? 4 : 6);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= layout << 61;
    return d;
}

// Unswizzled K-major operand descriptor: core matrices of 8 rows x 16 bytes (128 contiguous bytes), `lbo`
// bytes from one to the next along K, `sbo` bytes to the next 8 rows.
__device__ __forceinline__ uint64_t smem_desc_plain(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46; // descriptor version of this architecture
    return d;               // layout type 0: no swizzle
}

// K-major shared-memory operand descriptor: rows of `kb` bytes, 8-row swizzle atoms `8*kb`
// bytes apart (stride byte offset), swizzle mode matching the row length.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, int kb) {
    const uint64_t layout = kb == 128 ? 2 : (kb == 64 ? 4 : 6);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)((8 * kb) >> 4) << 32;         // stride byte offset
    d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
    d |= layout << 61;
    return d;
}

// An operand descriptor as two words: only the low one (start address >> 4 in its low 14 bits) changes from MMA to
// MMA, and the sums never carry out of that field (the stage ring stays below the field's 256 KB range), so
// advancing a descriptor is one 32-bit add and the high word is loop-invariant. The MMA loop is one thread's
// dependent instruction stream and paces the tensor pipe: with 64-bit descriptor arithmetic a K = 32 MMA took
// about 250 cycles.
struct Desc {
    uint32_t lo, hi;
    __device__ __forceinline__ Desc operator+(uint32_t o) const { return Desc{lo + o, hi}; }
    __device__ __forceinline__ Desc &operator+=(uint32_t o) {
        lo += o;
        return *this;
    }
};
__device__ __forceinline__ Desc make_desc(uint64_t d) { return Desc{(uint32_t)d, (uint32_t)(d >> 32)}; }
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, Desc a, Desc b, uint32_t idesc, uint32_t accum) {
    asm volatile("{\n.reg .pred p;\n.reg .b64 da, db;\nsetp.ne.b32 p, %6, 0;\n"
                 "mov.b64 da, {%1, %2};\nmov.b64 db, {%3, %4};\n"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n}"
                 ::"r"(tmem_d), "r"(a.lo), "r"(a.hi), "r"(b.lo), "r"(b.hi), "r"(idesc), "r"(accum)
                 : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                 "tcgen05.wait::ld.sync.aligned;"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
// Split form: the load is issued early; the registers hold the data only after tmem_ld_wait().
// Both are volatile statements with a memory clobber, which keeps them in program order; every
// use of the registers is written after the wait.
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, int (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld8_issue(uint32_t taddr, int (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The wait is part of the same statement so that no use of the result can be scheduled before it.
__device__ __forceinline__ void tmem_ld1(uint32_t taddr, int &r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];\ntcgen05.wait::ld.sync.aligned;"
                 : "=r"(r)
                 : "r"(taddr)
                 : "memory");
}

} // namespace dev

} // namespace nncb
