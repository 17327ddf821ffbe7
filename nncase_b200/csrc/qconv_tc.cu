// Quantized Conv2D / MatMul as an implicit GEMM on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, u8 activations x u8|i8 weights -> s32 in tensor memory).
//
//   GEMM view: M = n*oh*ow output pixels, N = output channels, K = kh*kw*c ordered (ky, kx, c).
//   A (activations, NHWC) is never materialised: each K block of one filter tap is fetched by
//   TMA -- a plain 2-D tile for 1x1/stride-1 convolutions and MatMul, the im2col tensor-map
//   mode otherwise (the hardware walks 128 consecutive output pixels, applies the tap offset
//   and zero-fills the padding). B (weights) is repacked once at plan creation into K-major
//   rows per N tile.
//
//   One persistent CTA per SM, warp-specialised:
//     warp 0       TMA producer   (one lane) fills a ring of shared-memory stages
//     warp 1       MMA issuer     (one lane) tcgen05.mma into one of two TMEM accumulators
//     warps 2..17  epilogue       tcgen05.ld the finished accumulator, requantise, store u8 (TMA stores)
//     warps 18, 19 a second MMA issuer and a second load warp, in plans with deep K loops
//   so the epilogue of tile i overlaps the main loop of tile i+1. Launched as a programmatic dependent of the
//   kernel before it in the stream: set-up runs during that kernel's last tiles, the first load of
//   activations (and of the residual) waits for its completion.
//
//   Zero points. The MMA accumulates raw sum(xq*wq); TMA fills padding with 0 (not with the
//   zero point), so with "valid" = taps inside the image
//     sum_valid (xq-zx)(wq-zw) = sum xq*wq - zx*sum_valid wq - zw*(sum_valid xq - cnt_valid*zx).
//   sum_valid wq depends only on the output pixel's border class and the channel: a table
//   corr[class][oc] built at plan creation. sum_valid xq is per pixel: it comes out of the same
//   MMA through one extra all-ones weight row per N tile (present only if some zw != 0).
//
//   Every wait in the kernel is bounded: when a barrier does not complete within about a second
//   the role records a code in the context's status word, raises a block-wide abort flag and
//   all roles leave their loops, free tensor memory and return.
#include "qconv.cuh"
#include "tc_dev.cuh"
#include <cmath>
#include <type_traits>
#include <vector>

namespace nncb {

// ------------------------------------------------------------------------------------------------
// plan
// ------------------------------------------------------------------------------------------------
// MODE_ROWS: an unpadded stride-1 convolution over few channels whose kw taps of one kernel row are
// contiguous in memory (kw * c is 32, 64 or 128 bytes): a plain tiled tensor map whose pixel stride
// is smaller than its row extent delivers the overlapping windows, one K block per kernel row, and
// the M tile is a bx x by patch of output pixels instead of 128 consecutive ones.
// MODE_PATCH: the same convolutions when c == 16 (space-to-depth image stems) and the weights stay resident.
// The M tile is an 8 x 16 patch of output pixels; ONE load brings its (8 + kw - 1) x (16 + kh - 1) input
// cells (16 bytes each, a few KB in a few long rows) and the overlapping windows are formed by the MMA's
// own operand addressing: in the unswizzled K-major layout a core matrix is 8 rows x 16 bytes = 8
// consecutive cells of a patch row, the next core matrix along K is the same row one cell further (leading
// offset 16 bytes, they overlap), the next 8 rows are the next patch row (stride offset = its pitch). MODE_ROWS
// moves kh x 128 short rows per tile for the same data and is bound by rows per clock.
// The same tile shape serves padded 3 x 3-like stride-1 convolutions over 64 or 128 channels with resident weights
// (cell = one pixel = one 64- or 128-byte swizzle row): the patch is loaded once per tile with the tensor map's
// swizzle, out-of-image cells zero-filled, and every tap addresses it through a swizzled descriptor whose start
// is moved by whole pixels -- the swizzle is a function of the shared-memory address, so a start inside the
// 8-row pattern and a stride offset that is not a multiple of it read what the load wrote. One ninth of the
// activation rows of the im2col form, which is bound by rows per clock at these channel counts.
enum { MODE_GEMM = 0, MODE_IM2COL = 1, MODE_ROWS = 2, MODE_PATCH = 3 };

// Division by a number fixed at plan creation (Granlund and Montgomery's multiply-and-shift): for n < 2^31,
// n / d == (umulhi(n, mul) + n) >> shift with shift = ceil(log2 d), mul = floor(2^32 (2^shift - d) / d) + 1.
// An integer division costs the kernel's one-thread roles some hundred dependent cycles and the epilogue
// warps some 25 issue slots each; the tile loops have several per tile.
struct FastDiv {
    uint32_t mul, shift, d;
};
static FastDiv make_fastdiv(int d) {
    FastDiv f;
    f.d = (uint32_t)(d < 1 ? 1 : d);
    f.shift = 0;
    while ((1ull << f.shift) < f.d)
        f.shift++;
    f.mul = (uint32_t)((((1ull << f.shift) - f.d) << 32) / f.d) + 1u;
    return f;
}
__device__ __forceinline__ int fdiv(int n, const FastDiv &f) { return (int)((__umulhi((uint32_t)n, f.mul) + (uint32_t)n) >> f.shift); }
// quotient and remainder
__device__ __forceinline__ int fdivmod(int n, const FastDiv &f, int &rem) {
    const int q = fdiv(n, f);
    rem = n - q * (int)f.d;
    return q;
}

struct TcGeom {
    int mode;
    int m_total;        // n*oh*ow
    int oc;             // real output channels
    int bn;             // output channels per N tile
    int bn_mma;         // MMA N (bn + 16 when the row-sum column is present), multiple of 16
    int n_tiles, m_tiles;
    int kb;             // bytes (= int8 elements) per K block: 32, 64 or 128
    int c_blocks;       // c / kb
    int taps;           // kh*kw
    int kw;
    int oh, ow;
    int stride_h, stride_w, pad_t, pad_l, dil_h, dil_w;
    int has_xsum;       // row-sum column present
    int x_zp;
    int c;              // input channels
    int n_cls_x;        // number of x border classes (corr index = ycls*n_cls_x + xcls)
    int stages;
    int tmem_cols;      // allocation (power of two >= 32)
    int acc_stride;     // TMEM columns between the two accumulators
    uint32_t idesc;
    int f32_out;
    int acc_arrivals;   // epilogue warps that release an accumulator buffer
    int issuers;        // 2: two warps issue the MMAs, taking the stages of the ring in turn (stages is even then)
    int load_warps;     // 2: two load warps
    int load_by_stage;  // ... that take the stages of the ring in turn (else: one loads activations, one weights)
    int kgroup;         // K blocks per pipeline stage (one barrier round trip and one commit for all of them)
    int b_resident;     // the whole weight matrix stays in shared memory (one N tile, small K): loaded once per CTA
    int bx_log2, tiles_x, tiles_y; // MODE_ROWS: patch width 2^bx_log2 (height 128 >> bx_log2), patches per image
    int patch_w, patch_h;          // MODE_PATCH: input cells per patch row, patch rows
    int kh, kw_cells;              // MODE_PATCH: kernel rows, cells per kernel row
    int cell;                      // MODE_PATCH: bytes per cell (16: unswizzled; 64 / 128: one swizzle row per pixel)
    FastDiv fd_m_tiles, fd_ow, fd_oh, fd_tiles_x, fd_tiles_y;
    unsigned wait_limit_us;        // waits give up after this long (context option, set per launch)
    int withhold;                  // self-test of the give-up path: CTA 0 expects bytes that never arrive
};

struct FastEpi;
struct TcPlan {
    TcGeom g;
    void *d_wpack = nullptr;       // [n_tiles][bn_mma][K] packed weights
    int32_t *d_corr = nullptr;     // [n_cls][oc_pad] zx * sum_valid(wq)
    int32_t *d_cnt = nullptr;      // [n_cls] valid taps * c
    uint8_t *d_ycls = nullptr;     // [oh]
    uint8_t *d_xcls = nullptr;     // [ow]
    int oc_pad = 0;
    CUtensorMap tmap_b;
    // The A map depends on the activation pointer; it is rebuilt when the pointer changes.
    CUtensorMap tmap_a;
    const void *a_ptr = nullptr;
    size_t smem_bytes = 0;
    // fast epilogue
    bool fast = false;
    FastEpi *f = nullptr;
    float4 *d_cst = nullptr;
    uint8_t *d_addtab = nullptr;   // [256][256] residual-add table
    CUtensorMap tmap_y, tmap_y2, tmap_res;
    const void *y_ptr = nullptr, *y2_ptr = nullptr, *res_ptr = nullptr;
};

static CUtensorMapSwizzle swizzle_for(int kb) {
    return kb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (kb == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

static bool rows_mode_applies(const nncb_conv2d_desc &d) {
    const int rb = d.kw * d.c;
    return d.groups == 1 && d.kw > 1 && d.stride_h == 1 && d.stride_w == 1 && d.dil_h == 1 && d.dil_w == 1 &&
           d.pad_t == 0 && d.pad_b == 0 && d.pad_l == 0 && d.pad_r == 0 && d.c % 16 == 0 &&
           (rb == 32 || rb == 64 || rb == 128) && d.h >= d.kh && d.w >= d.kw;
}

static bool patch_mode_applies(const nncb_conv2d_desc &d) {
    // cells of exactly one core-matrix width, an even number of them per kernel row (one MMA takes two),
    // one N tile whose weights stay in shared memory, no residual (its buffers and table need the room)
    if (!rows_mode_applies(d) || d.c != 16 || (d.kw & 1) || d.kh > 8 || d.oc > 128 || d.has_residual)
        return false;
    const size_t b_all = (size_t)d.kh * (((size_t)(d.oc + 31) * d.kw * 16 + 1023) & ~(size_t)1023);
    return b_all <= 48u * 1024u;
}

// the wide-cell form: padded or not, stride 1, dilation 1, c = 64 or 128, one N tile with resident weights
static bool patch_wide_applies(const nncb_conv2d_desc &d, const nncb_options &opt) {
    if (!opt.conv_wide_patch) // tuning override: keep these layers on the im2col form
        return false;
    if (d.groups != 1 || d.stride_h != 1 || d.stride_w != 1 || d.dil_h != 1 || d.dil_w != 1 || (d.c != 64 && d.c != 128) ||
        d.kh < 2 || d.kw < 2 || d.kh > 4 || d.kw > 4 || d.oc > 128 || d.oc % 16 != 0 || d.has_residual || d.f32_out)
        return false;
    if (d.pad_t >= d.kh || d.pad_b >= d.kh || d.pad_l >= d.kw || d.pad_r >= d.kw)
        return false;
    const size_t b_all = (size_t)d.kh * d.kw * (((size_t)(d.oc + 31) * d.c + 1023) & ~(size_t)1023);
    return b_all <= 64u * 1024u;
}

bool tc_conv_supported(const nncb_conv2d_desc &d, std::string *why) {
    auto no = [&](const char *m) {
        if (why)
            *why = m;
        return false;
    };
    if (d.groups != 1)
        return no("grouped convolution");
    if (d.c % 32 != 0 && !rows_mode_applies(d))
        return no("input channels not a multiple of 32");
    if ((size_t)d.kh * d.kw * d.c > (1u << 20))
        return no("K too large");
    if (d.kh > 255 || d.kw > 255)
        return no("filter too large");
    const int oh = conv_out_size(d.h, d.kh, d.stride_h, d.dil_h, d.pad_t, d.pad_b);
    const int ow = conv_out_size(d.w, d.kw, d.stride_w, d.dil_w, d.pad_l, d.pad_r);
    if ((long long)d.n * oh * ow > 0x7fffffffLL)
        return no("M too large");
    // im2col tensor maps hold the corner offsets in 8 bits (4-D tensors).
    const int upper_w = d.pad_r - (d.kw - 1) * d.dil_w, upper_h = d.pad_b - (d.kh - 1) * d.dil_h;
    const bool gemm = d.kh == 1 && d.kw == 1 && d.stride_h == 1 && d.stride_w == 1 && d.pad_t == 0 && d.pad_b == 0 &&
                      d.pad_l == 0 && d.pad_r == 0;
    if (!gemm) {
        if (d.pad_l > 128 || d.pad_t > 128 || upper_w < -128 || upper_w > 127 || upper_h < -128 || upper_h > 127)
            return no("padding / dilation outside the im2col corner range");
        if (d.stride_h > 8 || d.stride_w > 8)
            return no("stride > 8");
        if ((d.kw - 1) * d.dil_w > 255 || (d.kh - 1) * d.dil_h > 255)
            return no("tap offset > 255");
        // The hardware derives the output extent from the corners; it must agree with ours.
        if ((d.w + upper_w + d.pad_l - 1) / d.stride_w + 1 != ow || (d.h + upper_h + d.pad_t - 1) / d.stride_h + 1 != oh)
            return no("output extent not expressible by im2col corners");
    }
    return true;
}

static int make_tmap_a(TcPlan *tp, const nncb_conv2d_desc &d, const void *x) {
    const TcGeom &g = tp->g;
    CUresult r;
    if (g.mode == MODE_PATCH && g.cell != 16) {
        // one swizzle row per pixel; the box is the patch of pixels under an 8 x 16 output patch
        cuuint64_t dims[4] = {(cuuint64_t)d.c, (cuuint64_t)d.w, (cuuint64_t)d.h, (cuuint64_t)d.n};
        cuuint64_t strides[3] = {(cuuint64_t)d.c, (cuuint64_t)d.c * d.w, (cuuint64_t)d.c * d.w * d.h};
        cuuint32_t box[4] = {(cuuint32_t)g.cell, (cuuint32_t)g.patch_w, (cuuint32_t)g.patch_h, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        r = g_encode_tiled(&tp->tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(x), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(g.cell), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (g.mode == MODE_PATCH) {
        // rows of the image as bytes; the box is the patch of input cells under an 8 x 16 output patch
        cuuint64_t dims[3] = {(cuuint64_t)d.w * 16, (cuuint64_t)d.h, (cuuint64_t)d.n};
        cuuint64_t strides[2] = {(cuuint64_t)d.w * 16, (cuuint64_t)d.w * 16 * d.h};
        cuuint32_t box[3] = {(cuuint32_t)g.patch_w * 16, (cuuint32_t)g.patch_h, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        r = g_encode_tiled(&tp->tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(x), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (g.mode == MODE_ROWS) {
        // dimension 1 steps one pixel (c bytes) while dimension 0 spans kw pixels: overlapping windows
        cuuint64_t dims[4] = {(cuuint64_t)(d.kw * d.c), (cuuint64_t)g.ow, (cuuint64_t)d.h, (cuuint64_t)d.n};
        cuuint64_t strides[3] = {(cuuint64_t)d.c, (cuuint64_t)d.c * d.w, (cuuint64_t)d.c * d.w * d.h};
        cuuint32_t box[4] = {(cuuint32_t)g.kb, 1u << g.bx_log2, 128u >> g.bx_log2, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        r = g_encode_tiled(&tp->tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(x), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(g.kb), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (g.mode == MODE_GEMM) {
        cuuint64_t dims[2] = {(cuuint64_t)d.c, (cuuint64_t)g.m_total};
        cuuint64_t strides[1] = {(cuuint64_t)d.c};
        cuuint32_t box[2] = {(cuuint32_t)g.kb, 128};
        cuuint32_t estr[2] = {1, 1};
        r = g_encode_tiled(&tp->tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(x), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(g.kb), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        cuuint64_t dims[4] = {(cuuint64_t)d.c, (cuuint64_t)d.w, (cuuint64_t)d.h, (cuuint64_t)d.n};
        cuuint64_t strides[3] = {(cuuint64_t)d.c, (cuuint64_t)d.c * d.w, (cuuint64_t)d.c * d.w * d.h};
        int lower[2] = {-d.pad_l, -d.pad_t};
        int upper[2] = {d.pad_r - (d.kw - 1) * d.dil_w, d.pad_b - (d.kh - 1) * d.dil_h};
        cuuint32_t estr[4] = {1, (cuuint32_t)d.stride_w, (cuuint32_t)d.stride_h, 1};
        r = g_encode_im2col(&tp->tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(x), dims, strides, lower,
                            upper, (cuuint32_t)g.kb, 128, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(g.kb),
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        // Drivers up to CUDA 13.1 set a descriptor bit that misbehaves for tensors smaller than
        // 128 KiB in im2col mode; clearing bit 21 of the second 64-bit word is the published
        // remedy (CUTLASS does the same when it encodes im2col maps).
        int drv = 0;
        cudaDriverGetVersion(&drv);
        if (r == CUDA_SUCCESS && drv <= 13010 && (size_t)d.c * d.w * d.h * d.n < 131072)
            reinterpret_cast<uint64_t *>(&tp->tmap_a)[1] &= ~(1ull << 21);
    }
    if (r != CUDA_SUCCESS)
        return fail(-EIO, "encoding the activation tensor map failed (CUresult %d)", (int)r);
    tp->a_ptr = x;
    return 0;
}

// ------------------------------------------------------------------------------------------------
// device side
// ------------------------------------------------------------------------------------------------

// Extra constants of the fast epilogue (see epilogue_fast below).
struct FastEpi {
    uint32_t off_out, off_y2, off_res, off_cst, off_corr, off_lut2, off_tab; // byte offsets from the aligned smem base
    uint32_t res_pitch; // bytes between the residual staging buffers
    int lut_only; // the table maps the convolution's own output: only the mapped tile is stored
    int corr_pitch;     // bn + 1: distinct border classes fall into distinct banks
    int n_cls;
    int out_sw;         // swizzle span of the staging sub-tiles: 32 or 0
    int ncg, wcols;     // column groups per tile (2 to 4) and columns per epilogue warp (32 or 16)
    int halves;         // 2: tiles of 8 epilogue warps, the two halves of the warps take alternate tiles; else 1
    int fcorr;          // the integer corrections run in float (every intermediate is an integer below 2^24)
    float so, rso, zo;  // output scale, its correctly rounded reciprocal, zero point
    float one;          // 1.0f, as a kernel argument: a value the assembler cannot fold (see the bias add)
    float qlo, qhi;     // the fused clamp's bounds after quantization, within [0, 255]
    const float4 *cst;  // [oc_pad] {mult, bias, bits(corr of class 0), bits(-zw)}
    const uint8_t *add_table; // [256][256] quantized sum of (convolution output, residual), or null
    // the same chain in arithmetic (add_math): -(residual zero point), residual scale, the add's output scale as
    // correctly rounded reciprocal and negated, its zero point
    int add_math;
    float add_nzr, add_sr, add_rsa, add_nsa, add_za;
};

struct TcArgs {
    TcGeom g;
    EpiParams p;
    FastEpi f;
    const int32_t *corr;  // [n_cls][oc_pad]
    const int32_t *cnt;   // [n_cls]
    const uint8_t *ycls, *xcls;
    const int32_t *w_zp;  // [oc]
    int oc_pad;
    const uint8_t *res;
    void *y;
    uint8_t *y2;
    int *status;
};

enum { ERR_PRODUCER = 101, ERR_MMA_FULL = 102, ERR_MMA_ACC = 103, ERR_EPILOGUE = 104, ERR_RESIDUAL = 105 };

constexpr int EPI_WARPS = 16; // four per TMEM lane quadrant: enough warps per scheduler to hide TMEM and shared-memory latency
// warp 0: loads, warp 1: MMAs, warps 2 .. 17: epilogue, warp 18: the second MMA issuer, warp 19: the second
// load warp (idle in plans that use one of each)
constexpr int TC_THREADS = 64 + 32 * EPI_WARPS + 64;
constexpr int WARP_MMA2 = 2 + EPI_WARPS, WARP_LOAD2 = 3 + EPI_WARPS;
constexpr int MAX_STAGES = 8;
constexpr int RES_BUFS = 3; // residual sub-tiles in flight per epilogue warp: the fetch of tile i+3 starts when tile i is done
constexpr int ADD_TABLE_BYTES = 256 * 260; // fused residual add: rows of 256 entries, 260 bytes apart

struct TcShared {
    uint64_t bar_full[MAX_STAGES], bar_empty[MAX_STAGES], bar_acc_full[2], bar_acc_empty[2], bar_acc_init[2], bar_b, bar_res[EPI_WARPS * RES_BUFS];
    uint32_t tmem_base_slot;
    volatile int abort_flag;
    unsigned wait_limit_us; // must follow abort_flag: mbar_wait_slow reads it through the flag's address
};

struct StageGeom {
    uint32_t smem_base, a_stage_bytes, b_stage_bytes, stage_pitch;
    uint32_t kblock_pitch; // bytes between the K blocks of one stage
    uint32_t b_pitch;    // bytes between the K blocks of a resident weight matrix
    uint32_t b_resident; // its address (after the stage ring), or 0 when weights travel with the stages
};

__device__ __forceinline__ StageGeom stage_geom(const TcGeom &g, const uint8_t *smem_raw) {
    StageGeom sg;
    // stage ring, 1024-byte aligned (required by the 128-byte swizzle)
    sg.smem_base = (dev::smem_u32(smem_raw) + 1023u) & ~1023u;
    sg.a_stage_bytes = g.mode == MODE_PATCH ? (((uint32_t)g.patch_w * g.cell * g.patch_h + 1023u) & ~1023u) : 128u * g.kb;
    sg.b_stage_bytes = (uint32_t)g.bn_mma * g.kb;
    // keep every stage's A and B tile 1024-byte aligned (a_stage_bytes is a multiple of 1024)
    sg.b_pitch = (sg.b_stage_bytes + 1023u) & ~1023u;
    sg.kblock_pitch = sg.a_stage_bytes + (g.b_resident ? 0u : sg.b_pitch);
    sg.stage_pitch = (uint32_t)g.kgroup * sg.kblock_pitch;
    sg.b_resident = g.b_resident ? sg.smem_base + (uint32_t)g.stages * sg.stage_pitch : 0u;
    return sg;
}

__device__ __forceinline__ void tc_setup(const TcGeom &g, TcShared &sh, int warp) {
    using namespace dev;
    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        sh.wait_limit_us = g.wait_limit_us;
        for (int s = 0; s < g.stages; s++) {
            mbar_init(smem_u32(&sh.bar_full[s]), g.load_by_stage ? 1 : g.load_warps);
            mbar_init(smem_u32(&sh.bar_empty[s]), g.mode == MODE_PATCH ? g.issuers : 1);
        }
        mbar_init(smem_u32(&sh.bar_b), 1);
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&sh.bar_acc_full[b]), g.issuers);
            mbar_init(smem_u32(&sh.bar_acc_empty[b]), g.acc_arrivals);
            mbar_init(smem_u32(&sh.bar_acc_init[b]), 1);
        }
        for (int w = 0; w < EPI_WARPS * RES_BUFS; w++)
            mbar_init(smem_u32(&sh.bar_res[w]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base_slot)),
                     "r"((uint32_t)g.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
}

__device__ __forceinline__ void tc_teardown(const TcGeom &g, TcShared &sh, int warp, uint32_t tmem_base) {
    using namespace dev;
    if (sh.abort_flag) {
        // give loads that are still in flight time to land before shared memory is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {
        }
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)g.tmem_cols)
                     : "memory");
    }
}

// warp 0, one lane: fills the stage ring with the A (activation) and B (weight) tiles of every
// K block of every tile this CTA owns.
// `part`: 0 = this warp loads everything, 1 = the activations only, 2 = the weights only (two load warps: each
// announces its own bytes on the stage's barrier, which then counts two arrivals)
__device__ __forceinline__ void producer_loop(const TcGeom &g, const StageGeom &sg, TcShared &sh,
                                              const CUtensorMap *tmap_a, const CUtensorMap *tmap_b, int *status,
                                              const int part) {
    using namespace dev;
    const int k_blocks = g.taps * g.c_blocks;
    const int total_tiles = g.m_tiles * g.n_tiles;
    const bool gemm = g.mode == MODE_GEMM, rows = g.mode == MODE_ROWS;
    const int kb = g.kb, c_blocks = g.c_blocks, kw_ = g.kw;
    const uint32_t dil_w = g.dil_w, dil_h = g.dil_h, stages = g.stages;
    const bool b_res = sg.b_resident != 0;
    const bool load_a = part != 2, load_b = part != 1 && !b_res;
    const uint32_t kblock_bytes = (load_a ? sg.a_stage_bytes : 0u) + (load_b ? sg.b_stage_bytes : 0u);
    const bool by_stage = part >= 3;          // parts 3 and 4: the even and the odd stages of the ring, activations and weights
    const uint32_t my_parity = part == 4 ? 1u : 0u;
    const int kgroup = g.kgroup;
    const uint32_t bar_full0 = smem_u32(&sh.bar_full[0]), bar_empty0 = smem_u32(&sh.bar_empty[0]);
    uint32_t stage = 0, phase = 0;
    if (g.withhold && blockIdx.x == 0 && load_a && part != 4) // self-test: 16 bytes that no load delivers keep stage 0 from ever filling
        asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar_full0), "r"(16u) : "memory");
    if (b_res && (int)blockIdx.x < total_tiles && load_a && part != 4) {
        // the whole weight matrix, once
        const uint32_t bar_b = smem_u32(&sh.bar_b);
        mbar_expect_tx(bar_b, (uint32_t)k_blocks * sg.b_stage_bytes);
        for (int kbi = 0; kbi < k_blocks; kbi++)
            tma_load_2d(sg.b_resident + kbi * sg.b_pitch, tmap_b, bar_b, kbi * kb, 0);
    }
    grid_dependency_wait(); // activations are the previous kernel's output (the weights above are nobody's)
    if (g.mode == MODE_PATCH) {
        // one load per tile: the input cells under the output patch (weights are resident, one N tile)
        const uint32_t patch_bytes = (uint32_t)g.patch_w * g.cell * g.patch_h;
        const bool wide = g.cell != 16;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            int txi, tyi;
            const int r = fdivmod(tile, g.fd_tiles_x, txi);
            const int img = fdivmod(r, g.fd_tiles_y, tyi);
            if (!mbar_wait(bar_empty0 + stage * 8, phase ^ 1, &sh.abort_flag, status, ERR_PRODUCER))
                return;
            const uint32_t full = bar_full0 + stage * 8;
            mbar_expect_tx(full, patch_bytes);
            if (wide) // pixels as rows; the patch starts pad cells outside the output patch (zero fill outside the image)
                tma_load_4d(sg.smem_base + stage * sg.stage_pitch, tmap_a, full, 0, txi * 8 - g.pad_l, tyi * 16 - g.pad_t, img);
            else
                tma_load_3d(sg.smem_base + stage * sg.stage_pitch, tmap_a, full, (txi * 8) * 16, tyi * 16, img);
            if (++stage == stages) {
                stage = 0;
                phase ^= 1;
            }
        }
        return;
    }
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        int mt;
        const int nt = fdivmod(tile, g.fd_m_tiles, mt);
        const int m0 = mt * 128, n0 = nt * g.bn_mma;
        int cw = 0, chh = 0, cn = 0;
        if (rows) {
            int txi, tyi;
            const int r = fdivmod(mt, g.fd_tiles_x, txi);
            cn = fdivmod(r, g.fd_tiles_y, tyi);
            cw = txi << g.bx_log2;
            chh = tyi * (128 >> g.bx_log2);
        } else if (!gemm) {
            int q, pp;
            const int row_i = fdivmod(m0, g.fd_ow, q);
            cn = fdivmod(row_i, g.fd_oh, pp);
            cw = q * g.stride_w - g.pad_l;
            chh = pp * g.stride_h - g.pad_t;
        }
        // K blocks in (tap row, tap column, channel block) order; all indices advance by
        // increments -- this loop is one thread's dependent instruction stream
        int cb = 0, c_off = 0, k_off = 0;
        uint32_t off_w = 0, off_h = 0;
        int kx = 0;
        if (kgroup == 1) {
            // one K block per stage: the shortest instruction stream per block
            for (int kbi = 0; kbi < k_blocks; kbi++) {
                if (!by_stage || (stage & 1u) == my_parity) {
                    if (!mbar_wait(bar_empty0 + stage * 8, phase ^ 1, &sh.abort_flag, status, ERR_PRODUCER))
                        return;
                    const uint32_t full = bar_full0 + stage * 8;
                    const uint32_t sa = sg.smem_base + stage * sg.stage_pitch;
                    mbar_expect_tx(full, kblock_bytes);
                    if (load_a) {
                        if (gemm)
                            tma_load_2d(sa, tmap_a, full, c_off, m0);
                        else if (rows)
                            tma_load_4d(sa, tmap_a, full, 0, cw, chh + (int)off_h, cn);
                        else
                            tma_load_im2col_4d(sa, tmap_a, full, c_off, cw, chh, cn, (uint16_t)off_w, (uint16_t)off_h);
                    }
                    if (load_b)
                        tma_load_2d(sa + sg.a_stage_bytes, tmap_b, full, k_off, n0);
                }
                k_off += kb;
                c_off += kb;
                if (++cb == c_blocks) {
                    cb = 0, c_off = 0;
                    off_w += dil_w;
                    if (++kx == kw_)
                        kx = 0, off_w = 0, off_h += dil_h;
                }
                if (++stage == stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            continue;
        }
        for (int kb0 = 0; kb0 < k_blocks; kb0 += kgroup) {
            const bool mine = !by_stage || (stage & 1u) == my_parity;
            if (mine && !mbar_wait(bar_empty0 + stage * 8, phase ^ 1, &sh.abort_flag, status, ERR_PRODUCER))
                return;
            const uint32_t full = bar_full0 + stage * 8;
            const int cnt = min(kgroup, k_blocks - kb0); // K blocks of this stage
            if (mine)
                mbar_expect_tx(full, (uint32_t)cnt * kblock_bytes);
            uint32_t sa = sg.smem_base + stage * sg.stage_pitch;
            for (int i = 0; i < cnt; i++, sa += sg.kblock_pitch) {
                if (load_a && mine) {
                    if (gemm)
                        tma_load_2d(sa, tmap_a, full, c_off, m0);
                    else if (rows)
                        tma_load_4d(sa, tmap_a, full, 0, cw, chh + (int)off_h, cn); // kw = 1 here: off_h counts kernel rows
                    else
                        tma_load_im2col_4d(sa, tmap_a, full, c_off, cw, chh, cn, (uint16_t)off_w, (uint16_t)off_h);
                }
                if (load_b && mine)
                    tma_load_2d(sa + sg.a_stage_bytes, tmap_b, full, k_off, n0);
                k_off += kb;
                c_off += kb;
                if (++cb == c_blocks) {
                    cb = 0, c_off = 0;
                    off_w += dil_w;
                    if (++kx == kw_)
                        kx = 0, off_w = 0, off_h += dil_h;
                }
            }
            if (++stage == stages) {
                stage = 0;
                phase ^= 1;
            }
        }
    }
}

// The MMAs of one tile in patch mode for a filter size known at compile time: straight-line code (in the
// nested loops over taps each MMA pair cost about 390 cycles of the issuing thread, most of it loop overhead).
// WIDE: one pixel per swizzle row of `cell16` 16-byte units, a tap is `cell16 / 2` MMAs; else 16-byte cells and
// one MMA per pair of cells of a kernel row. With DUAL the taps go to the two issuers in turn; issuer 0 owns the
// first one, which overwrites the accumulator.
template <int KH, int KWC, bool WIDE>
__device__ __forceinline__ bool patch_taps(const bool DUAL, uint32_t tmem_d, const dev::Desc da0, const dev::Desc db0, const uint32_t row16,
                                           const uint32_t cell16, const uint32_t bres_pitch16, const uint32_t idesc,
                                           const uint32_t mi, const uint32_t bar_init, const uint32_t init_parity,
                                           volatile int *abort_flag, int *status) {
    using namespace dev;
    if (DUAL && mi == 1) {
        if (!mbar_wait(bar_init, init_parity, abort_flag, status, ERR_MMA_ACC))
            return false;
        fence_after_sync();
    }
    constexpr int PER_ROW = WIDE ? KWC : KWC / 2;
#pragma unroll
    for (int ky = 0; ky < KH; ky++) {
#pragma unroll
        for (int x = 0; x < PER_ROW; x++) {
            const int tap = ky * PER_ROW + x;
            if (DUAL && (uint32_t)(tap & 1) != mi)
                continue;
            if (WIDE) {
                const Desc da = da0 + ((uint32_t)ky * row16 + (uint32_t)x * cell16);
                const Desc db = db0 + (uint32_t)tap * bres_pitch16;
                mma_i8(tmem_d, da, db, idesc, tap != 0);
                mma_i8(tmem_d, da + 2, db + 2, idesc, 1);
                if (cell16 > 4) {
                    mma_i8(tmem_d, da + 4, db + 4, idesc, 1);
                    mma_i8(tmem_d, da + 6, db + 6, idesc, 1);
                }
            } else {
                const Desc da = da0 + ((uint32_t)ky * row16 + (uint32_t)(2 * x));
                const Desc db = db0 + ((uint32_t)ky * bres_pitch16 + (uint32_t)(2 * x));
                mma_i8(tmem_d, da, db, idesc, tap != 0);
            }
            if (DUAL && tap == 0) {
                fence_before_sync();
                mbar_arrive(bar_init);
            }
        }
    }
    return true;
}

// One lane of warp 1 (and, with two issuers, of warp 18): issues the MMAs of every K block into the tile's TMEM
// accumulator. One thread's stream per stage -- barrier probe, fence, descriptor arithmetic, four MMAs, commit,
// ring bookkeeping, each a dependent instruction or a branch of a lone warp -- takes 600 to 700 cycles, twice what
// the tensor pipe needs for the stage's MMAs at 144 columns. With DUAL (a run-time flag: one copy of the loop keeps
// the kernels' code, which every launch has to fetch, short) two threads take the stages of the ring in
// turn: stage index modulo 2 (with an odd stage count one of them takes the last and the first stage of the ring),
// so that a stage always belongs to the same thread and each of its barrier phases is seen in order by one
// waiter. Both accumulate into the same TMEM accumulator (32-bit integer sums do not depend on the order); the owner of a tile's first stage issues its
// first MMA, which overwrites the accumulator, and arrives on bar_acc_init; the other waits for that before its
// first MMA of the tile, with tcgen05 fences on both sides of the barrier. Each commits to the tile's
// bar_acc_full (count 2) after its last MMA.
__device__ __forceinline__ void mma_loop(const TcGeom &g, const StageGeom &sg, TcShared &sh, uint32_t tmem_base,
                                         int *status, const bool DUAL, const uint32_t mi) {
    using namespace dev;
    const int k_blocks = g.taps * g.c_blocks;
    const int total_tiles = g.m_tiles * g.n_tiles;
    uint32_t stage = 0, phase = 0;
    grid_dependency_wait(); // every bounded wait below starts its clock after the predecessor kernel has completed
    uint32_t acc_phase0 = 0, acc_phase1 = 0, init_phase = 0;
    int it = 0;
    // descriptors of stage 0; a stage further on adds its byte offset >> 4 to the address field
    // (the ring stays below the field's 256 KB range, so the sum never carries out of it)
    const Desc desc_a0 = make_desc(smem_desc(sg.smem_base, g.kb)), desc_b0 = make_desc(smem_desc(sg.smem_base + sg.a_stage_bytes, g.kb));
    const uint32_t pitch16 = sg.stage_pitch >> 4, stages = g.stages, idesc = g.idesc;
    const int kk = g.kb / 32; // 1, 2 or 4 MMAs of K = 32 per K block
    const uint32_t bar_full0 = smem_u32(&sh.bar_full[0]), bar_empty0 = smem_u32(&sh.bar_empty[0]);
    const bool b_res = sg.b_resident != 0;
    const Desc desc_bres = make_desc(smem_desc(sg.b_resident, g.kb));
    const uint32_t bres_pitch16 = sg.b_pitch >> 4, kblock_pitch16 = sg.kblock_pitch >> 4;
    const uint32_t b_step16 = b_res ? bres_pitch16 : kblock_pitch16; // from one K block's weights to the next
    const int kgroup = g.kgroup;
    if (b_res && (int)blockIdx.x < total_tiles) {
        if (!mbar_wait(smem_u32(&sh.bar_b), 0, &sh.abort_flag, status, ERR_MMA_FULL))
            return;
    }
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, it++) {
        const int buf = it & 1;
        const uint32_t ph = buf ? acc_phase1 : acc_phase0;
        if (!mbar_wait(smem_u32(&sh.bar_acc_empty[buf]), ph ^ 1, &sh.abort_flag, status, ERR_MMA_ACC))
            return;
        if (buf)
            acc_phase1 ^= 1;
        else
            acc_phase0 ^= 1;
        fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * g.acc_stride;
        bool joined = false; // DUAL: this thread has issued, or waited for, the tile's first MMA
        if (g.mode == MODE_PATCH) {
            if (!mbar_wait(bar_full0 + stage * 8, phase, &sh.abort_flag, status, ERR_MMA_FULL))
                return;
            fence_after_sync();
            // rows of the tile = (patch row y, x) with x fastest: 8-row groups step one patch row
            const uint32_t bar_init = smem_u32(&sh.bar_acc_init[buf]), init_parity = (init_phase >> buf) & 1;
            if (g.cell == 16 && g.kh == 4 && g.kw_cells == 4) {
                const uint32_t row16 = (uint32_t)g.patch_w;
                const Desc da = make_desc(smem_desc_plain(sg.smem_base, 16u, row16 * 16u)) + stage * pitch16;
                if (!patch_taps<4, 4, false>(DUAL, tmem_d, da, desc_bres, row16, 1u, bres_pitch16, idesc, mi, bar_init, init_parity,
                                                   &sh.abort_flag, status))
                    return;
            } else if (g.cell != 16 && g.kh == 3 && g.kw_cells == 3) {
                const uint32_t cell16 = (uint32_t)g.cell >> 4, row16 = (uint32_t)g.patch_w * cell16;
                const Desc da = make_desc(smem_desc_sbo(sg.smem_base, g.cell, row16 * 16u)) + stage * pitch16;
                if (!patch_taps<3, 3, true>(DUAL, tmem_d, da, desc_bres, row16, cell16, bres_pitch16, idesc, mi, bar_init, init_parity,
                                                  &sh.abort_flag, status))
                    return;
            } else if (g.cell == 16) {
                const uint32_t row16 = (uint32_t)g.patch_w; // patch row pitch in 16-byte units
                Desc da = make_desc(smem_desc_plain(sg.smem_base, 16u, row16 * 16u)) + stage * pitch16;
                Desc db = desc_bres;
                for (int ky = 0; ky < g.kh; ky++, da += row16, db += bres_pitch16)
                    for (int j = 0; j < g.kw_cells; j += 2) // one MMA: cells j, j + 1 of the kernel row (K = 32 bytes)
                        mma_i8(tmem_d, da + (uint32_t)j, db + (uint32_t)j, idesc, (ky | j) != 0);
            } else {
                // one pixel = one swizzle row: 8 consecutive pixels of a patch row are an 8-row group, the next
                // group is the next patch row; a tap moves the start by whole pixels
                const uint32_t cell16 = (uint32_t)g.cell >> 4, row16 = (uint32_t)g.patch_w * cell16;
                const Desc da0 = make_desc(smem_desc_sbo(sg.smem_base, g.cell, row16 * 16u)) + stage * pitch16;
                // (the shortest instruction stream per MMA: descriptors advance by increments)
                Desc db = desc_bres, da_row = da0;
                uint32_t accum = 0;
                for (int ky = 0; ky < g.kh; ky++, da_row += row16) {
                    Desc da = da_row;
                    for (int kx = 0; kx < g.kw_cells; kx++, da += cell16, db += bres_pitch16) {
                        mma_i8(tmem_d, da, db, idesc, accum); // K = 32 bytes per MMA
                        mma_i8(tmem_d, da + 2, db + 2, idesc, 1);
                        if (cell16 > 4) {
                            mma_i8(tmem_d, da + 4, db + 4, idesc, 1);
                            mma_i8(tmem_d, da + 6, db + 6, idesc, 1);
                        }
                        accum = 1;
                    }
                }
            }
            mma_commit(bar_empty0 + stage * 8); // (with two issuers the stage is free when both have committed)
            if (++stage == stages) {
                stage = 0;
                phase ^= 1;
            }
            mma_commit(smem_u32(&sh.bar_acc_full[buf]));
            init_phase ^= 1u << buf;
            continue;
        }
        if (kgroup == 1) {
            for (int kbi = 0; kbi < k_blocks; kbi++) {
                if (!DUAL || (stage & 1u) == mi) {
                    if (!mbar_wait(bar_full0 + stage * 8, phase, &sh.abort_flag, status, ERR_MMA_FULL))
                        return;
                    fence_after_sync();
                    if (DUAL && !joined) {
                        if (kbi != 0) {
                            if (!mbar_wait(smem_u32(&sh.bar_acc_init[buf]), (init_phase >> buf) & 1, &sh.abort_flag, status, ERR_MMA_ACC))
                                return;
                            fence_after_sync();
                        }
                        joined = true;
                    }
                    const Desc da = desc_a0 + stage * pitch16;
                    const Desc db = b_res ? desc_bres + (uint32_t)kbi * bres_pitch16 : desc_b0 + stage * pitch16;
                    mma_i8(tmem_d, da, db, idesc, kbi != 0);
                    if (DUAL && kbi == 0) {
                        fence_before_sync();
                        mbar_arrive(smem_u32(&sh.bar_acc_init[buf]));
                    }
                    if (kk > 1)
                        mma_i8(tmem_d, da + 2, db + 2, idesc, 1);
                    if (kk > 2) {
                        mma_i8(tmem_d, da + 4, db + 4, idesc, 1);
                        mma_i8(tmem_d, da + 6, db + 6, idesc, 1);
                    }
                    mma_commit(bar_empty0 + stage * 8); // frees the stage when these MMAs retire
                }
                if (++stage == stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            mma_commit(smem_u32(&sh.bar_acc_full[buf]));
            init_phase ^= 1u << buf;
            continue;
        }
        for (int kb0 = 0; kb0 < k_blocks; kb0 += kgroup) {
            if (!DUAL || (stage & 1u) == mi) {
                if (!mbar_wait(bar_full0 + stage * 8, phase, &sh.abort_flag, status, ERR_MMA_FULL))
                    return;
                fence_after_sync();
                if (DUAL && !joined) {
                    if (kb0 != 0) {
                        if (!mbar_wait(smem_u32(&sh.bar_acc_init[buf]), (init_phase >> buf) & 1, &sh.abort_flag, status, ERR_MMA_ACC))
                            return;
                        fence_after_sync();
                    }
                    joined = true;
                }
                const int cnt = min(kgroup, k_blocks - kb0);
                Desc da = desc_a0 + stage * pitch16;
                Desc db = b_res ? desc_bres + (uint32_t)kb0 * bres_pitch16 : desc_b0 + stage * pitch16;
                for (int i = 0; i < cnt; i++, da += kblock_pitch16, db += b_step16) {
                    mma_i8(tmem_d, da, db, idesc, (kb0 | i) != 0);
                    if (DUAL && (kb0 | i) == 0) {
                        fence_before_sync();
                        mbar_arrive(smem_u32(&sh.bar_acc_init[buf]));
                    }
                    if (kk > 1)
                        mma_i8(tmem_d, da + 2, db + 2, idesc, 1);
                    if (kk > 2) {
                        mma_i8(tmem_d, da + 4, db + 4, idesc, 1);
                        mma_i8(tmem_d, da + 6, db + 6, idesc, 1);
                    }
                }
                mma_commit(bar_empty0 + stage * 8); // frees the stage when these MMAs retire
            }
            if (++stage == stages) {
                stage = 0;
                phase ^= 1;
            }
        }
        mma_commit(smem_u32(&sh.bar_acc_full[buf]));
        init_phase ^= 1u << buf;
    }
}

// -------------------------------------------------------------------------------------------------
// generic epilogue: exact arithmetic per element, direct global stores. Takes every case
// (f32 output, activation table, channel counts that are not a multiple of 16).
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void epilogue_generic(const TcArgs &a, TcShared &sh, uint32_t tmem_base, int warp, int lane) {
    using namespace dev;
    const TcGeom &g = a.g;
    const int total_tiles = g.m_tiles * g.n_tiles;
    const int ew = warp - 2;
    const int lane_group = warp & 3; // TMEM lanes 32*lane_group .. +31 are this warp's
    const int grp = ew >> 2;         // the warps of a lane group take 16-column chunks in turn
    const int row = lane_group * 32 + lane;
    grid_dependency_wait(); // every bounded wait below starts its clock after the predecessor kernel has completed
    uint32_t acc_phase0 = 0, acc_phase1 = 0;
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, it++) {
        const int buf = it & 1;
        int mt;
        const int nt = fdivmod(tile, g.fd_m_tiles, mt);
        int m = mt * 128 + row;
        bool row_ok = m < g.m_total;
        int patch_cls = 0;
        if (g.mode == MODE_ROWS || g.mode == MODE_PATCH) {
            // the tile is a patch of output pixels: row -> (patch row, patch column)
            int txi, tyi;
            const int r2 = fdivmod(mt, g.fd_tiles_x, txi);
            const int img = fdivmod(r2, g.fd_tiles_y, tyi);
            const int ox = (txi << g.bx_log2) + (row & ((1 << g.bx_log2) - 1));
            const int oy = tyi * (128 >> g.bx_log2) + (row >> g.bx_log2);
            row_ok = ox < g.ow && oy < g.oh;
            m = (img * g.oh + oy) * g.ow + ox;
            patch_cls = row_ok ? (int)a.ycls[oy] * g.n_cls_x + (int)a.xcls[ox] : 0; // one class when unpadded
        }
        int cls = patch_cls; // border class of this output pixel
        if (g.mode == MODE_IM2COL && row_ok) {
            int ox, oy;
            fdivmod(fdivmod(m, g.fd_ow, ox), g.fd_oh, oy);
            cls = (int)a.ycls[oy] * g.n_cls_x + (int)a.xcls[ox];
        }
        const uint32_t ph = buf ? acc_phase1 : acc_phase0;
        if (!mbar_wait(smem_u32(&sh.bar_acc_full[buf]), ph, &sh.abort_flag, a.status, ERR_EPILOGUE))
            return;
        if (buf)
            acc_phase1 ^= 1;
        else
            acc_phase0 ^= 1;
        fence_after_sync();
        const uint32_t tbase = tmem_base + ((uint32_t)(lane_group * 32) << 16) + buf * g.acc_stride;
        int rsum = 0; // sum_valid xq - cnt_valid * zx
        if (g.has_xsum) {
            int xs;
            tmem_ld1(tbase + g.bn, xs);
            rsum = xs - a.cnt[cls] * g.x_zp;
        }
        const int32_t *corr = a.corr + (size_t)cls * a.oc_pad;
        const int oc0 = nt * g.bn;
        for (int c0 = grp * 16; c0 < g.bn; c0 += 16 * (EPI_WARPS / 4)) {
            int v[16];
            __syncwarp();
            tmem_ld16(tbase + c0, v);
            if (!row_ok || oc0 + c0 >= g.oc)
                continue;
            const size_t obase = (size_t)m * g.oc + oc0 + c0;
            if (g.f32_out) {
                float *yo = reinterpret_cast<float *>(a.y) + obase;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int oc = oc0 + c0 + j;
                    if (oc < g.oc) {
                        int acc = v[j] - corr[oc] - a.w_zp[oc] * rsum;
                        yo[j] = epi_real(acc, a.p.mult[oc], a.p.bias[oc], a.p.clamp_lo, a.p.clamp_hi);
                    }
                }
                continue;
            }
            uint32_t pk[4] = {0, 0, 0, 0}, pk2[4] = {0, 0, 0, 0};
            const bool full16 = (oc0 + c0 + 16 <= g.oc) && ((obase & 15) == 0);
            uint32_t rs[4] = {0, 0, 0, 0};
            if (a.p.has_res) {
                if (full16) {
                    uint4 r4 = *reinterpret_cast<const uint4 *>(a.res + obase);
                    rs[0] = r4.x, rs[1] = r4.y, rs[2] = r4.z, rs[3] = r4.w;
                } else {
                    for (int j = 0; j < 16; j++)
                        if (oc0 + c0 + j < g.oc)
                            rs[j >> 2] |= (uint32_t)a.res[obase + j] << (8 * (j & 3));
                }
            }
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const int oc = oc0 + c0 + j;
                if (oc < g.oc) {
                    int acc = v[j] - corr[oc] - a.w_zp[oc] * rsum;
                    int q = epi_u8(acc, a.p.mult[oc], a.p.bias[oc], a.p, (int)((rs[j >> 2] >> (8 * (j & 3))) & 255));
                    pk[j >> 2] |= (uint32_t)q << (8 * (j & 3));
                    if (a.y2)
                        pk2[j >> 2] |= (uint32_t)a.p.y2_lut[q] << (8 * (j & 3));
                }
            }
            uint8_t *yo = reinterpret_cast<uint8_t *>(a.y) + obase;
            if (full16) {
                *reinterpret_cast<uint4 *>(yo) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                if (a.y2)
                    *reinterpret_cast<uint4 *>(a.y2 + obase) = make_uint4(pk2[0], pk2[1], pk2[2], pk2[3]);
            } else {
                for (int j = 0; j < 16; j++)
                    if (oc0 + c0 + j < g.oc) {
                        yo[j] = (uint8_t)(pk[j >> 2] >> (8 * (j & 3)));
                        if (a.y2)
                            a.y2[obase + j] = (uint8_t)(pk2[j >> 2] >> (8 * (j & 3)));
                    }
            }
        }
        // this accumulator may be overwritten once all epilogue warps are done reading
        fence_before_sync();
        __syncwarp();
        if (lane == 0)
            mbar_arrive(smem_u32(&sh.bar_acc_empty[buf]));
    }
}

__global__ void __launch_bounds__(TC_THREADS, 1)
tc_conv_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const TcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) TcShared sh;
    const TcGeom &g = a.g;
    const StageGeom sg = stage_geom(g, smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    grid_dependency_release(); // the next kernel of the stream may take the SMs this one leaves
    tc_setup(g, sh, warp);
    const uint32_t tmem_base = sh.tmem_base_slot;
    if (warp == 0) {
        if (lane == 0)
            producer_loop(g, sg, sh, &tmap_a, &tmap_b, a.status, g.load_warps == 2 ? (g.load_by_stage ? 3 : 1) : 0);
    } else if (warp == 1) {
        if (lane == 0)
            mma_loop(g, sg, sh, tmem_base, a.status, g.issuers == 2, 0);
    } else if (warp == WARP_MMA2) {
        if (lane == 0 && g.issuers == 2)
            mma_loop(g, sg, sh, tmem_base, a.status, true, 1);
    } else if (warp == WARP_LOAD2) {
        if (lane == 0 && g.load_warps == 2)
            producer_loop(g, sg, sh, &tmap_a, &tmap_b, a.status, g.load_by_stage ? 4 : 2);
    } else {
        epilogue_generic(a, sh, tmem_base, warp, lane);
    }
    tc_teardown(g, sh, warp, tmem_base);
}

// -------------------------------------------------------------------------------------------------
// fast epilogue (u8 output, channel count a multiple of 16, N tile of 128, 64 or 32, no activation
// table). Same arithmetic as epi_u8 -- every IEEE operation of the requantisation chain, in the
// same order -- but organised for throughput:
//   * the two divisions (by the output scale, by the add-output scale) use a reciprocal that was
//     correctly rounded at plan creation: q0 = RN(x*r), rem = x - q0*s (exact, one fma),
//     q = RN(q0 + rem*r). With r = RN(1/s) this sequence returns RN(x/s), the IEEE quotient
//     (Markstein's theorem), in three fused operations instead of a division subroutine;
//   * per-channel constants are staged in shared memory per N tile and read as one broadcast
//     16-byte load per element;
//   * every epilogue warp stages its 32 x bn/2 sub-tile of the output (and of the optional second
//     output) in swizzled shared memory and writes it with its own TMA store; the residual
//     sub-tile is prefetched with a TMA load. No block-wide barrier in the steady state.
// -------------------------------------------------------------------------------------------------
namespace dev {
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory"); }
__device__ __forceinline__ bool epi_bar_or(bool v) {
    uint32_t out;
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.or.pred p, 1, %2, q;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(out)
                 : "r"((uint32_t)v), "n"(32 * EPI_WARPS)
                 : "memory");
    return out != 0;
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src),
                 "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// {a, b} and {c, d} of one 16-byte shared-memory word as two register pairs
__device__ __forceinline__ void lds128_2x64(uint32_t addr, uint64_t &lo, uint64_t &hi) {
    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(lo), "=l"(hi) : "r"(addr));
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts64(uint32_t addr, uint2 v) {
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// address of 16-byte chunk `chunk` of row `row` in a staging tile whose rows are `bn` bytes and
// which TMA reads / writes with swizzle span `sw`
__device__ __forceinline__ uint32_t stage_addr(uint32_t base, int row, int chunk, int bn, int sw) {
    const int x = sw == 128 ? (row & 7) : (sw == 64 ? ((row >> 1) & 3) : (sw == 32 ? ((row >> 2) & 1) : 0));
    return base + (uint32_t)(row * bn) + (uint32_t)((chunk ^ x) << 4);
}
} // namespace dev

// RES: 0 no residual, 1 fused add through the byte-pair table, 2 fused add as the float chain itself
template <int RES, bool Y2, bool XSUM, bool ROWS>
__device__ __forceinline__ void epilogue_fast(const TcArgs &a, const StageGeom &sg, TcShared &sh, uint32_t tmem_base,
                                              const CUtensorMap *tmap_y, const CUtensorMap *tmap_y2,
                                              const CUtensorMap *tmap_res, int warp, int lane) {
    using namespace dev;
    const TcGeom &g = a.g;
    const FastEpi &f = a.f;
    const int total_tiles = g.m_tiles * g.n_tiles;
    const int ew = warp - 2;
    const int et = ew * 32 + lane;   // index among the epilogue threads
    const int lane_group = warp & 3; // TMEM lanes 32*lane_group .. +31 are this warp's
    // which group of the tile's columns this warp owns, and (narrow tiles, f.halves == 2) which of the
    // alternating tiles: while one half of the warps waits for its accumulator, TMEM loads and stores, the
    // other half requantises the tile before
    const int grp = (ew >> 2) % f.ncg, half = (ew >> 2) / f.ncg;
    const bool active = half < f.halves; // some widths leave the last warps without columns
    const int row = lane_group * 32 + lane;
    const int hw = f.wcols;          // bytes per row of this warp's sub-tile (32 rows x hw columns)
    // Every warp stages, stores and prefetches its own 32 x hw sub-tile: no block-wide barrier in
    // the steady state.
    const uint32_t sub = (uint32_t)ew * 32u * hw;
    const uint32_t s_out = sg.smem_base + f.off_out + sub, s_y2 = sg.smem_base + f.off_y2 + sub;
    const uint32_t s_res = sg.smem_base + f.off_res + sub;
    const uint32_t s_cst = sg.smem_base + f.off_cst, s_corr = sg.smem_base + f.off_corr;
    const uint32_t s_lut2 = sg.smem_base + f.off_lut2, s_tab = sg.smem_base + f.off_tab;
    const uint32_t bar_res = smem_u32(&sh.bar_res[ew * RES_BUFS]);
    const bool multi_cls = f.n_cls > 1;
    const int clamp_level = f.qhi < 255.f ? 2 : (f.qlo > 0.f ? 1 : 0); // which bounds an activation moved inside 0..255
    const uint32_t res_bytes = 32u * hw;
    const int col_off = grp * hw;
    constexpr bool rows = ROWS; // the tile is a patch of pixels (MODE_ROWS)
    // Tensor-map coordinates of this warp's 32-row sub-tile of tile (mt, nt): 2-D {channel, pixel} in
    // general, 4-D {channel, x, y, image} when the tile is a patch of pixels. False when the sub-tile
    // lies wholly outside the output.
    auto sub_coords = [&](int mt, int nt, int (&c)[4]) {
        c[0] = nt * g.bn + col_off;
        if (!rows) {
            c[1] = mt * 128 + lane_group * 32;
            return c[1] < g.m_total;
        }
        int txi, tyi;
        const int r2 = fdivmod(mt, g.fd_tiles_x, txi), r0 = lane_group * 32;
        c[3] = fdivmod(r2, g.fd_tiles_y, tyi);
        c[1] = (txi << g.bx_log2) + (r0 & ((1 << g.bx_log2) - 1));
        c[2] = tyi * (128 >> g.bx_log2) + (r0 >> g.bx_log2);
        return c[1] < g.ow && c[2] < g.oh;
    };
    auto load_sub = [&](uint32_t dst, const CUtensorMap *map, uint32_t bar, const int (&c)[4]) {
        if (rows)
            tma_load_4d(dst, map, bar, c[0], c[1], c[2], c[3]);
        else
            tma_load_2d(dst, map, bar, c[0], c[1]);
    };
    auto store_sub = [&](const CUtensorMap *map, uint32_t src, const int (&c)[4]) {
        if (rows)
            tma_store_4d(map, src, c[0], c[1], c[2], c[3]);
        else
            tma_store_2d(map, src, c[0], c[1]);
    };
    if (RES == 1) {
        // the add table (65 KB), copied once per CTA
        const uint4 *src = reinterpret_cast<const uint4 *>(f.add_table);
        for (int i = et; i < ADD_TABLE_BYTES / 16; i += 32 * EPI_WARPS)
            sts128(s_tab + i * 16, __ldg(src + i));
    }
    if (Y2) {
        if (et < 64)
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(s_lut2 + et * 4),
                         "r"(reinterpret_cast<const uint32_t *>(a.p.y2_lut)[et])
                         : "memory");
    }
    // residual sub-tiles of this warp's next RES_BUFS tiles are always in flight
    const int tstep = f.halves * (int)gridDim.x; // distance between this warp's tiles
    if (RES && lane == 0 && active) {
        grid_dependency_wait(); // the residual is an earlier kernel's output
        int t = blockIdx.x + half * (int)gridDim.x;
        for (int b = 0; b < RES_BUFS && t < total_tiles; b++, t += tstep) {
            int c[4];
            int tm;
            const int tn = fdivmod(t, g.fd_m_tiles, tm);
            sub_coords(tm, tn, c); // a load outside the tensor still completes, with fill
            mbar_expect_tx(bar_res + b * 8, res_bytes);
            load_sub(s_res + b * f.res_pitch, tmap_res, bar_res + b * 8, c);
        }
    }
    grid_dependency_wait(); // every bounded wait below starts its clock after the predecessor kernel has completed
    uint32_t acc_phase0 = 0, acc_phase1 = 0, res_phase = 0; // res_phase: one parity bit per buffer
    int rb = 0;                                             // residual buffer of the current tile
    int it = 0, cur_nt = -1;
    bool dead = false; // after a failed wait the warp only keeps the block-wide barriers company
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, it++) {
        const int buf = it & 1;
        int mt;
        const int nt = fdivmod(tile, g.fd_m_tiles, mt);
        const int m = mt * 128 + row;
        const bool row_ok = m < g.m_total;
        const int oc0 = nt * g.bn;
        if (nt != cur_nt) {
            // (re)load the per-channel constants of this N tile; happens once or twice per CTA
            epi_bar_sync();
            // two columns share 32 bytes: {mult0, mult1, bias0, bias1} {corr0, corr1, -zw0, -zw1}, so that
            // the constants of a column pair arrive as register pairs
            for (int c = et; c < g.bn; c += 32 * EPI_WARPS) {
                const float4 k = f.cst[oc0 + c];
                const uint32_t dst = s_cst + (uint32_t)(c >> 1) * 32u + (uint32_t)(c & 1) * 4u;
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst), "f"(k.x) : "memory");
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst + 8), "f"(k.y) : "memory");
                // (float corrections: -corr and -zw as floats instead of integer bits)
                const float kz = f.fcorr ? -(float)__float_as_int(k.z) : k.z;
                const float kw_ = f.fcorr ? (float)__float_as_int(k.w) : k.w;
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst + 16), "f"(kz) : "memory");
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst + 24), "f"(kw_) : "memory");
            }
            if (multi_cls)
                for (int i = et; i < f.n_cls * g.bn; i += 32 * EPI_WARPS) {
                    const int cl = i / g.bn, c = i % g.bn;
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(s_corr + (cl * f.corr_pitch + c) * 4),
                                 "r"(a.corr[(size_t)cl * a.oc_pad + oc0 + c])
                                 : "memory");
                }
            cur_nt = nt;
            epi_bar_sync();
        }
        if (dead || !active || (f.halves == 2 && (it & 1) != half))
            continue;
        int cls = 0;
        if (g.mode == MODE_IM2COL && row_ok) {
            int ox, oy;
            fdivmod(fdivmod(m, g.fd_ow, ox), g.fd_oh, oy);
            cls = (int)a.ycls[oy] * g.n_cls_x + (int)a.xcls[ox];
        }
        if (rows && multi_cls) {
            // a padded patch-mode layer: the class of this lane's pixel of the patch
            int txi, tyi;
            fdivmod(fdivmod(mt, g.fd_tiles_x, txi), g.fd_tiles_y, tyi);
            const int ox = (txi << g.bx_log2) + (row & ((1 << g.bx_log2) - 1));
            const int oy = tyi * (128 >> g.bx_log2) + (row >> g.bx_log2);
            if (ox < g.ow && oy < g.oh)
                cls = (int)a.ycls[oy] * g.n_cls_x + (int)a.xcls[ox];
        }
        const uint32_t ph = buf ? acc_phase1 : acc_phase0;
        bool ok = mbar_wait(smem_u32(&sh.bar_acc_full[buf]), ph, &sh.abort_flag, a.status, ERR_EPILOGUE);
        if (RES && ok)
            ok = mbar_wait(bar_res + rb * 8, (res_phase >> rb) & 1, &sh.abort_flag, a.status, ERR_RESIDUAL);
        if (!ok) {
            dead = true;
            continue;
        }
        // this warp's previous TMA stores must have finished reading its staging sub-tiles
        if (lane == 0)
            tma_store_wait_read();
        __syncwarp();
        if (buf)
            acc_phase1 ^= 1;
        else
            acc_phase0 ^= 1;
        res_phase ^= 1u << rb;
        const uint32_t s_res_cur = s_res + rb * f.res_pitch;
        fence_after_sync();
        const uint32_t tbase = tmem_base + ((uint32_t)(lane_group * 32) << 16) + buf * g.acc_stride;
        int rsum = 0;
        if (XSUM) {
            int xs;
            tmem_ld1(tbase + g.bn, xs);
            rsum = xs - a.cnt[cls] * g.x_zp;
        }
        const uint32_t corr_row = s_corr + (uint32_t)(cls * f.corr_pitch) * 4;
        // eight columns at a time: short live ranges keep the 16 epilogue warps within the register file
        const uint64_t rso2 = pack2(f.rso, f.rso), nso2 = pack2(-f.so, -f.so), zo2 = pack2(f.zo, f.zo);
        const uint64_t one2 = pack2(f.one, f.one);
        const uint64_t rsumf2 = pack2((float)rsum, (float)rsum);
        const uint64_t add_nzo2 = pack2(-f.zo, -f.zo), add_so2 = pack2(f.so, f.so), add_nzr2 = pack2(f.add_nzr, f.add_nzr);
        const uint64_t add_sr2 = pack2(f.add_sr, f.add_sr), add_rsa2 = pack2(f.add_rsa, f.add_rsa);
        const uint64_t add_nsa2 = pack2(f.add_nsa, f.add_nsa), add_za2 = pack2(f.add_za, f.add_za);
        auto chunk = [&](const int (&v)[8], const int cc, auto multi_tag, auto clamp_tag, auto fc_tag) {
            constexpr bool MULTI = decltype(multi_tag)::value;
            constexpr bool FC = decltype(fc_tag)::value; // corrections in float (never with MULTI)
            constexpr int CL = decltype(clamp_tag)::value; // 0: no bound inside 0..255, 1: a lower one, 2: both
            const int c0 = col_off + cc; // column within the tile
            const uint32_t half16 = stage_addr(0, lane, cc >> 4, hw, f.out_sw) + (cc & 8); // offset in a sub-tile
            uint2 rw = make_uint2(0, 0);
            if (RES)
                rw = lds64(s_res_cur + half16);
            const uint32_t rwa[2] = {rw.x, rw.y};
            uint32_t bits[8];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                uint64_t mult2, bias2, ck_lo, ck_hi;
                lds128_2x64(s_cst + (c0 + j) * 16, mult2, bias2);      // {mult0, mult1} {bias0, bias1}
                lds128_2x64(s_cst + (c0 + j) * 16 + 16, ck_lo, ck_hi); // {corr0, corr1} {-zw0, -zw1}
                uint64_t accf2;
                if (FC) {
                    // acc - corr - zw * rowsum on integers below 2^24 held in floats: exact, and packed
                    accf2 = pack2((float)v[j], (float)v[j + 1]);
                    if (XSUM)
                        accf2 = fma2(ck_hi, rsumf2, accf2);
                    accf2 = add2(accf2, ck_lo);
                } else {
                    int corr0 = (int)(uint32_t)ck_lo, corr1 = (int)(uint32_t)(ck_lo >> 32);
                    if (MULTI) {
                        corr0 = (int)lds32(corr_row + (c0 + j) * 4);
                        corr1 = (int)lds32(corr_row + (c0 + j) * 4 + 4);
                    }
                    int acc0 = v[j] - corr0, acc1 = v[j + 1] - corr1;
                    if (XSUM) {
                        acc0 += (int)(uint32_t)ck_hi * rsum;
                        acc1 += (int)(uint32_t)(ck_hi >> 32) * rsum;
                    }
                    accf2 = pack2((float)acc0, (float)acc1);
                }
                // x = acc * mult + bias, then x / so correctly rounded: q0 = RN(x r), q = RN(q0 + RN(x - q0 so) r)
                // the product must round before the bias is added: the assembler contracts a packed multiply and a
                // packed add into one fused operation even when both carry .rn. So the add is a fused multiply-add
                // by one, RN(p * 1 + bias) = RN(p + bias), with the one a kernel argument that cannot be folded away.
                const uint64_t x2 = fma2(mul2(accf2, mult2), one2, bias2);
                const uint64_t q0 = mul2(x2, rso2);
                const uint64_t q2 = fma2(fma2(q0, nso2, x2), rso2, q0);
                // Quantization is monotone, so the fused clamp on the real value is a clamp of the
                // quantized value to the quantized bounds, and clamping before rounding to an integer is
                // the same as after. One saturating round-to-nearest-even conversion is rint + clamp to
                // 0..255; a bound that an activation moved inside that range is applied first.
                float u0, u1;
                unpack2(add2(q2, zo2), u0, u1);
                if (CL >= 1)
                    u0 = fmaxf(u0, f.qlo), u1 = fmaxf(u1, f.qlo);
                if (CL == 2)
                    u0 = fminf(u0, f.qhi), u1 = fminf(u1, f.qhi);
                asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(bits[j]) : "f"(u0));
                asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(bits[j + 1]) : "f"(u1));
                if (RES == 2) {
                    // dequantize both addends, add, requantise: the unfused chain itself, two outputs at a time.
                    // (q - zo) so and (r - zr) sr are rounded products; their sum is a fused multiply-add by one
                    // (see the bias add above); the division is the three-operation exact quotient.
                    const uint32_t r0 = __byte_perm(rwa[j >> 2], 0u, 0x4440 | (j & 3));
                    const uint32_t r1 = __byte_perm(rwa[j >> 2], 0u, 0x4440 | ((j + 1) & 3));
                    const uint64_t ya = mul2(add2(pack2((float)bits[j], (float)bits[j + 1]), add_nzo2), add_so2);
                    const uint64_t yb = mul2(add2(pack2((float)r0, (float)r1), add_nzr2), add_sr2);
                    const uint64_t sum = fma2(ya, one2, yb);
                    const uint64_t p0 = mul2(sum, add_rsa2);
                    const uint64_t p2 = fma2(fma2(p0, add_nsa2, sum), add_rsa2, p0);
                    float w0, w1;
                    unpack2(add2(p2, add_za2), w0, w1);
                    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(bits[j]) : "f"(w0));
                    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(bits[j + 1]) : "f"(w1));
                }
                if (RES == 1) {
                    // dequantize both addends, add, requantise -- as a table of all byte pairs. Rows of 260
                    // bytes: the bank of entry (q, r) is (q + r / 4) mod 32, so the pixels of one channel,
                    // which have similar q and similar r, spread over the banks.
                    const uint32_t r0 = __byte_perm(rwa[j >> 2], 0u, 0x4440 | (j & 3));
                    const uint32_t r1 = __byte_perm(rwa[j >> 2], 0u, 0x4440 | ((j + 1) & 3));
                    bits[j] = lds8(s_tab + bits[j] * 260u + r0);
                    bits[j + 1] = lds8(s_tab + bits[j + 1] * 260u + r1);
                }
            }
            uint2 o;
            o.x = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
            o.y = __byte_perm(__byte_perm(bits[4], bits[5], 0x0040), __byte_perm(bits[6], bits[7], 0x0040), 0x5410);
            sts64(s_out + half16, o);
            if (Y2) {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    bits[j] = lds8(s_lut2 + bits[j]);
                o.x = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
                o.y = __byte_perm(__byte_perm(bits[4], bits[5], 0x0040), __byte_perm(bits[6], bits[7], 0x0040), 0x5410);
                sts64(s_y2 + half16, o);
            }
        };
        // the TMEM load of the next eight columns is in flight while the current ones are requantised
        auto columns = [&](auto multi_tag, auto clamp_tag, auto fc_tag) {
            int va[8], vb[8];
            __syncwarp();
            tmem_ld8_issue(tbase + col_off, va);
            for (int cc = 0; cc < hw; cc += 16) { // hw is 16 or 32
                tmem_ld_wait();
                tmem_ld8_issue(tbase + col_off + cc + 8, vb);
                chunk(va, cc, multi_tag, clamp_tag, fc_tag);
                tmem_ld_wait();
                if (cc + 16 < hw)
                    tmem_ld8_issue(tbase + col_off + cc + 16, va);
                chunk(vb, cc + 8, multi_tag, clamp_tag, fc_tag);
            }
        };
        using cl0 = std::integral_constant<int, 0>;
        using cl1 = std::integral_constant<int, 1>;
        using cl2 = std::integral_constant<int, 2>;
        if (multi_cls) {
            if (clamp_level == 0)
                columns(std::true_type{}, cl0{}, std::false_type{});
            else if (clamp_level == 1)
                columns(std::true_type{}, cl1{}, std::false_type{});
            else
                columns(std::true_type{}, cl2{}, std::false_type{});
        } else if (f.fcorr) {
            if (clamp_level == 0)
                columns(std::false_type{}, cl0{}, std::true_type{});
            else if (clamp_level == 1)
                columns(std::false_type{}, cl1{}, std::true_type{});
            else
                columns(std::false_type{}, cl2{}, std::true_type{});
        } else {
            if (clamp_level == 0)
                columns(std::false_type{}, cl0{}, std::false_type{});
            else if (clamp_level == 1)
                columns(std::false_type{}, cl1{}, std::false_type{});
            else
                columns(std::false_type{}, cl2{}, std::false_type{});
        }
        // accumulator and residual sub-tile are consumed; staging sub-tiles are written
        fence_before_sync();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(smem_u32(&sh.bar_acc_empty[buf]));
            int c[4];
            if (sub_coords(mt, nt, c)) {
                if (!Y2 || !f.lut_only)
                    store_sub(tmap_y, s_out, c);
                if (Y2)
                    store_sub(tmap_y2, s_y2, c);
            }
            tma_store_commit();
            const int next = tile + RES_BUFS * tstep;
            if (RES && next < total_tiles) {
                int nm;
                const int nn = fdivmod(next, g.fd_m_tiles, nm);
                sub_coords(nm, nn, c);
                mbar_expect_tx(bar_res + rb * 8, res_bytes);
                load_sub(s_res_cur, tmap_res, bar_res + rb * 8, c);
            }
        }
        if (++rb == RES_BUFS)
            rb = 0;
    }
    if (lane == 0)
        tma_store_wait_all();
}

template <int RES, bool Y2, bool XSUM, bool ROWS>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_conv_fast_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ CUtensorMap tmap_y2,
                    const __grid_constant__ CUtensorMap tmap_res, const TcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) TcShared sh;
    const TcGeom &g = a.g;
    const StageGeom sg = stage_geom(g, smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    grid_dependency_release(); // the next kernel of the stream may take the SMs this one leaves
    tc_setup(g, sh, warp);
    const uint32_t tmem_base = sh.tmem_base_slot;
    if (warp == 0) {
        if (lane == 0)
            producer_loop(g, sg, sh, &tmap_a, &tmap_b, a.status, g.load_warps == 2 ? (g.load_by_stage ? 3 : 1) : 0);
    } else if (warp == 1) {
        if (lane == 0)
            mma_loop(g, sg, sh, tmem_base, a.status, g.issuers == 2, 0);
    } else if (warp == WARP_MMA2) {
        if (lane == 0 && g.issuers == 2)
            mma_loop(g, sg, sh, tmem_base, a.status, true, 1);
    } else if (warp == WARP_LOAD2) {
        if (lane == 0 && g.load_warps == 2)
            producer_loop(g, sg, sh, &tmap_a, &tmap_b, a.status, g.load_by_stage ? 4 : 2);
    } else {
        epilogue_fast<RES, Y2, XSUM, ROWS>(a, sg, sh, tmem_base, &tmap_y, &tmap_y2, &tmap_res, warp, lane);
    }
    tc_teardown(g, sh, warp, tmem_base);
}

// ------------------------------------------------------------------------------------------------
// host side: plan creation
// ------------------------------------------------------------------------------------------------
// RN(1/b) as a float, verified against its neighbours in extended precision. The three-operation
// division of the fast epilogue returns the IEEE quotient only with a correctly rounded
// reciprocal; scales far from 1 (where intermediate products could leave the normal range) are
// refused, and the generic epilogue takes the layer.
float rn_reciprocal(float b, bool *ok) {
    if (!(b > 1e-18f && b < 1e18f)) {
        *ok = false;
        return 0.f;
    }
    const long double lb = (long double)b;
    float best = (float)(1.0L / lb);
    const float cand[3] = {best, nextafterf(best, 0.f), nextafterf(best, INFINITY)};
    long double best_err = -1;
    for (float c : cand) {
        long double e = 1.0L - lb * (long double)c; // exact: 24 x 24 bit product, difference near 0
        if (e < 0)
            e = -e;
        if (best_err < 0 || e < best_err) {
            best_err = e;
            best = c;
        }
    }
    return best;
}

// Self-test of the reciprocal division: compares it with the IEEE division for `count` operands
// (random sign and mantissa, exponents spread over [2^-32, 2^32) times the divisor) and counts
// disagreements.
__global__ void reciprocal_division_selftest_kernel(float s, float r, unsigned long long count, unsigned long long seed,
                                                    unsigned long long *mismatches) {
    unsigned long long bad = 0;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (unsigned long long)gridDim.x * blockDim.x) {
        unsigned long long z = (i + seed) * 0x9E3779B97F4A7C15ull; // splitmix64
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        const uint32_t mant = (uint32_t)z & 0x7FFFFFu, sign = (uint32_t)(z >> 23) & 1u;
        const int e = (int)((z >> 24) & 63u) - 32;
        const float x = __uint_as_float((sign << 31) | ((uint32_t)(127 + e) << 23) | mant) * s;
        float q0 = __fmul_rn(x, r);
        q0 = __fmaf_rn(__fmaf_rn(-q0, s, x), r, q0);
        if (q0 != __fdiv_rn(x, s))
            bad++;
    }
    if (bad)
        atomicAdd(mismatches, bad);
}

int reciprocal_division_selftest(nncb_context *ctx, float scale, unsigned long long count, unsigned long long seed,
                                 unsigned long long *mismatches) {
    bool ok = true;
    const float r = rn_reciprocal(scale, &ok);
    if (!ok)
        return fail(-EINVAL, "scale %g is outside the range the reciprocal division accepts", (double)scale);
    unsigned long long *d = nullptr;
    NNCB_CUDA_TRY(cudaMalloc(&d, sizeof(*d)));
    NNCB_CUDA_TRY(cudaMemsetAsync(d, 0, sizeof(*d), ctx->stream));
    reciprocal_division_selftest_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(scale, r, count, seed, d);
    int rc = after_launch(ctx, "reciprocal_division_selftest");
    if (rc == 0) {
        cudaError_t e = cudaMemcpyAsync(mismatches, d, sizeof(*d), cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess)
            e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess)
            rc = fail(-EIO, "self-test copy failed: %s", cudaGetErrorString(e));
    }
    cudaFree(d);
    return rc;
}

// ------------------------------------------------------------------------------------------------
// Peak of the kind::i8 tensor pipe, measured: the denominator of every "fraction of int8 peak".
// One CTA per SM; one thread issues back-to-back tcgen05.mma kind::i8 of M = 128, N = 256, K = 32 on one
// resident pair of shared-memory operand tiles (128-byte swizzle, pseudo-random bytes) into two
// alternating TMEM accumulators. No global-memory traffic, no epilogue: nothing but the tensor pipe can
// bound it. Every `sync` MMAs the thread commits to an mbarrier and waits (bounded) so that the issue
// queue stays shallow.
// ------------------------------------------------------------------------------------------------
struct PeakShared {
    uint64_t bar;
    uint32_t tmem_slot;
    volatile int abort_flag;
    unsigned wait_limit_us; // must follow abort_flag (read by mbar_wait_slow through the flag's address)
};

__global__ void __launch_bounds__(128, 1) int8_peak_kernel(uint32_t mma_groups, uint32_t idesc, int *status, unsigned limit_us) {
    using namespace dev;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) PeakShared sh;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_tile = base, b_tile = base + 128u * 128u; // A: 128 rows x 128 B, B: 256 rows x 128 B
    for (uint32_t i = threadIdx.x; i < (128u + 256u) * 128u / 4u; i += blockDim.x) {
        uint32_t v = (i + 1u) * 2654435761u + blockIdx.x * 40503u;
        v ^= v >> 15;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(base + i * 4u), "r"(v) : "memory");
    }
    fence_async_smem();
    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        sh.wait_limit_us = limit_us;
        mbar_init(smem_u32(&sh.bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int warp = threadIdx.x >> 5;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = sh.tmem_slot;
    if (threadIdx.x == 32) {
        const Desc da = make_desc(smem_desc(a_tile, 128)), db = make_desc(smem_desc(b_tile, 128));
        const uint32_t bar = smem_u32(&sh.bar);
        uint32_t phase = 0;
        constexpr uint32_t sync_every = 64; // groups of four MMAs between two commits
        for (uint32_t g = 0; g < mma_groups; g++) {
            const uint32_t d = tmem + (g & 1u) * 256u;
            mma_i8(d, da, db, idesc, g > 1);
            mma_i8(d, da + 2, db + 2, idesc, 1);
            mma_i8(d, da + 4, db + 4, idesc, 1);
            mma_i8(d, da + 6, db + 6, idesc, 1);
            if ((g + 1) % sync_every == 0 || g + 1 == mma_groups) {
                mma_commit(bar);
                if (!mbar_wait(bar, phase, &sh.abort_flag, status, ERR_MMA_ACC))
                    break;
                phase ^= 1;
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

// Runs the loop `repeats` times (after one warm-up launch), each timed with CUDA events on the context's
// stream; returns the best and the mean rate in TOP/s (2 operations per multiply-accumulate).
int int8_peak_selftest(nncb_context *ctx, uint32_t mmas_per_sm, int repeats, int w_signed, double *best_tops, double *mean_tops) {
    if (mmas_per_sm < 4 || mmas_per_sm > (1u << 24) || repeats < 1 || repeats > 10000)
        return fail(-EINVAL, "int8 peak self-test: 4 <= mmas_per_sm <= 2^24, 1 <= repeats <= 10000");
    const uint32_t groups = mmas_per_sm / 4;
    const uint32_t idesc = (2u << 4) | ((w_signed ? 1u : 0u) << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const size_t smem = (128 + 256) * 128 + 1024;
    // more than half of an SM's shared memory would not be needed, but exactly one CTA (one 512-column TMEM
    // allocation) per SM is: ask for it explicitly
    const size_t smem_one_per_sm = 120 * 1024;
    NNCB_CUDA_TRY(cudaFuncSetAttribute(int8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_one_per_sm));
    (void)smem;
    cudaEvent_t e0, e1;
    NNCB_CUDA_TRY(cudaEventCreate(&e0));
    NNCB_CUDA_TRY(cudaEventCreate(&e1));
    double best = 0, sum = 0;
    int rc = 0;
    for (int r = -1; r < repeats && rc == 0; r++) {
        cudaEventRecord(e0, ctx->stream);
        int8_peak_kernel<<<ctx->sm_count, 128, smem_one_per_sm, ctx->stream>>>(groups, idesc, ctx->d_status, ctx->opt.wait_limit_us);
        rc = after_launch(ctx, "int8_peak");
        cudaEventRecord(e1, ctx->stream);
        cudaError_t e = cudaEventSynchronize(e1);
        if (e != cudaSuccess)
            rc = fail(-EIO, "int8 peak self-test: %s", cudaGetErrorString(e));
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        if (r >= 0 && rc == 0 && ms > 0) {
            const double tops = (double)ctx->sm_count * groups * 4.0 * 2.0 * 128.0 * 256.0 * 32.0 / (ms * 1e-3) / 1e12;
            best = tops > best ? tops : best;
            sum += tops;
        }
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc == 0) {
        *best_tops = best;
        *mean_tops = sum / repeats;
    }
    return rc;
}

// ------------------------------------------------------------------------------------------------
// Pace of MMA issue, measured: cycles per tcgen05.mma kind::i8 (M = 128, K = 32) of `n_cols` columns when one
// or two warps (one lane each) issue them back to back on operand tiles resident in shared memory, each warp into
// its own TMEM accumulator, four MMAs and one descriptor step per loop iteration. It is the floor of a
// convolution's K loop: measured, one issuer keeps the pipe's own pace from 144 columns up (72 cycles per MMA at
// n = 144, 128 at n = 256, i.e. n / 1.9 at 1.965 GHz) and takes 57 cycles at 64 columns, where two issuers reach
// the 48 cycles at which shared memory delivers the operands ((128 + n) / 4). What a real K loop adds per stage --
// a barrier probe, a fence, a commit, ring bookkeeping, each some tens of cycles in a lone thread's dependent
// stream -- is what separates it from these figures.
// ------------------------------------------------------------------------------------------------
struct IssueShared {
    uint64_t bar[2];
    uint32_t tmem_slot;
    volatile int abort_flag;
    unsigned wait_limit_us; // must follow abort_flag (read by mbar_wait_slow through the flag's address)
};

__global__ void __launch_bounds__(128, 1) mma_issue_kernel(uint32_t groups, uint32_t idesc, int issuers, unsigned long long *cycles,
                                                           int *status, unsigned limit_us) {
    using namespace dev;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) IssueShared sh;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_tile = base, b_tile = base + 48u * 1024u; // three A stages of 16 KB, B: 256 rows x 128 B
    for (uint32_t i = threadIdx.x; i < 80u * 1024u / 4u; i += blockDim.x) {
        uint32_t v = (i + 1u) * 2654435761u + blockIdx.x * 40503u;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(base + i * 4u), "r"(v ^ (v >> 15)) : "memory");
    }
    fence_async_smem();
    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        sh.wait_limit_us = limit_us;
        mbar_init(smem_u32(&sh.bar[0]), 1);
        mbar_init(smem_u32(&sh.bar[1]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = sh.tmem_slot;
    if (lane == 0 && warp >= 1 && warp <= issuers) {
        const Desc da0 = make_desc(smem_desc(a_tile, 128)), db = make_desc(smem_desc(b_tile, 128));
        const uint32_t bar = smem_u32(&sh.bar[warp - 1]), d = tmem + (uint32_t)(warp - 1) * 256u;
        uint32_t st = 0;
        const long long t0 = clock64();
        for (uint32_t g = 0; g < groups; g++) {
            const Desc da = da0 + st * 1024u; // a K block of another stage each time, as in a K loop
            mma_i8(d, da, db, idesc, g != 0);
            mma_i8(d, da + 2, db + 2, idesc, 1);
            mma_i8(d, da + 4, db + 4, idesc, 1);
            mma_i8(d, da + 6, db + 6, idesc, 1);
            if (++st == 3)
                st = 0;
        }
        mma_commit(bar);
        mbar_wait(bar, 0, &sh.abort_flag, status, ERR_MMA_ACC);
        const long long t1 = clock64();
        if (warp == 1)
            cycles[blockIdx.x] = (unsigned long long)(t1 - t0);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

// One launch after one warm-up; returns the mean over the SMs of cycles per MMA (all issuers' MMAs counted).
int mma_issue_selftest(nncb_context *ctx, int n_cols, int issuers, uint32_t mmas_per_issuer, double *cycles_per_mma) {
    if (n_cols < 16 || n_cols > 256 || n_cols % 16 != 0 || issuers < 1 || issuers > 2 || mmas_per_issuer < 4 ||
        mmas_per_issuer > (1u << 22))
        return fail(-EINVAL, "mma issue self-test: 16 <= n_cols <= 256 in steps of 16, issuers 1 or 2, 4 <= mmas <= 2^22");
    const uint32_t groups = mmas_per_issuer / 4;
    const uint32_t idesc = (2u << 4) | ((uint32_t)(n_cols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const size_t smem_one_per_sm = 120 * 1024; // more than half of an SM's shared memory: one CTA, one TMEM allocation per SM
    NNCB_CUDA_TRY(cudaFuncSetAttribute(mma_issue_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_one_per_sm));
    unsigned long long *d_cyc = nullptr;
    NNCB_CUDA_TRY(cudaMalloc(&d_cyc, sizeof(unsigned long long) * ctx->sm_count));
    int rc = 0;
    for (int r = 0; r < 2 && rc == 0; r++) {
        mma_issue_kernel<<<ctx->sm_count, 128, smem_one_per_sm, ctx->stream>>>(groups, idesc, issuers, d_cyc, ctx->d_status,
                                                                               ctx->opt.wait_limit_us);
        rc = after_launch(ctx, "mma_issue");
    }
    std::vector<unsigned long long> h(ctx->sm_count);
    if (rc == 0) {
        cudaError_t e = cudaMemcpyAsync(h.data(), d_cyc, sizeof(unsigned long long) * ctx->sm_count, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess)
            e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess)
            rc = fail(-EIO, "mma issue self-test: %s", cudaGetErrorString(e));
    }
    cudaFree(d_cyc);
    if (rc == 0) {
        double sum = 0;
        for (unsigned long long c : h)
            sum += (double)c;
        *cycles_per_mma = sum / ctx->sm_count / ((double)groups * 4.0 * issuers);
    }
    return rc;
}

static int pick_bn(int oc, long long K, const nncb_options &opt) {
    // N tile width. 128, 96, 64, 48 and 32 are the widths the fast epilogue stages; a layer whose channel
    // count is a multiple of 16 takes the one with the least modelled time per 128-pixel tile row. A tile costs
    // the larger of its epilogue (measured: about 1000 clocks of latency plus 22 per column) and its operand
    // loads ((128 + bn) K bytes at 40 per clock): 96 columns cover a 96- or 192-channel layer without waste and
    // in the fewest tiles, 48 a 144-channel one, wide tiles re-read the activations of a deep layer less often.
    if (oc % 16 != 0)
        return oc >= 128 ? 128 : ((oc + 15) / 16) * 16;
    if (opt.conv_tile_n) { // tuning override: force the N tile width (128, 96, 64, 48 or 32)
        const int v = opt.conv_tile_n;
        if (v == 128 || v == 96 || v == 64 || v == 48 || v == 32)
            return v;
    }
    static const int widths[5] = {128, 96, 64, 48, 32};
    int best = 128;
    long long best_cost = -1;
    for (int bn : widths) {
        const long long tiles = (oc + bn - 1) / bn;
        const long long epi = 1000 + 22ll * bn, load = (128ll + bn) * K / 40;
        const long long cost = tiles * (epi > load ? epi : load);
        if (best_cost < 0 || cost < best_cost)
            best_cost = cost, best = bn;
    }
    return best;
}

int tc_conv_create(nncb_context *ctx, nncb_qconv2d *cv, const void *w_host, const int32_t *wzp_host) {
    NNCB_TRY(load_driver_entry_points());
    const nncb_conv2d_desc &d = cv->d;
    TcPlan *tp = new TcPlan();
    cv->tc = tp;
    TcGeom &g = tp->g;
    const bool gemm = d.kh == 1 && d.kw == 1 && d.stride_h == 1 && d.stride_w == 1 && d.pad_t == 0 && d.pad_b == 0 &&
                      d.pad_l == 0 && d.pad_r == 0;
    const bool wide_patch = !gemm && patch_wide_applies(d, ctx->opt);
    g.mode = gemm ? MODE_GEMM
                  : ((wide_patch || patch_mode_applies(d)) ? MODE_PATCH : (rows_mode_applies(d) ? MODE_ROWS : MODE_IM2COL));
    g.oh = cv->oh, g.ow = cv->ow;
    g.wait_limit_us = 1000000, g.withhold = 0;
    g.m_total = d.n * cv->oh * cv->ow;
    g.oc = d.oc;
    bool any_zw = false;
    for (int i = 0; i < d.oc && wzp_host; i++)
        any_zw |= wzp_host[i] != 0;
    g.has_xsum = any_zw ? 1 : 0;
    g.bn = pick_bn(d.oc, (long long)d.kh * d.kw * d.c, ctx->opt);
    g.bn_mma = g.bn + (any_zw ? 16 : 0);
    g.n_tiles = (d.oc + g.bn - 1) / g.bn;
    g.m_tiles = (g.m_total + 127) / 128;
    g.kb = d.c % 128 == 0 ? 128 : (d.c % 64 == 0 ? 64 : 32);
    g.c_blocks = d.c / g.kb;
    g.taps = d.kh * d.kw;
    g.kw = d.kw;
    if (g.mode == MODE_ROWS) {
        // patch shape: the one that covers the output with the fewest wasted rows; wider on a tie
        long long best = -1;
        for (int l = 7; l >= 3; l--) {
            const int bx = 1 << l, by = 128 >> l;
            const long long area = (long long)((g.ow + bx - 1) / bx) * bx * ((g.oh + by - 1) / by) * by;
            if (best < 0 || area < best)
                best = area, g.bx_log2 = l;
        }
        const int bx = 1 << g.bx_log2, by = 128 >> g.bx_log2;
        g.tiles_x = (g.ow + bx - 1) / bx, g.tiles_y = (g.oh + by - 1) / by;
        g.m_tiles = d.n * g.tiles_x * g.tiles_y;
        g.kb = d.kw * d.c; // one K block per kernel row
        g.c_blocks = 1;
        g.taps = d.kh;
        g.kw = 1;
    }
    if (g.mode == MODE_PATCH) {
        g.bx_log2 = 3; // 8 x 16 output pixels
        g.tiles_x = (g.ow + 7) / 8, g.tiles_y = (g.oh + 15) / 16;
        g.m_tiles = d.n * g.tiles_x * g.tiles_y;
        g.kh = d.kh, g.kw_cells = d.kw;
        g.patch_w = 8 + d.kw - 1, g.patch_h = 16 + d.kh - 1;
        if (wide_patch) {
            g.cell = d.c; // the weights keep the layout of MODE_IM2COL: one K block of c bytes per tap
        } else {
            g.cell = 16;
            g.kb = d.kw * d.c; // the weights keep the layout of MODE_ROWS: one K block per kernel row
            g.c_blocks = 1;
            g.taps = d.kh;
            g.kw = 1;
        }
    }
    g.fd_m_tiles = make_fastdiv(g.m_tiles), g.fd_ow = make_fastdiv(g.ow), g.fd_oh = make_fastdiv(g.oh);
    g.fd_tiles_x = make_fastdiv(g.tiles_x), g.fd_tiles_y = make_fastdiv(g.tiles_y);
    g.stride_h = d.stride_h, g.stride_w = d.stride_w, g.pad_t = d.pad_t, g.pad_l = d.pad_l;
    g.dil_h = d.dil_h, g.dil_w = d.dil_w;
    g.x_zp = d.x_zp;
    g.c = d.c;
    g.f32_out = d.f32_out;
    g.acc_stride = g.bn_mma;
    int cols = 32;
    while (cols < 2 * g.acc_stride)
        cols *= 2;
    g.tmem_cols = cols;
    g.idesc = (2u << 4) | (0u << 7) | ((d.w_signed ? 1u : 0u) << 10) | ((uint32_t)(g.bn_mma >> 3) << 17) |
              ((uint32_t)(128 >> 4) << 24);
    // ---- fast epilogue: constants, error bounds and shared-memory layout ----
    // An activation table on the output runs through the second-output machinery (table in shared
    // memory, mapped tile staged and stored), with the unmapped tile left unstored.
    const bool lut_only = cv->d_lut != nullptr && !d.has_y2 && !d.has_residual;
    const bool fast_shape = !d.f32_out && (cv->d_lut == nullptr || lut_only) && d.oc % 16 == 0 &&
                            (g.bn == 128 || g.bn == 96 || g.bn == 64 || g.bn == 48 || g.bn == 32);
    tp->f = new FastEpi();
    FastEpi &fe = *tp->f;
    memset(&fe, 0, sizeof(fe));
    const uint32_t a_stage = g.mode == MODE_PATCH ? (((uint32_t)g.patch_w * g.cell * g.patch_h + 1023u) & ~1023u) : 128u * g.kb;
    const uint32_t b_pitch = ((uint32_t)g.bn_mma * g.kb + 1023u) & ~1023u;
    const uint32_t budget = 224u * 1024u - 1024u; // dynamic shared memory we may use, minus alignment slack
    uint32_t extras = 0;
    tp->fast = false;
    if (fast_shape) {
        // 64- and 32-column tiles: eight warps per tile (four lane quarters x two column groups), the two
        // halves of the sixteen take alternate tiles; every warp has its own staging sub-tile, so the
        // staging areas hold two tiles
        fe.halves = (g.bn == 64 || g.bn == 32) ? 2 : 1;
        const uint32_t tile_bytes = ((uint32_t)fe.halves * 128u * g.bn + 1023u) & ~1023u;
        uint32_t off = 0;
        fe.off_out = off, off += tile_bytes;
        fe.off_y2 = off, off += (d.has_y2 || lut_only) ? tile_bytes : 0;
        fe.lut_only = lut_only ? 1 : 0;
        fe.off_res = off, off += d.has_residual ? RES_BUFS * tile_bytes : 0;
        fe.res_pitch = tile_bytes;
        fe.off_cst = off, off += (uint32_t)g.bn * 16;
        fe.off_lut2 = off, off += 256;
        // The fused residual add: a look-up in a table of all byte pairs (65 KB of shared memory, one load per
        // output), or -- option conv.add_table = 2 -- the float chain itself on packed arithmetic (about six more
        // instructions per output, no table, room for four pipeline stages instead of two on a 128 x 144 tile with
        // several K blocks). Measured on the 16 such layers of ResNet-50 at 512 images, table -> arithmetic: 56 x 56
        // 434 -> 538 us, 28 x 28 233 -> 271, 14 x 14 (K 256) 137 -> 148, 7 x 7 (K 512) 91.5 -> 92.6; 3.33 -> 3.91 ms
        // in all. The table stays the default everywhere: the epilogue's instruction issue, not the table's
        // look-ups or the depth of the ring, is what these layers wait for.
        if (d.has_residual)
            fe.add_math = ctx->opt.conv_add_table == 2 ? 1 : 0;
        fe.off_tab = off, off += (d.has_residual && !fe.add_math) ? ADD_TABLE_BYTES : 0;
        fe.off_corr = off;
        extras = off; // the per-class table is appended once the classes are known
        // each epilogue warp stages a 32-row x wcols-byte sub-tile; 32-byte rows are the swizzle span
        fe.wcols = g.bn >= 64 ? 32 : 16;
        fe.ncg = g.bn / fe.wcols; // 128: 4 x 32, 96: 3 x 32, 64: 2 x 32, 48: 3 x 16, 32: 2 x 16
        fe.out_sw = fe.wcols == 32 ? 32 : 0;
        tp->fast = true;
    }
    // ---- weights: [n_tiles][bn_mma][K], K ordered (ky, kx, c) = the OHWI row as given ----
    const size_t K = (size_t)d.kh * d.kw * d.c;
    std::vector<uint8_t> wp((size_t)g.n_tiles * g.bn_mma * K, 0);
    const uint8_t *wsrc = reinterpret_cast<const uint8_t *>(w_host);
    for (int nt = 0; nt < g.n_tiles; nt++) {
        for (int r = 0; r < g.bn; r++) {
            int oc = nt * g.bn + r;
            if (oc < d.oc)
                memcpy(&wp[((size_t)nt * g.bn_mma + r) * K], wsrc + (size_t)oc * K, K);
        }
        if (any_zw)
            memset(&wp[((size_t)nt * g.bn_mma + g.bn) * K], 1, K); // all-ones row: per-pixel sum of xq
    }
    NNCB_CUDA_TRY(cudaMalloc(&tp->d_wpack, wp.size()));
    NNCB_CUDA_TRY(cudaMemcpyAsync(tp->d_wpack, wp.data(), wp.size(), cudaMemcpyHostToDevice, ctx->stream));
    NNCB_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    {
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)g.n_tiles * g.bn_mma};
        cuuint64_t strides[1] = {(cuuint64_t)K};
        cuuint32_t box[2] = {(cuuint32_t)g.kb, (cuuint32_t)g.bn_mma};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = g_encode_tiled(&tp->tmap_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, tp->d_wpack, dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(g.kb), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(-EIO, "encoding the weight tensor map failed (CUresult %d)", (int)r);
    }

    // ---- border classes: distinct ranges of valid taps along y and along x ----
    auto classes = [](int out, int in, int k, int stride, int pad, int dil, std::vector<uint8_t> &cls,
                      std::vector<std::pair<int, int>> &ranges) -> bool {
        cls.resize(out);
        for (int o = 0; o < out; o++) {
            int origin = o * stride - pad;
            int lo = 0, hi = k;
            while (lo < k && origin + lo * dil < 0)
                lo++;
            while (hi > lo && origin + (hi - 1) * dil >= in)
                hi--;
            std::pair<int, int> r(lo, hi);
            size_t idx = 0;
            for (; idx < ranges.size(); idx++)
                if (ranges[idx] == r)
                    break;
            if (idx == ranges.size())
                ranges.push_back(r);
            if (idx > 255)
                return false;
            cls[o] = (uint8_t)idx;
        }
        return true;
    };
    std::vector<uint8_t> ycls, xcls;
    std::vector<std::pair<int, int>> yr, xr;
    if (!classes(cv->oh, d.h, d.kh, d.stride_h, d.pad_t, d.dil_h, ycls, yr) ||
        !classes(cv->ow, d.w, d.kw, d.stride_w, d.pad_l, d.dil_w, xcls, xr))
        return fail(-ENOSYS, "tcgen05 conv: too many border classes");
    g.n_cls_x = (int)xr.size();
    const int n_cls = (int)(yr.size() * xr.size());
    tp->oc_pad = g.n_tiles * g.bn;
    // per-tap weight sums, then per-class sums
    const int all_taps = d.kh * d.kw; // g.taps counts K blocks per channel block, which MODE_ROWS merges
    std::vector<int64_t> tapsum((size_t)d.oc * all_taps, 0);
    for (int oc = 0; oc < d.oc; oc++)
        for (int t = 0; t < all_taps; t++) {
            int64_t s = 0;
            const uint8_t *p = wsrc + ((size_t)oc * all_taps + t) * d.c;
            for (int c = 0; c < d.c; c++)
                s += d.w_signed ? (int)(int8_t)p[c] : (int)p[c];
            tapsum[(size_t)oc * all_taps + t] = s;
        }
    std::vector<int32_t> corr((size_t)n_cls * tp->oc_pad, 0), cnt(n_cls, 0);
    for (size_t yc = 0; yc < yr.size(); yc++)
        for (size_t xc = 0; xc < xr.size(); xc++) {
            const int cls = (int)(yc * xr.size() + xc);
            cnt[cls] = (yr[yc].second - yr[yc].first) * (xr[xc].second - xr[xc].first) * d.c;
            for (int oc = 0; oc < d.oc; oc++) {
                int64_t s = 0;
                for (int ky = yr[yc].first; ky < yr[yc].second; ky++)
                    for (int kx = xr[xc].first; kx < xr[xc].second; kx++)
                        s += tapsum[(size_t)oc * all_taps + ky * d.kw + kx];
                corr[(size_t)cls * tp->oc_pad + oc] = (int32_t)(s * d.x_zp);
            }
        }
    NNCB_CUDA_TRY(cudaMalloc(&tp->d_corr, corr.size() * 4));
    NNCB_CUDA_TRY(cudaMalloc(&tp->d_cnt, cnt.size() * 4));
    NNCB_CUDA_TRY(cudaMalloc(&tp->d_ycls, ycls.size()));
    NNCB_CUDA_TRY(cudaMalloc(&tp->d_xcls, xcls.size()));
    NNCB_CUDA_TRY(cudaMemcpyAsync(tp->d_corr, corr.data(), corr.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    NNCB_CUDA_TRY(cudaMemcpyAsync(tp->d_cnt, cnt.data(), cnt.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    NNCB_CUDA_TRY(cudaMemcpyAsync(tp->d_ycls, ycls.data(), ycls.size(), cudaMemcpyHostToDevice, ctx->stream));
    NNCB_CUDA_TRY(cudaMemcpyAsync(tp->d_xcls, xcls.data(), xcls.size(), cudaMemcpyHostToDevice, ctx->stream));

    if (tp->fast) {
        fe.n_cls = n_cls;
        // |sum x w|, |zw rowsum| and |corr| are each at most 255 * 255 * K: with K <= 128 every intermediate of
        // acc - corr - zw * rowsum stays below 2^24 and float arithmetic on these integers is exact
        fe.fcorr = (n_cls == 1 && (long long)d.kh * d.kw * d.c <= 128) ? 1 : 0;
        fe.corr_pitch = g.bn + 1;
        if (n_cls > 1)
            extras += (uint32_t)n_cls * fe.corr_pitch * 4;
        extras = (extras + 1023u) & ~1023u;
        std::vector<float> hm(d.oc), hb(d.oc);
        NNCB_CUDA_TRY(cudaMemcpy(hm.data(), cv->d_mult, sizeof(float) * d.oc, cudaMemcpyDeviceToHost));
        NNCB_CUDA_TRY(cudaMemcpy(hb.data(), cv->d_bias, sizeof(float) * d.oc, cudaMemcpyDeviceToHost));
        std::vector<float4> cst(tp->oc_pad, make_float4(0, 0, 0, 0));
        for (int oc = 0; oc < d.oc; oc++) {
            const int32_t c0 = corr[oc], nzw = wzp_host ? -wzp_host[oc] : 0;
            float4 k;
            k.x = hm[oc], k.y = hb[oc];
            memcpy(&k.z, &c0, 4);
            memcpy(&k.w, &nzw, 4);
            cst[oc] = k;
        }
        bool ok = true;
        fe.so = d.out_scale, fe.zo = (float)d.out_zp;
        fe.rso = rn_reciprocal(d.out_scale, &ok);
        fe.one = 1.0f;
        // quantized clamp bounds: q(clamp(v, lo, hi)) == clamp(q(v), q(lo), q(hi)) for the monotone q
        auto quant = [&](float v) {
            if (std::isinf(v))
                return v < 0 ? 0.f : 255.f;
            const float t = v / d.out_scale;
            const float u = t + (float)d.out_zp;
            return std::fmin(std::fmax(rintf(u), 0.f), 255.f);
        };
        fe.qlo = quant(d.clamp_lo), fe.qhi = quant(d.clamp_hi);
        std::vector<uint8_t> addtab;
        if (d.has_residual) {
            // every (convolution output byte, residual byte) pair through the unfused chain:
            // dequantize both, add, divide by the output scale, add the zero point, round, clamp
            ok = ok && d.res_zp >= 0 && d.res_zp <= 255;
            addtab.assign(ADD_TABLE_BYTES, 0);
            const float so = d.out_scale, zo = (float)d.out_zp, sr = d.res_scale, zr = (float)d.res_zp;
            const float sa = d.add_out_scale, za = (float)d.add_out_zp;
            fe.add_nzr = -zr, fe.add_sr = sr, fe.add_za = za, fe.add_nsa = -sa;
            bool ok_sa = true;
            fe.add_rsa = rn_reciprocal(sa, &ok_sa);
            if (!ok_sa && fe.add_math)
                return fail(-ENOSYS, "tcgen05 conv: the fused add's output scale is outside the range of the exact division");
            for (int qa = 0; qa < 256; qa++) {
                const float da = (float)qa - zo;
                const float ya = da * so;
                for (int r = 0; r < 256; r++) {
                    const float dr = (float)r - zr;
                    const float yb = dr * sr;
                    const float sum = ya + yb;
                    const float p = sum / sa;
                    const float u = p + za;
                    addtab[qa * 260 + r] = (uint8_t)std::fmin(std::fmax(rintf(u), 0.f), 255.f);
                }
            }
        }
        if (!ok || std::isnan(d.clamp_lo) || std::isnan(d.clamp_hi))
            tp->fast = false; // scales outside the range the reciprocal division is proven for
        if (tp->fast) {
            NNCB_CUDA_TRY(cudaMalloc(&tp->d_cst, cst.size() * sizeof(float4)));
            NNCB_CUDA_TRY(cudaMemcpyAsync(tp->d_cst, cst.data(), cst.size() * sizeof(float4), cudaMemcpyHostToDevice, ctx->stream));
            fe.cst = tp->d_cst;
            if (!addtab.empty() && !fe.add_math) {
                NNCB_CUDA_TRY(cudaMalloc(&tp->d_addtab, addtab.size()));
                NNCB_CUDA_TRY(cudaMemcpyAsync(tp->d_addtab, addtab.data(), addtab.size(), cudaMemcpyHostToDevice, ctx->stream));
                fe.add_table = tp->d_addtab;
            }
        }
    }
    NNCB_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    if (!tp->fast)
        extras = 0;
    if (extras + 2 * (a_stage + b_pitch) > budget) {
        tp->fast = false; // not enough room for the staging tiles next to two pipeline stages
        extras = 0;
    }
    // A weight matrix of one N tile that fits beside four activation stages stays resident: the
    // loads are bound by rows moved per clock, and weights are 40 % of the rows of a 64-channel layer.
    const uint32_t k_blocks = (uint32_t)(g.taps * g.c_blocks);
    const uint32_t b_all = k_blocks * b_pitch;
    g.b_resident = g.n_tiles == 1 && b_all <= 64u * 1024u && extras + b_all + 4 * a_stage <= budget;
    const uint32_t per_kblock = a_stage + (g.b_resident ? 0u : b_pitch);
    // Several small K blocks share a stage: the barrier round trip and the commit cost a few hundred
    // cycles per stage whatever its size. Stages of up to 32 KB (larger K blocks already carry enough
    // MMA work each), a count that divides the K blocks if there is one, and at least three stages.
    const uint32_t room = budget - extras - (g.b_resident ? b_all : 0u);
    g.kgroup = 1;
    int fallback = 1;
    for (uint32_t k = 4; k >= 2; k--) {
        if (k > k_blocks || k * per_kblock > 32u * 1024u || 3 * k * per_kblock > room)
            continue;
        if (k_blocks % k == 0) {
            g.kgroup = (int)k;
            break;
        }
        if (fallback == 1)
            fallback = (int)k;
    }
    if (g.kgroup == 1)
        g.kgroup = fallback;
    if (g.mode == MODE_PATCH) {
        if (!g.b_resident || g.n_tiles != 1)
            return fail(-ENOSYS, "tcgen05 conv: patch mode without resident weights");
        g.kgroup = 1; // a stage is one tile's patch
    }
    const uint32_t per_stage = (uint32_t)g.kgroup * per_kblock;
    int stages = (int)(room / per_stage);
    if (stages > MAX_STAGES)
        stages = MAX_STAGES;
    if (stages < 2)
        return fail(-ENOSYS, "tcgen05 conv: tile does not fit shared memory");
    // Deep K loops are bound by the instruction streams of the one-thread roles and by the latency of the stage
    // ring, not by the tensor pipe or the load bandwidth: two MMA issuers and two load warps take the stages in
    // turn. Measured on ResNet-50 at 512 images: tiles of eight or more stages gain (3x3 layers over 256 and 512
    // channels 72 -> 67 us, 1x1 layers with K = 2048 40 -> 36 us), tiles of four stages lose a few per cent.
    const uint32_t stage_groups = (k_blocks + (uint32_t)g.kgroup - 1) / (uint32_t)g.kgroup;
    const bool deep = g.mode != MODE_PATCH && stage_groups >= 8;
    const int want_issuers = ctx->opt.conv_mma_issuers ? ctx->opt.conv_mma_issuers : (deep ? 2 : 1);
    const int want_loaders = ctx->opt.conv_load_warps ? ctx->opt.conv_load_warps : (deep ? 3 : 1);
    // (patch mode: the taps of a tile are dealt out instead; only the filter sizes with straight-line code)
    // 18 or 36 MMAs per tile pay for the second issuer; the 8 of a 4 x 4-cell stem do not (measured: 349 us with
    // one issuer, 377 us with two, ResNet-50 stem at 512 images)
    const bool patch_dual = g.mode == MODE_PATCH && g.cell != 16 && g.kh == 3 && g.kw_cells == 3;
    const int want_patch = ctx->opt.conv_mma_issuers ? ctx->opt.conv_mma_issuers : 2;
    g.issuers = g.mode == MODE_PATCH ? ((patch_dual && want_patch == 2) ? 2 : 1) : (want_issuers == 2 ? 2 : 1);
    g.load_by_stage = want_loaders == 3 && g.mode != MODE_PATCH ? 1 : 0;
    g.load_warps = (g.load_by_stage || (want_loaders == 2 && g.mode != MODE_PATCH && !g.b_resident)) ? 2 : 1;
    g.stages = stages;
    g.acc_arrivals = tp->fast ? 4 * fe.ncg : EPI_WARPS;
    const uint32_t ring = (uint32_t)stages * per_stage + (g.b_resident ? b_all : 0u);
    if (tp->fast) {
        fe.off_out += ring, fe.off_y2 += ring, fe.off_res += ring, fe.off_cst += ring;
        fe.off_lut2 += ring, fe.off_corr += ring, fe.off_tab += ring;
    }
    // More than half of an SM's shared memory, so exactly one CTA (and one TMEM allocation) per SM.
    tp->smem_bytes = (size_t)ring + extras + 1024;
    if (tp->smem_bytes < 120 * 1024)
        tp->smem_bytes = 120 * 1024;
    // The limit is a property of the function, not of the plan: raise it once to the most any
    // plan can ask for.
    const int lim = 226 * 1024;
    NNCB_CUDA_TRY(cudaFuncSetAttribute(tc_conv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    const void *fast_kernels[24] = {
#define NNCB_K(R, Y, X) (const void *)tc_conv_fast_kernel<R, Y, X, false>, (const void *)tc_conv_fast_kernel<R, Y, X, true>
        NNCB_K(0, false, false), NNCB_K(0, false, true), NNCB_K(0, true, false), NNCB_K(0, true, true),
        NNCB_K(1, false, false), NNCB_K(1, false, true), NNCB_K(1, true, false), NNCB_K(1, true, true),
        NNCB_K(2, false, false), NNCB_K(2, false, true), NNCB_K(2, true, false), NNCB_K(2, true, true)
#undef NNCB_K
    };
    for (const void *k : fast_kernels)
        NNCB_CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    return 0;
}

void tc_conv_destroy(nncb_qconv2d *cv) {
    TcPlan *tp = cv->tc;
    if (!tp)
        return;
    cudaFree(tp->d_wpack);
    cudaFree(tp->d_corr);
    cudaFree(tp->d_cnt);
    cudaFree(tp->d_ycls);
    cudaFree(tp->d_xcls);
    cudaFree(tp->d_cst);
    cudaFree(tp->d_addtab);
    delete tp->f;
    delete tp;
    cv->tc = nullptr;
}

static int make_tmap_out(CUtensorMap *map, const TcPlan *tp, const void *ptr) {
    const TcGeom &g = tp->g;
    const int sw = tp->f->out_sw;
    CUtensorMapSwizzle swz = sw == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                       : (sw == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                   : (sw == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE));
    CUresult r;
    if (g.mode == MODE_ROWS || g.mode == MODE_PATCH) {
        // a warp's 32 rows are sx x sy pixels of the patch
        const int bx = 1 << g.bx_log2, sx = bx < 32 ? bx : 32;
        const int n_img = g.m_total / (g.oh * g.ow);
        cuuint64_t dims[4] = {(cuuint64_t)g.oc, (cuuint64_t)g.ow, (cuuint64_t)g.oh, (cuuint64_t)n_img};
        cuuint64_t strides[3] = {(cuuint64_t)g.oc, (cuuint64_t)g.oc * g.ow, (cuuint64_t)g.oc * g.ow * g.oh};
        cuuint32_t box[4] = {(cuuint32_t)tp->f->wcols, (cuuint32_t)sx, (cuuint32_t)(32 / sx), 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        r = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        cuuint64_t dims[2] = {(cuuint64_t)g.oc, (cuuint64_t)g.m_total};
        cuuint64_t strides[1] = {(cuuint64_t)g.oc};
        cuuint32_t box[2] = {(cuuint32_t)tp->f->wcols, 32}; // one epilogue warp's sub-tile
        cuuint32_t estr[2] = {1, 1};
        r = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS)
        return fail(-EIO, "encoding an output tensor map failed (CUresult %d)", (int)r);
    return 0;
}

int tc_conv_run(nncb_context *ctx, nncb_qconv2d *cv, const uint8_t *x, const uint8_t *res, void *y, uint8_t *y2) {
    TcPlan *tp = cv->tc;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0)
        return fail(-EINVAL, "tcgen05 conv: activation pointer must be 16-byte aligned");
    if (tp->a_ptr != x)
        NNCB_TRY(make_tmap_a(tp, cv->d, x));
    TcArgs a;
    a.g = tp->g;
    a.g.wait_limit_us = ctx->opt.wait_limit_us;
    a.g.withhold = ctx->opt.debug_withhold_load;
    a.p = make_epi(cv);
    a.f = *tp->f;
    a.corr = tp->d_corr;
    a.cnt = tp->d_cnt;
    a.ycls = tp->d_ycls;
    a.xcls = tp->d_xcls;
    a.w_zp = cv->d_wzp;
    a.oc_pad = tp->oc_pad;
    a.res = res;
    a.y = y;
    a.y2 = y2;
    a.status = ctx->d_status;
    const int tiles = tp->g.m_tiles * tp->g.n_tiles;
    const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    // the two further role warps exist only in plans that use them: every warp of the block meets the set-up and
    // tear-down barriers, and short launches (single images, narrow layers) feel two idle warps
    const int threads = (tp->g.issuers == 2 || tp->g.load_warps == 2) ? TC_THREADS : TC_THREADS - 64;
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (tp->fast && al16(y) && al16(y2) && al16(res)) {
        if (tp->f->lut_only) {
            a.p.y2_lut = cv->d_lut;
            y2 = static_cast<uint8_t *>(y);
        }
        if (tp->y_ptr != y) {
            NNCB_TRY(make_tmap_out(&tp->tmap_y, tp, y));
            tp->y_ptr = y;
        }
        if (y2 && tp->y2_ptr != y2) {
            NNCB_TRY(make_tmap_out(&tp->tmap_y2, tp, y2));
            tp->y2_ptr = y2;
        }
        if (res && tp->res_ptr != res) {
            NNCB_TRY(make_tmap_out(&tp->tmap_res, tp, res));
            tp->res_ptr = res;
        }
        const CUtensorMap &my2 = y2 ? tp->tmap_y2 : tp->tmap_y, &mres = res ? tp->tmap_res : tp->tmap_y;
        const int variant = (res ? (tp->f->add_math ? 8 : 4) : 0) | (y2 ? 2 : 0) | (tp->g.has_xsum ? 1 : 0);
#define NNCB_LAUNCH_FAST(R, Y, C)                                                                                     \
    do {                                                                                                              \
        if (tp->g.mode == MODE_ROWS || tp->g.mode == MODE_PATCH)                                                      \
            launch_dependent(ctx, tc_conv_fast_kernel<R, Y, C, true>, dim3(grid), dim3(threads), tp->smem_bytes,        \
                             tp->tmap_a, tp->tmap_b, tp->tmap_y, my2, mres, a);                                       \
        else                                                                                                          \
            launch_dependent(ctx, tc_conv_fast_kernel<R, Y, C, false>, dim3(grid), dim3(threads), tp->smem_bytes,       \
                             tp->tmap_a, tp->tmap_b, tp->tmap_y, my2, mres, a);                                       \
    } while (0)
        switch (variant) {
        case 0: NNCB_LAUNCH_FAST(0, false, false); break;
        case 1: NNCB_LAUNCH_FAST(0, false, true); break;
        case 2: NNCB_LAUNCH_FAST(0, true, false); break;
        case 3: NNCB_LAUNCH_FAST(0, true, true); break;
        case 4: NNCB_LAUNCH_FAST(1, false, false); break;
        case 5: NNCB_LAUNCH_FAST(1, false, true); break;
        case 6: NNCB_LAUNCH_FAST(1, true, false); break;
        case 7: NNCB_LAUNCH_FAST(1, true, true); break;
        case 8: NNCB_LAUNCH_FAST(2, false, false); break;
        case 9: NNCB_LAUNCH_FAST(2, false, true); break;
        case 10: NNCB_LAUNCH_FAST(2, true, false); break;
        default: NNCB_LAUNCH_FAST(2, true, true); break;
        }
#undef NNCB_LAUNCH_FAST
        return after_launch(ctx, "tc_conv_fast");
    }
    launch_dependent(ctx, tc_conv_kernel, dim3(grid), dim3(threads), tp->smem_bytes, tp->tmap_a, tp->tmap_b, a);
    return after_launch(ctx, "tc_conv");
}

} // namespace nncb
