// CUDA-core quantized Conv2D: the general path (any stride, dilation, padding, groups --
// depthwise included -- and channel counts the tensor-core kernel does not take, such as the
// 3-channel stem). One thread per (output pixel, output channel); consecutive threads own
// consecutive output channels, so activation loads broadcast within a warp and stores coalesce.
#include "qconv.cuh"
#include <cmath>
#include <vector>

namespace nncb {

struct SimtGeom {
    int n, h, w, c, oc, kh, kw, sh, sw, pt, pl, dh, dw, groups, oh, ow, w_signed, x_zp, f32_out;
};

template <bool W_SIGNED>
__device__ __forceinline__ int load_w(const void *w, size_t i) {
    if (W_SIGNED)
        return (int)reinterpret_cast<const int8_t *>(w)[i];
    return (int)reinterpret_cast<const uint8_t *>(w)[i];
}

template <bool W_SIGNED>
__global__ void __launch_bounds__(256)
simt_conv_kernel(SimtGeom g, const uint8_t *__restrict__ x, const void *__restrict__ w,
                 const int32_t *__restrict__ w_zp, EpiParams p, const uint8_t *__restrict__ res,
                 void *__restrict__ y, uint8_t *__restrict__ y2) {
    grid_dependency_release(); // a tensor-core convolution that follows sets itself up meanwhile
    const int gic = g.c / g.groups, goc = g.oc / g.groups;
    const size_t total = (size_t)g.n * g.oh * g.ow * g.oc;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        // 32-bit index arithmetic when the index fits: a 64-bit division costs some seventy instructions
        int oc, ox, oy, b;
        if (i <= 0xffffffffull) {
            const uint32_t ii = (uint32_t)i, px = ii / (uint32_t)g.oc, row = px / (uint32_t)g.ow;
            oc = (int)(ii % (uint32_t)g.oc), ox = (int)(px % (uint32_t)g.ow);
            oy = (int)(row % (uint32_t)g.oh), b = (int)(row / (uint32_t)g.oh);
        } else {
            const size_t pix = i / g.oc;
            oc = (int)(i % g.oc);
            ox = (int)(pix % g.ow);
            oy = (int)((pix / g.ow) % g.oh);
            b = (int)(pix / ((size_t)g.ow * g.oh));
        }
        const int grp = oc / goc;
        const int zw = w_zp[oc];
        const int iy0 = oy * g.sh - g.pt, ix0 = ox * g.sw - g.pl;
        int acc = 0;
        const bool vec4 = (gic % 4 == 0) && (g.c % 4 == 0);
        for (int ky = 0; ky < g.kh; ky++) {
            const int iy = iy0 + ky * g.dh;
            if (iy < 0 || iy >= g.h)
                continue;
            for (int kx = 0; kx < g.kw; kx++) {
                const int ix = ix0 + kx * g.dw;
                if (ix < 0 || ix >= g.w)
                    continue;
                const uint8_t *xp = x + (((size_t)b * g.h + iy) * g.w + ix) * g.c + grp * gic;
                const size_t wo = (((size_t)oc * g.kh + ky) * g.kw + kx) * gic;
                if (vec4) {
                    // sum (x - zx)(w - zw) = sum x*w - zx*sum w - zw*sum x + cnt*zx*zw, via dp4a
                    const uint32_t *xv = reinterpret_cast<const uint32_t *>(xp);
                    const uint32_t *wv = reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(w) + wo);
                    int sxw = 0, sx = 0, sw_ = 0;
                    for (int k = 0; k < gic / 4; k++) {
                        uint32_t xa = __ldg(xv + k), wa = __ldg(wv + k);
                        if (W_SIGNED) {
                            // x unsigned, w signed
                            asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(sxw) : "r"(xa), "r"(wa), "r"(sxw));
                            asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(sw_) : "r"(wa), "r"(0x01010101u), "r"(sw_));
                        } else {
                            sxw = (int)__dp4a(xa, wa, (unsigned)sxw);
                            sw_ = (int)__dp4a(wa, 0x01010101u, (unsigned)sw_);
                        }
                        sx = (int)__dp4a(xa, 0x01010101u, (unsigned)sx);
                    }
                    acc += sxw - g.x_zp * sw_ - zw * sx + gic * g.x_zp * zw;
                } else {
                    int s = 0;
                    for (int ic = 0; ic < gic; ic++)
                        s += ((int)xp[ic] - g.x_zp) * (load_w<W_SIGNED>(w, wo + ic) - zw);
                    acc += s;
                }
            }
        }
        const float mult = p.mult[oc], bias = p.bias[oc];
        if (g.f32_out) {
            reinterpret_cast<float *>(y)[i] = epi_real(acc, mult, bias, p.clamp_lo, p.clamp_hi);
        } else {
            int q = epi_u8(acc, mult, bias, p, p.has_res ? (int)res[i] : 0);
            reinterpret_cast<uint8_t *>(y)[i] = (uint8_t)q;
            if (y2)
                y2[i] = p.y2_lut[q];
        }
    }
}

// ---- depthwise (groups == c == oc, c % 4 == 0, u8 output) ----------------------------------------
// A streaming kernel: one thread per (output pixel, four channels); a warp reads 128 contiguous bytes
// of every tap and writes 128 contiguous bytes. The weights are prepared at plan creation as
// (w - zw) in int16, tap-major, so that four channels of a tap are one 8-byte load. Padded taps are
// skipped, which is what the normative formulation says (they contribute (zx - zx) * w = 0).
struct DwFast {
    int on;            // no residual, no activation table: requantise without a division
    float so, rso, zo; // output scale, its verified reciprocal, zero point
    float qlo, qhi;    // the fused clamp as quantized bounds
};

// rint (nearest even) and clamp to 0..255 in one conversion
__device__ __forceinline__ uint32_t rint_sat_u8(float v) {
    uint32_t q;
    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q) : "f"(v));
    return q;
}

// The division-free exact requantisation on two accumulators at once (f32x2 instructions): v = acc * mult + bias,
// v / so as q0 = RN(v r), q = RN(q0 + RN(v - q0 so) r), + zo, the clamp folded into the quantized bounds, one
// saturating round-to-nearest-even conversion each.
__device__ __forceinline__ void dw_requant2(int a0, int a1, float m0, float m1, float b0, float b1, const DwFast &f, int &q0o,
                                            int &q1o) {
    // the product must round before the bias is added: the assembler contracts a packed multiply and a packed
    // add into one fused operation even when both carry .rn, so the add is two scalar ones
    float p0, p1;
    unpack2(mul2(pack2((float)a0, (float)a1), pack2(m0, m1)), p0, p1);
    const uint64_t v2 = pack2(__fadd_rn(p0, b0), __fadd_rn(p1, b1));
    const uint64_t r2 = pack2(f.rso, f.rso);
    const uint64_t q0 = mul2(v2, r2);
    const uint64_t q2 = fma2(fma2(q0, pack2(-f.so, -f.so), v2), r2, q0);
    float u0, u1;
    unpack2(add2(q2, pack2(f.zo, f.zo)), u0, u1);
    q0o = (int)rint_sat_u8(fminf(fmaxf(u0, f.qlo), f.qhi));
    q1o = (int)rint_sat_u8(fminf(fmaxf(u1, f.qlo), f.qhi));
}

__global__ void __launch_bounds__(256)
dw_conv_kernel(SimtGeom g, const uint8_t *__restrict__ x, const int16_t *__restrict__ wdw, EpiParams p, DwFast f,
               const uint8_t *__restrict__ res, uint8_t *__restrict__ y, uint8_t *__restrict__ y2) {
    grid_dependency_release(); // a tensor-core convolution that follows sets itself up meanwhile
    const int cq = g.c / 4;
    const size_t total = (size_t)g.n * g.oh * g.ow * cq;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        // 32-bit index arithmetic when the index fits: a 64-bit division costs some seventy instructions
        int c0, ox, oy, b;
        size_t pix;
        if (i <= 0xffffffffull) {
            const uint32_t ii = (uint32_t)i, px = ii / (uint32_t)cq, row = px / (uint32_t)g.ow;
            c0 = (int)(ii % (uint32_t)cq) * 4, ox = (int)(px % (uint32_t)g.ow);
            oy = (int)(row % (uint32_t)g.oh), b = (int)(row / (uint32_t)g.oh);
            pix = px;
        } else {
            c0 = (int)(i % cq) * 4;
            pix = i / cq;
            ox = (int)(pix % g.ow);
            oy = (int)((pix / g.ow) % g.oh);
            b = (int)(pix / ((size_t)g.ow * g.oh));
        }
        const int iy0 = oy * g.sh - g.pt, ix0 = ox * g.sw - g.pl;
        // valid tap ranges: no bounds test inside the loops
        int ky0 = 0, ky1 = g.kh, kx0 = 0, kx1 = g.kw;
        while (ky0 < ky1 && iy0 + ky0 * g.dh < 0)
            ky0++;
        while (ky1 > ky0 && iy0 + (ky1 - 1) * g.dh >= g.h)
            ky1--;
        while (kx0 < kx1 && ix0 + kx0 * g.dw < 0)
            kx0++;
        while (kx1 > kx0 && ix0 + (kx1 - 1) * g.dw >= g.w)
            kx1--;
        int acc[4] = {0, 0, 0, 0};
        for (int ky = ky0; ky < ky1; ky++) {
            const uint8_t *xrow = x + (((size_t)b * g.h + iy0 + ky * g.dh) * g.w + ix0) * g.c + c0;
            const int16_t *wrow = wdw + (size_t)(ky * g.kw) * g.c + c0;
            for (int kx = kx0; kx < kx1; kx++) {
                const uint32_t xv = __ldg(reinterpret_cast<const uint32_t *>(xrow + (size_t)kx * g.dw * g.c));
                const uint2 wv = __ldg(reinterpret_cast<const uint2 *>(wrow + (size_t)kx * g.c));
                acc[0] += ((int)(xv & 255u) - g.x_zp) * (int)(short)(wv.x & 0xffffu);
                acc[1] += ((int)((xv >> 8) & 255u) - g.x_zp) * ((int)wv.x >> 16);
                acc[2] += ((int)((xv >> 16) & 255u) - g.x_zp) * (int)(short)(wv.y & 0xffffu);
                acc[3] += ((int)(xv >> 24) - g.x_zp) * ((int)wv.y >> 16);
            }
        }
        const float4 mult = __ldg(reinterpret_cast<const float4 *>(p.mult + c0));
        const float4 bias = __ldg(reinterpret_cast<const float4 *>(p.bias + c0));
        const size_t o = pix * g.c + c0;
        int q[4];
        if (f.on) {
            dw_requant2(acc[0], acc[1], mult.x, mult.y, bias.x, bias.y, f, q[0], q[1]);
            dw_requant2(acc[2], acc[3], mult.z, mult.w, bias.z, bias.w, f, q[2], q[3]);
        } else {
            const uint32_t rv = p.has_res ? __ldg(reinterpret_cast<const uint32_t *>(res + o)) : 0u;
            q[0] = epi_u8(acc[0], mult.x, bias.x, p, (int)(rv & 255u));
            q[1] = epi_u8(acc[1], mult.y, bias.y, p, (int)((rv >> 8) & 255u));
            q[2] = epi_u8(acc[2], mult.z, bias.z, p, (int)((rv >> 16) & 255u));
            q[3] = epi_u8(acc[3], mult.w, bias.w, p, (int)(rv >> 24));
        }
        *reinterpret_cast<uint32_t *>(y + o) = (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) | ((uint32_t)q[3] << 24);
        if (y2)
            *reinterpret_cast<uint32_t *>(y2 + o) = (uint32_t)p.y2_lut[q[0]] | ((uint32_t)p.y2_lut[q[1]] << 8) |
                                                    ((uint32_t)p.y2_lut[q[2]] << 16) | ((uint32_t)p.y2_lut[q[3]] << 24);
    }
}

// requantises and stores the four outputs x four channels a thread of the 3x3 kernels holds
__device__ __forceinline__ void dw3x3_store(const SimtGeom &g, const EpiParams &p, const DwFast &f, const uint8_t *__restrict__ res,
                                            uint8_t *__restrict__ y, uint8_t *__restrict__ y2, const int (&acc)[4][4], int b, int oy,
                                            int ox0, int c0) {
    const float4 mult = __ldg(reinterpret_cast<const float4 *>(p.mult + c0));
    const float4 bias = __ldg(reinterpret_cast<const float4 *>(p.bias + c0));
    const float m4[4] = {mult.x, mult.y, mult.z, mult.w}, b4[4] = {bias.x, bias.y, bias.z, bias.w};
#pragma unroll
    for (int t = 0; t < 4; t++) {
        if (ox0 + t >= g.ow)
            break;
        const size_t o = ((((size_t)b * g.oh + oy) * g.ow) + ox0 + t) * g.c + c0;
        int q[4];
        if (f.on) {
            dw_requant2(acc[t][0], acc[t][1], m4[0], m4[1], b4[0], b4[1], f, q[0], q[1]);
            dw_requant2(acc[t][2], acc[t][3], m4[2], m4[3], b4[2], b4[3], f, q[2], q[3]);
        } else {
            const uint32_t rv = p.has_res ? __ldg(reinterpret_cast<const uint32_t *>(res + o)) : 0u;
#pragma unroll
            for (int e = 0; e < 4; e++)
                q[e] = epi_u8(acc[t][e], m4[e], b4[e], p, (int)((rv >> (8 * e)) & 255u));
        }
        *reinterpret_cast<uint32_t *>(y + o) = (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) | ((uint32_t)q[3] << 24);
        if (y2)
            *reinterpret_cast<uint32_t *>(y2 + o) = (uint32_t)p.y2_lut[q[0]] | ((uint32_t)p.y2_lut[q[1]] << 8) |
                                                    ((uint32_t)p.y2_lut[q[2]] << 16) | ((uint32_t)p.y2_lut[q[3]] << 24);
    }
}

// The tap sums as byte dot products. sum (x - zx)(w - zw) = sum x w - zw sum x + (9 zx zw - zx sum w) with padded
// taps holding zx: per kernel row the six (stride 1) or nine (stride 2) column words of four channels are
// transposed (eight PRMT per four columns) into words that hold four consecutive columns of ONE channel, and one
// dp4a against the row's three weight bytes -- in bytes 0..2 for the window that starts at the first column of
// the word, in bytes 1..3 for the one that starts at the second -- gives a row's share of one output; a second
// dp4a against ones gives sum x where some weight zero point is not zero. About 25 instructions per output
// channel against 40 of the multiply-add form.
template <bool W_SIGNED>
__device__ __forceinline__ int dot4(uint32_t xbytes, uint32_t wbytes, int acc) {
    int d;
    if (W_SIGNED)
        asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(xbytes), "r"(wbytes), "r"(acc));
    else
        asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(xbytes), "r"(wbytes), "r"(acc));
    return d;
}

template <int S, bool W_SIGNED, bool HAS_ZW>
__global__ void __launch_bounds__(256)
dw3x3_dp_kernel(SimtGeom g, const uint8_t *__restrict__ x, const uint32_t *__restrict__ wdp, const int32_t *__restrict__ cdp,
                const int32_t *__restrict__ w_zp, EpiParams p, DwFast f, const uint8_t *__restrict__ res,
                uint8_t *__restrict__ y, uint8_t *__restrict__ y2) {
    grid_dependency_release(); // a tensor-core convolution that follows sets itself up meanwhile
    constexpr int NC = 3 * S + 3;
    const uint32_t cq = (uint32_t)g.c / 4u, oxg = ((uint32_t)g.ow + 3u) / 4u;
    const uint32_t j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j < oxg * cq) {
        const int c0 = (int)(j % cq) * 4;
        const int ox0 = (int)(j / cq) * 4;
        const int oy = (int)(blockIdx.x % (uint32_t)g.oh), b = (int)(blockIdx.x / (uint32_t)g.oh);
        const int ix0 = ox0 * S - g.pl, iy0 = oy * S - g.pt;
        const uint32_t zxw = (uint32_t)g.x_zp * 0x01010101u; // a padded tap holds the zero point
        int acc[4][4], sx[4][4];
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int e = 0; e < 4; e++)
                acc[t][e] = 0, sx[t][e] = 0;
#pragma unroll
        for (int ky = 0; ky < 3; ky++) {
            const int iy = iy0 + ky;
            const bool row_ok = iy >= 0 && iy < g.h;
            const uint8_t *xrow = x + (((size_t)b * g.h + (row_ok ? iy : 0)) * g.w) * g.c + c0;
            uint32_t col[NC];
#pragma unroll
            for (int cidx = 0; cidx < NC; cidx++) {
                const int ix = ix0 + cidx;
                const bool valid = row_ok && ix >= 0 && ix < g.w;
                col[cidx] = valid ? __ldg(reinterpret_cast<const uint32_t *>(xrow + (size_t)ix * g.c)) : zxw;
            }
            const uint4 wl = __ldg(reinterpret_cast<const uint4 *>(wdp + (size_t)(ky * 2 + 0) * g.c + c0));
            const uint4 wh = __ldg(reinterpret_cast<const uint4 *>(wdp + (size_t)(ky * 2 + 1) * g.c + c0));
            const uint32_t wlo[4] = {wl.x, wl.y, wl.z, wl.w}, whi[4] = {wh.x, wh.y, wh.z, wh.w};
#pragma unroll
            for (int t = 0; t < 4; t++) {
                // the four-column word this output's window lies in, and whether it starts at its second column
                const int start = S == 1 ? (t / 2) * 2 : (t < 3 ? 2 * t : 5);
                const bool shifted = S == 1 ? (t & 1) != 0 : t == 3;
                const uint32_t a = __byte_perm(col[start], col[start + 1], 0x5140), b2 = __byte_perm(col[start + 2], col[start + 3], 0x5140);
                const uint32_t c = __byte_perm(col[start], col[start + 1], 0x7362), d2 = __byte_perm(col[start + 2], col[start + 3], 0x7362);
                const uint32_t tr[4] = {__byte_perm(a, b2, 0x5410), __byte_perm(a, b2, 0x7632), __byte_perm(c, d2, 0x5410),
                                        __byte_perm(c, d2, 0x7632)};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    acc[t][e] = dot4<W_SIGNED>(tr[e], shifted ? whi[e] : wlo[e], acc[t][e]);
                    if (HAS_ZW)
                        sx[t][e] = dot4<false>(tr[e], shifted ? 0x01010100u : 0x00010101u, sx[t][e]);
                }
            }
        }
        const int4 cd = __ldg(reinterpret_cast<const int4 *>(cdp + c0));
        const int cds[4] = {cd.x, cd.y, cd.z, cd.w};
        int zws[4] = {0, 0, 0, 0};
        if (HAS_ZW) {
            const int4 z = __ldg(reinterpret_cast<const int4 *>(w_zp + c0));
            zws[0] = z.x, zws[1] = z.y, zws[2] = z.z, zws[3] = z.w;
        }
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int e = 0; e < 4; e++)
                acc[t][e] += cds[e] - zws[e] * sx[t][e];
        dw3x3_store(g, p, f, res, y, y2, acc, b, oy, ox0, c0);
    }
}

// 3x3, dilation 1, stride S in {1, 2}: one thread computes FOUR horizontally adjacent outputs of four
// channels from a sliding window of 3 S + 3 input columns per kernel row held in registers, so every input
// word is loaded and unpacked once per row (instead of once per tap) and every weight once per four outputs.
template <int S>
__global__ void __launch_bounds__(256)
dw3x3_conv_kernel(SimtGeom g, const uint8_t *__restrict__ x, const int16_t *__restrict__ wdw, EpiParams p, DwFast f,
                  const uint8_t *__restrict__ res, uint8_t *__restrict__ y, uint8_t *__restrict__ y2) {
    grid_dependency_release(); // a tensor-core convolution that follows sets itself up meanwhile
    constexpr int NC = 3 * S + 3;
    // blockIdx.x = output row (image, oy); blockIdx.y * 256 + thread = (group of four outputs, channel quad) in it
    const uint32_t cq = (uint32_t)g.c / 4u, oxg = ((uint32_t)g.ow + 3u) / 4u;
    const uint32_t j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j < oxg * cq) {
        const int c0 = (int)(j % cq) * 4;
        const int ox0 = (int)(j / cq) * 4;
        const int oy = (int)(blockIdx.x % (uint32_t)g.oh), b = (int)(blockIdx.x / (uint32_t)g.oh);
        const int ix0 = ox0 * S - g.pl, iy0 = oy * S - g.pt;
        int acc[4][4];
#pragma unroll
        for (int t = 0; t < 4; t++)
            acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0;
#pragma unroll
        for (int ky = 0; ky < 3; ky++) {
            const int iy = iy0 + ky;
            if (iy < 0 || iy >= g.h)
                continue; // a padded row contributes (zx - zx) * w = 0
            const uint8_t *xrow = x + (((size_t)b * g.h + iy) * g.w) * g.c + c0;
            int xs[NC][4];
#pragma unroll
            for (int cidx = 0; cidx < NC; cidx++) {
                const int ix = ix0 + cidx;
                const bool valid = ix >= 0 && ix < g.w;
                const uint32_t v = valid ? __ldg(reinterpret_cast<const uint32_t *>(xrow + (size_t)ix * g.c)) : 0u;
                xs[cidx][0] = valid ? (int)(v & 255u) - g.x_zp : 0;
                xs[cidx][1] = valid ? (int)((v >> 8) & 255u) - g.x_zp : 0;
                xs[cidx][2] = valid ? (int)((v >> 16) & 255u) - g.x_zp : 0;
                xs[cidx][3] = valid ? (int)(v >> 24) - g.x_zp : 0;
            }
#pragma unroll
            for (int kx = 0; kx < 3; kx++) {
                const uint2 wv = __ldg(reinterpret_cast<const uint2 *>(wdw + (size_t)(ky * 3 + kx) * g.c + c0));
                const int w0 = (int)(short)(wv.x & 0xffffu), w1 = (int)wv.x >> 16;
                const int w2 = (int)(short)(wv.y & 0xffffu), w3 = (int)wv.y >> 16;
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    acc[t][0] += xs[t * S + kx][0] * w0;
                    acc[t][1] += xs[t * S + kx][1] * w1;
                    acc[t][2] += xs[t * S + kx][2] * w2;
                    acc[t][3] += xs[t * S + kx][3] * w3;
                }
            }
        }
        dw3x3_store(g, p, f, res, y, y2, acc, b, oy, ox0, c0);
    }
}

// (w - zw) as int16, [tap][channel], for dw_conv_kernel; null when the shape is not depthwise.
int simt_conv_prepare(nncb_context *ctx, nncb_qconv2d *cv, const void *w_host, const int32_t *wzp_host) {
    const nncb_conv2d_desc &d = cv->d;
    if (!(d.groups == d.c && d.oc == d.c && d.c % 4 == 0 && !d.f32_out))
        return 0;
    const int taps = d.kh * d.kw;
    std::vector<int16_t> t((size_t)taps * d.c);
    for (int c = 0; c < d.c; c++)
        for (int k = 0; k < taps; k++) {
            const int wv = d.w_signed ? (int)reinterpret_cast<const int8_t *>(w_host)[(size_t)c * taps + k]
                                      : (int)reinterpret_cast<const uint8_t *>(w_host)[(size_t)c * taps + k];
            t[(size_t)k * d.c + c] = (int16_t)(wv - (wzp_host ? wzp_host[c] : 0));
        }
    // constants of the division-free requantisation (no residual, no activation table)
    bool ok = true;
    cv->dw_rso = rn_reciprocal(d.out_scale, &ok);
    auto quant = [&](float v) {
        if (std::isinf(v))
            return v < 0 ? 0.f : 255.f;
        const float tq = v / d.out_scale;
        const float u = tq + (float)d.out_zp;
        return std::fmin(std::fmax(rintf(u), 0.f), 255.f);
    };
    cv->dw_qlo = quant(d.clamp_lo), cv->dw_qhi = quant(d.clamp_hi);
    cv->dw_fast = ok && !d.has_residual && cv->d_lut == nullptr && !std::isnan(d.clamp_lo) && !std::isnan(d.clamp_hi);
    if (d.kh == 3 && d.kw == 3) {
        // dp4a form: a kernel row's three raw weight bytes in bytes 0..2 (low) and in bytes 1..3 (shifted) of a word,
        // and the constant part of sum (x - zx)(w - zw) = sum x w - zw sum x - zx sum w + 9 zx zw
        std::vector<uint32_t> wd((size_t)3 * 2 * d.c);
        std::vector<int32_t> cd(d.c);
        for (int c = 0; c < d.c; c++) {
            int wsum = 0;
            for (int ky = 0; ky < 3; ky++) {
                uint32_t lo = 0;
                for (int kx = 0; kx < 3; kx++) {
                    const uint8_t b = reinterpret_cast<const uint8_t *>(w_host)[(size_t)c * 9 + ky * 3 + kx];
                    lo |= (uint32_t)b << (8 * kx);
                    wsum += d.w_signed ? (int)(int8_t)b : (int)b;
                }
                wd[((size_t)ky * 2 + 0) * d.c + c] = lo;
                wd[((size_t)ky * 2 + 1) * d.c + c] = lo << 8;
            }
            const int zw = wzp_host ? wzp_host[c] : 0;
            cv->dw_has_zw |= zw != 0;
            cd[c] = 9 * d.x_zp * zw - d.x_zp * wsum;
        }
        NNCB_CUDA_TRY(cudaMalloc(&cv->d_wdp, wd.size() * 4));
        NNCB_CUDA_TRY(cudaMalloc(&cv->d_cdp, cd.size() * 4));
        NNCB_CUDA_TRY(cudaMemcpyAsync(cv->d_wdp, wd.data(), wd.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
        NNCB_CUDA_TRY(cudaMemcpyAsync(cv->d_cdp, cd.data(), cd.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
        NNCB_CUDA_TRY(cudaStreamSynchronize(ctx->stream)); // the host vectors go out of scope
    }
    NNCB_CUDA_TRY(cudaMalloc(&cv->d_wdw, t.size() * sizeof(int16_t)));
    NNCB_CUDA_TRY(cudaMemcpyAsync(cv->d_wdw, t.data(), t.size() * sizeof(int16_t), cudaMemcpyHostToDevice, ctx->stream));
    NNCB_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return 0;
}

int simt_conv_run(nncb_context *ctx, nncb_qconv2d *cv, const uint8_t *x, const uint8_t *res, void *y, uint8_t *y2) {
    const nncb_conv2d_desc &d = cv->d;
    SimtGeom g{d.n, d.h, d.w, d.c, d.oc, d.kh, d.kw, d.stride_h, d.stride_w, d.pad_t, d.pad_l, d.dil_h,
               d.dil_w, d.groups, cv->oh, cv->ow, d.w_signed, d.x_zp, d.f32_out};
    EpiParams p = make_epi(cv);
    auto al4 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 3) == 0; };
    if (cv->d_wdw && al4(x) && al4(res) && al4(y) && al4(y2)) {
        const size_t quads = (size_t)d.n * cv->oh * cv->ow * (d.c / 4);
        const size_t nb = (quads + 255) / 256, capq = (size_t)ctx->sm_count * 32;
        DwFast f{cv->dw_fast ? 1 : 0, d.out_scale, cv->dw_rso, (float)d.out_zp, cv->dw_qlo, cv->dw_qhi};
        const bool k3 = d.kh == 3 && d.kw == 3 && d.dil_h == 1 && d.dil_w == 1 && d.stride_h == d.stride_w &&
                        (d.stride_h == 1 || d.stride_h == 2);
        if (k3) {
            const int row_items = ((cv->ow + 3) / 4) * (d.c / 4);
            const int bt = row_items >= 256 ? 256 : (row_items + 31) / 32 * 32;
            const dim3 grid3((unsigned)(d.n * cv->oh), (unsigned)((row_items + bt - 1) / bt));
            const bool al16 = (reinterpret_cast<uintptr_t>(cv->d_wdp) & 15) == 0;
            if (cv->d_wdp && cv->d_cdp && al16 && ctx->opt.depthwise_dot) { // (tuning override: 0 takes the multiply-add form)
#define NNCB_DWDP(S_, WS_, ZW_)                                                                                       \
    dw3x3_dp_kernel<S_, WS_, ZW_><<<grid3, bt, 0, ctx->stream>>>(g, x, cv->d_wdp, cv->d_cdp, cv->d_wzp, p, f, res,   \
                                                                 (uint8_t *)y, y2)
                const int v = (d.stride_h == 2 ? 4 : 0) | (d.w_signed ? 2 : 0) | (cv->dw_has_zw ? 1 : 0);
                switch (v) {
                case 0: NNCB_DWDP(1, false, false); break;
                case 1: NNCB_DWDP(1, false, true); break;
                case 2: NNCB_DWDP(1, true, false); break;
                case 3: NNCB_DWDP(1, true, true); break;
                case 4: NNCB_DWDP(2, false, false); break;
                case 5: NNCB_DWDP(2, false, true); break;
                case 6: NNCB_DWDP(2, true, false); break;
                default: NNCB_DWDP(2, true, true); break;
                }
#undef NNCB_DWDP
                return after_launch(ctx, "dw3x3_dp");
            }
            if (d.stride_h == 1)
                dw3x3_conv_kernel<1><<<grid3, bt, 0, ctx->stream>>>(g, x, cv->d_wdw, p, f, res, (uint8_t *)y, y2);
            else
                dw3x3_conv_kernel<2><<<grid3, bt, 0, ctx->stream>>>(g, x, cv->d_wdw, p, f, res, (uint8_t *)y, y2);
            return after_launch(ctx, "dw3x3_conv");
        }
        dw_conv_kernel<<<(int)(nb < capq ? nb : capq), 256, 0, ctx->stream>>>(g, x, cv->d_wdw, p, f, res, (uint8_t *)y, y2);
        return after_launch(ctx, "dw_conv");
    }
    size_t total = (size_t)d.n * cv->oh * cv->ow * d.oc;
    size_t blocks = (total + 255) / 256;
    size_t cap = (size_t)ctx->sm_count * 32;
    int grid = (int)(blocks < cap ? blocks : cap);
    if (d.w_signed)
        simt_conv_kernel<true><<<grid, 256, 0, ctx->stream>>>(g, x, cv->d_w, cv->d_wzp, p, res, y, y2);
    else
        simt_conv_kernel<false><<<grid, 256, 0, ctx->stream>>>(g, x, cv->d_w, cv->d_wzp, p, res, y, y2);
    return after_launch(ctx, "simt_conv");
}

} // namespace nncb
