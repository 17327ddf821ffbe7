// Quantized Conv2D / MatMul: the plan object shared by the CUDA-core and the tcgen05 kernels,
// and the requantising epilogue both use, so the two paths cannot differ in arithmetic.
#pragma once
#include "internal.cuh"
#include <cuda.h>

namespace nncb {

// Per-launch epilogue constants. Tables are device pointers indexed by output channel.
struct EpiParams {
    const float *mult;     // sx * sw[oc]
    const float *bias;     // f32 bias
    const uint8_t *lut;    // optional 256-entry activation table applied to the u8 result
    const uint8_t *y2_lut; // optional table producing the second output from the final u8
    float out_scale, out_zp;
    float clamp_lo, clamp_hi;
    int has_res;
    float res_scale, res_zp, add_scale, add_zp;
};

// Real value of the convolution before requantisation:
//   v = clamp((float)acc * mult + bias, lo, hi)        two roundings, no fma
__device__ __forceinline__ float epi_real(int acc, float mult, float bias, float lo, float hi) {
    float v = __fadd_rn(__fmul_rn((float)acc, mult), bias);
    return clamp_dev(v, lo, hi);
}

// Exact requantising epilogue for one element; `res` is the residual byte (ignored unless
// p.has_res). Returns the final u8.
__device__ __forceinline__ int epi_u8(int acc, float mult, float bias, const EpiParams &p, int res) {
    float v = epi_real(acc, mult, bias, p.clamp_lo, p.clamp_hi);
    int q = quant_dev(v, p.out_scale, p.out_zp, 0, 255);
    if (p.lut)
        q = p.lut[q];
    if (p.has_res) {
        float a = dequant_dev((float)q, p.out_zp, p.out_scale);
        float b = dequant_dev((float)res, p.res_zp, p.res_scale);
        q = quant_dev(__fadd_rn(a, b), p.add_scale, p.add_zp, 0, 255);
    }
    return q;
}

enum { PATH_SIMT = 1, PATH_TC = 2 };

struct TcPlan; // tcgen05 kernel's packed weights, tensor maps and tables (qconv_tc.cu)

} // namespace nncb

struct nncb_qconv2d {
    nncb_conv2d_desc d;
    int device = 0;
    int oh = 0, ow = 0;
    int path = 0;
    // device copies of the caller's tables
    void *d_w = nullptr;       // OHWI weights as given
    int16_t *d_wdw = nullptr;  // depthwise only: (w - zw) as int16, [tap][channel]
    uint32_t *d_wdp = nullptr; // depthwise 3x3 only: raw weight bytes of a kernel row as dp4a operands, [ky][low / shifted][channel]
    int32_t *d_cdp = nullptr;  // depthwise 3x3 only: per channel 9 zx zw - zx sum(w)
    bool dw_has_zw = false;    // some weight zero point is not 0
    // depthwise only: constants of the division-free exact requantisation (valid when dw_fast)
    bool dw_fast = false;
    float dw_rso = 0.f, dw_qlo = 0.f, dw_qhi = 255.f;
    int32_t *d_wzp = nullptr;  // per-oc weight zero points (always materialised)
    float *d_mult = nullptr;
    float *d_bias = nullptr;
    uint8_t *d_lut = nullptr;
    uint8_t *d_y2lut = nullptr;
    nncb::TcPlan *tc = nullptr;
};

namespace nncb {
EpiParams make_epi(const nncb_qconv2d *cv);
int simt_conv_run(nncb_context *ctx, nncb_qconv2d *cv, const uint8_t *x, const uint8_t *res, void *y, uint8_t *y2);
int simt_conv_prepare(nncb_context *ctx, nncb_qconv2d *cv, const void *w_host, const int32_t *wzp_host);
// RN(1/b) verified in extended precision; *ok = false for scales outside the range the three-operation
// division is proven for (qconv_tc.cu).
float rn_reciprocal(float b, bool *ok);
// tcgen05 path; tc_conv_supported says whether this shape can use it.
bool tc_conv_supported(const nncb_conv2d_desc &d, std::string *why);
int tc_conv_create(nncb_context *ctx, nncb_qconv2d *cv, const void *w_host, const int32_t *wzp_host);
void tc_conv_destroy(nncb_qconv2d *cv);
int tc_conv_run(nncb_context *ctx, nncb_qconv2d *cv, const uint8_t *x, const uint8_t *res, void *y, uint8_t *y2);
int reciprocal_division_selftest(nncb_context *ctx, float scale, unsigned long long count, unsigned long long seed,
                                 unsigned long long *mismatches);
// y = quantize(clamp(dequantize(x)))) for all 256 inputs, host arithmetic identical to the device's.
int make_activation_table(int kind, float si, int32_t zi, float so, int32_t zo, uint8_t table[256]);
void make_requant_table(float si, int32_t zi, float so, int32_t zo, float lo, float hi, uint8_t table[256]);
} // namespace nncb
