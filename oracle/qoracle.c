/* CPU oracle for the quantized-inference hot path.
 *
 * TEST INFRASTRUCTURE ONLY. Only tests/, the smoke check and the benchmark's CPU arms load
 * this library; the shipped CUDA library never does. Built by oracle/Makefile (`make port`)
 * with -ffp-contract=off so every float operation below rounds once, exactly as written.
 *
 * PARITY STATUS
 *   - quantize / dequantize restate the reference kernels one to one and are pinned against
 *     the reference's own compiled kernels (oracle/_ref) in tests/.
 *   - The integer conv / matmul / add / pooling functions have NO counterpart in the
 *     reference (its cpu target runs Conv2D and MatMul in float: reference/convolution.cpp:
 *     118-130, reference/matmul.cpp:28-51). They state the integer formulation that the CUDA
 *     kernels implement; against the reference's float composite
 *     dequantize -> conv2d(f32, fused clamp) -> quantize they agree except for rare 1-LSB
 *     differences caused by the reference's f32 accumulation order. Parity of these
 *     functions with the reference is therefore "unpinned" in the strict sense: it is pinned
 *     bit-exactly against this file, and statistically (<= 1 LSB, rate <= 1e-3) against
 *     oracle/_ref.
 *   - paged attention has no reference counterpart at all: parity unpinned.
 *
 * Layouts: activations NHWC (u8), conv weights OHWI (u8 or i8), per-output-channel tables.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Number of worker threads for the convolution loops (1 = the reference's default single
 * thread). Set with qo_set_threads(); results do not depend on it. */
static int g_threads = 1;
void qo_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
int qo_get_threads(void) { return g_threads; }

typedef void (*range_fn)(long begin, long end, void *arg);
typedef struct {
    range_fn fn;
    long begin, end;
    void *arg;
} range_job;
static void *range_tramp(void *p) {
    range_job *j = (range_job *)p;
    j->fn(j->begin, j->end, j->arg);
    return NULL;
}
static void parallel_ranges(long total, range_fn fn, void *arg) {
    int nt = g_threads;
    if (nt > total)
        nt = total > 0 ? (int)total : 1;
    if (nt <= 1) {
        fn(0, total, arg);
        return;
    }
    pthread_t th[256];
    range_job jobs[256];
    long chunk = (total + nt - 1) / nt;
    for (int t = 0; t < nt; t++) {
        jobs[t].fn = fn;
        jobs[t].begin = t * chunk;
        jobs[t].end = (t + 1) * chunk < total ? (t + 1) * chunk : total;
        jobs[t].arg = arg;
        pthread_create(&th[t], NULL, range_tramp, &jobs[t]);
    }
    for (int t = 0; t < nt; t++)
        pthread_join(th[t], NULL);
}

static inline int32_t clampi(int32_t v, int32_t lo, int32_t hi) {
    return v < lo ? lo : (v > hi ? hi : v);
}

/* kernels::detail::clamp = max(min(v, hi), lo)  (include/nncase/kernels/kernel_utils.h:123-130) */
static inline float clampf(float v, float lo, float hi) {
    float t = v < hi ? v : hi; /* std::min(value, max) */
    return t > lo ? t : lo;    /* std::max(.., min)    */
}

/* q = clamp((int32)rint(x / scale + zero_point), type_min, type_max)
 * reference/quantize.cpp:29-45 (lrintf) and optimized/quantize.cpp:59-72 (nearbyintf):
 * both round to nearest even; division, not reciprocal multiplication. */
static inline int32_t quant1(float x, float scale, float zp, int32_t lo, int32_t hi) {
    float v = x / scale + zp;
    int32_t q = (int32_t)lrintf(v);
    return clampi(q, lo, hi);
}

void qo_quantize_u8(const float *in, uint8_t *out, size_t n, float scale, int32_t zp) {
    for (size_t i = 0; i < n; i++)
        out[i] = (uint8_t)quant1(in[i], scale, (float)zp, 0, 255);
}

void qo_quantize_i8(const float *in, int8_t *out, size_t n, float scale, int32_t zp) {
    for (size_t i = 0; i < n; i++)
        out[i] = (int8_t)quant1(in[i], scale, (float)zp, -128, 127);
}

/* y = ((float)q - (float)zero_point) * scale   (reference/dequantize.cpp:29-43) */
void qo_dequantize_u8(const uint8_t *in, float *out, size_t n, float scale, int32_t zp) {
    for (size_t i = 0; i < n; i++)
        out[i] = ((float)in[i] - (float)zp) * scale;
}

void qo_dequantize_i8(const int8_t *in, float *out, size_t n, float scale, int32_t zp) {
    for (size_t i = 0; i < n; i++)
        out[i] = ((float)in[i] - (float)zp) * scale;
}

/* Fused input stage: f32 NCHW -> u8 NHWC (transpose + quantize). Element-wise it is
 * qo_quantize_u8. c_pad >= c: extra channels are filled with the zero point. */
void qo_quantize_nchw_to_nhwc_u8(const float *in, uint8_t *out, int n, int c, int h, int w,
                                 int c_pad, float scale, int32_t zp) {
    for (int b = 0; b < n; b++)
        for (int y = 0; y < h; y++)
            for (int x = 0; x < w; x++)
                for (int ch = 0; ch < c_pad; ch++) {
                    size_t o = (((size_t)b * h + y) * w + x) * c_pad + ch;
                    if (ch < c)
                        out[o] = (uint8_t)quant1(in[(((size_t)b * c + ch) * h + y) * w + x], scale,
                                                 (float)zp, 0, 255);
                    else
                        out[o] = (uint8_t)clampi(zp, 0, 255);
                }
}

/* Fused input stage with space-to-depth(2): out[n][Y][X][(dy*2+dx)*c + ch] =
 * quantize(in[n][ch][2Y+dy][2X+dx]); channels 4c..c_pad-1 hold the zero point. Element-wise it is
 * qo_quantize_u8; only the arrangement differs. */
void qo_quantize_nchw_to_s2d_u8(const float *in, uint8_t *out, int n, int c, int h, int w, int c_pad,
                                float scale, int32_t zp) {
    const int hc = h / 2, wc = w / 2;
    for (int b = 0; b < n; b++)
        for (int Y = 0; Y < hc; Y++)
            for (int X = 0; X < wc; X++) {
                uint8_t *o = out + (((size_t)b * hc + Y) * wc + X) * c_pad;
                for (int k = 0; k < c_pad; k++)
                    o[k] = (uint8_t)clampi(zp, 0, 255);
                for (int dy = 0; dy < 2; dy++)
                    for (int dx = 0; dx < 2; dx++)
                        for (int ch = 0; ch < c; ch++)
                            o[(dy * 2 + dx) * c + ch] = (uint8_t)quant1(
                                in[(((size_t)b * c + ch) * h + 2 * Y + dy) * w + 2 * X + dx], scale, (float)zp, 0, 255);
            }
}

/* Output size of a windowed op: kernels::detail::get_windowed_output_size
 * (include/nncase/kernels/kernel_utils.h). */
static inline int out_size(int in, int k, int stride, int dil, int pad_before, int pad_after) {
    int eff = (k - 1) * dil + 1;
    return (in + pad_before + pad_after - eff) / stride + 1;
}

typedef struct {
    int32_t n, h, w, c;       /* input NHWC                                   */
    int32_t oc, kh, kw;       /* weights [oc][kh][kw][c/groups]               */
    int32_t stride_h, stride_w;
    int32_t pad_t, pad_b, pad_l, pad_r;
    int32_t dil_h, dil_w;
    int32_t groups;
    int32_t w_signed;         /* 0: weights are u8, 1: weights are i8         */
    int32_t x_zp;             /* activation zero point                        */
    float out_scale;          /* output quant param                           */
    int32_t out_zp;
    float clamp_lo, clamp_hi; /* fused_clamp on the real-valued result        */
} qo_conv_desc;

/* Integer Conv2D with requantisation. For every output element
 *   acc = sum over in-image taps of (xq - zx) * (wq - zw[oc])           (int32, exact)
 *   y   = clamp((float)acc * mult[oc] + bias[oc], lo, hi)                (mult = sx * sw[oc], f32)
 *   yq  = clamp(rint(y / so + zo), 0, 255)
 * Out-of-image taps are skipped, as the reference's loop-bound clipping does
 * (reference/convolution.cpp:59-74); bias is added in float (":75"); clamp is the fused
 * activation (":99-101"); the last line is the reference quantize. w_zp may be NULL (all 0).
 * lut, if non-NULL, maps the u8 result through a 256-entry table (u8 activation such as
 * SiLU evaluated on the quantized value). acc_out, if non-NULL, receives the raw int32 acc. */
typedef struct {
    const qo_conv_desc *d;
    const uint8_t *x;
    const void *wv;
    const int32_t *w_zp;
    const float *mult, *bias;
    const uint8_t *lut;
    uint8_t *y;
    int32_t *acc_out;
    int oh, ow;
} conv_args;

static void conv_range(long p0, long p1, void *argp) {
    const conv_args *a = (const conv_args *)argp;
    const qo_conv_desc *d = a->d;
    const int oh = a->oh, ow = a->ow;
    const int gic = d->c / d->groups, goc = d->oc / d->groups;
    const uint8_t *wu = (const uint8_t *)a->wv;
    const int8_t *ws = (const int8_t *)a->wv;
    for (long p = p0; p < p1; p++) {
        int b = (int)(p / ((long)oh * ow));
        int r = (int)(p % ((long)oh * ow));
        int oy = r / ow, ox = r % ow;
        int iy0 = oy * d->stride_h - d->pad_t, ix0 = ox * d->stride_w - d->pad_l;
        for (int oc = 0; oc < d->oc; oc++) {
            int g = oc / goc;
            int32_t zw = a->w_zp ? a->w_zp[oc] : 0;
            int32_t acc = 0;
            for (int ky = 0; ky < d->kh; ky++) {
                int iy = iy0 + ky * d->dil_h;
                if (iy < 0 || iy >= d->h)
                    continue;
                for (int kx = 0; kx < d->kw; kx++) {
                    int ix = ix0 + kx * d->dil_w;
                    if (ix < 0 || ix >= d->w)
                        continue;
                    const uint8_t *xp =
                        a->x + (((size_t)b * d->h + iy) * d->w + ix) * d->c + g * gic;
                    size_t wo = (((size_t)oc * d->kh + ky) * d->kw + kx) * gic;
                    int32_t s = 0;
                    if (d->w_signed) {
                        const int8_t *wp = ws + wo;
                        for (int ic = 0; ic < gic; ic++)
                            s += ((int32_t)xp[ic] - d->x_zp) * ((int32_t)wp[ic] - zw);
                    } else {
                        const uint8_t *wp = wu + wo;
                        for (int ic = 0; ic < gic; ic++)
                            s += ((int32_t)xp[ic] - d->x_zp) * ((int32_t)wp[ic] - zw);
                    }
                    acc += s;
                }
            }
            size_t o = (size_t)p * d->oc + oc;
            if (a->acc_out)
                a->acc_out[o] = acc;
            float v = (float)acc * a->mult[oc];
            v = v + a->bias[oc];
            v = clampf(v, d->clamp_lo, d->clamp_hi);
            uint8_t q = (uint8_t)quant1(v, d->out_scale, (float)d->out_zp, 0, 255);
            a->y[o] = a->lut ? a->lut[q] : q;
        }
    }
}

void qo_qconv2d_u8(const qo_conv_desc *d, const uint8_t *x, const void *wv, const int32_t *w_zp,
                   const float *mult, const float *bias, const uint8_t *lut, uint8_t *y,
                   int32_t *acc_out) {
    conv_args a = {d, x, wv, w_zp, mult, bias, lut, y, acc_out, 0, 0};
    a.oh = out_size(d->h, d->kh, d->stride_h, d->dil_h, d->pad_t, d->pad_b);
    a.ow = out_size(d->w, d->kw, d->stride_w, d->dil_w, d->pad_l, d->pad_r);
    parallel_ranges((long)d->n * a.oh * a.ow, conv_range, &a);
}

/* Same accumulation and float epilogue, but the real-valued result is stored as f32 instead
 * of being requantised (used for the classifier logits: MatMul -> Dequantize-free output). */
void qo_qconv2d_f32out(const qo_conv_desc *d, const uint8_t *x, const void *wv,
                       const int32_t *w_zp, const float *mult, const float *bias, float *y) {
    const int oh = out_size(d->h, d->kh, d->stride_h, d->dil_h, d->pad_t, d->pad_b);
    const int ow = out_size(d->w, d->kw, d->stride_w, d->dil_w, d->pad_l, d->pad_r);
    const long total = (long)d->n * oh * ow * d->oc;
    int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)total);
    uint8_t *tmp = (uint8_t *)malloc((size_t)total);
    qo_qconv2d_u8(d, x, wv, w_zp, mult, bias, NULL, tmp, acc);
    for (long i = 0; i < total; i++) {
        int oc = (int)(i % d->oc);
        float v = (float)acc[i] * mult[oc];
        v = v + bias[oc];
        y[i] = clampf(v, d->clamp_lo, d->clamp_hi);
    }
    free(acc);
    free(tmp);
}

/* Residual add on quantized tensors: the reference executes binary(add) on dequantized f32
 * values (reference/binary.cpp:28-123) between a dequantize and a quantize, so
 *   yq = quantize(dequantize(a) + dequantize(b)). */
void qo_qadd_u8(const uint8_t *a, const uint8_t *b, uint8_t *y, size_t n, float sa, int32_t za,
                float sb, int32_t zb, float so, int32_t zo) {
    for (size_t i = 0; i < n; i++) {
        float fa = ((float)a[i] - (float)za) * sa;
        float fb = ((float)b[i] - (float)zb) * sb;
        float s = fa + fb;
        y[i] = (uint8_t)quant1(s, so, (float)zo, 0, 255);
    }
}

/* Requantise a u8 tensor to new parameters, optionally through clamp [lo, hi] on the real
 * value (ReLU = [0, +inf)): yq = quantize(clamp(dequantize(x))). */
void qo_requant_u8(const uint8_t *x, uint8_t *y, size_t n, float si, int32_t zi, float so,
                   int32_t zo, float lo, float hi) {
    for (size_t i = 0; i < n; i++) {
        float f = ((float)x[i] - (float)zi) * si;
        f = clampf(f, lo, hi);
        y[i] = (uint8_t)quant1(f, so, (float)zo, 0, 255);
    }
}

/* Unary activations between quant params as a 256-entry table:
 *   table[q] = quantize((float)f((double)dequantize(q)))
 * f evaluated in double and cast to float like the reference's UNARY_TEMPLATE
 * (reference/kernel_template.h:19-50) with the formulas of reference/activation.cpp:32-38.
 * kind: 0 relu, 1 sigmoid, 2 swish, 3 hard_swish. */
int qo_activation_table(int kind, float si, int32_t zi, float so, int32_t zo, uint8_t *table) {
    for (int q = 0; q < 256; q++) {
        float xf = ((float)q - (float)zi) * si;
        double x = (double)xf, y;
        switch (kind) {
        case 0:
            y = x > 0 ? x : 0;
            break;
        case 1:
            y = 1 / (1 + exp(-x));
            break;
        case 2:
            y = x / (1 + exp(-x));
            break;
        case 3: {
            double t = (double)(1.f / 6 * x + 0.5);
            t = t < 1.0 ? t : 1.0;
            t = t > 0.0 ? t : 0.0;
            y = x * t;
            break;
        }
        default:
            return -1;
        }
        table[q] = (uint8_t)quant1((float)y, so, (float)zo, 0, 255);
    }
    return 0;
}

void qo_lut_u8(const uint8_t *x, uint8_t *y, size_t n, const uint8_t *table) {
    for (size_t i = 0; i < n; i++)
        y[i] = table[x[i]];
}

/* Channel-block copy through an optional table: concat (per-input requantisation) and split. */
void qo_copy_channels_u8(const uint8_t *src, int src_c, int src_off, uint8_t *dst, int dst_c, int dst_off, int len,
                         size_t pixels, const uint8_t *table) {
    for (size_t p = 0; p < pixels; p++)
        for (int j = 0; j < len; j++) {
            uint8_t q = src[p * src_c + src_off + j];
            dst[p * dst_c + dst_off + j] = table ? table[q] : q;
        }
}

/* Nearest-neighbour resize by integer factors, asymmetric coordinates, floor (NHWC). */
void qo_resize_nearest_u8(const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int fy, int fx) {
    const int oh = h * fy, ow = w * fx;
    for (int b = 0; b < n; b++)
        for (int oy = 0; oy < oh; oy++)
            for (int ox = 0; ox < ow; ox++)
                memcpy(y + (((size_t)b * oh + oy) * ow + ox) * c, x + (((size_t)b * h + oy / fy) * w + ox / fx) * c, c);
}

/* softmax over the last axis, f32 (reference/softmax.cpp:30-80): max, (x - max) * beta, expf,
 * sequential sum, multiply by 1/sum. */
void qo_softmax_f32(const float *in, float *out, size_t rows, int cols, float beta) {
    for (size_t r = 0; r < rows; r++) {
        const float *x = in + r * cols;
        float *y = out + r * cols;
        float mx = x[0];
        for (int j = 0; j < cols; j++)
            mx = x[j] > mx ? x[j] : mx;
        float sum = 0;
        for (int j = 0; j < cols; j++) {
            y[j] = expf((x[j] - mx) * beta);
            sum += y[j];
        }
        float inv = 1.0f / sum;
        for (int j = 0; j < cols; j++)
            y[j] *= inv;
    }
}

/* Max pooling on u8 NHWC with input and output sharing one quant param (max commutes with
 * the monotone dequantize/quantize pair). A window that overlaps the padding also takes the
 * real value 0, i.e. the zero point, into the max: reduce_window2d applies
 * binary_op(value, 0) once per padded tap (reference/reduce_window.cpp:86-90). */
void qo_maxpool_u8(const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int kh, int kw,
                   int sh, int sw, int pt, int pb, int pl, int pr, int32_t zp) {
    const int oh = out_size(h, kh, sh, 1, pt, pb), ow = out_size(w, kw, sw, 1, pl, pr);
    for (int b = 0; b < n; b++)
        for (int oy = 0; oy < oh; oy++)
            for (int ox = 0; ox < ow; ox++)
                for (int ch = 0; ch < c; ch++) {
                    int m = -1, cnt = 0;
                    for (int ky = 0; ky < kh; ky++) {
                        int iy = oy * sh - pt + ky;
                        if (iy < 0 || iy >= h)
                            continue;
                        for (int kx = 0; kx < kw; kx++) {
                            int ix = ox * sw - pl + kx;
                            if (ix < 0 || ix >= w)
                                continue;
                            int v = x[(((size_t)b * h + iy) * w + ix) * c + ch];
                            m = v > m ? v : m;
                            cnt++;
                        }
                    }
                    if (cnt < kh * kw) {
                        int z = clampi(zp, 0, 255);
                        m = z > m ? z : m;
                    }
                    y[(((size_t)b * oh + oy) * ow + ox) * c + ch] = (uint8_t)m;
                }
}


/* reduce_window2d (kernels::stackvm::reduce_window2d, reference/reduce_window.cpp:35-182) between quantized
 * tensors, u8 NHWC. op follows reduce_op_t: 0 mean, 1 min, 2 max, 3 sum. A tap outside the image contributes
 * the real value 0 (:86-90), i.e. the input zero point. max / min are monotone, so they run on the bytes and the
 * result is requantised from (si, zi) to (so, zo); sum and mean accumulate exactly in integers:
 *   v = (float)(sum_valid q - cnt_valid * zi) * si;   mean: v / (float)(count_include_pad ? kh*kw : cnt_valid)
 *   y = quantize(v, so, zo)
 * (the reference sums the dequantized floats tap by tap; the two agree up to its float summation order). */
void qo_reduce_window2d_u8(int op, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int kh, int kw,
                           int sh, int sw, int pt, int pb, int pl, int pr, int count_include_pad, float si,
                           int32_t zi, float so, int32_t zo) {
    const int oh = out_size(h, kh, sh, 1, pt, pb), ow = out_size(w, kw, sw, 1, pl, pr);
    for (int b = 0; b < n; b++)
        for (int oy = 0; oy < oh; oy++)
            for (int ox = 0; ox < ow; ox++)
                for (int ch = 0; ch < c; ch++) {
                    int mx = -1, mn = 256, cnt = 0;
                    int32_t sum = 0;
                    for (int ky = 0; ky < kh; ky++) {
                        int iy = oy * sh - pt + ky;
                        if (iy < 0 || iy >= h)
                            continue;
                        for (int kx = 0; kx < kw; kx++) {
                            int ix = ox * sw - pl + kx;
                            if (ix < 0 || ix >= w)
                                continue;
                            int v = x[(((size_t)b * h + iy) * w + ix) * c + ch];
                            mx = v > mx ? v : mx;
                            mn = v < mn ? v : mn;
                            sum += v;
                            cnt++;
                        }
                    }
                    float r;
                    if (op == 1 || op == 2) {
                        int q = op == 2 ? mx : mn;
                        if (cnt < kh * kw) {
                            int z = clampi(zi, 0, 255);
                            q = op == 2 ? (z > q ? z : q) : (z < q ? z : q);
                        }
                        r = ((float)q - (float)zi) * si;
                    } else {
                        r = (float)(sum - cnt * zi) * si;
                        if (op == 0)
                            r = r / (float)(count_include_pad ? kh * kw : cnt);
                    }
                    y[(((size_t)b * oh + oy) * ow + ox) * c + ch] = (uint8_t)quant1(r, so, (float)zo, 0, 255);
                }
}

/* Element-wise binary operators between quantized tensors (kernels::stackvm::binary, reference/binary.cpp:28-123):
 *   y = quantize(op(dequantize(a), dequantize(b)));  op follows binary_op_t: 0 add, 1 sub, 2 mul, 5 min, 6 max. */
int qo_qbinary_u8(int op, const uint8_t *a, const uint8_t *b, uint8_t *y, size_t n, float sa, int32_t za,
                  float sb, int32_t zb, float so, int32_t zo) {
    if (op != 0 && op != 1 && op != 2 && op != 5 && op != 6)
        return -1;
    for (size_t i = 0; i < n; i++) {
        float fa = ((float)a[i] - (float)za) * sa;
        float fb = ((float)b[i] - (float)zb) * sb;
        float r = op == 0 ? fa + fb : op == 1 ? fa - fb : op == 2 ? fa * fb : op == 5 ? (fa < fb ? fa : fb) : (fa > fb ? fa : fb);
        y[i] = (uint8_t)quant1(r, so, (float)zo, 0, 255);
    }
    return 0;
}

/* Global mean over H x W (reduce_window2d mean with the window covering the image,
 * reference/reduce_window.cpp:133-135) on u8 NHWC:
 *   mean = ((float)(sum q - cnt * zi) * si) / (float)cnt ;  yq = quantize(mean).
 * The integer sum makes the result independent of summation order. */
void qo_global_avgpool_u8(const uint8_t *x, uint8_t *y, int n, int h, int w, int c, float si,
                          int32_t zi, float so, int32_t zo) {
    const int cnt = h * w;
    for (int b = 0; b < n; b++)
        for (int ch = 0; ch < c; ch++) {
            int32_t s = 0;
            for (int p = 0; p < cnt; p++)
                s += x[((size_t)b * cnt + p) * c + ch];
            s -= cnt * zi;
            float m = ((float)s * si) / (float)cnt;
            y[(size_t)b * c + ch] = (uint8_t)quant1(m, so, (float)zo, 0, 255);
        }
}

/* u8 NHWC -> f32 NCHW with dequantize (output stage). */
void qo_dequantize_nhwc_to_nchw_f32(const uint8_t *in, float *out, int n, int h, int w, int c,
                                    float scale, int32_t zp) {
    for (int b = 0; b < n; b++)
        for (int ch = 0; ch < c; ch++)
            for (int y = 0; y < h; y++)
                for (int x = 0; x < w; x++)
                    out[(((size_t)b * c + ch) * h + y) * w + x] =
                        ((float)in[(((size_t)b * h + y) * w + x) * c + ch] - (float)zp) * scale;
}

#ifdef __cplusplus
}
#endif
