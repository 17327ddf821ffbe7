/* nncase_b200 -- C ABI of the B200 (sm_100a) kernels behind nncase's `cuda` module.
 *
 * This is the thin extern "C" boundary that a runtime_module / custom-call plugin of the
 * nncase native runtime (and its C# P/Invoke or Python ctypes callers) binds to. Plain
 * pointers and sizes only. Every function returns 0 on success or a negative errno-style
 * code, the convention of the reference's own C API (src/Native/src/api.cpp:25-49,
 * managed side: src/Nncase.Simulator/Runtime/Interop/ErrorCode.cs:23-31):
 *   -EINVAL  bad argument            -ENOMEM    device allocation failed
 *   -ENOSYS  unsupported combination -EIO       a CUDA call or kernel failed
 *   -ETIMEDOUT a kernel-internal wait ran out (the kernel returned, the context is usable)
 * nncb_last_error() gives the text of the calling thread's last failure.
 *
 * Unless a function says "host", pointers are DEVICE pointers valid on the context's device.
 * Calls enqueue work on the context's stream and return without synchronising; the *_host
 * variants copy in, run, copy out and synchronise (the contract of the reference's
 * synchronous kernels, src/Native/src/kernels/stackvm/tensor_ops.cpp).
 *
 * Quantized tensors: activations are u8, NHWC. Convolution weights are u8 or i8, OHWI
 * ([oc][kh][kw][ic/groups]). Arithmetic of every quantized op is specified with the op and
 * is bit-exact with the CPU oracle shipped in oracle/qoracle.c.
 */
#ifndef NNCASE_B200_H
#define NNCASE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define NNCB_API __declspec(dllexport)
#else
#define NNCB_API __attribute__((visibility("default")))
#endif

typedef struct nncb_context nncb_context;
typedef struct nncb_qconv2d nncb_qconv2d;

/* element types, numbered like nncase's typecode_t for the types used here
 * (src/Native/include/nncase/runtime/typecodes.def) */
typedef enum nncb_dtype { NNCB_I8 = 2, NNCB_I16 = 3, NNCB_U8 = 6, NNCB_F16 = 10, NNCB_F32 = 11 } nncb_dtype;

/* ---- context: device + stream (replaces kernels::kernel_context,
 *      src/Native/include/nncase/kernels/kernel_context.h) ------------------------------ */
/* stream: the cudaStream_t to launch on; NULL is the CUDA default stream. The caller owns it.
 * Every call that takes a context makes the context's device the calling thread's current CUDA
 * device (cudaSetDevice) and leaves it so: a caller that works with several devices sets its own
 * device again afterwards. */
NNCB_API int nncb_context_create(int device, void *stream, nncb_context **out);
NNCB_API int nncb_context_destroy(nncb_context *ctx);
NNCB_API int nncb_context_set_stream(nncb_context *ctx, void *stream);
NNCB_API void *nncb_context_stream(nncb_context *ctx);
NNCB_API int nncb_synchronize(nncb_context *ctx);
/* Per-context options, by name (the role of the reference interpreter's options_dict,
 * src/Native/src/runtime/interpreter.cpp:29-31). Read when a plan is created or a kernel is launched.
 *   "launch.overlap"         1: tensor-core convolutions are launched as programmatic dependents of the kernel before them in
 *                            the stream (their set-up overlaps its last tiles); 0: plain launches
 *   "matmul.tensor_core"     1: nncb_gemv_w8a16 / _swiglu run on the tcgen05 form for more than 32 tokens on matrices of 128 K
 *                            weights or more (K a multiple of 64); 2: for every shape that fits; 0: mma.sync form always
 *   "wait_limit_us"          kernel-internal waits give up after this long (default 1,000,000)
 *   "peer_wait_limit_us"     waits for another rank's flag (nncb_peer_allreduce_add_rmsnorm_f16) give up after this long (default 30,000,000)
 *   "conv.tile_n"            force the N tile of the tensor-core convolution: 128, 96, 64, 48, 32 (0 = choose)
 *   "conv.mma_issuers"       force the number of warps that issue the convolution's MMAs: 1 or 2 (0 = choose)
 *   "conv.load_warps"        force its load warps: 1, 2 = one for activations and one for weights, 3 = two that take the stages in turn (0 = choose)
 *   "conv.wide_patch"        0: keep 64-/128-channel stride-1 convolutions on the im2col form (default 1)
 *   "conv.add_table"         the fused residual add of the tensor-core convolution: 2 = the unfused float chain on packed arithmetic
 *                            instead of the look-up in a table of all byte pairs (default 0; same bits, measured slower)
 *   "depthwise.dot_product"  0: multiply-add form of the 3x3 depthwise kernel (default 1)
 *   "attention.warps"        force the CTA width of paged attention: 4 or 8 (0 = choose)
 *   "attention.splits"       force its number of context splits (0 = choose)
 *   "debug.withhold_load"    1: the tensor-core convolution's loader leaves out one operand load, so that
 *                            the consumer's wait runs out; exercises the give-up path (see
 *                            nncb_check_device_status). Results of such a run are undefined.
 * Unknown names and negative values: -EINVAL. */
NNCB_API int nncb_context_set_option(nncb_context *ctx, const char *name, int64_t value);
NNCB_API int nncb_context_get_option(nncb_context *ctx, const char *name, int64_t *value);
/* Number of kernels this context has launched so far. */
NNCB_API uint64_t nncb_launch_count(nncb_context *ctx);
/* Reads and clears the device-side status word (0 = none); synchronises the stream.
 *   -ETIMEDOUT  a kernel-internal wait ran out (role codes 101-105 of the tensor-core convolution);
 *               the kernel returned early, its outputs are undefined, the context stays usable
 *   -ERANGE     a kernel met an index from device memory that it refused to follow: a position,
 *               context length or page id outside the bounds the call was given (codes 201, 202);
 *               nothing was read or written through it */
NNCB_API int nncb_check_device_status(nncb_context *ctx);
NNCB_API const char *nncb_last_error(void);
NNCB_API const char *nncb_version(void);

/* ---- device memory (stands in for host_buffer, the only memory the reference has:
 *      src/Native/include/nncase/runtime/host_buffer.h:46-84) ---------------------------- */
NNCB_API int nncb_malloc(nncb_context *ctx, size_t bytes, void **dptr);
NNCB_API int nncb_free(nncb_context *ctx, void *dptr);
NNCB_API int nncb_memcpy_h2d(nncb_context *ctx, void *dst, const void *host_src, size_t bytes);
NNCB_API int nncb_memcpy_d2h(nncb_context *ctx, void *host_dst, const void *src, size_t bytes);
NNCB_API int nncb_memset(nncb_context *ctx, void *dst, int value, size_t bytes);

/* ---- QuantParam math (host; replaces QuantUtility.GetQuantParam / FixupRange,
 *      src/Nncase.Core/Utilities/QuantUtility.cs:41-97) ---------------------------------- */
typedef enum nncb_quant_mode { NNCB_UNSIGNED = 0, NNCB_SIGNED_SYMMETRIC = 1, NNCB_SIGNED_ASYMMETRIC = 2 } nncb_quant_mode;
NNCB_API int nncb_fixup_range(float *rmin, float *rmax, int symmetric);
NNCB_API int nncb_get_quant_param(float rmin, float rmax, int bits, int mode, int32_t *zero_point, float *scale);

/* ---- Quantize / Dequantize (replace kernels::stackvm::quantize / dequantize,
 *      src/Native/src/kernels/stackvm/tensor_ops.cpp:681-695 and :268-283; arithmetic of
 *      optimized/quantize.cpp:59-72 and optimized/dequantize.cpp:49-60) -------------------
 *   q = clamp(rint(x / scale + zero_point), type_min, type_max)   (ties to even, true division)
 *   y = ((float)q - (float)zero_point) * scale
 * qtype: NNCB_U8, NNCB_I8 or NNCB_I16. Any n (n == 0 is a no-op). */
NNCB_API int nncb_quantize(nncb_context *ctx, const float *in, void *out, size_t n, float scale, int32_t zero_point, int qtype);
NNCB_API int nncb_dequantize(nncb_context *ctx, const void *in, float *out, size_t n, float scale, int32_t zero_point, int qtype);
/* host-buffer forms: in/out are HOST pointers (synchronous). */
NNCB_API int nncb_quantize_host(nncb_context *ctx, const float *in, void *out, size_t n, float scale, int32_t zero_point, int qtype);
NNCB_API int nncb_dequantize_host(nncb_context *ctx, const void *in, float *out, size_t n, float scale, int32_t zero_point, int qtype);

/* Module input/output stages: the reference's tensors are NCHW f32 at the module boundary;
 * the kernels keep u8 NHWC inside. c_pad >= c pads the channel dimension with the zero point. */
NNCB_API int nncb_quantize_nchw_to_nhwc_u8(nncb_context *ctx, const float *in, uint8_t *out, int n, int c, int h, int w, int c_pad, float scale, int32_t zero_point);
/* Quantize + space-to-depth(2): out[n][Y][X][(dy*2+dx)*c + ch] = quantize(in[n][ch][2Y+dy][2X+dx]),
 * channels 4c..c_pad-1 = zero point (c_pad 16 or 32; h, w even). A stride-2 convolution over few
 * input channels becomes a stride-1 convolution over c_pad channels with rearranged weights. */
NNCB_API int nncb_quantize_nchw_to_s2d_u8(nncb_context *ctx, const float *in, uint8_t *out, int n, int c, int h, int w, int c_pad, float scale, int32_t zero_point);
/* the same from an NHWC f32 input [n][h][w][c] */
NNCB_API int nncb_quantize_nhwc_to_s2d_u8(nncb_context *ctx, const float *in, uint8_t *out, int n, int h, int w, int c, int c_pad, float scale, int32_t zero_point);
/* the same with the convolution's padding materialised: out is [n][h/2+pad_t+pad_b][w/2+pad_l+pad_r][c_pad]
 * and the border cells hold the zero point, so that the consumer is an unpadded convolution
 * (Conv2D's zero padding, src/Native/src/kernels/stackvm/reference/convolution.cpp:56-66, as data).
 * in_nhwc != 0: the f32 input is [n][h][w][c], else [n][c][h][w]. */
NNCB_API int nncb_quantize_to_s2d_padded_u8(nncb_context *ctx, const float *in, int in_nhwc, uint8_t *out, int n, int c, int h, int w, int c_pad, int pad_t, int pad_b, int pad_l, int pad_r, float scale, int32_t zero_point);
NNCB_API int nncb_dequantize_nhwc_to_nchw_f32(nncb_context *ctx, const uint8_t *in, float *out, int n, int h, int w, int c, float scale, int32_t zero_point);
/* u8 layout changes without arithmetic */
NNCB_API int nncb_nchw_to_nhwc_u8(nncb_context *ctx, const uint8_t *in, uint8_t *out, int n, int c, int h, int w);
NNCB_API int nncb_nhwc_to_nchw_u8(nncb_context *ctx, const uint8_t *in, uint8_t *out, int n, int h, int w, int c);

/* ---- element-wise and pooling ops on u8 NHWC ------------------------------------------ */
/* binary add (kernels::stackvm::binary, tensor_ops.cpp:70-89) between quantized tensors:
 *   y = quantize(dequantize(a) + dequantize(b)) */
NNCB_API int nncb_qadd_u8(nncb_context *ctx, const uint8_t *a, const uint8_t *b, uint8_t *y, size_t n, float sa, int32_t za, float sb, int32_t zb, float so, int32_t zo);
/* the other binary operators of kernels::stackvm::binary (reference/binary.cpp:28-123), numbered like the reference's
 * binary_op_t: 0 add, 1 sub, 2 mul, 5 min, 6 max:   y = quantize(op(dequantize(a), dequantize(b))) */
NNCB_API int nncb_qbinary_u8(nncb_context *ctx, int op, const uint8_t *a, const uint8_t *b, uint8_t *y, size_t n, float sa, int32_t za, float sb, int32_t zb, float so, int32_t zo);
/* y = quantize(clamp(dequantize(x), lo, hi)) -- clamp/relu/relu6 between quant params
 * (kernels::stackvm::clamp / relu, reference/activation.cpp:32-55). Runs as a 256-entry table. */
NNCB_API int nncb_requant_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, size_t n, float si, int32_t zi, float so, int32_t zo, float lo, float hi);
/* Unary activations on u8 (kernels::stackvm::relu / sigmoid / swish / hard_swish,
 * src/Native/src/kernels/stackvm/reference/activation.cpp:32-38, evaluated in double like the
 * reference's UNARY_TEMPLATE, kernel_template.h:19-50):
 *   y = quantize((float)f((double)dequantize(x)))   as a 256-entry table.
 * nncb_make_activation_table / nncb_make_requant_table (host) give the tables themselves, e.g. to
 * fuse an activation into a convolution through its `lut` argument. */
typedef enum nncb_activation { NNCB_ACT_RELU = 0, NNCB_ACT_SIGMOID = 1, NNCB_ACT_SWISH = 2, NNCB_ACT_HARD_SWISH = 3 } nncb_activation;
NNCB_API int nncb_activation_u8(nncb_context *ctx, int kind, const uint8_t *x, uint8_t *y, size_t n, float si, int32_t zi, float so, int32_t zo);
NNCB_API int nncb_make_activation_table(int kind, float si, int32_t zi, float so, int32_t zo, uint8_t *table);
NNCB_API int nncb_make_requant_table(float si, int32_t zi, float so, int32_t zo, float lo, float hi, uint8_t *table);
/* softmax over the last axis of a [rows, cols] f32 tensor (kernels::stackvm::softmax,
 * tensor_ops.cpp:1054-1071; reference/softmax.cpp:30-80): exp((x - max) * beta) / sum. */
NNCB_API int nncb_softmax_f32(nncb_context *ctx, const float *in, float *out, size_t rows, int cols, float beta);
/* Channel-block copy between NHWC u8 tensors, optionally through a 256-entry table (HOST pointer or
 * NULL): dst[p][dst_off + j] = table[src[p][src_off + j]], j < len, p < pixels. This is
 * kernels::stackvm::concat (tensor_ops.cpp: concat) on the channel axis between quant params -- one
 * call per input, the table requantising it into the output's param -- and split / slice without one. */
NNCB_API int nncb_copy_channels_u8(nncb_context *ctx, const uint8_t *src, int src_c, int src_off, uint8_t *dst, int dst_c, int dst_off, int len, size_t pixels, const uint8_t *host_table);
/* kernels::stackvm::resize_image, nearest neighbour with asymmetric coordinates and floor rounding,
 * for integer factors: y[n][oy][ox] = x[n][oy / fy][ox / fx]  (NHWC u8). */
NNCB_API int nncb_resize_nearest_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int fy, int fx);
/* y[i] = table[x[i]]; table: 256 bytes, HOST pointer. */
NNCB_API int nncb_lut_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, size_t n, const uint8_t *host_table);
/* reduce_window2d max (tensor_ops.cpp: reduce_window2d, reference/reduce_window.cpp:35-105):
 * windows overlapping the padding also take the real value 0 (the zero point) into the max. */
NNCB_API int nncb_maxpool_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int kh, int kw, int stride_h, int stride_w, int pad_t, int pad_b, int pad_l, int pad_r, int32_t zero_point);
/* reduce_window2d with any reducer of the reference (reduce_op_t: 0 mean, 1 min, 2 max, 3 sum; reference/reduce_window.cpp:
 * 35-182) between quant params (si, zi) -> (so, zo). Taps outside the image contribute the real value 0. max / min work on
 * the bytes and requantise; sum and mean accumulate exactly:
 *   v = (float)(sum_valid q - cnt_valid * zi) * si;  mean: v / (float)(count_include_pad ? kh*kw : cnt_valid);  y = quantize(v) */
NNCB_API int nncb_reduce_window2d_u8(nncb_context *ctx, int op, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, int kh, int kw, int stride_h, int stride_w, int pad_t, int pad_b, int pad_l, int pad_r, int count_include_pad, float si, int32_t zi, float so, int32_t zo);
/* reduce_window2d mean over the whole image:
 *   mean = ((float)(sum q - cnt*zi) * si) / (float)cnt ; y = quantize(mean, so, zo) */
NNCB_API int nncb_global_avgpool_u8(nncb_context *ctx, const uint8_t *x, uint8_t *y, int n, int h, int w, int c, float si, int32_t zi, float so, int32_t zo);

/* ---- quantized Conv2D / MatMul (replace kernels::stackvm::conv2d, tensor_ops.cpp:181-220,
 *      and kernels::stackvm::mat_mul, tensor_ops.cpp:553-565, for u8 x u8|i8 operands) ------
 *   acc = sum over in-image taps of (xq - x_zp) * (wq - w_zp[oc])                 int32
 *   v   = clamp((float)acc * mult[oc] + bias[oc], clamp_lo, clamp_hi)              f32, no fma
 *   q   = clamp(rint(v / out_scale + out_zp), 0, 255) ; q = lut ? lut[q] : q
 * optional fused residual add (res != NULL at run):  q = quantize(deq(q; out) + deq(res; res), add_out)
 * optional second output y2 = quantize(clamp(deq(q'), y2_lo, y2_hi); y2_out) of the final q'.
 * A MatMul [M,K]x[K,N] is the 1x1 case: n=1,h=1,w=M,c=K,oc=N with weights [N][K]. */
typedef struct nncb_conv2d_desc {
    int32_t n, h, w, c;
    int32_t oc, kh, kw;
    int32_t stride_h, stride_w;
    int32_t pad_t, pad_b, pad_l, pad_r;
    int32_t dil_h, dil_w;
    int32_t groups;
    int32_t w_signed;    /* 0: u8 weights, 1: i8 weights */
    int32_t x_zp;
    float out_scale;
    int32_t out_zp;
    float clamp_lo, clamp_hi;
    /* fused residual add (used when has_residual != 0) */
    int32_t has_residual;
    float res_scale;
    int32_t res_zp;
    float add_out_scale;
    int32_t add_out_zp;
    /* second output (used when has_y2 != 0) */
    int32_t has_y2;
    float y2_scale;
    int32_t y2_zp;
    float y2_lo, y2_hi;
    /* output as f32 real values (v above, no requantisation) instead of u8 */
    int32_t f32_out;
    /* 0: choose automatically; 1: force the CUDA-core kernel; 2: force the tcgen05 kernel */
    int32_t force_path;
} nncb_conv2d_desc;

/* weights/w_zp/mult/bias/lut are HOST pointers, copied and repacked at creation.
 * w_zp may be NULL (all zero); lut may be NULL. */
NNCB_API int nncb_qconv2d_create(nncb_context *ctx, const nncb_conv2d_desc *desc, const void *weights, const int32_t *w_zp, const float *mult, const float *bias, const uint8_t *lut, nncb_qconv2d **out);
NNCB_API int nncb_qconv2d_destroy(nncb_qconv2d *conv);
/* 1 = CUDA-core kernel, 2 = tcgen05 tensor-core kernel */
NNCB_API int nncb_qconv2d_path(const nncb_qconv2d *conv);
NNCB_API int nncb_qconv2d_out_shape(const nncb_qconv2d *conv, int *oh, int *ow);
/* y: u8 NHWC [n,oh,ow,oc] (or f32 when f32_out); res and y2 may be NULL when unused. */
NNCB_API int nncb_qconv2d_run(nncb_context *ctx, nncb_qconv2d *conv, const uint8_t *x, const uint8_t *res, void *y, uint8_t *y2);
/* One-shot with HOST buffers: x u8 NHWC in, y out; weights as in create. */
NNCB_API int nncb_qconv2d_host(nncb_context *ctx, const nncb_conv2d_desc *desc, const void *weights, const int32_t *w_zp, const float *mult, const float *bias, const uint8_t *lut, const uint8_t *x, const uint8_t *res, void *y, uint8_t *y2);

/* ---- decode-step operators of a transformer with i8 weights and f16 activations -----------
 * None of these has a reference operator; they extend kernels::stackvm::mat_mul's convention
 * (f32 accumulation, reference/matmul.cpp:28-51) to weight-only quantization, with f16 storage
 * between operators. All pointers are device pointers.
 *   gemv_w8a16:  y[m][n] = f16( (sum_k x[m][k]*w[n][k]) * scale[n] + bias[n] + residual[m][n] )
 *                x f16 [m<=64][k], w i8 [n][k], scale f16 [n]; bias, residual may be NULL; k % 64 == 0.
 *   add_rmsnorm: if delta: x <- f16(x + delta) in place;  h = f16(x * rsqrt(mean(x^2) + eps) * weight)
 *   rope_kv_append: rotary embedding ("rotate half", cos/sin table [max_pos][32] f32) of the q and k
 *                parts of qkv [batch][(q_heads + 2 kv_heads) * 64]; rotated q to q_out [batch][q_heads][64],
 *                rotated k and v to page block_table[b][pos/16], slot pos%16 of the pools (the layouts
 *                nncb_paged_attention_decode reads).
 *   swiglu:      out[m][j] = f16( silu(gate_up[m][j]) * gate_up[m][inter + j] )
 *   embedding:   out[m][:] = table[ids[m]][:] */
NNCB_API int nncb_gemv_w8a16(nncb_context *ctx, const void *x, const int8_t *w, const void *scale, const void *bias, const void *residual, void *y, int m, int n, int k);
/* The gate/up MatMul with SwiGLU in its epilogue: the n weight rows come in blocks of 16 = the gate rows of 8
 * outputs followed by their up rows (scale and bias ordered alike), y is [m][n / 2] and
 * y[m][8 b + r] = f16( silu(f16(gate)) * f16(up) ) for rows r and r + 8 of block b: bit-identical to
 * nncb_gemv_w8a16 followed by nncb_swiglu_f16 on the un-interleaved rows, without the [m][n] round trip. */
NNCB_API int nncb_gemv_w8a16_swiglu(nncb_context *ctx, const void *x, const int8_t *w, const void *scale, const void *bias, void *y, int m, int n, int k);
NNCB_API int nncb_add_rmsnorm_f16(nncb_context *ctx, void *x, const void *delta, const void *weight, void *h, int rows, int cols, float eps);
/* max_pos: rows of the cos/sin tables; num_pages: pages in the pools. A position outside [0, max_pos) or beyond
 * the block-table row, or a page id outside [0, num_pages), stores nothing for that sequence and sets the
 * status word (-ERANGE from nncb_check_device_status). */
NNCB_API int nncb_rope_kv_append_f16(nncb_context *ctx, const void *qkv, void *q_out, const float *cos_table, const float *sin_table, const int32_t *positions, const int32_t *block_table, void *k_pool, void *v_pool, int batch, int q_heads, int kv_heads, int head_dim, int page_size, int max_pages, int max_pos, int num_pages);
NNCB_API int nncb_swiglu_f16(nncb_context *ctx, const void *gate_up, void *out, int rows, int inter);
NNCB_API int nncb_embedding_f16(nncb_context *ctx, const void *table, const int32_t *ids, void *out, int rows, int cols, int vocab);

/* ---- tensor-parallel decode: the all-reduce after a row-split projection, over peer memory ----------------
 * One process per GPU. Every rank allocates, with nncb_malloc, a buffer for its partial results and a flag block of
 * 128 zeroed bytes, exports both (nncb_ipc_export gives the 64-byte CUDA IPC handle to send to the other ranks) and
 * maps the other ranks' (nncb_ipc_import, in another process than the one that exported: CUDA IPC does not open a
 * process's own handles; nncb_ipc_close before the owner frees). One allocation may hold the partial buffers of both
 * slots and the flag block. (No counterpart in the reference, whose runtime is single-device.)
 * nncb_peer_allreduce_add_rmsnorm_f16 is the exchange and what follows it in a decoder block, in one launch:
 *   delta = f16( sum over ranks r = 0 .. world-1, in that order, of partials[r] in f32 );
 *   x <- f16(x + delta) in place;  h = f16(x * rsqrt(mean(x^2) + eps) * weight)          (as nncb_add_rmsnorm_f16)
 * partials[r] / flags[r]: host arrays of `world` device pointers (rank r's partial [rows][cols] f16 and flag block;
 * the own entries are local memory). Launch it after the MatMul that wrote partials[rank], on the same stream, on
 * every rank with the same slot (0 or 1: two consecutive exchanges must use different slots and different partial
 * buffers -- a rank may be one exchange ahead of a peer that still reads). The kernel tells the peers that this rank's
 * partial is ready, waits until every peer has said the same (option "peer_wait_limit_us", default 30 s; a wait that
 * runs out sets the status word, -ETIMEDOUT from nncb_check_device_status, reads no peer, and later launches
 * on the context do not wait again until the status has been read), then reads the peers' rows over NVLink with
 * plain loads. No multicast, no NCCL; works inside a captured CUDA graph (sequence numbers live in the flag blocks).
 * world 2..8; cols a multiple of 4, at most 2048. */
NNCB_API int nncb_ipc_export(nncb_context *ctx, const void *dptr, void *handle, size_t handle_bytes);
NNCB_API int nncb_ipc_import(nncb_context *ctx, const void *handle, size_t handle_bytes, void **dptr);
NNCB_API int nncb_ipc_close(nncb_context *ctx, void *dptr);
NNCB_API int nncb_peer_allreduce_add_rmsnorm_f16(nncb_context *ctx, void *x, const void *const *partials, void *const *flags, int world, int rank, int slot, const void *weight, void *h, int rows, int cols, float eps);

/* ---- paged-attention decode ---------------------------------------------------------------
 * The reference has no attention, KV-cache or softmax-over-pages operator (its native op list is
 * src/Native/include/nncase/kernels/stackvm/tensor_ops.h:29-479); this entry point defines one.
 * Math follows the reference's mat_mul and softmax kernels (reference/matmul.cpp:28-51,
 * reference/softmax.cpp:30-80): f32 scores, max-subtracted softmax, f32 value sum.
 *   q [batch][q_heads][head_dim] f16; k_pool, v_pool [num_pages][kv_heads][page_size][head_dim] f16;
 *   block_table [batch][max_pages] int32 page ids; context_lens [batch] int32 (0 gives a zero row);
 *   out [batch][q_heads][head_dim] f16.  Query head h reads kv head h / (q_heads / kv_heads).
 * Built for head_dim 64, page_size 16, q_heads / kv_heads <= 8 (others: -ENOSYS).
 * The context is split across CTAs; partial results go through `workspace` (device memory, size
 * from nncb_paged_attention_workspace_size, may be 0).
 * num_pages = pages in the pools. Indices read from device memory are bounded: a context length is
 * clamped to [0, max_pages * page_size], a page id outside [0, num_pages) contributes zeros; either sets
 * the status word (-ERANGE from nncb_check_device_status). */
NNCB_API int nncb_paged_attention_workspace_size(nncb_context *ctx, int batch, int q_heads, int kv_heads, int head_dim, int page_size, int max_pages, size_t *bytes);
NNCB_API int nncb_paged_attention_decode(nncb_context *ctx, const void *q, const void *k_pool, const void *v_pool, const int32_t *block_table, const int32_t *context_lens, void *out, int batch, int q_heads, int kv_heads, int head_dim, int page_size, int max_pages, int num_pages, float scale, void *workspace, size_t workspace_bytes);

/* The same with the step's rotary embedding and KV append inside (one launch instead of nncb_rope_kv_append_f16 +
 * nncb_paged_attention_decode, bit-identical results): qkv [batch][(q_heads + 2 kv_heads) * 64] f16 holds the
 * unrotated q, k and v heads of the new token of every sequence, positions [batch] int32 its position
 * (context_lens[b] must be positions[b] + 1 or more), cos / sin tables [max_pos][32] f32. Each CTA rotates the q
 * heads it reads; the CTA whose part of the context holds page positions[b] / 16 writes the rotated k and the v
 * into that page before it loads it. A position outside [0, max_pos), beyond the block-table row or not covered
 * by the context length appends nothing and sets the status word. */
NNCB_API int nncb_paged_attention_decode_rope(nncb_context *ctx, const void *qkv, const float *cos_table, const float *sin_table, const int32_t *positions, void *k_pool, void *v_pool, const int32_t *block_table, const int32_t *context_lens, void *out, int batch, int q_heads, int kv_heads, int head_dim, int page_size, int max_pages, int max_pos, int num_pages, float scale, void *workspace, size_t workspace_bytes);

/* Paged-attention decode for callers that must not allocate. (No counterpart in the reference.)
 *
 * Some hosts of this library hand out all device memory up front and forbid the allocator
 * afterwards: a runtime that plans every buffer when the model is loaded, an inference loop with a
 * fixed memory budget owned by another framework, code running while a stream is being captured.
 * They cannot provide (or size) the workspace that nncb_paged_attention_decode wants. This variant
 * takes the same inputs and outputs and keeps the split partials in a 768 KiB array that is part of
 * the library image on every GPU that loads it. It calls no cudaMalloc, cudaFree or other allocating
 * routine.
 *  - Limit: batch * q_heads * splits * 264 bytes must fit 768 KiB; larger problems return -E2BIG with a
 *    message that names both sizes. The library splits the context only while (sequence, kv head) pairs
 *    are too few to fill the GPU, so batch * kv_heads * splits stays near the number of CTA slots: on a
 *    148-SM part the partials reach about 625 KiB at most. A large batch such as the Qwen2-0.5B decode
 *    shape (64 sequences x 2 kv heads) runs unsplit and uses none of the array.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 *    device current) and remembers it; make that first call before starting any stream capture.
 *  - All calls on a device share the one array. Nothing in it has to be cleared between calls (every
 *    entry that is read is written first by the same call), but two calls that overlap on the GPU
 *    -- different streams, or different contexts -- race on it: serialise them.
 * Results are identical to nncb_paged_attention_decode. */
NNCB_API int nncb_paged_attention_decode_noalloc(nncb_context *ctx, const void *q, const void *k_pool, const void *v_pool, const int32_t *block_table, const int32_t *context_lens, void *out, int batch, int q_heads, int kv_heads, int head_dim, int page_size, int max_pages, int num_pages, float scale);

/* ---- float kernels for calibration ---------------------------------------------------------------
 * The forward pass the reference's Quantizer runs per calibration sample to collect ranges
 * (src/Nncase.Quantization/Quantization/Quantizer.cs:389-409) and the range reduction over finite values
 * (Quantizer.Algorithms.cs:14-30), on the GPU. Semantics of the reference's float kernels: conv2d = bias + sum over
 * in-image taps, then the fused clamp (reference/convolution.cpp:50-106); max pooling injects the value 0 for taps
 * outside the image (reference/reduce_window.cpp:86-90); swish in double (kernel_template.h:33-47).
 * NCHW f32 tensors, OIHW weights, device pointers; bias may be NULL; groups == 1 or depthwise or any divisor. */
NNCB_API int nncb_conv2d_f32(nncb_context *ctx, const float *x, const float *w, const float *bias, float *y, int n, int c, int h, int wd, int oc, int kh, int kw, int stride_h, int stride_w, int pad_t, int pad_b, int pad_l, int pad_r, int dil_h, int dil_w, int groups, float clamp_lo, float clamp_hi);
NNCB_API int nncb_clamp_f32(nncb_context *ctx, const float *x, float *y, size_t n, float lo, float hi);
NNCB_API int nncb_swish_f32(nncb_context *ctx, const float *x, float *y, size_t n);
NNCB_API int nncb_add_f32(nncb_context *ctx, const float *a, const float *b, float *y, size_t n);
NNCB_API int nncb_maxpool_f32(nncb_context *ctx, const float *x, float *y, int n, int c, int h, int w, int kh, int kw, int stride_h, int stride_w, int pad_t, int pad_b, int pad_l, int pad_r);
NNCB_API int nncb_global_mean_f32(nncb_context *ctx, const float *x, float *y, size_t planes, int hw);
/* min and max over the finite values of x (HOST results; synchronises); (FLT_MAX, -FLT_MAX) when there is none. */
NNCB_API int nncb_minmax_f32(nncb_context *ctx, const float *x, size_t n, float *min_out, float *max_out);

/* ---- a whole quantized program: the body of one kmodel function of module kind "cuda" -----------
 * The native side of the `cuda` module's runtime_function (the reference's contract:
 * src/Native/include/nncase/runtime/runtime_function.h:59-63 -- initialize_core once, invoke_core per
 * call; its StackVM counterpart is src/Native/src/runtime/stackvm/runtime_function.run.cpp:34-63).
 *   nncb_program_create   parses the function's ".desc" section and the module's ".rdata" section (HOST
 *                         pointers; the formats are written by nncase_b200/kmodel.py and described in
 *                         INTEGRATION.md), uploads weights, plans every convolution and allocates every
 *                         tensor for the batch the descriptor names. Malformed input: -EINVAL, never a crash.
 *   nncb_program_run      enqueues all kernels of one call; x is the f32 input ON THE DEVICE
 *                         ([n,c,h,w], or [n,h,w,c] when the descriptor says so). Nothing is allocated.
 *   nncb_program_run_host the same with HOST buffers: input copied in, every output copied out
 *                         (outs[i] must hold the bytes nncb_program_tensor reports for output i), then
 *                         synchronised -- the contract of the reference's synchronous functions.
 *   nncb_program_info / _output / _tensor   shapes, types, quant params and device pointers.
 *   nncb_program_set_profiling, _profile_text, _profile_ms   per-operator CUDA-event times of the last call,
 *                         as the two tables of the reference's op_profile::print
 *                         (src/Native/src/runtime/stackvm/op_profile.cpp:25-111) or as numbers. */
typedef struct nncb_program nncb_program;
NNCB_API int nncb_program_create(nncb_context *ctx, const void *desc, size_t desc_bytes, const void *rdata, size_t rdata_bytes, nncb_program **out);
NNCB_API int nncb_program_destroy(nncb_program *program);
NNCB_API int nncb_program_run(nncb_context *ctx, nncb_program *program, const float *x);
NNCB_API int nncb_program_run_host(nncb_context *ctx, nncb_program *program, const float *x_host, void *const *outs_host, int32_t n_outs);
NNCB_API int nncb_program_info(const nncb_program *program, int32_t *batch, int32_t *in_nhwc, int32_t in_chw[3], int32_t *n_outputs, int32_t *n_ops, int32_t *n_tensors);
NNCB_API int nncb_program_output(const nncb_program *program, int32_t index, int32_t *tensor);
NNCB_API int nncb_program_tensor(const nncb_program *program, int32_t tensor, void **dptr, int32_t hwc[3], int32_t *dtype, float *scale, int32_t *zero_point, size_t *bytes);
NNCB_API int nncb_program_set_profiling(nncb_program *program, int enabled);
NNCB_API uint64_t nncb_program_launches_per_call(const nncb_program *program);
NNCB_API int nncb_program_profile_text(const nncb_program *program, char *buf, size_t cap);
NNCB_API int nncb_program_profile_ms(const nncb_program *program, float *ms, int32_t n);

/* Diagnostic: the tensor-core kernel divides by a layer's output scale with a three-operation
 * sequence around a correctly rounded reciprocal. This runs that sequence against the IEEE
 * division for `count` pseudo-random operands on the device and returns how many differ
 * (expected: 0). No counterpart in the reference. */
NNCB_API int nncb_selftest_reciprocal_division(nncb_context *ctx, float scale, uint64_t count, uint64_t seed, uint64_t *mismatches);

/* Diagnostic: the measured peak of the kind::i8 tensor pipe on this GPU, the denominator of every
 * "fraction of int8 peak" this library's benchmarks report. One CTA per SM issues `mmas_per_sm`
 * back-to-back tcgen05.mma (M 128, N 256, K 32; u8 x u8, or u8 x i8 when w_signed) on operand tiles
 * resident in shared memory; no global-memory traffic, no epilogue. Timed with CUDA events on the context's
 * stream, `repeats` launches after one warm-up; returns the best and the mean rate in TOP/s (2 operations
 * per multiply-accumulate). Synchronises. No counterpart in the reference. */
NNCB_API int nncb_selftest_int8_peak(nncb_context *ctx, uint32_t mmas_per_sm, int repeats, int w_signed, double *best_tops, double *mean_tops);

/* Diagnostic: the pace at which MMAs can be issued. One CTA per SM; `issuers` warps (1 or 2, one lane each)
 * issue `mmas_per_issuer` back-to-back tcgen05.mma kind::i8 of M 128, N `n_cols` (16 .. 256, a multiple of 16),
 * K 32 on operand tiles resident in shared memory, each warp into its own TMEM accumulator, in a loop shaped
 * like a convolution's K loop (four MMAs and one descriptor step per iteration). Returns the mean over the SMs
 * of SM cycles per MMA, all issuers' MMAs counted: the floor of a K loop's pace, to set beside the tensor
 * pipe's own rate (nncb_selftest_int8_peak). Synchronises. No counterpart in the reference. */
NNCB_API int nncb_selftest_mma_issue(nncb_context *ctx, int n_cols, int issuers, uint32_t mmas_per_issuer, double *cycles_per_mma);

#ifdef __cplusplus
}
#endif
#endif /* NNCASE_B200_H */
