// The `cuda` module's runtime function, native side: executes a quantized program (the body of one
// kmodel function of module kind "cuda") on one device.
//
// This is what a runtime_function subclass of the reference's native runtime does
// (src/Native/include/nncase/runtime/runtime_function.h:59-63): initialize_core = parse the
// function's sections, upload weights and plan every buffer and convolution once
// (nncb_program_create); invoke_core = run the kernels for one call (nncb_program_run /
// nncb_program_run_host). It replaces the per-op fetch / pop / allocate / call loop of the StackVM
// (src/Native/src/runtime/stackvm/runtime_function.run.cpp:34-63) by a launch list that is fixed at
// load time: nothing is allocated or uploaded per call. With profiling on, every operator is
// bracketed by CUDA events on the context's stream and the result is printed in the two tables of
// the reference's op_profile (src/Native/src/runtime/stackvm/op_profile.cpp:25-111).
//
// Section format (little endian; written by nncase_b200/kmodel.py, documented in INTEGRATION.md):
//   ".desc"  (function section)  DescHeader, n_outputs x u32 tensor index, n_tensors x DescTensor,
//                                n_ops x DescOp
//   ".rdata" (module section)    weights and per-channel tables, addressed by byte offset from DescOp
// Host code only: the kernels are the ones behind the per-operator entry points of the C ABI.
#include "internal.cuh"
#include <algorithm>
#include <map>
#include <sstream>
#include <iomanip>
#include <vector>

namespace nncb {

constexpr uint32_t DESC_MAGIC = 0x4455434Eu; // "NCUD"
constexpr uint32_t DESC_VERSION = 1;

struct DescHeader {
    uint32_t magic, version, batch, n_tensors, n_ops;
    uint32_t input_tensor; // index of the tensor the input stage writes
    uint32_t input_nhwc;   // the f32 input is [n][h][w][c] (else [n][c][h][w])
    uint32_t in_c, in_h, in_w;
    uint32_t n_outputs, reserved;
};
struct DescTensor {
    uint32_t h, w, c;
    uint32_t dtype; // 0: u8, 1: f32
    int32_t zero_point;
    float scale;
};
// kind-specific fields: see the switch in nncb_program_create
struct DescOp {
    uint32_t kind;
    char name[28];
    int32_t i[24];
    float f[8];
};
enum OpKind : uint32_t { OP_QUANT_INPUT = 0, OP_CONV = 1, OP_MAXPOOL = 2, OP_REQUANT = 3, OP_ADD = 4, OP_SLICE = 5,
                         OP_CONCAT_PART = 6, OP_UPSAMPLE = 7, OP_GAP = 8, OP_KINDS = 9 };
// names as the reference's tensor functions are called (src/Native/include/nncase/kernels/stackvm/tensor_ops.h)
static const char *kind_name(uint32_t k) {
    static const char *names[OP_KINDS] = {"quantize", "conv2d", "reduce_window2d", "clamp", "binary", "slice", "concat",
                                          "resize_image", "reduce_window2d(mean)"};
    return k < OP_KINDS ? names[k] : "?";
}

} // namespace nncb

struct nncb_program {
    nncb::DescHeader h{};
    int device = 0;
    std::vector<uint32_t> outputs;
    std::vector<nncb::DescTensor> tensors;
    std::vector<nncb::DescOp> ops;
    std::vector<void *> bufs;           // one device buffer per tensor
    std::vector<nncb_qconv2d *> convs;  // per op (null unless OP_CONV)
    std::vector<std::vector<uint8_t>> tables; // per op: 256-entry host table (concat parts), empty if none
    bool profiling = false;
    std::vector<cudaEvent_t> ev;        // n_ops + 1 events when profiling
    std::vector<float> op_ms;           // last profiled call
    uint64_t launches_per_call = 0;
};

using namespace nncb;

static size_t tensor_bytes(const nncb_program *p, uint32_t t) {
    const DescTensor &d = p->tensors[t];
    return (size_t)p->h.batch * d.h * d.w * d.c * (d.dtype == 1 ? 4 : 1);
}

extern "C" {

int nncb_program_destroy(nncb_program *p) {
    if (!p)
        return 0;
    cudaSetDevice(p->device);
    for (nncb_qconv2d *c : p->convs)
        nncb_qconv2d_destroy(c);
    for (void *b : p->bufs)
        cudaFree(b);
    for (cudaEvent_t e : p->ev)
        cudaEventDestroy(e);
    delete p;
    return 0;
}

int nncb_program_create(nncb_context *ctx, const void *desc, size_t desc_bytes, const void *rdata, size_t rdata_bytes,
                        nncb_program **out) {
    if (!ctx)
        return fail(-EINVAL, "null context");
    NNCB_CUDA_TRY(cudaSetDevice(ctx->device));
    if (!desc || !out || desc_bytes < sizeof(DescHeader))
        return fail(-EINVAL, "nncb_program_create: descriptor missing or truncated");
    const uint8_t *p0 = static_cast<const uint8_t *>(desc);
    DescHeader h;
    memcpy(&h, p0, sizeof(h));
    if (h.magic != DESC_MAGIC)
        return fail(-EINVAL, "nncb_program_create: not a cuda function descriptor (magic %08x)", h.magic);
    if (h.version != DESC_VERSION)
        return fail(-ENOSYS, "nncb_program_create: descriptor version %u, this library reads version %u", h.version,
                    DESC_VERSION);
    const size_t need = sizeof(DescHeader) + (size_t)h.n_outputs * 4 + (size_t)h.n_tensors * sizeof(DescTensor) +
                        (size_t)h.n_ops * sizeof(DescOp);
    if (h.batch == 0 || h.n_tensors == 0 || h.n_ops == 0 || h.n_outputs == 0 || h.n_tensors > 65536 || h.n_ops > 65536 ||
        h.n_outputs > h.n_tensors || desc_bytes < need || h.input_tensor >= h.n_tensors)
        return fail(-EINVAL, "nncb_program_create: inconsistent descriptor header");
    nncb_program *p = new nncb_program();
    p->h = h;
    p->device = ctx->device;
    const uint8_t *q = p0 + sizeof(DescHeader);
    p->outputs.resize(h.n_outputs);
    memcpy(p->outputs.data(), q, (size_t)h.n_outputs * 4);
    q += (size_t)h.n_outputs * 4;
    p->tensors.resize(h.n_tensors);
    memcpy(p->tensors.data(), q, (size_t)h.n_tensors * sizeof(DescTensor));
    q += (size_t)h.n_tensors * sizeof(DescTensor);
    p->ops.resize(h.n_ops);
    memcpy(p->ops.data(), q, (size_t)h.n_ops * sizeof(DescOp));
    p->convs.assign(h.n_ops, nullptr);
    p->tables.assign(h.n_ops, {});
    p->bufs.assign(h.n_tensors, nullptr);
    int rc = 0;
    auto bad = [&](const char *what, uint32_t op) {
        rc = fail(-EINVAL, "nncb_program_create: op %u (%.27s): %s", op, p->ops[op].name, what);
    };
    auto tidx = [&](int32_t t) { return t >= 0 && (uint32_t)t < h.n_tensors; };
    for (uint32_t t : p->outputs)
        if (t >= h.n_tensors)
            rc = fail(-EINVAL, "nncb_program_create: output tensor index out of range");
    for (uint32_t t = 0; t < h.n_tensors && rc == 0; t++) {
        const DescTensor &d = p->tensors[t];
        if (d.h == 0 || d.w == 0 || d.c == 0 || d.dtype > 1) {
            rc = fail(-EINVAL, "nncb_program_create: tensor %u has an empty shape or an unknown type", t);
            break;
        }
        cudaError_t e = cudaMalloc(&p->bufs[t], tensor_bytes(p, t));
        if (e != cudaSuccess) {
            cudaGetLastError();
            rc = fail(-ENOMEM, "nncb_program_create: cudaMalloc(%zu) for tensor %u failed: %s", tensor_bytes(p, t), t,
                      cudaGetErrorString(e));
        }
    }
    const uint8_t *rd = static_cast<const uint8_t *>(rdata);
    auto blob = [&](int32_t off, size_t bytes) -> const void * {
        if (off < 0)
            return nullptr;
        if (!rd || (size_t)off + bytes > rdata_bytes)
            return (const void *)(uintptr_t)1; // marks "out of range"
        return rd + off;
    };
    for (uint32_t k = 0; k < h.n_ops && rc == 0; k++) {
        DescOp &op = p->ops[k];
        op.name[27] = 0;
        const int32_t *I = op.i;
        switch (op.kind) {
        case OP_QUANT_INPUT: // i: out, c, c_pad, s2d, pad t b l r
            if (!tidx(I[0]) || (uint32_t)I[0] != h.input_tensor)
                bad("input stage must write the declared input tensor", k);
            break;
        case OP_CONV: {
            // i: in, out, res, y2, oc, kh, kw, stride h w, pad t b l r, dil h w, groups, w_signed, f32_out,
            //    [18] activation table offset, [19] weights, [20] weight zero points, [21] multipliers, [22] bias
            //    (byte offsets into .rdata, -1 = absent), [23] zero point of the convolution's own output;
            //    f: clamp lo, clamp hi, scale of the convolution's own output
            if (!tidx(I[0]) || !tidx(I[1]) || (I[2] >= 0 && !tidx(I[2])) || (I[3] >= 0 && !tidx(I[3]))) {
                bad("tensor index out of range", k);
                break;
            }
            const DescTensor &ti = p->tensors[I[0]], &to = p->tensors[I[1]];
            nncb_conv2d_desc d;
            memset(&d, 0, sizeof(d));
            d.n = (int)h.batch, d.h = (int)ti.h, d.w = (int)ti.w, d.c = (int)ti.c;
            d.oc = I[4], d.kh = I[5], d.kw = I[6], d.stride_h = I[7], d.stride_w = I[8];
            d.pad_t = I[9], d.pad_b = I[10], d.pad_l = I[11], d.pad_r = I[12], d.dil_h = I[13], d.dil_w = I[14];
            d.groups = I[15], d.w_signed = I[16], d.f32_out = I[17];
            d.x_zp = ti.zero_point;
            d.clamp_lo = op.f[0], d.clamp_hi = op.f[1];
            // the convolution's own quant param (before a fused add): f[2] scale, i[23] zero point
            d.out_scale = d.f32_out ? 1.f : op.f[2], d.out_zp = d.f32_out ? 0 : I[23];
            if (I[2] >= 0) {
                d.has_residual = 1;
                d.res_scale = p->tensors[I[2]].scale, d.res_zp = p->tensors[I[2]].zero_point;
                d.add_out_scale = to.scale, d.add_out_zp = to.zero_point;
            }
            if (I[3] >= 0) {
                d.has_y2 = 1;
                d.y2_scale = p->tensors[I[3]].scale, d.y2_zp = p->tensors[I[3]].zero_point;
                d.y2_lo = 0.f, d.y2_hi = INFINITY; // the second output is the ReLU of the first
            }
            if (d.oc <= 0 || d.kh <= 0 || d.kw <= 0 || d.groups <= 0 || d.c % d.groups != 0) {
                bad("bad convolution geometry", k);
                break;
            }
            const size_t wbytes = (size_t)d.oc * d.kh * d.kw * (d.c / d.groups);
            const void *w = blob(I[19], wbytes), *wz = blob(I[20], (size_t)d.oc * 4), *mu = blob(I[21], (size_t)d.oc * 4),
                       *bi = blob(I[22], (size_t)d.oc * 4), *lutp = blob(I[18], 256);
            const void *oob = (const void *)(uintptr_t)1;
            if (!w || !mu || !bi || w == oob || wz == oob || mu == oob || bi == oob || lutp == oob) {
                bad("weights or tables outside the .rdata section", k);
                break;
            }
            rc = nncb_qconv2d_create(ctx, &d, w, (const int32_t *)wz, (const float *)mu, (const float *)bi,
                                     (const uint8_t *)lutp, &p->convs[k]);
            if (rc == 0) {
                int oh = 0, ow = 0;
                nncb_qconv2d_out_shape(p->convs[k], &oh, &ow);
                if ((uint32_t)oh != to.h || (uint32_t)ow != to.w || (uint32_t)d.oc != to.c || to.dtype != (uint32_t)d.f32_out)
                    bad("output tensor does not match the convolution's result", k);
            }
            break;
        }
        case OP_MAXPOOL: // i: in, out, k h w, stride h w, pad t b l r
        case OP_REQUANT: // i: in, out; f: lo hi
        case OP_SLICE:   // i: in, out, begin, end
        case OP_UPSAMPLE: // i: in, out, factor
        case OP_GAP:     // i: in, out
            if (!tidx(I[0]) || !tidx(I[1]))
                bad("tensor index out of range", k);
            break;
        case OP_ADD: // i: a, b, out
            if (!tidx(I[0]) || !tidx(I[1]) || !tidx(I[2]))
                bad("tensor index out of range", k);
            break;
        case OP_CONCAT_PART: { // i: in, out, channel offset in out
            if (!tidx(I[0]) || !tidx(I[1])) {
                bad("tensor index out of range", k);
                break;
            }
            const DescTensor &ti = p->tensors[I[0]], &to = p->tensors[I[1]];
            if (ti.scale != to.scale || ti.zero_point != to.zero_point) {
                p->tables[k].resize(256);
                rc = nncb_make_requant_table(ti.scale, ti.zero_point, to.scale, to.zero_point, -INFINITY, INFINITY,
                                             p->tables[k].data());
            }
            break;
        }
        default:
            bad("unknown operator kind", k);
        }
    }
    if (rc != 0) {
        nncb_program_destroy(p);
        return rc;
    }
    *out = p;
    return 0;
}

// Enqueues every kernel of one call on the context's stream. x_dev: the f32 input on the device.
int nncb_program_run(nncb_context *ctx, nncb_program *p, const float *x_dev) {
    if (!ctx || !p || !x_dev)
        return fail(-EINVAL, "nncb_program_run: null argument");
    if (p->device != ctx->device)
        return fail(-EINVAL, "nncb_program_run: program belongs to device %d, context to %d", p->device, ctx->device);
    NNCB_CUDA_TRY(cudaSetDevice(ctx->device));
    const DescHeader &h = p->h;
    const int B = (int)h.batch;
    const uint64_t l0 = nncb_launch_count(ctx);
    if (p->profiling) {
        if (p->ev.size() != p->ops.size() + 1) {
            p->ev.resize(p->ops.size() + 1);
            for (auto &e : p->ev)
                NNCB_CUDA_TRY(cudaEventCreate(&e));
        }
        NNCB_CUDA_TRY(cudaEventRecord(p->ev[0], ctx->stream));
    }
    for (size_t k = 0; k < p->ops.size(); k++) {
        const DescOp &op = p->ops[k];
        const int32_t *I = op.i;
        auto T = [&](int32_t t) -> const DescTensor & { return p->tensors[t]; };
        auto U8 = [&](int32_t t) { return static_cast<uint8_t *>(p->bufs[t]); };
        switch (op.kind) {
        case OP_QUANT_INPUT: {
            const DescTensor &to = T(I[0]);
            const int c = I[1], c_pad = I[2];
            if (I[3] && (I[4] | I[5] | I[6] | I[7])) {
                NNCB_TRY(nncb_quantize_to_s2d_padded_u8(ctx, x_dev, (int)h.input_nhwc, U8(I[0]), B, c, (int)h.in_h, (int)h.in_w,
                                                        c_pad, I[4], I[5], I[6], I[7], to.scale, to.zero_point));
            } else if (h.input_nhwc) {
                if (I[3])
                    NNCB_TRY(nncb_quantize_nhwc_to_s2d_u8(ctx, x_dev, U8(I[0]), B, (int)h.in_h, (int)h.in_w, c, c_pad, to.scale,
                                                          to.zero_point));
                else if (c_pad == c)
                    NNCB_TRY(nncb_quantize(ctx, x_dev, U8(I[0]), (size_t)B * h.in_h * h.in_w * c, to.scale, to.zero_point,
                                           NNCB_U8));
                else
                    return fail(-ENOSYS, "nncb_program_run: NHWC input with channel padding is only built for stride-2 stems");
            } else if (I[3]) {
                NNCB_TRY(nncb_quantize_nchw_to_s2d_u8(ctx, x_dev, U8(I[0]), B, c, (int)h.in_h, (int)h.in_w, c_pad, to.scale,
                                                      to.zero_point));
            } else {
                NNCB_TRY(nncb_quantize_nchw_to_nhwc_u8(ctx, x_dev, U8(I[0]), B, c, (int)h.in_h, (int)h.in_w, c_pad, to.scale,
                                                       to.zero_point));
            }
            break;
        }
        case OP_CONV:
            NNCB_TRY(nncb_qconv2d_run(ctx, p->convs[k], U8(I[0]), I[2] >= 0 ? U8(I[2]) : nullptr, p->bufs[I[1]],
                                      I[3] >= 0 ? U8(I[3]) : nullptr));
            break;
        case OP_MAXPOOL:
            NNCB_TRY(nncb_maxpool_u8(ctx, U8(I[0]), U8(I[1]), B, (int)T(I[0]).h, (int)T(I[0]).w, (int)T(I[0]).c, I[2], I[3], I[4],
                                     I[5], I[6], I[7], I[8], I[9], T(I[0]).zero_point));
            break;
        case OP_REQUANT:
            NNCB_TRY(nncb_requant_u8(ctx, U8(I[0]), U8(I[1]), tensor_bytes(p, I[0]), T(I[0]).scale, T(I[0]).zero_point,
                                     T(I[1]).scale, T(I[1]).zero_point, op.f[0], op.f[1]));
            break;
        case OP_ADD:
            NNCB_TRY(nncb_qadd_u8(ctx, U8(I[0]), U8(I[1]), U8(I[2]), tensor_bytes(p, I[2]), T(I[0]).scale, T(I[0]).zero_point,
                                  T(I[1]).scale, T(I[1]).zero_point, T(I[2]).scale, T(I[2]).zero_point));
            break;
        case OP_SLICE:
            NNCB_TRY(nncb_copy_channels_u8(ctx, U8(I[0]), (int)T(I[0]).c, I[2], U8(I[1]), I[3] - I[2], 0, I[3] - I[2],
                                           (size_t)B * T(I[0]).h * T(I[0]).w, nullptr));
            break;
        case OP_CONCAT_PART:
            NNCB_TRY(nncb_copy_channels_u8(ctx, U8(I[0]), (int)T(I[0]).c, 0, U8(I[1]), (int)T(I[1]).c, I[2], (int)T(I[0]).c,
                                           (size_t)B * T(I[1]).h * T(I[1]).w,
                                           p->tables[k].empty() ? nullptr : p->tables[k].data()));
            break;
        case OP_UPSAMPLE:
            NNCB_TRY(nncb_resize_nearest_u8(ctx, U8(I[0]), U8(I[1]), B, (int)T(I[0]).h, (int)T(I[0]).w, (int)T(I[0]).c, I[2],
                                            I[2]));
            break;
        case OP_GAP:
            NNCB_TRY(nncb_global_avgpool_u8(ctx, U8(I[0]), U8(I[1]), B, (int)T(I[0]).h, (int)T(I[0]).w, (int)T(I[0]).c,
                                            T(I[0]).scale, T(I[0]).zero_point, T(I[1]).scale, T(I[1]).zero_point));
            break;
        default:
            return fail(-EINVAL, "nncb_program_run: unknown operator kind %u", op.kind);
        }
        if (p->profiling)
            NNCB_CUDA_TRY(cudaEventRecord(p->ev[k + 1], ctx->stream));
    }
    p->launches_per_call = nncb_launch_count(ctx) - l0;
    if (p->profiling) {
        NNCB_CUDA_TRY(cudaEventSynchronize(p->ev.back()));
        p->op_ms.assign(p->ops.size(), 0.f);
        for (size_t k = 0; k < p->ops.size(); k++)
            cudaEventElapsedTime(&p->op_ms[k], p->ev[k], p->ev[k + 1]);
    }
    return 0;
}

int nncb_program_info(const nncb_program *p, int32_t *batch, int32_t *in_nhwc, int32_t in_chw[3], int32_t *n_outputs,
                      int32_t *n_ops, int32_t *n_tensors) {
    if (!p)
        return fail(-EINVAL, "nncb_program_info: null program");
    if (batch)
        *batch = (int32_t)p->h.batch;
    if (in_nhwc)
        *in_nhwc = (int32_t)p->h.input_nhwc;
    if (in_chw)
        in_chw[0] = (int32_t)p->h.in_c, in_chw[1] = (int32_t)p->h.in_h, in_chw[2] = (int32_t)p->h.in_w;
    if (n_outputs)
        *n_outputs = (int32_t)p->h.n_outputs;
    if (n_ops)
        *n_ops = (int32_t)p->h.n_ops;
    if (n_tensors)
        *n_tensors = (int32_t)p->h.n_tensors;
    return 0;
}

int nncb_program_tensor(const nncb_program *p, int32_t tensor, void **dptr, int32_t hwc[3], int32_t *dtype, float *scale,
                        int32_t *zero_point, size_t *bytes) {
    if (!p || tensor < 0 || (size_t)tensor >= p->tensors.size())
        return fail(-EINVAL, "nncb_program_tensor: bad argument");
    const DescTensor &d = p->tensors[tensor];
    if (dptr)
        *dptr = p->bufs[tensor];
    if (hwc)
        hwc[0] = (int32_t)d.h, hwc[1] = (int32_t)d.w, hwc[2] = (int32_t)d.c;
    if (dtype)
        *dtype = d.dtype == 1 ? NNCB_F32 : NNCB_U8;
    if (scale)
        *scale = d.scale;
    if (zero_point)
        *zero_point = d.zero_point;
    if (bytes)
        *bytes = tensor_bytes(p, tensor);
    return 0;
}

int nncb_program_output(const nncb_program *p, int32_t index, int32_t *tensor) {
    if (!p || !tensor || index < 0 || (size_t)index >= p->outputs.size())
        return fail(-EINVAL, "nncb_program_output: bad argument");
    *tensor = (int32_t)p->outputs[index];
    return 0;
}

// Host in, host out: copies the f32 input to a staging buffer on the device, runs, copies every output
// back and synchronises -- the contract of the reference's synchronous functions.
int nncb_program_run_host(nncb_context *ctx, nncb_program *p, const float *x_host, void *const *outs_host, int32_t n_outs) {
    if (!ctx || !p || !x_host || !outs_host)
        return fail(-EINVAL, "nncb_program_run_host: null argument");
    if (n_outs != (int32_t)p->outputs.size())
        return fail(-EINVAL, "nncb_program_run_host: the program has %zu outputs, %d buffers given", p->outputs.size(), n_outs);
    NNCB_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t in_bytes = (size_t)p->h.batch * p->h.in_c * p->h.in_h * p->h.in_w * sizeof(float);
    float *xd = nullptr;
    cudaError_t e = cudaMalloc(&xd, in_bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(-ENOMEM, "nncb_program_run_host: cudaMalloc(%zu) failed: %s", in_bytes, cudaGetErrorString(e));
    }
    int rc = 0;
    e = cudaMemcpyAsync(xd, x_host, in_bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess)
        rc = fail(-EIO, "nncb_program_run_host: input copy failed: %s", cudaGetErrorString(e));
    if (rc == 0)
        rc = nncb_program_run(ctx, p, xd);
    for (size_t i = 0; i < p->outputs.size() && rc == 0; i++) {
        e = cudaMemcpyAsync(outs_host[i], p->bufs[p->outputs[i]], tensor_bytes(p, p->outputs[i]), cudaMemcpyDeviceToHost,
                            ctx->stream);
        if (e != cudaSuccess)
            rc = fail(-EIO, "nncb_program_run_host: output copy failed: %s", cudaGetErrorString(e));
    }
    e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess && rc == 0)
        rc = fail(-EIO, "nncb_program_run_host: %s", cudaGetErrorString(e));
    cudaFree(xd);
    return rc;
}

int nncb_program_set_profiling(nncb_program *p, int enabled) {
    if (!p)
        return fail(-EINVAL, "nncb_program_set_profiling: null program");
    p->profiling = enabled != 0;
    return 0;
}

uint64_t nncb_program_launches_per_call(const nncb_program *p) { return p ? p->launches_per_call : 0; }

// The two tables of the reference's op_profile::print for the last profiled call: the timeline (one row per
// operator: name, start, end, duration in ms relative to the first operator) and the per-kind summary sorted
// by time (count, ms, percent). Returns the number of bytes the full text needs (excluding the terminator);
// at most cap - 1 bytes are written.
int nncb_program_profile_text(const nncb_program *p, char *buf, size_t cap) {
    if (!p)
        return fail(-EINVAL, "nncb_program_profile_text: null program");
    if (p->op_ms.size() != p->ops.size())
        return fail(-ENODATA, "nncb_program_profile_text: no profiled call yet (nncb_program_set_profiling, then run)");
    std::ostringstream os;
    auto cell = [&](int w, const std::string &s) { os << "|" << std::setw(w) << std::left << s; };
    auto num = [](double v) {
        std::ostringstream t;
        t << v;
        return t.str();
    };
    os << "stack OPs timeline\n";
    cell(24, "cuda tensor op"), cell(28, "name"), cell(24, "start timing(ms)"), cell(24, "end timing(ms)"), cell(24, "cast(ms)");
    os << "|\n";
    cell(24, "---"), cell(28, "---"), cell(24, "---"), cell(24, "---"), cell(24, "---");
    os << "|\n";
    double t = 0, total = 0;
    std::map<std::string, std::pair<size_t, double>> agg;
    for (size_t k = 0; k < p->ops.size(); k++) {
        const double dt = p->op_ms[k];
        cell(24, kind_name(p->ops[k].kind)), cell(28, p->ops[k].name), cell(24, num(t)), cell(24, num(t + dt)), cell(24, num(dt));
        os << "|\n";
        t += dt, total += dt;
        auto &a = agg[kind_name(p->ops[k].kind)];
        a.first++, a.second += dt;
    }
    std::vector<std::pair<std::string, std::pair<size_t, double>>> v(agg.begin(), agg.end());
    std::sort(v.begin(), v.end(), [](const auto &a, const auto &b) { return a.second.second > b.second.second; });
    os << "\ncuda OPs profile\n";
    cell(24, "cuda tensor op"), cell(6, "count"), cell(12, "timing(ms)"), cell(12, "percent(%)");
    os << "|\n";
    cell(24, "---"), cell(6, "---"), cell(12, "---"), cell(12, "---");
    os << "|\n";
    size_t count = 0;
    for (auto &e : v) {
        cell(24, e.first), cell(6, std::to_string(e.second.first)), cell(12, num(e.second.second)),
            cell(12, num(total > 0 ? e.second.second / total * 100 : 0));
        os << "|\n";
        count += e.second.first;
    }
    cell(24, "total"), cell(6, std::to_string(count)), cell(12, num(total)), cell(12, "100");
    os << "|\n";
    const std::string s = os.str();
    if (buf && cap) {
        const size_t n = std::min(cap - 1, s.size());
        memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    return (int)s.size();
}

// Per-operator milliseconds of the last profiled call (n values), for callers that want numbers, not text.
int nncb_program_profile_ms(const nncb_program *p, float *ms, int32_t n) {
    if (!p || !ms)
        return fail(-EINVAL, "nncb_program_profile_ms: null argument");
    if (p->op_ms.size() != p->ops.size() || n != (int32_t)p->ops.size())
        return fail(-ENODATA, "nncb_program_profile_ms: no profiled call yet, or n is not the operator count");
    memcpy(ms, p->op_ms.data(), sizeof(float) * p->ops.size());
    return 0;
}

} // extern "C"
