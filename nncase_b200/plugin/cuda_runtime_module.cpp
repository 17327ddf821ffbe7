// `cuda` module plugin for the nncase native runtime.
//
// Compiled against the reference's own headers into libnncase.simulator.cuda.so, the file name
// the interpreter dlopens for a kmodel module of kind "cuda"
// (src/Native/src/runtime/runtime_loader.cpp:58-90). Exports the two C-linkage entry points of
// the plugin contract (src/Native/include/nncase/runtime/runtime_loader.h:24-37):
//   create_runtime_module  -> a runtime_module whose lifetime owns the device context
//   collect_custom_call    -> operator-level plugins, invoked by the StackVM's CUSCALL opcode
//                             (src/Native/src/runtime/stackvm/ops/control.cpp:80-106)
// Custom calls take and return HOST tensors, like every kernel of the reference; device memory is
// internal. Each one follows the argument meaning of the kernels::stackvm function it replaces
// and forwards to the C ABI of libnncase_b200.so. Failures of the CUDA library become
// result<> errors (std::errc from the negative errno), never exceptions.
//
// This file contains no kernel code: it is glue between the reference's types (value_t, tensor,
// result<T>) and plain pointers.
#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <nncase/kernels/kernel_context.h>
#include <nncase/runtime/interpreter.h>
#include <nncase/runtime/runtime_function.h>
#include <nncase/runtime/runtime_loader.h>
#include <nncase/runtime/runtime_module.h>
#include <nncase/runtime/runtime_tensor.h>
#include <nncase/runtime/util.h>

#include "../../include/nncase_b200.h"

using namespace nncase;
using namespace nncase::runtime;

namespace {

std::error_condition to_errc(int rc) {
    // negative errno from the C ABI -> the generic category the reference's result<> carries
    return std::error_condition(-rc, std::generic_category());
}

#define NNCB_OK_OR_ERR(expr)                                                                     \
    {                                                                                            \
        int rc__ = (expr);                                                                       \
        if (rc__ < 0)                                                                            \
            return err(to_errc(rc__));                                                           \
    }

// One device context per process for operator-level calls (they have no module instance).
// Device from NNCASE_CUDA_DEVICE (default 0).
result<nncb_context *> shared_context() {
    static std::mutex mu;
    static nncb_context *ctx = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!ctx) {
        const char *e = std::getenv("NNCASE_CUDA_DEVICE");
        NNCB_OK_OR_ERR(nncb_context_create(e ? std::atoi(e) : 0, nullptr, &ctx));
    }
    return ok(ctx);
}

int qtype_of(typecode_t t) {
    switch (t) {
    case dt_uint8:
        return NNCB_U8;
    case dt_int8:
        return NNCB_I8;
    case dt_int16:
        return NNCB_I16;
    default:
        return -1;
    }
}

// cuda.quantize -- kernels::stackvm::quantize(target_type, input, quant_param)
// (src/Native/src/kernels/stackvm/tensor_ops.cpp:681-695).
// fields: int32 target typecode. args: [input f32, quant_param (quant_param_t)].
result<value_t> cuda_quantize(gsl::span<const gsl::byte> fields, const std::vector<value_t> &args,
                              const kernels::kernel_context &) {
    if (fields.size() < sizeof(int32_t) || args.size() != 2)
        return err(std::errc::invalid_argument);
    int32_t target;
    std::memcpy(&target, fields.data(), sizeof(target));
    const int qtype = qtype_of((typecode_t)target);
    if (qtype < 0)
        return err(std::errc::not_supported);
    value_t input = args[0], quant_param = args[1], output;
    try_f32_input(input_mem, input);
    try_input_with_value_type(qp, quant_param, quant_param_t);
    try_output(out_mem, output, datatype_t::from_typecode((typecode_t)target).unwrap(), input_tensor->shape());
    if (!is_contiguous(input_tensor))
        return err(std::errc::not_supported);
    try_var(ctx, shared_context());
    NNCB_OK_OR_ERR(nncb_quantize_host(ctx, input_mem, out_mem, compute_size(input_tensor->shape()), qp->scale,
                                      qp->zero_point, qtype));
    return ok(output);
}

// cuda.dequantize -- kernels::stackvm::dequantize(target_type, input, dequant_param)
// (tensor_ops.cpp:268-283). fields: int32 target typecode (f32). args: [input u8|i8|i16, param].
result<value_t> cuda_dequantize(gsl::span<const gsl::byte> fields, const std::vector<value_t> &args,
                                const kernels::kernel_context &) {
    if (fields.size() < sizeof(int32_t) || args.size() != 2)
        return err(std::errc::invalid_argument);
    int32_t target;
    std::memcpy(&target, fields.data(), sizeof(target));
    if ((typecode_t)target != dt_float32)
        return err(std::errc::not_supported);
    value_t input = args[0], dequant_param = args[1], output;
    try_input(input_mem, input);
    try_input_with_value_type(qp, dequant_param, quant_param_t);
    try_var(in_code, to_typecode(input_tensor->dtype()));
    const int qtype = qtype_of(in_code);
    if (qtype < 0 || !is_contiguous(input_tensor))
        return err(std::errc::not_supported);
    try_f32_output(out_mem, output, input_tensor->shape());
    try_var(ctx, shared_context());
    NNCB_OK_OR_ERR(nncb_dequantize_host(ctx, input_mem, out_mem, compute_size(input_tensor->shape()), qp->scale,
                                        qp->zero_point, qtype));
    return ok(output);
}

// cuda.qconv2d -- kernels::stackvm::conv2d (tensor_ops.cpp:181-220) on quantized operands.
// fields: nncb_conv2d_desc (n/h/w/c are overwritten from the input tensor).
// args: [x u8 NHWC, weights u8|i8 OHWI, w_zp i32[oc], mult f32[oc], bias f32[oc], (residual u8)].
// Returns the u8 (or f32, desc.f32_out) NHWC result; a second output is not exposed here.
result<value_t> cuda_qconv2d(gsl::span<const gsl::byte> fields, const std::vector<value_t> &args,
                             const kernels::kernel_context &) {
    if (fields.size() < sizeof(nncb_conv2d_desc) || args.size() < 5 || args.size() > 6)
        return err(std::errc::invalid_argument);
    nncb_conv2d_desc d;
    std::memcpy(&d, fields.data(), sizeof(d));
    value_t x = args[0], w = args[1], wzp = args[2], mult = args[3], bias = args[4], output;
    try_input(x_mem, x);
    try_input(w_mem, w);
    try_input(wzp_mem, wzp);
    try_f32_input(mult_mem, mult);
    try_f32_input(bias_mem, bias);
    if (x_tensor->shape().size() != 4 || w_tensor->shape().size() != 4 || !is_contiguous(x_tensor) ||
        !is_contiguous(w_tensor))
        return err(std::errc::invalid_argument);
    try_var(w_code, to_typecode(w_tensor->dtype()));
    try_var(x_code, to_typecode(x_tensor->dtype()));
    try_var(z_code, to_typecode(wzp_tensor->dtype()));
    if (w_code != dt_uint8 && w_code != dt_int8)
        return err(std::errc::not_supported);
    if (x_code != dt_uint8 || z_code != dt_int32)
        return err(std::errc::invalid_argument);
    d.n = (int32_t)x_tensor->shape()[0], d.h = (int32_t)x_tensor->shape()[1];
    d.w = (int32_t)x_tensor->shape()[2], d.c = (int32_t)x_tensor->shape()[3];
    d.oc = (int32_t)w_tensor->shape()[0], d.kh = (int32_t)w_tensor->shape()[1], d.kw = (int32_t)w_tensor->shape()[2];
    d.w_signed = w_code == dt_int8;
    d.has_y2 = 0;
    // the tensors come from a kmodel: every element count is checked before a byte is read through them
    if (d.groups <= 0 || d.c % d.groups != 0 || w_tensor->shape()[3] != (size_t)(d.c / d.groups) ||
        compute_size(wzp_tensor->shape()) != (size_t)d.oc || compute_size(mult_tensor->shape()) != (size_t)d.oc ||
        compute_size(bias_tensor->shape()) != (size_t)d.oc)
        return err(std::errc::invalid_argument);
    if (d.stride_h <= 0 || d.stride_w <= 0 || d.dil_h <= 0 || d.dil_w <= 0 || d.pad_t < 0 || d.pad_b < 0 || d.pad_l < 0 ||
        d.pad_r < 0)
        return err(std::errc::invalid_argument);
    // signed arithmetic: a kernel extent beyond the padded input must not wrap into a huge shape
    const int64_t oh = ((int64_t)d.h + d.pad_t + d.pad_b - ((int64_t)(d.kh - 1) * d.dil_h + 1)) / d.stride_h + 1;
    const int64_t ow = ((int64_t)d.w + d.pad_l + d.pad_r - ((int64_t)(d.kw - 1) * d.dil_w + 1)) / d.stride_w + 1;
    if ((int64_t)d.h + d.pad_t + d.pad_b < (int64_t)(d.kh - 1) * d.dil_h + 1 ||
        (int64_t)d.w + d.pad_l + d.pad_r < (int64_t)(d.kw - 1) * d.dil_w + 1 || oh <= 0 || ow <= 0)
        return err(std::errc::invalid_argument);
    dims_t out_shape{(size_t)d.n, (size_t)oh, (size_t)ow, (size_t)d.oc};
    const gsl::byte *res_mem = nullptr;
    if (args.size() == 6) {
        value_t res = args[5];
        try_input(r_mem, res);
        try_var(r_code, to_typecode(res_tensor->dtype()));
        if (r_code != dt_uint8 || compute_size(res_tensor->shape()) != compute_size(out_shape) || !is_contiguous(res_tensor))
            return err(std::errc::invalid_argument);
        res_mem = r_mem;
        d.has_residual = 1;
    } else {
        d.has_residual = 0;
    }
    try_output(out_mem, output, d.f32_out ? dt_float32 : dt_uint8, out_shape);
    try_var(ctx, shared_context());
    NNCB_OK_OR_ERR(nncb_qconv2d_host(ctx, &d, w_mem, reinterpret_cast<const int32_t *>(wzp_mem), mult_mem, bias_mem,
                                     nullptr, reinterpret_cast<const uint8_t *>(x_mem),
                                     reinterpret_cast<const uint8_t *>(res_mem), out_mem, nullptr));
    return ok(output);
}

// A function of the cuda module = one quantized program (sections written by nncase_b200/kmodel.py):
//   module section ".rdata"  weights and per-channel tables
//   function section ".desc" the launch list (tensor table + operator records)
// initialize_core hands both to the native executor of libnncase_b200.so (nncb_program_create: upload once,
// plan every buffer and convolution); invoke_core takes the f32 host tensor the interpreter passes, runs the
// kernels and returns host tensor(s) -- device memory never crosses the plugin boundary, so the callers of the
// reference's C API (src/Native/src/api.cpp:83-154) need nothing new.
class cuda_runtime_module;

class cuda_runtime_function final : public runtime_function {
  public:
    using runtime_function::runtime_function;
    ~cuda_runtime_function() override { nncb_program_destroy(program_); }

  protected:
    result<void> initialize_core(runtime_function_init_context &context) noexcept override;
    result<value_t> invoke_core(gsl::span<value_t> parameters, value_t return_value) noexcept override;

  private:
    nncb_program *program_ = nullptr;
    host_buffer_t desc_storage_;
};

class cuda_runtime_module final : public runtime_module {
  public:
    gsl::span<const gsl::byte> rdata() const noexcept { return rdata_; }

  protected:
    result<void> initialize_before_functions(runtime_module_init_context &context) noexcept override {
        try_var(ctx, shared_context()); // fails loudly when no B200 is present
        (void)ctx;
        if (context.header().version != 1)
            return err(std::errc::not_supported);
        try_set(rdata_, context.get_or_read_section(".rdata", rdata_storage_, false));
        return ok();
    }
    result<std::unique_ptr<runtime_function>> create_function() noexcept override {
        std::unique_ptr<runtime_function> fn(new (std::nothrow) cuda_runtime_function(*this));
        if (fn)
            return ok(std::move(fn));
        return err(std::errc::not_enough_memory);
    }

  private:
    gsl::span<const gsl::byte> rdata_;
    host_buffer_t rdata_storage_;
};

result<void> cuda_runtime_function::initialize_core(runtime_function_init_context &context) noexcept {
    try_var(desc, context.get_or_read_section(".desc", desc_storage_, false));
    try_var(ctx, shared_context());
    auto rdata = static_cast<cuda_runtime_module &>(module()).rdata();
    NNCB_OK_OR_ERR(nncb_program_create(ctx, desc.data(), desc.size(), rdata.data(), rdata.size(), &program_));
    uint8_t profiling = 0;
    auto opt = module().interp().options().get_scalar_opt<uint8_t>("profiling");
    if (opt.is_ok())
        profiling = opt.unwrap();
    NNCB_OK_OR_ERR(nncb_program_set_profiling(program_, profiling));
    return ok();
}

result<value_t> cuda_runtime_function::invoke_core(gsl::span<value_t> parameters, value_t) noexcept {
    if (!program_ || parameters.size() != 1)
        return err(std::errc::invalid_argument);
    int32_t batch = 0, nhwc = 0, chw[3] = {0, 0, 0}, n_out = 0;
    NNCB_OK_OR_ERR(nncb_program_info(program_, &batch, &nhwc, chw, &n_out, nullptr, nullptr));
    value_t input = parameters[0];
    try_f32_input(in_mem, input);
    const dims_t want = nhwc ? dims_t{(size_t)batch, (size_t)chw[1], (size_t)chw[2], (size_t)chw[0]}
                             : dims_t{(size_t)batch, (size_t)chw[0], (size_t)chw[1], (size_t)chw[2]};
    auto in_shape = input_tensor->shape();
    if (in_shape.size() != want.size() || !std::equal(in_shape.begin(), in_shape.end(), want.begin()) ||
        !is_contiguous(input_tensor))
        return err(std::errc::invalid_argument);
    std::vector<value_t> outs(n_out);
    std::vector<void *> out_ptrs(n_out);
    for (int32_t i = 0; i < n_out; i++) {
        int32_t t = 0, hwc[3] = {0, 0, 0}, dtype = 0;
        NNCB_OK_OR_ERR(nncb_program_output(program_, i, &t));
        NNCB_OK_OR_ERR(nncb_program_tensor(program_, t, nullptr, hwc, &dtype, nullptr, nullptr, nullptr));
        value_t output;
        dims_t shape{(size_t)batch, (size_t)hwc[0], (size_t)hwc[1], (size_t)hwc[2]};
        try_output(out_mem, output, dtype == NNCB_F32 ? dt_float32 : dt_uint8, shape);
        outs[i] = output;
        out_ptrs[i] = out_mem;
    }
    try_var(ctx, shared_context());
    uint8_t profiling = 0;
    auto opt = module().interp().options().get_scalar_opt<uint8_t>("profiling");
    if (opt.is_ok())
        profiling = opt.unwrap();
    NNCB_OK_OR_ERR(nncb_program_set_profiling(program_, profiling));
    NNCB_OK_OR_ERR(nncb_program_run_host(ctx, program_, in_mem, out_ptrs.data(), n_out));
    NNCB_OK_OR_ERR(nncb_check_device_status(ctx));
    if (profiling) {
        // the cuda function's own per-operator table, in the form of the reference's op_profile::print
        const int need = nncb_program_profile_text(program_, nullptr, 0);
        if (need > 0) {
            std::string text((size_t)need + 1, '\0');
            nncb_program_profile_text(program_, text.data(), text.size());
            std::fputs(text.c_str(), stdout);
        }
    }
    if (n_out == 1)
        return ok(outs[0]);
    return ok<value_t>(tuple(std::in_place, std::move(outs)));
}

} // namespace

extern "C" {
__attribute__((visibility("default"))) void
RUNTIME_MODULE_ACTIVATOR_NAME(result<std::unique_ptr<runtime_module>> &result) {
    std::unique_ptr<runtime_module> mod(new (std::nothrow) cuda_runtime_module());
    if (mod)
        result = ok(std::move(mod));
    else
        result = err(std::errc::not_enough_memory);
}

__attribute__((visibility("default"))) void RUNTIME_MODULE_COLLECTOR_NAME(
    result<std::vector<std::pair<std::string, runtime_module::custom_call_type>>> &result) {
    std::vector<std::pair<std::string, runtime_module::custom_call_type>> calls;
    calls.emplace_back("cuda.quantize", &cuda_quantize);
    calls.emplace_back("cuda.dequantize", &cuda_dequantize);
    calls.emplace_back("cuda.qconv2d", &cuda_qconv2d);
    result = ok(std::move(calls));
}
}
