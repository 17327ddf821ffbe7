// Test harness: drives the `cuda` plugin the way the reference runtime does.
//
// Compiled against the reference's headers and linked with the reference's own native runtime
// (oracle/_ref/libnncase_ref.so, simulator mode). It asks the REFERENCE's loader for the module
// kind "cuda" -- runtime_module::collect / runtime_module::create
// (src/Native/src/runtime/runtime_loader.cpp:118-144), which dlopens
// libnncase.simulator.cuda.so and resolves collect_custom_call / create_runtime_module -- and
// invokes the custom calls with host tensors exactly as the StackVM's CUSCALL opcode does
// (src/Native/src/runtime/stackvm/ops/control.cpp:80-106).
#include <cstring>
#include <nncase/runtime/runtime_module.h>
#include <nncase/runtime/runtime_tensor.h>
#include <nncase/runtime/util.h>
#include <string>

using namespace nncase;
using namespace nncase::runtime;

namespace {
module_kind_t cuda_kind() {
    module_kind_t k{};
    std::strncpy(k.data(), "cuda", k.size() - 1);
    return k;
}

result<runtime_module::custom_call_type> find_call(const char *name) {
    try_var(table, runtime_module::collect(cuda_kind()));
    for (auto &p : table)
        if (p.first == name)
            return ok(p.second);
    return err(std::errc::no_such_file_or_directory);
}

result<value_t> host_tensor(typecode_t dt, dims_t shape, const void *data, size_t bytes) {
    try_var(t, hrt::create(dt, shape, {(gsl::byte *)data, bytes}, true, hrt::pool_cpu_only));
    return ok<value_t>(t.impl());
}

int code_of(const std::error_condition &e) { return e.value() > 0 ? -e.value() : (e.value() ? e.value() : -1); }

result<void> copy_out(value_t val, void *dst, size_t bytes) {
    try_var(t, val.as<tensor>());
    try_var(src, get_input_data(t));
    std::memcpy(dst, src, bytes);
    return ok();
}
} // namespace

extern "C" {

// Names of the custom calls the plugin registers, '\n'-separated; returns the count or < 0.
int harness_list_custom_calls(char *buf, size_t cap) {
    auto r = runtime_module::collect(cuda_kind());
    if (!r.is_ok())
        return code_of(r.unwrap_err());
    std::string s;
    for (auto &p : r.unwrap())
        s += p.first + "\n";
    std::strncpy(buf, s.c_str(), cap - 1);
    buf[cap - 1] = 0;
    return (int)r.unwrap().size();
}

// 0 when the reference's loader can activate a module of kind "cuda".
int harness_create_module(void) {
    auto r = runtime_module::create(cuda_kind());
    return r.is_ok() ? 0 : code_of(r.unwrap_err());
}

int harness_quantize(const float *in, size_t n, float scale, int32_t zp, int32_t target_typecode, void *out,
                     size_t out_elem_bytes) {
    auto run = [&]() -> result<void> {
        try_var(call, find_call("cuda.quantize"));
        try_var(x, host_tensor(dt_float32, dims_t{n}, in, n * 4));
        quant_param_t qp{zp, scale};
        try_var(q, host_tensor(dt_uint8, dims_t{sizeof(qp)}, &qp, sizeof(qp)));
        std::vector<value_t> args{x, q};
        try_var(y, call({(const gsl::byte *)&target_typecode, sizeof(int32_t)}, args, kernels::default_kernel_context()));
        return copy_out(y, out, n * out_elem_bytes);
    };
    auto r = run();
    return r.is_ok() ? 0 : code_of(r.unwrap_err());
}

int harness_dequantize(const uint8_t *in, size_t n, float scale, int32_t zp, float *out) {
    auto run = [&]() -> result<void> {
        try_var(call, find_call("cuda.dequantize"));
        try_var(x, host_tensor(dt_uint8, dims_t{n}, in, n));
        quant_param_t qp{zp, scale};
        try_var(q, host_tensor(dt_uint8, dims_t{sizeof(qp)}, &qp, sizeof(qp)));
        std::vector<value_t> args{x, q};
        int32_t target = dt_float32;
        try_var(y, call({(const gsl::byte *)&target, sizeof(int32_t)}, args, kernels::default_kernel_context()));
        return copy_out(y, out, n * 4);
    };
    auto r = run();
    return r.is_ok() ? 0 : code_of(r.unwrap_err());
}

// desc: bytes of nncb_conv2d_desc. x [n,h,w,c] u8, w [oc,kh,kw,gic] u8 (w_signed 0) or i8 (1).
int harness_qconv2d(const void *desc, size_t desc_bytes, const uint8_t *x, const size_t *x_shape, const void *w,
                    const size_t *w_shape, int w_signed, const int32_t *w_zp, const float *mult, const float *bias,
                    const uint8_t *res, uint8_t *out, size_t out_bytes) {
    auto run = [&]() -> result<void> {
        try_var(call, find_call("cuda.qconv2d"));
        dims_t xs(x_shape, x_shape + 4), ws(w_shape, w_shape + 4);
        const size_t oc = ws[0];
        try_var(tx, host_tensor(dt_uint8, xs, x, xs[0] * xs[1] * xs[2] * xs[3]));
        try_var(tw, host_tensor(w_signed ? dt_int8 : dt_uint8, ws, w, ws[0] * ws[1] * ws[2] * ws[3]));
        try_var(tz, host_tensor(dt_int32, dims_t{oc}, w_zp, oc * 4));
        try_var(tm, host_tensor(dt_float32, dims_t{oc}, mult, oc * 4));
        try_var(tb, host_tensor(dt_float32, dims_t{oc}, bias, oc * 4));
        std::vector<value_t> args{tx, tw, tz, tm, tb};
        if (res) {
            try_var(tr, host_tensor(dt_uint8, dims_t{out_bytes}, res, out_bytes));
            args.push_back(tr);
        }
        try_var(y, call({(const gsl::byte *)desc, desc_bytes}, args, kernels::default_kernel_context()));
        return copy_out(y, out, out_bytes);
    };
    auto r = run();
    return r.is_ok() ? 0 : code_of(r.unwrap_err());
}
}
