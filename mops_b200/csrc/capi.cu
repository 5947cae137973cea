// The C ABI (include/mops.h) over the C++ API (mops.hpp).
//
// Same mechanics as the reference's shims (mops/src/*/capi.cpp, mops/include/mops/capi.hpp:
// 13-25, mops/src/capi.cpp:4-12): int64 shapes are range-checked and converted to size_t,
// the C++ call is wrapped in try/catch, std::exception -> status 1 with the message kept
// in a thread_local string, anything else -> status 2.
#include <string>

#include "../../include/mops.h"
#include "mops.hpp"
#include "runtime.hpp"

namespace {

thread_local std::string g_last_error;

size_t to_size(int64_t value) {
    if (value < 0 || static_cast<uint64_t>(value) > static_cast<uint64_t>(SIZE_MAX)) {
        throw std::runtime_error("integer value '" + std::to_string(value) +
                                 "' does not fit in size_t");
    }
    return static_cast<size_t>(value);
}

#define MOPS_B200_CONVERT(CTYPE, SCALAR, NDIM)                                                     \
    mops::Tensor<SCALAR, NDIM> cpp(const CTYPE& t) {                                               \
        mops::Tensor<SCALAR, NDIM> out;                                                            \
        out.data = t.data;                                                                         \
        for (int d = 0; d < NDIM; d++) out.shape[d] = to_size(t.shape[d]);                         \
        return out;                                                                                \
    }
MOPS_B200_CONVERT(mops_tensor_1d_f32_t, float, 1)
MOPS_B200_CONVERT(mops_tensor_2d_f32_t, float, 2)
MOPS_B200_CONVERT(mops_tensor_3d_f32_t, float, 3)
MOPS_B200_CONVERT(mops_tensor_1d_f64_t, double, 1)
MOPS_B200_CONVERT(mops_tensor_2d_f64_t, double, 2)
MOPS_B200_CONVERT(mops_tensor_3d_f64_t, double, 3)
MOPS_B200_CONVERT(mops_tensor_1d_i32_t, int32_t, 1)
MOPS_B200_CONVERT(mops_tensor_2d_i32_t, int32_t, 2)

// The SASAW second-order prototype types grad_grad_W as 2-D while the C++ API takes 3-D
// (include/mops.h); the extra extent is unknown from the C struct, which is harmless because
// that entry point only reports "Not implemented".
mops::Tensor<float, 3> widen(const mops_tensor_2d_f32_t& t) {
    return {t.data, {to_size(t.shape[0]), to_size(t.shape[1]), 0}};
}
mops::Tensor<double, 3> widen(const mops_tensor_2d_f64_t& t) {
    return {t.data, {to_size(t.shape[0]), to_size(t.shape[1]), 0}};
}

template <typename F> int guarded(F&& body) {
    try {
        body();
        return 0;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return 1;
    } catch (...) {
        g_last_error = "unknown error";
        return 2;
    }
}

} // namespace

// Argument names of every entry point, in prototype order.
#define NAMES_HPE(F) F(output), F(A), F(C), F(indices_A)
#define NAMES_HPE_VJP(F) F(grad_A), F(grad_output), F(A), F(C), F(indices_A)
#define NAMES_HPE_VJP_VJP(F)                                                                       \
    F(grad_grad_output), F(grad_A_2), F(grad_grad_A), F(grad_output), F(A), F(C), F(indices_A)
#define NAMES_SAP(F) F(output), F(A), F(B), F(C), F(indices_A), F(indices_B), F(indices_output)
#define NAMES_SAP_VJP(F)                                                                           \
    F(grad_A), F(grad_B), F(grad_output), F(A), F(B), F(C), F(indices_A), F(indices_B),            \
        F(indices_output)
#define NAMES_SAP_VJP_VJP(F)                                                                       \
    F(grad_grad_output), F(grad_A_2), F(grad_B_2), F(grad_grad_A), F(grad_grad_B),                 \
        F(grad_output), F(A), F(B), F(C), F(indices_A), F(indices_B), F(indices_output)
#define NAMES_OPSA(F) F(output), F(A), F(B), F(indices_output)
#define NAMES_OPSA_VJP(F) F(grad_A), F(grad_B), F(grad_output), F(A), F(B), F(indices_output)
#define NAMES_OPSA_VJP_VJP(F)                                                                      \
    F(grad_grad_output), F(grad_A_2), F(grad_B_2), F(grad_grad_A), F(grad_grad_B),                 \
        F(grad_output), F(A), F(B), F(indices_output)
#define NAMES_OPSAW(F) F(output), F(A), F(B), F(W), F(indices_W), F(indices_output)
#define NAMES_OPSAW_VJP(F)                                                                         \
    F(grad_A), F(grad_B), F(grad_W), F(grad_output), F(A), F(B), F(W), F(indices_W),               \
        F(indices_output)
#define NAMES_OPSAW_VJP_VJP(F)                                                                     \
    F(grad_grad_output), F(grad_A_2), F(grad_B_2), F(grad_W_2), F(grad_grad_A), F(grad_grad_B),    \
        F(grad_grad_W), F(grad_output), F(A), F(B), F(W), F(indices_W), F(indices_output)
#define NAMES_SASAW(F)                                                                             \
    F(output), F(A), F(B), F(C), F(W), F(indices_A), F(indices_W_1), F(indices_W_2),               \
        F(indices_output_1), F(indices_output_2)
#define NAMES_SASAW_VJP(F)                                                                         \
    F(grad_A), F(grad_B), F(grad_W), F(grad_output), F(A), F(B), F(C), F(W), F(indices_A),         \
        F(indices_W_1), F(indices_W_2), F(indices_output_1), F(indices_output_2)
#define NAMES_SASAW_VJP_VJP(F)                                                                     \
    F(grad_grad_output), F(grad_A_2), F(grad_B_2), F(grad_W_2), F(grad_grad_A), F(grad_grad_B),    \
        widen(grad_grad_W), F(grad_output), F(A), F(B), F(C), F(W), F(indices_A),                  \
        F(indices_W_1), F(indices_W_2), F(indices_output_1), F(indices_output_2)

#define AS_CPP(x) cpp(x)

// Device entry points call mops::cuda::<op>; host entry points call mops::<op>, which in this
// build throws (there is no CPU implementation here by design).
#define DEFINE_ENTRY(name, ARGS, NAMES)                                                            \
    extern "C" int mops_cuda_##name##_f32(ARGS(f32)) {                                             \
        return guarded([&] { mops::cuda::name<float>(NAMES(AS_CPP)); });                           \
    }                                                                                              \
    extern "C" int mops_cuda_##name##_f64(ARGS(f64)) {                                             \
        return guarded([&] { mops::cuda::name<double>(NAMES(AS_CPP)); });                          \
    }                                                                                              \
    extern "C" int mops_##name##_f32(ARGS(f32)) {                                                  \
        return guarded([&] { mops::name<float>(NAMES(AS_CPP)); });                                 \
    }                                                                                              \
    extern "C" int mops_##name##_f64(ARGS(f64)) {                                                  \
        return guarded([&] { mops::name<double>(NAMES(AS_CPP)); });                                \
    }

DEFINE_ENTRY(homogeneous_polynomial_evaluation, MOPS_ARGS_HPE, NAMES_HPE)
DEFINE_ENTRY(homogeneous_polynomial_evaluation_vjp, MOPS_ARGS_HPE_VJP, NAMES_HPE_VJP)
DEFINE_ENTRY(homogeneous_polynomial_evaluation_vjp_vjp, MOPS_ARGS_HPE_VJP_VJP, NAMES_HPE_VJP_VJP)
DEFINE_ENTRY(sparse_accumulation_of_products, MOPS_ARGS_SAP, NAMES_SAP)
DEFINE_ENTRY(sparse_accumulation_of_products_vjp, MOPS_ARGS_SAP_VJP, NAMES_SAP_VJP)
DEFINE_ENTRY(sparse_accumulation_of_products_vjp_vjp, MOPS_ARGS_SAP_VJP_VJP, NAMES_SAP_VJP_VJP)
DEFINE_ENTRY(outer_product_scatter_add, MOPS_ARGS_OPSA, NAMES_OPSA)
DEFINE_ENTRY(outer_product_scatter_add_vjp, MOPS_ARGS_OPSA_VJP, NAMES_OPSA_VJP)
DEFINE_ENTRY(outer_product_scatter_add_vjp_vjp, MOPS_ARGS_OPSA_VJP_VJP, NAMES_OPSA_VJP_VJP)
DEFINE_ENTRY(outer_product_scatter_add_with_weights, MOPS_ARGS_OPSAW, NAMES_OPSAW)
DEFINE_ENTRY(outer_product_scatter_add_with_weights_vjp, MOPS_ARGS_OPSAW_VJP, NAMES_OPSAW_VJP)
DEFINE_ENTRY(outer_product_scatter_add_with_weights_vjp_vjp, MOPS_ARGS_OPSAW_VJP_VJP,
             NAMES_OPSAW_VJP_VJP)
DEFINE_ENTRY(sparse_accumulation_scatter_add_with_weights, MOPS_ARGS_SASAW, NAMES_SASAW)
DEFINE_ENTRY(sparse_accumulation_scatter_add_with_weights_vjp, MOPS_ARGS_SASAW_VJP,
             NAMES_SASAW_VJP)
DEFINE_ENTRY(sparse_accumulation_scatter_add_with_weights_vjp_vjp, MOPS_ARGS_SASAW_VJP_VJP,
             NAMES_SASAW_VJP_VJP)

namespace mops_b200 {
void sasaw_forward_noalloc_f64(mops::Tensor<double, 3>, mops::Tensor<double, 2>,
                               mops::Tensor<double, 2>, mops::Tensor<double, 1>,
                               mops::Tensor<double, 3>, mops::Tensor<int32_t, 1>,
                               mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>,
                               mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>);
}

// Allocation-free SASAW forward (see sasaw.cu); same arguments and status convention as
// mops_cuda_sparse_accumulation_scatter_add_with_weights_f64.
extern "C" int mops_b200_cuda_sparse_accumulation_scatter_add_with_weights_noalloc_f64(
    MOPS_ARGS_SASAW(f64)) {
    return guarded([&] { mops_b200::sasaw_forward_noalloc_f64(NAMES_SASAW(AS_CPP)); });
}

extern "C" const char* mops_get_last_error_message(void) { return g_last_error.c_str(); }

extern "C" void mops_b200_set_stream(void* stream) { mops_b200::set_stream(stream); }
extern "C" void* mops_b200_get_stream(void) { return mops_b200::get_stream(); }
extern "C" void mops_b200_set_wait(int wait) { mops_b200::set_wait(wait != 0); }
extern "C" int mops_b200_get_wait(void) { return mops_b200::get_wait() ? 1 : 0; }
namespace mops_b200 {
void sort_index(mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>, int64_t);
}
extern "C" int mops_b200_cuda_sort_index(mops_tensor_1d_i32_t sorted,
                                         mops_tensor_1d_i32_t permutation,
                                         mops_tensor_1d_i32_t indices, int64_t n_rows) {
    return guarded([&] { mops_b200::sort_index(cpp(sorted), cpp(permutation), cpp(indices), n_rows); });
}

extern "C" int mops_b200_plan_create(mops_b200_plan_t** plan) {
    return guarded([&] {
        if (plan == nullptr) throw std::runtime_error("mops_b200_plan_create: plan is NULL");
        *plan = reinterpret_cast<mops_b200_plan_t*>(mops_b200::plan_create());
    });
}
extern "C" int mops_b200_plan_destroy(mops_b200_plan_t* plan) {
    return guarded([&] { mops_b200::plan_destroy(reinterpret_cast<mops_b200::TablePlan*>(plan)); });
}
extern "C" void mops_b200_plan_bind(mops_b200_plan_t* plan) {
    mops_b200::plan_bind(reinterpret_cast<mops_b200::TablePlan*>(plan));
}
extern "C" mops_b200_plan_t* mops_b200_plan_bound(void) {
    return reinterpret_cast<mops_b200_plan_t*>(mops_b200::plan_bound());
}
extern "C" int mops_b200_plan_tables(const mops_b200_plan_t* plan) {
    return mops_b200::plan_table_count(reinterpret_cast<const mops_b200::TablePlan*>(plan));
}

extern "C" const char* mops_b200_last_kernels(void) { return mops_b200::last_kernels(); }
extern "C" const char* mops_b200_version(void) { return "mops-b200 0.1 (sm_100a)"; }
