// Host (`mops::*`) entry points of the C++ API. This build has no CPU implementation by
// design: the product is the sm_100a path, and a silent CPU route would hide a missing or
// broken CUDA build. The symbols exist so that every caller links; each one throws, the
// same way the reference's CUDA entry points do when it is built without CUDA
// (mops/src/hpe/hpe.cpp:48-65).
#include <stdexcept>

#include "mops.hpp"

namespace {
[[noreturn]] void no_cpu() {
    throw std::runtime_error(
        "this build of mops provides the CUDA (sm_100a) implementations only; "
        "call the mops_cuda_* / mops::cuda::* entry points with device pointers");
}
} // namespace

#define V1(S) mops::Tensor<S, 1>
#define V2(S) mops::Tensor<S, 2>
#define V3(S) mops::Tensor<S, 3>
#define I1 mops::Tensor<int32_t, 1>
#define I2 mops::Tensor<int32_t, 2>

#define P_HPE(S) V1(S), V2(S), V1(S), I2
#define P_HPE_VJP(S) V2(S), V1(S), V2(S), V1(S), I2
#define P_HPE_VJP_VJP(S) V1(S), V2(S), V2(S), V1(S), V2(S), V1(S), I2
#define P_SAP(S) V2(S), V2(S), V2(S), V1(S), I1, I1, I1
#define P_SAP_VJP(S) V2(S), V2(S), V2(S), V2(S), V2(S), V1(S), I1, I1, I1
#define P_SAP_VJP_VJP(S) V2(S), V2(S), V2(S), V2(S), V2(S), V2(S), V2(S), V2(S), V1(S), I1, I1, I1
#define P_OPSA(S) V3(S), V2(S), V2(S), I1
#define P_OPSA_VJP(S) V2(S), V2(S), V3(S), V2(S), V2(S), I1
#define P_OPSA_VJP_VJP(S) V3(S), V2(S), V2(S), V2(S), V2(S), V3(S), V2(S), V2(S), I1
#define P_OPSAW(S) V3(S), V2(S), V2(S), V2(S), I1, I1
#define P_OPSAW_VJP(S) V2(S), V2(S), V2(S), V3(S), V2(S), V2(S), V2(S), I1, I1
#define P_OPSAW_VJP_VJP(S)                                                                         \
    V3(S), V2(S), V2(S), V2(S), V2(S), V2(S), V2(S), V3(S), V2(S), V2(S), V2(S), I1, I1
#define P_SASAW(S) V3(S), V2(S), V2(S), V1(S), V3(S), I1, I1, I1, I1, I1
#define P_SASAW_VJP(S) V2(S), V2(S), V3(S), V3(S), V2(S), V2(S), V1(S), V3(S), I1, I1, I1, I1, I1
#define P_SASAW_VJP_VJP(S)                                                                         \
    V3(S), V2(S), V2(S), V3(S), V2(S), V2(S), V3(S), V3(S), V2(S), V2(S), V1(S), V3(S), I1, I1,    \
        I1, I1, I1

#define HOST_STUB(name, P)                                                                         \
    template <typename scalar_t> void mops::name(P(scalar_t)) { no_cpu(); }                        \
    template void mops::name<float>(P(float));                                                     \
    template void mops::name<double>(P(double));

HOST_STUB(homogeneous_polynomial_evaluation, P_HPE)
HOST_STUB(homogeneous_polynomial_evaluation_vjp, P_HPE_VJP)
HOST_STUB(homogeneous_polynomial_evaluation_vjp_vjp, P_HPE_VJP_VJP)
HOST_STUB(sparse_accumulation_of_products, P_SAP)
HOST_STUB(sparse_accumulation_of_products_vjp, P_SAP_VJP)
HOST_STUB(sparse_accumulation_of_products_vjp_vjp, P_SAP_VJP_VJP)
HOST_STUB(outer_product_scatter_add, P_OPSA)
HOST_STUB(outer_product_scatter_add_vjp, P_OPSA_VJP)
HOST_STUB(outer_product_scatter_add_vjp_vjp, P_OPSA_VJP_VJP)
HOST_STUB(outer_product_scatter_add_with_weights, P_OPSAW)
HOST_STUB(outer_product_scatter_add_with_weights_vjp, P_OPSAW_VJP)
HOST_STUB(outer_product_scatter_add_with_weights_vjp_vjp, P_OPSAW_VJP_VJP)
HOST_STUB(sparse_accumulation_scatter_add_with_weights, P_SASAW)
HOST_STUB(sparse_accumulation_scatter_add_with_weights_vjp, P_SASAW_VJP)
HOST_STUB(sparse_accumulation_scatter_add_with_weights_vjp_vjp, P_SASAW_VJP_VJP)
