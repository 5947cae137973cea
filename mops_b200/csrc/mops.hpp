// C++ API of the B200 build: the same entry points, argument order and tensor view as the
// reference's public headers, so that code written against `mops::cuda::*` links unchanged.
//
//   Tensor view           mops/include/mops/tensor.hpp:7-13
//   HPE                   mops/include/mops/hpe.hpp:24-37, 123-192
//   SAP                   mops/include/mops/sap.hpp:184-303
//   OPSA                  mops/include/mops/opsa.hpp:145-231
//   OPSAW                 mops/include/mops/opsaw.hpp:188-307
//   SASAW                 mops/include/mops/sasaw.hpp:243-398
//
// Conventions (identical to the reference): tensors are row-major and contiguous, index
// tensors are int32 and zero-based, the caller allocates every output, outputs are fully
// overwritten, a gradient output whose `data` is nullptr is skipped. `mops::cuda::*` take
// device pointers. Errors are thrown as std::runtime_error.
//
// This build contains CUDA implementations only: the host-side `mops::*` functions exist so
// that every symbol resolves, and throw.
#ifndef MOPS_B200_MOPS_HPP
#define MOPS_B200_MOPS_HPP

#include <cstddef>
#include <cstdint>

#if defined(__GNUC__)
#define MOPS_EXPORT __attribute__((visibility("default")))
#else
#define MOPS_EXPORT
#endif

namespace mops {

template <typename scalar_t, size_t N_DIMS> struct Tensor {
    scalar_t* __restrict__ data; // first element; contiguous, row-major
    size_t shape[N_DIMS];
};

// Short names used only inside this header.
#define T1 Tensor<scalar_t, 1>
#define T2 Tensor<scalar_t, 2>
#define T3 Tensor<scalar_t, 3>
#define I1 Tensor<int32_t, 1>
#define I2 Tensor<int32_t, 2>

// The fifteen operations, declared once and stamped into both namespaces.
#define MOPS_B200_DECLARE_API                                                                      \
    /* O[i] = sum_j C[j] prod_k A[i, P[j,k]] */                                                    \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT homogeneous_polynomial_evaluation(T1 output, T2 A, T1 C, I2 indices_A);       \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT homogeneous_polynomial_evaluation_vjp(                                        \
        T2 grad_A, T1 grad_output, T2 A, T1 C, I2 indices_A);                                      \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT homogeneous_polynomial_evaluation_vjp_vjp(                                    \
        T1 grad_grad_output, T2 grad_A_2, T2 grad_grad_A, T1 grad_output, T2 A, T1 C,              \
        I2 indices_A);                                                                             \
    /* O[i, PO[k]] += C[k] A[i,PA[k]] B[i,PB[k]] */                                                \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT sparse_accumulation_of_products(                                              \
        T2 output, T2 A, T2 B, T1 C, I1 indices_A, I1 indices_B, I1 indices_output);               \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT sparse_accumulation_of_products_vjp(                                          \
        T2 grad_A, T2 grad_B, T2 grad_output, T2 A, T2 B, T1 C, I1 indices_A, I1 indices_B,        \
        I1 indices_output);                                                                        \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT sparse_accumulation_of_products_vjp_vjp(                                      \
        T2 grad_grad_output, T2 grad_A_2, T2 grad_B_2, T2 grad_grad_A, T2 grad_grad_B,             \
        T2 grad_output, T2 A, T2 B, T1 C, I1 indices_A, I1 indices_B, I1 indices_output);          \
    /* O[P[j],k,l] += A[j,k] B[j,l] */                                                             \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT outer_product_scatter_add(T3 output, T2 A, T2 B, I1 indices_output);          \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT outer_product_scatter_add_vjp(                                                \
        T2 grad_A, T2 grad_B, T3 grad_output, T2 A, T2 B, I1 indices_output);                      \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT outer_product_scatter_add_vjp_vjp(                                            \
        T3 grad_grad_output, T2 grad_A_2, T2 grad_B_2, T2 grad_grad_A, T2 grad_grad_B,             \
        T3 grad_output, T2 A, T2 B, I1 indices_output);                                            \
    /* O[PO[e],k,l] += A[e,k] B[e,l] W[PW[e],l] */                                                 \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT outer_product_scatter_add_with_weights(                                       \
        T3 output, T2 A, T2 B, T2 W, I1 indices_W, I1 indices_output);                             \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT outer_product_scatter_add_with_weights_vjp(                                   \
        T2 grad_A, T2 grad_B, T2 grad_W, T3 grad_output, T2 A, T2 B, T2 W, I1 indices_W,           \
        I1 indices_output);                                                                        \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT outer_product_scatter_add_with_weights_vjp_vjp(                               \
        T3 grad_grad_output, T2 grad_A_2, T2 grad_B_2, T2 grad_W_2, T2 grad_grad_A,                \
        T2 grad_grad_B, T2 grad_grad_W, T3 grad_output, T2 A, T2 B, T2 W, I1 indices_W,            \
        I1 indices_output);                                                                        \
    /* O[I[e],M3[n],:] += C[n] A[e,M1[n]] B[e,:] W[J[e],M2[n],:] */                                \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT sparse_accumulation_scatter_add_with_weights(                                 \
        T3 output, T2 A, T2 B, T1 C, T3 W, I1 indices_A, I1 indices_W_1, I1 indices_W_2,           \
        I1 indices_output_1, I1 indices_output_2);                                                 \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT sparse_accumulation_scatter_add_with_weights_vjp(                             \
        T2 grad_A, T2 grad_B, T3 grad_W, T3 grad_output, T2 A, T2 B, T1 C, T3 W, I1 indices_A,     \
        I1 indices_W_1, I1 indices_W_2, I1 indices_output_1, I1 indices_output_2);                 \
    template <typename scalar_t>                                                                   \
    void MOPS_EXPORT sparse_accumulation_scatter_add_with_weights_vjp_vjp(                         \
        T3 grad_grad_output, T2 grad_A_2, T2 grad_B_2, T3 grad_W_2, T2 grad_grad_A,                \
        T2 grad_grad_B, T3 grad_grad_W, T3 grad_output, T2 A, T2 B, T1 C, T3 W, I1 indices_A,      \
        I1 indices_W_1, I1 indices_W_2, I1 indices_output_1, I1 indices_output_2);

MOPS_B200_DECLARE_API
namespace cuda {
MOPS_B200_DECLARE_API
} // namespace cuda

#undef T1
#undef T2
#undef T3
#undef I1
#undef I2

} // namespace mops

#endif
