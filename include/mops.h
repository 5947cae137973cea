/* C ABI of the B200 build of the mops sparse operations.
 *
 * Binary-compatible with the C ABI of lab-cosmo/mops: the same 60 entry points plus the
 * error getter, the same by-value tensor structs, the same argument order and the same
 * status convention. A program or binding written against the reference's `mops.h`
 * (ctypes in python/mops/src/mops/_c_api.py:60-872, any C caller) can load this library
 * instead of the reference's `libmops.so` without being rebuilt.
 *
 * Interfaces replaced, by file in the reference tree:
 *   tensor structs                         mops/include/mops/tensor.h:11-49
 *   mops_get_last_error_message            mops/include/mops.h:16, mops/src/capi.cpp:4-12
 *   homogeneous_polynomial_evaluation      mops/include/mops/hpe.h:12-125
 *   sparse_accumulation_of_products        mops/include/mops/sap.h:12-169
 *   outer_product_scatter_add              mops/include/mops/opsa.h:12-133
 *   outer_product_scatter_add_with_weights mops/include/mops/opsaw.h:12-170
 *   sparse_accumulation_scatter_add_with_weights   mops/include/mops/sasaw.h:12-226
 *
 * Every operation <op> exists as
 *     int mops_<op>_{f32,f64}(...)        host pointers  -- NOT implemented in this build:
 *                                         returns 1 with an explanatory message
 *     int mops_cuda_<op>_{f32,f64}(...)   device pointers -- the sm_100a kernels
 * for <op> itself, <op>_vjp and <op>_vjp_vjp.
 *
 * Conventions (as in the reference):
 *   - tensors are passed by value as {data, shape[N]}; data is contiguous, row-major;
 *     index tensors are int32 and zero-based; mops_cuda_* take device pointers of the
 *     current CUDA device;
 *   - the caller allocates every output; outputs are fully overwritten;
 *   - a gradient output with data == NULL is skipped;
 *   - return 0 on success, 1 on error (message stored per thread), 2 on unknown error;
 *   - mops_cuda_* return when the results are complete.
 * Differences from the reference CUDA path, all on the safe side: index arrays are
 * range-checked on the device and reported (status 1) instead of being trusted; scatter
 * indices (indices_output, indices_output_1) need not be sorted, sorted input is merely the
 * fast path; CUDA errors are reported through the status instead of terminating the process.
 */
#ifndef MOPS_H
#define MOPS_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define MOPS_EXPORT __attribute__((visibility("default")))
#else
#define MOPS_EXPORT
#endif

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__cplusplus) || defined(__GNUC__)
#define MOPS_RESTRICT __restrict__
#else
#define MOPS_RESTRICT restrict
#endif

#define MOPS_TENSOR_STRUCT(name, type, ndim)                                                       \
    struct name {                                                                                  \
        type* MOPS_RESTRICT data;                                                                  \
        int64_t shape[ndim];                                                                       \
    };                                                                                             \
    typedef struct name name

MOPS_TENSOR_STRUCT(mops_tensor_1d_f32_t, float, 1);
MOPS_TENSOR_STRUCT(mops_tensor_2d_f32_t, float, 2);
MOPS_TENSOR_STRUCT(mops_tensor_3d_f32_t, float, 3);
MOPS_TENSOR_STRUCT(mops_tensor_1d_f64_t, double, 1);
MOPS_TENSOR_STRUCT(mops_tensor_2d_f64_t, double, 2);
MOPS_TENSOR_STRUCT(mops_tensor_3d_f64_t, double, 3);
MOPS_TENSOR_STRUCT(mops_tensor_1d_i32_t, int32_t, 1);
MOPS_TENSOR_STRUCT(mops_tensor_2d_i32_t, int32_t, 2);

/* Parameter lists, S = f32 or f64. Outputs first, then grad_output, inputs, indices. */
#define MOPS_V1(S) mops_tensor_1d_##S##_t
#define MOPS_V2(S) mops_tensor_2d_##S##_t
#define MOPS_V3(S) mops_tensor_3d_##S##_t
#define MOPS_I1 mops_tensor_1d_i32_t
#define MOPS_I2 mops_tensor_2d_i32_t

/* O[i] = sum_j C[j] prod_k A[i, indices_A[j,k]] */
#define MOPS_ARGS_HPE(S) MOPS_V1(S) output, MOPS_V2(S) A, MOPS_V1(S) C, MOPS_I2 indices_A
#define MOPS_ARGS_HPE_VJP(S)                                                                       \
    MOPS_V2(S) grad_A, MOPS_V1(S) grad_output, MOPS_V2(S) A, MOPS_V1(S) C, MOPS_I2 indices_A
#define MOPS_ARGS_HPE_VJP_VJP(S)                                                                   \
    MOPS_V1(S) grad_grad_output, MOPS_V2(S) grad_A_2, MOPS_V2(S) grad_grad_A,                      \
        MOPS_V1(S) grad_output, MOPS_V2(S) A, MOPS_V1(S) C, MOPS_I2 indices_A

/* O[i, indices_output[k]] += C[k] A[i, indices_A[k]] B[i, indices_B[k]] */
#define MOPS_ARGS_SAP(S)                                                                           \
    MOPS_V2(S) output, MOPS_V2(S) A, MOPS_V2(S) B, MOPS_V1(S) C, MOPS_I1 indices_A,                \
        MOPS_I1 indices_B, MOPS_I1 indices_output
#define MOPS_ARGS_SAP_VJP(S)                                                                       \
    MOPS_V2(S) grad_A, MOPS_V2(S) grad_B, MOPS_V2(S) grad_output, MOPS_V2(S) A, MOPS_V2(S) B,      \
        MOPS_V1(S) C, MOPS_I1 indices_A, MOPS_I1 indices_B, MOPS_I1 indices_output
#define MOPS_ARGS_SAP_VJP_VJP(S)                                                                   \
    MOPS_V2(S) grad_grad_output, MOPS_V2(S) grad_A_2, MOPS_V2(S) grad_B_2,                         \
        MOPS_V2(S) grad_grad_A, MOPS_V2(S) grad_grad_B, MOPS_V2(S) grad_output, MOPS_V2(S) A,      \
        MOPS_V2(S) B, MOPS_V1(S) C, MOPS_I1 indices_A, MOPS_I1 indices_B, MOPS_I1 indices_output

/* O[indices_output[j], k, l] += A[j,k] B[j,l] */
#define MOPS_ARGS_OPSA(S) MOPS_V3(S) output, MOPS_V2(S) A, MOPS_V2(S) B, MOPS_I1 indices_output
#define MOPS_ARGS_OPSA_VJP(S)                                                                      \
    MOPS_V2(S) grad_A, MOPS_V2(S) grad_B, MOPS_V3(S) grad_output, MOPS_V2(S) A, MOPS_V2(S) B,      \
        MOPS_I1 indices_output
#define MOPS_ARGS_OPSA_VJP_VJP(S)                                                                  \
    MOPS_V3(S) grad_grad_output, MOPS_V2(S) grad_A_2, MOPS_V2(S) grad_B_2,                         \
        MOPS_V2(S) grad_grad_A, MOPS_V2(S) grad_grad_B, MOPS_V3(S) grad_output, MOPS_V2(S) A,      \
        MOPS_V2(S) B, MOPS_I1 indices_output

/* O[indices_output[e], k, l] += A[e,k] B[e,l] W[indices_W[e], l] */
#define MOPS_ARGS_OPSAW(S)                                                                         \
    MOPS_V3(S) output, MOPS_V2(S) A, MOPS_V2(S) B, MOPS_V2(S) W, MOPS_I1 indices_W,                \
        MOPS_I1 indices_output
#define MOPS_ARGS_OPSAW_VJP(S)                                                                     \
    MOPS_V2(S) grad_A, MOPS_V2(S) grad_B, MOPS_V2(S) grad_W, MOPS_V3(S) grad_output,               \
        MOPS_V2(S) A, MOPS_V2(S) B, MOPS_V2(S) W, MOPS_I1 indices_W, MOPS_I1 indices_output
#define MOPS_ARGS_OPSAW_VJP_VJP(S)                                                                 \
    MOPS_V3(S) grad_grad_output, MOPS_V2(S) grad_A_2, MOPS_V2(S) grad_B_2, MOPS_V2(S) grad_W_2,    \
        MOPS_V2(S) grad_grad_A, MOPS_V2(S) grad_grad_B, MOPS_V2(S) grad_grad_W,                    \
        MOPS_V3(S) grad_output, MOPS_V2(S) A, MOPS_V2(S) B, MOPS_V2(S) W, MOPS_I1 indices_W,       \
        MOPS_I1 indices_output

/* O[indices_output_1[e], indices_output_2[n], :] +=
 *     C[n] A[e, indices_A[n]] B[e, :] W[indices_W_1[e], indices_W_2[n], :] */
#define MOPS_ARGS_SASAW(S)                                                                         \
    MOPS_V3(S) output, MOPS_V2(S) A, MOPS_V2(S) B, MOPS_V1(S) C, MOPS_V3(S) W,                     \
        MOPS_I1 indices_A, MOPS_I1 indices_W_1, MOPS_I1 indices_W_2, MOPS_I1 indices_output_1,     \
        MOPS_I1 indices_output_2
#define MOPS_ARGS_SASAW_VJP(S)                                                                     \
    MOPS_V2(S) grad_A, MOPS_V2(S) grad_B, MOPS_V3(S) grad_W, MOPS_V3(S) grad_output,               \
        MOPS_V2(S) A, MOPS_V2(S) B, MOPS_V1(S) C, MOPS_V3(S) W, MOPS_I1 indices_A,                 \
        MOPS_I1 indices_W_1, MOPS_I1 indices_W_2, MOPS_I1 indices_output_1,                        \
        MOPS_I1 indices_output_2
/* grad_grad_W is declared 2-D in the reference's C header (sasaw.h:84); kept as is. */
#define MOPS_ARGS_SASAW_VJP_VJP(S)                                                                 \
    MOPS_V3(S) grad_grad_output, MOPS_V2(S) grad_A_2, MOPS_V2(S) grad_B_2, MOPS_V3(S) grad_W_2,    \
        MOPS_V2(S) grad_grad_A, MOPS_V2(S) grad_grad_B, MOPS_V2(S) grad_grad_W,                    \
        MOPS_V3(S) grad_output, MOPS_V2(S) A, MOPS_V2(S) B, MOPS_V1(S) C, MOPS_V3(S) W,            \
        MOPS_I1 indices_A, MOPS_I1 indices_W_1, MOPS_I1 indices_W_2, MOPS_I1 indices_output_1,     \
        MOPS_I1 indices_output_2

/* Four entry points per (operation, level): host/device x f32/f64. */
#define MOPS_DECLARE(name, ARGS)                                                                   \
    MOPS_EXPORT int mops_##name##_f32(ARGS(f32));                                                  \
    MOPS_EXPORT int mops_##name##_f64(ARGS(f64));                                                  \
    MOPS_EXPORT int mops_cuda_##name##_f32(ARGS(f32));                                             \
    MOPS_EXPORT int mops_cuda_##name##_f64(ARGS(f64));

#define MOPS_FOR_EACH_ENTRY(X)                                                                     \
    X(homogeneous_polynomial_evaluation, MOPS_ARGS_HPE)                                            \
    X(homogeneous_polynomial_evaluation_vjp, MOPS_ARGS_HPE_VJP)                                    \
    X(homogeneous_polynomial_evaluation_vjp_vjp, MOPS_ARGS_HPE_VJP_VJP)                            \
    X(sparse_accumulation_of_products, MOPS_ARGS_SAP)                                              \
    X(sparse_accumulation_of_products_vjp, MOPS_ARGS_SAP_VJP)                                      \
    X(sparse_accumulation_of_products_vjp_vjp, MOPS_ARGS_SAP_VJP_VJP)                              \
    X(outer_product_scatter_add, MOPS_ARGS_OPSA)                                                   \
    X(outer_product_scatter_add_vjp, MOPS_ARGS_OPSA_VJP)                                           \
    X(outer_product_scatter_add_vjp_vjp, MOPS_ARGS_OPSA_VJP_VJP)                                   \
    X(outer_product_scatter_add_with_weights, MOPS_ARGS_OPSAW)                                     \
    X(outer_product_scatter_add_with_weights_vjp, MOPS_ARGS_OPSAW_VJP)                             \
    X(outer_product_scatter_add_with_weights_vjp_vjp, MOPS_ARGS_OPSAW_VJP_VJP)                     \
    X(sparse_accumulation_scatter_add_with_weights, MOPS_ARGS_SASAW)                               \
    X(sparse_accumulation_scatter_add_with_weights_vjp, MOPS_ARGS_SASAW_VJP)                       \
    X(sparse_accumulation_scatter_add_with_weights_vjp_vjp, MOPS_ARGS_SASAW_VJP_VJP)

MOPS_FOR_EACH_ENTRY(MOPS_DECLARE)

/* Message of the last error on the calling thread; valid until that thread's next failing
 * call. (mops/include/mops.h:16) */
MOPS_EXPORT const char* mops_get_last_error_message(void);

/* ---- Extensions of this build (no counterpart in the reference ABI) ------------------- */

/* CUDA stream (a cudaStream_t) on which the calling thread's mops_cuda_* calls run.
 * NULL selects the legacy default stream, which is what the reference uses. */
MOPS_EXPORT void mops_b200_set_stream(void* stream);
MOPS_EXPORT void* mops_b200_get_stream(void);

/* wait != 0 (default): mops_cuda_* return when results are complete, as in the reference.
 * wait == 0: they return after enqueueing on the stream; index errors found by the kernels
 * are then not reported by that call. Per thread. */
MOPS_EXPORT void mops_b200_set_wait(int wait);
MOPS_EXPORT int mops_b200_get_wait(void);
/* Concurrency: any number of threads may call at the same time. The few status words through
 * which the kernels report unsorted or out-of-range indices are kept per (calling thread,
 * device, stream): calls that one thread issues on one stream run in order and share them
 * safely; calls on different streams, which may overlap on the GPU when wait == 0, each have
 * their own. Do not hand one thread's stream to mops_b200_set_stream of another thread while
 * asynchronous calls of both are in flight on it unless the application orders them itself. */

/* ---- Plans: device tables built once and reused (no counterpart in the reference, which
 * rebuilds its first-occurrence table on every call, mops/src/internal/
 * cuda_first_occurences.cu:82-117, and has no caller-visible object for it).
 * Every operation first turns its index (and coefficient) arrays into a device table: the
 * segment offsets of a scatter index (indices_output of OPSA / OPSAW, indices_output_1 of
 * SASAW), HPE's packed monomial records, SAP's sorted triplets, SASAW's grouped coupling
 * table. While a plan is bound to the calling thread, each such table is built by the first
 * mops_cuda_* call that needs it and kept in the plan; later calls whose index arrays have
 * the same device addresses and sizes reuse it. The forward and the VJP of one graph then
 * share one segment table, no table is rebuilt, and calls with a sorted scatter index no
 * longer wait for the device in mid-call to learn that it is sorted.
 * Contract: while a plan holds tables derived from an array, the caller must not change that
 * array's contents (or free it and reuse the address for other data); destroy the plan, or
 * use a new one, when the graph changes. An unsorted scatter index, or one with out-of-range
 * values, is not kept: such calls behave as without a plan. The call that builds a table
 * waits for the stream once. Plans may be bound in several threads at the same time.
 * mops_b200_plan_create / _destroy return 0 on success, 1 on error. */
typedef struct mops_b200_plan mops_b200_plan_t;
MOPS_EXPORT int mops_b200_plan_create(mops_b200_plan_t** plan);
MOPS_EXPORT int mops_b200_plan_destroy(mops_b200_plan_t* plan);
/* Binds `plan` to the calling thread (NULL unbinds). */
MOPS_EXPORT void mops_b200_plan_bind(mops_b200_plan_t* plan);
MOPS_EXPORT mops_b200_plan_t* mops_b200_plan_bound(void);
/* Number of tables the plan currently holds. */
MOPS_EXPORT int mops_b200_plan_tables(const mops_b200_plan_t* plan);

/* Stable sort of a scatter index on the device (no counterpart in the reference, whose callers
 * sort on the host before the call, python/mops/tests/opsa.py:96): on return sorted[i] =
 * indices[permutation[i]] is ascending and entries with equal values keep their input order.
 * All three are device arrays of the same length (< 2^31); values must lie in [0, n_rows).
 * Apply `permutation` to the rows of A, B (and indices_W) to obtain the sorted problem the
 * scatter operations run fastest on; applied to indices_W / indices_W_1 it groups the grad_W
 * contributions by row of W. Same status convention, stream and completion rules as the
 * mops_cuda_* entry points. */
MOPS_EXPORT int mops_b200_cuda_sort_index(mops_tensor_1d_i32_t sorted,
                                          mops_tensor_1d_i32_t permutation,
                                          mops_tensor_1d_i32_t indices, int64_t n_rows);

/* Names (with template arguments) of the main kernels the calling thread's last mops_cuda_*
 * call dispatched to, "; "-separated; valid until that thread's next call. For tools that
 * pair a timing with the profile of the same kernel instantiation. */
MOPS_EXPORT const char* mops_b200_last_kernels(void);

/* SASAW forward for callers that cannot allocate device memory at the time they call: a
 * host program whose own pool has reserved the whole device, where a cudaMalloc made by a
 * library fails or fragments that pool, and latency-critical loops, where a driver
 * allocation may block or synchronise the device.
 * No counterpart in the reference. Same arguments, result and status convention as
 * mops_cuda_sparse_accumulation_scatter_add_with_weights_f64, but its internal scratch (the
 * grouped coupling table and the status words) is a fixed array inside the library instead
 * of call-scoped allocations: it calls no cudaMalloc/cudaFree or other allocating routine.
 * Limits: C.shape[0] <= 4096 coupling entries and output.shape[1] * W.shape[1] <= 1024;
 * beyond that it returns 1 with a message. All calls share the one array per GPU (held until
 * the process exits, about 100 KB), so calls whose GPU work overlaps race: serialise them.
 * The first call on each device looks up the array's address and must be made outside any
 * stream capture; the first launch of each kernel may also make the driver load its code.
 * Runs on the thread's stream (mops_b200_set_stream) and returns when done. */
MOPS_EXPORT int mops_b200_cuda_sparse_accumulation_scatter_add_with_weights_noalloc_f64(
    MOPS_ARGS_SASAW(f64));

/* Version string of this build. */
MOPS_EXPORT const char* mops_b200_version(void);

#ifdef __cplusplus
}
#endif

#endif
