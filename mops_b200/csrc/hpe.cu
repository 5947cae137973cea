// Homogeneous polynomial evaluation: forward and VJP, f32 and f64, for sm_100a.
//
//   O[i]     = sum_j C[j] prod_k A[i, P[j,k]]                              (hpe.hpp:10-27)
//   gA[i,n] += gO[i] C[j] prod_{l != k} A[i, P[j,l]]   for every (j,k) with P[j,k] = n
//
// Replaces mops/src/hpe/hpe.cu, which runs one block per batch row, so that every block
// re-reads the whole monomial table, and gathers factors with conflicting shared-memory
// reads and shared-memory atomics.
//
// Here the batch dimension is the parallel one. A block takes 32 consecutive rows of A,
// loads them with coalesced reads and keeps them transposed in shared memory ([factor][row],
// padded), so that "factor P[j,k] of my row" is a conflict-free read at a warp-uniform
// offset: lane = row. Monomials are warp-uniform; their indices and coefficients come
// through L1 as broadcasts. Forward: the block's warps split the monomials and add their
// partial sums at the end. VJP: each lane owns its row of the gradient tile in shared
// memory, so the scatter into gA needs no atomics; the K leave-one-out products are built
// from running prefix and suffix products (2K multiplications instead of K^2).
#include "checks.hpp"
#include "device.cuh"

namespace mops_b200 {
namespace {

constexpr int kRows = 32;       // batch rows per block (one per lane)
constexpr int kPad = kRows + 1; // shared-memory row stride of a transposed tile
constexpr int kFwdWarps = 4;
constexpr int kMaxOrder = 10;

// Loads rows [i0, i0+32) of a row-major [I][N] matrix into tile[n*kPad + row].
template <typename T>
__device__ __forceinline__ void load_tile_transposed(T* tile, const T* __restrict__ M, int64_t i0,
                                                     int64_t I, int N, int tid, int nthreads) {
    const int64_t rows = I - i0 < kRows ? I - i0 : kRows;
    const int total = kRows * N;
    const int64_t valid = rows * N;
    const T* src = M + i0 * N;
    for (int idx = tid; idx < total; idx += nthreads) {
        const int row = idx / N, n = idx - row * N;
        tile[n * kPad + row] = idx < valid ? src[idx] : T(0);
    }
}

template <typename T, int K>
__global__ void __launch_bounds__(kFwdWarps * 32)
hpe_fwd_tile(T* __restrict__ O, const T* __restrict__ A, const T* __restrict__ C,
             const int32_t* __restrict__ P, int64_t I, int N, int64_t J, Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* At = reinterpret_cast<T*>(smem_raw); // [N][kPad]
    T* partial = At + static_cast<size_t>(N) * kPad; // [kFwdWarps][32]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * kRows;
    const bool reporter = blockIdx.x == 0;

    load_tile_transposed(At, A, i0, I, N, tid, kFwdWarps * 32);
    __syncthreads();

    const T* col = At + lane;
    T acc = T(0);
#pragma unroll 4
    for (int64_t j = warp; j < J; j += kFwdWarps) {
        T prod = __ldg(C + j);
#pragma unroll
        for (int k = 0; k < K; k++) {
            int32_t p = __ldg(P + j * K + k);
            if (clamp_index(p, N) && reporter && lane == 0) report_bad_index(st, 0);
            prod *= col[p * kPad];
        }
        acc += prod;
    }
    partial[warp * 32 + lane] = acc;
    __syncthreads();
    if (warp == 0 && i0 + lane < I) {
        T sum = partial[lane];
#pragma unroll
        for (int w = 1; w < kFwdWarps; w++) sum += partial[w * 32 + lane];
        O[i0 + lane] = sum;
    }
}

template <typename T, int K>
__global__ void __launch_bounds__(32)
hpe_vjp_tile(T* __restrict__ gA, const T* __restrict__ gO, const T* __restrict__ A,
             const T* __restrict__ C, const int32_t* __restrict__ P, int64_t I, int N, int64_t J,
             Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* At = reinterpret_cast<T*>(smem_raw);          // [N][kPad]
    T* Gt = At + static_cast<size_t>(N) * kPad;      // [N][kPad]
    const int lane = threadIdx.x;
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * kRows;
    const bool reporter = blockIdx.x == 0;

    load_tile_transposed(At, A, i0, I, N, lane, 32);
    for (int idx = lane; idx < N * kPad; idx += 32) Gt[idx] = T(0);
    __syncwarp();

    const T go = i0 + lane < I ? gO[i0 + lane] : T(0);
    const T* a_col = At + lane;
    T* g_col = Gt + lane;
    for (int64_t j = 0; j < J; j++) {
        int32_t p[K > 0 ? K : 1];
        T a[K > 0 ? K : 1];
#pragma unroll
        for (int k = 0; k < K; k++) {
            p[k] = __ldg(P + j * K + k);
            if (clamp_index(p[k], N) && reporter && lane == 0) report_bad_index(st, 0);
            a[k] = a_col[p[k] * kPad];
        }
        // suffix[k] = prod_{l > k} a[l]
        T suffix[K > 0 ? K : 1];
        if constexpr (K > 0) suffix[K - 1] = T(1);
#pragma unroll
        for (int k = K - 2; k >= 0; k--) suffix[k] = suffix[k + 1] * a[k + 1];
        T prefix = __ldg(C + j) * go; // times prod_{l < k} a[l]
#pragma unroll
        for (int k = 0; k < K; k++) {
            g_col[p[k] * kPad] += prefix * suffix[k];
            prefix *= a[k];
        }
    }
    __syncwarp();

    const int64_t rows = I - i0 < kRows ? I - i0 : kRows;
    const int64_t valid = rows * N;
    T* dst = gA + i0 * N;
    for (int idx = lane; idx < kRows * N; idx += 32) {
        const int row = idx / N, n = idx - row * N;
        if (idx < valid) dst[idx] = Gt[n * kPad + row];
    }
}

// Any N: one thread per row, factors straight from global memory. Used when a 32-row tile of
// A (and, for the VJP, of gA) does not fit in shared memory.
template <typename T>
__global__ void hpe_fwd_wide(T* __restrict__ O, const T* __restrict__ A, const T* __restrict__ C,
                             const int32_t* __restrict__ P, int64_t I, int N, int64_t J, int K,
                             Status st) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= I) return;
    const T* a = A + i * N;
    T acc = T(0);
    for (int64_t j = 0; j < J; j++) {
        T prod = __ldg(C + j);
        for (int k = 0; k < K; k++) {
            int32_t p = __ldg(P + j * K + k);
            if (clamp_index(p, N) && i == 0) report_bad_index(st, 0);
            prod *= a[p];
        }
        acc += prod;
    }
    O[i] = acc;
}

template <typename T>
__global__ void hpe_vjp_wide(T* __restrict__ gA, const T* __restrict__ gO,
                             const T* __restrict__ A, const T* __restrict__ C,
                             const int32_t* __restrict__ P, int64_t I, int N, int64_t J, int K,
                             Status st) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= I) return;
    const T* a = A + i * N;
    T* g = gA + i * N;
    for (int n = 0; n < N; n++) g[n] = T(0);
    const T go = gO[i];
    for (int64_t j = 0; j < J; j++) {
        const T base = __ldg(C + j) * go;
        for (int k = 0; k < K; k++) {
            T term = base;
            for (int l = 0; l < K; l++) {
                if (l == k) continue;
                int32_t p = __ldg(P + j * K + l);
                clamp_index(p, N);
                term *= a[p];
            }
            int32_t p = __ldg(P + j * K + k);
            if (clamp_index(p, N) && i == 0) report_bad_index(st, 0);
            g[p] += term;
        }
    }
}

template <typename T, int K>
void launch_fwd(const Call& call, size_t smem, T* O, const T* A, const T* C, const int32_t* P,
                int64_t I, int N, int64_t J) {
    auto kernel = hpe_fwd_tile<T, K>;
    if (smem > 48 * 1024)
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
    kernel<<<static_cast<unsigned>(ceil_div(I, kRows)), kFwdWarps * 32, smem, call.stream>>>(
        O, A, C, P, I, N, J, call.status);
}

template <typename T, int K>
void launch_vjp(const Call& call, size_t smem, T* gA, const T* gO, const T* A, const T* C,
                const int32_t* P, int64_t I, int N, int64_t J) {
    auto kernel = hpe_vjp_tile<T, K>;
    if (smem > 48 * 1024)
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
    kernel<<<static_cast<unsigned>(ceil_div(I, kRows)), 32, smem, call.stream>>>(
        gA, gO, A, C, P, I, N, J, call.status);
}

#define MOPS_B200_ORDER_SWITCH(K, CALL)                                                            \
    switch (K) {                                                                                   \
    case 0: CALL(0); break;                                                                        \
    case 1: CALL(1); break;                                                                        \
    case 2: CALL(2); break;                                                                        \
    case 3: CALL(3); break;                                                                        \
    case 4: CALL(4); break;                                                                        \
    case 5: CALL(5); break;                                                                        \
    case 6: CALL(6); break;                                                                        \
    case 7: CALL(7); break;                                                                        \
    case 8: CALL(8); break;                                                                        \
    case 9: CALL(9); break;                                                                        \
    default: CALL(10); break;                                                                      \
    }

const char* const kIndexNames[] = {"indices_A"};

void check_order(size_t K) {
    // Same limit and text as the reference CPU code (mops/src/hpe/cpu.tpp:129); the reference
    // CUDA launcher silently does nothing for larger orders (mops/src/hpe/hpe.cu:183-185).
    if (K > static_cast<size_t>(kMaxOrder)) {
        throw std::runtime_error("Only up to polynomial order 10 is supported at the moment. "
                                 "Please contact the developers for more");
    }
}

} // namespace
} // namespace mops_b200

using namespace mops_b200;

template <typename scalar_t>
void mops::cuda::homogeneous_polynomial_evaluation(Tensor<scalar_t, 1> output,
                                                   Tensor<scalar_t, 2> A, Tensor<scalar_t, 1> C,
                                                   Tensor<int32_t, 2> indices_A) {
    const std::string op = "cuda_homogeneous_polynomial_evaluation";
    // The reference names `output` "grad_output" in this message (checks/hpe.hpp:16).
    same_size(A, "A", 0, output, "grad_output", 0, op);
    same_size(C, "C", 0, indices_A, "indices_A", 0, op);
    check_order(indices_A.shape[1]);
    fits_int32(A.shape[1], "A.shape[1]", op);
    const int64_t I = static_cast<int64_t>(A.shape[0]), J = static_cast<int64_t>(C.shape[0]);
    const int N = static_cast<int>(A.shape[1]), K = static_cast<int>(indices_A.shape[1]);
    if (I == 0) return;
    Call call = begin_call();
    if (N == 0 && K > 0) {
        // No factor to gather: with J > 0 every index is out of range; with J == 0 the sum is empty.
        if (J > 0)
            throw std::runtime_error("Index array indices_A in operation " + op +
                                     " refers to columns of an A that has none");
        MOPS_CUDA_OK(cudaMemsetAsync(output.data, 0, I * sizeof(scalar_t), call.stream));
        end_call(call, op.c_str(), kIndexNames, 1);
        return;
    }
    const size_t smem = (static_cast<size_t>(N) * kPad + kFwdWarps * 32) * sizeof(scalar_t);
    if (smem <= static_cast<size_t>(max_optin_smem(call.device))) {
#define CALL(KK)                                                                                   \
    launch_fwd<scalar_t, KK>(call, smem, output.data, A.data, C.data, indices_A.data, I, N, J)
        MOPS_B200_ORDER_SWITCH(K, CALL)
#undef CALL
    } else {
        hpe_fwd_wide<scalar_t><<<static_cast<unsigned>(ceil_div(I, 128)), 128, 0, call.stream>>>(
            output.data, A.data, C.data, indices_A.data, I, N, J, K, call.status);
    }
    end_call(call, op.c_str(), kIndexNames, 1);
}

template <typename scalar_t>
void mops::cuda::homogeneous_polynomial_evaluation_vjp(Tensor<scalar_t, 2> grad_A,
                                                       Tensor<scalar_t, 1> grad_output,
                                                       Tensor<scalar_t, 2> A,
                                                       Tensor<scalar_t, 1> C,
                                                       Tensor<int32_t, 2> indices_A) {
    const std::string op = "cuda_homogeneous_polynomial_evaluation_vjp";
    grad_like(grad_A, "grad_A", A, "A", op);
    same_size(A, "A", 0, grad_output, "grad_output", 0, op);
    same_size(C, "C", 0, indices_A, "indices_A", 0, op);
    check_order(indices_A.shape[1]);
    fits_int32(A.shape[1], "A.shape[1]", op);
    if (grad_A.data == nullptr) return;
    const int64_t I = static_cast<int64_t>(A.shape[0]), J = static_cast<int64_t>(C.shape[0]);
    const int N = static_cast<int>(A.shape[1]), K = static_cast<int>(indices_A.shape[1]);
    if (I == 0 || N == 0) return;
    Call call = begin_call();
    const size_t smem = 2 * static_cast<size_t>(N) * kPad * sizeof(scalar_t);
    if (smem <= static_cast<size_t>(max_optin_smem(call.device))) {
#define CALL(KK)                                                                                   \
    launch_vjp<scalar_t, KK>(call, smem, grad_A.data, grad_output.data, A.data, C.data,            \
                             indices_A.data, I, N, J)
        MOPS_B200_ORDER_SWITCH(K, CALL)
#undef CALL
    } else {
        hpe_vjp_wide<scalar_t><<<static_cast<unsigned>(ceil_div(I, 128)), 128, 0, call.stream>>>(
            grad_A.data, grad_output.data, A.data, C.data, indices_A.data, I, N, J, K,
            call.status);
    }
    end_call(call, op.c_str(), kIndexNames, 1);
}

template <typename scalar_t>
void mops::cuda::homogeneous_polynomial_evaluation_vjp_vjp(
    Tensor<scalar_t, 1>, Tensor<scalar_t, 2>, Tensor<scalar_t, 2>, Tensor<scalar_t, 1>,
    Tensor<scalar_t, 2>, Tensor<scalar_t, 1>, Tensor<int32_t, 2>) {
    // Same behaviour as the reference CUDA build (mops/src/hpe/hpe.cu:402-413).
    throw std::runtime_error("Not implemented");
}

#define INSTANTIATE(T)                                                                             \
    template void mops::cuda::homogeneous_polynomial_evaluation<T>(                               \
        mops::Tensor<T, 1>, mops::Tensor<T, 2>, mops::Tensor<T, 1>, mops::Tensor<int32_t, 2>);    \
    template void mops::cuda::homogeneous_polynomial_evaluation_vjp<T>(                           \
        mops::Tensor<T, 2>, mops::Tensor<T, 1>, mops::Tensor<T, 2>, mops::Tensor<T, 1>,           \
        mops::Tensor<int32_t, 2>);                                                                \
    template void mops::cuda::homogeneous_polynomial_evaluation_vjp_vjp<T>(                       \
        mops::Tensor<T, 1>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 1>,           \
        mops::Tensor<T, 2>, mops::Tensor<T, 1>, mops::Tensor<int32_t, 2>);

INSTANTIATE(float)
INSTANTIATE(double)
