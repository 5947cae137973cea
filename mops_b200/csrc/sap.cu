// Sparse accumulation of products: forward, VJP and second-order VJP, f32 and f64, sm_100a.
//
//   O[i, PO[k]]  += C[k] A[i,PA[k]] B[i,PB[k]]                             (sap.hpp:10-42)
//   gA[i, PA[k]] += gO[i,PO[k]] C[k] B[i,PB[k]];  gB[i, PB[k]] += gO[i,PO[k]] C[k] A[i,PA[k]]
//   ggO[i,PO_k]  += C_k (ggA[i,PA_k] B[i,PB_k] + ggB[i,PB_k] A[i,PA_k])
//   gA2[i,PA_k]  += C_k ggB[i,PB_k] gO[i,PO_k];   gB2[i,PB_k] += C_k ggA[i,PA_k] gO[i,PO_k]
//
// Replaces mops/src/sap/sap.cu: 32 rows per block with strided (uncoalesced) tile loads, one
// shared-memory atomic per (row, triplet), and the three indices of a triplet packed into 8
// bits each, which silently breaks for any dimension above 255.
//
// Here the batch dimension is the parallel one: lane = row. A block loads its rows of every
// operand with coalesced reads and keeps them transposed in shared memory ([column][row],
// padded), so that each triplet's operands are conflict-free reads at warp-uniform offsets,
// and each lane owns its row of every output tile: the scatter needs no atomics at all.
// Consecutive triplets with the same output column (indices_output is usually sorted) are
// summed in a register and flushed once. Outputs go back with coalesced stores. Indices are
// plain int32, any size.
#include "checks.hpp"
#include "device.cuh"

namespace mops_b200 {
namespace {

// A transposed operand tile in shared memory: element (row, col) at data[col * stride + row].
template <typename T> struct Tile {
    T* data;
    int cols;
};

template <typename T>
__device__ __forceinline__ void tile_load(Tile<T> t, const T* __restrict__ M, int64_t i0, int64_t I,
                                          int R, int stride) {
    const int64_t rows = I - i0 < R ? I - i0 : R;
    const int64_t valid = rows * t.cols;
    const int total = R * t.cols;
    const T* src = M == nullptr ? nullptr : M + i0 * t.cols;
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int row = idx / t.cols, c = idx - row * t.cols;
        t.data[c * stride + row] = (src != nullptr && idx < valid) ? src[idx] : T(0);
    }
}

template <typename T>
__device__ __forceinline__ void tile_store(Tile<T> t, T* __restrict__ M, int64_t i0, int64_t I,
                                           int R, int stride) {
    if (M == nullptr) return;
    const int64_t rows = I - i0 < R ? I - i0 : R;
    const int64_t valid = rows * t.cols;
    T* dst = M + i0 * t.cols;
    for (int idx = threadIdx.x; idx < valid; idx += blockDim.x) {
        const int row = idx / t.cols, c = idx - row * t.cols;
        dst[idx] = t.data[c * stride + row];
    }
}

struct Triplet {
    int32_t pa, pb, po;
};

// Reads triplet k (warp-uniform), clamping bad indices; block 0 reports them.
__device__ __forceinline__ Triplet read_triplet(const int32_t* __restrict__ PA,
                                                const int32_t* __restrict__ PB,
                                                const int32_t* __restrict__ PO, int64_t k, int nA,
                                                int nB, int nO, const Status& st) {
    Triplet t{__ldg(PA + k), __ldg(PB + k), __ldg(PO + k)};
    const bool ba = clamp_index(t.pa, nA), bb = clamp_index(t.pb, nB), bo = clamp_index(t.po, nO);
    if ((ba || bb || bo) && blockIdx.x == 0 && threadIdx.x == 0) {
        if (ba) report_bad_index(st, 0);
        if (bb) report_bad_index(st, 1);
        if (bo) report_bad_index(st, 2);
    }
    return t;
}

template <typename T>
__global__ void sap_fwd_tile(T* __restrict__ O, const T* __restrict__ A, const T* __restrict__ B,
                             const T* __restrict__ C, const int32_t* __restrict__ PA,
                             const int32_t* __restrict__ PB, const int32_t* __restrict__ PO,
                             int64_t I, int nA, int nB, int nO, int64_t K, Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = blockDim.x, S = R + 1, tid = threadIdx.x;
    Tile<T> At{reinterpret_cast<T*>(smem_raw), nA};
    Tile<T> Bt{At.data + static_cast<size_t>(nA) * S, nB};
    Tile<T> Ot{Bt.data + static_cast<size_t>(nB) * S, nO};
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * R;

    tile_load(At, A, i0, I, R, S);
    tile_load(Bt, B, i0, I, R, S);
    for (int idx = tid; idx < nO * S; idx += R) Ot.data[idx] = T(0);
    __syncthreads();

    const T* a = At.data + tid;
    const T* b = Bt.data + tid;
    T* o = Ot.data + tid;
    int cur = -1;
    T acc = T(0);
    for (int64_t k = 0; k < K; k++) {
        const Triplet t = read_triplet(PA, PB, PO, k, nA, nB, nO, st);
        const T v = __ldg(C + k) * a[t.pa * S] * b[t.pb * S];
        if (t.po == cur) {
            acc += v;
        } else {
            if (cur >= 0) o[cur * S] += acc;
            cur = t.po;
            acc = v;
        }
    }
    if (cur >= 0) o[cur * S] += acc;
    __syncthreads();
    tile_store(Ot, O, i0, I, R, S);
}

template <typename T>
__global__ void sap_vjp_tile(T* __restrict__ gA, T* __restrict__ gB, const T* __restrict__ gO,
                             const T* __restrict__ A, const T* __restrict__ B,
                             const T* __restrict__ C, const int32_t* __restrict__ PA,
                             const int32_t* __restrict__ PB, const int32_t* __restrict__ PO,
                             int64_t I, int nA, int nB, int nO, int64_t K, Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = blockDim.x, S = R + 1, tid = threadIdx.x;
    Tile<T> At{reinterpret_cast<T*>(smem_raw), nA};
    Tile<T> Bt{At.data + static_cast<size_t>(nA) * S, nB};
    Tile<T> Gt{Bt.data + static_cast<size_t>(nB) * S, nO};
    Tile<T> gAt{Gt.data + static_cast<size_t>(nO) * S, nA};
    Tile<T> gBt{gAt.data + static_cast<size_t>(nA) * S, nB};
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * R;

    tile_load(At, A, i0, I, R, S);
    tile_load(Bt, B, i0, I, R, S);
    tile_load(Gt, gO, i0, I, R, S);
    for (int idx = tid; idx < (nA + nB) * S; idx += R) gAt.data[idx] = T(0); // gAt and gBt are adjacent
    __syncthreads();

    const T *a = At.data + tid, *b = Bt.data + tid, *g = Gt.data + tid;
    T *ga = gAt.data + tid, *gb = gBt.data + tid;
    const bool want_a = gA != nullptr, want_b = gB != nullptr;
    for (int64_t k = 0; k < K; k++) {
        const Triplet t = read_triplet(PA, PB, PO, k, nA, nB, nO, st);
        const T gc = g[t.po * S] * __ldg(C + k);
        if (want_a) ga[t.pa * S] += gc * b[t.pb * S];
        if (want_b) gb[t.pb * S] += gc * a[t.pa * S];
    }
    __syncthreads();
    tile_store(gAt, gA, i0, I, R, S);
    tile_store(gBt, gB, i0, I, R, S);
}

template <typename T>
__global__ void sap_vjp_vjp_tile(T* __restrict__ ggO, T* __restrict__ gA2, T* __restrict__ gB2,
                                 const T* __restrict__ ggA, const T* __restrict__ ggB,
                                 const T* __restrict__ gO, const T* __restrict__ A,
                                 const T* __restrict__ B, const T* __restrict__ C,
                                 const int32_t* __restrict__ PA, const int32_t* __restrict__ PB,
                                 const int32_t* __restrict__ PO, int64_t I, int nA, int nB, int nO,
                                 int64_t K, Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = blockDim.x, S = R + 1, tid = threadIdx.x;
    T* p = reinterpret_cast<T*>(smem_raw);
    auto take = [&](int cols) {
        Tile<T> t{p, cols};
        p += static_cast<size_t>(cols) * S;
        return t;
    };
    Tile<T> At = take(nA), Bt = take(nB), Gt = take(nO), hAt = take(nA), hBt = take(nB);
    Tile<T> ggOt = take(nO), gA2t = take(nA), gB2t = take(nB); // outputs, adjacent
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * R;

    tile_load(At, A, i0, I, R, S);
    tile_load(Bt, B, i0, I, R, S);
    tile_load(Gt, gO, i0, I, R, S);
    tile_load(hAt, ggA, i0, I, R, S); // a missing second-order input reads as zeros
    tile_load(hBt, ggB, i0, I, R, S);
    for (int idx = tid; idx < (nO + nA + nB) * S; idx += R) ggOt.data[idx] = T(0);
    __syncthreads();

    const T *a = At.data + tid, *b = Bt.data + tid, *g = Gt.data + tid;
    const T *ha = hAt.data + tid, *hb = hBt.data + tid;
    T *o = ggOt.data + tid, *oa = gA2t.data + tid, *ob = gB2t.data + tid;
    const bool have_a = ggA != nullptr, have_b = ggB != nullptr;
    for (int64_t k = 0; k < K; k++) {
        const Triplet t = read_triplet(PA, PB, PO, k, nA, nB, nO, st);
        const T c = __ldg(C + k);
        const T go = g[t.po * S];
        if (have_a) {
            const T h = ha[t.pa * S];
            o[t.po * S] += h * b[t.pb * S] * c;
            ob[t.pb * S] += h * go * c;
        }
        if (have_b) {
            const T h = hb[t.pb * S];
            o[t.po * S] += h * a[t.pa * S] * c;
            oa[t.pa * S] += h * go * c;
        }
    }
    __syncthreads();
    tile_store(ggOt, ggO, i0, I, R, S);
    tile_store(gA2t, gA2, i0, I, R, S);
    tile_store(gB2t, gB2, i0, I, R, S);
}

// Any width: one thread per row working directly on its rows in global memory. Used when the
// tiles of 32 rows do not fit in shared memory.
template <typename T>
__global__ void sap_wide(int level, T* __restrict__ out0, T* __restrict__ out1,
                         T* __restrict__ out2, const T* __restrict__ ggA,
                         const T* __restrict__ ggB, const T* __restrict__ gO,
                         const T* __restrict__ A, const T* __restrict__ B, const T* __restrict__ C,
                         const int32_t* __restrict__ PA, const int32_t* __restrict__ PB,
                         const int32_t* __restrict__ PO, int64_t I, int nA, int nB, int nO,
                         int64_t K, Status st) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= I) return;
    // level 0: out0 = O.  level 1: out0 = gA, out1 = gB.  level 2: out0 = ggO, out1 = gA2, out2 = gB2.
    T* o_row = level == 1 ? nullptr : (out0 ? out0 + i * nO : nullptr);
    T* a_row = level == 1 ? (out0 ? out0 + i * nA : nullptr) : (level == 2 && out1 ? out1 + i * nA : nullptr);
    T* b_row = level == 1 ? (out1 ? out1 + i * nB : nullptr) : (level == 2 && out2 ? out2 + i * nB : nullptr);
    if (o_row) for (int n = 0; n < nO; n++) o_row[n] = T(0);
    if (a_row) for (int n = 0; n < nA; n++) a_row[n] = T(0);
    if (b_row) for (int n = 0; n < nB; n++) b_row[n] = T(0);
    for (int64_t k = 0; k < K; k++) {
        Triplet t{__ldg(PA + k), __ldg(PB + k), __ldg(PO + k)};
        const bool ba = clamp_index(t.pa, nA), bb = clamp_index(t.pb, nB), bo = clamp_index(t.po, nO);
        if (i == 0) {
            if (ba) report_bad_index(st, 0);
            if (bb) report_bad_index(st, 1);
            if (bo) report_bad_index(st, 2);
        }
        const T c = __ldg(C + k), a = A[i * nA + t.pa], b = B[i * nB + t.pb];
        if (level == 0) {
            o_row[t.po] += c * a * b;
        } else if (level == 1) {
            const T gc = gO[i * nO + t.po] * c;
            if (a_row) a_row[t.pa] += gc * b;
            if (b_row) b_row[t.pb] += gc * a;
        } else {
            const T go = gO[i * nO + t.po];
            if (ggA) {
                const T h = ggA[i * nA + t.pa];
                if (o_row) o_row[t.po] += h * b * c;
                if (b_row) b_row[t.pb] += h * go * c;
            }
            if (ggB) {
                const T h = ggB[i * nB + t.pb];
                if (o_row) o_row[t.po] += h * a * c;
                if (a_row) a_row[t.pa] += h * go * c;
            }
        }
    }
}

// Rows per block: the largest of 128/64/32 whose tiles stay under ~100 KB (so that at least
// two blocks share an SM); 0 if not even 32 rows fit in the opt-in limit.
template <typename T> int rows_per_block(const Call& call, int cols, size_t* smem) {
    for (int R : {128, 64, 32}) {
        const size_t bytes = static_cast<size_t>(cols) * (R + 1) * sizeof(T);
        const size_t limit = R == 32 ? static_cast<size_t>(max_optin_smem(call.device)) : 100 * 1024;
        if (bytes <= limit) {
            *smem = bytes;
            return R;
        }
    }
    return 0;
}

template <typename Kernel> void allow_smem(Kernel kernel, size_t smem) {
    if (smem > 48 * 1024)
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
}

const char* const kIndexNames[] = {"indices_A", "indices_B", "indices_output"};

template <typename scalar_t>
void check_sap_shapes(const mops::Tensor<scalar_t, 2>& output, const mops::Tensor<scalar_t, 2>& A,
                      const mops::Tensor<scalar_t, 2>& B, const mops::Tensor<scalar_t, 1>& C,
                      const mops::Tensor<int32_t, 1>& indices_A,
                      const mops::Tensor<int32_t, 1>& indices_B,
                      const mops::Tensor<int32_t, 1>& indices_output, const std::string& op) {
    same_size(A, "A", 0, B, "B", 0, op);
    same_size(A, "A", 0, output, "output", 0, op);
    same_size(C, "C", 0, indices_A, "indices_A", 0, op);
    same_size(C, "C", 0, indices_B, "indices_B", 0, op);
    same_size(C, "C", 0, indices_output, "indices_output", 0, op);
    fits_int32(A.shape[1], "A.shape[1]", op);
    fits_int32(B.shape[1], "B.shape[1]", op);
    fits_int32(output.shape[1], "output.shape[1]", op);
}

} // namespace
} // namespace mops_b200

using namespace mops_b200;

template <typename scalar_t>
void mops::cuda::sparse_accumulation_of_products(Tensor<scalar_t, 2> output, Tensor<scalar_t, 2> A,
                                                 Tensor<scalar_t, 2> B, Tensor<scalar_t, 1> C,
                                                 Tensor<int32_t, 1> indices_A,
                                                 Tensor<int32_t, 1> indices_B,
                                                 Tensor<int32_t, 1> indices_output) {
    const std::string op = "cuda_sparse_accumulation_of_products";
    check_sap_shapes(output, A, B, C, indices_A, indices_B, indices_output, op);
    const int64_t I = static_cast<int64_t>(A.shape[0]), K = static_cast<int64_t>(C.shape[0]);
    const int nA = static_cast<int>(A.shape[1]), nB = static_cast<int>(B.shape[1]);
    const int nO = static_cast<int>(output.shape[1]);
    if (I == 0 || nO == 0) return;
    Call call = begin_call();
    if (K == 0 || nA == 0 || nB == 0) {
        if (K > 0)
            throw std::runtime_error("Index arrays in operation " + op +
                                     " refer to columns of an operand that has none");
        MOPS_CUDA_OK(cudaMemsetAsync(output.data, 0, I * nO * sizeof(scalar_t), call.stream));
        end_call(call, op.c_str(), kIndexNames, 3);
        return;
    }
    size_t smem = 0;
    const int R = rows_per_block<scalar_t>(call, nA + nB + nO, &smem);
    if (R > 0) {
        allow_smem(sap_fwd_tile<scalar_t>, smem);
        sap_fwd_tile<scalar_t><<<static_cast<unsigned>(ceil_div(I, R)), R, smem, call.stream>>>(
            output.data, A.data, B.data, C.data, indices_A.data, indices_B.data,
            indices_output.data, I, nA, nB, nO, K, call.status);
    } else {
        sap_wide<scalar_t><<<static_cast<unsigned>(ceil_div(I, 128)), 128, 0, call.stream>>>(
            0, output.data, nullptr, nullptr, nullptr, nullptr, nullptr, A.data, B.data, C.data,
            indices_A.data, indices_B.data, indices_output.data, I, nA, nB, nO, K, call.status);
    }
    end_call(call, op.c_str(), kIndexNames, 3);
}

template <typename scalar_t>
void mops::cuda::sparse_accumulation_of_products_vjp(
    Tensor<scalar_t, 2> grad_A, Tensor<scalar_t, 2> grad_B, Tensor<scalar_t, 2> grad_output,
    Tensor<scalar_t, 2> A, Tensor<scalar_t, 2> B, Tensor<scalar_t, 1> C,
    Tensor<int32_t, 1> indices_A, Tensor<int32_t, 1> indices_B,
    Tensor<int32_t, 1> indices_output) {
    const std::string op = "cuda_sparse_accumulation_of_products_vjp";
    grad_like(grad_A, "grad_A", A, "A", op);
    grad_like(grad_B, "grad_B", B, "B", op);
    check_sap_shapes(grad_output, A, B, C, indices_A, indices_B, indices_output, op);
    if (grad_A.data == nullptr && grad_B.data == nullptr) return;
    const int64_t I = static_cast<int64_t>(A.shape[0]), K = static_cast<int64_t>(C.shape[0]);
    const int nA = static_cast<int>(A.shape[1]), nB = static_cast<int>(B.shape[1]);
    const int nO = static_cast<int>(grad_output.shape[1]);
    if (I == 0) return;
    Call call = begin_call();
    if (K == 0 || nA == 0 || nB == 0 || nO == 0) {
        if (K > 0)
            throw std::runtime_error("Index arrays in operation " + op +
                                     " refer to columns of an operand that has none");
        if (grad_A.data != nullptr && nA > 0)
            MOPS_CUDA_OK(cudaMemsetAsync(grad_A.data, 0, I * nA * sizeof(scalar_t), call.stream));
        if (grad_B.data != nullptr && nB > 0)
            MOPS_CUDA_OK(cudaMemsetAsync(grad_B.data, 0, I * nB * sizeof(scalar_t), call.stream));
        end_call(call, op.c_str(), kIndexNames, 3);
        return;
    }
    size_t smem = 0;
    const int R = rows_per_block<scalar_t>(call, 2 * nA + 2 * nB + nO, &smem);
    if (R > 0) {
        allow_smem(sap_vjp_tile<scalar_t>, smem);
        sap_vjp_tile<scalar_t><<<static_cast<unsigned>(ceil_div(I, R)), R, smem, call.stream>>>(
            grad_A.data, grad_B.data, grad_output.data, A.data, B.data, C.data, indices_A.data,
            indices_B.data, indices_output.data, I, nA, nB, nO, K, call.status);
    } else {
        sap_wide<scalar_t><<<static_cast<unsigned>(ceil_div(I, 128)), 128, 0, call.stream>>>(
            1, grad_A.data, grad_B.data, nullptr, nullptr, nullptr, grad_output.data, A.data,
            B.data, C.data, indices_A.data, indices_B.data, indices_output.data, I, nA, nB, nO, K,
            call.status);
    }
    end_call(call, op.c_str(), kIndexNames, 3);
}

template <typename scalar_t>
void mops::cuda::sparse_accumulation_of_products_vjp_vjp(
    Tensor<scalar_t, 2> grad_grad_output, Tensor<scalar_t, 2> grad_A_2,
    Tensor<scalar_t, 2> grad_B_2, Tensor<scalar_t, 2> grad_grad_A,
    Tensor<scalar_t, 2> grad_grad_B, Tensor<scalar_t, 2> grad_output, Tensor<scalar_t, 2> A,
    Tensor<scalar_t, 2> B, Tensor<scalar_t, 1> C, Tensor<int32_t, 1> indices_A,
    Tensor<int32_t, 1> indices_B, Tensor<int32_t, 1> indices_output) {
    const std::string op = "cuda_sparse_accumulation_of_products_vjp_vjp";
    grad_like(grad_grad_output, "grad_grad_output", grad_output, "grad_output", op);
    grad_like(grad_A_2, "grad_A_2", A, "A", op);
    grad_like(grad_B_2, "grad_B_2", B, "B", op);
    grad_like(grad_grad_A, "grad_grad_A", A, "A", op);
    grad_like(grad_grad_B, "grad_grad_B", B, "B", op);
    check_sap_shapes(grad_output, A, B, C, indices_A, indices_B, indices_output, op);
    if (grad_grad_output.data == nullptr && grad_A_2.data == nullptr && grad_B_2.data == nullptr)
        return;
    const int64_t I = static_cast<int64_t>(A.shape[0]), K = static_cast<int64_t>(C.shape[0]);
    const int nA = static_cast<int>(A.shape[1]), nB = static_cast<int>(B.shape[1]);
    const int nO = static_cast<int>(grad_output.shape[1]);
    if (I == 0) return;
    Call call = begin_call();
    if (K == 0 || nA == 0 || nB == 0 || nO == 0) {
        if (K > 0)
            throw std::runtime_error("Index arrays in operation " + op +
                                     " refer to columns of an operand that has none");
        if (grad_grad_output.data != nullptr && nO > 0)
            MOPS_CUDA_OK(cudaMemsetAsync(grad_grad_output.data, 0, I * nO * sizeof(scalar_t),
                                         call.stream));
        if (grad_A_2.data != nullptr && nA > 0)
            MOPS_CUDA_OK(cudaMemsetAsync(grad_A_2.data, 0, I * nA * sizeof(scalar_t), call.stream));
        if (grad_B_2.data != nullptr && nB > 0)
            MOPS_CUDA_OK(cudaMemsetAsync(grad_B_2.data, 0, I * nB * sizeof(scalar_t), call.stream));
        end_call(call, op.c_str(), kIndexNames, 3);
        return;
    }
    size_t smem = 0;
    const int R = rows_per_block<scalar_t>(call, 3 * nA + 3 * nB + 2 * nO, &smem);
    if (R > 0) {
        allow_smem(sap_vjp_vjp_tile<scalar_t>, smem);
        sap_vjp_vjp_tile<scalar_t>
            <<<static_cast<unsigned>(ceil_div(I, R)), R, smem, call.stream>>>(
                grad_grad_output.data, grad_A_2.data, grad_B_2.data, grad_grad_A.data,
                grad_grad_B.data, grad_output.data, A.data, B.data, C.data, indices_A.data,
                indices_B.data, indices_output.data, I, nA, nB, nO, K, call.status);
    } else {
        sap_wide<scalar_t><<<static_cast<unsigned>(ceil_div(I, 128)), 128, 0, call.stream>>>(
            2, grad_grad_output.data, grad_A_2.data, grad_B_2.data, grad_grad_A.data,
            grad_grad_B.data, grad_output.data, A.data, B.data, C.data, indices_A.data,
            indices_B.data, indices_output.data, I, nA, nB, nO, K, call.status);
    }
    end_call(call, op.c_str(), kIndexNames, 3);
}

#define INSTANTIATE(T)                                                                             \
    template void mops::cuda::sparse_accumulation_of_products<T>(                                 \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 1>,           \
        mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>);            \
    template void mops::cuda::sparse_accumulation_of_products_vjp<T>(                             \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>,           \
        mops::Tensor<T, 2>, mops::Tensor<T, 1>, mops::Tensor<int32_t, 1>,                         \
        mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>);                                      \
    template void mops::cuda::sparse_accumulation_of_products_vjp_vjp<T>(                         \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>,           \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>,           \
        mops::Tensor<T, 1>, mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>,                   \
        mops::Tensor<int32_t, 1>);

INSTANTIATE(float)
INSTANTIATE(double)
