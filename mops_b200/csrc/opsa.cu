// Outer-product scatter-add, without (OPSA) and with (OPSAW) per-row weights: forward and
// VJP, f32 and f64, for sm_100a.
//
//   OPSA   O[P[j],k,l]  = sum_j A[j,k] B[j,l]                       (opsa.hpp:10-38)
//          gA[j,k] = sum_l gO[P[j],k,l] B[j,l];  gB[j,l] = sum_k gO[P[j],k,l] A[j,k]
//   OPSAW  O[PO[e],k,l] = sum_e A[e,k] B[e,l] W[PW[e],l]            (opsaw.hpp:10-39)
//          S[e,l] = sum_k gO[PO[e],k,l] A[e,k]
//          gA[e,k] = sum_l gO[PO[e],k,l] B[e,l] W[PW[e],l]
//          gB[e,l] = S[e,l] W[PW[e],l];  gW[PW[e],l] += S[e,l] B[e,l]
//
// These replace mops/src/opsa/opsa.cu (one 128-thread block per output row reading A and B
// from global memory once per (k, l-chunk); a warp-per-entry VJP with K serial shuffle
// reductions) and the OPSAW stubs that throw (mops/src/opsaw/cuda.tpp:5-49).
//
// Forward: a segmented reduction over the sorted scatter index. One warp owns one output
// row; it finds the row's entry range with a 32-way search (device.cuh), streams the
// contiguous A and B slices of that range through shared memory in coalesced chunks, keeps
// a TK x TL tile of the K x L result per lane in registers and writes the row once. No
// atomics, no zero-fill pass, empty rows are written as zeros by their warp. If the index
// turns out not to be sorted (the reference CPU code accepts that), the same call falls
// back to a zero-fill plus global-atomic kernel, so the result is right either way.
//
// VJP: entry-parallel, one lane per entry, so it does not depend on the index order. A block
// stages its entries' A and B rows in shared memory with coalesced loads, each lane keeps its
// A row and the gA accumulators in registers and walks over l; gO rows come through L1 as
// warp-wide broadcasts because neighbouring entries share an output row. Results are
// staged back in place and written with coalesced stores; gW is accumulated with RED.
#include <algorithm>

#include "checks.hpp"
#include "device.cuh"

namespace mops_b200 {
namespace {

constexpr int kFwdWarps = 8;
constexpr int kMaxTK = 8;

template <typename T, int N> struct VecOf;
template <> struct VecOf<float, 1> { using type = float; };
template <> struct VecOf<float, 2> { using type = float2; };
template <> struct VecOf<float, 4> { using type = float4; };
template <> struct VecOf<double, 1> { using type = double; };
template <> struct VecOf<double, 2> { using type = double2; };

template <typename T, int N> __device__ __forceinline__ void load_vec(const T* p, T (&out)[N]) {
    using V = typename VecOf<T, N>::type;
    union {
        V v;
        T s[N];
    } u;
    u.v = *reinterpret_cast<const V*>(p);
#pragma unroll
    for (int i = 0; i < N; i++) out[i] = u.s[i];
}

template <typename T, int N> __device__ __forceinline__ void store_vec(T* p, const T (&in)[N]) {
    using V = typename VecOf<T, N>::type;
    union {
        V v;
        T s[N];
    } u;
#pragma unroll
    for (int i = 0; i < N; i++) u.s[i] = in[i];
    *reinterpret_cast<V*>(p) = u.v;
}

// ------------------------------------------------------------------------------ forward
struct FwdPlan {
    int TK, TL; // register tile per lane
    int LL, LK; // lane grid: LL lanes along l, LK along k (LL*LK <= 32)
    int CH;     // entries staged per chunk
    size_t smem_per_warp;
};

template <typename T, int TK, int TL, bool WEIGHTED>
__global__ void __launch_bounds__(kFwdWarps * 32)
opsa_fwd_segmented(T* __restrict__ O, const T* __restrict__ A, const T* __restrict__ B,
                   const T* __restrict__ W, const int32_t* __restrict__ PW,
                   const int32_t* __restrict__ P, int64_t J, int K, int L, int64_t nO,
                   FwdPlan plan, Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * kFwdWarps + warp;

    check_sorted_slice(P, J, nO, r, static_cast<int64_t>(gridDim.x) * kFwdWarps, lane, st);
    if (r >= nO) return;

    const int CH = plan.CH;
    T* Bs = reinterpret_cast<T*>(smem_raw + warp * plan.smem_per_warp); // [CH][L], 16-byte aligned
    T* As = Bs + static_cast<size_t>(CH) * L;                            // [CH][K]

    int64_t begin, end;
    warp_segment(P, J, static_cast<int32_t>(r), lane, begin, end);

    const int ll = lane % plan.LL, lk = lane / plan.LL;
    const bool active = lk < plan.LK;
    T* Orow = O + r * K * L;

    for (int kb = 0; kb < K; kb += plan.LK * TK) {
        for (int lb = 0; lb < L; lb += plan.LL * TL) {
            const int k0 = kb + lk * TK, l0 = lb + ll * TL;
            T acc[TK][TL];
#pragma unroll
            for (int t = 0; t < TK; t++)
#pragma unroll
                for (int u = 0; u < TL; u++) acc[t][u] = T(0);

            for (int64_t c0 = begin; c0 < end; c0 += CH) {
                const int n = static_cast<int>(end - c0 < CH ? end - c0 : CH);
                __syncwarp();
                if (WEIGHTED) {
                    for (int jj = 0; jj < n; jj++) {
                        int32_t pw = __ldg(PW + c0 + jj);
                        if (clamp_index(pw, static_cast<int32_t>(nO)) && lane == 0)
                            report_bad_index(st, 1);
                        const T* b = B + (c0 + jj) * L;
                        const T* w = W + static_cast<int64_t>(pw) * L;
                        for (int l = lane; l < L; l += 32) Bs[jj * L + l] = b[l] * __ldg(w + l);
                    }
                } else {
                    const T* b = B + c0 * L;
                    for (int idx = lane; idx < n * L; idx += 32) Bs[idx] = b[idx];
                }
                {
                    const T* a = A + c0 * K;
                    for (int idx = lane; idx < n * K; idx += 32) As[idx] = a[idx];
                }
                __syncwarp();
                if (active && l0 < L) {
                    for (int jj = 0; jj < n; jj++) {
                        T a[TK], b[TL];
#pragma unroll
                        for (int t = 0; t < TK; t++)
                            a[t] = (k0 + t < K) ? As[jj * K + k0 + t] : T(0);
                        if (TL > 1) {
                            load_vec<T, TL>(Bs + jj * L + l0, b);
                        } else {
                            b[0] = Bs[jj * L + l0];
                        }
#pragma unroll
                        for (int t = 0; t < TK; t++)
#pragma unroll
                            for (int u = 0; u < TL; u++) acc[t][u] += a[t] * b[u];
                    }
                }
            }
            if (active && l0 < L) {
#pragma unroll
                for (int t = 0; t < TK; t++) {
                    if (k0 + t < K) {
#pragma unroll
                        for (int u = 0; u < TL; u++) Orow[(k0 + t) * L + l0 + u] = acc[t][u];
                    }
                }
            }
        }
    }
}

template <typename T, bool WEIGHTED>
__global__ void opsa_fwd_atomic(T* __restrict__ O, const T* __restrict__ A,
                                const T* __restrict__ B, const T* __restrict__ W,
                                const int32_t* __restrict__ PW, const int32_t* __restrict__ P,
                                int64_t J, int K, int L, int64_t nO, bool always, Status st) {
    if (!always && !saw_unsorted(st)) return;
    const int64_t KL = static_cast<int64_t>(K) * L;
    const int64_t total = J * KL;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t j = i / KL;
        const int x = static_cast<int>(i - j * KL);
        const int k = x / L, l = x - k * L;
        int32_t row = __ldg(P + j);
        if (clamp_index(row, static_cast<int32_t>(nO))) {
            report_bad_index(st, 0);
            continue;
        }
        T v = A[j * K + k] * B[j * L + l];
        if (WEIGHTED) {
            int32_t pw = __ldg(PW + j);
            if (clamp_index(pw, static_cast<int32_t>(nO))) {
                report_bad_index(st, 1);
                continue;
            }
            v *= __ldg(W + static_cast<int64_t>(pw) * L + l);
        }
        red_add(O + row * KL + x, v);
    }
}

template <typename T> FwdPlan plan_forward(int K, int L, bool l_aligned) {
    FwdPlan p;
    const int widest = 16 / static_cast<int>(sizeof(T));
    p.TL = 1;
    if (l_aligned) {
        for (int tl = widest; tl > 1; tl /= 2) {
            if (L % tl == 0) {
                p.TL = tl;
                break;
            }
        }
    }
    p.LL = static_cast<int>(std::min<int64_t>(32, ceil_div(L, p.TL)));
    p.LK = 32 / p.LL;
    if (p.LK > K) p.LK = K;
    p.TK = static_cast<int>(std::min<int64_t>(kMaxTK, ceil_div(K, p.LK)));
    p.CH = 32;
    const size_t row_bytes = static_cast<size_t>(K + L) * sizeof(T);
    while (p.CH > 1 && p.CH * row_bytes > 12 * 1024) p.CH /= 2;
    p.smem_per_warp = (p.CH * row_bytes + 15) / 16 * 16;
    return p;
}

template <typename T, int TK, int TL, bool WEIGHTED>
void launch_fwd_tile(const Call& call, const FwdPlan& plan, T* O, const T* A, const T* B,
                     const T* W, const int32_t* PW, const int32_t* P, int64_t J, int K, int L,
                     int64_t nO) {
    auto kernel = opsa_fwd_segmented<T, TK, TL, WEIGHTED>;
    const size_t smem = plan.smem_per_warp * kFwdWarps;
    if (smem > 48 * 1024) {
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
    }
    const int64_t blocks = ceil_div(nO, kFwdWarps);
    kernel<<<static_cast<unsigned>(blocks), kFwdWarps * 32, smem, call.stream>>>(
        O, A, B, W, PW, P, J, K, L, nO, plan, call.status);
}

template <typename T, int TL, bool WEIGHTED, typename... Args>
void dispatch_tk(int TK, Args... args) {
    switch (TK) {
    case 1: launch_fwd_tile<T, 1, TL, WEIGHTED>(args...); break;
    case 2: launch_fwd_tile<T, 2, TL, WEIGHTED>(args...); break;
    case 3: launch_fwd_tile<T, 3, TL, WEIGHTED>(args...); break;
    case 4: launch_fwd_tile<T, 4, TL, WEIGHTED>(args...); break;
    case 5: launch_fwd_tile<T, 5, TL, WEIGHTED>(args...); break;
    case 6: launch_fwd_tile<T, 6, TL, WEIGHTED>(args...); break;
    case 7: launch_fwd_tile<T, 7, TL, WEIGHTED>(args...); break;
    default: launch_fwd_tile<T, 8, TL, WEIGHTED>(args...); break;
    }
}

template <typename T, bool WEIGHTED>
void forward(const Call& call, T* O, const T* A, const T* B, const T* W, const int32_t* PW,
             const int32_t* P, int64_t J, int K, int L, int64_t nO) {
    const int64_t KL = static_cast<int64_t>(K) * L;
    if (nO == 0 || KL == 0) return;
    if (J == 0) {
        MOPS_CUDA_OK(cudaMemsetAsync(O, 0, nO * KL * sizeof(T), call.stream));
        return;
    }
    const bool aligned = reinterpret_cast<uintptr_t>(O) % 16 == 0;
    FwdPlan plan = plan_forward<T>(K, L, aligned);
    const size_t smem = plan.smem_per_warp * kFwdWarps;
    const bool segmented = smem <= static_cast<size_t>(max_optin_smem(call.device));
    const int grid_generic = sm_count(call.device) * 8;

    if (segmented) {
        if constexpr (sizeof(T) == 8) {
            if (plan.TL == 2)
                dispatch_tk<T, 2, WEIGHTED>(plan.TK, call, plan, O, A, B, W, PW, P, J, K, L, nO);
            else
                dispatch_tk<T, 1, WEIGHTED>(plan.TK, call, plan, O, A, B, W, PW, P, J, K, L, nO);
        } else {
            if (plan.TL == 4)
                dispatch_tk<T, 4, WEIGHTED>(plan.TK, call, plan, O, A, B, W, PW, P, J, K, L, nO);
            else if (plan.TL == 2)
                dispatch_tk<T, 2, WEIGHTED>(plan.TK, call, plan, O, A, B, W, PW, P, J, K, L, nO);
            else
                dispatch_tk<T, 1, WEIGHTED>(plan.TK, call, plan, O, A, B, W, PW, P, J, K, L, nO);
        }
        MOPS_CUDA_OK(cudaGetLastError());
        bool need_fallback = true; // asynchronous calls cannot look: always enqueue
        if (call.wait) {
            wait_stream(call);
            need_fallback = host_saw_unsorted(call);
        }
        if (need_fallback) {
            zero_if_unsorted<T><<<grid_generic, 256, 0, call.stream>>>(O, nO * KL, call.status);
            opsa_fwd_atomic<T, WEIGHTED><<<grid_generic, 256, 0, call.stream>>>(
                O, A, B, W, PW, P, J, K, L, nO, false, call.status);
        }
    } else {
        // Rows too wide for the staged kernel: zero-fill and accumulate with atomics.
        MOPS_CUDA_OK(cudaMemsetAsync(O, 0, nO * KL * sizeof(T), call.stream));
        opsa_fwd_atomic<T, WEIGHTED><<<grid_generic, 256, 0, call.stream>>>(
            O, A, B, W, PW, P, J, K, L, nO, true, call.status);
    }
    MOPS_CUDA_OK(cudaGetLastError());
}

// ---------------------------------------------------------------------------------- VJP
struct VjpPlan {
    int Kp, Lp; // shared-memory row strides (odd: conflict-free row-per-lane access)
    int nkc;    // number of KP-wide chunks of K
    int threads;
    size_t smem;
};

template <typename T, int KP, int VL, bool WEIGHTED>
__global__ void __launch_bounds__(128)
opsa_vjp_entries(T* __restrict__ gA, T* __restrict__ gB, T* __restrict__ gW,
                 const T* __restrict__ gO, const T* __restrict__ A, const T* __restrict__ B,
                 const T* __restrict__ W, const int32_t* __restrict__ PW,
                 const int32_t* __restrict__ P, int64_t J, int K, int L, int64_t nO,
                 VjpPlan plan, Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, EPB = blockDim.x;
    const int Kp = plan.Kp, Lp = plan.Lp, nkc = plan.nkc;
    T* As = reinterpret_cast<T*>(smem_raw);              // [EPB][Kp]  A rows, then gA rows
    T* Bs = As + static_cast<size_t>(EPB) * Kp;          // [EPB][Lp]  B rows, then gB rows
    T* Ws = Bs + static_cast<size_t>(EPB) * Lp;          // [EPB][Lp]  W rows, then gW terms
    T* Ss = WEIGHTED ? Ws + static_cast<size_t>(EPB) * Lp : Ws; // [EPB][Lp] S, only if nkc > 1

    const int64_t base = static_cast<int64_t>(blockIdx.x) * EPB;
    const int n = static_cast<int>(J - base < EPB ? J - base : EPB);

    for (int idx = tid; idx < n * K; idx += EPB) {
        const int jj = idx / K, k = idx - jj * K;
        As[jj * Kp + k] = A[base * K + idx];
    }
    for (int idx = tid; idx < n * L; idx += EPB) {
        const int jj = idx / L, l = idx - jj * L;
        Bs[jj * Lp + l] = B[base * L + idx];
        if (WEIGHTED) {
            int32_t pw = __ldg(PW + base + jj);
            if (clamp_index(pw, static_cast<int32_t>(nO))) report_bad_index(st, 1);
            Ws[jj * Lp + l] = __ldg(W + static_cast<int64_t>(pw) * L + l);
        }
    }
    __syncthreads();

    if (tid < n) {
        int32_t row = __ldg(P + base + tid);
        if (clamp_index(row, static_cast<int32_t>(nO))) report_bad_index(st, 0);
        const T* g = gO + static_cast<int64_t>(row) * K * L;
        T* a_row = As + tid * Kp;
        T* b_row = Bs + tid * Lp;
        T* w_row = Ws + tid * Lp;
        T* s_row = Ss + tid * Lp;

        for (int kc = 0; kc < nkc; kc++) {
            const int kbase = kc * KP;
            T a[KP], ga[KP];
#pragma unroll
            for (int t = 0; t < KP; t++) {
                a[t] = (kbase + t < K) ? a_row[kbase + t] : T(0);
                ga[t] = T(0);
            }
            for (int l0 = 0; l0 < L; l0 += VL) {
                T b[VL], w[VL], bw[VL], s[VL];
#pragma unroll
                for (int u = 0; u < VL; u++) {
                    b[u] = b_row[l0 + u];
                    w[u] = WEIGHTED ? w_row[l0 + u] : T(1);
                    bw[u] = WEIGHTED ? b[u] * w[u] : b[u];
                    s[u] = T(0);
                }
#pragma unroll
                for (int t = 0; t < KP; t++) {
                    if (kbase + t < K) {
                        T gv[VL];
                        if (VL > 1) {
                            load_vec<T, VL>(g + static_cast<int64_t>(kbase + t) * L + l0, gv);
                        } else {
                            gv[0] = __ldg(g + static_cast<int64_t>(kbase + t) * L + l0);
                        }
#pragma unroll
                        for (int u = 0; u < VL; u++) {
                            ga[t] += gv[u] * bw[u];
                            s[u] += gv[u] * a[t];
                        }
                    }
                }
                if (nkc == 1) {
#pragma unroll
                    for (int u = 0; u < VL; u++) {
                        b_row[l0 + u] = WEIGHTED ? s[u] * w[u] : s[u];
                        if (WEIGHTED) w_row[l0 + u] = s[u] * b[u];
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < VL; u++) {
                        if (kc == 0)
                            s_row[l0 + u] = s[u];
                        else
                            s_row[l0 + u] += s[u];
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < KP; t++)
                if (kbase + t < K) a_row[kbase + t] = ga[t];
        }
        if (nkc > 1) {
            for (int l = 0; l < L; l++) {
                const T s = s_row[l], b = b_row[l];
                if (WEIGHTED) {
                    const T w = w_row[l];
                    b_row[l] = s * w;
                    w_row[l] = s * b;
                } else {
                    b_row[l] = s;
                }
            }
        }
    }
    __syncthreads();

    if (gA != nullptr) {
        for (int idx = tid; idx < n * K; idx += EPB) {
            const int jj = idx / K, k = idx - jj * K;
            gA[base * K + idx] = As[jj * Kp + k];
        }
    }
    if (gB != nullptr || (WEIGHTED && gW != nullptr)) {
        for (int idx = tid; idx < n * L; idx += EPB) {
            const int jj = idx / L, l = idx - jj * L;
            if (gB != nullptr) gB[base * L + idx] = Bs[jj * Lp + l];
            if (WEIGHTED && gW != nullptr) {
                int32_t pw = __ldg(PW + base + jj);
                if (!clamp_index(pw, static_cast<int32_t>(nO)))
                    red_add(gW + static_cast<int64_t>(pw) * L + l, Ws[jj * Lp + l]);
            }
        }
    }
}

// Any K and L: one thread per gradient element, straight from global memory.
template <typename T, bool WEIGHTED>
__global__ void opsa_vjp_wide(T* __restrict__ gA, T* __restrict__ gB, T* __restrict__ gW,
                              const T* __restrict__ gO, const T* __restrict__ A,
                              const T* __restrict__ B, const T* __restrict__ W,
                              const int32_t* __restrict__ PW, const int32_t* __restrict__ P,
                              int64_t J, int K, int L, int64_t nO, Status st) {
    const int64_t per = static_cast<int64_t>(K) + L;
    const int64_t total = J * per;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t j = i / per;
        const int c = static_cast<int>(i - j * per);
        int32_t row = __ldg(P + j);
        if (clamp_index(row, static_cast<int32_t>(nO))) report_bad_index(st, 0);
        int32_t pw = 0;
        if (WEIGHTED) {
            pw = __ldg(PW + j);
            if (clamp_index(pw, static_cast<int32_t>(nO))) report_bad_index(st, 1);
        }
        const T* g = gO + static_cast<int64_t>(row) * K * L;
        const T* w = WEIGHTED ? W + static_cast<int64_t>(pw) * L : nullptr;
        if (c < K) {
            if (gA == nullptr) continue;
            T s = T(0);
            for (int l = 0; l < L; l++) {
                T bw = B[j * L + l];
                if (WEIGHTED) bw *= w[l];
                s += g[static_cast<int64_t>(c) * L + l] * bw;
            }
            gA[j * K + c] = s;
        } else {
            const int l = c - K;
            T s = T(0);
            for (int k = 0; k < K; k++) s += g[static_cast<int64_t>(k) * L + l] * A[j * K + k];
            if (gB != nullptr) gB[j * L + l] = WEIGHTED ? s * w[l] : s;
            if (WEIGHTED && gW != nullptr)
                red_add(gW + static_cast<int64_t>(pw) * L + l, s * B[j * L + l]);
        }
    }
}

template <typename T, int KP, int VL, bool WEIGHTED, typename... Args>
void launch_vjp_tile(const Call& call, const VjpPlan& plan, int64_t J, Args... args) {
    auto kernel = opsa_vjp_entries<T, KP, VL, WEIGHTED>;
    if (plan.smem > 48 * 1024) {
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(plan.smem)));
    }
    const int64_t blocks = ceil_div(J, plan.threads);
    kernel<<<static_cast<unsigned>(blocks), plan.threads, plan.smem, call.stream>>>(args..., plan,
                                                                                   call.status);
}

template <typename T, int VL, bool WEIGHTED, typename... Args>
void dispatch_kp(int K, Args... args) {
    if (K <= 4)
        launch_vjp_tile<T, 4, VL, WEIGHTED>(args...);
    else if (K <= 8)
        launch_vjp_tile<T, 8, VL, WEIGHTED>(args...);
    else
        launch_vjp_tile<T, 16, VL, WEIGHTED>(args...);
}

template <typename T, bool WEIGHTED>
void backward(const Call& call, T* gA, T* gB, T* gW, const T* gO, const T* A, const T* B,
              const T* W, const int32_t* PW, const int32_t* P, int64_t J, int K, int L,
              int64_t nO) {
    if (gA == nullptr && gB == nullptr && gW == nullptr) return;
    if (WEIGHTED && gW != nullptr && nO * L > 0)
        MOPS_CUDA_OK(cudaMemsetAsync(gW, 0, nO * static_cast<int64_t>(L) * sizeof(T), call.stream));
    if (J == 0 || (K == 0 && L == 0)) return;
    if (K == 0 || L == 0) {
        // One of the factors is empty: every requested gradient is zero.
        if (gA != nullptr && K > 0)
            MOPS_CUDA_OK(cudaMemsetAsync(gA, 0, J * K * sizeof(T), call.stream));
        if (gB != nullptr && L > 0)
            MOPS_CUDA_OK(cudaMemsetAsync(gB, 0, J * L * sizeof(T), call.stream));
        return;
    }

    VjpPlan plan;
    const int KP = K <= 4 ? 4 : (K <= 8 ? 8 : 16);
    plan.nkc = static_cast<int>(ceil_div(K, KP));
    plan.Kp = K | 1;
    plan.Lp = L | 1;
    const int tiles_l = 1 + (WEIGHTED ? 1 : 0) + (plan.nkc > 1 ? 1 : 0);
    const size_t per_entry = (plan.Kp + static_cast<size_t>(tiles_l) * plan.Lp) * sizeof(T);
    plan.threads = 128;
    while (plan.threads > 32 && plan.threads * per_entry > 96 * 1024) plan.threads /= 2;
    plan.smem = plan.threads * per_entry;

    const int widest = 16 / static_cast<int>(sizeof(T));
    int VL = 1;
    for (int v = widest; v > 1; v /= 2) {
        if (L % v == 0 && reinterpret_cast<uintptr_t>(gO) % (v * sizeof(T)) == 0) {
            VL = v;
            break;
        }
    }

    if (plan.smem <= static_cast<size_t>(max_optin_smem(call.device))) {
        if constexpr (sizeof(T) == 8) {
            if (VL == 2)
                dispatch_kp<T, 2, WEIGHTED>(K, call, plan, J, gA, gB, gW, gO, A, B, W, PW, P, J, K,
                                            L, nO);
            else
                dispatch_kp<T, 1, WEIGHTED>(K, call, plan, J, gA, gB, gW, gO, A, B, W, PW, P, J, K,
                                            L, nO);
        } else {
            if (VL == 4)
                dispatch_kp<T, 4, WEIGHTED>(K, call, plan, J, gA, gB, gW, gO, A, B, W, PW, P, J, K,
                                            L, nO);
            else if (VL == 2)
                dispatch_kp<T, 2, WEIGHTED>(K, call, plan, J, gA, gB, gW, gO, A, B, W, PW, P, J, K,
                                            L, nO);
            else
                dispatch_kp<T, 1, WEIGHTED>(K, call, plan, J, gA, gB, gW, gO, A, B, W, PW, P, J, K,
                                            L, nO);
        }
    } else {
        opsa_vjp_wide<T, WEIGHTED><<<sm_count(call.device) * 8, 256, 0, call.stream>>>(
            gA, gB, gW, gO, A, B, W, PW, P, J, K, L, nO, call.status);
    }
    MOPS_CUDA_OK(cudaGetLastError());
}

const char* const kOpsaIndexNames[] = {"indices_output"};
const char* const kOpsawIndexNames[] = {"indices_output", "indices_W"};

} // namespace
} // namespace mops_b200

// ------------------------------------------------------------------------------ public API
using namespace mops_b200;

template <typename scalar_t>
void mops::cuda::outer_product_scatter_add(Tensor<scalar_t, 3> output, Tensor<scalar_t, 2> A,
                                           Tensor<scalar_t, 2> B,
                                           Tensor<int32_t, 1> indices_output) {
    const std::string op = "cuda_outer_product_scatter_add";
    same_size(A, "A", 0, B, "B", 0, op);
    same_size(A, "A", 1, output, "output", 1, op);
    same_size(B, "B", 1, output, "output", 2, op);
    same_size(A, "A", 0, indices_output, "indices_output", 0, op);
    fits_int32(output.shape[0], "output.shape[0]", op);
    fits_int32(A.shape[1], "A.shape[1]", op);
    fits_int32(B.shape[1], "B.shape[1]", op);
    Call call = begin_call();
    forward<scalar_t, false>(call, output.data, A.data, B.data, nullptr, nullptr,
                             indices_output.data, static_cast<int64_t>(A.shape[0]),
                             static_cast<int>(A.shape[1]), static_cast<int>(B.shape[1]),
                             static_cast<int64_t>(output.shape[0]));
    end_call(call, op.c_str(), kOpsaIndexNames, 1);
}

template <typename scalar_t>
void mops::cuda::outer_product_scatter_add_vjp(Tensor<scalar_t, 2> grad_A,
                                               Tensor<scalar_t, 2> grad_B,
                                               Tensor<scalar_t, 3> grad_output,
                                               Tensor<scalar_t, 2> A, Tensor<scalar_t, 2> B,
                                               Tensor<int32_t, 1> indices_output) {
    const std::string op = "cuda_outer_product_scatter_add_vjp";
    grad_like(grad_A, "grad_A", A, "A", op);
    grad_like(grad_B, "grad_B", B, "B", op);
    same_size(A, "A", 0, B, "B", 0, op);
    same_size(A, "A", 1, grad_output, "output", 1, op);
    same_size(B, "B", 1, grad_output, "output", 2, op);
    same_size(A, "A", 0, indices_output, "indices_output", 0, op);
    fits_int32(grad_output.shape[0], "grad_output.shape[0]", op);
    fits_int32(A.shape[1], "A.shape[1]", op);
    fits_int32(B.shape[1], "B.shape[1]", op);
    Call call = begin_call();
    backward<scalar_t, false>(call, grad_A.data, grad_B.data, nullptr, grad_output.data, A.data,
                              B.data, nullptr, nullptr, indices_output.data,
                              static_cast<int64_t>(A.shape[0]), static_cast<int>(A.shape[1]),
                              static_cast<int>(B.shape[1]),
                              static_cast<int64_t>(grad_output.shape[0]));
    end_call(call, op.c_str(), kOpsaIndexNames, 1);
}

template <typename scalar_t>
void mops::cuda::outer_product_scatter_add_vjp_vjp(
    Tensor<scalar_t, 3>, Tensor<scalar_t, 2>, Tensor<scalar_t, 2>, Tensor<scalar_t, 2>,
    Tensor<scalar_t, 2>, Tensor<scalar_t, 3>, Tensor<scalar_t, 2>, Tensor<scalar_t, 2>,
    Tensor<int32_t, 1>) {
    // Same behaviour as the reference CUDA build (mops/src/opsa/opsa.cu:305-318).
    throw std::runtime_error("Not implemented");
}

template <typename scalar_t>
static void check_opsaw_shapes(const mops::Tensor<scalar_t, 3>& output,
                               const mops::Tensor<scalar_t, 2>& A,
                               const mops::Tensor<scalar_t, 2>& B,
                               const mops::Tensor<scalar_t, 2>& W,
                               const mops::Tensor<int32_t, 1>& indices_W,
                               const mops::Tensor<int32_t, 1>& indices_output,
                               const std::string& op) {
    same_size(A, "A", 0, B, "B", 0, op);
    same_size(A, "A", 1, output, "output", 1, op);
    same_size(B, "B", 1, output, "output", 2, op);
    same_size(A, "A", 0, indices_output, "indices_output", 0, op);
    same_size(A, "A", 0, indices_W, "indices_W", 0, op);
    same_size(W, "W", 0, output, "output", 0, op);
    same_size(B, "B", 1, W, "W", 1, op);
    fits_int32(output.shape[0], "output.shape[0]", op);
    fits_int32(A.shape[1], "A.shape[1]", op);
    fits_int32(B.shape[1], "B.shape[1]", op);
}

template <typename scalar_t>
void mops::cuda::outer_product_scatter_add_with_weights(
    Tensor<scalar_t, 3> output, Tensor<scalar_t, 2> A, Tensor<scalar_t, 2> B,
    Tensor<scalar_t, 2> W, Tensor<int32_t, 1> indices_W, Tensor<int32_t, 1> indices_output) {
    const std::string op = "cuda_outer_product_scatter_add_with_weights";
    check_opsaw_shapes(output, A, B, W, indices_W, indices_output, op);
    Call call = begin_call();
    forward<scalar_t, true>(call, output.data, A.data, B.data, W.data, indices_W.data,
                            indices_output.data, static_cast<int64_t>(A.shape[0]),
                            static_cast<int>(A.shape[1]), static_cast<int>(B.shape[1]),
                            static_cast<int64_t>(output.shape[0]));
    end_call(call, op.c_str(), kOpsawIndexNames, 2);
}

template <typename scalar_t>
void mops::cuda::outer_product_scatter_add_with_weights_vjp(
    Tensor<scalar_t, 2> grad_A, Tensor<scalar_t, 2> grad_B, Tensor<scalar_t, 2> grad_W,
    Tensor<scalar_t, 3> grad_output, Tensor<scalar_t, 2> A, Tensor<scalar_t, 2> B,
    Tensor<scalar_t, 2> W, Tensor<int32_t, 1> indices_W, Tensor<int32_t, 1> indices_output) {
    const std::string op = "cuda_outer_product_scatter_add_with_weights_vjp";
    grad_like(grad_A, "grad_A", A, "A", op);
    grad_like(grad_B, "grad_B", B, "B", op);
    grad_like(grad_W, "grad_W", W, "W", op);
    check_opsaw_shapes(grad_output, A, B, W, indices_W, indices_output, op);
    Call call = begin_call();
    backward<scalar_t, true>(call, grad_A.data, grad_B.data, grad_W.data, grad_output.data,
                             A.data, B.data, W.data, indices_W.data, indices_output.data,
                             static_cast<int64_t>(A.shape[0]), static_cast<int>(A.shape[1]),
                             static_cast<int>(B.shape[1]),
                             static_cast<int64_t>(grad_output.shape[0]));
    end_call(call, op.c_str(), kOpsawIndexNames, 2);
}

template <typename scalar_t>
void mops::cuda::outer_product_scatter_add_with_weights_vjp_vjp(
    Tensor<scalar_t, 3>, Tensor<scalar_t, 2>, Tensor<scalar_t, 2>, Tensor<scalar_t, 2>,
    Tensor<scalar_t, 2>, Tensor<scalar_t, 2>, Tensor<scalar_t, 2>, Tensor<scalar_t, 3>,
    Tensor<scalar_t, 2>, Tensor<scalar_t, 2>, Tensor<scalar_t, 2>, Tensor<int32_t, 1>,
    Tensor<int32_t, 1>) {
    // The reference has no second-order OPSAW on any device (mops/src/opsaw/cpu.tpp:149).
    throw std::runtime_error("Not implemented");
}

#define INSTANTIATE(T)                                                                             \
    template void mops::cuda::outer_product_scatter_add<T>(                                       \
        mops::Tensor<T, 3>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<int32_t, 1>);    \
    template void mops::cuda::outer_product_scatter_add_vjp<T>(                                   \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 3>, mops::Tensor<T, 2>,           \
        mops::Tensor<T, 2>, mops::Tensor<int32_t, 1>);                                            \
    template void mops::cuda::outer_product_scatter_add_vjp_vjp<T>(                               \
        mops::Tensor<T, 3>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>,           \
        mops::Tensor<T, 2>, mops::Tensor<T, 3>, mops::Tensor<T, 2>, mops::Tensor<T, 2>,           \
        mops::Tensor<int32_t, 1>);                                                                \
    template void mops::cuda::outer_product_scatter_add_with_weights<T>(                          \
        mops::Tensor<T, 3>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>,           \
        mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>);                                      \
    template void mops::cuda::outer_product_scatter_add_with_weights_vjp<T>(                      \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 3>,           \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<int32_t, 1>,     \
        mops::Tensor<int32_t, 1>);                                                                \
    template void mops::cuda::outer_product_scatter_add_with_weights_vjp_vjp<T>(                  \
        mops::Tensor<T, 3>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>,           \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 3>,           \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<int32_t, 1>,     \
        mops::Tensor<int32_t, 1>);

INSTANTIATE(float)
INSTANTIATE(double)
