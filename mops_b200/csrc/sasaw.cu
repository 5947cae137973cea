// Sparse accumulation scatter-add with weights: forward and VJP, f32 and f64, for sm_100a.
//
//   O[I[e], M3[n], b] += C[n] A[e,M1[n]] B[e,b] W[J[e], M2[n], b]          (sasaw.hpp:10-52)
//   gA[e,M1[n]]       += C[n] sum_b gO[I[e],M3[n],b] B[e,b] W[J[e],M2[n],b]
//   gB[e,b]           += sum_n C[n] A[e,M1[n]] gO[I[e],M3[n],b] W[J[e],M2[n],b]
//   gW[J[e],M2[n],b]  += C[n] A[e,M1[n]] B[e,b] gO[I[e],M3[n],b]
// (I = indices_output_1, J = indices_W_1, M1 = indices_A, M2 = indices_W_2,
//  M3 = indices_output_2.)
//
// The reference has no CUDA implementation of this operation: its entry points throw
// (mops/src/sasaw/cuda.tpp:5-61). The CPU code (mops/src/sasaw/cpu.tpp:8-171) walks all N
// coupling entries for every edge and every b.
//
// These kernels first contract the coupling table with the edge's A row:
//     T_e[m3,m2] = sum_{n : M3[n]=m3, M2[n]=m2} C[n] A[e,M1[n]]
// which does not depend on b, and then use the small dense T_e:
//     O[I_e,m3,b]  += B[e,b] sum_m2 T_e[m3,m2] W[J_e,m2,b]
//     gB[e,b]       = sum_m2 W[J_e,m2,b] sum_m3 T_e[m3,m2] gO[I_e,m3,b]
//     gW[J_e,m2,b] += B[e,b] sum_m3 T_e[m3,m2] gO[I_e,m3,b]
//     gA[e,M1[n]]  += C[n] U_e[M3[n],M2[n]],  U_e[m3,m2] = sum_b gO[I_e,m3,b] B[e,b] W[J_e,m2,b]
// For 500 coupling entries on a 9x9 grid of cells this is about seven times fewer
// multiply-adds than the direct form. A one-block kernel groups the coupling entries by cell
// once per call (counting sort, entries of a cell kept in ascending n so the sums are
// reproducible); the grouped table is call-scoped scratch memory.
//
// Forward: segmented reduction, one warp per output row (lane = b), accumulators for the row
// in shared memory, one plain store per output row; atomic fallback when the scatter index
// is not sorted. VJP: one warp per edge (lane = b), independent of the index order; gW is
// accumulated with RED because indices_W_1 is not sorted.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "checks.hpp"
#include "device.cuh"

namespace mops_b200 {
namespace {

// Index arrays in status-bit order.
const char* const kIndexNames[] = {"indices_output_1", "indices_A", "indices_W_1", "indices_W_2",
                                   "indices_output_2"};
enum { kBitI = 0, kBitM1 = 1, kBitJ = 2, kBitM2 = 3, kBitM3 = 4 };

// Coupling entries grouped by cell (m3 * nW1 + m2), in global scratch memory.
template <typename T> struct Coupling {
    T* C;           // [N]  coefficients in grouped order
    int32_t* M1;    // [N]  A column of each grouped entry
    int32_t* cell;  // [N]  cell of each grouped entry
    int32_t* start; // [ncell + 1]  first grouped position of each cell
    int32_t* order; // [N]  scratch for the sort
    int N, ncell;
    // Optional dense form for the fast kernels: D[cc][m1] = sum of C[n] over the entries of
    // compact cell cc = m3 * nW1 + m2 with M1[n] = m1; rows of d_stride scalars.
    // With d_padded the rows are numbered like the cells (m3 * cell_stride + m2) and the rows
    // of padding cells are zero.
    T* D;
    int d_stride;
    bool d_padded;
};

constexpr int kBuildThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kBuildThreads)
sasaw_group_coupling(Coupling<T> cp, const T* __restrict__ C, const int32_t* __restrict__ M1,
                     const int32_t* __restrict__ M2, const int32_t* __restrict__ M3, int nA,
                     int nW1, int nO1, Status st) {
    // cells are numbered m3 * stride + m2; stride > nW1 leaves empty padding cells
    const int cell_stride = cp.ncell / nO1;
    extern __shared__ int32_t cursor[]; // [ncell]
    __shared__ int32_t chunk_sum[kBuildThreads];
    const int tid = threadIdx.x, N = cp.N, ncell = cp.ncell;

    for (int c = tid; c < ncell; c += kBuildThreads) cursor[c] = 0;
    __syncthreads();
    for (int n = tid; n < N; n += kBuildThreads) {
        int32_t m1 = M1[n], m2 = M2[n], m3 = M3[n];
        if (clamp_index(m1, nA)) report_bad_index(st, kBitM1);
        if (clamp_index(m2, nW1)) report_bad_index(st, kBitM2);
        if (clamp_index(m3, nO1)) report_bad_index(st, kBitM3);
        atomicAdd(&cursor[m3 * cell_stride + m2], 1);
    }
    __syncthreads();
    // Exclusive scan of the per-cell counts: each thread scans a contiguous chunk.
    const int per = (ncell + kBuildThreads - 1) / kBuildThreads;
    const int c_lo = min(tid * per, ncell), c_hi = min(c_lo + per, ncell);
    int local = 0;
    for (int c = c_lo; c < c_hi; c++) local += cursor[c];
    chunk_sum[tid] = local;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int t = 0; t < kBuildThreads; t++) {
            const int v = chunk_sum[t];
            chunk_sum[t] = run;
            run += v;
        }
    }
    __syncthreads();
    int run = chunk_sum[tid];
    for (int c = c_lo; c < c_hi; c++) {
        const int v = cursor[c];
        cp.start[c] = run;
        cursor[c] = run;
        run += v;
    }
    if (tid == 0) cp.start[ncell] = N;
    __syncthreads();
    for (int n = tid; n < N; n += kBuildThreads) {
        int32_t m2 = M2[n], m3 = M3[n];
        clamp_index(m2, nW1);
        clamp_index(m3, nO1);
        cp.order[atomicAdd(&cursor[m3 * cell_stride + m2], 1)] = n;
    }
    __syncthreads();
    // Entries of one cell in ascending n (they were placed in arbitrary order).
    for (int c = tid; c < ncell; c += kBuildThreads) {
        const int lo = cp.start[c], hi = cursor[c];
        for (int i = lo + 1; i < hi; i++) {
            const int32_t v = cp.order[i];
            int j = i - 1;
            while (j >= lo && cp.order[j] > v) {
                cp.order[j + 1] = cp.order[j];
                j--;
            }
            cp.order[j + 1] = v;
        }
        for (int i = lo; i < hi; i++) cp.cell[i] = c;
    }
    __syncthreads();
    for (int pos = tid; pos < N; pos += kBuildThreads) {
        const int32_t n = cp.order[pos];
        int32_t m1 = M1[n];
        clamp_index(m1, nA);
        cp.C[pos] = C[n];
        cp.M1[pos] = m1;
    }
    if (cp.D != nullptr) {
        __syncthreads();
        // one thread per cell, entries in ascending n: reproducible sums
        for (int c = tid; c < ncell; c += kBuildThreads) {
            const int m3 = c / cell_stride, m2 = c - m3 * cell_stride;
            if (m2 >= nW1 && !cp.d_padded) continue;
            T* row = cp.D + static_cast<size_t>(cp.d_padded ? c : m3 * nW1 + m2) * cp.d_stride;
            for (int m = 0; m < cp.d_stride; m++) row[m] = T(0);
            for (int pos = cp.start[c]; pos < cp.start[c + 1]; pos++) row[cp.M1[pos]] += cp.C[pos];
        }
    }
}

// Shared-memory carve-up common to the forward and VJP kernels.
template <typename T> struct Shared {
    T* C;           // [N]
    T* warp_base;   // per-warp scalars start here
    int32_t* M1;    // [N]
    int32_t* cell;  // [N] (VJP only)
    int32_t* start; // [ncell + 1]
};

template <typename T>
__device__ __forceinline__ Shared<T> carve(unsigned char* raw, const Coupling<T>& cp,
                                           size_t per_warp_scalars, int warps, bool with_cell) {
    Shared<T> s;
    s.C = reinterpret_cast<T*>(raw);
    s.warp_base = s.C + cp.N;
    T* end = s.warp_base + per_warp_scalars * warps;
    s.M1 = reinterpret_cast<int32_t*>(end);
    s.cell = s.M1 + cp.N;
    s.start = with_cell ? s.cell + cp.N : s.cell;
    return s;
}

template <typename T>
__device__ __forceinline__ void load_coupling(const Shared<T>& s, const Coupling<T>& cp,
                                              bool with_cell) {
    for (int i = threadIdx.x; i < cp.N; i += blockDim.x) {
        s.C[i] = cp.C[i];
        s.M1[i] = cp.M1[i];
        if (with_cell) s.cell[i] = cp.cell[i];
    }
    for (int i = threadIdx.x; i <= cp.ncell; i += blockDim.x) s.start[i] = cp.start[i];
}

// T_e[cell] for one edge; a_s and T_s are this warp's buffers.
template <typename T>
__device__ __forceinline__ void contract_coupling(const Shared<T>& s, int ncell,
                                                  const T* __restrict__ a_row, int nA, T* a_s,
                                                  T* T_s, int lane) {
    __syncwarp();
    for (int m = lane; m < nA; m += 32) a_s[m] = a_row[m];
    __syncwarp();
    for (int c = lane; c < ncell; c += 32) {
        T t = T(0);
        for (int pos = s.start[c]; pos < s.start[c + 1]; pos++) t += s.C[pos] * a_s[s.M1[pos]];
        T_s[c] = t;
    }
    __syncwarp();
}

template <typename T, bool SEGMENTED>
__global__ void sasaw_fwd(T* __restrict__ O, const T* __restrict__ A, const T* __restrict__ B,
                          const T* __restrict__ W, const int32_t* __restrict__ Jw,
                          const int32_t* __restrict__ Io, Coupling<T> cp, int64_t E, int nA, int L,
                          int64_t nW0, int nW1, int nO1, bool always, Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ncell = cp.ncell;
    const size_t per_warp = static_cast<size_t>(nA) + ncell + (SEGMENTED ? static_cast<size_t>(nO1) * L : 0);
    if (!SEGMENTED && !always && !saw_unsorted(st)) return;
    Shared<T> s = carve<T>(smem_raw, cp, per_warp, warps, false);
    load_coupling(s, cp, false);
    __syncthreads();
    T* a_s = s.warp_base + per_warp * warp;
    T* T_s = a_s + nA;
    T* Oacc = T_s + ncell;
    const int64_t rowsize = static_cast<int64_t>(nO1) * L;

    auto edge = [&](int64_t e, int64_t out_row) {
        int32_t j = __ldg(Jw + e);
        if (clamp_index(j, static_cast<int32_t>(nW0)) && lane == 0) report_bad_index(st, kBitJ);
        contract_coupling(s, ncell, A + e * nA, nA, a_s, T_s, lane);
        const T* w = W + static_cast<int64_t>(j) * nW1 * L;
        for (int b = lane; b < L; b += 32) {
            const T Bb = B[e * L + b];
            for (int m3 = 0; m3 < nO1; m3++) {
                T p = T(0);
                for (int m2 = 0; m2 < nW1; m2++) {
                    const int c = m3 * nW1 + m2;
                    if (s.start[c + 1] > s.start[c]) p += T_s[c] * __ldg(w + m2 * L + b);
                }
                if (SEGMENTED)
                    Oacc[m3 * L + b] += Bb * p;
                else
                    red_add(O + out_row * rowsize + m3 * L + b, Bb * p);
            }
        }
    };

    if (SEGMENTED) {
        const int64_t r = static_cast<int64_t>(blockIdx.x) * warps + warp;
        check_sorted_slice(Io, E, nW0, r, static_cast<int64_t>(gridDim.x) * warps, lane, st);
        if (r >= nW0) return;
        int64_t begin, end;
        warp_segment(Io, E, static_cast<int32_t>(r), lane, begin, end);
        for (int idx = lane; idx < rowsize; idx += 32) Oacc[idx] = T(0);
        for (int64_t e = begin; e < end; e++) edge(e, r);
        __syncwarp();
        T* dst = O + r * rowsize;
        for (int idx = lane; idx < rowsize; idx += 32) dst[idx] = Oacc[idx];
    } else {
        const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps;
        for (int64_t e = static_cast<int64_t>(blockIdx.x) * warps + warp; e < E; e += nwarps) {
            int32_t row = __ldg(Io + e);
            if (clamp_index(row, static_cast<int32_t>(nW0))) {
                if (lane == 0) report_bad_index(st, kBitI);
                continue;
            }
            edge(e, row);
        }
    }
}

template <typename T>
__global__ void sasaw_vjp(T* __restrict__ gA, T* __restrict__ gB, T* __restrict__ gW,
                          const T* __restrict__ gO, const T* __restrict__ A,
                          const T* __restrict__ B, const T* __restrict__ W,
                          const int32_t* __restrict__ Jw, const int32_t* __restrict__ Io,
                          Coupling<T> cp, int64_t E, int nA, int L, int64_t nW0, int nW1, int nO1,
                          Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ncell = cp.ncell, N = cp.N;
    const size_t per_warp = static_cast<size_t>(nA) + 2 * static_cast<size_t>(ncell) + static_cast<size_t>(nA) * 33;
    Shared<T> s = carve<T>(smem_raw, cp, per_warp, warps, true);
    load_coupling(s, cp, true);
    __syncthreads();
    T* a_s = s.warp_base + per_warp * warp;
    T* T_s = a_s + nA;
    T* U_s = T_s + ncell;
    T* ga_priv = U_s + ncell; // [nA][33]: one private column per lane
    const int64_t rowsize = static_cast<int64_t>(nO1) * L;
    const bool want_a = gA != nullptr, want_b = gB != nullptr, want_w = gW != nullptr;

    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * warps + warp; e < E; e += nwarps) {
        int32_t row = __ldg(Io + e), j = __ldg(Jw + e);
        if (clamp_index(row, static_cast<int32_t>(nW0)) && lane == 0) report_bad_index(st, kBitI);
        if (clamp_index(j, static_cast<int32_t>(nW0)) && lane == 0) report_bad_index(st, kBitJ);
        contract_coupling(s, ncell, A + e * nA, nA, a_s, T_s, lane);
        for (int c = lane; c < ncell; c += 32) U_s[c] = T(0);
        __syncwarp();
        const T* g = gO + static_cast<int64_t>(row) * rowsize;
        const T* w = W + static_cast<int64_t>(j) * nW1 * L;
        T* gw = want_w ? gW + static_cast<int64_t>(j) * nW1 * L : nullptr;
        for (int b0 = 0; b0 < L; b0 += 32) {
            const int b = b0 + lane;
            const bool valid = b < L;
            const T Bb = valid ? B[e * L + b] : T(0);
            T gb = T(0);
            for (int m2 = 0; m2 < nW1; m2++) {
                const T wv = valid ? __ldg(w + m2 * L + b) : T(0);
                T accw = T(0);
                for (int m3 = 0; m3 < nO1; m3++) {
                    const int c = m3 * nW1 + m2;
                    if (s.start[c + 1] == s.start[c]) continue;
                    const T gv = valid ? __ldg(g + m3 * L + b) : T(0);
                    accw += T_s[c] * gv;
                    if (want_a) {
                        const T u = warp_sum(gv * wv * Bb);
                        if (lane == 0) U_s[c] += u;
                    }
                }
                gb += wv * accw;
                if (want_w && valid) red_add(gw + m2 * L + b, Bb * accw);
            }
            if (want_b && valid) gB[e * L + b] = gb;
        }
        if (want_a) {
            __syncwarp();
            for (int idx = lane; idx < nA * 33; idx += 32) ga_priv[idx] = T(0);
            __syncwarp();
            for (int pos = lane; pos < N; pos += 32)
                ga_priv[s.M1[pos] * 33 + lane] += s.C[pos] * U_s[s.cell[pos]];
            __syncwarp();
            for (int m = lane; m < nA; m += 32) {
                T sum = T(0);
                for (int l = 0; l < 32; l++) sum += ga_priv[m * 33 + l];
                gA[e * nA + m] = sum;
            }
        }
    }
}

// ---------------------------------------------------------------------------- fast kernels
// For A.shape[1] <= 16 and W.shape[1] <= 16 (angular channels up to l = 3). Template
// parameters: TP = W.shape[1] rounded up to a multiple of four, NAP = A.shape[1] rounded up
// likewise. Differences from the general kernels above:
//   * the coupling table is used in dense form D[cell][m1] (built once per call), so that
//     T_e = D a_e is a branch-free matrix-vector product with lanes over cells and the A row
//     in registers, and the reverse contraction gA_e = D^T U_e likewise;
//   * T_e rows are padded to TP and read as 16-byte broadcasts;
//   * the edge's W values W[J_e, :, b] sit in registers (one load each per edge instead of
//     one per cell);
//   * sums over the 32 lanes (U_e, gA_e) use a recursive-halving shuffle reduction.

__host__ __device__ inline size_t round4(size_t n) { return (n + 3) / 4 * 4; }

template <typename T, int N> struct Vec;
template <> struct Vec<double, 2> { using type = double2; };
template <> struct Vec<float, 4> { using type = float4; };

// Block-shared part of the fast kernels' shared memory.
template <typename T> struct Dense {
    T* D;          // [ncc][ds]
    int32_t* tpos; // [ncc] position of compact cell cc in a padded T_e / U_e
    T* warp_base;  // per-warp scalars start here (16-byte aligned)
};

template <typename T>
__device__ __forceinline__ Dense<T> carve_dense(unsigned char* raw, int ncc, int ds) {
    Dense<T> d;
    d.D = reinterpret_cast<T*>(raw);
    const size_t d_scalars = round4(static_cast<size_t>(ncc) * ds);
    d.warp_base = d.D + d_scalars;
    d.tpos = nullptr; // set by the caller after the per-warp area
    return d;
}

// `stride`: row stride of the per-edge T_e buffer; `transposed`: T_e stored as [m2][m3].
template <typename T>
__device__ __forceinline__ void load_dense(const Dense<T>& d, const Coupling<T>& cp, int ncc,
                                           int ds, int nW1, int stride, bool transposed = false) {
    for (int i = threadIdx.x; i < ncc * ds; i += blockDim.x) d.D[i] = cp.D[i];
    for (int cc = threadIdx.x; cc < ncc; cc += blockDim.x) {
        const int m3 = cc / nW1, m2 = cc - m3 * nW1;
        d.tpos[cc] = transposed ? m2 * stride + m3 : m3 * stride + m2;
    }
}

// T_e = D a_e: lanes over compact cells, the A row in registers.
template <typename T, int NAP>
__device__ __forceinline__ void dense_contract(const Dense<T>& d, int ncc, int ds,
                                               const T* __restrict__ a_row, int nA, T* T_s,
                                               T* U_s, int lane) {
    T a[NAP];
#pragma unroll
    for (int m = 0; m < NAP; m++) a[m] = m < nA ? __ldg(a_row + m) : T(0);
    __syncwarp(); // the previous edge's readers of T_s / U_s are done
    for (int cc = lane; cc < ncc; cc += 32) {
        const T* row = d.D + cc * ds;
        T t = T(0);
#pragma unroll
        for (int m = 0; m < NAP; m++) t += row[m] * a[m];
        const int pos = d.tpos[cc];
        T_s[pos] = t;
        if (U_s != nullptr) U_s[pos] = T(0);
    }
    __syncwarp();
}

// Same, with the A row already in registers.
template <typename T, int NAP>
__device__ __forceinline__ void dense_contract_regs(const Dense<T>& d, int ncc, int ds,
                                                    const T (&a)[NAP], T* T_s, int lane) {
    __syncwarp(); // the previous edge's readers of T_s are done
    for (int cc = lane; cc < ncc; cc += 32) {
        const T* row = d.D + cc * ds;
        T t = T(0);
#pragma unroll
        for (int m = 0; m < NAP; m++) t += row[m] * a[m];
        T_s[d.tpos[cc]] = t;
    }
    __syncwarp();
}

template <typename T, int TP>
__device__ __forceinline__ T dot_row(const T* __restrict__ row, const T (&w)[TP]) {
    constexpr int V = 16 / sizeof(T);
    using VT = typename Vec<T, V>::type;
    T p = T(0);
#pragma unroll
    for (int q = 0; q < TP / V; q++) {
        union {
            VT v;
            T s[V];
        } u;
        u.v = *reinterpret_cast<const VT*>(row + q * V);
#pragma unroll
        for (int i = 0; i < V; i++) p += u.s[i] * w[q * V + i];
    }
    return p;
}

template <typename T, int TP, int NAP, bool SEGMENTED>
__global__ void sasaw_fwd_fast(T* __restrict__ O, const T* __restrict__ A, const T* __restrict__ B,
                               const T* __restrict__ W, const int32_t* __restrict__ Jw,
                               const int32_t* __restrict__ Io,
                               const int64_t* __restrict__ offsets, Coupling<T> cp, int64_t E,
                               int nA, int L, int64_t nW0, int nW1, int nO1, bool always,
                               Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ncc = nO1 * nW1, ds = cp.d_stride, tsize = nO1 * TP;
    const size_t rowsize = static_cast<size_t>(nO1) * L;
    const size_t per_warp = round4(tsize) + (SEGMENTED ? round4(rowsize) : 0);
    if (SEGMENTED ? saw_unsorted(st) : (!always && !saw_unsorted(st))) return;
    Dense<T> d = carve_dense<T>(smem_raw, ncc, ds);
    d.tpos = reinterpret_cast<int32_t*>(d.warp_base + per_warp * warps);
    load_dense(d, cp, ncc, ds, nW1, TP);
    T* T_s = d.warp_base + per_warp * warp; // [nO1][TP], 16-byte aligned
    T* Oacc = T_s + round4(tsize);
    for (int i = lane; i < tsize; i += 32) T_s[i] = T(0); // padding columns stay zero
    __syncthreads();

    auto edge = [&](int64_t e, int64_t out_row) {
        int32_t j = __ldg(Jw + e);
        if (clamp_index(j, static_cast<int32_t>(nW0)) && lane == 0) report_bad_index(st, kBitJ);
        dense_contract<T, NAP>(d, ncc, ds, A + e * nA, nA, T_s, static_cast<T*>(nullptr), lane);
        const T* wrow = W + static_cast<int64_t>(j) * nW1 * L;
        for (int b0 = 0; b0 < L; b0 += 32) {
            const int b = b0 + lane;
            const bool valid = b < L;
            T w[TP];
#pragma unroll
            for (int m2 = 0; m2 < TP; m2++)
                w[m2] = (valid && m2 < nW1) ? __ldg(wrow + m2 * L + b) : T(0);
            const T Bb = valid ? B[e * L + b] : T(0);
            for (int m3 = 0; m3 < nO1; m3++) {
                const T p = dot_row<T, TP>(T_s + m3 * TP, w);
                if (valid) {
                    if (SEGMENTED)
                        Oacc[m3 * L + b] += Bb * p;
                    else
                        red_add(O + out_row * rowsize + m3 * L + b, Bb * p);
                }
            }
        }
    };

    if (SEGMENTED) {
        const int64_t r = static_cast<int64_t>(blockIdx.x) * warps + warp;
        if (r >= nW0) return;
        const int64_t begin = offsets[r], end = offsets[r + 1];
        for (int idx = lane; idx < static_cast<int>(rowsize); idx += 32) Oacc[idx] = T(0);
        for (int64_t e = begin; e < end; e++) edge(e, r);
        __syncwarp();
        T* dst = O + r * rowsize;
        for (int idx = lane; idx < static_cast<int>(rowsize); idx += 32) dst[idx] = Oacc[idx];
    } else {
        const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps;
        for (int64_t e = static_cast<int64_t>(blockIdx.x) * warps + warp; e < E; e += nwarps) {
            int32_t row = __ldg(Io + e);
            if (clamp_index(row, static_cast<int32_t>(nW0))) {
                if (lane == 0) report_bad_index(st, kBitI);
                continue;
            }
            edge(e, row);
        }
    }
}

// Sums VP values over the 32 lanes with VP - 1 + log2(32 / VP) shuffles (recursive halving):
// afterwards every lane holds the total of value number lane >> (5 - log2(VP)).
template <typename T, int VP> __device__ __forceinline__ T reduce_to_lanes(T (&v)[VP], int lane) {
    int d = 16;
#pragma unroll
    for (int half = VP / 2; half >= 1; half >>= 1, d >>= 1) {
        const bool upper = (lane & d) != 0;
#pragma unroll
        for (int i = 0; i < half; i++) {
            const T keep = upper ? v[i + half] : v[i];
            const T send = upper ? v[i] : v[i + half];
            v[i] = keep + __shfl_xor_sync(kFullMask, send, d);
        }
    }
    T r = v[0];
    for (; d >= 1; d >>= 1) r += __shfl_xor_sync(kFullMask, r, d);
    return r;
}

template <int TP> struct Pow2 { static constexpr int value = TP <= 4 ? 4 : TP <= 8 ? 8 : 16; };
template <int VP> struct Log2 { static constexpr int value = VP == 4 ? 2 : VP == 8 ? 3 : 4; };

template <typename T, int TP, int NAP>
__global__ void sasaw_vjp_fast(T* __restrict__ gA, T* __restrict__ gB, T* __restrict__ gW,
                               const T* __restrict__ gO, const T* __restrict__ A,
                               const T* __restrict__ B, const T* __restrict__ W,
                               const int32_t* __restrict__ Jw, const int32_t* __restrict__ Io,
                               Coupling<T> cp, int64_t E, int nA, int L, int64_t nW0, int nW1,
                               int nO1, Status st) {
    constexpr int VP = Pow2<TP>::value;
    constexpr int kShift = 5 - Log2<VP>::value;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ncc = nO1 * nW1, ds = cp.d_stride, tsize = nO1 * TP;
    const size_t per_warp = 2 * round4(tsize);
    Dense<T> d = carve_dense<T>(smem_raw, ncc, ds);
    d.tpos = reinterpret_cast<int32_t*>(d.warp_base + per_warp * warps);
    load_dense(d, cp, ncc, ds, nW1, TP);
    T* T_s = d.warp_base + per_warp * warp;
    T* U_s = T_s + round4(tsize);
    for (int i = lane; i < tsize; i += 32) T_s[i] = T(0);
    __syncthreads();
    const int64_t rowsize = static_cast<int64_t>(nO1) * L;
    const bool want_a = gA != nullptr, want_b = gB != nullptr, want_w = gW != nullptr;
    const int my_value = lane >> kShift;
    const bool writer = (lane & ((1 << kShift) - 1)) == 0 && my_value < nW1;

    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * warps + warp; e < E; e += nwarps) {
        int32_t row = __ldg(Io + e), j = __ldg(Jw + e);
        if (clamp_index(row, static_cast<int32_t>(nW0)) && lane == 0) report_bad_index(st, kBitI);
        if (clamp_index(j, static_cast<int32_t>(nW0)) && lane == 0) report_bad_index(st, kBitJ);
        dense_contract<T, NAP>(d, ncc, ds, A + e * nA, nA, T_s, U_s, lane);
        const T* g = gO + static_cast<int64_t>(row) * rowsize;
        const T* wrow = W + static_cast<int64_t>(j) * nW1 * L;
        T* gw = want_w ? gW + static_cast<int64_t>(j) * nW1 * L : nullptr;
        for (int b0 = 0; b0 < L; b0 += 32) {
            const int b = b0 + lane;
            const bool valid = b < L;
            T w[TP], accw[TP];
#pragma unroll
            for (int m2 = 0; m2 < TP; m2++) {
                w[m2] = (valid && m2 < nW1) ? __ldg(wrow + m2 * L + b) : T(0);
                accw[m2] = T(0);
            }
            const T Bb = valid ? B[e * L + b] : T(0);
            for (int m3 = 0; m3 < nO1; m3++) {
                const T gv = valid ? __ldg(g + m3 * L + b) : T(0);
                const T* trow = T_s + m3 * TP;
                constexpr int V = 16 / sizeof(T);
                using VT = typename Vec<T, V>::type;
#pragma unroll
                for (int q = 0; q < TP / V; q++) {
                    union {
                        VT v;
                        T s[V];
                    } u;
                    u.v = *reinterpret_cast<const VT*>(trow + q * V);
#pragma unroll
                    for (int i = 0; i < V; i++) accw[q * V + i] += u.s[i] * gv;
                }
                if (want_a) {
                    // U_e[m3, m2] = sum_b gO[m3,b] B[b] W[m2,b]: TP lane-partials, summed over lanes
                    const T gb_ = gv * Bb;
                    T up[VP];
#pragma unroll
                    for (int m2 = 0; m2 < VP; m2++) up[m2] = m2 < TP ? gb_ * w[m2 < TP ? m2 : 0] : T(0);
                    const T total = reduce_to_lanes<T, VP>(up, lane);
                    if (writer) U_s[m3 * TP + my_value] += total;
                }
            }
            T gb = T(0);
#pragma unroll
            for (int m2 = 0; m2 < TP; m2++) {
                gb += w[m2] * accw[m2];
                if (want_w && valid && m2 < nW1) red_add(gw + m2 * L + b, Bb * accw[m2]);
            }
            if (want_b && valid) gB[e * L + b] = gb;
        }
        if (want_a) {
            // gA_e = D^T U_e: lanes over cells, then one sum over lanes per component
            __syncwarp();
            T ga[16];
#pragma unroll
            for (int m = 0; m < 16; m++) ga[m] = T(0);
            for (int cc = lane; cc < ncc; cc += 32) {
                const T u = U_s[d.tpos[cc]];
                const T* drow = d.D + cc * ds;
#pragma unroll
                for (int m = 0; m < NAP; m++) ga[m] += drow[m] * u;
            }
            const T total = reduce_to_lanes<T, 16>(ga, lane);
            const int m = lane >> 1;
            if ((lane & 1) == 0 && m < nA) gA[e * nA + m] = total;
        }
    }
}

// ------------------------------------------------------------------- tensor-core kernels
// f64 only, A.shape[1], W.shape[1] and output_size all <= 16. Profiling the kernels above
// showed the small dense contractions per edge (9x9 by 9x32 at the benchmark shape), their
// operand reads and, in the VJP, the shuffle reductions dominating the instruction stream.
// The kernels below run every contraction on the FP64 tensor-core path (mma.sync m8n8k4: 256
// multiply-adds per warp instruction instead of 32).
// Fragment layout of m8n8k4 (lane = 4*qr + qc): A[qr][qc], B[k = qc][n = qr],
// C[qr][2*qc + {0,1}].


// Row stride for an A-operand matrix read as 8 rows x 4 columns per fragment: a multiple of
// four that is 4 or 12 modulo 16, so that the eight rows fall on distinct banks.
__host__ __device__ constexpr int a_stride(int cols4) { return cols4 % 8 == 4 ? cols4 : cols4 + 4; }
// VJP, f64 only, A.shape[1], W.shape[1] and output_size all <= 16. The shuffle reductions of
// the kernel above made it issue-bound (about 2600 warp instructions per edge). Here every
// contraction runs on the FP64 tensor-core path and a warp works on eight consecutive edges at
// a time:
//   phase A  T[cell, e] = sum_m D[cell, m] A[e, m] for the eight edges at once (edges are the
//            n dimension of the MMA), written to one shared-memory slot per edge;
//   phase B  per edge: X^T[b, m2] = sum_m3 gO[I_e, m3, b] T_e[m3, m2]  -> grad_B, grad_W,
//            U_e[m3, m2] = sum_b gO[I_e, m3, b] (B[e, b] W[J_e, m2, b]) -> the edge's slot;
//   phase C  grad_A[e, m] = sum_cell U[e, cell] D[cell, m] for the eight edges at once.
// The gO fragments stay in registers while consecutive edges share the output row (always, for
// a sorted scatter index); W rows and B arrive by cp.async one edge ahead. Cells are numbered
// m3 * TS + m2 (padding cells have zero rows in D), so T_e and U_e share one layout.

template <int TP> struct VjpMma {
    static constexpr int TS = a_stride(TP);  // row stride of T_e / U_e
    static constexpr int WS = 36;            // row stride of a staged W[J_e] chunk
    static constexpr int NT2 = TP > 8 ? 2 : 1;  // 8-wide tiles over m2
    __host__ __device__ static int ncell(int nO1) { return nO1 * TS; }
    // Distance between the slots of consecutive edges: 4 modulo 8, so that the eight slots read
    // or written by one fragment access fall on distinct banks. Cells are written in whole
    // tiles of eight; the last of the four spare scalars is never written and serves as the
    // zero that out-of-range fragment elements read.
    __host__ __device__ static int slot(int nO1) { return (ncell(nO1) + 7) / 8 * 8 + 4; }
    // One stage: rows 0..nW1-1 a 32-wide chunk of W[J_e], row nW1 the chunk of B[e], row
    // nW1+1 zeros.
    __host__ __device__ static int stage(int nW1) { return (nW1 + 2) * WS; }
    __host__ __device__ static size_t per_warp(int nO1, int nW1) {
        return 8 * static_cast<size_t>(slot(nO1)) + 2 * static_cast<size_t>(stage(nW1));
    }
    // row stride of D: A.shape[1] rounded up to 4 or 12 modulo 16
    __host__ __device__ static int d_stride(int nA) { return a_stride((nA + 3) / 4 * 4); }
    __host__ __device__ static size_t d_scalars(int nO1, int nA) {
        return static_cast<size_t>((ncell(nO1) + 7) / 8 * 8) * d_stride(nA);
    }
};


// KS3 = number of four-row k-steps that cover output_size.
// Predicated forms (one instruction each, no branch around them).
template <int BYTE_OFFSET>
__device__ __forceinline__ void red_add_if(bool p, double* addr, double v) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %2, 0;\n @p red.global.add.f64 [%0 + %3], %1;\n}\n"
                 :: "l"(addr), "d"(v), "r"(static_cast<int>(p)), "n"(BYTE_OFFSET)
                 : "memory");
}
template <int BYTE_OFFSET> __device__ __forceinline__ void red_add_at(double* addr, double v) {
    asm volatile("red.global.add.f64 [%0 + %2], %1;\n" ::"l"(addr), "d"(v), "n"(BYTE_OFFSET) : "memory");
}
// Copies 16 bytes if p; src_bytes = 0 writes zeros instead of reading.
__device__ __forceinline__ void cp_async16_if(bool p, void* smem_dst, const void* global_src,
                                              int src_bytes) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %3, 0;\n"
                 " @p cp.async.ca.shared.global [%0], [%1], 16, %2;\n}\n"
                 :: "r"(dst), "l"(global_src), "r"(src_bytes), "r"(static_cast<int>(p))
                 : "memory");
}

template <int TP, int KS3>
__global__ void __launch_bounds__(128, 3)
sasaw_vjp_mma(double* __restrict__ gA, double* __restrict__ gB, double* __restrict__ gW,
              const double* __restrict__ gO, const double* __restrict__ A,
              const double* __restrict__ B, const double* __restrict__ W,
              const int32_t* __restrict__ Jw, const int32_t* __restrict__ Io,
              Coupling<double> cp, int64_t E, int nA, int L, int64_t nW0, int nW1, int nO1,
              bool wide_copies, bool only_if_unsorted, Status st) {
    using T = double;
    using Lay = VjpMma<TP>;
    constexpr int TS = Lay::TS, WS = Lay::WS, NT2 = Lay::NT2;
    constexpr int MT3 = KS3 > 2 ? 2 : 1; // 8-high tiles over m3
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // (a kernel for sorted input ran before this one and has done the work unless it stood down)
    if (only_if_unsorted && !saw_unsorted(st)) return;
    // the shuffle tells the compiler that the warp number is the same in all lanes, so that
    // everything derived from it (edge ranges, loop counts) stays in uniform control flow
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0);
    const int qr = lane >> 2, qc = lane & 3;
    const int ncell = Lay::ncell(nO1), nct = (ncell + 7) / 8, ES = Lay::slot(nO1);
    const int stage = Lay::stage(nW1), DS = cp.d_stride;
    T* D_s = reinterpret_cast<T*>(smem_raw); // [8 * nct][DS], rows >= ncell zero
    const int d_scalars = static_cast<int>(Lay::d_scalars(nO1, nA));
    const size_t per_warp = Lay::per_warp(nO1, nW1);
    T* slots = D_s + d_scalars + per_warp * warp; // [8][ES]
    T* stages = slots + 8 * ES;                   // [2][nW1 + 2][WS]
    for (int i = threadIdx.x; i < d_scalars; i += blockDim.x)
        D_s[i] = i < ncell * DS ? cp.D[i] : T(0);
    for (int i = lane; i < static_cast<int>(per_warp); i += 32) slots[i] = T(0);
    __syncthreads();

    const bool want_a = gA != nullptr, want_bw = gB != nullptr || gW != nullptr;
    const int64_t rowsize = static_cast<int64_t>(nO1) * L;
    const int nchunks = (L + 31) / 32;
    const int ksa = (nA + 3) / 4;    // k-steps over m1
    const int nta = nA > 8 ? 2 : 1;  // 8-wide tiles over m1

    // Per-lane offsets of the fragment elements, fixed for the whole kernel; elements outside
    // the operands point at a zero.
    int t_off[KS3][NT2]; // T_e[m3 = 4 ks + qc][m2 = 8 nt + qr] in a slot
#pragma unroll
    for (int ks = 0; ks < KS3; ks++)
#pragma unroll
        for (int nt = 0; nt < NT2; nt++) {
            const int m3 = 4 * ks + qc, m2 = 8 * nt + qr;
            t_off[ks][nt] = (m3 < nO1 && m2 < nW1) ? m3 * TS + m2 : ES - 1;
        }
    int wk_off[NT2]; // W chunk [m2 = 8 nt + qr][qc + 4 kb]
#pragma unroll
    for (int nt = 0; nt < NT2; nt++)
        wk_off[nt] = (8 * nt + qr < nW1 ? 8 * nt + qr : nW1 + 1) * WS + qc;
    int wc_off[NT2][2]; // W chunk [m2 = 8 nt + 2 qc + h][qr + 8 mt]
#pragma unroll
    for (int nt = 0; nt < NT2; nt++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int m2 = 8 * nt + 2 * qc + h;
            wc_off[nt][h] = (m2 < nW1 ? m2 : nW1 + 1) * WS + qr;
        }

    // this warp's contiguous range of eight-edge batches
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps;
    const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * warps + warp;
    const int64_t nbatch = (E + 7) / 8;
    const int64_t e_begin = nbatch * gwarp / nwarps * 8;
    const int64_t e_end = min(nbatch * (gwarp + 1) / nwarps * 8, E);
    if (e_begin >= e_end) return;

    // Indices of the batch's edges (lane & 7 holds edge number lane & 7).
    auto load_meta = [&](int64_t eb, int32_t& jv, int32_t& rv) {
        const int64_t e = eb + (lane & 7);
        jv = 0, rv = 0;
        if (e < E) {
            jv = __ldg(Jw + e);
            rv = __ldg(Io + e);
            if (clamp_index(jv, static_cast<int32_t>(nW0)) && lane < 8) report_bad_index(st, kBitJ);
            if (clamp_index(rv, static_cast<int32_t>(nW0)) && lane < 8) report_bad_index(st, kBitI);
        }
    };
    // A fragments of phase A: edge qr of the batch, component 4 ks + qc.
    auto load_a = [&](int64_t eb, T (&af)[4]) {
        const int64_t ea = eb + qr;
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            const int m = 4 * ks + qc;
            af[ks] = (ea < E && m < nA) ? __ldg(A + ea * nA + m) : T(0);
        }
    };
    // Asynchronous copies of W[j, :, b0..b0+31] and B[e, b0..b0+31] into stage s. With
    // wide_copies (L even, 16-byte aligned operands) a lane moves two scalars per copy and the
    // B chunk rides along as row nW1.
    auto issue = [&](int s, int64_t e, int32_t j, int b0) {
        T* w_s = stages + s * stage;
        const T* wsrc = W + static_cast<int64_t>(j) * nW1 * L + b0;
        const T* bsrc = B + e * L + b0;
        if (wide_copies) {
            const int col = 2 * (lane & 15);
            const int bytes = b0 + col < L ? 16 : 0; // 0: zero fill
            const int scol = bytes != 0 ? col : 0;   // keeps the unused source address valid
            int r = lane >> 4;
            const T* src = wsrc + r * L + scol;
            T* dst = w_s + r * WS + col;
#pragma unroll
            for (int it = 0; it < TP / 2; it++, r += 2, src += 2 * L, dst += 2 * WS)
                if (2 * it < nW1) cp_async16_if(r < nW1, dst, src, bytes);
            cp_async16_if(lane < 16, w_s + nW1 * WS + col, bsrc + scol, bytes);
        } else {
            const bool inside = b0 + lane < L;
            for (int r = 0; r <= nW1; r++) {
                T* dst = w_s + r * WS + lane;
                if (inside)
                    cp_async<8>(dst, (r < nW1 ? wsrc + r * L : bsrc) + lane);
                else
                    dst[0] = T(0);
            }
        }
        cp_async_commit();
    };

    // gO fragments of one (row, chunk): gt[mt][ks] = gO[row, 4 ks + qc, b0 + 8 mt + qr] (the A
    // operand of X^T), gu[mt][kb] = gO[row, 8 mt + qr, b0 + 4 kb + qc] (the A operand of U).
    T gt[4][KS3], gu[MT3][8];
    auto load_g = [&](int32_t row, int b0) {
        const T* g = gO + static_cast<int64_t>(row) * rowsize;
#pragma unroll
        for (int mt = 0; mt < 4; mt++)
#pragma unroll
            for (int ks = 0; ks < KS3; ks++) {
                const int m3 = 4 * ks + qc, b = b0 + 8 * mt + qr;
                gt[mt][ks] = (want_bw && m3 < nO1 && b < L) ? __ldg(g + m3 * L + b) : T(0);
            }
#pragma unroll
        for (int mt = 0; mt < MT3; mt++)
#pragma unroll
            for (int kb = 0; kb < 8; kb++) {
                const int m3 = 8 * mt + qr, b = b0 + 4 * kb + qc;
                gu[mt][kb] = (want_a && m3 < nO1 && b < L) ? __ldg(g + m3 * L + b) : T(0);
            }
    };

    int32_t jv, rv, jv_n = 0, rv_n = 0;
    load_meta(e_begin, jv, rv);
    issue(0, e_begin, __shfl_sync(kFullMask, jv, 0), 0);
    int s = 0;
    int32_t cached_row = -1;

    for (int64_t eb = e_begin; eb < e_end; eb += 8) {
        const int nvalid = static_cast<int>(min(static_cast<int64_t>(8), e_end - eb));
        const bool more = eb + 8 < e_end;
        if (more) load_meta(eb + 8, jv_n, rv_n);

        // ---- phase A: T for the eight edges
        if (want_bw) {
            T af[4];
            load_a(eb, af);
            const T* drow = D_s + qr * DS + qc;
            T* dst = slots + (2 * qc) * ES + qr;
            for (int t = 0; t < nct; t++, drow += 8 * DS, dst += 8) {
                T c[2];
                dmma0(c, drow[0], af[0]);
#pragma unroll
                for (int ks = 1; ks < 4; ks++)
                    if (ks < ksa) dmma(c, drow[4 * ks], af[ks]);
                dst[0] = c[0]; // cells >= ncell of the last tile get zeros
                dst[ES] = c[1];
            }
        }
        __syncwarp();

        // ---- phase B: edge by edge
        for (int i = 0; i < nvalid; i++) {
            const int64_t e = eb + i;
            const int32_t j = __shfl_sync(kFullMask, jv, i);
            const int32_t row = __shfl_sync(kFullMask, rv, i);
            T* slot = slots + i * ES;
            T u[MT3][NT2][2];

            for (int c = 0; c < nchunks; c++) {
                const int b0 = 32 * c;
                // the copies of the next (edge, chunk) go out before this one is used
                bool has_next = true;
                if (c + 1 < nchunks)
                    issue(s ^ 1, e, j, b0 + 32);
                else if (i + 1 < nvalid)
                    issue(s ^ 1, e + 1, __shfl_sync(kFullMask, jv, i + 1), 0);
                else if (more)
                    issue(s ^ 1, eb + 8, __shfl_sync(kFullMask, jv_n, 0), 0);
                else
                    has_next = false;
                if (has_next)
                    cp_async_wait<1>();
                else
                    cp_async_wait<0>();
                __syncwarp();
                if (nchunks > 1 || row != cached_row) {
                    load_g(row, b0);
                    cached_row = row;
                }
                const T* w_s = stages + s * stage;
                const T* b_s = w_s + nW1 * WS;

                if (want_bw) {
                    // X^T[b = 8 mt + qr][m2 = 8 nt + 2 qc + {0,1}]
                    T x[4][NT2][2];
#pragma unroll
                    for (int ks = 0; ks < KS3; ks++) {
                        T bt[NT2];
#pragma unroll
                        for (int nt = 0; nt < NT2; nt++) bt[nt] = slot[t_off[ks][nt]];
#pragma unroll
                        for (int mt = 0; mt < 4; mt++)
#pragma unroll
                            for (int nt = 0; nt < NT2; nt++) {
                                if (ks == 0)
                                    dmma0(x[mt][nt], gt[mt][ks], bt[nt]);
                                else
                                    dmma(x[mt][nt], gt[mt][ks], bt[nt]);
                            }
                    }
                    T part[4] = {T(0), T(0), T(0), T(0)};
                    T bv[4];
#pragma unroll
                    for (int mt = 0; mt < 4; mt++) bv[mt] = b_s[8 * mt + qr];
                    const int width = L - b0; // columns of this chunk
                    T* gw = gW != nullptr
                                ? gW + static_cast<int64_t>(j) * nW1 * L + b0 + 2 * qc * L + qr
                                : nullptr;
#pragma unroll
                    for (int nt = 0; nt < NT2; nt++)
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (8 * nt + h >= nW1) continue; // no lane has a valid m2
                            const T* wcol = w_s + wc_off[nt][h];
#pragma unroll
                            for (int mt = 0; mt < 4; mt++) part[mt] += x[mt][nt][h] * wcol[8 * mt];
                            if (gw == nullptr) continue;
                            T* gdst = gw + (8 * nt + h) * L;
                            if (8 * nt + 8 <= nW1 && width >= 32) { // every lane has an element
                                red_add_at<0>(gdst, x[0][nt][h] * bv[0]);
                                red_add_at<64>(gdst, x[1][nt][h] * bv[1]);
                                red_add_at<128>(gdst, x[2][nt][h] * bv[2]);
                                red_add_at<192>(gdst, x[3][nt][h] * bv[3]);
                            } else {
                                const bool ok = 8 * nt + 2 * qc + h < nW1;
                                red_add_if<0>(ok && qr < width, gdst, x[0][nt][h] * bv[0]);
                                red_add_if<64>(ok && 8 + qr < width, gdst, x[1][nt][h] * bv[1]);
                                red_add_if<128>(ok && 16 + qr < width, gdst, x[2][nt][h] * bv[2]);
                                red_add_if<192>(ok && 24 + qr < width, gdst, x[3][nt][h] * bv[3]);
                            }
                        }
                    if (gB != nullptr) {
                        // sum over the four lanes of a quad; lane (qr, qc) ends with b = 8 qc + qr
                        const bool up2 = (qc & 2) != 0, up1 = (qc & 1) != 0;
                        const T r0 = (up2 ? part[2] : part[0]) +
                                     __shfl_xor_sync(kFullMask, up2 ? part[0] : part[2], 2);
                        const T r1 = (up2 ? part[3] : part[1]) +
                                     __shfl_xor_sync(kFullMask, up2 ? part[1] : part[3], 2);
                        const T gb = (up1 ? r1 : r0) + __shfl_xor_sync(kFullMask, up1 ? r0 : r1, 1);
                        const int b = b0 + 8 * qc + qr;
                        if (b < L) gB[e * L + b] = gb;
                    }
                }
                if (want_a) {
                    // U[m3 = 8 mt + qr][m2 = 8 nt + 2 qc + {0,1}] += sum_b gO[m3, b] (B[b] W[m2, b])
#pragma unroll
                    for (int kb = 0; kb < 8; kb++) {
                        const T bb = b_s[4 * kb + qc];
                        T bw[NT2];
#pragma unroll
                        for (int nt = 0; nt < NT2; nt++) bw[nt] = w_s[wk_off[nt] + 4 * kb] * bb;
#pragma unroll
                        for (int nt = 0; nt < NT2; nt++) {
#pragma unroll
                            for (int mt = 0; mt < MT3; mt++) {
                                if (kb == 0 && c == 0)
                                    dmma0(u[mt][nt], gu[mt][kb], bw[nt]);
                                else
                                    dmma(u[mt][nt], gu[mt][kb], bw[nt]);
                            }
                        }
                    }
                }
                __syncwarp(); // stage s is overwritten by the copies issued next round
                s ^= 1;
            }
            if (want_a) {
                // T_e is no longer needed: the slot now holds U_e (padding cells stay zero)
#pragma unroll
                for (int mt = 0; mt < MT3; mt++)
#pragma unroll
                    for (int nt = 0; nt < NT2; nt++) {
                        const int m3 = 8 * mt + qr, m2 = 8 * nt + 2 * qc;
                        T* dst = slot + m3 * TS + m2;
                        if (8 * mt + 8 <= nO1 && 8 * nt + 8 <= nW1) { // whole tile inside
                            *reinterpret_cast<double2*>(dst) = make_double2(u[mt][nt][0], u[mt][nt][1]);
                        } else {
                            if (m3 < nO1 && m2 < nW1) dst[0] = u[mt][nt][0];
                            if (m3 < nO1 && m2 + 1 < nW1) dst[1] = u[mt][nt][1];
                        }
                    }
            }
        }

        // ---- phase C: grad_A for the eight edges
        if (want_a) {
            __syncwarp();
            T ga[2][2] = {{T(0), T(0)}, {T(0), T(0)}};
            const T* urow = slots + qr * ES + qc;
            const T* dcol = D_s + qc * DS + qr;
#pragma unroll 3
            for (int kc = 0; kc < ncell / 4; kc++, dcol += 4 * DS) {
                const T au = urow[4 * kc];
                dmma(ga[0], au, dcol[0]);
                if (nta > 1) dmma(ga[1], au, dcol[8]);
            }
            const int64_t ea = eb + qr;
            if (ea < e_end) {
#pragma unroll
                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const int m = 8 * nt + 2 * qc + h;
                        if (m < nA) gA[ea * nA + m] = ga[nt][h];
                    }
            }
        }
        __syncwarp(); // the slots are rewritten by the next batch's phase A
        jv = jv_n;
        rv = rv_n;
    }
}

// Forward, f64, A.shape[1], W.shape[1] and output_size all <= 16: the same eight-edge batches
// as the VJP above. Phase A builds T_e for eight edges with one pass of MMAs; then, per edge,
//     O[I_e, m3, b] += sum_m2 T_e[m3, m2] (B[e, b] W[J_e, m2, b])
// accumulates straight into the output fragments, which stay in registers for the whole
// segment of edges that share the output row (SEGMENTED, one plain store per element), or
// are flushed with atomics after every edge (unsorted scatter index).
template <int TP, bool SEGMENTED>
__global__ void __launch_bounds__(128, 3)
sasaw_fwd_mma(double* __restrict__ O, const double* __restrict__ A, const double* __restrict__ B,
              const double* __restrict__ W, const int32_t* __restrict__ Jw,
              const int32_t* __restrict__ Io, const int64_t* __restrict__ offsets,
              Coupling<double> cp, int64_t E, int nA, int L, int64_t nW0, int nW1, int nO1,
              bool wide_copies, Status st) {
    using T = double;
    using Lay = VjpMma<TP>;
    constexpr int TS = Lay::TS, WS = Lay::WS, KS2 = TP / 4;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0); // uniform for the compiler
    const int qr = lane >> 2, qc = lane & 3;
    if (SEGMENTED ? saw_unsorted(st) : !saw_unsorted(st)) return;
    const int ncell = Lay::ncell(nO1), nct = (ncell + 7) / 8, ES = Lay::slot(nO1);
    const int stage = Lay::stage(nW1), DS = cp.d_stride;
    T* D_s = reinterpret_cast<T*>(smem_raw); // [8 * nct][DS], rows >= ncell zero
    const int d_scalars = static_cast<int>(Lay::d_scalars(nO1, nA));
    const size_t per_warp = Lay::per_warp(nO1, nW1);
    T* slots = D_s + d_scalars + per_warp * warp; // [8][ES]
    T* stages = slots + 8 * ES;                   // [2][nW1 + 2][WS]
    for (int i = threadIdx.x; i < d_scalars; i += blockDim.x)
        D_s[i] = i < ncell * DS ? cp.D[i] : T(0);
    for (int i = lane; i < static_cast<int>(per_warp); i += 32) slots[i] = T(0);
    __syncthreads();

    const size_t rowsize = static_cast<size_t>(nO1) * L;
    const int ksa = (nA + 3) / 4;
    const bool two_tiles = nO1 > 8; // 8-high tiles over m3

    // Per-lane fragment offsets: T_e[m3 = 8 mt + qr][m2 = 4 ks + qc] in a slot (rows past the
    // output read the slot's zero) and W chunk row 4 ks + qc (rows past W read the zero row).
    int t_off[2][KS2], w_off[KS2];
#pragma unroll
    for (int ks = 0; ks < KS2; ks++) {
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
            t_off[mt][ks] = 8 * mt + qr < nO1 ? (8 * mt + qr) * TS + 4 * ks + qc : ES - 1;
        w_off[ks] = (4 * ks + qc < nW1 ? 4 * ks + qc : nW1 + 1) * WS + qr;
    }

    auto load_meta = [&](int64_t eb, int64_t hi, int32_t& jv, int32_t& rv) {
        const int64_t e = eb + (lane & 7);
        jv = 0, rv = 0;
        if (e < hi) {
            jv = __ldg(Jw + e);
            if (clamp_index(jv, static_cast<int32_t>(nW0)) && lane < 8) report_bad_index(st, kBitJ);
            if (!SEGMENTED) {
                rv = __ldg(Io + e);
                if (clamp_index(rv, static_cast<int32_t>(nW0)) && lane < 8) {
                    report_bad_index(st, kBitI);
                    rv = -1; // skipped below
                }
            }
        }
    };
    auto load_a = [&](int64_t eb, int64_t hi, T (&af)[4]) {
        const int64_t ea = eb + qr;
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            const int m = 4 * ks + qc;
            af[ks] = (ea < hi && m < nA) ? __ldg(A + ea * nA + m) : T(0);
        }
    };
    auto issue = [&](int s, int64_t e, int32_t j, int b0) {
        T* w_s = stages + s * stage;
        const T* wsrc = W + static_cast<int64_t>(j) * nW1 * L + b0;
        const T* bsrc = B + e * L + b0;
        if (wide_copies) {
            const int col = 2 * (lane & 15);
            const int bytes = b0 + col < L ? 16 : 0; // 0: zero fill
            const int scol = bytes != 0 ? col : 0;   // keeps the unused source address valid
            int r = lane >> 4;
            const T* src = wsrc + r * L + scol;
            T* dst = w_s + r * WS + col;
#pragma unroll
            for (int it = 0; it < TP / 2; it++, r += 2, src += 2 * L, dst += 2 * WS)
                if (2 * it < nW1) cp_async16_if(r < nW1, dst, src, bytes);
            cp_async16_if(lane < 16, w_s + nW1 * WS + col, bsrc + scol, bytes);
        } else {
            const bool inside = b0 + lane < L;
            for (int r = 0; r <= nW1; r++) {
                T* dst = w_s + r * WS + lane;
                if (inside)
                    cp_async<8>(dst, (r < nW1 ? wsrc + r * L : bsrc) + lane);
                else
                    dst[0] = T(0);
            }
        }
        cp_async_commit();
    };

    // fragment element (mt, nt, h) is output element [m3 = 8 mt + qr][b = b0 + 8 nt + 2 qc + h]
    T acc[2][4][2];
    auto clear = [&] {
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int nt = 0; nt < 4; nt++) acc[mt][nt][0] = acc[mt][nt][1] = T(0);
    };
    auto flush = [&](int64_t out_row, int b0) {
        T* dst = O + out_row * rowsize + b0 + 2 * qc;
        const int width = L - b0;
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            const int m3 = 8 * mt + qr;
            if (m3 >= nO1) continue;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                T* d2 = dst + m3 * L + 8 * nt;
                if (SEGMENTED) {
                    if (wide_copies && width >= 32) {
                        *reinterpret_cast<double2*>(d2) = make_double2(acc[mt][nt][0], acc[mt][nt][1]);
                    } else {
                        if (8 * nt + 2 * qc < width) d2[0] = acc[mt][nt][0];
                        if (8 * nt + 2 * qc + 1 < width) d2[1] = acc[mt][nt][1];
                    }
                } else {
                    if (8 * nt + 2 * qc < width) red_add(d2, acc[mt][nt][0]);
                    if (8 * nt + 2 * qc + 1 < width) red_add(d2 + 1, acc[mt][nt][1]);
                }
            }
        }
    };

    // All edges of [lo, hi) for one 32-wide chunk of b.
    auto run = [&](int64_t lo, int64_t hi, int64_t out_row, int b0) {
        int32_t jv, rv, jv_n = 0, rv_n = 0;
        T af[4], af_n[4];
        load_meta(lo, hi, jv, rv);
        load_a(lo, hi, af);
        __syncwarp();
        issue(0, lo, __shfl_sync(kFullMask, jv, 0), b0);
        int s = 0;
        for (int64_t eb = lo; eb < hi; eb += 8) {
            const int nvalid = static_cast<int>(min(static_cast<int64_t>(8), hi - eb));
            const bool more = eb + 8 < hi;
            if (more) {
                load_meta(eb + 8, hi, jv_n, rv_n);
                load_a(eb + 8, hi, af_n);
            }
            // ---- phase A: T for the eight edges
            {
                const T* drow = D_s + qr * DS + qc;
                T* dst = slots + (2 * qc) * ES + qr;
                for (int t = 0; t < nct; t++, drow += 8 * DS, dst += 8) {
                    T c[2];
                    dmma0(c, drow[0], af[0]);
#pragma unroll
                    for (int ks = 1; ks < 4; ks++)
                        if (ks < ksa) dmma(c, drow[4 * ks], af[ks]);
                    dst[0] = c[0]; // cells >= ncell of the last tile get zeros
                    dst[ES] = c[1];
                }
            }
            __syncwarp();
            // ---- phase B: edge by edge
            for (int i = 0; i < nvalid; i++) {
                bool has_next = true;
                if (i + 1 < nvalid)
                    issue(s ^ 1, eb + i + 1, __shfl_sync(kFullMask, jv, i + 1), b0);
                else if (more)
                    issue(s ^ 1, eb + 8, __shfl_sync(kFullMask, jv_n, 0), b0);
                else
                    has_next = false;
                if (has_next)
                    cp_async_wait<1>();
                else
                    cp_async_wait<0>();
                __syncwarp();
                const T* slot = slots + i * ES;
                const T* w_s = stages + s * stage;
                const T* b_s = w_s + nW1 * WS;
                T bb[4];
#pragma unroll
                for (int nt = 0; nt < 4; nt++) bb[nt] = b_s[8 * nt + qr];
#pragma unroll
                for (int ks = 0; ks < KS2; ks++) {
                    if (4 * ks < nW1) {
                        const T a0 = slot[t_off[0][ks]];
                        const T a1 = two_tiles ? slot[t_off[1][ks]] : T(0);
                        const T* wrow = w_s + w_off[ks];
#pragma unroll
                        for (int nt = 0; nt < 4; nt++) {
                            const T bw = wrow[8 * nt] * bb[nt];
                            dmma(acc[0][nt], a0, bw);
                            if (two_tiles) dmma(acc[1][nt], a1, bw);
                        }
                    }
                }
                if (!SEGMENTED) {
                    const int32_t row = __shfl_sync(kFullMask, rv, i);
                    if (row >= 0) flush(row, b0);
                    clear();
                }
                __syncwarp(); // stage s is overwritten by the copies issued next round
                s ^= 1;
            }
            __syncwarp(); // the slots are rewritten by the next batch's phase A
            jv = jv_n;
            rv = rv_n;
#pragma unroll
            for (int ks = 0; ks < 4; ks++) af[ks] = af_n[ks];
        }
        if (SEGMENTED) flush(out_row, b0);
    };

    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps;
    const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * warps + warp;
    if (SEGMENTED) {
        for (int64_t r = gwarp; r < nW0; r += nwarps) {
            const int64_t lo = offsets[r], hi = offsets[r + 1];
            for (int b0 = 0; b0 < L; b0 += 32) {
                clear();
                if (lo < hi)
                    run(lo, hi, r, b0);
                else
                    flush(r, b0);
            }
        }
    } else {
        const int64_t nbatch = (E + 7) / 8;
        const int64_t lo = nbatch * gwarp / nwarps * 8;
        const int64_t hi = min(nbatch * (gwarp + 1) / nwarps * 8, E);
        if (lo < hi)
            for (int b0 = 0; b0 < L; b0 += 32) {
                clear();
                run(lo, hi, 0, b0);
            }
    }
}

// ----------------------------------------------------------- tensor-core kernels, quads
// The kernels above spend most of their FP64 tensor-core issue slots on padding: with nine
// angular channels every dimension is padded to 12 or 16, the ninth output row costs a whole
// second 8-row tile, and only about four in ten issued MMA lanes do useful work. The kernels
// below remove the padding by choosing which index goes where in the m8n8k4 shape:
//   * cells are numbered compactly (m3 * W.shape[1] + m2), so T for eight edges takes
//     ceil(cells / 8) tiles instead of ceil(padded cells / 8);
//   * a contraction length of 4 k + 1 (nine components of A) is 4 k by MMA plus one
//     multiply-add per accumulator element for the last component;
//   * phase B contracts over (m2, edge) together: edges of one output row are taken four at
//     a time and one k-step holds one m2 of four edges, so nine channels take nine k-steps
//     with no padding at all (instead of three padded k-steps per edge = twelve per four edges);
//   * the ninth output row is not a second MMA tile: its sums are formed by the FP64 FMA pipe
//     from the very fragment registers the MMA consumes (one multiply-add per fragment element),
//     and its four partial sums per quad of lanes are added once per output row.
// A warp owns a contiguous range of output rows and walks their edges in quads; the (W rows,
// B row) blocks of the next quad are in flight (16-byte asynchronous copies by all lanes)
// while the current one is consumed, across row boundaries.

struct QuadLayout {
    int ncc;  // compact cells: output_size * W.shape[1]
    int nct;  // 8-cell tiles
    int DS;   // row stride of D (A.shape[1] rounded up to 4 or 12 modulo 16: conflict-free)
    int ES;   // distance between the T slots of consecutive edges (4 modulo 16)
    int EB;   // distance between the staged blocks of consecutive edges (4 modulo 16)
    int d_scalars;
    int warp_scalars;
};

__host__ __device__ constexpr QuadLayout quad_layout(int nA, int nW1, int nO1) {
    QuadLayout q{};
    q.ncc = nO1 * nW1;
    q.nct = (q.ncc + 7) / 8;
    q.DS = a_stride((nA + 3) / 4 * 4);
    q.ES = q.ncc + ((4 - q.ncc % 16) + 16) % 16;
    q.EB = (nW1 + 1) * 32 + 4;
    q.d_scalars = q.nct * 8 * q.DS;
    q.warp_scalars = 8 * q.ES + 2 * 4 * q.EB;
    return q;
}

// Copies 16 bytes, or writes 16 zero bytes when src_bytes == 0 (the source is not read then).
__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* global_src,
                                                 int src_bytes) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(global_src),
                 "r"(src_bytes)
                 : "memory");
}

// Where a warp is in its walk over the quads of its rows; edges are counted from the warp's
// first edge and rows from its first row, so the bookkeeping is 32-bit.
struct QuadPos {
    int row, lo, hi, e; // output row, its edges [lo, hi), first edge of the quad
    bool valid;
};

// MODE 0: output_size <= 8; MODE 1: output_size == 9 (eight rows by MMA, one by FMA);
// MODE 2: 10..16 (two MMA tiles). NA, NW, NO: A.shape[1], W.shape[1], output_size when they
// are known at compile time (all loops unroll and all shared-memory offsets are immediates:
// a quarter of the instructions of the generic form), 0 = taken from the arguments.
// f64, all three <= 16, L even, 16-byte aligned W, B and O, sorted scatter index.
template <int MODE, int NA, int NW, int NO>
__global__ void __launch_bounds__(256, 1)
sasaw_fwd_quad(double* __restrict__ O, const double* __restrict__ A, const double* __restrict__ B,
               const double* __restrict__ W, const int32_t* __restrict__ Jw,
               const int64_t* __restrict__ offsets, Coupling<double> cp, int64_t E, int nA_arg,
               int L, int64_t nW0, int nW1_arg, int nO1_arg, Status st) {
    using T = double;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    if (saw_unsorted(st)) return; // the kernels for unsorted input do the work
    const int nA = NA > 0 ? NA : nA_arg, nW1 = NW > 0 ? NW : nW1_arg, nO1 = NO > 0 ? NO : nO1_arg;
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0); // uniform for the compiler
    const int qr = lane >> 2, qc = lane & 3;
    const QuadLayout q = quad_layout(nA, nW1, nO1);
    T* D_s = reinterpret_cast<T*>(smem_raw); // [8 * nct][DS], rows >= ncc zero
    T* slots = D_s + q.d_scalars + static_cast<size_t>(q.warp_scalars) * warp; // [8][ES]
    T* stages = slots + 8 * q.ES;                                              // [2][4][EB]
    for (int i = threadIdx.x; i < q.d_scalars; i += blockDim.x)
        D_s[i] = i < q.ncc * q.DS ? cp.D[i] : T(0);
    for (int i = lane; i < q.warp_scalars; i += 32) slots[i] = T(0);
    __syncthreads();

    const int64_t total_warps = static_cast<int64_t>(gridDim.x) * warps;
    const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * warps + warp;
    const int64_t r0 = balanced_row_split(offsets, nW0, gwarp, total_warps, lane);
    const int64_t r1 = balanced_row_split(offsets, nW0, gwarp + 1, total_warps, lane);
    if (r0 >= r1) return;
    const int nrows = static_cast<int>(r1 - r0);
    // this warp's edges, operands and output, rebased to its first edge / row
    const int64_t e_base = offsets[r0];
    const T* A0 = A + e_base * nA;
    const T* B0 = B + e_base * L;
    const int32_t* J0 = Jw + e_base;
    const size_t rowsize = static_cast<size_t>(nO1) * L;
    T* O0 = O + r0 * rowsize;

    const int ksa = nA / 4;                          // whole k-steps over the components of A
    const bool rank1 = nA % 4 == 1;                  // the last component by multiply-add
    const int ksa_mma = ksa + (nA % 4 >= 2 ? 1 : 0); // else one more, partly filled, k-step

    // segment ends of 32 rows at a time: lane i holds offsets[r0 + wbase + 1 + i] - e_base
    int wbase = 0, win = 0;
    auto load_window = [&](int base) {
        const int64_t i = r0 + base + 1 + lane;
        return static_cast<int>(offsets[i < nW0 ? i : nW0] - e_base);
    };
    auto row_end = [&](int r) -> int {
        if (r - wbase >= 32) {
            wbase = r;
            win = load_window(wbase);
        }
        return __shfl_sync(kFullMask, win, r - wbase);
    };

    // fragment element (nt, h) of tile 0 is output element [m3 = qr][b = b0 + 8 nt + 2 qc + h];
    // x1: MODE 1 partial sums of row 8 for b = b0 + 8 nt + qr over this lane's edges (lane
    // qc takes edge qc of every quad); MODE 2 the second tile, rows 8 + qr
    T acc0[4][2], x1[4][2];
    auto clear = [&] {
#pragma unroll
        for (int nt = 0; nt < 4; nt++)
            acc0[nt][0] = acc0[nt][1] = x1[nt][0] = x1[nt][1] = T(0);
    };
    auto store_pair = [&](T* d2, int b, int width, T v0, T v1) {
        if (b + 1 < width) {
            *reinterpret_cast<double2*>(d2) = make_double2(v0, v1);
        } else if (b < width) {
            d2[0] = v0;
        }
    };
    auto flush = [&](int row, int b0) {
        T* dst = O0 + row * rowsize + b0;
        const int width = L - b0;
        if (MODE != 0 || qr < nO1) {
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
                store_pair(dst + qr * L + 8 * nt + 2 * qc, 8 * nt + 2 * qc, width, acc0[nt][0],
                           acc0[nt][1]);
        }
        if (MODE == 2 && 8 + qr < nO1) {
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
                store_pair(dst + (8 + qr) * L + 8 * nt + 2 * qc, 8 * nt + 2 * qc, width, x1[nt][0],
                           x1[nt][1]);
        }
        if (MODE == 1) {
            // add the four lanes of a quad; lane (qr, qc) ends with b = 8 qc + qr
            const bool up2 = (qc & 2) != 0, up1 = (qc & 1) != 0;
            const T s0 = (up2 ? x1[2][0] : x1[0][0]) +
                         __shfl_xor_sync(kFullMask, up2 ? x1[0][0] : x1[2][0], 2);
            const T s1 = (up2 ? x1[3][0] : x1[1][0]) +
                         __shfl_xor_sync(kFullMask, up2 ? x1[1][0] : x1[3][0], 2);
            const T v = (up1 ? s1 : s0) + __shfl_xor_sync(kFullMask, up1 ? s0 : s1, 1);
            const int b = 8 * qc + qr;
            if (b < width) dst[8 * L + b] = v;
        }
    };
    auto zero_row = [&](int row, int b0) {
        T* dst = O0 + row * rowsize + b0;
        const int width = L - b0 < 32 ? L - b0 : 32;
        for (int m3 = 0; m3 < nO1; m3++)
            if (lane < width) dst[m3 * L + lane] = T(0);
    };

    // A fragments of a batch of eight edges: af[ks] = A[eb + qr][4 ks + qc] (the B operand of
    // phase A: k = component, n = edge), al[h] = last component of edge eb + 2 qc + h
    auto load_a = [&](int eb, int hi, T (&af)[4], T (&al)[2]) {
        const int ea = eb + qr;
        const T* a = A0 + static_cast<int64_t>(ea) * nA + qc;
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
            af[ks] = (ks < ksa_mma && ea < hi && 4 * ks + qc < nA) ? __ldg(a + 4 * ks) : T(0);
        const int e2 = eb + 2 * qc;
        const T* a2 = A0 + static_cast<int64_t>(e2) * nA + nA - 1;
        al[0] = (rank1 && e2 < hi) ? __ldg(a2) : T(0);
        al[1] = (rank1 && e2 + 1 < hi) ? __ldg(a2 + nA) : T(0);
    };
    // T[cell, edge] = sum_m D[cell, m] A[edge, m] for the eight edges of a batch
    auto phase_a = [&](const T (&af)[4], const T (&al)[2]) {
        const T* drow = D_s + qr * q.DS + qc;
        T* dst = slots + (2 * qc) * q.ES + qr;
#pragma unroll
        for (int t = 0; t < (NO > 0 ? (NO * NW + 7) / 8 : 32); t++) {
            if (NO == 0 && t >= q.nct) break;
            T c[2] = {T(0), T(0)};
#pragma unroll
            for (int ks = 0; ks < 4; ks++)
                if (ks < ksa_mma) dmma(c, drow[t * 8 * q.DS + 4 * ks], af[ks]);
            if (rank1) {
                const T dl = drow[t * 8 * q.DS + nA - 1 - qc];
                c[0] = fma(dl, al[0], c[0]);
                c[1] = fma(dl, al[1], c[1]);
            }
            if (8 * t + qr < q.ncc) {
                dst[8 * t] = c[0];
                dst[8 * t + q.ES] = c[1];
            }
        }
    };
    // Lane i < 4 takes the W row index of edge e + i.
    auto load_j = [&](const QuadPos& p) -> int32_t {
        int32_t j = 0;
        if (p.valid && lane < 4 && p.e + lane < p.hi) {
            j = __ldg(J0 + p.e + lane);
            if (clamp_index(j, static_cast<int32_t>(nW0))) report_bad_index(st, kBitJ);
        }
        return j;
    };
    // Asynchronous copies of W[J_e, :, b0 .. b0+31] and B[e, b0 .. b0+31] of the four edges of
    // a quad into stage s: a lane moves 16 bytes per copy, two rows per round; blocks of
    // edges past the row's end and columns past L are zero-filled. Always commits a group.
    const int64_t w_stride = static_cast<int64_t>(nW1) * L;
    auto issue = [&](int s, const QuadPos& p, int32_t j_lane, int b0) {
        if (p.valid) {
            const int col = 2 * (lane & 15);
            const bool col_ok = b0 + col < L;
            T* buf = stages + s * 4 * q.EB + col + (lane >> 4) * 32;
            const int src_col = b0 + (col_ok ? col : 0);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int32_t j = __shfl_sync(kFullMask, j_lane, i);
                const bool ok = col_ok && p.e + i < p.hi;
                const T* wsrc = W + j * w_stride + src_col + (lane >> 4) * L;
                const T* bsrc = B0 + static_cast<int64_t>(ok ? p.e + i : p.e) * L + src_col;
                T* dst = buf + i * q.EB;
                const int bytes = ok ? 16 : 0;
#pragma unroll
                for (int rr = 0; rr < (NW > 0 ? (NW + 2) / 2 : 9); rr++) {
                    const int r = 2 * rr + (lane >> 4);
                    if (r <= nW1)
                        cp_async16_zfill(dst + rr * 64, r < nW1 ? wsrc + static_cast<int64_t>(2 * rr) * L : bsrc,
                                         bytes);
                }
            }
        }
        cp_async_commit();
    };
    // O[m3, b] += sum over (m2, edge of the quad) of T_edge[m3, m2] (B_edge[b] W[J_edge, m2, b]):
    // one k-step per m2, lane qc holds edge qc of the quad.
    auto phase_b = [&](int s, int quad_in_batch) {
        const T* wl = stages + s * 4 * q.EB + qc * q.EB + qr; // + m2 * 32 + 8 nt
        const T* tl = slots + (4 * quad_in_batch + qc) * q.ES; // T of this lane's edge
        T bb[4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++) bb[nt] = wl[nW1 * 32 + 8 * nt];
        const bool row_ok = MODE != 0 || qr < nO1;
        const bool row1_ok = MODE == 2 && 8 + qr < nO1;
        const T* t0 = tl + (row_ok ? qr * nW1 : 0);
        const T* t1 = tl + (MODE == 1 ? 8 * nW1 : (row1_ok ? (8 + qr) * nW1 : 0));
#pragma unroll
        for (int m2 = 0; m2 < (NW > 0 ? NW : 16); m2++) {
            if (NW == 0 && m2 >= nW1) break;
            const T a0 = row_ok ? t0[m2] : T(0);
            T a1 = T(0);
            if (MODE == 1) a1 = t1[m2];
            if (MODE == 2) a1 = row1_ok ? t1[m2] : T(0);
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const T bw = wl[m2 * 32 + 8 * nt] * bb[nt];
                dmma(acc0[nt], a0, bw);
                if (MODE == 1) x1[nt][0] = fma(a1, bw, x1[nt][0]);
                if (MODE == 2) dmma(x1[nt], a1, bw);
            }
        }
    };

    for (int b0 = 0; b0 < L; b0 += 32) {
        wbase = 0;
        win = load_window(0);
        // next quad after p; rows without edges are written as zeros on the way
        auto advance = [&](QuadPos p) -> QuadPos {
            if (!p.valid) return p;
            p.e += 4;
            while (p.e >= p.hi) {
                p.row++;
                if (p.row >= nrows) {
                    p.valid = false;
                    return p;
                }
                p.lo = p.hi;
                p.hi = row_end(p.row);
                p.e = p.lo;
                if (p.hi == p.lo) zero_row(p.row, b0);
            }
            return p;
        };
        QuadPos start;
        start.row = -1, start.valid = true;
        start.lo = start.hi = 0;
        start.e = -4;
        QuadPos p0 = advance(start);
        QuadPos p1 = advance(p0), p2 = advance(p1), p3 = advance(p2);
        int32_t j2 = load_j(p2), j3 = load_j(p3);
        issue(0, p0, load_j(p0), b0);
        issue(1, p1, load_j(p1), b0);
        T af[4], al[2], af_n[4], al_n[2];
        if (p0.valid) load_a(p0.e, p0.hi, af, al);
        if (p1.valid && ((p1.e - p1.lo) & 7) == 0) load_a(p1.e, p1.hi, af_n, al_n);
        clear();
        int s = 0;
        while (p0.valid) {
            const int in_row = p0.e - p0.lo;
            if ((in_row & 7) == 0) { // first quad of a batch of eight edges
                phase_a(af, al);
            }
            cp_async_wait<1>();
            __syncwarp();
            phase_b(s, (in_row >> 2) & 1);
            __syncwarp(); // stage s and (after the batch's second quad) the slots are free
            issue(s, p2, j2, b0);
            if (!p1.valid || p1.row != p0.row) {
                flush(p0.row, b0);
                clear();
            }
            if (p1.valid && ((p1.e - p1.lo) & 7) == 0) {
#pragma unroll
                for (int ks = 0; ks < 4; ks++) af[ks] = af_n[ks];
                al[0] = al_n[0], al[1] = al_n[1];
            }
            p0 = p1, p1 = p2, p2 = p3, j2 = j3;
            p3 = advance(p3);
            j3 = load_j(p3);
            if (p1.valid && ((p1.e - p1.lo) & 7) == 0) load_a(p1.e, p1.hi, af_n, al_n);
            s ^= 1;
        }
        cp_async_wait<0>();
        __syncwarp();
    }
}

// VJP over quads of edges, for a sorted scatter index and compile-time widths NA = A.shape[1],
// NW = W.shape[1], NO = output_size (LL = B.shape[1] when known at compile time, else 0).
// Per batch of eight edges of one output row r (T, U in one slot per edge, cells compact):
//   phase A  T[cell, e] = sum_m D[cell, m] A[e, m]                       (as in the forward)
//   per quad X[(m2, e), b] = sum_m3 T_e[m3, m2] gO[r, m3, b]: the rows of the MMA are (m2
//            pair, edge of the quad), so nine channels fill 4.5 tiles instead of 8; a ninth
//            m3 is one multiply-add per accumulator element. grad_B[e, b] = sum_m2 X W[J_e,
//            m2, b] is summed in registers (one exchange between two lanes per quad),
//            grad_W[J_e, m2, b] += X B[e, b] goes out by RED straight from the fragments;
//            U[m3, (m2, e)] = sum_b gO[r, m3, b] (B[e, b] W[J_e, m2, b]) with the columns
//            numbered the same way (a ninth m3 again on the FMA pipe), written over T_e;
//   phase C  grad_A[e, m] = sum_cell U[e, cell] D[cell, m] for the eight edges at once.
// About 25 tensor-core instructions per edge instead of 74.
template <int NA, int NW, int NO, int LL>
__global__ void __launch_bounds__(256, 1)
sasaw_vjp_quad(double* __restrict__ gA, double* __restrict__ gB, double* __restrict__ gW,
               const double* __restrict__ gO, const double* __restrict__ A,
               const double* __restrict__ B, const double* __restrict__ W,
               const int32_t* __restrict__ Jw, const int64_t* __restrict__ offsets,
               Coupling<double> cp, int L_arg, int64_t nW0, Status st) {
    using T = double;
    constexpr QuadLayout q = quad_layout(NA, NW, NO);
    constexpr int ES = q.ES, EB = q.EB, DS = q.DS;
    constexpr int KSA = NA / 4 + (NA % 4 >= 2 ? 1 : 0); // phase A: k-steps over m1
    constexpr bool RANK_A = NA % 4 == 1;                // ... and the last component by FMA
    constexpr int NMT = (NW + 1) / 2;                   // tiles over (m2 pair, edge of the quad)
    constexpr int KS3 = NO / 4 + (NO % 4 >= 2 ? 1 : 0); // X: k-steps over m3
    constexpr bool RANK_3 = NO % 4 == 1;                // ... and the last m3 by FMA
    constexpr int MT3 = NO > 9 ? 2 : 1;                 // U: 8-row tiles over m3
    constexpr bool ROW8 = NO == 9;                      // ... and the ninth row by FMA
    constexpr int NTA = NA > 9 ? 2 : 1;                 // phase C: 8-wide tiles over m1
    constexpr bool COL8 = NA == 9;                      // ... and the ninth column by FMA
    constexpr int KC = (q.ncc + 3) / 4;                 // phase C: k-steps over the cells
    extern __shared__ __align__(16) unsigned char smem_raw[];
    if (saw_unsorted(st)) return; // the edge-by-edge kernel of the same call does the work
    const int L = LL > 0 ? LL : L_arg;
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0); // uniform for the compiler
    const int qr = lane >> 2, qc = lane & 3;
    const int qe = qr & 3, qh = qr >> 2; // as a row of an (m2 pair, edge) tile: edge, which m2
    T* D_s = reinterpret_cast<T*>(smem_raw); // [8 * nct][DS], rows >= ncc zero
    T* slots = D_s + q.d_scalars + static_cast<size_t>(q.warp_scalars) * warp; // [8][ES]
    T* stages = slots + 8 * ES;                                               // [2][4][EB]
    for (int i = threadIdx.x; i < q.d_scalars; i += blockDim.x)
        D_s[i] = i < q.ncc * DS ? cp.D[i] : T(0);
    for (int i = lane; i < q.warp_scalars; i += 32) slots[i] = T(0);
    __syncthreads();

    const int64_t total_warps = static_cast<int64_t>(gridDim.x) * warps;
    const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * warps + warp;
    const int64_t r0 = balanced_row_split(offsets, nW0, gwarp, total_warps, lane);
    const int64_t r1 = balanced_row_split(offsets, nW0, gwarp + 1, total_warps, lane);
    if (r0 >= r1) return;
    const int nrows = static_cast<int>(r1 - r0);
    const int64_t e_base = offsets[r0];
    const T* A0 = A + e_base * NA;
    const T* B0 = B + e_base * L;
    const int32_t* J0 = Jw + e_base;
    T* gA0 = gA != nullptr ? gA + e_base * NA : nullptr;
    T* gB0 = gB != nullptr ? gB + e_base * L : nullptr;
    const size_t rowsize = static_cast<size_t>(NO) * L;
    const T* gO0 = gO + r0 * rowsize;
    const int64_t w_stride = static_cast<int64_t>(NW) * L;
    const bool want_a = gA != nullptr, want_bw = gB != nullptr || gW != nullptr;

    int wbase = 0, win = 0;
    auto load_window = [&](int base) {
        const int64_t i = r0 + base + 1 + lane;
        return static_cast<int>(offsets[i < nW0 ? i : nW0] - e_base);
    };
    auto row_end = [&](int r) -> int {
        if (r - wbase >= 32) {
            wbase = r;
            win = load_window(wbase);
        }
        return __shfl_sync(kFullMask, win, r - wbase);
    };
    auto advance = [&](QuadPos p) -> QuadPos {
        if (!p.valid) return p;
        p.e += 4;
        while (p.e >= p.hi) {
            p.row++;
            if (p.row >= nrows) {
                p.valid = false;
                return p;
            }
            p.lo = p.hi;
            p.hi = row_end(p.row);
            p.e = p.lo;
        }
        return p;
    };
    auto load_j = [&](const QuadPos& p) -> int32_t {
        int32_t j = 0;
        if (p.valid && lane < 4 && p.e + lane < p.hi) {
            j = __ldg(J0 + p.e + lane);
            if (clamp_index(j, static_cast<int32_t>(nW0))) report_bad_index(st, kBitJ);
        }
        return j;
    };
    auto load_a = [&](int eb, int hi, T (&af)[4], T (&al)[2]) {
        const int ea = eb + qr;
        const T* a = A0 + static_cast<int64_t>(ea) * NA + qc;
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
            af[ks] = (ks < KSA && ea < hi && 4 * ks + qc < NA) ? __ldg(a + 4 * ks) : T(0);
        const int e2 = eb + 2 * qc;
        const T* a2 = A0 + static_cast<int64_t>(e2) * NA + NA - 1;
        al[0] = (RANK_A && e2 < hi) ? __ldg(a2) : T(0);
        al[1] = (RANK_A && e2 + 1 < hi) ? __ldg(a2 + NA) : T(0);
    };
    auto phase_a = [&](const T (&af)[4], const T (&al)[2]) {
        const T* drow = D_s + qr * DS + qc;
        T* dst = slots + (2 * qc) * ES + qr;
#pragma unroll
        for (int t = 0; t < q.nct; t++) {
            T c[2] = {T(0), T(0)};
#pragma unroll
            for (int ks = 0; ks < KSA; ks++) dmma(c, drow[t * 8 * DS + 4 * ks], af[ks]);
            if (RANK_A) {
                const T dl = drow[t * 8 * DS + NA - 1 - qc];
                c[0] = fma(dl, al[0], c[0]);
                c[1] = fma(dl, al[1], c[1]);
            }
            if (8 * t + qr < q.ncc) {
                dst[8 * t] = c[0];
                dst[8 * t + ES] = c[1];
            }
        }
    };
    auto issue = [&](int s, const QuadPos& p, int32_t j_lane, int b0) {
        if (p.valid) {
            const int col = 2 * (lane & 15);
            const bool col_ok = b0 + col < L;
            T* buf = stages + s * 4 * EB + col + (lane >> 4) * 32;
            const int src_col = b0 + (col_ok ? col : 0);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int32_t j = __shfl_sync(kFullMask, j_lane, i);
                const bool ok = col_ok && p.e + i < p.hi;
                const T* wsrc = W + j * w_stride + src_col + (lane >> 4) * L;
                const T* bsrc = B0 + static_cast<int64_t>(ok ? p.e + i : p.e) * L + src_col;
                T* dst = buf + i * EB;
                const int bytes = ok ? 16 : 0;
#pragma unroll
                for (int rr = 0; rr < (NW + 2) / 2; rr++) {
                    const int r = 2 * rr + (lane >> 4);
                    if (r <= NW)
                        cp_async16_zfill(dst + rr * 64,
                                         r < NW ? wsrc + static_cast<int64_t>(2 * rr) * L : bsrc, bytes);
                }
            }
        }
        cp_async_commit();
    };

    // grad_output fragments of the current output row and 32-wide chunk of b
    T gx[KS3 > 0 ? KS3 : 1][4]; // X: B operand gO[m3 = 4 ks + qc][b0 + 8 nt + qr]
    T gx8[4][2];                // RANK_3: gO[NO - 1][b0 + 8 nt + 2 qc + h]
    T gu[MT3][8];               // U: A operand gO[m3 = 8 mt + qr][b0 + 4 kb + qc]
    T gu8[8];                   // ROW8: gO[8][b0 + 4 kb + qc]
    auto load_g = [&](int row, int b0) {
        const T* g = gO0 + row * rowsize + b0;
        const int width = L - b0;
#pragma unroll
        for (int ks = 0; ks < KS3; ks++)
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const int m3 = 4 * ks + qc, b = 8 * nt + qr;
                gx[ks][nt] = (want_bw && m3 < NO - (RANK_3 ? 1 : 0) && b < width) ? __ldg(g + m3 * L + b) : T(0);
            }
#pragma unroll
        for (int nt = 0; nt < 4; nt++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int b = 8 * nt + 2 * qc + h;
                gx8[nt][h] = (RANK_3 && want_bw && b < width) ? __ldg(g + (NO - 1) * L + b) : T(0);
            }
#pragma unroll
        for (int mt = 0; mt < MT3; mt++)
#pragma unroll
            for (int kb = 0; kb < 8; kb++) {
                const int m3 = 8 * mt + qr, b = 4 * kb + qc;
                gu[mt][kb] = (want_a && m3 < NO - (ROW8 ? 1 : 0) && b < width) ? __ldg(g + m3 * L + b) : T(0);
            }
#pragma unroll
        for (int kb = 0; kb < 8; kb++) {
            const int b = 4 * kb + qc;
            gu8[kb] = (ROW8 && want_a && b < width) ? __ldg(g + 8 * L + b) : T(0);
        }
    };

    for (int b0 = 0; b0 < L; b0 += 32) {
        const int width = L - b0;
        wbase = 0;
        win = load_window(0);
        QuadPos start;
        start.row = -1, start.valid = true;
        start.lo = start.hi = 0;
        start.e = -4;
        QuadPos p0 = advance(start);
        QuadPos p1 = advance(p0), p2 = advance(p1), p3 = advance(p2);
        int32_t j0 = load_j(p0), j1 = load_j(p1), j2 = load_j(p2), j3 = load_j(p3);
        issue(0, p0, j0, b0);
        issue(1, p1, j1, b0);
        T af[4], al[2], af_n[4], al_n[2];
        if (p0.valid) load_a(p0.e, p0.hi, af, al);
        if (p1.valid && ((p1.e - p1.lo) & 7) == 0) load_a(p1.e, p1.hi, af_n, al_n);
        int s = 0, cur_row = -1;
        while (p0.valid) {
            const int in_row = p0.e - p0.lo;
            const int qi = (in_row >> 2) & 1; // which quad of the batch
            if ((in_row & 7) == 0 && want_bw) phase_a(af, al);
            cp_async_wait<1>();
            __syncwarp();
            if (p0.row != cur_row) {
                load_g(p0.row, b0);
                cur_row = p0.row;
            }
            const T* stage = stages + s * 4 * EB;
            const int my_e = p0.e + qe;        // this lane's edge as a tile row / column
            const bool ev = my_e < p0.hi;
            const int32_t jq = __shfl_sync(kFullMask, j0, qe);

            if (want_bw) {
                const T* tb = slots + (4 * qi + qe) * ES + qc * NW + qh; // + 4 ks NW + 2 mt
                const T* t8 = slots + (4 * qi + qe) * ES + (NO - 1) * NW + qh;
                const T* wv = stage + qe * EB + qh * 32 + 2 * qc; // + 2 mt * 32 + 8 nt
                const T* bv = stage + qe * EB + NW * 32 + 2 * qc; // + 8 nt
                T* gwp = gW != nullptr
                             ? gW + jq * w_stride + static_cast<int64_t>(qh) * L + b0 + 2 * qc
                             : nullptr;
                T gb[4][2], b2[4][2];
#pragma unroll
                for (int nt = 0; nt < 4; nt++) {
                    const double2 v = *reinterpret_cast<const double2*>(bv + 8 * nt);
                    b2[nt][0] = v.x, b2[nt][1] = v.y;
                    gb[nt][0] = gb[nt][1] = T(0);
                }
#pragma unroll
                for (int mt = 0; mt < NMT; mt++) {
                    const bool m2_ok = 2 * mt + 1 < NW || qh == 0; // lane's m2 = 2 mt + qh
                    T a[KS3 > 0 ? KS3 : 1];
#pragma unroll
                    for (int ks = 0; ks < KS3; ks++)
                        a[ks] = (m2_ok && 4 * ks + qc < NO - (RANK_3 ? 1 : 0)) ? tb[4 * ks * NW + 2 * mt] : T(0);
                    const T a8 = (RANK_3 && m2_ok) ? t8[2 * mt] : T(0);
#pragma unroll
                    for (int nt = 0; nt < 4; nt++) {
                        T c[2] = {T(0), T(0)};
#pragma unroll
                        for (int ks = 0; ks < KS3; ks++) dmma(c, a[ks], gx[ks][nt]);
                        if (RANK_3) {
                            c[0] = fma(a8, gx8[nt][0], c[0]);
                            c[1] = fma(a8, gx8[nt][1], c[1]);
                        }
                        const int b = 8 * nt + 2 * qc;
                        if (m2_ok) {
                            const double2 w2 = *reinterpret_cast<const double2*>(wv + 2 * mt * 32 + 8 * nt);
                            gb[nt][0] = fma(c[0], w2.x, gb[nt][0]);
                            gb[nt][1] = fma(c[1], w2.y, gb[nt][1]);
                            if (gwp != nullptr && ev) {
                                T* gw = gwp + static_cast<int64_t>(2 * mt) * L + 8 * nt;
                                if (b < width) red_add(gw, c[0] * b2[nt][0]);
                                if (b + 1 < width) red_add(gw + 1, c[1] * b2[nt][1]);
                            }
                        }
                    }
                }
                if (gB0 != nullptr) {
                    // lanes qh = 0 and qh = 1 hold the two halves of the sum over m2: exchange,
                    // so that qh = 0 ends with nt = 0, 1 and qh = 1 with nt = 2, 3
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        T v[2];
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const T keep = qh ? gb[2 + i][h] : gb[i][h];
                            const T send = qh ? gb[i][h] : gb[2 + i][h];
                            v[h] = keep + __shfl_xor_sync(kFullMask, send, 16);
                        }
                        const int b = 8 * (2 * qh + i) + 2 * qc;
                        T* dst = gB0 + static_cast<int64_t>(my_e) * L + b0 + b;
                        if (ev && b + 1 < width)
                            *reinterpret_cast<double2*>(dst) = make_double2(v[0], v[1]);
                        else if (ev && b < width)
                            dst[0] = v[0];
                    }
                }
            }
            __syncwarp(); // every lane has read T of this quad: the slots may take U
            if (want_a) {
                const T* wu = stage + qe * EB + qh * 32 + qc; // + 2 nt * 32 + 4 kb
                const T* bu = stage + qe * EB + NW * 32 + qc; // + 4 kb
                T bbu[8];
#pragma unroll
                for (int kb = 0; kb < 8; kb++) bbu[kb] = bu[4 * kb];
                // column n = 2 qc + h of tile nt is (edge 2 (qc & 1) + h, m2 = 2 nt + (qc >> 1))
                T* us = slots + (4 * qi + 2 * (qc & 1)) * ES + qr * NW + (qc >> 1);
#pragma unroll
                for (int nt = 0; nt < NMT; nt++) {
                    T u[MT3][2], u8 = T(0);
#pragma unroll
                    for (int mt = 0; mt < MT3; mt++) u[mt][0] = u[mt][1] = T(0);
#pragma unroll
                    for (int kb = 0; kb < 8; kb++) {
                        const T bw = wu[2 * nt * 32 + 4 * kb] * bbu[kb];
#pragma unroll
                        for (int mt = 0; mt < MT3; mt++) dmma(u[mt], gu[mt][kb], bw);
                        if (ROW8) u8 = fma(gu8[kb], bw, u8);
                    }
                    const bool col_ok = 2 * nt + 1 < NW || (qc >> 1) == 0;
#pragma unroll
                    for (int mt = 0; mt < MT3; mt++) {
                        if (col_ok && 8 * mt + qr < NO - (ROW8 ? 1 : 0)) {
                            us[8 * mt * NW + 2 * nt] = u[mt][0];
                            us[8 * mt * NW + 2 * nt + ES] = u[mt][1];
                        }
                    }
                    if (ROW8) {
                        u8 += __shfl_xor_sync(kFullMask, u8, 1);
                        u8 += __shfl_xor_sync(kFullMask, u8, 2);
                        // the lane's column as the B operand: edge qe, m2 = 2 nt + qh
                        if (qc == 0 && (2 * nt + 1 < NW || qh == 0))
                            slots[(4 * qi + qe) * ES + 8 * NW + 2 * nt + qh] = u8;
                    }
                }
            }
            __syncwarp(); // stage s is free; U of this quad is in the slots
            issue(s, p2, j2, b0);
            const bool batch_end = !p1.valid || ((p1.e - p1.lo) & 7) == 0;
            if (want_a && batch_end) {
                // grad_A[e, m] = sum_cell U[e, cell] D[cell, m] for the batch's eight edges
                T ga[NTA][2], ga8 = T(0);
#pragma unroll
                for (int nt = 0; nt < NTA; nt++) ga[nt][0] = ga[nt][1] = T(0);
                const T* ur = slots + qr * ES + qc;
                const T* dc = D_s + qc * DS + qr;
#pragma unroll 7
                for (int kc = 0; kc < KC; kc++) {
                    const T au = ur[4 * kc];
#pragma unroll
                    for (int nt = 0; nt < NTA; nt++) dmma(ga[nt], au, dc[4 * kc * DS + 8 * nt]);
                    if (COL8) ga8 = fma(au, D_s[(4 * kc + qc) * DS + 8], ga8);
                }
                const int eb = p0.e - (in_row & 4);
                const bool ok = eb + qr < p0.hi;
                T* dst = gA0 + static_cast<int64_t>(eb + qr) * NA;
#pragma unroll
                for (int nt = 0; nt < NTA; nt++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const int m = 8 * nt + 2 * qc + h;
                        if (ok && m < NA - (COL8 ? 1 : 0))
                            dst[m] = b0 > 0 ? dst[m] + ga[nt][h] : ga[nt][h];
                    }
                if (COL8) {
                    ga8 += __shfl_xor_sync(kFullMask, ga8, 1);
                    ga8 += __shfl_xor_sync(kFullMask, ga8, 2);
                    if (ok && qc == 0) dst[8] = b0 > 0 ? dst[8] + ga8 : ga8;
                }
                __syncwarp(); // the slots are rewritten by the next batch's phase A
            }
            if (p1.valid && ((p1.e - p1.lo) & 7) == 0) {
#pragma unroll
                for (int ks = 0; ks < 4; ks++) af[ks] = af_n[ks];
                al[0] = al_n[0], al[1] = al_n[1];
            }
            p0 = p1, p1 = p2, p2 = p3;
            j0 = j1, j1 = j2, j2 = j3;
            p3 = advance(p3);
            j3 = load_j(p3);
            if (p1.valid && ((p1.e - p1.lo) & 7) == 0) load_a(p1.e, p1.hi, af_n, al_n);
            s ^= 1;
        }
        cp_async_wait<0>();
        __syncwarp();
    }
}

// Any sizes, no shared memory: one thread per (edge, b) walking the whole coupling table.
// Needs zero-filled O (forward) / gA, gW (VJP).
template <typename T>
__global__ void sasaw_fwd_wide(T* __restrict__ O, const T* __restrict__ A, const T* __restrict__ B,
                               const T* __restrict__ C, const T* __restrict__ W,
                               const int32_t* __restrict__ M1, const int32_t* __restrict__ Jw,
                               const int32_t* __restrict__ M2, const int32_t* __restrict__ Io,
                               const int32_t* __restrict__ M3, int64_t E, int nA, int L, int N,
                               int64_t nW0, int nW1, int nO1, Status st) {
    const int64_t total = E * L;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t e = i / L;
        const int b = static_cast<int>(i - e * L);
        int32_t row = __ldg(Io + e), j = __ldg(Jw + e);
        if (clamp_index(row, static_cast<int32_t>(nW0))) { report_bad_index(st, kBitI); continue; }
        if (clamp_index(j, static_cast<int32_t>(nW0))) { report_bad_index(st, kBitJ); continue; }
        const T Bb = B[i];
        for (int n = 0; n < N; n++) {
            int32_t m1 = __ldg(M1 + n), m2 = __ldg(M2 + n), m3 = __ldg(M3 + n);
            const bool b1 = clamp_index(m1, nA), b2 = clamp_index(m2, nW1), b3 = clamp_index(m3, nO1);
            if (b1 || b2 || b3) {
                if (b1) report_bad_index(st, kBitM1);
                if (b2) report_bad_index(st, kBitM2);
                if (b3) report_bad_index(st, kBitM3);
                continue;
            }
            const T v = __ldg(C + n) * A[e * nA + m1] * Bb *
                        __ldg(W + (static_cast<int64_t>(j) * nW1 + m2) * L + b);
            red_add(O + (static_cast<int64_t>(row) * nO1 + m3) * L + b, v);
        }
    }
}

template <typename T>
__global__ void sasaw_vjp_wide(T* __restrict__ gA, T* __restrict__ gB, T* __restrict__ gW,
                               const T* __restrict__ gO, const T* __restrict__ A,
                               const T* __restrict__ B, const T* __restrict__ C,
                               const T* __restrict__ W, const int32_t* __restrict__ M1,
                               const int32_t* __restrict__ Jw, const int32_t* __restrict__ M2,
                               const int32_t* __restrict__ Io, const int32_t* __restrict__ M3,
                               int64_t E, int nA, int L, int N, int64_t nW0, int nW1, int nO1,
                               Status st) {
    const int64_t total = E * L;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t e = i / L;
        const int b = static_cast<int>(i - e * L);
        int32_t row = __ldg(Io + e), j = __ldg(Jw + e);
        if (clamp_index(row, static_cast<int32_t>(nW0))) report_bad_index(st, kBitI);
        if (clamp_index(j, static_cast<int32_t>(nW0))) report_bad_index(st, kBitJ);
        const T Bb = B[i];
        T gb = T(0);
        for (int n = 0; n < N; n++) {
            int32_t m1 = __ldg(M1 + n), m2 = __ldg(M2 + n), m3 = __ldg(M3 + n);
            const bool b1 = clamp_index(m1, nA), b2 = clamp_index(m2, nW1), b3 = clamp_index(m3, nO1);
            if (b1 || b2 || b3) {
                if (b1) report_bad_index(st, kBitM1);
                if (b2) report_bad_index(st, kBitM2);
                if (b3) report_bad_index(st, kBitM3);
                continue;
            }
            const T c = __ldg(C + n), a = A[e * nA + m1];
            const T gv = __ldg(gO + (static_cast<int64_t>(row) * nO1 + m3) * L + b);
            const int64_t wi = (static_cast<int64_t>(j) * nW1 + m2) * L + b;
            const T wv = __ldg(W + wi);
            if (gA != nullptr) red_add(gA + e * nA + m1, gv * c * Bb * wv);
            gb += gv * c * a * wv;
            if (gW != nullptr) red_add(gW + wi, gv * c * a * Bb);
        }
        if (gB != nullptr) gB[i] = gb;
    }
}

template <typename T> struct Problem {
    const T *A, *B, *C, *W;
    const int32_t *M1, *Jw, *M2, *Io, *M3;
    int64_t E, nW0;
    int nA, L, N, nW1, nO1;
};

// Allocates and fills the grouped coupling table; returns false when the grouped kernels
// cannot be used (cell grid too large for one block's shared memory).
template <typename T>
bool build_coupling(const Call& call, const Problem<T>& p, Coupling<T>& cp, TableRef* table,
                    int cell_stride = 0, int d_stride = 0, bool d_padded = false) {
    if (cell_stride == 0) cell_stride = p.nW1;
    const int64_t ncell64 = static_cast<int64_t>(p.nO1) * cell_stride;
    if (ncell64 > 8192 || ncell64 == 0) return false;
    cp.N = p.N;
    cp.ncell = static_cast<int>(ncell64);
    const size_t nT = (static_cast<size_t>(p.N) * sizeof(T) + 15) / 16 * 16;
    const size_t nI = static_cast<size_t>(p.N) * sizeof(int32_t);
    const size_t nStart = ((cp.ncell + 1) * sizeof(int32_t) + 15) / 16 * 16;
    const size_t nD =
        static_cast<size_t>(d_stride) * p.nO1 * (d_padded ? cell_stride : p.nW1) * sizeof(T);
    const size_t bytes = nT + 3 * nI + nStart + 16 + nD;
    TableKey key{};
    key.kind = kSasawCouplingTable;
    key.scalar_bytes = static_cast<int>(sizeof(T));
    key.ptr[0] = p.C, key.ptr[1] = p.M1, key.ptr[2] = p.M2, key.ptr[3] = p.M3;
    key.n[0] = p.N, key.n[1] = p.nA, key.n[2] = p.nW1, key.n[3] = p.nO1;
    key.n[4] = cell_stride, key.n[5] = d_stride, key.n[6] = d_padded ? 1 : 0;
    *table = acquire_table(call, key, bytes);
    unsigned char* base = static_cast<unsigned char*>(table->ptr);
    cp.d_stride = d_stride;
    cp.d_padded = d_padded;
    cp.D = d_stride > 0
               ? reinterpret_cast<T*>(base + (nT + 3 * nI + nStart + 15) / 16 * 16)
               : nullptr;
    cp.C = reinterpret_cast<T*>(base);
    cp.M1 = reinterpret_cast<int32_t*>(base + nT);
    cp.cell = cp.M1 + p.N;
    cp.order = cp.cell + p.N;
    cp.start = cp.order + p.N;
    if (table->fresh) {
        sasaw_group_coupling<T><<<1, kBuildThreads, cp.ncell * sizeof(int32_t), call.stream>>>(
            cp, p.C, p.M1, p.M2, p.M3, p.nA, p.nW1, p.nO1, call.status);
        MOPS_CUDA_OK(cudaGetLastError());
        commit_table(call, *table);
    }
    return true;
}

template <typename T>
size_t block_smem(const Coupling<T>& cp, size_t per_warp_scalars, int warps, bool with_cell) {
    return (static_cast<size_t>(cp.N) + per_warp_scalars * warps) * sizeof(T) +
           (static_cast<size_t>(cp.N) * (with_cell ? 2 : 1) + cp.ncell + 1) * sizeof(int32_t);
}

// Largest warp count (8, 4, 2, 1) whose shared memory fits; 0 if none does.
template <typename T>
int pick_warps(const Call& call, const Coupling<T>& cp, size_t per_warp_scalars, bool with_cell,
               size_t* smem) {
    for (int warps : {8, 4, 2, 1}) {
        const size_t bytes = block_smem(cp, per_warp_scalars, warps, with_cell);
        const size_t limit = warps == 1 ? static_cast<size_t>(max_optin_smem(call.device)) : 100 * 1024;
        if (bytes <= limit) {
            *smem = bytes;
            return warps;
        }
    }
    return 0;
}

template <typename Kernel> void allow_smem(Kernel kernel, size_t smem) {
    if (smem > 48 * 1024)
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
}

// Shared memory of a fast-kernel block, and the largest warp count (8, 4, 2, 1) that fits.
template <typename T>
int pick_warps_fast(const Call& call, int ncc, int ds, size_t per_warp, size_t* smem) {
    for (int warps : {8, 4, 2, 1}) {
        const size_t bytes = (round4(static_cast<size_t>(ncc) * ds) + per_warp * warps) * sizeof(T) +
                             static_cast<size_t>(ncc) * sizeof(int32_t);
        const size_t limit = warps == 1 ? static_cast<size_t>(max_optin_smem(call.device)) : 100 * 1024;
        if (bytes <= limit) {
            *smem = bytes;
            return warps;
        }
    }
    return 0;
}

// Padded widths used by the fast kernels (0: not applicable).
inline int fast_width(int n) { return n >= 1 && n <= 16 ? (n + 3) / 4 * 4 : 0; }

template <typename T, int TP, int NAP>
bool forward_fast(const Call& call, T* O, const Problem<T>& p) {
    const int64_t rowsize = static_cast<int64_t>(p.nO1) * p.L;
    const int ncc = p.nO1 * p.nW1, ds = NAP + 1; // odd row stride: conflict-free row-per-lane reads
    if (static_cast<int64_t>(p.nO1) * p.nW1 > 1024) return false;
    const int grid_generic = sm_count(call.device) * 8;
    size_t smem_seg = 0, smem_edge = 0;
    const size_t tsize = round4(static_cast<size_t>(p.nO1) * TP);
    const int warps_seg = pick_warps_fast<T>(call, ncc, ds, tsize + round4(rowsize), &smem_seg);
    const int warps_edge = pick_warps_fast<T>(call, ncc, ds, tsize, &smem_edge);
    if (warps_seg == 0 || warps_edge == 0) return false;
    Coupling<T> cp{};
    TableRef scratch{};
    if (!build_coupling(call, p, cp, &scratch, TP, ds)) return false;
    SegmentTable seg = segment_table(call, p.Io, p.E, p.nW0);
    const int64_t* offsets = seg.offsets;
    allow_smem(sasaw_fwd_fast<T, TP, NAP, true>, smem_seg);
    note_kernel_f("sasaw_fwd_fast<%s,TP=%d,NAP=%d>", scalar_name<T>(), TP, NAP);
    sasaw_fwd_fast<T, TP, NAP, true><<<static_cast<unsigned>(ceil_div(p.nW0, warps_seg)),
                                       warps_seg * 32, smem_seg, call.stream>>>(
        O, p.A, p.B, p.W, p.Jw, p.Io, offsets, cp, p.E, p.nA, p.L, p.nW0, p.nW1, p.nO1, false,
        call.status);
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, seg.ref);
    bool need_fallback = !seg.known_sorted; // asynchronous calls cannot look: always enqueue
    if (need_fallback && call.wait) {
        wait_stream(call);
        need_fallback = host_saw_unsorted(call);
    }
    if (need_fallback) {
        zero_if_unsorted<T><<<grid_generic, 256, 0, call.stream>>>(O, p.nW0 * rowsize, call.status);
        allow_smem(sasaw_fwd_fast<T, TP, NAP, false>, smem_edge);
        const int64_t blocks = std::min<int64_t>(ceil_div(p.E, warps_edge), grid_generic);
        sasaw_fwd_fast<T, TP, NAP, false><<<static_cast<unsigned>(blocks), warps_edge * 32,
                                            smem_edge, call.stream>>>(
            O, p.A, p.B, p.W, p.Jw, p.Io, nullptr, cp, p.E, p.nA, p.L, p.nW0, p.nW1, p.nO1, false,
            call.status);
    }
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, scratch);
    return true;
}

template <typename T, int TP, int NAP>
bool backward_fast(const Call& call, T* gA, T* gB, T* gW, const T* gO, const Problem<T>& p) {
    const int ncc = p.nO1 * p.nW1, ds = NAP + 1;
    if (static_cast<int64_t>(p.nO1) * p.nW1 > 1024) return false;
    size_t smem = 0;
    const int warps =
        pick_warps_fast<T>(call, ncc, ds, 2 * round4(static_cast<size_t>(p.nO1) * TP), &smem);
    if (warps == 0) return false;
    Coupling<T> cp{};
    TableRef scratch{};
    if (!build_coupling(call, p, cp, &scratch, TP, ds)) return false;
    allow_smem(sasaw_vjp_fast<T, TP, NAP>, smem);
    note_kernel_f("sasaw_vjp_fast<%s,TP=%d,NAP=%d>", scalar_name<T>(), TP, NAP);
    const int64_t blocks =
        std::min<int64_t>(ceil_div(p.E, warps), static_cast<int64_t>(sm_count(call.device)) * 16);
    sasaw_vjp_fast<T, TP, NAP><<<static_cast<unsigned>(blocks), warps * 32, smem, call.stream>>>(
        gA, gB, gW, gO, p.A, p.B, p.W, p.Jw, p.Io, cp, p.E, p.nA, p.L, p.nW0, p.nW1, p.nO1,
        call.status);
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, scratch);
    return true;
}

// Tensor-core variants (f64, output_size <= 16 as well).
// `segmented_done`: another kernel has already handled sorted input; only the kernels for an
// unsorted scatter index are enqueued (they stand down by themselves when it was sorted).
template <typename T, int TP>
bool forward_mma_launch(const Call& call, T* O, const Problem<T>& p, bool segmented_done = false) {
    using Lay = VjpMma<TP>;
    const int warps = 4;
    const size_t smem =
        (Lay::d_scalars(p.nO1, p.nA) + Lay::per_warp(p.nO1, p.nW1) * warps) * sizeof(T);
    if (smem > 74 * 1024) return false; // three blocks per SM
    const int64_t rowsize = static_cast<int64_t>(p.nO1) * p.L;
    const int sms = sm_count(call.device);
    Coupling<T> cp{};
    TableRef scratch{};
    if (!build_coupling(call, p, cp, &scratch, Lay::TS, Lay::d_stride(p.nA), true)) return false;
    const bool wide_copies = p.L % 2 == 0 && reinterpret_cast<uintptr_t>(p.W) % 16 == 0 &&
                             reinterpret_cast<uintptr_t>(p.B) % 16 == 0 &&
                             reinterpret_cast<uintptr_t>(O) % 16 == 0;
    bool known_sorted = false;
    if (!segmented_done) {
        SegmentTable seg = segment_table(call, p.Io, p.E, p.nW0);
        const int64_t* offsets = seg.offsets;
        known_sorted = seg.known_sorted;
        allow_smem(sasaw_fwd_mma<TP, true>, smem);
        note_kernel_f("sasaw_fwd_mma<TP=%d,SEG=1>", TP);
        const int64_t seg_blocks = std::min<int64_t>(ceil_div(p.nW0, warps), sms * 3);
        sasaw_fwd_mma<TP, true><<<static_cast<unsigned>(seg_blocks), warps * 32, smem,
                                  call.stream>>>(O, p.A, p.B, p.W, p.Jw, p.Io, offsets, cp, p.E,
                                                 p.nA, p.L, p.nW0, p.nW1, p.nO1, wide_copies,
                                                 call.status);
        MOPS_CUDA_OK(cudaGetLastError());
        release_table(call, seg.ref);
    }
    bool need_fallback = !known_sorted; // asynchronous calls cannot look: always enqueue
    if (need_fallback && call.wait && !segmented_done) {
        wait_stream(call);
        need_fallback = host_saw_unsorted(call);
    }
    if (need_fallback) {
        zero_if_unsorted<T><<<sms * 8, 256, 0, call.stream>>>(O, p.nW0 * rowsize, call.status);
        allow_smem(sasaw_fwd_mma<TP, false>, smem);
        const int64_t blocks = std::min<int64_t>(ceil_div(ceil_div(p.E, 8), warps), sms * 3);
        sasaw_fwd_mma<TP, false><<<static_cast<unsigned>(blocks), warps * 32, smem, call.stream>>>(
            O, p.A, p.B, p.W, p.Jw, p.Io, nullptr, cp, p.E, p.nA, p.L, p.nW0, p.nW1, p.nO1,
            wide_copies, call.status);
    }
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, scratch);
    return true;
}

inline int env_flag(const char* name, int fallback) {
    const char* v = std::getenv(name);
    return v != nullptr && *v != '\0' ? std::atoi(v) : fallback;
}

// Sorted scatter index through the quad kernel. Returns 0 when it does not apply, 1 when it
// ran and the index was seen to be sorted (nothing left to do), 2 when it was launched but
// the kernels for unsorted input must still be enqueued (asynchronous call, or the index
// turned out unsorted).
template <typename T> int forward_quad(const Call& call, T* O, const Problem<T>& p) {
    if constexpr (!std::is_same<T, double>::value) {
        return 0;
    } else {
        // (MOPS_B200_SASAW_QUAD=0: development switch back to the batch-of-eight kernels)
        if (env_flag("MOPS_B200_SASAW_QUAD", 1) == 0) return 0;
        auto aligned = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
        if (p.L % 2 != 0 || !aligned(p.W) || !aligned(p.B) || !aligned(O)) return 0;
        const QuadLayout q = quad_layout(p.nA, p.nW1, p.nO1);
        const size_t d_bytes = static_cast<size_t>(q.d_scalars) * sizeof(T);
        const size_t warp_bytes = static_cast<size_t>(q.warp_scalars) * sizeof(T);
        const size_t limit = static_cast<size_t>(max_optin_smem(call.device));
        if (d_bytes + 2 * warp_bytes > limit) return 0;
        const int warps = static_cast<int>(std::min<size_t>(8, (limit - d_bytes) / warp_bytes));
        const size_t smem = d_bytes + warps * warp_bytes;
        const int sms = sm_count(call.device);
        Coupling<T> cp{};
        TableRef scratch{};
        if (!build_coupling(call, p, cp, &scratch, p.nW1, q.DS, false)) return 0;
        SegmentTable seg = segment_table(call, p.Io, p.E, p.nW0);
    const int64_t* offsets = seg.offsets;
        const int mode = p.nO1 <= 8 ? 0 : (p.nO1 == 9 ? 1 : 2);
        const unsigned blocks = static_cast<unsigned>(std::min<int64_t>(ceil_div(p.nW0, warps), sms));
        const bool fixed = p.nA == p.nW1 && p.nA == p.nO1 && (p.nA == 4 || p.nA == 9 || p.nA == 16);
        note_kernel_f("sasaw_fwd_quad<MODE=%d,%s> warps=%d", mode, fixed ? "fixed widths" : "any widths", warps);
#define MOPS_B200_CASE(MODE_, NA_, NW_, NO_)                                                       \
    {                                                                                              \
        allow_smem(sasaw_fwd_quad<MODE_, NA_, NW_, NO_>, smem);                                    \
        sasaw_fwd_quad<MODE_, NA_, NW_, NO_><<<blocks, warps * 32, smem, call.stream>>>(           \
            O, p.A, p.B, p.W, p.Jw, offsets, cp, p.E, p.nA, p.L, p.nW0, p.nW1, p.nO1, call.status); \
    }
        // the widths of l <= 1, 2, 3 spherical-harmonic channels are compiled in
        if (p.nA == 9 && p.nW1 == 9 && p.nO1 == 9) MOPS_B200_CASE(1, 9, 9, 9)
        else if (p.nA == 4 && p.nW1 == 4 && p.nO1 == 4) MOPS_B200_CASE(0, 4, 4, 4)
        else if (p.nA == 16 && p.nW1 == 16 && p.nO1 == 16) MOPS_B200_CASE(2, 16, 16, 16)
        else if (mode == 0) MOPS_B200_CASE(0, 0, 0, 0)
        else if (mode == 1) MOPS_B200_CASE(1, 0, 0, 0)
        else MOPS_B200_CASE(2, 0, 0, 0)
#undef MOPS_B200_CASE
        MOPS_CUDA_OK(cudaGetLastError());
        release_table(call, seg.ref);
        release_table(call, scratch);
        if (seg.known_sorted) return 1;
        if (call.wait) {
            wait_stream(call);
            if (!host_saw_unsorted(call)) return 1;
        }
        return 2;
    }
}

template <typename T> bool forward_mma(const Call& call, T* O, const Problem<T>& p) {
    if constexpr (!std::is_same<T, double>::value) {
        return false;
    } else {
        if (fast_width(p.nO1) == 0 || fast_width(p.nA) == 0 || fast_width(p.nW1) == 0)
            return false;
        const int quad = forward_quad(call, O, p);
        if (quad == 1) return true;
        switch (fast_width(p.nW1)) {
        case 4: return forward_mma_launch<T, 4>(call, O, p, quad == 2);
        case 8: return forward_mma_launch<T, 8>(call, O, p, quad == 2);
        case 12: return forward_mma_launch<T, 12>(call, O, p, quad == 2);
        case 16: return forward_mma_launch<T, 16>(call, O, p, quad == 2);
        default: return false;
        }
    }
}

template <typename T, int TP, int KS3>
bool backward_mma_launch(const Call& call, T* gA, T* gB, T* gW, const T* gO, const Problem<T>& p,
                         bool only_if_unsorted) {
    using Lay = VjpMma<TP>;
    const int warps = 4;
    const size_t smem =
        (Lay::d_scalars(p.nO1, p.nA) + Lay::per_warp(p.nO1, p.nW1) * warps) * sizeof(T);
    if (smem > 74 * 1024) return false; // three blocks per SM
    Coupling<T> cp{};
    TableRef scratch{};
    if (!build_coupling(call, p, cp, &scratch, Lay::TS, Lay::d_stride(p.nA), true)) return false;
    allow_smem(sasaw_vjp_mma<TP, KS3>, smem);
    if (!only_if_unsorted) note_kernel_f("sasaw_vjp_mma<TP=%d,KS3=%d>", TP, KS3);
    const bool wide_copies = p.L % 2 == 0 && reinterpret_cast<uintptr_t>(p.W) % 16 == 0 &&
                             reinterpret_cast<uintptr_t>(p.B) % 16 == 0;
    const int64_t blocks = std::min<int64_t>(ceil_div(ceil_div(p.E, 8), warps),
                                             static_cast<int64_t>(sm_count(call.device)) * 3);
    sasaw_vjp_mma<TP, KS3><<<static_cast<unsigned>(blocks), warps * 32, smem, call.stream>>>(
        gA, gB, gW, gO, p.A, p.B, p.W, p.Jw, p.Io, cp, p.E, p.nA, p.L, p.nW0, p.nW1, p.nO1,
        wide_copies, only_if_unsorted, call.status);
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, scratch);
    return true;
}

// VJP through the quad kernel (sorted scatter index, compiled-in widths). Returns 0 when it
// does not apply, 1 when it ran and the index was seen to be sorted, 2 when it was launched
// but the edge-by-edge kernel must still be enqueued for the unsorted case.
template <typename T>
int backward_quad(const Call& call, T* gA, T* gB, T* gW, const T* gO, const Problem<T>& p) {
    if constexpr (!std::is_same<T, double>::value) {
        return 0;
    } else {
        if (env_flag("MOPS_B200_SASAW_QUAD", 1) == 0) return 0;
        if (!(p.nA == 9 && p.nW1 == 9 && p.nO1 == 9)) return 0;
        auto aligned = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
        if (p.L % 2 != 0 || !aligned(p.W) || !aligned(p.B) || !aligned(gB)) return 0;
        constexpr QuadLayout q = quad_layout(9, 9, 9);
        const size_t d_bytes = static_cast<size_t>(q.d_scalars) * sizeof(T);
        const size_t warp_bytes = static_cast<size_t>(q.warp_scalars) * sizeof(T);
        const size_t limit = static_cast<size_t>(max_optin_smem(call.device));
        if (d_bytes + 2 * warp_bytes > limit) return 0;
        const int warps = static_cast<int>(std::min<size_t>(8, (limit - d_bytes) / warp_bytes));
        const size_t smem = d_bytes + warps * warp_bytes;
        const int sms = sm_count(call.device);
        Coupling<T> cp{};
        TableRef scratch{};
        if (!build_coupling(call, p, cp, &scratch, p.nW1, q.DS, false)) return 0;
        SegmentTable seg = segment_table(call, p.Io, p.E, p.nW0);
    const int64_t* offsets = seg.offsets;
        const unsigned blocks = static_cast<unsigned>(std::min<int64_t>(ceil_div(p.nW0, warps), sms));
        note_kernel_f("sasaw_vjp_quad<9,9,9,L=%d> warps=%d", p.L == 32 ? 32 : 0, warps);
        if (p.L == 32) {
            allow_smem(sasaw_vjp_quad<9, 9, 9, 32>, smem);
            sasaw_vjp_quad<9, 9, 9, 32><<<blocks, warps * 32, smem, call.stream>>>(
                gA, gB, gW, gO, p.A, p.B, p.W, p.Jw, offsets, cp, p.L, p.nW0, call.status);
        } else {
            allow_smem(sasaw_vjp_quad<9, 9, 9, 0>, smem);
            sasaw_vjp_quad<9, 9, 9, 0><<<blocks, warps * 32, smem, call.stream>>>(
                gA, gB, gW, gO, p.A, p.B, p.W, p.Jw, offsets, cp, p.L, p.nW0, call.status);
        }
        MOPS_CUDA_OK(cudaGetLastError());
        release_table(call, seg.ref);
        release_table(call, scratch);
        if (seg.known_sorted) return 1;
        if (call.wait) {
            wait_stream(call);
            if (!host_saw_unsorted(call)) return 1;
        }
        return 2;
    }
}

// Tensor-core VJP: f64, A.shape[1], W.shape[1] and output_size all between 1 and 16.
template <typename T>
bool backward_mma(const Call& call, T* gA, T* gB, T* gW, const T* gO, const Problem<T>& p) {
    if constexpr (!std::is_same<T, double>::value) {
        return false;
    } else {
        const int tp = fast_width(p.nW1), op = fast_width(p.nO1);
        if (tp == 0 || op == 0 || fast_width(p.nA) == 0) return false;
        const int quad = backward_quad(call, gA, gB, gW, gO, p);
        if (quad == 1) return true;
        const bool rest = quad == 2; // only what the quad kernel left: an unsorted index
        switch (tp * 100 + op) {
#define MOPS_B200_CASE(TP_, OP_)                                                                   \
    case TP_ * 100 + OP_:                                                                          \
        return backward_mma_launch<T, TP_, OP_ / 4>(call, gA, gB, gW, gO, p, rest);
            MOPS_B200_CASE(4, 4) MOPS_B200_CASE(4, 8) MOPS_B200_CASE(4, 12) MOPS_B200_CASE(4, 16)
            MOPS_B200_CASE(8, 4) MOPS_B200_CASE(8, 8) MOPS_B200_CASE(8, 12) MOPS_B200_CASE(8, 16)
            MOPS_B200_CASE(12, 4) MOPS_B200_CASE(12, 8) MOPS_B200_CASE(12, 12) MOPS_B200_CASE(12, 16)
            MOPS_B200_CASE(16, 4) MOPS_B200_CASE(16, 8) MOPS_B200_CASE(16, 12) MOPS_B200_CASE(16, 16)
#undef MOPS_B200_CASE
        default: return false;
        }
    }
}

// Dispatch on the two padded widths; returns false when the fast kernels do not apply.
#define MOPS_B200_SASAW_FAST(FN, ...)                                                              \
    [&]() -> bool {                                                                                \
        const int tp = fast_width(p.nW1), nap = fast_width(p.nA);                                  \
        if (tp == 0 || nap == 0) return false;                                                     \
        switch (tp * 100 + nap) {                                                                  \
        case 404: return FN<T, 4, 4>(__VA_ARGS__);                                                 \
        case 408: return FN<T, 4, 8>(__VA_ARGS__);                                                 \
        case 412: return FN<T, 4, 12>(__VA_ARGS__);                                                \
        case 416: return FN<T, 4, 16>(__VA_ARGS__);                                                \
        case 804: return FN<T, 8, 4>(__VA_ARGS__);                                                 \
        case 808: return FN<T, 8, 8>(__VA_ARGS__);                                                 \
        case 812: return FN<T, 8, 12>(__VA_ARGS__);                                                \
        case 816: return FN<T, 8, 16>(__VA_ARGS__);                                                \
        case 1204: return FN<T, 12, 4>(__VA_ARGS__);                                               \
        case 1208: return FN<T, 12, 8>(__VA_ARGS__);                                               \
        case 1212: return FN<T, 12, 12>(__VA_ARGS__);                                              \
        case 1216: return FN<T, 12, 16>(__VA_ARGS__);                                              \
        case 1604: return FN<T, 16, 4>(__VA_ARGS__);                                               \
        case 1608: return FN<T, 16, 8>(__VA_ARGS__);                                               \
        case 1612: return FN<T, 16, 12>(__VA_ARGS__);                                              \
        default: return FN<T, 16, 16>(__VA_ARGS__);                                                \
        }                                                                                          \
    }()

template <typename T> void forward(const Call& call, T* O, const Problem<T>& p) {
    const int64_t rowsize = static_cast<int64_t>(p.nO1) * p.L;
    if (p.nW0 == 0 || rowsize == 0) return;
    if (p.E == 0 || p.N == 0) {
        MOPS_CUDA_OK(cudaMemsetAsync(O, 0, p.nW0 * rowsize * sizeof(T), call.stream));
        return;
    }
    if (forward_mma(call, O, p)) return;
    if (MOPS_B200_SASAW_FAST(forward_fast, call, O, p)) return;
    const int grid_generic = sm_count(call.device) * 8;
    Coupling<T> cp{};
    TableRef scratch{};
    const bool grouped = build_coupling(call, p, cp, &scratch);
    size_t smem_seg = 0, smem_edge = 0;
    int warps_seg = 0, warps_edge = 0;
    if (grouped) {
        warps_seg = pick_warps(call, cp, static_cast<size_t>(p.nA) + cp.ncell + rowsize, false,
                               &smem_seg);
        warps_edge = pick_warps(call, cp, static_cast<size_t>(p.nA) + cp.ncell, false, &smem_edge);
    }
    if (grouped && warps_seg > 0 && warps_edge > 0) {
        allow_smem(sasaw_fwd<T, true>, smem_seg);
        sasaw_fwd<T, true><<<static_cast<unsigned>(ceil_div(p.nW0, warps_seg)), warps_seg * 32,
                             smem_seg, call.stream>>>(O, p.A, p.B, p.W, p.Jw, p.Io, cp, p.E, p.nA,
                                                      p.L, p.nW0, p.nW1, p.nO1, false, call.status);
        MOPS_CUDA_OK(cudaGetLastError());
        bool need_fallback = true; // asynchronous calls cannot look: always enqueue
        if (call.wait) {
            wait_stream(call);
            need_fallback = host_saw_unsorted(call);
        }
        if (need_fallback) {
            zero_if_unsorted<T><<<grid_generic, 256, 0, call.stream>>>(O, p.nW0 * rowsize,
                                                                       call.status);
            allow_smem(sasaw_fwd<T, false>, smem_edge);
            const int64_t blocks = std::min<int64_t>(ceil_div(p.E, warps_edge), grid_generic);
            sasaw_fwd<T, false><<<static_cast<unsigned>(blocks), warps_edge * 32, smem_edge,
                                  call.stream>>>(O, p.A, p.B, p.W, p.Jw, p.Io, cp, p.E, p.nA, p.L,
                                                 p.nW0, p.nW1, p.nO1, false, call.status);
        }
    } else {
        MOPS_CUDA_OK(cudaMemsetAsync(O, 0, p.nW0 * rowsize * sizeof(T), call.stream));
        sasaw_fwd_wide<T><<<grid_generic, 256, 0, call.stream>>>(
            O, p.A, p.B, p.C, p.W, p.M1, p.Jw, p.M2, p.Io, p.M3, p.E, p.nA, p.L, p.N, p.nW0, p.nW1,
            p.nO1, call.status);
    }
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, scratch);
}

template <typename T>
void backward(const Call& call, T* gA, T* gB, T* gW, const T* gO, const Problem<T>& p) {
    if (gA == nullptr && gB == nullptr && gW == nullptr) return;
    const int64_t wsize = p.nW0 * static_cast<int64_t>(p.nW1) * p.L;
    if (gW != nullptr && wsize > 0)
        MOPS_CUDA_OK(cudaMemsetAsync(gW, 0, wsize * sizeof(T), call.stream));
    if (p.E == 0) return;
    const bool empty = p.N == 0 || p.L == 0 || p.nO1 == 0 || p.nW1 == 0 || p.nA == 0;
    if (!empty && backward_mma(call, gA, gB, gW, gO, p)) return;
    if (!empty && MOPS_B200_SASAW_FAST(backward_fast, call, gA, gB, gW, gO, p)) return;
    Coupling<T> cp{};
    TableRef scratch{};
    const bool grouped = !empty && build_coupling(call, p, cp, &scratch);
    size_t smem = 0;
    int warps = 0;
    if (grouped)
        warps = pick_warps(call, cp, static_cast<size_t>(p.nA) * 34 + 2 * static_cast<size_t>(cp.ncell),
                           true, &smem);
    if (empty) {
        if (gA != nullptr && p.nA > 0)
            MOPS_CUDA_OK(cudaMemsetAsync(gA, 0, p.E * p.nA * sizeof(T), call.stream));
        if (gB != nullptr && p.L > 0)
            MOPS_CUDA_OK(cudaMemsetAsync(gB, 0, p.E * p.L * sizeof(T), call.stream));
    } else if (grouped && warps > 0) {
        allow_smem(sasaw_vjp<T>, smem);
        const int64_t blocks =
            std::min<int64_t>(ceil_div(p.E, warps), static_cast<int64_t>(sm_count(call.device)) * 16);
        sasaw_vjp<T><<<static_cast<unsigned>(blocks), warps * 32, smem, call.stream>>>(
            gA, gB, gW, gO, p.A, p.B, p.W, p.Jw, p.Io, cp, p.E, p.nA, p.L, p.nW0, p.nW1, p.nO1,
            call.status);
    } else {
        if (gA != nullptr)
            MOPS_CUDA_OK(cudaMemsetAsync(gA, 0, p.E * p.nA * sizeof(T), call.stream));
        sasaw_vjp_wide<T><<<sm_count(call.device) * 8, 256, 0, call.stream>>>(
            gA, gB, gW, gO, p.A, p.B, p.C, p.W, p.M1, p.Jw, p.M2, p.Io, p.M3, p.E, p.nA, p.L, p.N,
            p.nW0, p.nW1, p.nO1, call.status);
    }
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, scratch);
}

template <typename scalar_t>
Problem<scalar_t> check_and_pack(const mops::Tensor<scalar_t, 3>& output,
                                 const mops::Tensor<scalar_t, 2>& A,
                                 const mops::Tensor<scalar_t, 2>& B,
                                 const mops::Tensor<scalar_t, 1>& C,
                                 const mops::Tensor<scalar_t, 3>& W,
                                 const mops::Tensor<int32_t, 1>& indices_A,
                                 const mops::Tensor<int32_t, 1>& indices_W_1,
                                 const mops::Tensor<int32_t, 1>& indices_W_2,
                                 const mops::Tensor<int32_t, 1>& indices_output_1,
                                 const mops::Tensor<int32_t, 1>& indices_output_2,
                                 const std::string& op) {
    same_size(A, "A", 0, B, "B", 0, op);
    same_size(W, "W", 0, output, "output", 0, op);
    same_size(B, "B", 1, W, "W", 2, op);
    same_size(C, "C", 0, indices_A, "indices_A", 0, op);
    same_size(C, "C", 0, indices_W_2, "indices_W_2", 0, op);
    same_size(C, "C", 0, indices_output_2, "indices_output_2", 0, op);
    same_size(A, "A", 0, indices_output_1, "indices_output_1", 0, op);
    same_size(A, "A", 0, indices_W_1, "indices_W_1", 0, op);
    // Not checked by the reference (checks/sasaw.hpp:22-29), needed for memory safety here:
    same_size(B, "B", 1, output, "output", 2, op);
    fits_int32(W.shape[0], "W.shape[0]", op);
    fits_int32(W.shape[1], "W.shape[1]", op);
    fits_int32(A.shape[1], "A.shape[1]", op);
    fits_int32(B.shape[1], "B.shape[1]", op);
    fits_int32(C.shape[0], "C.shape[0]", op);
    fits_int32(output.shape[1], "output.shape[1]", op);
    Problem<scalar_t> p;
    p.A = A.data;
    p.B = B.data;
    p.C = C.data;
    p.W = W.data;
    p.M1 = indices_A.data;
    p.Jw = indices_W_1.data;
    p.M2 = indices_W_2.data;
    p.Io = indices_output_1.data;
    p.M3 = indices_output_2.data;
    p.E = static_cast<int64_t>(A.shape[0]);
    p.nW0 = static_cast<int64_t>(W.shape[0]);
    p.nA = static_cast<int>(A.shape[1]);
    p.L = static_cast<int>(B.shape[1]);
    p.N = static_cast<int>(C.shape[0]);
    p.nW1 = static_cast<int>(W.shape[1]);
    p.nO1 = static_cast<int>(output.shape[1]);
    return p;
}

} // namespace
} // namespace mops_b200

using namespace mops_b200;

template <typename scalar_t>
void mops::cuda::sparse_accumulation_scatter_add_with_weights(
    Tensor<scalar_t, 3> output, Tensor<scalar_t, 2> A, Tensor<scalar_t, 2> B,
    Tensor<scalar_t, 1> C, Tensor<scalar_t, 3> W, Tensor<int32_t, 1> indices_A,
    Tensor<int32_t, 1> indices_W_1, Tensor<int32_t, 1> indices_W_2,
    Tensor<int32_t, 1> indices_output_1, Tensor<int32_t, 1> indices_output_2) {
    const std::string op = "cuda_sparse_accumulation_scatter_add_with_weights";
    Problem<scalar_t> p = check_and_pack(output, A, B, C, W, indices_A, indices_W_1, indices_W_2,
                                         indices_output_1, indices_output_2, op);
    Call call = begin_call();
    forward<scalar_t>(call, output.data, p);
    end_call(call, op.c_str(), kIndexNames, 5);
}

template <typename scalar_t>
void mops::cuda::sparse_accumulation_scatter_add_with_weights_vjp(
    Tensor<scalar_t, 2> grad_A, Tensor<scalar_t, 2> grad_B, Tensor<scalar_t, 3> grad_W,
    Tensor<scalar_t, 3> grad_output, Tensor<scalar_t, 2> A, Tensor<scalar_t, 2> B,
    Tensor<scalar_t, 1> C, Tensor<scalar_t, 3> W, Tensor<int32_t, 1> indices_A,
    Tensor<int32_t, 1> indices_W_1, Tensor<int32_t, 1> indices_W_2,
    Tensor<int32_t, 1> indices_output_1, Tensor<int32_t, 1> indices_output_2) {
    const std::string op = "cuda_sparse_accumulation_scatter_add_with_weights_vjp";
    grad_like(grad_A, "grad_A", A, "A", op);
    grad_like(grad_B, "grad_B", B, "B", op);
    grad_like(grad_W, "grad_W", W, "W", op);
    Problem<scalar_t> p = check_and_pack(grad_output, A, B, C, W, indices_A, indices_W_1,
                                         indices_W_2, indices_output_1, indices_output_2, op);
    Call call = begin_call();
    backward<scalar_t>(call, grad_A.data, grad_B.data, grad_W.data, grad_output.data, p);
    end_call(call, op.c_str(), kIndexNames, 5);
}

template <typename scalar_t>
void mops::cuda::sparse_accumulation_scatter_add_with_weights_vjp_vjp(
    Tensor<scalar_t, 3>, Tensor<scalar_t, 2>, Tensor<scalar_t, 2>, Tensor<scalar_t, 3>,
    Tensor<scalar_t, 2>, Tensor<scalar_t, 2>, Tensor<scalar_t, 3>, Tensor<scalar_t, 3>,
    Tensor<scalar_t, 2>, Tensor<scalar_t, 2>, Tensor<scalar_t, 1>, Tensor<scalar_t, 3>,
    Tensor<int32_t, 1>, Tensor<int32_t, 1>, Tensor<int32_t, 1>, Tensor<int32_t, 1>,
    Tensor<int32_t, 1>) {
    // The reference has no second-order SASAW on any device (mops/src/sasaw/cpu.tpp:193).
    throw std::runtime_error("Not implemented");
}

#define INSTANTIATE(T)                                                                             \
    template void mops::cuda::sparse_accumulation_scatter_add_with_weights<T>(                    \
        mops::Tensor<T, 3>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 1>,           \
        mops::Tensor<T, 3>, mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>,                   \
        mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>);            \
    template void mops::cuda::sparse_accumulation_scatter_add_with_weights_vjp<T>(                \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 3>, mops::Tensor<T, 3>,           \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 1>, mops::Tensor<T, 3>,           \
        mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>,             \
        mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>);                                      \
    template void mops::cuda::sparse_accumulation_scatter_add_with_weights_vjp_vjp<T>(            \
        mops::Tensor<T, 3>, mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 3>,           \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 3>, mops::Tensor<T, 3>,           \
        mops::Tensor<T, 2>, mops::Tensor<T, 2>, mops::Tensor<T, 1>, mops::Tensor<T, 3>,           \
        mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>,             \
        mops::Tensor<int32_t, 1>, mops::Tensor<int32_t, 1>);

INSTANTIATE(float)
INSTANTIATE(double)

// ------------------------------------------------------------ allocation-free SASAW forward
//
// mops_b200_cuda_sparse_accumulation_scatter_add_with_weights_noalloc_f64: the forward above
// for callers that cannot allocate device memory at the time they call: a host program
// whose own memory pool has reserved the whole device (a simulation code or a serving
// process that takes all of HBM at start-up, where a cudaMalloc from a library fails or
// fragments the pool), and latency-critical loops, where a driver allocation may block or
// synchronise the device. It computes exactly what
// mops_cuda_sparse_accumulation_scatter_add_with_weights_f64 computes, but everything the
// normal path allocates (the grouped coupling table and the status words the kernels report
// through) lives in the fixed device array below, so the entry point calls no cudaMalloc,
// cudaFree, cudaMallocAsync or any other allocating routine. The caller still passes all
// inputs and the output.
//
// Limits and rules:
//   * at most kNoAllocMaxEntries coupling entries (C.shape[0]) and kNoAllocMaxCells cells
//     (output.shape[1] * W.shape[1]); larger problems are rejected with status 1;
//   * every GPU that loads this library holds the array (about 100 KB) until the process ends;
//   * all calls share the array and it keeps the previous call's contents: the status words
//     are cleared at the start of each call, the table is rewritten in full; two calls whose
//     GPU work overlaps (different streams or threads) race on it, so serialise them;
//   * the first call on each device looks up the array's device address
//     (cudaGetSymbolAddress); make that first call outside any stream capture;
//   * runs on the calling thread's stream (mops_b200_set_stream) and returns when the result
//     is complete.
namespace mops_b200 {
namespace {

constexpr int kNoAllocMaxEntries = 4096;
constexpr int kNoAllocMaxCells = 1024;
constexpr size_t kNoAllocStatusBytes = 256; // status words, padded so the table stays aligned
constexpr size_t kNoAllocBytes = kNoAllocStatusBytes + kNoAllocMaxEntries * sizeof(double) +
                                 3 * kNoAllocMaxEntries * sizeof(int32_t) +
                                 (kNoAllocMaxCells + 1) * sizeof(int32_t) + 252;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mutex;
unsigned char* g_noalloc_address[kNoAllocMaxDevices] = {};
uint32_t g_noalloc_epoch = 0;

// Device address of the scratch array on the current device (looked up once per device).
unsigned char* noalloc_scratch_for_current_device(int* device_out) {
    int device = 0;
    MOPS_CUDA_OK(cudaGetDevice(&device));
    if (device < 0 || device >= kNoAllocMaxDevices)
        throw std::runtime_error("device ordinal out of range for the allocation-free entry point");
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_address[device] == nullptr) {
        void* ptr = nullptr;
        MOPS_CUDA_OK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        g_noalloc_address[device] = static_cast<unsigned char*>(ptr);
    }
    *device_out = device;
    return g_noalloc_address[device];
}

void forward_noalloc(double* O, const Problem<double>& p) {
    using T = double;
    const int64_t rowsize = static_cast<int64_t>(p.nO1) * p.L;
    const int64_t ncell = static_cast<int64_t>(p.nO1) * p.nW1;
    if (p.N > kNoAllocMaxEntries || ncell > kNoAllocMaxCells) {
        throw std::runtime_error(
            "the allocation-free SASAW entry point supports at most " +
            std::to_string(kNoAllocMaxEntries) + " coupling entries and " +
            std::to_string(kNoAllocMaxCells) + " (output_size x W.shape[1]) cells; got " +
            std::to_string(p.N) + " and " + std::to_string(ncell) +
            ". Use mops_cuda_sparse_accumulation_scatter_add_with_weights_f64 instead");
    }
    if (ncell == 0 && rowsize > 0 && p.nW0 > 0 && p.E > 0 && p.N > 0) {
        // W.shape[1] == 0 with a non-empty coupling table: every indices_W_2 entry is out of
        // range. The regular entry point reports the same (its table builder stands down and
        // the entry-wise kernel finds the bad indices); here it is decided on the host, before
        // any launch, because the grouping kernel cannot run on an empty cell grid.
        throw std::runtime_error(
            "Index array indices_W_2 in operation "
            "cuda_sparse_accumulation_scatter_add_with_weights (allocation-free) contains "
            "negative or too large elements; this would cause out-of-bounds accesses");
    }
    Call call;
    unsigned char* base = noalloc_scratch_for_current_device(&call.device);
    call.stream = static_cast<cudaStream_t>(get_stream());
    call.wait = true;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        g_noalloc_epoch += 1;
        if (g_noalloc_epoch == 0) g_noalloc_epoch = 1;
        call.status.epoch = g_noalloc_epoch;
    }
    // Both views of the status block are the device array: nothing here is host-mapped.
    call.status.dev = reinterpret_cast<uint32_t*>(base);
    call.status.host = call.status.dev;
    MOPS_CUDA_OK(cudaMemsetAsync(base, 0, kNoAllocStatusBytes, call.stream));

    if (p.nW0 == 0 || rowsize == 0) return;
    if (p.E == 0 || p.N == 0) {
        MOPS_CUDA_OK(cudaMemsetAsync(O, 0, p.nW0 * rowsize * sizeof(T), call.stream));
        MOPS_CUDA_OK(cudaStreamSynchronize(call.stream));
        return;
    }

    Coupling<T> cp{};
    cp.N = p.N;
    cp.ncell = static_cast<int>(ncell);
    unsigned char* table = base + kNoAllocStatusBytes;
    cp.C = reinterpret_cast<T*>(table);
    cp.M1 = reinterpret_cast<int32_t*>(table + kNoAllocMaxEntries * sizeof(T));
    cp.cell = cp.M1 + kNoAllocMaxEntries;
    cp.order = cp.cell + kNoAllocMaxEntries;
    cp.start = cp.order + kNoAllocMaxEntries;
    sasaw_group_coupling<T><<<1, kBuildThreads, cp.ncell * sizeof(int32_t), call.stream>>>(
        cp, p.C, p.M1, p.M2, p.M3, p.nA, p.nW1, p.nO1, call.status);
    MOPS_CUDA_OK(cudaGetLastError());

    size_t smem_seg = 0, smem_edge = 0;
    const int warps_seg =
        pick_warps(call, cp, static_cast<size_t>(p.nA) + cp.ncell + rowsize, false, &smem_seg);
    const int warps_edge =
        pick_warps(call, cp, static_cast<size_t>(p.nA) + cp.ncell, false, &smem_edge);
    if (warps_seg == 0 || warps_edge == 0) {
        throw std::runtime_error("rows of this size do not fit the allocation-free SASAW entry "
                                 "point's shared-memory kernels; use "
                                 "mops_cuda_sparse_accumulation_scatter_add_with_weights_f64");
    }
    allow_smem(sasaw_fwd<T, true>, smem_seg);
    sasaw_fwd<T, true><<<static_cast<unsigned>(ceil_div(p.nW0, warps_seg)), warps_seg * 32,
                         smem_seg, call.stream>>>(O, p.A, p.B, p.W, p.Jw, p.Io, cp, p.E, p.nA, p.L,
                                                  p.nW0, p.nW1, p.nO1, false, call.status);
    MOPS_CUDA_OK(cudaGetLastError());
    MOPS_CUDA_OK(cudaStreamSynchronize(call.stream));

    uint32_t words[kStatusWords];
    MOPS_CUDA_OK(cudaMemcpy(words, base, sizeof(words), cudaMemcpyDeviceToHost));
    if (words[kUnsortedEpoch] == call.status.epoch) {
        const int grid_generic = sm_count(call.device) * 8;
        zero_if_unsorted<T><<<grid_generic, 256, 0, call.stream>>>(O, p.nW0 * rowsize, call.status);
        allow_smem(sasaw_fwd<T, false>, smem_edge);
        const int64_t blocks = std::min<int64_t>(ceil_div(p.E, warps_edge), grid_generic);
        sasaw_fwd<T, false><<<static_cast<unsigned>(blocks), warps_edge * 32, smem_edge,
                              call.stream>>>(O, p.A, p.B, p.W, p.Jw, p.Io, cp, p.E, p.nA, p.L,
                                             p.nW0, p.nW1, p.nO1, false, call.status);
        MOPS_CUDA_OK(cudaGetLastError());
        MOPS_CUDA_OK(cudaStreamSynchronize(call.stream));
        MOPS_CUDA_OK(cudaMemcpy(words, base, sizeof(words), cudaMemcpyDeviceToHost));
    }
    std::string names;
    for (int i = 0; i < 5; i++) {
        if (words[kBadIndex0 + i] == call.status.epoch) {
            if (!names.empty()) names += ", ";
            names += kIndexNames[i];
        }
    }
    if (!names.empty()) {
        throw std::runtime_error(
            "Index array " + names + " in operation "
            "cuda_sparse_accumulation_scatter_add_with_weights (allocation-free) contains "
            "negative or too large elements; this would cause out-of-bounds accesses");
    }
}

} // namespace

// Called by the C entry point in capi.cu.
void sasaw_forward_noalloc_f64(mops::Tensor<double, 3> output, mops::Tensor<double, 2> A,
                               mops::Tensor<double, 2> B, mops::Tensor<double, 1> C,
                               mops::Tensor<double, 3> W, mops::Tensor<int32_t, 1> indices_A,
                               mops::Tensor<int32_t, 1> indices_W_1,
                               mops::Tensor<int32_t, 1> indices_W_2,
                               mops::Tensor<int32_t, 1> indices_output_1,
                               mops::Tensor<int32_t, 1> indices_output_2) {
    const std::string op = "cuda_sparse_accumulation_scatter_add_with_weights";
    Problem<double> p = check_and_pack(output, A, B, C, W, indices_A, indices_W_1, indices_W_2,
                                       indices_output_1, indices_output_2, op);
    forward_noalloc(output.data, p);
}

} // namespace mops_b200
