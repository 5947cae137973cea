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
#include <cstdlib>
#include <type_traits>

#include "bulk.cuh"
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

#include "opsa_pipe.cuh"

// ------------------------------------------------------------------------------ forward
struct FwdPlan {
    int G;      // lanes that share one entry; 32 / G entries are processed side by side
    int LL, LK; // lane grid inside a group: LL lanes along l, LK along k (LL*LK <= G)
    int TK;     // k values per lane (contiguous)
    int NV;     // l vector chunks per lane (chunk q = ll + v*LL covers l in [q*VEC, q*VEC+VEC))
    int VEC;    // scalars per l chunk (16-byte loads when > 1)
    int CH;     // entries per staged chunk (<= 32)
    int stage_scalars; // scalars of one stage: CH*L (B) [+ CH*L (W rows)] + CH*K (A) + padding
    size_t smem_per_warp;
};

// One warp per output row. The row's entries [offsets[r], offsets[r+1]) are contiguous in A
// and B; they stream through two shared-memory stages with cp.async, the next chunk in
// flight while the current one is consumed. The 32 lanes form 32/G groups that take
// alternate entries; inside a group, lane (lk, ll) keeps a TK x (NV*VEC) tile of the K x L
// result in registers. Fewer lanes per entry mean larger register tiles, hence fewer
// shared-memory operand reads per multiply-add (the limiter of this kernel after HBM); the
// groups' partial tiles are added with shuffles once per row.
template <typename T, int TK, int NV, int VEC, bool WEIGHTED>
__global__ void __launch_bounds__(kFwdWarps * 32, 2)
opsa_fwd_rows(T* __restrict__ O, const T* __restrict__ A, const T* __restrict__ B,
              const T* __restrict__ W, const int32_t* __restrict__ PW,
              const int64_t* __restrict__ offsets, int K, int L, int64_t nO, FwdPlan plan,
              Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    if (saw_unsorted(st)) return; // the atomic kernel of the same call does the work
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * kFwdWarps + warp;
    if (r >= nO) return;

    const int CH = plan.CH;
    T* stage0 = reinterpret_cast<T*>(smem_raw + warp * plan.smem_per_warp);
    // stage layout: Bs [CH][L] | Ws [CH][L] (weighted only) | As [CH][K] | padding
    const int a_off = (WEIGHTED ? 2 : 1) * CH * L;
    const int64_t begin = offsets[r], end = offsets[r + 1];

    const int G = plan.G, slots = 32 / G;
    const int slot = lane / G, g = lane - slot * G;
    const int ll = g % plan.LL, lk = g / plan.LL;
    T* Orow = O + r * K * L;

    // Issues the copies of chunk [c0, c0+n) into stage `buf`. pw_lane: lane jj holds PW[c0+jj].
    auto issue = [&](int buf, int64_t c0, int n, int32_t pw_lane) {
        T* Bs = stage0 + buf * plan.stage_scalars;
        const T* b = B + c0 * L;
        for (int idx = lane; idx < n * L; idx += 32) cp_async<sizeof(T)>(Bs + idx, b + idx);
        T* As = Bs + a_off;
        const T* a = A + c0 * K;
        for (int idx = lane; idx < n * K; idx += 32) cp_async<sizeof(T)>(As + idx, a + idx);
        if (WEIGHTED) {
            T* Ws = Bs + CH * L;
            for (int jj = 0; jj < n; jj++) {
                const int32_t pw = __shfl_sync(kFullMask, pw_lane, jj);
                const T* w = W + static_cast<int64_t>(pw) * L;
                for (int l = lane; l < L; l += 32) cp_async<sizeof(T)>(Ws + jj * L + l, w + l);
            }
        }
        cp_async_commit();
    };
    auto load_pw = [&](int64_t c0, int n) -> int32_t {
        int32_t pw = 0;
        if (WEIGHTED && lane < n) {
            pw = __ldg(PW + c0 + lane);
            if (clamp_index(pw, static_cast<int32_t>(nO))) report_bad_index(st, 1);
        }
        return pw;
    };

    const int l_span = plan.LL * NV * VEC; // l values one pass covers
    for (int kb = 0; kb < K; kb += plan.LK * TK) {
        for (int lb = 0; lb < L; lb += l_span) {
            const int k0 = kb + lk * TK;
            const bool active = lk < plan.LK && k0 < K;
            int l_of[NV]; // first l of each of this lane's chunks
#pragma unroll
            for (int v = 0; v < NV; v++) l_of[v] = lb + (ll + v * plan.LL) * VEC;
            T acc[TK][NV * VEC];
#pragma unroll
            for (int t = 0; t < TK; t++)
#pragma unroll
                for (int u = 0; u < NV * VEC; u++) acc[t][u] = T(0);

            const int64_t total = end - begin;
            const int nchunks = static_cast<int>((total + CH - 1) / CH);
            __syncwarp();
            if (nchunks > 0) {
                const int n0 = static_cast<int>(total < CH ? total : CH);
                issue(0, begin, n0, load_pw(begin, n0));
            }
            int32_t pw_next = 0;
            if (nchunks > 1) {
                const int64_t c1 = begin + CH;
                pw_next = load_pw(c1, static_cast<int>(end - c1 < CH ? end - c1 : CH));
            }
            for (int c = 0; c < nchunks; c++) {
                const int64_t c0 = begin + static_cast<int64_t>(c) * CH;
                const int n = static_cast<int>(end - c0 < CH ? end - c0 : CH);
                if (c + 1 < nchunks) {
                    const int64_t c1 = c0 + CH;
                    issue((c + 1) & 1, c1, static_cast<int>(end - c1 < CH ? end - c1 : CH), pw_next);
                    if (c + 2 < nchunks) {
                        const int64_t c2 = c1 + CH;
                        pw_next = load_pw(c2, static_cast<int>(end - c2 < CH ? end - c2 : CH));
                    }
                    cp_async_wait<1>();
                } else {
                    cp_async_wait<0>();
                }
                __syncwarp();
                if (active) {
                    const T* Bs = stage0 + (c & 1) * plan.stage_scalars;
                    const T* pb = Bs + slot * L;
                    const T* pa = Bs + a_off + slot * K + k0;
                    for (int jj = slot; jj < n; jj += slots) {
                        T a[TK], b[NV * VEC];
                        // k0+t beyond K reads the next row or the padding: those
                        // accumulators are never stored.
#pragma unroll
                        for (int t = 0; t < TK; t++) a[t] = pa[t];
#pragma unroll
                        for (int v = 0; v < NV; v++) {
                            T bv[VEC];
                            if (l_of[v] < L) {
                                if (VEC > 1) {
                                    load_vec<T, VEC>(pb + l_of[v], bv);
                                } else {
                                    bv[0] = pb[l_of[v]];
                                }
                                if (WEIGHTED) {
                                    T wv[VEC];
                                    if (VEC > 1) {
                                        load_vec<T, VEC>(pb + CH * L + l_of[v], wv);
                                    } else {
                                        wv[0] = pb[CH * L + l_of[v]];
                                    }
#pragma unroll
                                    for (int u = 0; u < VEC; u++) bv[u] *= wv[u];
                                }
                            } else {
#pragma unroll
                                for (int u = 0; u < VEC; u++) bv[u] = T(0);
                            }
#pragma unroll
                            for (int u = 0; u < VEC; u++) b[v * VEC + u] = bv[u];
                        }
#pragma unroll
                        for (int t = 0; t < TK; t++)
#pragma unroll
                            for (int u = 0; u < NV * VEC; u++) acc[t][u] += a[t] * b[u];
                        pa += slots * K;
                        pb += slots * L;
                    }
                }
                __syncwarp(); // stage (c & 1) may be overwritten by the copy issued next round
            }
            // add the groups' partial tiles (all lanes take part in the shuffles)
            for (int d = G; d < 32; d <<= 1) {
#pragma unroll
                for (int t = 0; t < TK; t++)
#pragma unroll
                    for (int u = 0; u < NV * VEC; u++)
                        acc[t][u] += __shfl_xor_sync(kFullMask, acc[t][u], d);
            }
            if (active && slot == 0) {
#pragma unroll
                for (int t = 0; t < TK; t++) {
                    if (k0 + t < K) {
#pragma unroll
                        for (int v = 0; v < NV; v++) {
                            if (l_of[v] < L) {
                                T out[VEC];
#pragma unroll
                                for (int u = 0; u < VEC; u++) out[u] = acc[t][v * VEC + u];
                                if (VEC > 1) {
                                    store_vec<T, VEC>(Orow + (k0 + t) * L + l_of[v], out);
                                } else {
                                    Orow[(k0 + t) * L + l_of[v]] = out[0];
                                }
                            }
                        }
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

constexpr int kMaxNV = 3;

// Chooses the lane grouping and register tile that minimise shared-memory operand traffic
// per entry, within a register budget.
template <typename T, bool WEIGHTED> FwdPlan plan_forward(int K, int L, bool l_aligned) {
    const int words = static_cast<int>(sizeof(T)) / 4; // 32-bit words per scalar
    const int widest = 16 / static_cast<int>(sizeof(T));
    FwdPlan best{};
    double best_cost = 1e30;
    for (int VEC : {widest, 1}) {
        if (VEC > 1 && (!l_aligned || L % VEC != 0)) continue;
        const int nchunks_l = static_cast<int>(ceil_div(L, VEC));
        for (int G : {32, 16, 8, 4}) {
            for (int LL = 1; LL <= G; LL++) {
                int LK = G / LL;
                if (LK > K) LK = K;
                const int NV = static_cast<int>(ceil_div(nchunks_l, LL));
                const int TK = static_cast<int>(ceil_div(K, LK));
                if (NV > kMaxNV || TK > kMaxTK) continue;
                const int acc = TK * NV * VEC;
                if (acc * words > 64) continue; // register budget: two 8-warp blocks per SM
                // shared-memory passes per entry: a w-byte load costs w/4 of a 32-lane pass
                const double operand =
                    (TK + (WEIGHTED ? 2 : 1) * NV * VEC) * words * (G / 32.0);
                // shuffles that add the 32/G partial tiles, spread over ~48 entries per row
                int steps = 0;
                for (int d = G; d < 32; d <<= 1) steps++;
                const double reduce = acc * words * steps / 48.0;
                // idle lanes and padded tile elements waste issue slots
                const double waste = 0.02 * (TK * LK * NV * LL * VEC) / std::max(1, K * L);
                const double cost = operand + reduce + waste;
                if (cost < best_cost) {
                    best_cost = cost;
                    best.G = G;
                    best.LL = LL;
                    best.LK = LK;
                    best.TK = TK;
                    best.NV = NV;
                    best.VEC = VEC;
                }
            }
        }
        if (best_cost < 1e30) break; // the widest usable vector is always the better choice
    }
    if (best_cost >= 1e30) {
        // very large K x L: tile in passes with the largest tile
        best.VEC = (l_aligned && L % widest == 0) ? widest : 1;
        best.G = 32;
        best.LL = static_cast<int>(std::min<int64_t>(32, ceil_div(ceil_div(L, best.VEC), kMaxNV)));
        best.LK = std::max(1, 32 / best.LL);
        best.NV = static_cast<int>(std::min<int64_t>(kMaxNV, ceil_div(ceil_div(L, best.VEC), best.LL)));
        best.TK = static_cast<int>(std::min<int64_t>(kMaxTK, ceil_div(K, best.LK)));
        while (best.TK * best.NV * best.VEC * words > 64 && best.TK > 1) best.TK--;
    }
    FwdPlan p = best;
    // Two stages per warp, about 9 KB together, so that three 8-warp blocks share an SM.
    const size_t row_bytes = (static_cast<size_t>(K) + (WEIGHTED ? 2 : 1) * L) * sizeof(T);
    p.CH = 32;
    while (p.CH > 1 && 2 * p.CH * row_bytes > 9 * 1024) p.CH /= 2;
    // padding: TK scalars so the unguarded A reads of the last row stay inside the stage;
    // rounded so that every stage starts 16-byte aligned
    const int per16 = 16 / static_cast<int>(sizeof(T));
    int scalars = p.CH * (K + (WEIGHTED ? 2 : 1) * L) + kMaxTK;
    scalars = (scalars + per16 - 1) / per16 * per16;
    p.stage_scalars = scalars;
    p.smem_per_warp = 2 * static_cast<size_t>(scalars) * sizeof(T);
    return p;
}

template <typename T, int TK, int NV, int VEC, bool WEIGHTED>
void launch_fwd_tile(const Call& call, const FwdPlan& plan, T* O, const T* A, const T* B,
                     const T* W, const int32_t* PW, const int64_t* offsets, int K, int L,
                     int64_t nO) {
    auto kernel = opsa_fwd_rows<T, TK, NV, VEC, WEIGHTED>;
    note_kernel_f("opsa_fwd_rows<%s,TK=%d,NV=%d,VEC=%d,W=%d>", scalar_name<T>(), TK, NV, VEC,
                  WEIGHTED ? 1 : 0);
    const size_t smem = plan.smem_per_warp * kFwdWarps;
    if (smem > 48 * 1024) {
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
    }
    const int64_t blocks = ceil_div(nO, kFwdWarps);
    kernel<<<static_cast<unsigned>(blocks), kFwdWarps * 32, smem, call.stream>>>(
        O, A, B, W, PW, offsets, K, L, nO, plan, call.status);
}

template <typename T, int NV, int VEC, bool WEIGHTED, typename... Args>
void dispatch_tk(int TK, Args... args) {
    switch (TK) {
    case 1: launch_fwd_tile<T, 1, NV, VEC, WEIGHTED>(args...); break;
    case 2: launch_fwd_tile<T, 2, NV, VEC, WEIGHTED>(args...); break;
    case 3: launch_fwd_tile<T, 3, NV, VEC, WEIGHTED>(args...); break;
    case 4: launch_fwd_tile<T, 4, NV, VEC, WEIGHTED>(args...); break;
    case 5: launch_fwd_tile<T, 5, NV, VEC, WEIGHTED>(args...); break;
    case 6: launch_fwd_tile<T, 6, NV, VEC, WEIGHTED>(args...); break;
    case 7: launch_fwd_tile<T, 7, NV, VEC, WEIGHTED>(args...); break;
    default: launch_fwd_tile<T, 8, NV, VEC, WEIGHTED>(args...); break;
    }
}

template <typename T, int VEC, bool WEIGHTED, typename... Args>
void dispatch_nv(int NV, int TK, Args... args) {
    switch (NV) {
    case 1: dispatch_tk<T, 1, VEC, WEIGHTED>(TK, args...); break;
    case 2: dispatch_tk<T, 2, VEC, WEIGHTED>(TK, args...); break;
    default: dispatch_tk<T, 3, VEC, WEIGHTED>(TK, args...); break;
    }
}

// ------------------------------------------------------------------- forward, tensor cores
// f64, K <= 16, L <= 32, entries sorted by output row. The row's sum of outer products is a
// matrix product over its entries,  O[p] = A[seg, :]^T (B[seg, :] * W[PW[seg], :]),  with
// the entries as the MMA's k dimension: a warp takes one output row, keeps O[p] in its MMA
// accumulators and consumes four entries per step, reading the A and B fragments straight
// from global memory (a fragment row is 64 contiguous bytes of one entry).
// MT = ceil(K / 8), NT = ceil(L / 8).
template <int MT, int NT, bool WEIGHTED>
__global__ void __launch_bounds__(128, 4)
opsa_fwd_mma(double* __restrict__ O, const double* __restrict__ A, const double* __restrict__ B,
             const double* __restrict__ W, const int32_t* __restrict__ PW,
             const int64_t* __restrict__ offsets, int K, int L, int64_t nO, Status st) {
    using T = double;
    if (saw_unsorted(st)) return; // the atomic kernel of the same call does the work
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0); // uniform for the compiler
    const int qr = lane >> 2, qc = lane & 3;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps;
    const int64_t rowsize = static_cast<int64_t>(K) * L;
    const bool pair_ok = L % 2 == 0 && reinterpret_cast<uintptr_t>(O) % 16 == 0;

    // fragments of the four entries e0 .. e0+3: A^T[k = 8 mt + qr][entry qc] and
    // (B*W)[entry qc][l = 8 nt + qr]
    auto load_step = [&](int64_t e0, int64_t hi, T (&af)[MT], T (&bf)[NT]) {
        const int64_t e = e0 + qc;
        const bool valid = e < hi;
        int32_t wrow = 0;
        if (WEIGHTED && valid) {
            wrow = __ldg(PW + e);
            if (clamp_index(wrow, static_cast<int32_t>(nO))) report_bad_index(st, 1);
        }
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const int k = 8 * mt + qr;
            af[mt] = (valid && k < K) ? __ldg(A + e * K + k) : T(0);
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int l = 8 * nt + qr;
            T v = (valid && l < L) ? __ldg(B + e * L + l) : T(0);
            if (WEIGHTED && valid && l < L) v *= __ldg(W + static_cast<int64_t>(wrow) * L + l);
            bf[nt] = v;
        }
    };

    // Neighbouring warps take neighbouring rows, so a block reads one contiguous stretch of
    // the entries at a time. (Giving each warp its own contiguous range of rows, with the
    // loads running on across row boundaries, measured slower: 0.88 against 0.63 ms.)
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * warps + warp; r < nO; r += nwarps) {
        const int64_t lo = offsets[r], hi = offsets[r + 1];
        T acc[MT][NT][2];
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) acc[mt][nt][0] = acc[mt][nt][1] = T(0);
        if (lo < hi) {
            T af[MT], bf[NT], af_n[MT], bf_n[NT], af_m[MT], bf_m[NT];
            load_step(lo, hi, af, bf);
            load_step(lo + 4, hi, af_n, bf_n);
            for (int64_t e0 = lo; e0 < hi; e0 += 4) {
                load_step(e0 + 8, hi, af_m, bf_m); // two steps ahead
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) dmma(acc[mt][nt], af[mt], bf[nt]);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) af[mt] = af_n[mt], af_n[mt] = af_m[mt];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) bf[nt] = bf_n[nt], bf_n[nt] = bf_m[nt];
            }
        }
        // element (mt, nt, h) is O[r, k = 8 mt + qr, l = 8 nt + 2 qc + h]
        T* dst = O + r * rowsize;
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const int k = 8 * mt + qr;
            if (k >= K) continue;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int l = 8 * nt + 2 * qc;
                if (l >= L) continue;
                T* d2 = dst + k * L + l;
                if (pair_ok) {
                    *reinterpret_cast<double2*>(d2) = make_double2(acc[mt][nt][0], acc[mt][nt][1]);
                } else {
                    d2[0] = acc[mt][nt][0];
                    if (l + 1 < L) d2[1] = acc[mt][nt][1];
                }
            }
        }
    }
}

template <int MT, bool WEIGHTED, typename... Args>
void launch_fwd_mma_l(int L, unsigned blocks, cudaStream_t stream, Args... args) {
    switch ((L + 7) / 8) {
    case 1: opsa_fwd_mma<MT, 1, WEIGHTED><<<blocks, 128, 0, stream>>>(args...); break;
    case 2: opsa_fwd_mma<MT, 2, WEIGHTED><<<blocks, 128, 0, stream>>>(args...); break;
    case 3: opsa_fwd_mma<MT, 3, WEIGHTED><<<blocks, 128, 0, stream>>>(args...); break;
    default: opsa_fwd_mma<MT, 4, WEIGHTED><<<blocks, 128, 0, stream>>>(args...); break;
    }
}

// ------------------------------------------------------------- streaming kernels, host side
// Tuning overrides (development aid): MOPS_B200_PIPE=0 turns the streaming kernels off,
// MOPS_B200_PIPE_CH / MOPS_B200_PIPE_STAGES change the ring geometry.
inline int env_int(const char* name, int fallback) {
    const char* v = std::getenv(name);
    return v != nullptr && *v != '\0' ? std::atoi(v) : fallback;
}

template <typename T, bool WEIGHTED>
bool pipe_usable(const T* A, const T* B, const T* W, const void* extra, int K, int L, bool vjp) {
    auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (env_int("MOPS_B200_PIPE", 1) == 0) return false;
    if (K < 1 || K > 16 || L < 1 || L > 32) return false;
    if (!aligned(A) || !aligned(B) || !aligned(extra)) return false;
    if (WEIGHTED && (!aligned(W) || (L * sizeof(T)) % 16 != 0)) return false;
    if (vjp && (static_cast<size_t>(K) * L * sizeof(T)) % 16 != 0) return false;
    return true;
}

// Shapes of the weighted operation that have kernels with K and L fixed at compile time:
// L = 32 columns and K = 9, 13 or 16 (angular channels up to l = 4, 6, and (l + 1)^2 for l = 3).
inline bool fixed_shape(int K, int L) { return L == 32 && (K == 9 || K == 13 || K == 16); }

template <typename T, bool WEIGHTED> PipeLayout choose_pipe_layout(int K, int L, bool vjp) {
    // Measured on B200 (J = 2^24 / E = 2^22): without weights two stages of 32 entries per
    // warp are best for f64 (forward 0.92 ms, VJP 1.60 ms against 0.97 / 1.84 with four stages
    // of 16): the smaller ring lets more warps share an SM, and one chunk in flight per warp
    // already keeps about 100 KB per SM in flight; f32 takes 64 entries (the same bytes:
    // forward 0.52 ms, VJP 0.95 ms against 0.56 / 1.09 with 32). With weights a stage also
    // holds the padded B and W rows (680 bytes per entry), so chunks of 8 keep the warp count
    // up (forward 0.49 ms, VJP 1.00 ms against 0.54 / 1.02 with 16; four stages of 4 or 8:
    // 0.54 / 1.49 and 0.74 / 1.23). The stage count is rounded to a power of two.
    int ch = env_int("MOPS_B200_PIPE_CH", WEIGHTED ? 8 : sizeof(T) == 4 ? 64 : 32);
    int stages = env_int("MOPS_B200_PIPE_STAGES", 2);
    ch = std::max(4, std::min(WEIGHTED ? 32 : 128, ch / 4 * 4)); // weighted: one lane per entry
    stages = std::max(2, std::min(8, stages));
    return pipe_layout(sizeof(T), K, L, WEIGHTED, vjp, ch, stages);
}

// Grid of a VJP streaming kernel, whose warps split the entries: at most one warp per chunk.
template <typename Kernel>
unsigned pipe_grid_entries(const Call& call, Kernel kernel, size_t smem, int64_t J, int ch) {
    if (smem > 48 * 1024)
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
    int per_sm = 0;
    MOPS_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kPipeWarps * 32, smem));
    per_sm = std::max(1, per_sm);
    return static_cast<unsigned>(std::max<int64_t>(
        1, std::min<int64_t>(ceil_div(J, static_cast<int64_t>(kPipeWarps) * ch),
                             static_cast<int64_t>(sm_count(call.device)) * per_sm)));
}

template <typename Kernel>
unsigned pipe_grid(const Call& call, Kernel kernel, size_t smem, int64_t nO) {
    if (smem > 48 * 1024)
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
    int per_sm = 0;
    MOPS_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kPipeWarps * 32, smem));
    per_sm = std::max(1, per_sm);
    return static_cast<unsigned>(std::min<int64_t>(
        ceil_div(nO, kPipeWarps), static_cast<int64_t>(sm_count(call.device)) * per_sm));
}

template <typename T, int MT, bool WEIGHTED, typename... Args>
void launch_fwd_pipe_l(const Call& call, const PipeLayout& lay, int64_t nO, Args... args) {
    const size_t smem = static_cast<size_t>(lay.warp_bytes) * kPipeWarps;
#define MOPS_B200_CASE(NT_)                                                                        \
    {                                                                                              \
        auto kernel = opsa_fwd_pipe<T, MT, NT_, WEIGHTED>;                                         \
        const unsigned blocks = pipe_grid(call, kernel, smem, nO);                                 \
        kernel<<<blocks, kPipeWarps * 32, smem, call.stream>>>(args..., lay, call.status);         \
    }
    switch ((lay.L + 7) / 8) {
    case 1: MOPS_B200_CASE(1) break;
    case 2: MOPS_B200_CASE(2) break;
    case 3: MOPS_B200_CASE(3) break;
    default: MOPS_B200_CASE(4) break;
    }
#undef MOPS_B200_CASE
}

// Forward through the streaming kernel; false when it does not apply (the caller then takes
// another kernel).
template <typename T, bool WEIGHTED>
bool forward_pipe(const Call& call, T* O, const T* A, const T* B, const T* W, const int32_t* PW,
                  const int64_t* offsets, int64_t J, int K, int L, int64_t nO) {
    if (!pipe_usable<T, WEIGHTED>(A, B, W, nullptr, K, L, false)) return false;
    const PipeLayout lay = choose_pipe_layout<T, WEIGHTED>(K, L, false);
    if (static_cast<size_t>(lay.warp_bytes) * kPipeWarps > static_cast<size_t>(max_optin_smem(call.device)))
        return false;
    if constexpr (std::is_same<T, float>::value && !WEIGHTED) {
        // f32 without weights: the TF32 tensor path (MOPS_B200_TF32=0: development switch back
        // to the FP64 MMA route)
        if (env_int("MOPS_B200_TF32", 1) != 0) {
            const size_t smem = static_cast<size_t>(lay.warp_bytes) * kPipeWarps;
            note_kernel_f("opsa_fwd_pipe_tf32<NT=%d> ch=%d stages=%d", (L + 7) / 8, lay.ch,
                          lay.stages);
#define MOPS_B200_CASE(NT_)                                                                        \
    {                                                                                              \
        auto kernel = opsa_fwd_pipe_tf32<NT_>;                                                     \
        const unsigned blocks = pipe_grid(call, kernel, smem, nO);                                 \
        kernel<<<blocks, kPipeWarps * 32, smem, call.stream>>>(O, A, B, offsets, J, nO, lay,       \
                                                               call.status);                      \
    }
            switch ((L + 7) / 8) {
            case 1: MOPS_B200_CASE(1) break;
            case 2: MOPS_B200_CASE(2) break;
            case 3: MOPS_B200_CASE(3) break;
            default: MOPS_B200_CASE(4) break;
            }
#undef MOPS_B200_CASE
            MOPS_CUDA_OK(cudaGetLastError());
            return true;
        }
    }
    if constexpr (WEIGHTED) {
        // common shapes with K and L fixed at compile time (MOPS_B200_FIXED=0: development
        // switch back to the run-time widths)
        if (fixed_shape(K, L) && lay.ch == kFixedChunk<true> && lay.stages == 2 &&
            env_int("MOPS_B200_FIXED", 1) != 0) {
            const size_t smem = static_cast<size_t>(lay.warp_bytes) * kPipeWarps;
            note_kernel_f("opsa_fwd_pipe<%s,W=1,K=%d,L=%d> ch=%d stages=2", scalar_name<T>(), K, L, lay.ch);
#define MOPS_B200_CASE(K_)                                                                         \
    {                                                                                              \
        auto kernel = opsa_fwd_pipe<T, 2, 4, true, K_, 32>;                                        \
        const unsigned blocks = pipe_grid(call, kernel, smem, nO);                                 \
        kernel<<<blocks, kPipeWarps * 32, smem, call.stream>>>(O, A, B, W, PW, offsets, J, nO, nO, \
                                                               lay, call.status);                 \
    }
            switch (K) {
            case 9: MOPS_B200_CASE(9) break;
            case 13: MOPS_B200_CASE(13) break;
            default: MOPS_B200_CASE(16) break;
            }
#undef MOPS_B200_CASE
            MOPS_CUDA_OK(cudaGetLastError());
            return true;
        }
    }
    note_kernel_f("opsa_fwd_pipe<%s,MT=%d,NT=%d,W=%d> ch=%d stages=%d", scalar_name<T>(),
                  K <= 8 ? 1 : 2, (L + 7) / 8, WEIGHTED ? 1 : 0, lay.ch, lay.stages);
    if (K <= 8)
        launch_fwd_pipe_l<T, 1, WEIGHTED>(call, lay, nO, O, A, B, W, PW, offsets, J, nO, nO);
    else
        launch_fwd_pipe_l<T, 2, WEIGHTED>(call, lay, nO, O, A, B, W, PW, offsets, J, nO, nO);
    MOPS_CUDA_OK(cudaGetLastError());
    return true;
}

template <typename T, int KT, bool WEIGHTED, typename... Args>
void launch_vjp_pipe_l(const Call& call, const PipeLayout& lay, int64_t J, Args... args) {
    const size_t smem = static_cast<size_t>(lay.warp_bytes) * kPipeWarps;
#define MOPS_B200_CASE(LT_)                                                                        \
    {                                                                                              \
        auto kernel = opsa_vjp_pipe<T, KT, LT_, WEIGHTED>;                                         \
        const unsigned blocks = pipe_grid_entries(call, kernel, smem, J, lay.ch);                  \
        kernel<<<blocks, kPipeWarps * 32, smem, call.stream>>>(args..., lay, call.status);         \
    }
    switch ((lay.L + 7) / 8) {
    case 1: MOPS_B200_CASE(1) break;
    case 2: MOPS_B200_CASE(2) break;
    case 3: MOPS_B200_CASE(3) break;
    default: MOPS_B200_CASE(4) break;
    }
#undef MOPS_B200_CASE
}

template <typename T, bool WEIGHTED>
bool backward_pipe(const Call& call, T* gA, T* gB, T* gW, const T* gO, const T* A, const T* B,
                   const T* W, const int32_t* PW, const int64_t* offsets, int64_t J, int K, int L,
                   int64_t nO) {
    const PipeLayout lay = choose_pipe_layout<T, WEIGHTED>(K, L, true);
    if (static_cast<size_t>(lay.warp_bytes) * kPipeWarps > static_cast<size_t>(max_optin_smem(call.device)))
        return false;
    if constexpr (std::is_same<T, float>::value && !WEIGHTED) {
        if (env_int("MOPS_B200_TF32", 1) != 0) {
            const size_t smem = static_cast<size_t>(lay.warp_bytes) * kPipeWarps;
            note_kernel_f("opsa_vjp_pipe_tf32<KS=%d,LS=%d> ch=%d stages=%d", (K + 7) / 8,
                          (L + 7) / 8, lay.ch, lay.stages);
#define MOPS_B200_CASE(KS_, LS_)                                                                   \
    {                                                                                              \
        auto kernel = opsa_vjp_pipe_tf32<KS_, LS_>;                                                \
        const unsigned blocks = pipe_grid_entries(call, kernel, smem, J, lay.ch);                  \
        kernel<<<blocks, kPipeWarps * 32, smem, call.stream>>>(gA, gB, gO, A, B, offsets, J, nO,   \
                                                               lay, call.status);                 \
    }
            switch (((K + 7) / 8) * 10 + (L + 7) / 8) {
            case 11: MOPS_B200_CASE(1, 1) break;
            case 12: MOPS_B200_CASE(1, 2) break;
            case 13: MOPS_B200_CASE(1, 3) break;
            case 14: MOPS_B200_CASE(1, 4) break;
            case 21: MOPS_B200_CASE(2, 1) break;
            case 22: MOPS_B200_CASE(2, 2) break;
            case 23: MOPS_B200_CASE(2, 3) break;
            default: MOPS_B200_CASE(2, 4) break;
            }
#undef MOPS_B200_CASE
            MOPS_CUDA_OK(cudaGetLastError());
            return true;
        }
    }
    if constexpr (WEIGHTED) {
        if (fixed_shape(K, L) && lay.ch == kFixedChunk<true> && lay.stages == 2 &&
            env_int("MOPS_B200_FIXED", 1) != 0) {
            const PipeLayout& lay2 = lay;
            // Rows of 32 entries or more: one grad_output slot per warp instead of two (the
            // copy of the next row then has the whole current row to arrive), which is what
            // lets a fourth block fit an SM's shared memory (forward / VJP at E = 2^22,
            // 2^16 rows: 0.99 ms with two slots and three blocks).
            const bool long_rows = J / std::max<int64_t>(nO, 1) >= 32;
            const PipeLayout lay = pipe_layout(sizeof(T), K, L, true, true, lay2.ch, 2, long_rows ? 1 : 2);
            const size_t smem = static_cast<size_t>(lay.warp_bytes) * kPipeWarps;
            note_kernel_f("opsa_vjp_pipe<%s,W=1,K=%d,L=%d> ch=%d stages=2 g=%d", scalar_name<T>(), K, L, lay.ch,
                          lay.g_slots);
#define MOPS_B200_CASE(K_)                                                                         \
    {                                                                                              \
        auto kernel = opsa_vjp_pipe<T, (K_ + 3) / 4, 4, true, K_, 32>;                             \
        const unsigned blocks = pipe_grid_entries(call, kernel, smem, J, lay.ch);                  \
        kernel<<<blocks, kPipeWarps * 32, smem, call.stream>>>(gA, gB, gW, gO, A, B, W, PW,        \
                                                               offsets, J, nO, nO, lay,           \
                                                               call.status);                      \
    }
            switch (K) {
            case 9: MOPS_B200_CASE(9) break;
            case 13: MOPS_B200_CASE(13) break;
            default: MOPS_B200_CASE(16) break;
            }
#undef MOPS_B200_CASE
            MOPS_CUDA_OK(cudaGetLastError());
            return true;
        }
    }
    note_kernel_f("opsa_vjp_pipe<%s,KT=%d,LT8=%d,W=%d> ch=%d stages=%d", scalar_name<T>(),
                  (K + 3) / 4, (L + 7) / 8, WEIGHTED ? 1 : 0, lay.ch, lay.stages);
    switch ((K + 3) / 4) {
    case 1: launch_vjp_pipe_l<T, 1, WEIGHTED>(call, lay, J, gA, gB, gW, gO, A, B, W, PW, offsets, J, nO, nO); break;
    case 2: launch_vjp_pipe_l<T, 2, WEIGHTED>(call, lay, J, gA, gB, gW, gO, A, B, W, PW, offsets, J, nO, nO); break;
    case 3: launch_vjp_pipe_l<T, 3, WEIGHTED>(call, lay, J, gA, gB, gW, gO, A, B, W, PW, offsets, J, nO, nO); break;
    default: launch_vjp_pipe_l<T, 4, WEIGHTED>(call, lay, J, gA, gB, gW, gO, A, B, W, PW, offsets, J, nO, nO); break;
    }
    MOPS_CUDA_OK(cudaGetLastError());
    return true;
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
    FwdPlan plan = plan_forward<T, WEIGHTED>(K, L, aligned);
    const size_t smem = plan.smem_per_warp * kFwdWarps;
    const bool segmented = smem <= static_cast<size_t>(max_optin_smem(call.device));
    const int grid_generic = sm_count(call.device) * 8;

    if (segmented) {
        // Segment table: call-scoped scratch, (nO + 1) offsets.
        SegmentTable seg = segment_table(call, P, J, nO);
        const int64_t* offsets = seg.offsets;
        constexpr int widest = 16 / static_cast<int>(sizeof(T));
        bool on_tensor_cores = forward_pipe<T, WEIGHTED>(call, O, A, B, W, PW, offsets, J, K, L, nO);
        if constexpr (sizeof(T) == 8 && WEIGHTED) {
            if (!on_tensor_cores)
            // (without weights the staged kernel below measured as fast: 1.24 against 1.26 ms)
            if (K <= 16 && L <= 32) {
                const unsigned blocks = static_cast<unsigned>(
                    std::min<int64_t>(ceil_div(nO, 4), static_cast<int64_t>(sm_count(call.device)) * 4));
                note_kernel_f("opsa_fwd_mma<MT=%d,NT=%d,W=%d>", K <= 8 ? 1 : 2, (L + 7) / 8,
                              WEIGHTED ? 1 : 0);
                if (K <= 8)
                    launch_fwd_mma_l<1, WEIGHTED>(L, blocks, call.stream, O, A, B, W, PW, offsets, K,
                                                  L, nO, call.status);
                else
                    launch_fwd_mma_l<2, WEIGHTED>(L, blocks, call.stream, O, A, B, W, PW, offsets, K,
                                                  L, nO, call.status);
                on_tensor_cores = true;
            }
        }
        if (on_tensor_cores) {
        } else if (plan.VEC == widest)
            dispatch_nv<T, widest, WEIGHTED>(plan.NV, plan.TK, call, plan, O, A, B, W, PW, offsets,
                                             K, L, nO);
        else
            dispatch_nv<T, 1, WEIGHTED>(plan.NV, plan.TK, call, plan, O, A, B, W, PW, offsets, K,
                                        L, nO);
        MOPS_CUDA_OK(cudaGetLastError());
        release_table(call, seg.ref);
        bool need_fallback = !seg.known_sorted; // asynchronous calls cannot look: always enqueue
        if (need_fallback && call.wait) {
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
    bool only_if_unsorted; // run only when the segmented kernel of the same call stood down
};

template <typename T, int KP, int VL, bool WEIGHTED>
__global__ void __launch_bounds__(128, 4)
opsa_vjp_entries(T* __restrict__ gA, T* __restrict__ gB, T* __restrict__ gW,
                 const T* __restrict__ gO, const T* __restrict__ A, const T* __restrict__ B,
                 const T* __restrict__ W, const int32_t* __restrict__ PW,
                 const int32_t* __restrict__ P, int64_t J, int K, int L, int64_t nO,
                 VjpPlan plan, Status st) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    if (plan.only_if_unsorted && !saw_unsorted(st)) return;
    const int tid = threadIdx.x, EPB = blockDim.x;
    const int Kp = plan.Kp, Lp = plan.Lp, nkc = plan.nkc;
    T* As = reinterpret_cast<T*>(smem_raw);              // [EPB][Kp]  A rows, then gA rows
    T* Bs = As + static_cast<size_t>(EPB) * Kp;          // [EPB][Lp]  B rows, then gB rows
    T* Ws = Bs + static_cast<size_t>(EPB) * Lp;          // [EPB][Lp]  W rows, then gW terms
    T* Ss = WEIGHTED ? Ws + static_cast<size_t>(EPB) * Lp : Ws; // [EPB][Lp] S, only if nkc > 1

    const int64_t base = static_cast<int64_t>(blockIdx.x) * EPB;
    const int n = static_cast<int>(J - base < EPB ? J - base : EPB);
    int32_t* pws = reinterpret_cast<int32_t*>(Ss + (nkc > 1 ? static_cast<size_t>(EPB) * Lp : 0));

    // Stage the entries' rows: element idx of the contiguous slice -> (entry, column), tracked
    // incrementally (no division per element), copied asynchronously so that all of a
    // thread's loads are in flight together.
    {
        const int dj = EPB / K, dk = EPB - dj * K;
        int jj = tid / K, k = tid - jj * K;
        const T* src = A + base * K;
        for (int idx = tid; idx < n * K; idx += EPB) {
            cp_async<sizeof(T)>(As + jj * Kp + k, src + idx);
            jj += dj;
            k += dk;
            if (k >= K) {
                k -= K;
                jj++;
            }
        }
    }
    {
        const int dj = EPB / L, dl = EPB - dj * L;
        int jj = tid / L, l = tid - jj * L;
        const T* src = B + base * L;
        for (int idx = tid; idx < n * L; idx += EPB) {
            cp_async<sizeof(T)>(Bs + jj * Lp + l, src + idx);
            jj += dj;
            l += dl;
            if (l >= L) {
                l -= L;
                jj++;
            }
        }
    }
    if (WEIGHTED) {
        if (tid < n) {
            int32_t pw = __ldg(PW + base + tid);
            if (clamp_index(pw, static_cast<int32_t>(nO))) report_bad_index(st, 1);
            pws[tid] = pw;
        }
        __syncthreads();
        const int dj = EPB / L, dl = EPB - dj * L;
        int jj = tid / L, l = tid - jj * L;
        for (int idx = tid; idx < n * L; idx += EPB) {
            cp_async<sizeof(T)>(Ws + jj * Lp + l, W + static_cast<int64_t>(pws[jj]) * L + l);
            jj += dj;
            l += dl;
            if (l >= L) {
                l -= L;
                jj++;
            }
        }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    if (tid < n) {
        int32_t row = __ldg(P + base + tid);
        if (clamp_index(row, static_cast<int32_t>(nO))) report_bad_index(st, 0);
        const T* g = gO + static_cast<int64_t>(row) * K * L;
        T* a_row = As + tid * Kp;
        T* b_row = Bs + tid * Lp;
        T* w_row = Ws + tid * Lp;
        T* s_row = Ss + tid * Lp;

        // Byte offset of gO row t of a chunk, kept in registers so that every gO load is
        // "running pointer + 32-bit offset" instead of a 64-bit multiply-add per load.
        unsigned t_off[KP];
#pragma unroll
        for (int t = 0; t < KP; t++) t_off[t] = static_cast<unsigned>(t) * L * sizeof(T);

        for (int kc = 0; kc < nkc; kc++) {
            const int kbase = kc * KP;
            T a[KP], ga[KP];
#pragma unroll
            for (int t = 0; t < KP; t++) {
                a[t] = (kbase + t < K) ? a_row[kbase + t] : T(0);
                ga[t] = T(0);
            }
            const char* g_l = reinterpret_cast<const char*>(g + static_cast<int64_t>(kbase) * L);
            for (int l0 = 0; l0 < L; l0 += VL, g_l += VL * sizeof(T)) {
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
                        const T* src = reinterpret_cast<const T*>(g_l + t_off[t]);
                        if (VL > 1) {
                            load_vec<T, VL>(src, gv);
                        } else {
                            gv[0] = __ldg(src);
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
        const int dj = EPB / K, dk = EPB - dj * K;
        int jj = tid / K, k = tid - jj * K;
        T* dst = gA + base * K;
        for (int idx = tid; idx < n * K; idx += EPB) {
            dst[idx] = As[jj * Kp + k];
            jj += dj;
            k += dk;
            if (k >= K) {
                k -= K;
                jj++;
            }
        }
    }
    if (gB != nullptr || (WEIGHTED && gW != nullptr)) {
        const int dj = EPB / L, dl = EPB - dj * L;
        int jj = tid / L, l = tid - jj * L;
        for (int idx = tid; idx < n * L; idx += EPB) {
            if (gB != nullptr) gB[base * L + idx] = Bs[jj * Lp + l];
            if (WEIGHTED && gW != nullptr)
                red_add(gW + static_cast<int64_t>(pws[jj]) * L + l, Ws[jj * Lp + l]);
            jj += dj;
            l += dl;
            if (l >= L) {
                l -= L;
                jj++;
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
                              int64_t J, int K, int L, int64_t nO, bool only_if_unsorted, Status st) {
    if (only_if_unsorted && !saw_unsorted(st)) return;
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

// ----------------------------------------------------------------------- VJP, tensor cores
// K <= 16, L <= 32, entries sorted by output row (f32 operands are widened to f64 in
// registers: the products are then exact and the sums far inside the f32 tolerance). For the entries of one output row the
// two gradients are small matrix products with the row's grad_output as the common factor,
//     grad_A[seg, :] = B[seg, :] gO[p]^T      grad_B[seg, :] = A[seg, :] gO[p]
// so a warp takes one output row, keeps gO[p] in registers as MMA fragments and walks the
// row's entries eight at a time (the eight entries are the MMA's m dimension). The A and B
// fragments come straight from global memory (a fragment row is one 32-byte sector) and the
// results go straight back; nothing is staged. With weights, grad_A uses B*W[PW[e]], and
// X = A gO gives grad_B = X*W[PW[e]] and grad_W[PW[e]] += X*B.
// KT = ceil(K / 4), LT8 = ceil(L / 8).
template <typename S, int KT, int LT8, bool WEIGHTED>
__global__ void __launch_bounds__(128, 3)
opsa_vjp_mma(S* __restrict__ gA, S* __restrict__ gB, S* __restrict__ gW,
             const S* __restrict__ gO, const S* __restrict__ A, const S* __restrict__ B,
             const S* __restrict__ W, const int32_t* __restrict__ PW,
             const int64_t* __restrict__ offsets, int K, int L, int64_t nO, int64_t nW, Status st) {
    using T = double;
    using S2 = typename VecOf<S, 2>::type;
    constexpr int NTK = (KT + 1) / 2; // 8-wide tiles over K
    constexpr int KSL = 2 * LT8;      // k-steps over L
    constexpr int NTL = LT8;          // 8-wide tiles over L
    constexpr int KSK = KT;           // k-steps over K
    // Eight-entry tiles loaded per iteration (and again one iteration ahead): narrower scalars
    // need more tiles for the same number of bytes in flight.
    constexpr int TILES = sizeof(S) == 8 ? 1 : (WEIGHTED ? 2 : 4);
    struct RawTile {
        S a[KSK], b[KSL]; // b already multiplied by W[PW[e]] when there are weights
        int32_t wrow;
    };
    if (saw_unsorted(st)) return;     // the entry-per-lane kernel of the same call does the work
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0); // uniform for the compiler
    const int qr = lane >> 2, qc = lane & 3;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps;
    const int64_t rowsize = static_cast<int64_t>(K) * L;
    const bool want_a = gA != nullptr, want_b = gB != nullptr || (WEIGHTED && gW != nullptr);
    // two-scalar accesses to rows of B, W, grad_B: rows of even length in 16-byte (8-byte for
    // f32) aligned arrays; this kernel is the one that serves unaligned operands
    auto pair_aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % (2 * sizeof(S)) == 0; };
    const bool pair_ok = L % 2 == 0 && pair_aligned(gB) && (!WEIGHTED || (pair_aligned(B) && pair_aligned(W)));

    for (int64_t r = static_cast<int64_t>(blockIdx.x) * warps + warp; r < nO; r += nwarps) {
        const int64_t lo = offsets[r], hi = offsets[r + 1];
        if (lo >= hi) continue;
        const S* g = gO + r * rowsize;
        // gO[p] as the B operand of both products
        T ga_k[NTK][KSL]; // [k-step over l][n = k]: gO[k = 8 nt + qr][l = 4 ks + qc]
        T gb_k[NTL][KSK]; // [k-step over k][n = l]: gO[k = 4 ks + qc][l = 8 nt + qr]
#pragma unroll
        for (int nt = 0; nt < NTK; nt++)
#pragma unroll
            for (int ks = 0; ks < KSL; ks++) {
                const int k = 8 * nt + qr, l = 4 * ks + qc;
                ga_k[nt][ks] = (want_a && k < K && l < L) ? static_cast<T>(__ldg(g + k * L + l)) : T(0);
            }
#pragma unroll
        for (int nt = 0; nt < NTL; nt++)
#pragma unroll
            for (int ks = 0; ks < KSK; ks++) {
                const int k = 4 * ks + qc, l = 8 * nt + qr;
                gb_k[nt][ks] = (want_b && k < K && l < L) ? static_cast<T>(__ldg(g + k * L + l)) : T(0);
            }

        // A-operand fragments of the tile that starts at e0, as loaded: entry e0 + qr, column
        // 4 ks + qc of A and B (times W[PW[e]]).
        auto load_tile = [&](int64_t e0, RawTile& t) {
            const int64_t e = e0 + qr;
            const bool valid = e < hi;
            t.wrow = 0;
            if (WEIGHTED && valid) {
                t.wrow = __ldg(PW + e);
                if (clamp_index(t.wrow, static_cast<int32_t>(nW))) report_bad_index(st, 1);
            }
#pragma unroll
            for (int ks = 0; ks < KSK; ks++) {
                const int k = 4 * ks + qc;
                t.a[ks] = (want_b && valid && k < K) ? __ldg(A + e * K + k) : S(0);
            }
#pragma unroll
            for (int ks = 0; ks < KSL; ks++) {
                const int l = 4 * ks + qc;
                const bool in = want_a && valid && l < L;
                S v = in ? __ldg(B + e * L + l) : S(0);
                if (WEIGHTED && in) v *= __ldg(W + static_cast<int64_t>(t.wrow) * L + l);
                t.b[ks] = v;
            }
        };

        RawTile cur[TILES], nxt[TILES];
#pragma unroll
        for (int t = 0; t < TILES; t++) load_tile(lo + 8 * t, cur[t]);
        for (int64_t e_it = lo; e_it < hi; e_it += 8 * TILES) {
            if (e_it + 8 * TILES < hi) {
#pragma unroll
                for (int t = 0; t < TILES; t++) load_tile(e_it + 8 * TILES + 8 * t, nxt[t]);
            }
#pragma unroll
            for (int t = 0; t < TILES; t++) {
                const int64_t e0 = e_it + 8 * t;
                if (e0 >= hi) break;
                const int64_t e = e0 + qr;
                const bool valid = e < hi;
                const int32_t wrow = cur[t].wrow;
                if (want_a) {
                    T bf[KSL];
#pragma unroll
                    for (int ks = 0; ks < KSL; ks++) bf[ks] = static_cast<T>(cur[t].b[ks]);
#pragma unroll
                    for (int nt = 0; nt < NTK; nt++) {
                        T c[2];
                        dmma0(c, bf[0], ga_k[nt][0]);
#pragma unroll
                        for (int ks = 1; ks < KSL; ks++) dmma(c, bf[ks], ga_k[nt][ks]);
                        const int k = 8 * nt + 2 * qc;
                        S* dst = gA + e * K + k;
                        if (valid && k < K) dst[0] = static_cast<S>(c[0]);
                        if (valid && k + 1 < K) dst[1] = static_cast<S>(c[1]);
                    }
                }
                if (want_b) {
                    T af[KSK];
#pragma unroll
                    for (int ks = 0; ks < KSK; ks++) af[ks] = static_cast<T>(cur[t].a[ks]);
#pragma unroll
                    for (int nt = 0; nt < NTL; nt++) {
                        T c[2];
                        dmma0(c, af[0], gb_k[nt][0]);
#pragma unroll
                        for (int ks = 1; ks < KSK; ks++) dmma(c, af[ks], gb_k[nt][ks]);
                        const int l = 8 * nt + 2 * qc;
                        if (!valid || l >= L) continue;
                        const bool two = l + 1 < L;
                        if (WEIGHTED) {
                            const S* wp = W + static_cast<int64_t>(wrow) * L + l;
                            const S* bp = B + e * L + l;
                            T w0, w1 = T(0), b0, b1 = T(0);
                            if (pair_ok) {
                                const S2 w2 = *reinterpret_cast<const S2*>(wp);
                                const S2 b2 = *reinterpret_cast<const S2*>(bp);
                                w0 = w2.x, w1 = w2.y, b0 = b2.x, b1 = b2.y;
                            } else {
                                w0 = wp[0], b0 = bp[0];
                                if (two) w1 = wp[1], b1 = bp[1];
                            }
                            if (gW != nullptr) {
                                S* gw = gW + static_cast<int64_t>(wrow) * L + l;
                                red_add(gw, static_cast<S>(c[0] * b0));
                                if (two) red_add(gw + 1, static_cast<S>(c[1] * b1));
                            }
                            c[0] *= w0;
                            c[1] *= w1;
                        }
                        if (gB != nullptr) {
                            S* dst = gB + e * L + l;
                            if (pair_ok) {
                                S2 v2;
                                v2.x = static_cast<S>(c[0]), v2.y = static_cast<S>(c[1]);
                                *reinterpret_cast<S2*>(dst) = v2;
                            } else {
                                dst[0] = static_cast<S>(c[0]);
                                if (two) dst[1] = static_cast<S>(c[1]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < TILES; t++) cur[t] = nxt[t];
        }
    }
}

template <typename S, int KT, bool WEIGHTED, typename... Args>
void launch_vjp_mma_l(int L, unsigned blocks, cudaStream_t stream, Args... args) {
    switch ((L + 7) / 8) {
    case 1: opsa_vjp_mma<S, KT, 1, WEIGHTED><<<blocks, 128, 0, stream>>>(args...); break;
    case 2: opsa_vjp_mma<S, KT, 2, WEIGHTED><<<blocks, 128, 0, stream>>>(args...); break;
    case 3: opsa_vjp_mma<S, KT, 3, WEIGHTED><<<blocks, 128, 0, stream>>>(args...); break;
    default: opsa_vjp_mma<S, KT, 4, WEIGHTED><<<blocks, 128, 0, stream>>>(args...); break;
    }
}

template <typename S, bool WEIGHTED, typename... Args>
void launch_vjp_mma(int K, int L, unsigned blocks, cudaStream_t stream, Args... args) {
    switch ((K + 3) / 4) {
    case 1: launch_vjp_mma_l<S, 1, WEIGHTED>(L, blocks, stream, args...); break;
    case 2: launch_vjp_mma_l<S, 2, WEIGHTED>(L, blocks, stream, args...); break;
    case 3: launch_vjp_mma_l<S, 3, WEIGHTED>(L, blocks, stream, args...); break;
    default: launch_vjp_mma_l<S, 4, WEIGHTED>(L, blocks, stream, args...); break;
    }
}

template <typename T, int KP, int VL, bool WEIGHTED, typename... Args>
void launch_vjp_tile(const Call& call, const VjpPlan& plan, int64_t J, Args... args) {
    auto kernel = opsa_vjp_entries<T, KP, VL, WEIGHTED>;
    if (!plan.only_if_unsorted)
        note_kernel_f("opsa_vjp_entries<%s,KP=%d,VL=%d,W=%d>", scalar_name<T>(), KP, VL,
                      WEIGHTED ? 1 : 0);
    if (plan.smem > 48 * 1024) {
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(plan.smem)));
    }
    const int64_t blocks = ceil_div(J, plan.threads);
    kernel<<<static_cast<unsigned>(blocks), plan.threads, plan.smem, call.stream>>>(args..., plan,
                                                                                   call.status);
}

// Register-tile width along K: exact for K <= 8, next even value up to 16, chunks of 16 above.
inline int vjp_tile_k(int K) { return K <= 8 ? K : (K <= 16 ? (K + 1) / 2 * 2 : 16); }

template <typename T, int VL, bool WEIGHTED, typename... Args>
void dispatch_kp(int K, Args... args) {
    switch (vjp_tile_k(K)) {
    case 1: launch_vjp_tile<T, 1, VL, WEIGHTED>(args...); break;
    case 2: launch_vjp_tile<T, 2, VL, WEIGHTED>(args...); break;
    case 3: launch_vjp_tile<T, 3, VL, WEIGHTED>(args...); break;
    case 4: launch_vjp_tile<T, 4, VL, WEIGHTED>(args...); break;
    case 5: launch_vjp_tile<T, 5, VL, WEIGHTED>(args...); break;
    case 6: launch_vjp_tile<T, 6, VL, WEIGHTED>(args...); break;
    case 7: launch_vjp_tile<T, 7, VL, WEIGHTED>(args...); break;
    case 8: launch_vjp_tile<T, 8, VL, WEIGHTED>(args...); break;
    case 10: launch_vjp_tile<T, 10, VL, WEIGHTED>(args...); break;
    case 12: launch_vjp_tile<T, 12, VL, WEIGHTED>(args...); break;
    case 14: launch_vjp_tile<T, 14, VL, WEIGHTED>(args...); break;
    default: launch_vjp_tile<T, 16, VL, WEIGHTED>(args...); break;
    }
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
    plan.only_if_unsorted = false;
    // Sorted scatter index (checked on the device): the streaming tensor-core kernel, or for
    // f64 operands it cannot take (alignment) the kernel that loads its fragments from global
    // memory; otherwise, and whenever the index turns out unsorted, the entry-per-lane kernels
    // below do the work.
    const bool streaming = pipe_usable<T, WEIGHTED>(A, B, W, gO, K, L, true);
    if (K <= 16 && L <= 32 && (streaming || sizeof(T) == 8)) {
        const int sms = sm_count(call.device);
        SegmentTable seg = segment_table(call, P, J, nO);
        const int64_t* offsets = seg.offsets;
        bool launched = streaming && backward_pipe<T, WEIGHTED>(call, gA, gB, gW, gO, A, B, W, PW,
                                                                offsets, J, K, L, nO);
        if constexpr (sizeof(T) == 8) {
            if (!launched) {
                const unsigned blocks =
                    static_cast<unsigned>(std::min<int64_t>(ceil_div(nO, 4), sms * 3));
                note_kernel_f("opsa_vjp_mma<%s,KT=%d,LT8=%d,W=%d>", scalar_name<T>(), (K + 3) / 4,
                              (L + 7) / 8, WEIGHTED ? 1 : 0);
                launch_vjp_mma<T, WEIGHTED>(K, L, blocks, call.stream, gA, gB, gW, gO, A, B, W, PW,
                                            offsets, K, L, nO, nO, call.status);
                launched = true;
            }
        }
        MOPS_CUDA_OK(cudaGetLastError());
        release_table(call, seg.ref);
        if (launched) {
            if (seg.known_sorted) return;
            if (call.wait) {
                wait_stream(call);
                if (!host_saw_unsorted(call)) return;
            }
            plan.only_if_unsorted = true; // asynchronous calls cannot look: always enqueue
        }
    }
    const int KP = vjp_tile_k(K);
    plan.nkc = static_cast<int>(ceil_div(K, KP));
    plan.Kp = K | 1;
    plan.Lp = L | 1;
    const int tiles_l = 1 + (WEIGHTED ? 1 : 0) + (plan.nkc > 1 ? 1 : 0);
    const size_t per_entry = (plan.Kp + static_cast<size_t>(tiles_l) * plan.Lp) * sizeof(T);
    plan.threads = 128;
    while (plan.threads > 32 && plan.threads * per_entry > 96 * 1024) plan.threads /= 2;
    plan.smem = plan.threads * (per_entry + sizeof(int32_t));

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
            gA, gB, gW, gO, A, B, W, PW, P, J, K, L, nO, plan.only_if_unsorted, call.status);
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

// Second order, by composition of the first-order kernels (mops/src/opsa/cpu.tpp:114-246; the
// reference CUDA build throws "Not implemented", mops/src/opsa/opsa.cu:305-318):
//   ggO  = opsa(ggA, B) + opsa(A, ggB)
//   gA2  = grad_A of opsa_vjp(gO; ., B := ggB),   gB2 = grad_B of opsa_vjp(gO; A := ggA, .)
// A missing grad_grad input makes its terms vanish; a missing output is skipped.
template <typename T>
static __global__ void add_into(T* __restrict__ dst, const T* __restrict__ src, int64_t n) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        dst[i] += src[i];
}

template <typename scalar_t>
void mops::cuda::outer_product_scatter_add_vjp_vjp(
    Tensor<scalar_t, 3> grad_grad_output, Tensor<scalar_t, 2> grad_A_2,
    Tensor<scalar_t, 2> grad_B_2, Tensor<scalar_t, 2> grad_grad_A,
    Tensor<scalar_t, 2> grad_grad_B, Tensor<scalar_t, 3> grad_output, Tensor<scalar_t, 2> A,
    Tensor<scalar_t, 2> B, Tensor<int32_t, 1> indices_output) {
    const std::string op = "cuda_outer_product_scatter_add_vjp_vjp";
    grad_like(grad_grad_output, "grad_grad_output", grad_output, "grad_output", op);
    grad_like(grad_A_2, "grad_A_2", A, "A", op);
    grad_like(grad_B_2, "grad_B_2", B, "B", op);
    grad_like(grad_grad_A, "grad_grad_A", A, "A", op);
    grad_like(grad_grad_B, "grad_grad_B", B, "B", op);
    same_size(A, "A", 0, B, "B", 0, op);
    same_size(A, "A", 1, grad_output, "grad_output", 1, op);
    same_size(B, "B", 1, grad_output, "grad_output", 2, op);
    same_size(A, "A", 0, indices_output, "indices_output", 0, op);
    fits_int32(grad_output.shape[0], "grad_output.shape[0]", op);
    fits_int32(A.shape[1], "A.shape[1]", op);
    fits_int32(B.shape[1], "B.shape[1]", op);
    if (grad_grad_output.data == nullptr && grad_A_2.data == nullptr && grad_B_2.data == nullptr)
        return;
    const int64_t J = static_cast<int64_t>(A.shape[0]);
    const int K = static_cast<int>(A.shape[1]), L = static_cast<int>(B.shape[1]);
    const int64_t nO = static_cast<int64_t>(grad_output.shape[0]);
    const int64_t out_size = nO * K * L;
    const scalar_t *ggA = grad_grad_A.data, *ggB = grad_grad_B.data;
    const int32_t* P = indices_output.data;
    Call call = begin_call();
    if (grad_grad_output.data != nullptr && out_size > 0) {
        scalar_t* ggO = grad_grad_output.data;
        if (ggA != nullptr && ggB != nullptr) {
            forward<scalar_t, false>(call, ggO, ggA, B.data, nullptr, nullptr, P, J, K, L, nO);
            scalar_t* tmp =
                static_cast<scalar_t*>(scratch_alloc(call, out_size * sizeof(scalar_t)));
            forward<scalar_t, false>(call, tmp, A.data, ggB, nullptr, nullptr, P, J, K, L, nO);
            add_into<scalar_t><<<sm_count(call.device) * 8, 256, 0, call.stream>>>(ggO, tmp, out_size);
            MOPS_CUDA_OK(cudaGetLastError());
            scratch_free(call, tmp);
        } else if (ggA != nullptr) {
            forward<scalar_t, false>(call, ggO, ggA, B.data, nullptr, nullptr, P, J, K, L, nO);
        } else if (ggB != nullptr) {
            forward<scalar_t, false>(call, ggO, A.data, ggB, nullptr, nullptr, P, J, K, L, nO);
        } else {
            MOPS_CUDA_OK(cudaMemsetAsync(ggO, 0, out_size * sizeof(scalar_t), call.stream));
        }
    }
    if (grad_A_2.data != nullptr && J * K > 0) {
        if (ggB != nullptr)
            backward<scalar_t, false>(call, grad_A_2.data, nullptr, nullptr, grad_output.data,
                                      A.data, ggB, nullptr, nullptr, P, J, K, L, nO);
        else
            MOPS_CUDA_OK(cudaMemsetAsync(grad_A_2.data, 0, J * K * sizeof(scalar_t), call.stream));
    }
    if (grad_B_2.data != nullptr && J * L > 0) {
        if (ggA != nullptr)
            backward<scalar_t, false>(call, nullptr, grad_B_2.data, nullptr, grad_output.data, ggA,
                                      B.data, nullptr, nullptr, P, J, K, L, nO);
        else
            MOPS_CUDA_OK(cudaMemsetAsync(grad_B_2.data, 0, J * L * sizeof(scalar_t), call.stream));
    }
    end_call(call, op.c_str(), kOpsaIndexNames, 1);
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
