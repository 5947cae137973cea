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
// Design. The batch dimension is the parallel one: lane = row. A block loads its rows of
// every input with coalesced asynchronous copies and keeps them transposed in shared memory
// ([column][row], padded), so that each triplet's operands are conflict-free reads at
// warp-uniform offsets. The triplet list is the same for every row, so it is compiled once
// per call by a one-block "plan" kernel into tables the row kernels stream through L1 as
// 16-byte broadcasts: coefficients with ready-made shared-memory offsets, in three orders:
//   * by k, cut into runs of equal output column, for O and ggO;
//   * grouped by indices_A (stable), for gA and gA2;
//   * grouped by indices_B (stable), for gB and gB2.
// Every output element is then a plain sum over one group, accumulated in a register in
// ascending k (the order of the reference CPU loops) and stored once: no atomics, no
// read-modify-write chains in shared memory, no output tiles. Indices are range-checked by
// the plan kernel; they are plain int32, any size.
#include <algorithm>
#include <cstring>

#include "checks.hpp"
#include "device.cuh"

namespace mops_b200 {
namespace {

constexpr int kPlanThreads = 256;
constexpr uint32_t kFirstRun = 0x80000000u; // flag in run_col: first run of this output column

// One triplet with its operand offsets already multiplied by the tile stride.
template <typename T> struct alignas(16) Entry {
    T c;
    int32_t o1, o2;
};

template <typename T> struct Plan {
    // by k: (c, A offset, B offset); runs of equal output column
    Entry<T>* by_k;
    int32_t* run_end; // [n_runs] one past the last k of the run
    uint32_t* run_col; // [n_runs] output column | kFirstRun
    int32_t* zero_cols; // [n_zero] output columns no triplet writes
    // grouped by indices_A: (c, gO offset, B offset); grouped by indices_B: (c, gO offset, A offset)
    Entry<T>* by_a;
    Entry<T>* by_b;
    int32_t* a_start; // [nA + 1]
    int32_t* b_start; // [nB + 1]
    int32_t* first_k; // [nO] scratch: smallest k writing each output column
    int32_t* counts;  // [0] n_runs, [1] n_zero
    int32_t* cursor;  // [max(nA, nB) + 1] scratch for the sorts
};

// Stable counting sort of k = 0..K-1 by key[k] in [0, nbins), done by one warp so that equal
// keys keep ascending k. `emit(pos, k)` stores element k at sorted position pos.
template <typename Emit>
__device__ __forceinline__ void warp_stable_group(const int32_t* __restrict__ key, int nkeys,
                                                  int K, int nbins, int32_t* start,
                                                  int32_t* cursor, int lane, Emit emit) {
    for (int b = lane; b <= nbins; b += 32) cursor[b] = 0;
    __syncwarp();
    for (int k = lane; k < K; k += 32) {
        int32_t v = key[k];
        clamp_index(v, nkeys);
        atomicAdd(&cursor[v], 1);
    }
    __syncwarp();
    int run = 0;
    for (int b0 = 0; b0 <= nbins; b0 += 32) {
        const int b = b0 + lane;
        const int v = b < nbins ? cursor[b] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(kFullMask, incl, o);
            if (lane >= o) incl += t;
        }
        if (b <= nbins) {
            start[b] = run + incl - v;
            cursor[b] = run + incl - v;
        }
        run += __shfl_sync(kFullMask, incl, 31);
    }
    __syncwarp();
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int k = k0 + lane;
        const bool live = k < K;
        int32_t v = live ? key[k] : -1 - lane; // distinct dummies for idle lanes
        if (live) clamp_index(v, nkeys);
        const unsigned same = __match_any_sync(kFullMask, v);
        const int rank = __popc(same & ((1u << lane) - 1));
        const int leader = __ffs(same) - 1;
        int base = 0;
        if (live && lane == leader) {
            base = cursor[v];
            cursor[v] = base + __popc(same);
        }
        base = __shfl_sync(kFullMask, base, leader);
        if (live) emit(base + rank, k);
        __syncwarp();
    }
}

template <typename T>
__global__ void __launch_bounds__(kPlanThreads)
sap_plan(Plan<T> plan, const T* __restrict__ C, const int32_t* __restrict__ PA,
         const int32_t* __restrict__ PB, const int32_t* __restrict__ PO, int K, int nA, int nB,
         int nO, int stride, bool want_runs, bool want_groups, Status st) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ int n_runs_shared;

    // Range checks once for the whole call.
    for (int k = tid; k < K; k += kPlanThreads) {
        int32_t pa = PA[k], pb = PB[k], po = PO[k];
        if (clamp_index(pa, nA)) report_bad_index(st, 0);
        if (clamp_index(pb, nB)) report_bad_index(st, 1);
        if (clamp_index(po, nO)) report_bad_index(st, 2);
    }
    if (want_runs) {
        for (int o = tid; o < nO; o += kPlanThreads) plan.first_k[o] = INT32_MAX;
        __syncthreads();
        for (int k = tid; k < K; k += kPlanThreads) {
            int32_t pa = PA[k], pb = PB[k], po = PO[k];
            clamp_index(pa, nA);
            clamp_index(pb, nB);
            clamp_index(po, nO);
            plan.by_k[k] = Entry<T>{C[k], pa * stride, pb * stride};
            // a run starts where the output column changes
            int32_t prev = k == 0 ? -1 : PO[k - 1];
            if (k > 0) clamp_index(prev, nO);
            if (po != prev) atomicMin(&plan.first_k[po], k);
        }
        __syncthreads();
        if (warp == 0) {
            // compact the run starts, in order
            int n_runs = 0;
            for (int k0 = 0; k0 < K; k0 += 32) {
                const int k = k0 + lane;
                int32_t po = -1, prev = -1;
                if (k < K) {
                    po = PO[k];
                    clamp_index(po, nO);
                    if (k > 0) {
                        prev = PO[k - 1];
                        clamp_index(prev, nO);
                    }
                }
                const bool starts = k < K && po != prev;
                const unsigned m = __ballot_sync(kFullMask, starts);
                if (starts) {
                    const int r = n_runs + __popc(m & ((1u << lane) - 1));
                    plan.run_col[r] = static_cast<uint32_t>(po) |
                                      (plan.first_k[po] == k ? kFirstRun : 0u);
                    if (r > 0) plan.run_end[r - 1] = k;
                }
                n_runs += __popc(m);
            }
            if (lane == 0) {
                if (n_runs > 0) plan.run_end[n_runs - 1] = K;
                plan.counts[0] = n_runs;
                n_runs_shared = n_runs;
            }
        } else if (warp == 1) {
            // output columns nobody writes
            int n_zero = 0;
            for (int o0 = 0; o0 < nO; o0 += 32) {
                const int o = o0 + lane;
                const bool empty = o < nO && plan.first_k[o] == INT32_MAX;
                const unsigned m = __ballot_sync(kFullMask, empty);
                if (empty) plan.zero_cols[n_zero + __popc(m & ((1u << lane) - 1))] = o;
                n_zero += __popc(m);
            }
            if (lane == 0) plan.counts[1] = n_zero;
        }
    }
    __syncthreads();
    if (want_groups && warp == 0) {
        warp_stable_group(PA, nA, K, nA, plan.a_start, plan.cursor, lane, [&](int pos, int k) {
            int32_t pb = PB[k], po = PO[k];
            clamp_index(pb, nB);
            clamp_index(po, nO);
            plan.by_a[pos] = Entry<T>{C[k], po * stride, pb * stride};
        });
        warp_stable_group(PB, nB, K, nB, plan.b_start, plan.cursor, lane, [&](int pos, int k) {
            int32_t pa = PA[k], po = PO[k];
            clamp_index(pa, nA);
            clamp_index(po, nO);
            plan.by_b[pos] = Entry<T>{C[k], po * stride, pa * stride};
        });
    }
    (void)n_runs_shared;
}

// A transposed operand tile in shared memory: element (row, col) at data[col * stride + row].
template <typename T>
__device__ __forceinline__ void tile_load(T* tile, int cols, const T* __restrict__ M, int64_t i0,
                                          int64_t I, int R, int stride) {
    const int tid = threadIdx.x;
    const int64_t rows = I - i0 < R ? I - i0 : R;
    const int valid = static_cast<int>(rows) * cols, total = R * cols;
    const T* src = M == nullptr ? nullptr : M + i0 * cols;
    const int dr = R / cols, dc = R - dr * cols;
    int row = tid / cols, c = tid - row * cols;
    for (int idx = tid; idx < total; idx += R) {
        if (src != nullptr && idx < valid)
            cp_async<sizeof(T)>(tile + c * stride + row, src + idx);
        else
            tile[c * stride + row] = T(0);
        row += dr;
        c += dc;
        if (c >= cols) {
            c -= cols;
            row++;
        }
    }
}

template <typename T> __device__ __forceinline__ Entry<T> fetch(const Entry<T>* p) {
    static_assert(sizeof(Entry<T>) == 16, "table entries are read as one 16-byte broadcast");
    const int4 raw = __ldg(reinterpret_cast<const int4*>(p));
    Entry<T> e;
    memcpy(&e, &raw, 16);
    return e;
}

// Shared-memory entry read: one 16-byte broadcast.
template <typename T> __device__ __forceinline__ Entry<T> fetch_shared(const Entry<T>* p) {
    const int4 raw = *reinterpret_cast<const int4*>(p);
    Entry<T> e;
    memcpy(&e, &raw, 16);
    return e;
}

template <bool IN_SMEM, typename T>
__device__ __forceinline__ Entry<T> get(const Entry<T>* p) {
    return IN_SMEM ? fetch_shared(p) : fetch(p);
}

// Copies a plan table into shared memory (the row tiles stream through L1 and would evict
// it there); returns the pointer the row loop should read. `slot` is 16-byte aligned.
template <bool IN_SMEM, typename T>
__device__ __forceinline__ const Entry<T>* stage_table(const Entry<T>* table, int K,
                                                       unsigned char* slot) {
    if (!IN_SMEM) return table;
    Entry<T>* dst = reinterpret_cast<Entry<T>*>(slot);
    for (int k = threadIdx.x; k < K; k += blockDim.x) cp_async<16>(dst + k, table + k);
    return dst;
}

__host__ __device__ inline size_t up16(size_t n) { return (n + 15) / 16 * 16; }

template <typename T, bool IN_SMEM>
__global__ void sap_fwd_rows(T* __restrict__ O, const T* __restrict__ A, const T* __restrict__ B,
                             Plan<T> plan, int64_t I, int nA, int nB, int nO, int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = blockDim.x, S = R + 1, tid = threadIdx.x;
    T* At = reinterpret_cast<T*>(smem_raw);
    T* Bt = At + static_cast<size_t>(nA) * S;
    unsigned char* tables = smem_raw + up16(static_cast<size_t>(nA + nB) * S * sizeof(T));
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * R;
    tile_load(At, nA, A, i0, I, R, S);
    tile_load(Bt, nB, B, i0, I, R, S);
    const Entry<T>* by_k = stage_table<IN_SMEM>(plan.by_k, K, tables);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    if (i0 + tid >= I) return;

    const T* a = At + tid;
    const T* b = Bt + tid;
    T* o = O + (i0 + tid) * nO;
    const int n_runs = plan.counts[0], n_zero = plan.counts[1];
    int k = 0;
    for (int r = 0; r < n_runs; r++) {
        const int end = __ldg(plan.run_end + r);
        const uint32_t col = __ldg(plan.run_col + r);
        T acc = T(0);
#pragma unroll 4
        for (; k < end; k++) {
            const Entry<T> e = get<IN_SMEM>(by_k + k);
            acc += e.c * a[e.o1] * b[e.o2];
        }
        T* dst = o + (col & ~kFirstRun);
        if (col & kFirstRun)
            *dst = acc;
        else
            *dst += acc; // unsorted indices_output: a later run of an earlier column
    }
    for (int z = 0; z < n_zero; z++) o[__ldg(plan.zero_cols + z)] = T(0);
}

// gX[i, x] = sum over the group of x of (G[i, o1] * c) * Y[i, o2], for both groupings.
template <bool IN_SMEM, typename T>
__device__ __forceinline__ void grouped_sums(T* __restrict__ out_row, int n_groups,
                                             const int32_t* __restrict__ start,
                                             const Entry<T>* __restrict__ table, const T* g,
                                             const T* y) {
    int x = __ldg(start);
    for (int grp = 0; grp < n_groups; grp++) {
        const int end = __ldg(start + grp + 1);
        T acc = T(0);
#pragma unroll 4
        for (; x < end; x++) {
            const Entry<T> e = get<IN_SMEM>(table + x);
            acc += g[e.o1] * e.c * y[e.o2];
        }
        out_row[grp] = acc;
    }
}

template <typename T, bool IN_SMEM>
__global__ void sap_vjp_rows(T* __restrict__ gA, T* __restrict__ gB, const T* __restrict__ gO,
                             const T* __restrict__ A, const T* __restrict__ B, Plan<T> plan,
                             int64_t I, int nA, int nB, int nO, int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = blockDim.x, S = R + 1, tid = threadIdx.x;
    T* At = reinterpret_cast<T*>(smem_raw);
    T* Bt = At + static_cast<size_t>(nA) * S;
    T* Gt = Bt + static_cast<size_t>(nB) * S;
    unsigned char* tables = smem_raw + up16(static_cast<size_t>(nA + nB + nO) * S * sizeof(T));
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * R;
    if (gB != nullptr) tile_load(At, nA, A, i0, I, R, S);
    if (gA != nullptr) tile_load(Bt, nB, B, i0, I, R, S);
    tile_load(Gt, nO, gO, i0, I, R, S);
    const Entry<T>* by_a = stage_table<IN_SMEM>(plan.by_a, gA != nullptr ? K : 0, tables);
    const Entry<T>* by_b = stage_table<IN_SMEM>(plan.by_b, gB != nullptr ? K : 0,
                                                tables + static_cast<size_t>(K) * sizeof(Entry<T>));
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    if (i0 + tid >= I) return;
    const int64_t i = i0 + tid;
    if (gA != nullptr)
        grouped_sums<IN_SMEM>(gA + i * nA, nA, plan.a_start, by_a, Gt + tid, Bt + tid);
    if (gB != nullptr)
        grouped_sums<IN_SMEM>(gB + i * nB, nB, plan.b_start, by_b, Gt + tid, At + tid);
}

template <typename T, bool IN_SMEM>
__global__ void sap_vjp_vjp_rows(T* __restrict__ ggO, T* __restrict__ gA2, T* __restrict__ gB2,
                                 const T* __restrict__ ggA, const T* __restrict__ ggB,
                                 const T* __restrict__ gO, const T* __restrict__ A,
                                 const T* __restrict__ B, Plan<T> plan, int64_t I, int nA, int nB,
                                 int nO, int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = blockDim.x, S = R + 1, tid = threadIdx.x;
    T* At = reinterpret_cast<T*>(smem_raw);
    T* Bt = At + static_cast<size_t>(nA) * S;
    T* Gt = Bt + static_cast<size_t>(nB) * S;
    T* hAt = Gt + static_cast<size_t>(nO) * S;
    T* hBt = hAt + static_cast<size_t>(nA) * S;
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * R;
    tile_load(At, nA, A, i0, I, R, S);
    tile_load(Bt, nB, B, i0, I, R, S);
    tile_load(Gt, nO, gO, i0, I, R, S);
    tile_load(hAt, nA, ggA, i0, I, R, S); // a missing second-order input reads as zeros
    tile_load(hBt, nB, ggB, i0, I, R, S);
    unsigned char* tables =
        smem_raw + up16(static_cast<size_t>(2 * nA + 2 * nB + nO) * S * sizeof(T));
    const size_t table_bytes = static_cast<size_t>(K) * sizeof(Entry<T>);
    const Entry<T>* by_k = stage_table<IN_SMEM>(plan.by_k, ggO != nullptr ? K : 0, tables);
    const Entry<T>* by_a = stage_table<IN_SMEM>(plan.by_a, gA2 != nullptr ? K : 0, tables + table_bytes);
    const Entry<T>* by_b = stage_table<IN_SMEM>(plan.by_b, gB2 != nullptr ? K : 0, tables + 2 * table_bytes);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    if (i0 + tid >= I) return;
    const int64_t i = i0 + tid;
    if (ggO != nullptr) {
        const T *a = At + tid, *b = Bt + tid, *ha = hAt + tid, *hb = hBt + tid;
        T* o = ggO + i * nO;
        const int n_runs = plan.counts[0], n_zero = plan.counts[1];
        int k = 0;
        for (int r = 0; r < n_runs; r++) {
            const int end = __ldg(plan.run_end + r);
            const uint32_t col = __ldg(plan.run_col + r);
            T acc = T(0);
            for (; k < end; k++) {
                const Entry<T> e = get<IN_SMEM>(by_k + k);
                acc += ha[e.o1] * b[e.o2] * e.c;
                acc += hb[e.o2] * a[e.o1] * e.c;
            }
            T* dst = o + (col & ~kFirstRun);
            if (col & kFirstRun)
                *dst = acc;
            else
                *dst += acc;
        }
        for (int z = 0; z < n_zero; z++) o[__ldg(plan.zero_cols + z)] = T(0);
    }
    // gA2[i,pa] = sum c ggB[i,pb] gO[i,po];  gB2[i,pb] = sum c ggA[i,pa] gO[i,po]
    if (gA2 != nullptr)
        grouped_sums<IN_SMEM>(gA2 + i * nA, nA, plan.a_start, by_a, Gt + tid, hBt + tid);
    if (gB2 != nullptr)
        grouped_sums<IN_SMEM>(gB2 + i * nB, nB, plan.b_start, by_b, Gt + tid, hAt + tid);
}

struct Triplet {
    int32_t pa, pb, po;
};

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

// Rows per block and whether the plan tables go to shared memory. Prefers the tables in
// shared memory and a footprint that lets two blocks share an SM; returns 0 rows if not even
// 32 rows of tiles fit in the opt-in limit (then the global-memory kernel is used).
template <typename T>
int rows_per_block(const Call& call, int cols, int n_tables, int64_t K, size_t* smem,
                   bool* tables_in_smem) {
    const size_t limit = static_cast<size_t>(max_optin_smem(call.device));
    const size_t tables = static_cast<size_t>(n_tables) * K * sizeof(Entry<T>);
    for (int pass = 0; pass < 3; pass++) {
        for (int R : {128, 64, 32}) {
            const size_t tiles = up16(static_cast<size_t>(cols) * (R + 1) * sizeof(T));
            const size_t total = tiles + (pass < 2 ? tables : 0);
            const size_t cap = pass == 0 ? 112 * 1024 : limit;
            if (total <= cap) {
                *smem = total;
                *tables_in_smem = pass < 2;
                return R;
            }
        }
    }
    return 0;
}

template <typename Kernel> void allow_smem(Kernel kernel, size_t smem) {
    if (smem > 48 * 1024)
        MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
}

// Allocates the call-scoped plan tables and runs the plan kernel.
template <typename T>
Plan<T> make_plan(const Call& call, TableRef* scratch, const T* C, const int32_t* PA,
                  const int32_t* PB, const int32_t* PO, int64_t K, int nA, int nB, int nO,
                  int stride, bool want_runs, bool want_groups) {
    const size_t table = up16(static_cast<size_t>(K) * sizeof(Entry<T>));
    const size_t ints_k = up16(static_cast<size_t>(K) * sizeof(int32_t));
    const size_t ints_o = up16(static_cast<size_t>(nO) * sizeof(int32_t));
    const size_t ints_a = up16((static_cast<size_t>(nA) + 1) * sizeof(int32_t));
    const size_t ints_b = up16((static_cast<size_t>(nB) + 1) * sizeof(int32_t));
    const size_t total = 3 * table + 2 * ints_k + 2 * ints_o + 2 * ints_a + 2 * ints_b + 16 +
                         std::max(ints_a, ints_b);
    TableKey key{};
    key.kind = kSapTable;
    key.scalar_bytes = static_cast<int>(sizeof(T));
    key.ptr[0] = C, key.ptr[1] = PA, key.ptr[2] = PB, key.ptr[3] = PO;
    key.n[0] = K, key.n[1] = nA, key.n[2] = nB, key.n[3] = nO, key.n[4] = stride;
    key.n[5] = want_runs ? 1 : 0, key.n[6] = want_groups ? 1 : 0;
    *scratch = acquire_table(call, key, total);
    unsigned char* p = static_cast<unsigned char*>(scratch->ptr);
    Plan<T> plan;
    auto take = [&](size_t bytes) {
        unsigned char* q = p;
        p += bytes;
        return q;
    };
    plan.by_k = reinterpret_cast<Entry<T>*>(take(table));
    plan.by_a = reinterpret_cast<Entry<T>*>(take(table));
    plan.by_b = reinterpret_cast<Entry<T>*>(take(table));
    plan.run_end = reinterpret_cast<int32_t*>(take(ints_k));
    plan.run_col = reinterpret_cast<uint32_t*>(take(ints_k));
    plan.zero_cols = reinterpret_cast<int32_t*>(take(ints_o));
    plan.first_k = reinterpret_cast<int32_t*>(take(ints_o));
    plan.a_start = reinterpret_cast<int32_t*>(take(ints_a));
    plan.b_start = reinterpret_cast<int32_t*>(take(ints_b));
    plan.counts = reinterpret_cast<int32_t*>(take(16));
    plan.cursor = reinterpret_cast<int32_t*>(take(std::max(ints_a, ints_b)));
    if (scratch->fresh) {
        sap_plan<T><<<1, kPlanThreads, 0, call.stream>>>(plan, C, PA, PB, PO, static_cast<int>(K),
                                                         nA, nB, nO, stride, want_runs,
                                                         want_groups, call.status);
        MOPS_CUDA_OK(cudaGetLastError());
        commit_table(call, *scratch);
    }
    return plan;
}

// ------------------------------------------------------------ small-operand kernels
// When one of A, B has at most 16 columns (angular channels up to l = 7) its row fits in
// registers. Call it S and the other operand T. Sorting the triplets by (output column, S
// column) turns the forward sum into
//     O[i, o] = sum_s S[i, s] * ( sum_{k in (o, s)} C_k T[i, PT_k] ),
// with s a compile-time index in the unrolled loop, so only T is read from shared memory: one
// operand read per triplet instead of two. Sorted by (T column, S column) the VJP becomes
//     inner = sum_{k in (t, s)} C_k gO[i, PO_k]
//     gT[i, t] = sum_s S[i, s] inner,      gS[i, s] = sum_t T[i, t] inner,
// one operand read per triplet instead of four, and gS accumulates in registers.
constexpr int kSmallPad = 2; // zero entries after the last triplet (the row loops read ahead)

template <typename T> struct SmallPlan {
    Entry<T>* table; // sorted triplets: (c, tile offset of the streamed operand, unused)
    int32_t* start;  // [groups * NS + 1] first triplet of every (group, s)
    int32_t* cursor; // scratch of the same size
};

// mode 0 (forward): groups = output columns, streamed operand = T.
// mode 1 (VJP):     groups = T columns,      streamed operand = gO.
template <typename T>
__global__ void __launch_bounds__(kPlanThreads)
sap_plan_small(SmallPlan<T> plan, const T* __restrict__ C, const int32_t* __restrict__ PS,
               const int32_t* __restrict__ PT, const int32_t* __restrict__ PO, int K, int nS,
               int nT, int nO, int NS, int stride, int mode, int bit_s, int bit_t, Status st) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < kSmallPad) plan.table[K + tid] = Entry<T>{T(0), 0, 0}; // read ahead by the row loops
    for (int k = tid; k < K; k += kPlanThreads) {
        int32_t ps = PS[k], pt = PT[k], po = PO[k];
        if (clamp_index(ps, nS)) report_bad_index(st, bit_s);
        if (clamp_index(pt, nT)) report_bad_index(st, bit_t);
        if (clamp_index(po, nO)) report_bad_index(st, 2);
    }
    if (warp != 0) return;
    const int groups = mode == 0 ? nO : nT, nbins = groups * NS;
    auto key_of = [&](int k) {
        int32_t ps = PS[k], g = mode == 0 ? PO[k] : PT[k];
        clamp_index(ps, nS);
        clamp_index(g, groups);
        return g * NS + ps;
    };
    int32_t* cursor = plan.cursor;
    for (int b = lane; b <= nbins; b += 32) cursor[b] = 0;
    __syncwarp();
    for (int k = lane; k < K; k += 32) atomicAdd(&cursor[key_of(k)], 1);
    __syncwarp();
    int run = 0;
    for (int b0 = 0; b0 <= nbins; b0 += 32) {
        const int b = b0 + lane;
        const int v = b < nbins ? cursor[b] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(kFullMask, incl, o);
            if (lane >= o) incl += t;
        }
        if (b <= nbins) {
            plan.start[b] = run + incl - v;
            cursor[b] = run + incl - v;
        }
        run += __shfl_sync(kFullMask, incl, 31);
    }
    __syncwarp();
    for (int k0 = 0; k0 < K; k0 += 32) { // stable: equal keys keep ascending k
        const int k = k0 + lane;
        const bool live = k < K;
        const int32_t v = live ? key_of(k) : -1 - lane;
        const unsigned same = __match_any_sync(kFullMask, v);
        const int rank = __popc(same & ((1u << lane) - 1));
        const int leader = __ffs(same) - 1;
        int base = 0;
        if (live && lane == leader) {
            base = cursor[v];
            cursor[v] = base + __popc(same);
        }
        base = __shfl_sync(kFullMask, base, leader);
        if (live) {
            int32_t x = mode == 0 ? PT[k] : PO[k];
            clamp_index(x, mode == 0 ? nT : nO);
            plan.table[base + rank] = Entry<T>{C[k], x * stride, 0};
        }
        __syncwarp();
    }
}

// Row i of the small operand into registers (zero beyond its width).
template <typename T, int NS>
__device__ __forceinline__ void load_small_row(T (&s)[NS], const T* __restrict__ S, int64_t i,
                                               int nS) {
#pragma unroll
    for (int q = 0; q < NS; q++) s[q] = q < nS ? __ldg(S + i * nS + q) : T(0);
}

// Copies the plan's tables into shared memory behind the tiles.
template <typename T>
__device__ __forceinline__ void stage_small(const SmallPlan<T>& plan, int K, int nbins,
                                            unsigned char* slot, const Entry<T>*& table,
                                            const int32_t*& start) {
    Entry<T>* t = reinterpret_cast<Entry<T>*>(slot);
    int32_t* st =
        reinterpret_cast<int32_t*>(slot + static_cast<size_t>(K + kSmallPad) * sizeof(Entry<T>));
    for (int k = threadIdx.x; k < K + kSmallPad; k += blockDim.x)
        cp_async<16>(t + k, plan.table + k);
    for (int b = threadIdx.x; b <= nbins; b += blockDim.x) cp_async<4>(st + b, plan.start + b);
    table = t;
    start = st;
}

template <typename T, int NS>
__global__ void sap_fwd_small(T* __restrict__ O, const T* __restrict__ S, const T* __restrict__ Tm,
                              SmallPlan<T> plan, int64_t I, int nS, int nT, int nO, int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = blockDim.x, stride = R + 1, tid = threadIdx.x;
    T* Tt = reinterpret_cast<T*>(smem_raw);
    unsigned char* tables = smem_raw + up16(static_cast<size_t>(nT) * stride * sizeof(T));
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * R;
    tile_load(Tt, nT, Tm, i0, I, R, stride);
    const Entry<T>* table;
    const int32_t* start;
    stage_small(plan, K, nO * NS, tables, table, start);
    cp_async_commit();
    const int64_t i = i0 + tid;
    T sreg[NS];
    load_small_row<T, NS>(sreg, S, i < I ? i : I - 1, nS);
    cp_async_wait<0>();
    __syncthreads();
    if (i >= I) return;
    const T* t = Tt + tid;
    T* o = O + i * nO;
    // The triplets are one stream across all groups, read two ahead: (c0, v0) is triplet k with
    // its operand already loaded, e1 is triplet k + 1.
    // (small batches: gridDim.y blocks share a block of rows, each takes a range of columns)
    const int col_lo = static_cast<int>(static_cast<int64_t>(nO) * blockIdx.y / gridDim.y);
    const int col_hi = static_cast<int>(static_cast<int64_t>(nO) * (blockIdx.y + 1) / gridDim.y);
    int k = start[col_lo * NS];
    Entry<T> e1 = fetch_shared(table + k);
    T c0 = e1.c, v0 = t[e1.o1];
    e1 = fetch_shared(table + k + 1);
    for (int col = col_lo; col < col_hi; col++) {
        const int32_t* bounds = start + col * NS + 1;
        T acc = T(0);
#pragma unroll
        for (int q = 0; q < NS; q++) {
            const int end = bounds[q];
            T inner = T(0);
            for (; k < end; k++) {
                const Entry<T> e2 = fetch_shared(table + k + 2);
                const T v1 = t[e1.o1];
                inner += c0 * v0;
                c0 = e1.c, v0 = v1, e1 = e2;
            }
            acc += sreg[q] * inner;
        }
        o[col] = acc;
    }
}

template <typename T, int NS>
__global__ void sap_vjp_small(T* __restrict__ gS, T* __restrict__ gT, const T* __restrict__ gO,
                              const T* __restrict__ S, const T* __restrict__ Tm,
                              SmallPlan<T> plan, int64_t I, int nS, int nT, int nO, int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = blockDim.x, stride = R + 1, tid = threadIdx.x;
    // only gO is gathered by runtime column: T[i, t] is read once per t, straight from global
    // memory (the row's few sectors stay in L1), which leaves the shared memory to more rows
    T* Gt = reinterpret_cast<T*>(smem_raw);
    unsigned char* tables = smem_raw + up16(static_cast<size_t>(nO) * stride * sizeof(T));
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * R;
    tile_load(Gt, nO, gO, i0, I, R, stride);
    const Entry<T>* table;
    const int32_t* start;
    stage_small(plan, K, nT * NS, tables, table, start);
    cp_async_commit();
    const int64_t i = i0 + tid;
    T sreg[NS], gs[NS];
    load_small_row<T, NS>(sreg, S, i < I ? i : I - 1, nS);
#pragma unroll
    for (int q = 0; q < NS; q++) gs[q] = T(0);
    cp_async_wait<0>();
    __syncthreads();
    if (i >= I) return;
    const T* g = Gt + tid;
    const T* t = Tm + i * nT;
    int k = 0; // one stream of triplets read two ahead, as in the forward kernel
    Entry<T> e1 = fetch_shared(table);
    T c0 = e1.c, v0 = g[e1.o1];
    e1 = fetch_shared(table + 1);
    for (int col = 0; col < nT; col++) {
        const int32_t* bounds = start + col * NS + 1;
        const T tv = gS != nullptr ? __ldg(t + col) : T(0);
        T acc = T(0);
#pragma unroll
        for (int q = 0; q < NS; q++) {
            const int end = bounds[q];
            T inner = T(0);
            for (; k < end; k++) {
                const Entry<T> e2 = fetch_shared(table + k + 2);
                const T v1 = g[e1.o1];
                inner += c0 * v0;
                c0 = e1.c, v0 = v1, e1 = e2;
            }
            acc += sreg[q] * inner;
            gs[q] += tv * inner;
        }
        if (gT != nullptr) gT[i * nT + col] = acc;
    }
    if (gS != nullptr) {
#pragma unroll
        for (int q = 0; q < NS; q++)
            if (q < nS) gS[i * nS + q] = gs[q];
    }
}

// Width of the register-resident operand (4, 8 or 16), or 0 when neither operand is small.
inline int small_width(int nA, int nB) {
    const int n = std::min(nA, nB);
    return n <= 4 ? 4 : n <= 8 ? 8 : n <= 16 ? 16 : 0;
}

// Rows per block for tiles of `cols` columns plus the small plan's tables: the block size that
// puts the most warps on an SM within its shared memory and registers (the tables are per
// block, the tiles per row); 0 if 32 rows do not fit.
template <typename T>
int rows_small(const Call& call, const void* kernel, int cols, int64_t K, int nbins,
               size_t* smem, int64_t batch) {
    cudaFuncAttributes attr{};
    MOPS_CUDA_OK(cudaFuncGetAttributes(&attr, kernel));
    const int regs = std::max(attr.numRegs, 1);
    const size_t limit = static_cast<size_t>(max_optin_smem(call.device));
    const size_t per_sm = 228 * 1024, reserved = 1024;
    const size_t tables = up16(static_cast<size_t>(K + kSmallPad) * sizeof(Entry<T>) +
                               (static_cast<size_t>(nbins) + 1) * 4);
    int best_r = 0, best_warps = 0;
    for (int R : {32, 64, 96, 128, 160, 192, 256, 320, 384, 512}) {
        const size_t total = up16(static_cast<size_t>(cols) * (R + 1) * sizeof(T)) + tables;
        if (total > limit || R * regs > 65536) break;
        const int by_smem = static_cast<int>(std::min<size_t>(per_sm / (total + reserved), 32));
        const int blocks = std::min(by_smem, 65536 / (regs * R));
        const int warps = std::min(blocks * (R / 32), 64);
        if (warps > best_warps) {
            best_warps = warps;
            best_r = R;
            *smem = total;
        }
        // A batch too small to give every SM a block of this size: the smallest block spreads
        // the rows over the most SMs (the work per row does not depend on the block size).
        if (R == 32 && batch <= static_cast<int64_t>(sm_count(call.device)) * 64) return R;
    }
    return best_r;
}

template <typename T>
SmallPlan<T> make_small_plan(const Call& call, TableRef* scratch, const T* C, const int32_t* PS,
                             const int32_t* PT, const int32_t* PO, int64_t K, int nS, int nT,
                             int nO, int NS, int stride, int mode, int bit_s, int bit_t) {
    const size_t nbins = static_cast<size_t>(mode == 0 ? nO : nT) * NS;
    const size_t table = up16(static_cast<size_t>(K + kSmallPad) * sizeof(Entry<T>));
    const size_t ints = up16((nbins + 1) * sizeof(int32_t));
    TableKey key{};
    key.kind = kSapSmallTable;
    key.scalar_bytes = static_cast<int>(sizeof(T));
    key.ptr[0] = C, key.ptr[1] = PS, key.ptr[2] = PT, key.ptr[3] = PO;
    key.n[0] = K, key.n[1] = nS, key.n[2] = nT, key.n[3] = nO, key.n[4] = NS, key.n[5] = stride;
    key.n[6] = mode, key.n[7] = bit_s, key.n[8] = bit_t;
    *scratch = acquire_table(call, key, table + 2 * ints);
    unsigned char* p = static_cast<unsigned char*>(scratch->ptr);
    SmallPlan<T> plan;
    plan.table = reinterpret_cast<Entry<T>*>(p);
    plan.start = reinterpret_cast<int32_t*>(p + table);
    plan.cursor = reinterpret_cast<int32_t*>(p + table + ints);
    if (scratch->fresh) {
        sap_plan_small<T><<<1, kPlanThreads, 0, call.stream>>>(
            plan, C, PS, PT, PO, static_cast<int>(K), nS, nT, nO, NS, stride, mode, bit_s, bit_t,
            call.status);
        MOPS_CUDA_OK(cudaGetLastError());
        commit_table(call, *scratch);
    }
    return plan;
}

// Forward with the narrower of A, B in registers. Returns false if it does not apply.
template <typename T>
bool forward_small(const Call& call, T* O, const T* A, const T* B, const T* C, const int32_t* PA,
                   const int32_t* PB, const int32_t* PO, int64_t I, int64_t K, int nA, int nB,
                   int nO) {
    const int NS = small_width(nA, nB);
    if (NS == 0 || static_cast<int64_t>(nO) * NS > (1 << 20)) return false;
    const bool b_small = nB <= nA;
    const T *S = b_small ? B : A, *Tm = b_small ? A : B;
    const int32_t *PS = b_small ? PB : PA, *PT = b_small ? PA : PB;
    const int nS = b_small ? nB : nA, nT = b_small ? nA : nB;
    size_t smem = 0;
    const void* kernel = NS == 4   ? reinterpret_cast<const void*>(sap_fwd_small<T, 4>)
                         : NS == 8 ? reinterpret_cast<const void*>(sap_fwd_small<T, 8>)
                                   : reinterpret_cast<const void*>(sap_fwd_small<T, 16>);
    const int R = rows_small<T>(call, kernel, nT, K, nO * NS, &smem, I);
    if (R == 0) return false;
    TableRef scratch{};
    SmallPlan<T> plan = make_small_plan<T>(call, &scratch, C, PS, PT, PO, K, nS, nT, nO, NS, R + 1,
                                           0, b_small ? 1 : 0, b_small ? 0 : 1);
    const int64_t row_blocks = ceil_div(I, R);
    // few row blocks: split the output columns over up to eight blocks per block of rows
    const int col_parts = static_cast<int>(std::max<int64_t>(
        1, std::min<int64_t>(std::min(nO, 8), 2 * sm_count(call.device) / row_blocks)));
    const dim3 blocks(static_cast<unsigned>(row_blocks), static_cast<unsigned>(col_parts));
    note_kernel_f("sap_fwd_small<%s,NS=%d> rows/block=%d", scalar_name<T>(), NS, R);
#define MOPS_B200_LAUNCH(NS_)                                                                      \
    {                                                                                              \
        allow_smem(sap_fwd_small<T, NS_>, smem);                                                   \
        sap_fwd_small<T, NS_><<<blocks, R, smem, call.stream>>>(O, S, Tm, plan, I, nS, nT, nO,     \
                                                                static_cast<int>(K));              \
    }
    if (NS == 4) MOPS_B200_LAUNCH(4) else if (NS == 8) MOPS_B200_LAUNCH(8) else MOPS_B200_LAUNCH(16)
#undef MOPS_B200_LAUNCH
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, scratch);
    return true;
}

template <typename T>
bool backward_small(const Call& call, T* gA, T* gB, const T* gO, const T* A, const T* B,
                    const T* C, const int32_t* PA, const int32_t* PB, const int32_t* PO, int64_t I,
                    int64_t K, int nA, int nB, int nO) {
    const int NS = small_width(nA, nB);
    if (NS == 0) return false;
    const bool b_small = nB <= nA;
    const T *S = b_small ? B : A, *Tm = b_small ? A : B;
    T *gS = b_small ? gB : gA, *gT = b_small ? gA : gB;
    const int32_t *PS = b_small ? PB : PA, *PT = b_small ? PA : PB;
    const int nS = b_small ? nB : nA, nT = b_small ? nA : nB;
    if (static_cast<int64_t>(nT) * NS > (1 << 20)) return false;
    size_t smem = 0;
    const void* kernel = NS == 4   ? reinterpret_cast<const void*>(sap_vjp_small<T, 4>)
                         : NS == 8 ? reinterpret_cast<const void*>(sap_vjp_small<T, 8>)
                                   : reinterpret_cast<const void*>(sap_vjp_small<T, 16>);
    const int R = rows_small<T>(call, kernel, nO, K, nT * NS, &smem, I);
    if (R == 0) return false;
    TableRef scratch{};
    SmallPlan<T> plan = make_small_plan<T>(call, &scratch, C, PS, PT, PO, K, nS, nT, nO, NS, R + 1,
                                           1, b_small ? 1 : 0, b_small ? 0 : 1);
    const unsigned blocks = static_cast<unsigned>(ceil_div(I, R));
    note_kernel_f("sap_vjp_small<%s,NS=%d> rows/block=%d", scalar_name<T>(), NS, R);
#define MOPS_B200_LAUNCH(NS_)                                                                      \
    {                                                                                              \
        allow_smem(sap_vjp_small<T, NS_>, smem);                                                   \
        sap_vjp_small<T, NS_><<<blocks, R, smem, call.stream>>>(gS, gT, gO, S, Tm, plan, I, nS,    \
                                                                nT, nO, static_cast<int>(K));      \
    }
    if (NS == 4) MOPS_B200_LAUNCH(4) else if (NS == 8) MOPS_B200_LAUNCH(8) else MOPS_B200_LAUNCH(16)
#undef MOPS_B200_LAUNCH
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, scratch);
    return true;
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
    fits_int32(C.shape[0], "C.shape[0]", op);
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
    if (forward_small<scalar_t>(call, output.data, A.data, B.data, C.data, indices_A.data,
                                indices_B.data, indices_output.data, I, K, nA, nB, nO)) {
        end_call(call, op.c_str(), kIndexNames, 3);
        return;
    }
    size_t smem = 0;
    bool in_smem = false;
    const int R = rows_per_block<scalar_t>(call, nA + nB, 1, K, &smem, &in_smem);
    if (R > 0) {
        TableRef scratch{};
        Plan<scalar_t> plan = make_plan<scalar_t>(call, &scratch, C.data, indices_A.data,
                                                  indices_B.data, indices_output.data, K, nA, nB,
                                                  nO, R + 1, true, false);
        auto kernel = in_smem ? sap_fwd_rows<scalar_t, true> : sap_fwd_rows<scalar_t, false>;
        note_kernel_f("sap_fwd_rows<%s,smem=%d>", scalar_name<scalar_t>(), in_smem ? 1 : 0);
        allow_smem(kernel, smem);
        kernel<<<static_cast<unsigned>(ceil_div(I, R)), R, smem, call.stream>>>(
            output.data, A.data, B.data, plan, I, nA, nB, nO, static_cast<int>(K));
        MOPS_CUDA_OK(cudaGetLastError());
        release_table(call, scratch);
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
    if (backward_small<scalar_t>(call, grad_A.data, grad_B.data, grad_output.data, A.data, B.data,
                                 C.data, indices_A.data, indices_B.data, indices_output.data, I, K,
                                 nA, nB, nO)) {
        end_call(call, op.c_str(), kIndexNames, 3);
        return;
    }
    size_t smem = 0;
    bool in_smem = false;
    const int R = rows_per_block<scalar_t>(call, nA + nB + nO, 2, K, &smem, &in_smem);
    if (R > 0) {
        TableRef scratch{};
        Plan<scalar_t> plan = make_plan<scalar_t>(call, &scratch, C.data, indices_A.data,
                                                  indices_B.data, indices_output.data, K, nA, nB,
                                                  nO, R + 1, false, true);
        auto kernel = in_smem ? sap_vjp_rows<scalar_t, true> : sap_vjp_rows<scalar_t, false>;
        allow_smem(kernel, smem);
        kernel<<<static_cast<unsigned>(ceil_div(I, R)), R, smem, call.stream>>>(
            grad_A.data, grad_B.data, grad_output.data, A.data, B.data, plan, I, nA, nB, nO,
            static_cast<int>(K));
        MOPS_CUDA_OK(cudaGetLastError());
        release_table(call, scratch);
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
    bool in_smem = false;
    const int R = rows_per_block<scalar_t>(call, 2 * nA + 2 * nB + nO, 3, K, &smem, &in_smem);
    if (R > 0) {
        TableRef scratch{};
        Plan<scalar_t> plan = make_plan<scalar_t>(call, &scratch, C.data, indices_A.data,
                                                  indices_B.data, indices_output.data, K, nA, nB,
                                                  nO, R + 1, true, true);
        auto kernel =
            in_smem ? sap_vjp_vjp_rows<scalar_t, true> : sap_vjp_vjp_rows<scalar_t, false>;
        allow_smem(kernel, smem);
        kernel<<<static_cast<unsigned>(ceil_div(I, R)), R, smem, call.stream>>>(
            grad_grad_output.data, grad_A_2.data, grad_B_2.data, grad_grad_A.data,
            grad_grad_B.data, grad_output.data, A.data, B.data, plan, I, nA, nB, nO,
            static_cast<int>(K));
        MOPS_CUDA_OK(cudaGetLastError());
        release_table(call, scratch);
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
