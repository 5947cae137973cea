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
// loads them with coalesced asynchronous copies and keeps them transposed in shared memory
// ([factor][row], padded), so that "factor P[j,k] of my row" is a conflict-free read at a
// warp-uniform offset: lane = row. The monomial table is the same for every row, so a
// one-block plan kernel compiles it once per call into packed tables of ready-made
// shared-memory offsets, which the row kernels stream through double-buffered shared-memory
// stages (cp.async) and read as 16-byte broadcasts:
//   forward: the monomials in order; the block's four warps take interleaved monomials and
//            add their partial sums at the end;
//   VJP:     the (j,k) incidences grouped by the factor n they differentiate (stable
//            counting sort), each with the offsets of the monomial's other K-1 factors. Then
//            gA[i,n] is a plain sum over group n, accumulated in a register and stored once:
//            no atomics and no read-modify-write chain; the four warps take disjoint ranges
//            of n, balanced by incidence count.
#include <algorithm>

#include "checks.hpp"
#include "device.cuh"

namespace mops_b200 {
namespace {

constexpr int kRows = 32;       // batch rows per block (one per lane)
constexpr int kPad = kRows + 1; // shared-memory row stride of a transposed tile
constexpr int kWarps = 4;
constexpr int kMaxOrder = 10;
constexpr int kPlanThreads = 256;
constexpr int kFwdChunk = 256; // monomials per forward stage (whole block)
constexpr int kVjpChunk = 64;  // incidences per VJP stage (per warp)

// One table record: a coefficient followed by NF 16-bit tile offsets (in scalars: column
// n of the transposed tile starts at n * kPad, which fits 16 bits for every tile that fits in
// shared memory), padded to 8, 16 or 32 bytes so that one or two broadcast loads fetch it.
__host__ __device__ constexpr int record_bytes(int scalar_bytes, int nf) {
    const int raw = scalar_bytes + 2 * (nf > 0 ? nf : 0);
    return raw <= 8 ? 8 : raw <= 16 ? 16 : 32;
}
constexpr int kMaxTileColumns = 65535 / kPad;

template <typename T, int NF>
__device__ __forceinline__ T read_record(const unsigned char* rec, int (&o)[NF > 0 ? NF : 1]) {
    constexpr int B = record_bytes(sizeof(T), NF);
    unsigned w[B / 4];
    if constexpr (B == 8) {
        const uint2 v = *reinterpret_cast<const uint2*>(rec);
        w[0] = v.x, w[1] = v.y;
    } else {
#pragma unroll
        for (int q = 0; q < B / 16; q++) {
            const uint4 v = *reinterpret_cast<const uint4*>(rec + 16 * q);
            w[4 * q] = v.x, w[4 * q + 1] = v.y, w[4 * q + 2] = v.z, w[4 * q + 3] = v.w;
        }
    }
    constexpr int first = sizeof(T) / 4; // word where the offsets start
#pragma unroll
    for (int k = 0; k < NF; k++) {
        const unsigned word = w[first + k / 2];
        o[k] = (k & 1) ? (word >> 16) : (word & 0xffffu);
    }
    if constexpr (sizeof(T) == 8)
        return __hiloint2double(static_cast<int>(w[1]), static_cast<int>(w[0]));
    else
        return __uint_as_float(w[0]);
}

template <typename T>
__device__ __forceinline__ void write_record(unsigned char* rec, int bytes, T coef) {
    for (int q = 0; q < bytes / 4; q++) reinterpret_cast<unsigned*>(rec)[q] = 0u;
    *reinterpret_cast<T*>(rec) = coef;
}
template <typename T>
__device__ __forceinline__ void write_offset(unsigned char* rec, int q, int offset) {
    reinterpret_cast<uint16_t*>(rec + sizeof(T))[q] = static_cast<uint16_t>(offset);
}

struct HpePlan {
    unsigned char* fwd_rec; // [J]    C[j] and the tile offsets of monomial j's K factors
    unsigned char* vjp_rec; // [J*K]  grouped by differentiated factor: C[j], the other K-1 offsets
    int32_t* n_start;       // [N + 1]       first incidence of every factor
    int32_t* split;         // [kWarps + 1]  factor ranges of the block's warps
    int32_t* cursor;        // [plan warps][N + 1] scratch
};

// Loads rows [i0, i0+rows) of a row-major [I][N] matrix into tile[n*(rows+1) + row].
template <typename T>
__device__ __forceinline__ void load_tile_transposed(T* tile, const T* __restrict__ M, int64_t i0,
                                                     int64_t I, int N, int tid, int nthreads,
                                                     int rows = kRows) {
    const int pad = rows + 1;
    const int64_t have = I - i0 < rows ? I - i0 : rows;
    const int total = rows * N;
    const int valid = static_cast<int>(have) * N;
    const T* src = M + i0 * N;
    const int dr = nthreads / N, dn = nthreads - dr * N;
    int row = tid / N, n = tid - row * N;
    for (int idx = tid; idx < total; idx += nthreads) {
        if (idx < valid)
            cp_async<sizeof(T)>(tile + n * pad + row, src + idx);
        else
            tile[n * pad + row] = T(0);
        row += dr;
        n += dn;
        if (n >= N) {
            n -= N;
            row++;
        }
    }
}

// Builds the packed tables. One block; the grouping is a stable counting sort (equal factors
// keep ascending (j,k), so the sums are reproducible).
template <typename T>
__global__ void __launch_bounds__(kPlanThreads)
hpe_plan(HpePlan plan, const T* __restrict__ C, const int32_t* __restrict__ P, int J, int K,
         int N, bool want_fwd, bool want_vjp, int pad, Status st) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int fwd_bytes = record_bytes(sizeof(T), K), vjp_bytes = record_bytes(sizeof(T), K - 1);
    const int M = J * K;
    for (int x = tid; x < M; x += kPlanThreads) {
        int32_t p = P[x];
        if (clamp_index(p, N)) report_bad_index(st, 0);
    }
    if (want_fwd) {
        for (int j = tid; j < J; j += kPlanThreads) {
            unsigned char* rec = plan.fwd_rec + static_cast<size_t>(j) * fwd_bytes;
            write_record<T>(rec, fwd_bytes, C[j]);
            for (int k = 0; k < K; k++) {
                int32_t p = P[j * K + k];
                clamp_index(p, N);
                write_offset<T>(rec, k, p * pad);
            }
        }
    }
    if (!want_vjp || M == 0) return;
    // Stable counting sort of the J*K incidences by factor. Every warp takes a contiguous
    // chunk of the incidences; per-(warp, factor) counts turn into each warp's own write
    // cursors, so equal factors keep ascending (j, k) across and within the chunks.
    constexpr int kPlanWarps = kPlanThreads / 32;
    const int stride = N + 1;
    int32_t* cnt = plan.cursor; // [kPlanWarps][N + 1]
    const int chunk = ((M + kPlanWarps - 1) / kPlanWarps + 31) / 32 * 32;
    const int x_lo = min(warp * chunk, M), x_hi = min(x_lo + chunk, M);
    for (int i = tid; i < kPlanWarps * stride; i += kPlanThreads) cnt[i] = 0;
    __syncthreads();
    for (int x = x_lo + lane; x < x_hi; x += 32) {
        int32_t p = P[x];
        clamp_index(p, N);
        atomicAdd(&cnt[warp * stride + p], 1);
    }
    __syncthreads();
    for (int b = tid; b < N; b += kPlanThreads) { // counts -> offsets of each warp inside factor b
        int run = 0;
        for (int w = 0; w < kPlanWarps; w++) {
            const int v = cnt[w * stride + b];
            cnt[w * stride + b] = run;
            run += v;
        }
        plan.n_start[b] = run; // total, scanned below
    }
    __syncthreads();
    if (warp == 0) {
        int run = 0;
        for (int b0 = 0; b0 <= N; b0 += 32) {
            const int b = b0 + lane;
            const int v = b < N ? plan.n_start[b] : 0;
            int incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(kFullMask, incl, o);
                if (lane >= o) incl += t;
            }
            if (b <= N) plan.n_start[b] = run + incl - v;
            run += __shfl_sync(kFullMask, incl, 31);
        }
    }
    __syncthreads();
    for (int i = tid; i < kPlanWarps * N; i += kPlanThreads) {
        const int w = i / N, b = i - w * N;
        cnt[w * stride + b] += plan.n_start[b];
    }
    __syncthreads();
    int32_t* cursor = cnt + warp * stride;
    for (int x0 = x_lo; x0 < x_hi; x0 += 32) {
        const int x = x0 + lane;
        const bool live = x < x_hi;
        int32_t key = -1 - lane;
        if (live) {
            key = P[x];
            clamp_index(key, N);
        }
        const unsigned same = __match_any_sync(kFullMask, key);
        const int rank = __popc(same & ((1u << lane) - 1));
        const int leader = __ffs(same) - 1;
        int base = 0;
        if (live && lane == leader) {
            base = cursor[key];
            cursor[key] = base + __popc(same);
        }
        base = __shfl_sync(kFullMask, base, leader);
        if (live) {
            const int pos = base + rank, j = x / K, k = x - j * K;
            unsigned char* rec = plan.vjp_rec + static_cast<size_t>(pos) * vjp_bytes;
            write_record<T>(rec, vjp_bytes, C[j]);
            int q = 0;
            for (int l = 0; l < K; l++) {
                if (l == k) continue;
                int32_t p = P[j * K + l];
                clamp_index(p, N);
                write_offset<T>(rec, q++, p * pad);
            }
        }
        __syncwarp();
    }
    // Factor ranges of the row kernel's four warps, balanced by incidence count.
    if (warp == 0 && lane <= kWarps) {
        int n = 0;
        if (lane == kWarps) {
            n = N;
        } else if (lane > 0) {
            const int target = static_cast<int>(static_cast<int64_t>(M) * lane / kWarps);
            int lo = 0, hi = N; // first n with n_start[n] >= target
            while (lo < hi) {
                const int mid = (lo + hi) / 2;
                if (plan.n_start[mid] < target)
                    lo = mid + 1;
                else
                    hi = mid;
            }
            n = lo;
        }
        plan.split[lane] = n;
    }
}

// R rows per lane (lane works on rows lane + 32 r of the block's 32 R-row tile): one record read
// serves R rows.
template <typename T, int K, int R>
__global__ void __launch_bounds__(kWarps * 32)
hpe_fwd_rows(T* __restrict__ O, const T* __restrict__ A, const unsigned char* __restrict__ records,
             int64_t I, int N, int J) {
    constexpr int RB = record_bytes(sizeof(T), K);
    constexpr int kStageBytes = kFwdChunk * RB;
    constexpr int unit = RB >= 16 ? 16 : 8;
    constexpr int kTileRows = 32 * R;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // layout: stage 0 records | stage 1 records | A tile | partial
    T* At = reinterpret_cast<T*>(smem_raw + 2 * kStageBytes);
    T* partial = At + static_cast<size_t>(N) * (kTileRows + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * kTileRows;

    auto issue = [&](int stage, int m0) {
        const int mc = J - m0 < kFwdChunk ? J - m0 : kFwdChunk;
        const unsigned char* src = records + static_cast<int64_t>(m0) * RB;
        unsigned char* dst = smem_raw + stage * kStageBytes;
        for (int x = tid * unit; x < mc * RB; x += kWarps * 32 * unit) cp_async<unit>(dst + x, src + x);
        cp_async_commit();
    };

    load_tile_transposed(At, A, i0, I, N, tid, kWarps * 32, kTileRows);
    if (J > 0) issue(0, 0);

    const T* col = At + lane;
    T acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = T(0);
    int stage = 0;
    for (int m0 = 0; m0 < J; m0 += kFwdChunk, stage ^= 1) {
        const int mc = J - m0 < kFwdChunk ? J - m0 : kFwdChunk;
        if (m0 + kFwdChunk < J) {
            issue(stage ^ 1, m0 + kFwdChunk);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const unsigned char* recs = smem_raw + stage * kStageBytes;
#pragma unroll 4
        for (int m = warp; m < mc; m += kWarps) {
            int o[K > 0 ? K : 1];
            const T c = read_record<T, K>(recs + m * RB, o);
#pragma unroll
            for (int r = 0; r < R; r++) {
                T prod = c;
#pragma unroll
                for (int k = 0; k < K; k++) prod *= col[o[k] + 32 * r];
                acc[r] += prod;
            }
        }
        __syncthreads(); // the stage is overwritten by the copy issued next round
    }
    if (J == 0) {
        cp_async_wait<0>();
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < R; r++) partial[warp * kTileRows + 32 * r + lane] = acc[r];
    __syncthreads();
    for (int row = tid; row < kTileRows; row += kWarps * 32) {
        if (i0 + row < I) {
            T sum = partial[row];
#pragma unroll
            for (int w = 1; w < kWarps; w++) sum += partial[w * kTileRows + row];
            O[i0 + row] = sum;
        }
    }
}

// R rows per lane (lane works on rows lane + 32 r of the block's 32 R-row tile): one record read
// serves R rows.
template <typename T, int K, int R>
__global__ void __launch_bounds__(kWarps * 32)
hpe_vjp_rows(T* __restrict__ gA, const T* __restrict__ gO, const T* __restrict__ A, HpePlan plan,
             int64_t I, int N) {
    constexpr int NF = K - 1 > 0 ? K - 1 : 0;
    constexpr int RB = record_bytes(sizeof(T), NF);
    constexpr int kStageBytes = kVjpChunk * RB;
    constexpr int unit = RB >= 16 ? 16 : 8;
    constexpr int kTileRows = 32 * R;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // layout: per warp 2 stages of records | A tile
    T* At = reinterpret_cast<T*>(smem_raw + kWarps * 2 * kStageBytes);
    const int tid = threadIdx.x, lane = tid & 31;
    // the shuffle tells the compiler that the warp number (and the incidence range and loop
    // counts derived from it) is the same in all lanes
    const int warp = __shfl_sync(kFullMask, tid >> 5, 0);
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * kTileRows;
    unsigned char* recs_w = smem_raw + warp * 2 * kStageBytes;

    load_tile_transposed(At, A, i0, I, N, tid, kWarps * 32, kTileRows);
    cp_async_commit();

    const int n_lo = __ldg(plan.split + warp), n_hi = __ldg(plan.split + warp + 1);
    const int x_lo = __ldg(plan.n_start + n_lo), x_hi = __ldg(plan.n_start + n_hi);

    auto issue = [&](int stage, int x0) {
        const int xc = x_hi - x0 < kVjpChunk ? x_hi - x0 : kVjpChunk;
        const unsigned char* src = plan.vjp_rec + static_cast<int64_t>(x0) * RB;
        unsigned char* dst = recs_w + stage * kStageBytes;
        for (int y = lane * unit; y < xc * RB; y += 32 * unit) cp_async<unit>(dst + y, src + y);
        cp_async_commit();
    };
    if (x_lo < x_hi) issue(0, x_lo);
    // The A tile was committed first: waiting for "all but the newest group" covers it.
    if (x_lo < x_hi)
        cp_async_wait<1>();
    else
        cp_async_wait<0>();
    __syncthreads();

    T go[R];
    bool live[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        live[r] = i0 + lane + 32 * r < I;
        go[r] = live[r] ? gO[i0 + lane + 32 * r] : T(0);
    }
    const T* col = At + lane;
    T* out = gA + (i0 + lane) * N;
    constexpr int U = R == 1 ? 4 : R == 2 ? 2 : 1; // independent partial sums per row

    int n = n_lo;
    int end_n = n < n_hi ? __ldg(plan.n_start + n + 1) : x_hi;
    T acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = T(0);
    auto close_group = [&] {
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (live[r]) out[static_cast<int64_t>(32 * r) * N + n] = go[r] * acc[r];
            acc[r] = T(0);
        }
    };
    int stage = 0;
    for (int x0 = x_lo; x0 < x_hi; x0 += kVjpChunk, stage ^= 1) {
        const int xc = x_hi - x0 < kVjpChunk ? x_hi - x0 : kVjpChunk;
        if (x0 + kVjpChunk < x_hi) {
            issue(stage ^ 1, x0 + kVjpChunk);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        const unsigned char* recs = recs_w + stage * kStageBytes;
        // One term per row: C_j times the other K-1 factors of incidence y of this stage.
        auto add_term = [&](int y, T (&sum)[R]) {
            int o[NF > 0 ? NF : 1];
            const T c = read_record<T, NF>(recs + y * RB, o);
#pragma unroll
            for (int r = 0; r < R; r++) {
                T prod = c;
#pragma unroll
                for (int k = 0; k < NF; k++) prod *= col[o[k] + 32 * r];
                sum[r] += prod;
            }
        };
        int y = 0;
        while (y < xc) {
            while (x0 + y == end_n) { // group n is complete (possibly empty)
                close_group();
                n++;
                end_n = __ldg(plan.n_start + n + 1);
            }
            // the rest of group n that lies in this stage: no group test inside
            const int run_end = min(xc, end_n - x0);
            T part[U > 1 ? U - 1 : 1][R];
#pragma unroll
            for (int u = 0; u < U - 1; u++)
#pragma unroll
                for (int r = 0; r < R; r++) part[u][r] = T(0);
            for (; y + U <= run_end; y += U) {
                add_term(y, acc);
#pragma unroll
                for (int u = 1; u < U; u++) add_term(y + u, part[u - 1]);
            }
            for (; y < run_end; y++) add_term(y, acc);
#pragma unroll
            for (int u = 0; u < U - 1; u++)
#pragma unroll
                for (int r = 0; r < R; r++) acc[r] += part[u][r];
        }
        __syncwarp(); // the stage is overwritten by the copy issued next round
    }
    // Close the last group and any empty groups after it.
    for (; n < n_hi; n++) close_group();
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

template <typename T, int K> size_t fwd_smem(int N, int rows_per_lane = 1) {
    const int rows = 32 * rows_per_lane;
    return 2 * kFwdChunk * record_bytes(sizeof(T), K) +
           (static_cast<size_t>(N) * (rows + 1) + kWarps * rows) * sizeof(T);
}

template <typename T, int K> size_t vjp_smem(int N, int rows_per_lane = 1) {
    return kWarps * 2 * kVjpChunk * record_bytes(sizeof(T), K - 1) +
           static_cast<size_t>(N) * (32 * rows_per_lane + 1) * sizeof(T);
}

// Allocates the call-scoped tables and runs the plan kernel.
template <typename T>
HpePlan make_plan(const Call& call, TableRef* scratch, const T* C, const int32_t* P, int64_t J,
                  int K, int N, bool want_fwd, bool want_vjp, int pad = kPad) {
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    const size_t M = static_cast<size_t>(J) * K;
    const size_t b_fwd = want_fwd ? up(static_cast<size_t>(J) * record_bytes(sizeof(T), K)) : 0;
    const size_t b_vjp = want_vjp ? up(M * record_bytes(sizeof(T), K - 1)) : 0;
    const size_t b_n = up((static_cast<size_t>(N) + 1) * sizeof(int32_t));
    const size_t b_cur = up((kPlanThreads / 32) * (static_cast<size_t>(N) + 1) * sizeof(int32_t));
    TableKey key{};
    key.kind = kHpeTable;
    key.scalar_bytes = static_cast<int>(sizeof(T));
    key.ptr[0] = C, key.ptr[1] = P;
    key.n[0] = J, key.n[1] = K, key.n[2] = N, key.n[3] = want_fwd ? 1 : 0;
    key.n[4] = want_vjp ? 1 : 0, key.n[5] = pad;
    *scratch = acquire_table(call, key, b_fwd + b_vjp + b_n + b_cur + 256);
    unsigned char* p = static_cast<unsigned char*>(scratch->ptr);
    HpePlan plan;
    plan.fwd_rec = p;
    p += b_fwd;
    plan.vjp_rec = p;
    p += b_vjp;
    plan.n_start = reinterpret_cast<int32_t*>(p);
    p += b_n;
    plan.cursor = reinterpret_cast<int32_t*>(p);
    p += b_cur;
    plan.split = reinterpret_cast<int32_t*>(p);
    if (scratch->fresh) {
        hpe_plan<T><<<1, kPlanThreads, 0, call.stream>>>(plan, C, P, static_cast<int>(J), K, N,
                                                         want_fwd, want_vjp, pad, call.status);
        MOPS_CUDA_OK(cudaGetLastError());
        commit_table(call, *scratch);
    }
    return plan;
}

// ---------------------------------------------------------------- small batches
// With one lane per batch row, a batch of a thousand rows is 32 blocks and most of the GPU
// idles while every block walks the whole table. For small batches the roles are swapped: one
// warp per batch row (its A row in shared memory, record offsets = column numbers), lanes over
// the monomials (forward) or over the incidences of one factor (VJP), one shuffle reduction per
// result. A thousand rows are then a thousand warps.
constexpr int kSmallWarps = 8;
constexpr int64_t kSmallBatch = 8192; // rows up to which the warp-per-row kernels are used

template <typename T, int K>
__global__ void __launch_bounds__(kSmallWarps * 32)
hpe_fwd_warp(T* __restrict__ O, const T* __restrict__ A, const unsigned char* __restrict__ rec,
             int64_t I, int N, int J) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int RB = record_bytes(sizeof(T), K);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * kSmallWarps + warp;
    if (i >= I) return;
    T* row = reinterpret_cast<T*>(smem_raw) + static_cast<size_t>(warp) * N;
    for (int n = lane; n < N; n += 32) row[n] = A[i * N + n];
    __syncwarp();
    T acc = T(0);
    for (int j = lane; j < J; j += 32) {
        int o[K > 0 ? K : 1];
        T term = read_record<T, K>(rec + static_cast<size_t>(j) * RB, o);
#pragma unroll
        for (int k = 0; k < K; k++) term *= row[o[k]];
        acc += term;
    }
    acc = warp_sum(acc);
    if (lane == 0) O[i] = acc;
}

template <typename T, int K>
__global__ void __launch_bounds__(kSmallWarps * 32)
hpe_vjp_warp(T* __restrict__ gA, const T* __restrict__ gO, const T* __restrict__ A, HpePlan plan,
             int64_t I, int N) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int NF = K - 1;
    constexpr int RB = record_bytes(sizeof(T), NF);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * kSmallWarps + warp;
    int32_t* starts = reinterpret_cast<int32_t*>(
        smem_raw + static_cast<size_t>(N) * kSmallWarps * sizeof(T)); // [N + 1]
    for (int n = threadIdx.x; n <= N; n += blockDim.x) starts[n] = plan.n_start[n];
    __syncthreads();
    if (i >= I) return;
    T* row = reinterpret_cast<T*>(smem_raw) + static_cast<size_t>(warp) * N;
    for (int n = lane; n < N; n += 32) row[n] = A[i * N + n];
    __syncwarp();
    const T g = gO[i];
    T mine = T(0); // lane (n & 31) keeps the result of factor n until 32 of them go out together
    // four factors at a time, so that their shuffle reductions overlap
    for (int n0 = 0; n0 < N; n0 += 4) {
        T acc[4];
#pragma unroll
        for (int f = 0; f < 4; f++) {
            acc[f] = T(0);
            const int n = n0 + f < N ? n0 + f : N - 1;
            const int lo = starts[n], hi = n0 + f < N ? starts[n + 1] : lo;
            for (int x = lo + lane; x < hi; x += 32) {
                int o[NF > 0 ? NF : 1];
                T term = read_record<T, NF>(plan.vjp_rec + static_cast<size_t>(x) * RB, o);
#pragma unroll
                for (int k = 0; k < NF; k++) term *= row[o[k]];
                acc[f] += term;
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1)
#pragma unroll
            for (int f = 0; f < 4; f++) acc[f] += __shfl_xor_sync(kFullMask, acc[f], d);
#pragma unroll
        for (int f = 0; f < 4; f++)
            if (lane == ((n0 + f) & 31)) mine = g * acc[f];
        const int last = n0 + 3 < N ? n0 + 3 : N - 1;
        if ((last & 31) == 31 || last == N - 1) {
            const int col = (last & ~31) + lane;
            if (col <= last) gA[i * N + col] = mine;
        }
    }
}

template <typename T, int K>
void launch_fwd(const Call& call, T* O, const T* A, const T* C, const int32_t* P, int64_t I,
                int N, int64_t J) {
    if (I <= kSmallBatch && static_cast<size_t>(N) * kSmallWarps * sizeof(T) <= 48 * 1024) {
        TableRef scratch{};
        HpePlan plan = make_plan<T>(call, &scratch, C, P, J, K, N, true, false, 1);
        note_kernel_f("hpe_fwd_warp<%s,K=%d>", scalar_name<T>(), K);
        hpe_fwd_warp<T, K><<<static_cast<unsigned>(ceil_div(I, kSmallWarps)), kSmallWarps * 32,
                             static_cast<size_t>(N) * kSmallWarps * sizeof(T), call.stream>>>(
            O, A, plan.fwd_rec, I, N, static_cast<int>(J));
        MOPS_CUDA_OK(cudaGetLastError());
        release_table(call, scratch);
        return;
    }
    // Two rows per lane when the batch still fills the GPU that way and the wider tile fits.
    const size_t smem2 = fwd_smem<T, K>(N, 2);
    const bool two = I >= static_cast<int64_t>(sm_count(call.device)) * 64 * 8 &&
                     smem2 <= 75 * 1024 && static_cast<int64_t>(N) * 65 <= 65535;
    const size_t smem = two ? smem2 : fwd_smem<T, K>(N);
    TableRef scratch{};
    HpePlan plan = make_plan<T>(call, &scratch, C, P, J, K, N, true, false, two ? 65 : kPad);
    note_kernel_f("hpe_fwd_rows<%s,K=%d,R=%d>", scalar_name<T>(), K, two ? 2 : 1);
    if (two) {
        auto kernel = hpe_fwd_rows<T, K, 2>;
        if (smem > 48 * 1024)
            MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              static_cast<int>(smem)));
        kernel<<<static_cast<unsigned>(ceil_div(I, 64)), kWarps * 32, smem, call.stream>>>(
            O, A, plan.fwd_rec, I, N, static_cast<int>(J));
    } else {
        auto kernel = hpe_fwd_rows<T, K, 1>;
        if (smem > 48 * 1024)
            MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              static_cast<int>(smem)));
        kernel<<<static_cast<unsigned>(ceil_div(I, kRows)), kWarps * 32, smem, call.stream>>>(
            O, A, plan.fwd_rec, I, N, static_cast<int>(J));
    }
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, scratch);
}

template <typename T, int K>
void launch_vjp(const Call& call, T* gA, const T* gO, const T* A, const T* C, const int32_t* P,
                int64_t I, int N, int64_t J) {
    if (K == 0 || J == 0) { // no factor depends on A
        MOPS_CUDA_OK(cudaMemsetAsync(gA, 0, I * N * sizeof(T), call.stream));
        return;
    }
    if (I <= kSmallBatch && static_cast<size_t>(N) * kSmallWarps * sizeof(T) +
                                    (static_cast<size_t>(N) + 1) * sizeof(int32_t) <= 48 * 1024) {
        TableRef scratch{};
        HpePlan plan = make_plan<T>(call, &scratch, C, P, J, K, N, false, true, 1);
        note_kernel_f("hpe_vjp_warp<%s,K=%d>", scalar_name<T>(), K);
        hpe_vjp_warp<T, K><<<static_cast<unsigned>(ceil_div(I, kSmallWarps)), kSmallWarps * 32,
                             static_cast<size_t>(N) * kSmallWarps * sizeof(T) +
                                 (static_cast<size_t>(N) + 1) * sizeof(int32_t),
                             call.stream>>>(
            gA, gO, A, plan, I, N);
        MOPS_CUDA_OK(cudaGetLastError());
        release_table(call, scratch);
        return;
    }
    // Several rows per lane when the batch still fills the GPU that way and the wider tile fits.
    int rpl = 1;
    for (int r : {4, 2}) {
        if (I >= static_cast<int64_t>(sm_count(call.device)) * 32 * r * 8 &&
            vjp_smem<T, K>(N, r) <= 112 * 1024 &&
            static_cast<int64_t>(N) * (32 * r + 1) <= 65535) {
            rpl = r;
            break;
        }
    }
    const size_t smem = vjp_smem<T, K>(N, rpl);
    TableRef scratch{};
    HpePlan plan = make_plan<T>(call, &scratch, C, P, J, K, N, false, true, 32 * rpl + 1);
    auto launch = [&](auto kernel) {
        if (smem > 48 * 1024)
            MOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              static_cast<int>(smem)));
        kernel<<<static_cast<unsigned>(ceil_div(I, 32 * rpl)), kWarps * 32, smem, call.stream>>>(
            gA, gO, A, plan, I, N);
    };
    note_kernel_f("hpe_vjp_rows<%s,K=%d,R=%d>", scalar_name<T>(), K, rpl);
    if (rpl == 4)
        launch(hpe_vjp_rows<T, K, 4>);
    else if (rpl == 2)
        launch(hpe_vjp_rows<T, K, 2>);
    else
        launch(hpe_vjp_rows<T, K, 1>);
    MOPS_CUDA_OK(cudaGetLastError());
    release_table(call, scratch);
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

// Forward / VJP of an already checked problem on the call's stream (tile kernels when a
// 32-row tile of A fits in shared memory, the global-memory kernels otherwise).
template <typename T>
void run_forward(const Call& call, T* O, const T* A, const T* C, const int32_t* P, int64_t I,
                 int N, int64_t J, int K) {
    const size_t smem = fwd_smem<T, kMaxOrder>(N); // the largest any order needs
    if (smem <= static_cast<size_t>(max_optin_smem(call.device)) && N <= kMaxTileColumns) {
#define CALL(KK) launch_fwd<T, KK>(call, O, A, C, P, I, N, J)
        MOPS_B200_ORDER_SWITCH(K, CALL)
#undef CALL
    } else {
        note_kernel_f("hpe_fwd_wide<%s>", scalar_name<T>());
        hpe_fwd_wide<T><<<static_cast<unsigned>(ceil_div(I, 128)), 128, 0, call.stream>>>(
            O, A, C, P, I, N, J, K, call.status);
    }
    MOPS_CUDA_OK(cudaGetLastError());
}

template <typename T>
void run_backward(const Call& call, T* gA, const T* gO, const T* A, const T* C, const int32_t* P,
                  int64_t I, int N, int64_t J, int K) {
    const size_t smem = vjp_smem<T, kMaxOrder>(N);
    if (smem <= static_cast<size_t>(max_optin_smem(call.device)) && N <= kMaxTileColumns) {
#define CALL(KK) launch_vjp<T, KK>(call, gA, gO, A, C, P, I, N, J)
        MOPS_B200_ORDER_SWITCH(K, CALL)
#undef CALL
    } else {
        note_kernel_f("hpe_vjp_wide<%s>", scalar_name<T>());
        hpe_vjp_wide<T><<<static_cast<unsigned>(ceil_div(I, 128)), 128, 0, call.stream>>>(
            gA, gO, A, C, P, I, N, J, K, call.status);
    }
    MOPS_CUDA_OK(cudaGetLastError());
}

// ---- second order, as a first-order problem on augmented operands
// With A2 = [A | ggA] (2N columns) and, for every monomial j and position k, the monomial
// (j, k) whose k-th factor is taken from the ggA half,
//     Q(A2) = sum_{j,k} C_j ggA[i, P_jk] prod_{l != k} A[i, P_jl],
// the second-order terms of mops/src/hpe/cpu.tpp:275-539 are
//     ggO[i] = Q(A2)[i],      gA2[i, n] = gO[i] dQ/dA[i, n]   (the first N columns of Q's VJP).
template <typename T>
__global__ void hpe_augment_rows(T* __restrict__ A2, const T* __restrict__ A,
                                 const T* __restrict__ ggA, int64_t I, int N) {
    const int64_t total = I * 2 * N;
    for (int64_t x = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; x < total;
         x += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t i = x / (2 * N);
        const int n = static_cast<int>(x - i * 2 * N);
        A2[x] = n < N ? A[i * N + n] : ggA[i * N + n - N];
    }
}

template <typename T>
__global__ void hpe_augment_table(T* __restrict__ C2, int32_t* __restrict__ P2,
                                  const T* __restrict__ C, const int32_t* __restrict__ P, int J,
                                  int K, int N, Status st) {
    const int total = J * K;
    for (int x = blockIdx.x * blockDim.x + threadIdx.x; x < total; x += gridDim.x * blockDim.x) {
        const int j = x / K, k = x - j * K;
        C2[x] = C[j];
        for (int l = 0; l < K; l++) {
            int32_t p = P[j * K + l];
            if (clamp_index(p, N)) report_bad_index(st, 0);
            P2[static_cast<int64_t>(x) * K + l] = l == k ? N + p : p;
        }
    }
}

template <typename T>
__global__ void hpe_take_left_half(T* __restrict__ out, const T* __restrict__ in2, int64_t I,
                                   int N) {
    const int64_t total = I * N;
    for (int64_t x = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; x < total;
         x += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t i = x / N;
        out[x] = in2[i * 2 * N + (x - i * N)];
    }
}


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
    fits_int32(C.shape[0] * std::max<size_t>(indices_A.shape[1], 1) * 16, "the monomial table", op);
    run_forward<scalar_t>(call, output.data, A.data, C.data, indices_A.data, I, N, J, K);
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
    fits_int32(C.shape[0] * std::max<size_t>(indices_A.shape[1], 1) * 16, "the monomial table", op);
    run_backward<scalar_t>(call, grad_A.data, grad_output.data, A.data, C.data, indices_A.data, I,
                           N, J, K);
    end_call(call, op.c_str(), kIndexNames, 1);
}

template <typename scalar_t>
void mops::cuda::homogeneous_polynomial_evaluation_vjp_vjp(
    Tensor<scalar_t, 1> grad_grad_output, Tensor<scalar_t, 2> grad_A_2,
    Tensor<scalar_t, 2> grad_grad_A, Tensor<scalar_t, 1> grad_output, Tensor<scalar_t, 2> A,
    Tensor<scalar_t, 1> C, Tensor<int32_t, 2> indices_A) {
    // The reference CUDA build throws "Not implemented" (mops/src/hpe/hpe.cu:402-413); the
    // semantics are those of its CPU code (mops/src/hpe/cpu.tpp:275-539).
    const std::string op = "cuda_homogeneous_polynomial_evaluation_vjp_vjp";
    grad_like(grad_grad_output, "grad_grad_output", grad_output, "grad_output", op);
    grad_like(grad_A_2, "grad_A_2", A, "A", op);
    grad_like(grad_grad_A, "grad_grad_A", A, "A", op);
    same_size(A, "A", 0, grad_output, "grad_output", 0, op);
    same_size(C, "C", 0, indices_A, "indices_A", 0, op);
    check_order(indices_A.shape[1]);
    fits_int32(2 * A.shape[1], "2 * A.shape[1]", op);
    if (grad_grad_output.data == nullptr && grad_A_2.data == nullptr) return;
    const int64_t I = static_cast<int64_t>(A.shape[0]), J = static_cast<int64_t>(C.shape[0]);
    const int N = static_cast<int>(A.shape[1]), K = static_cast<int>(indices_A.shape[1]);
    if (I == 0) return;
    Call call = begin_call();
    const bool trivial = grad_grad_A.data == nullptr || K == 0 || J == 0 || N == 0;
    if (trivial) { // no dependence on grad_grad_A: both second-order terms vanish
        if (N == 0 && K > 0 && J > 0)
            throw std::runtime_error("Index array indices_A in operation " + op +
                                     " refers to columns of an A that has none");
        if (grad_grad_output.data != nullptr)
            MOPS_CUDA_OK(cudaMemsetAsync(grad_grad_output.data, 0, I * sizeof(scalar_t), call.stream));
        if (grad_A_2.data != nullptr && N > 0)
            MOPS_CUDA_OK(cudaMemsetAsync(grad_A_2.data, 0, I * N * sizeof(scalar_t), call.stream));
        end_call(call, op.c_str(), kIndexNames, 1);
        return;
    }
    fits_int32(C.shape[0] * indices_A.shape[1] * indices_A.shape[1] * 16, "the monomial table", op);
    const int64_t J2 = J * K;
    const int N2 = 2 * N, grid = sm_count(call.device) * 8;
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    const size_t b_a2 = up(static_cast<size_t>(I) * N2 * sizeof(scalar_t));
    const size_t b_c2 = up(static_cast<size_t>(J2) * sizeof(scalar_t));
    const size_t b_p2 = up(static_cast<size_t>(J2) * K * sizeof(int32_t));
    const size_t b_g2 = grad_A_2.data != nullptr ? b_a2 : 0;
    // The augmented coefficient and index arrays below are temporaries whose addresses repeat
    // from call to call: tables derived from them must not be kept by a plan.
    PlanSuspended no_plan;
    unsigned char* base = static_cast<unsigned char*>(scratch_alloc(call, b_a2 + b_c2 + b_p2 + b_g2));
    scalar_t* A2 = reinterpret_cast<scalar_t*>(base);
    scalar_t* C2 = reinterpret_cast<scalar_t*>(base + b_a2);
    int32_t* P2 = reinterpret_cast<int32_t*>(base + b_a2 + b_c2);
    scalar_t* G2 = reinterpret_cast<scalar_t*>(base + b_a2 + b_c2 + b_p2);
    hpe_augment_rows<scalar_t><<<grid, 256, 0, call.stream>>>(A2, A.data, grad_grad_A.data, I, N);
    hpe_augment_table<scalar_t><<<grid, 256, 0, call.stream>>>(
        C2, P2, C.data, indices_A.data, static_cast<int>(J), K, N, call.status);
    MOPS_CUDA_OK(cudaGetLastError());
    if (grad_grad_output.data != nullptr)
        run_forward<scalar_t>(call, grad_grad_output.data, A2, C2, P2, I, N2, J2, K);
    if (grad_A_2.data != nullptr) {
        run_backward<scalar_t>(call, G2, grad_output.data, A2, C2, P2, I, N2, J2, K);
        hpe_take_left_half<scalar_t><<<grid, 256, 0, call.stream>>>(grad_A_2.data, G2, I, N);
        MOPS_CUDA_OK(cudaGetLastError());
    }
    scratch_free(call, base);
    end_call(call, op.c_str(), kIndexNames, 1);
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
