// Device-side helpers shared by the kernels: status reporting, the segment search over a
// sorted scatter index, the sortedness check, and reductions.
//
// Replaces mops/src/internal/cuda_utils.{cuh,cu} (atomic add with a pre-sm_60 fallback, the
// shared-memory bump allocator) and mops/src/internal/cuda_first_occurences.cu (a memset + a
// kernel + a device synchronisation that write a first/last-occurrence table into a cached,
// process-wide global buffer before every scatter op). Here `segment_offsets` writes the
// table of segment starts in one launch on the call's stream (no memset, no synchronisation,
// call-scoped or plan-owned memory) and checks order and range in the same pass; the
// warp-wide search (`warp_segment`) serves the kernels that work without a table.
#ifndef MOPS_B200_DEVICE_CUH
#define MOPS_B200_DEVICE_CUH

#include <algorithm>
#include <cstdint>

#include "runtime.hpp"

namespace mops_b200 {

constexpr unsigned kFullMask = 0xffffffffu;

__device__ __forceinline__ void report_unsorted(const Status& st) {
    st.dev[kUnsortedEpoch] = st.epoch;
    st.host[kUnsortedEpoch] = st.epoch;
    __threadfence_system();
}

__device__ __forceinline__ void report_bad_index(const Status& st, int which) {
    st.dev[kBadIndex0 + which] = st.epoch;
    st.host[kBadIndex0 + which] = st.epoch;
    __threadfence_system();
}

__device__ __forceinline__ bool saw_unsorted(const Status& st) {
    return *reinterpret_cast<volatile uint32_t*>(st.dev + kUnsortedEpoch) == st.epoch;
}

// Clamp an index read from a user array into [0, n) so that a bad value can never address
// memory outside the operand; returns whether it had to.
__device__ __forceinline__ bool clamp_index(int32_t& v, int32_t n) {
    bool bad = static_cast<uint32_t>(v) >= static_cast<uint32_t>(n);
    if (bad) v = 0;
    return bad;
}

// First position in the ascending array P[lo, hi) whose value is >= r, found by the whole
// warp: every round the 32 lanes probe 32 evenly spaced positions and one ballot narrows
// the range 32-fold (five rounds for 2^24 entries, each a single coalescable load per lane).
// All lanes must call it with the same arguments; all get the result. On an unsorted array
// the result is some position in [lo, hi]; callers detect that case separately.
__device__ __forceinline__ int64_t warp_lower_bound(const int32_t* __restrict__ P, int64_t lo,
                                                    int64_t hi, int32_t r, int lane) {
    while (hi > lo) {
        int64_t n = hi - lo;
        int64_t chunk = (n + 31) / 32; // >= 1
        int64_t probe = lo + (lane + 1) * chunk - 1;
        bool below = (probe < hi) && (__ldg(P + probe) < r);
        int c = __popc(__ballot_sync(kFullMask, below));
        int64_t new_lo = lo + c * chunk;
        if (new_lo >= hi) {
            lo = hi;
            break;
        }
        // The answer is in [new_lo, new_lo + chunk - 1]: position new_lo + chunk - 1 was
        // probed and is >= r (or lies at/after hi).
        int64_t new_hi = new_lo + chunk - 1;
        if (new_hi > hi) new_hi = hi;
        lo = new_lo;
        hi = new_hi;
    }
    return lo;
}

// Number of i in [0, n) with t[i] + row_weight * i <= x, for an ascending table t, found by
// the whole warp with 32-way probes (as warp_lower_bound). All lanes call it with the same
// arguments.
__device__ __forceinline__ int64_t warp_count_weighted_le(const int64_t* __restrict__ t, int64_t n,
                                                          int64_t row_weight, int64_t x, int lane) {
    int64_t lo = 0, hi = n;
    while (hi > lo) {
        const int64_t len = hi - lo;
        const int64_t chunk = (len + 31) / 32; // >= 1
        const int64_t probe = lo + (lane + 1) * chunk - 1;
        const bool le = (probe < hi) && (t[probe] + row_weight * probe <= x);
        const int c = __popc(__ballot_sync(kFullMask, le));
        const int64_t new_lo = lo + c * chunk;
        if (new_lo >= hi) {
            lo = hi;
            break;
        }
        int64_t new_hi = new_lo + chunk - 1;
        if (new_hi > hi) new_hi = hi;
        lo = new_lo;
        hi = new_hi;
    }
    return lo;
}

// Splits the rows of a segment table among `parts` workers so that every worker gets whole
// rows and about the same amount of work, counted as entries + kRowWeight per row: not the
// same number of rows (the rows of a shard of a larger problem, or of an uneven graph, can be
// mostly empty), and not entries alone either (a long run of empty rows still has to be
// written). offsets[0 .. n_rows] ascending, offsets[n_rows] = number of entries. Returns the
// first row of worker `part`, who owns rows [split(part), split(part + 1)). All lanes of a
// warp call it together.
constexpr int64_t kRowWeight = 4;
__device__ __forceinline__ int64_t balanced_row_split(const int64_t* __restrict__ offsets,
                                                      int64_t n_rows, int64_t part, int64_t parts,
                                                      int lane) {
    if (part <= 0) return 0;
    if (part >= parts) return n_rows;
    const int64_t total = offsets[n_rows] + kRowWeight * n_rows;
    const int64_t target = total / parts * part + total % parts * part / parts;
    // the last row whose weighted start is <= target
    const int64_t r = warp_count_weighted_le(offsets, n_rows + 1, kRowWeight, target, lane) - 1;
    return r < 0 ? 0 : (r > n_rows ? n_rows : r);
}

// Bounds [begin, end) of the entries whose (sorted) index equals r.
__device__ __forceinline__ void warp_segment(const int32_t* __restrict__ P, int64_t J, int32_t r,
                                             int lane, int64_t& begin, int64_t& end) {
    begin = warp_lower_bound(P, 0, J, r, lane);
    // Segments are short in practice: look in a window after `begin` first.
    int64_t stop = begin + 1024 < J ? begin + 1024 : J;
    end = warp_lower_bound(P, begin, stop, r + 1, lane);
    if (end == stop && stop < J) end = warp_lower_bound(P, stop, J, r + 1, lane);
}

// Every warp of a grid checks one slice of the scatter index for ascending order and for
// range; together the slices cover all adjacent pairs, so "no report" proves the index is
// sorted and inside [0, n_rows). `part` in [0, n_parts).
__device__ __forceinline__ void check_sorted_slice(const int32_t* __restrict__ P, int64_t J,
                                                   int64_t n_rows, int64_t part, int64_t n_parts,
                                                   int lane, const Status& st) {
    if (J == 0) return;
    int64_t per = (J + n_parts - 1) / n_parts;
    int64_t a = part * per;
    int64_t b = a + per < J ? a + per : J;
    bool unsorted = false, bad = false;
    for (int64_t j = a + lane; j < b; j += 32) {
        int32_t v = __ldg(P + j);
        int32_t next = (j + 1 < J) ? __ldg(P + j + 1) : v;
        unsorted |= next < v;
        bad |= (v < 0) || (static_cast<int64_t>(v) >= n_rows);
    }
    if (__any_sync(kFullMask, unsorted) && lane == 0) report_unsorted(st);
    // Bit 0 is the scatter index of every scatter op.
    if (__any_sync(kFullMask, bad) && lane == 0) report_bad_index(st, 0);
}

template <typename T> __device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
    return v;
}

// Fire-and-forget global accumulation (compiles to RED: no value comes back).
// Reductions without a return value (atomicAdd with an unused result can still be compiled
// to the returning form, which holds a register and a scoreboard until the L2 answers).
__device__ __forceinline__ void red_add(double* addr, double v) {
    asm volatile("red.global.add.f64 [%0], %1;\n" ::"l"(addr), "d"(v) : "memory");
}
__device__ __forceinline__ void red_add(float* addr, float v) {
    asm volatile("red.global.add.f32 [%0], %1;\n" ::"l"(addr), "f"(v) : "memory");
}

// Unsorted index: runs only when the segmented kernel of the same call reported it.
template <typename T>
__global__ void zero_if_unsorted(T* __restrict__ out, int64_t n, Status st) {
    if (!saw_unsorted(st)) return;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[i] = T(0);
}


// ---------------------------------------------------------------- FP64 tensor-core MMA
// mma.sync m8n8k4, f64. Fragment layout (lane = 4*qr + qc): A[qr][qc], B[k = qc][n = qr],
// C[qr][2*qc + {0,1}].
__device__ __forceinline__ void dmma(double (&c)[2], double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};\n"
                 : "+d"(c[0]), "+d"(c[1])
                 : "d"(a), "d"(b));
}
// c = a b (no accumulator input)
__device__ __forceinline__ void dmma0(double (&c)[2], double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%4,%4};\n"
                 : "=d"(c[0]), "=d"(c[1])
                 : "d"(a), "d"(b), "d"(0.0));
}

// ---------------------------------------------------------------- asynchronous staging
// Element-wise global -> shared copies that do not pass through registers (LDGSTS): a lane
// can put a whole chunk in flight and go on; completion is tracked per committed group.
template <int BYTES>
__device__ __forceinline__ void cp_async(void* smem_dst, const void* global_src) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(dst), "l"(global_src),
                 "n"(BYTES)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- segment offsets
// offsets[r] = first position of the ascending index P whose value is >= r, for r in
// [0, n_rows]; offsets[n_rows] = J. One thread per boundary between neighbouring entries:
// entry j starts every row in (P[j-1], P[j]]. The same pass checks order and range, so the
// kernels that consume the table can trust it, or skip their work when the index was not
// sorted (saw_unsorted). Long runs of empty rows are filled by the whole warp.
// Replaces the reference's first-occurrence pass (memset + kernel + device synchronisation
// into a cached global buffer, mops/src/internal/cuda_first_occurences.cu:82-117).
static __global__ void segment_offsets(const int32_t* __restrict__ P, int64_t J, int64_t n_rows,
                                       int64_t* __restrict__ offsets, Status st) {
    const int lane = threadIdx.x & 31;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    // Whole warps iterate together so that the cooperative fill below sees all 32 lanes.
    const int64_t rounds = (J + 1 + stride - 1) / stride;
    int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (int64_t it = 0; it < rounds; it++, j += stride) {
        int64_t prev = 0, cur = -1; // empty range by default
        if (j <= J) {
            const int64_t p_raw = j == 0 ? -1 : static_cast<int64_t>(__ldg(P + j - 1));
            const int64_t c_raw = j == J ? n_rows : static_cast<int64_t>(__ldg(P + j));
            if (j < J && (c_raw < 0 || c_raw >= n_rows)) report_bad_index(st, 0);
            if (c_raw < p_raw) report_unsorted(st);
            prev = p_raw < -1 ? -1 : (p_raw > n_rows ? n_rows : p_raw);
            cur = c_raw < -1 ? -1 : (c_raw > n_rows ? n_rows : c_raw);
        }
        // rows prev+1 .. cur start at entry j
        if (cur > prev) offsets[prev + 1] = j;
        unsigned wide = __ballot_sync(kFullMask, cur > prev + 1);
        while (wide) {
            const int src = __ffs(wide) - 1;
            wide &= wide - 1;
            const int64_t lo = __shfl_sync(kFullMask, prev, src) + 2;
            const int64_t hi = __shfl_sync(kFullMask, cur, src);
            const int64_t at = __shfl_sync(kFullMask, j, src);
            for (int64_t r = lo + lane; r <= hi; r += 32) offsets[r] = at;
        }
    }
}

__host__ __device__ constexpr int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// The segment table of a scatter index for one call: taken from the calling thread's plan when
// it has one for this index (then the index is known to be sorted and nothing is launched),
// else built on the call's stream into call-scoped (or, for a plan's first use, plan-owned)
// memory. release_table(call, t.ref) when the kernels that read it are enqueued.
struct SegmentTable {
    int64_t* offsets;
    TableRef ref;
    bool known_sorted; // no need to ask the device, no fallback kernels
};

inline SegmentTable segment_table(const Call& call, const int32_t* P, int64_t J, int64_t n_rows) {
    TableKey key{};
    key.kind = kSegmentTable;
    key.ptr[0] = P;
    key.n[0] = J;
    key.n[1] = n_rows;
    SegmentTable t;
    t.ref = acquire_table(call, key, static_cast<size_t>(n_rows + 1) * sizeof(int64_t));
    t.offsets = static_cast<int64_t*>(t.ref.ptr);
    if (t.ref.fresh) {
        const int64_t blocks =
            std::min<int64_t>(ceil_div(J + 1, 256), static_cast<int64_t>(sm_count(call.device)) * 32);
        segment_offsets<<<static_cast<unsigned>(blocks > 0 ? blocks : 1), 256, 0, call.stream>>>(
            P, J, n_rows, t.offsets, call.status);
        MOPS_CUDA_OK(cudaGetLastError());
        commit_table(call, t.ref);
    }
    t.known_sorted = t.ref.owned_by_plan && t.ref.sorted;
    return t;
}

} // namespace mops_b200

#endif
