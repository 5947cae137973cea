// Stable sort of a scatter index on the device, with the permutation that sorts it.
//
// The scatter operations (OPSA, OPSAW, SASAW) are segmented reductions over an ascending
// scatter index; callers of the reference sort their entries on the host before the call
// (python/mops/tests/opsa.py:96 sorts with NumPy; the reference CUDA OPSA silently requires
// it, mops/src/opsa/opsa.cu:73-75). This is that step on the device: a least-significant-digit
// radix sort, eight bits per pass, as many passes as the row count needs (three up to 2^24
// rows). Every pass is stable, so entries of one output row keep their input order and the
// sums a kernel forms over a row's entries are taken in the same order as on unsorted input.
// The same routine applied to indices_W (OPSAW) or indices_W_1 (SASAW) gives the permutation
// that groups the grad_W contributions by row of W.
#include <algorithm>

#include "checks.hpp"
#include "device.cuh"

namespace mops_b200 {
namespace {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortItems = 16;                         // per thread
constexpr int kSortTile = kSortThreads * kSortItems;   // per block
constexpr int kWarpChunk = 32 * kSortItems;            // consecutive elements of one warp

// Element `i` of warp `w`'s chunk, round `r`: position w * kWarpChunk + r * 32 + lane, so
// that positions ascend with (warp, round, lane).
__device__ __forceinline__ int64_t sort_position(int64_t tile0, int warp, int round, int lane) {
    return tile0 + warp * kWarpChunk + round * 32 + lane;
}

__device__ __forceinline__ int sort_digit(int32_t key, int shift) { return (key >> shift) & 255; }

// hist[d * blocks + b] = number of keys of block b's tile whose digit is d. The first pass
// also checks the range of the values.
__global__ void __launch_bounds__(kSortThreads)
radix_histogram(const int32_t* __restrict__ keys, int64_t n, int shift, int64_t n_rows,
                bool check_range, int32_t* __restrict__ hist, Status st) {
    __shared__ int32_t h[256];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    h[tid] = 0;
    __syncthreads();
    const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * kSortTile;
    for (int r = 0; r < kSortItems; r++) {
        const int64_t pos = sort_position(tile0, warp, r, lane);
        if (pos < n) {
            int32_t key = __ldg(keys + pos);
            if (check_range && (key < 0 || key >= n_rows)) {
                report_bad_index(st, 0);
                key = 0;
            }
            atomicAdd(&h[sort_digit(key, shift)], 1);
        }
    }
    __syncthreads();
    hist[static_cast<int64_t>(tid) * gridDim.x + blockIdx.x] = h[tid];
}

// Block d turns row d of the histogram (the counts of digit d in every tile, in tile order)
// into its exclusive prefix sums, in place, and stores the row's total.
__global__ void __launch_bounds__(1024)
radix_scan_rows(int32_t* __restrict__ hist, int64_t blocks, int32_t* __restrict__ totals) {
    __shared__ int32_t partial[1024];
    const int tid = threadIdx.x;
    int32_t* row = hist + static_cast<int64_t>(blockIdx.x) * blocks;
    const int64_t per = (blocks + 1023) / 1024;
    const int64_t lo = tid * per < blocks ? tid * per : blocks;
    const int64_t hi = lo + per < blocks ? lo + per : blocks;
    int32_t sum = 0;
    for (int64_t i = lo; i < hi; i++) sum += row[i];
    partial[tid] = sum;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) { // Hillis-Steele over the 1024 partial sums
        const int32_t v = tid >= d ? partial[tid - d] : 0;
        __syncthreads();
        partial[tid] += v;
        __syncthreads();
    }
    int32_t run = partial[tid] - sum; // exclusive
    for (int64_t i = lo; i < hi; i++) {
        const int32_t v = row[i];
        row[i] = run;
        run += v;
    }
    if (tid == 1023) totals[blockIdx.x] = partial[1023];
}

// Moves every element of the block's tile to its place: scanned[d * blocks + b] is where block
// b's first key with digit d goes; inside the tile, keys with the same digit keep their order.
// vals_in == nullptr: the values are the positions themselves (first pass).
__global__ void __launch_bounds__(kSortThreads)
radix_scatter(const int32_t* __restrict__ keys_in, const int32_t* __restrict__ vals_in,
              int32_t* __restrict__ keys_out, int32_t* __restrict__ vals_out, int64_t n, int shift,
              int64_t n_rows, bool clamp, const int32_t* __restrict__ scanned,
              const int32_t* __restrict__ totals) {
    __shared__ int32_t next[kSortWarps][256]; // per warp: where its next key of each digit goes
    __shared__ int32_t digit_base[256];       // keys with a smaller digit, over all tiles
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * kSortTile;
    for (int w = 0; w < kSortWarps; w++) next[w][tid] = 0;
    {
        const int32_t mine = totals[tid];
        digit_base[tid] = mine;
        __syncthreads();
        for (int d = 1; d < 256; d <<= 1) {
            const int32_t v = tid >= d ? digit_base[tid - d] : 0;
            __syncthreads();
            digit_base[tid] += v;
            __syncthreads();
        }
        digit_base[tid] -= mine; // exclusive
    }
    __syncthreads();
    int32_t key[kSortItems], val[kSortItems];
    // 1. every warp counts the digits of its own chunk
    for (int r = 0; r < kSortItems; r++) {
        const int64_t pos = sort_position(tile0, warp, r, lane);
        const bool in = pos < n;
        key[r] = in ? __ldg(keys_in + pos) : 0;
        if (clamp && (key[r] < 0 || key[r] >= n_rows)) key[r] = 0; // reported by the histogram pass
        val[r] = in ? (vals_in != nullptr ? __ldg(vals_in + pos) : static_cast<int32_t>(pos)) : 0;
        const int d = in ? sort_digit(key[r], shift) : 256 + lane; // out-of-range lanes match nobody
        const unsigned peers = __match_any_sync(kFullMask, d);
        if (in && (peers & ((1u << lane) - 1)) == 0) next[warp][d] += __popc(peers);
        __syncwarp();
    }
    __syncthreads();
    // 2. digit by digit: global start of the block's keys, then warp after warp
    {
        int32_t run = digit_base[tid] + scanned[static_cast<int64_t>(tid) * gridDim.x + blockIdx.x];
        for (int w = 0; w < kSortWarps; w++) {
            const int32_t c = next[w][tid];
            next[w][tid] = run;
            run += c;
        }
    }
    __syncthreads();
    // 3. every warp walks its chunk again, in order
    for (int r = 0; r < kSortItems; r++) {
        const int64_t pos = sort_position(tile0, warp, r, lane);
        const bool in = pos < n;
        const int d = in ? sort_digit(key[r], shift) : 256 + lane;
        const unsigned peers = __match_any_sync(kFullMask, d);
        const int rank = __popc(peers & ((1u << lane) - 1));
        int32_t base = 0;
        if (in && rank == 0) {
            base = next[warp][d];
            next[warp][d] = base + __popc(peers);
        }
        base = __shfl_sync(kFullMask, base, __ffs(peers) - 1);
        if (in) {
            keys_out[base + rank] = key[r];
            vals_out[base + rank] = val[r];
        }
        __syncwarp();
    }
}

const char* const kSortIndexNames[] = {"indices"};

} // namespace

void sort_index(mops::Tensor<int32_t, 1> sorted, mops::Tensor<int32_t, 1> permutation,
                mops::Tensor<int32_t, 1> indices, int64_t n_rows) {
    const std::string op = "cuda_sort_index";
    same_size(indices, "indices", 0, sorted, "sorted", 0, op);
    same_size(indices, "indices", 0, permutation, "permutation", 0, op);
    fits_int32(indices.shape[0], "indices.shape[0]", op);
    if (n_rows < 0 || n_rows > INT32_MAX)
        throw std::runtime_error("n_rows does not fit the int32 index type in " + op);
    const int64_t n = static_cast<int64_t>(indices.shape[0]);
    if (n == 0) return;
    Call call = begin_call();
    int bits = 1;
    while ((int64_t(1) << bits) < n_rows) bits++;
    const int passes = (bits + 7) / 8;
    const int64_t blocks = ceil_div(n, kSortTile);
    const size_t hist_bytes = static_cast<size_t>(256) * blocks * sizeof(int32_t);
    const size_t buf_bytes = (static_cast<size_t>(n) * sizeof(int32_t) + 255) / 256 * 256;
    const size_t hist_room = (hist_bytes + 255) / 256 * 256;
    unsigned char* scratch = static_cast<unsigned char*>(
        scratch_alloc(call, hist_room + 1024 + (passes > 1 ? 4 * buf_bytes : 0)));
    int32_t* hist = reinterpret_cast<int32_t*>(scratch);
    int32_t* totals = reinterpret_cast<int32_t*>(scratch + hist_room);
    unsigned char* bufs = scratch + hist_room + 1024;
    int32_t* tmp_keys[2] = {reinterpret_cast<int32_t*>(bufs), reinterpret_cast<int32_t*>(bufs + buf_bytes)};
    int32_t* tmp_vals[2] = {reinterpret_cast<int32_t*>(bufs + 2 * buf_bytes),
                            reinterpret_cast<int32_t*>(bufs + 3 * buf_bytes)};
    const int32_t* keys_in = indices.data;
    const int32_t* vals_in = nullptr;
    for (int pass = 0; pass < passes; pass++) {
        const bool last = pass == passes - 1;
        int32_t* keys_out = last ? sorted.data : tmp_keys[pass & 1];
        int32_t* vals_out = last ? permutation.data : tmp_vals[pass & 1];
        radix_histogram<<<static_cast<unsigned>(blocks), kSortThreads, 0, call.stream>>>(
            keys_in, n, 8 * pass, n_rows, pass == 0, hist, call.status);
        radix_scan_rows<<<256, 1024, 0, call.stream>>>(hist, blocks, totals);
        radix_scatter<<<static_cast<unsigned>(blocks), kSortThreads, 0, call.stream>>>(
            keys_in, vals_in, keys_out, vals_out, n, 8 * pass, n_rows, pass == 0, hist, totals);
        MOPS_CUDA_OK(cudaGetLastError());
        keys_in = keys_out;
        vals_in = vals_out;
    }
    note_kernel_f("radix sort, %d passes", passes);
    scratch_free(call, scratch);
    end_call(call, op.c_str(), kSortIndexNames, 1);
}

} // namespace mops_b200
