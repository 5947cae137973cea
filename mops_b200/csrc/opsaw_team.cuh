// Outer-product scatter-add with weights, forward and VJP, by teams of warps.
//
// In the per-warp streaming kernels (opsa_pipe.cuh) every warp owns a ring of stages and does
// all the work of its entries. With weights a staged entry takes 680 bytes of shared memory
// (A, the padded B row and the gathered, padded W row), so chunks must stay at eight entries to
// keep sixteen warps on an SM; the bookkeeping per chunk (issuing the copies, the barrier, the
// segment walk) then costs more instructions than the contraction itself, and the measured time
// follows the instruction count, not the bytes. Here the warps of a block share ONE ring with
// chunks of up to 32 entries: the block owns a contiguous range of output rows, every warp
// stages its share of the rows of a chunk, and the warps split the contraction by columns of B
// (warp w owns l in [8 w, 8 w + 8)). The per-chunk bookkeeping is spread over four times as
// many entries, the accumulators of a warp shrink to one column tile, and the block
// synchronises once per chunk (the stage that every warp has left is refilled).
//
// Included by opsa.cu (inside its unnamed namespace) after opsa_pipe.cuh.

__device__ __forceinline__ void mbarrier_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_address(bar)) : "memory");
}

// Stage barriers (2), grad_output barriers (2), "every warp has taken this grad_output row" (2).
constexpr int kTeamBarriers = 6;

inline PipeLayout team_layout(size_t s, int K, int L, bool vjp, int ch) {
    PipeLayout p = pipe_layout(s, K, L, true, vjp, ch, 2);
    p.warp_bytes = (p.bar_off + 8 * kTeamBarriers + 127) / 128 * 128; // here: bytes of the block
    return p;
}

// Rows and entries of the block (the PipeWarp of a whole block).
__device__ __forceinline__ PipeWarp team_partition(const int64_t* __restrict__ offsets, int64_t nO,
                                                   int ch) {
    PipeWarp w;
    const int lane = threadIdx.x & 31;
    w.r0 = balanced_row_split(offsets, nO, blockIdx.x, gridDim.x, lane);
    w.r1 = balanced_row_split(offsets, nO, static_cast<int64_t>(blockIdx.x) + 1, gridDim.x, lane);
    w.e_begin = offsets[w.r0];
    w.e_last = offsets[w.r1];
    w.e_first = w.e_begin & ~static_cast<int64_t>(3);
    w.nchunks = w.e_last > w.e_begin ? static_cast<int>((w.e_last - w.e_first + ch - 1) / ch) : 0;
    return w;
}

// Every warp of the block calls this for the chunk that starts at entry e0: warp 0 starts the
// bulk copy of the A slice and stores the W rows' numbers, every warp copies its share of the
// B rows and of the gathered W rows (16 bytes per lane copy), every lane arrives on `bar` when
// its copies are complete. pw_lane: lane i holds the (range-checked) W row of entry e0 + i.
// Plain stores made here (the last scalars of A at the end of the array, the row numbers) are
// ordered before their readers by the block barrier that precedes the chunk's consumption.
template <typename S, int NW>
__device__ __forceinline__ void team_issue_chunk(const PipeLayout& lay, unsigned char* stage,
                                                 uint64_t* bar, const S* __restrict__ A,
                                                 const S* __restrict__ B, const S* __restrict__ W,
                                                 int64_t e0, int64_t J, int32_t pw_lane, int warp,
                                                 int lane) {
    const int K = lay.K, L = lay.L, LP = lay.LP;
    const int n = static_cast<int>(J - e0 < lay.ch ? J - e0 : lay.ch);
    S* As = reinterpret_cast<S*>(stage + lay.a_off);
    S* Bs = reinterpret_cast<S*>(stage + lay.b_off);
    if (warp == 0) {
        const unsigned a_bytes = static_cast<unsigned>(n) * K * sizeof(S), a_bulk = a_bytes & ~15u;
        if (lane == 0) {
            mbarrier_arrive_expect(bar, a_bulk);
            if (a_bulk) bulk_copy_in(As, A + e0 * K, a_bulk, bar);
        }
        int32_t* pws = reinterpret_cast<int32_t*>(stage + lay.pw_off);
        if (lane < n) pws[lane] = pw_lane;
        if (a_bulk != a_bytes)
            for (int i = a_bulk / sizeof(S) + lane; i < n * K; i += 32) As[i] = A[e0 * K + i];
    }
    constexpr int kPer = 16 / static_cast<int>(sizeof(S)); // scalars per piece
    const unsigned w_delta = static_cast<unsigned>(lay.w_off - lay.b_off);
    if (lay.row_pieces_log2 >= 0) {
        // a lane keeps its piece column; a warp instruction covers 32 / row_pieces rows
        const int per_round = 32 >> lay.row_pieces_log2, stride = NW * per_round;
        const int col = (lane & (lay.row_pieces - 1)) * kPer;
        int r = warp * per_round + (lane >> lay.row_pieces_log2);
        unsigned dst = smem_address(Bs + r * LP + col);
        const unsigned dst_step = static_cast<unsigned>(stride * LP * sizeof(S));
        const S* bsrc = B + (e0 + r) * L + col;
        const S* wsrc = W + col;
        const int64_t src_step = static_cast<int64_t>(stride) * L;
        for (int rb = warp * per_round; rb < n; rb += stride, r += stride, dst += dst_step, bsrc += src_step) {
            const int32_t wrow = __shfl_sync(kFullMask, pw_lane, r & 31);
            if (r < n) {
                lane_copy16_to(dst, bsrc);
                lane_copy16_to(dst + w_delta, wsrc + static_cast<int64_t>(wrow) * L);
            }
        }
    } else {
        const int pieces = n * lay.row_pieces;
        for (int ib = warp * 32; ib < pieces; ib += NW * 32) {
            const int i = ib + lane;
            const int r = i / lay.row_pieces;
            const int32_t wrow = __shfl_sync(kFullMask, pw_lane, r & 31);
            if (i < pieces) {
                const int col = (i - r * lay.row_pieces) * kPer;
                const unsigned dst = smem_address(Bs + r * LP + col);
                lane_copy16_to(dst, B + (e0 + r) * L + col);
                lane_copy16_to(dst + w_delta, W + static_cast<int64_t>(wrow) * L + col);
            }
        }
    }
    lane_copies_arrive(bar);
}

// ------------------------------------------------------------------------------- forward
// O[r][:, 8 w .. 8 w + 8) = A[seg]^T (B[seg] * W[PW[seg]])[:, 8 w .. 8 w + 8) in warp w, the
// entries as the MMA's k dimension, four per step. MT = ceil(K / 8), NW = ceil(L / 8) warps.
template <typename S, int MT, int NW>
__global__ void __launch_bounds__(NW * 32)
opsaw_fwd_team(S* __restrict__ O, const S* __restrict__ A, const S* __restrict__ B,
               const S* __restrict__ W, const int32_t* __restrict__ PW,
               const int64_t* __restrict__ offsets, int64_t J, int64_t nO, int64_t nW,
               PipeLayout lay, Status st) {
    using T = double;
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    if (saw_unsorted(st)) return; // the atomic kernel of the same call does the work
    const int lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0); // uniform for the compiler
    const int qr = lane >> 2, qc = lane & 3;
    const int K = lay.K, L = lay.L, LP = lay.LP, CH = lay.ch;
    uint64_t* bars = reinterpret_cast<uint64_t*>(pipe_smem + lay.bar_off);
    if (threadIdx.x == 0) {
        mbarrier_init(bars, NW * 32 + 1);
        mbarrier_init(bars + 1, NW * 32 + 1);
        mbarrier_init_fence();
    }
    __syncthreads();
    const PipeWarp w = team_partition(offsets, nO, CH);
    if (w.r0 >= w.r1) return;

    auto load_pw = [&](int c) -> int32_t {
        int32_t pw = 0;
        const int64_t e = w.e_first + static_cast<int64_t>(c) * CH + lane;
        if (c < w.nchunks && lane < CH && e < J) {
            pw = __ldg(PW + e);
            if (clamp_index(pw, static_cast<int32_t>(nW)) && warp == 0) report_bad_index(st, 1);
        }
        return pw;
    };
    int32_t pw_reg = load_pw(0);
    auto issue = [&](int c) {
        if (c < w.nchunks) {
            team_issue_chunk<S, NW>(lay, pipe_smem + (c & 1) * lay.stage_bytes, bars + (c & 1), A, B,
                                    W, w.e_first + static_cast<int64_t>(c) * CH, J, pw_reg, warp,
                                    lane);
            pw_reg = load_pw(c + 1);
        }
    };
    issue(0);

    // segment ends of 32 rows at a time: lane i holds offsets[wbase + 1 + i]
    int64_t wbase = w.r0;
    auto load_window = [&](int64_t base) {
        const int64_t i = base + 1 + lane;
        return offsets[i < nO ? i : nO];
    };
    int64_t win = load_window(wbase);
    auto row_end = [&](int64_t r) -> int64_t {
        if (r - wbase >= 32) {
            wbase = r;
            win = load_window(wbase);
        }
        return __shfl_sync(kFullMask, win, static_cast<int>(r - wbase));
    };

    T acc[MT][2];
    auto clear = [&] {
#pragma unroll
        for (int mt = 0; mt < MT; mt++) acc[mt][0] = acc[mt][1] = T(0);
    };
    const int64_t rowsize = static_cast<int64_t>(K) * L;
    const bool pair_ok = L % 2 == 0 && reinterpret_cast<uintptr_t>(O) % (2 * sizeof(S)) == 0;
    const int l_out = 8 * warp + 2 * qc; // element (mt, h) is O[r, k = 8 mt + qr, l = l_out + h]
    auto flush = [&](int64_t r) {
        if (l_out >= L) return;
        S* dst = O + r * rowsize + l_out;
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const int k = 8 * mt + qr;
            if (k >= K) continue;
            S* d2 = dst + k * L;
            if (pair_ok) {
                typename VecOf<S, 2>::type v2;
                v2.x = static_cast<S>(acc[mt][0]), v2.y = static_cast<S>(acc[mt][1]);
                *reinterpret_cast<typename VecOf<S, 2>::type*>(d2) = v2;
            } else {
                d2[0] = static_cast<S>(acc[mt][0]);
                if (l_out + 1 < L) d2[1] = static_cast<S>(acc[mt][1]);
            }
        }
    };

    clear();
    // positions of entries below are relative to e_first (the block's range fits an int)
    int64_t row = w.r0;
    int e = static_cast<int>(w.e_begin - w.e_first);
    const int e_stop = static_cast<int>(w.e_last - w.e_first);
    int hi = static_cast<int>(row_end(row) - w.e_first);
    auto finish_rows = [&] {
        while (row < w.r1 && e == hi) {
            flush(row);
            clear();
            row++;
            if (row < w.r1) hi = static_cast<int>(row_end(row) - w.e_first);
        }
    };
    int c_lo = 0;
    for (int c = 0; c < w.nchunks; c++, c_lo += CH) {
        __syncthreads(); // every warp has left the other stage: refill it
        issue(c + 1);
        if (!mbarrier_wait(bars + (c & 1), (c >> 1) & 1)) {
            if (lane == 0) report_stalled(st);
            return;
        }
        const unsigned char* stage = pipe_smem + (c & 1) * lay.stage_bytes;
        const S* As = reinterpret_cast<const S*>(stage + lay.a_off) + qr;
        const S* Bs = reinterpret_cast<const S*>(stage + lay.b_off) + 8 * warp + qr;
        const S* Ws = reinterpret_cast<const S*>(stage + lay.w_off) + 8 * warp + qr;
        const int c_hi = c_lo + CH < e_stop ? c_lo + CH : e_stop;
        while (true) {
            finish_rows();
            if (row >= w.r1 || e >= c_hi) break;
            const int seg_end = hi < c_hi ? hi : c_hi;
            // entries [e, seg_end) of the current row, four per MMA step: fragment
            // A^T[k = 8 mt + qr][entry qc], (B*W)[entry qc][l = 8 w + qr]
            // Whole steps take their fragments unguarded: rows k >= K of A^T and columns
            // l >= L of B*W (whatever lies behind them in the stage) only reach elements of
            // the accumulators that are never stored.
            const int first = e - c_lo, last = seg_end - c_lo;
            const S* ap = As + (first + qc) * K;
            const S* bp = Bs + (first + qc) * LP;
            const S* wp = Ws + (first + qc) * LP;
            int s0 = first;
#pragma unroll 2
            for (; s0 + 4 <= last; s0 += 4, ap += 4 * K, bp += 4 * LP, wp += 4 * LP) {
                T af[MT];
#pragma unroll
                for (int mt = 0; mt < MT; mt++) af[mt] = static_cast<T>(ap[8 * mt]);
                const T v = static_cast<T>(bp[0]) * static_cast<T>(wp[0]);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) dmma(acc[mt], af[mt], v);
            }
            if (s0 < last) { // the last, ragged step: entries past the segment count as zero
                const bool valid = s0 + qc < last;
                T af[MT];
#pragma unroll
                for (int mt = 0; mt < MT; mt++) af[mt] = valid ? static_cast<T>(ap[8 * mt]) : T(0);
                const T v = valid ? static_cast<T>(bp[0]) * static_cast<T>(wp[0]) : T(0);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) dmma(acc[mt], af[mt], v);
            }
            e = seg_end;
        }
    }
    finish_rows();
}

// ----------------------------------------------------------------------------------- VJP
// For the entries of one output row, with gO[r] as the common factor kept in registers:
//   X[seg] = A[seg] gO[r], grad_B = X * W, grad_W[PW] += X * B: warp w computes the columns
//     l in [8 w, 8 w + 8) of every tile of eight entries;
//   grad_A[seg] = (B*W)[seg] gO[r]^T (a contraction over all of l): the tiles of eight entries
//     go to the warps in turn.
// grad_output rows pass through a ring of two slots shared by the block; a slot is refilled
// when every warp has taken its fragments of the row it held. KT = ceil(K / 4), NW = ceil(L / 8).
template <typename S, int KT, int NW>
__global__ void __launch_bounds__(NW * 32)
opsaw_vjp_team(S* __restrict__ gA, S* __restrict__ gB, S* __restrict__ gW,
               const S* __restrict__ gO, const S* __restrict__ A, const S* __restrict__ B,
               const S* __restrict__ W, const int32_t* __restrict__ PW,
               const int64_t* __restrict__ offsets, int64_t J, int64_t nO, int64_t nW,
               PipeLayout lay, Status st) {
    using T = double;
    using S2 = typename VecOf<S, 2>::type;
    constexpr int NTK = (KT + 1) / 2; // 8-wide tiles over K
    constexpr int KSL = 2 * NW;       // k-steps over L
    constexpr int KSK = KT;           // k-steps over K
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    if (saw_unsorted(st)) return; // the entry-per-lane kernel of the same call does the work
    const int lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0);
    const int qr = lane >> 2, qc = lane & 3;
    const int K = lay.K, L = lay.L, LP = lay.LP, CH = lay.ch;
    uint64_t* bars = reinterpret_cast<uint64_t*>(pipe_smem + lay.bar_off);
    uint64_t* gbars = bars + 2;  // grad_output row has arrived
    uint64_t* gfree = bars + 4;  // every warp has taken its fragments of the row
    if (threadIdx.x == 0) {
        mbarrier_init(bars, NW * 32 + 1);
        mbarrier_init(bars + 1, NW * 32 + 1);
        mbarrier_init(gbars, 1);
        mbarrier_init(gbars + 1, 1);
        mbarrier_init(gfree, NW);
        mbarrier_init(gfree + 1, NW);
        mbarrier_init_fence();
    }
    __syncthreads();
    const PipeWarp w = team_partition(offsets, nO, CH);
    if (w.r0 >= w.r1 || w.nchunks == 0) return; // gradients exist per entry only

    const bool want_a = gA != nullptr, want_b = gB != nullptr || gW != nullptr;
    const bool pair_ok = L % 2 == 0 && (gB == nullptr || reinterpret_cast<uintptr_t>(gB) % (2 * sizeof(S)) == 0);
    const int64_t rowsize = static_cast<int64_t>(K) * L;
    const int g_slot_bytes = (lay.g_bytes + 15) / 16 * 16;

    auto load_pw = [&](int c) -> int32_t {
        int32_t pw = 0;
        const int64_t e = w.e_first + static_cast<int64_t>(c) * CH + lane;
        if (c < w.nchunks && lane < CH && e < J) {
            pw = __ldg(PW + e);
            if (clamp_index(pw, static_cast<int32_t>(nW)) && warp == 0) report_bad_index(st, 1);
        }
        return pw;
    };
    int32_t pw_reg = load_pw(0);
    auto issue = [&](int c) {
        if (c < w.nchunks) {
            team_issue_chunk<S, NW>(lay, pipe_smem + (c & 1) * lay.stage_bytes, bars + (c & 1), A, B,
                                    W, w.e_first + static_cast<int64_t>(c) * CH, J, pw_reg, warp,
                                    lane);
            pw_reg = load_pw(c + 1);
        }
    };
    // grad_output rows r0, r0 + 1, ... go through the two slots in turn (thread 0 issues)
    auto issue_g = [&](int64_t r) {
        if (r < w.r1 && threadIdx.x == 0) {
            const int slot = static_cast<int>(r - w.r0) & 1;
            mbarrier_arrive_expect(gbars + slot, static_cast<unsigned>(lay.g_bytes));
            bulk_copy_in(pipe_smem + lay.g_off + slot * g_slot_bytes, gO + r * rowsize,
                         static_cast<unsigned>(lay.g_bytes), gbars + slot);
        }
    };
    issue_g(w.r0);
    issue_g(w.r0 + 1);
    issue(0);

    int64_t wbase = w.r0;
    auto load_window = [&](int64_t base) {
        const int64_t i = base + 1 + lane;
        return offsets[i < nO ? i : nO];
    };
    int64_t win = load_window(wbase);
    auto row_end = [&](int64_t r) -> int64_t {
        if (r - wbase >= 32) {
            wbase = r;
            win = load_window(wbase);
        }
        return __shfl_sync(kFullMask, win, static_cast<int>(r - wbase));
    };

    // gO[r] as the B operand of both products
    T ga_k[NTK][KSL]; // [k-step over l][n = k]: gO[k = 8 nt + qr][l = 4 ks + qc]
    T gb_k[KSK];      // [k-step over k][n = l]: gO[k = 4 ks + qc][l = 8 w + qr]
    bool stalled = false;
    // Waits for row r's grad_output, takes the warp's fragments (if the row has entries) and
    // says so; warp 0 then waits until every warp has, and starts the copy of row r + 2 into
    // the slot. The other warps reach this point for the same row within the same chunk, so
    // the wait is short.
    auto enter_row = [&](int64_t r, bool has_entries) {
        const int use = static_cast<int>(r - w.r0);
        const int slot = use & 1;
        const unsigned phase = (use >> 1) & 1;
        if (!mbarrier_wait(gbars + slot, phase)) {
            stalled = true;
            return;
        }
        if (has_entries) {
            const S* g = reinterpret_cast<const S*>(pipe_smem + lay.g_off + slot * g_slot_bytes);
#pragma unroll
            for (int nt = 0; nt < NTK; nt++)
#pragma unroll
                for (int ks = 0; ks < KSL; ks++) {
                    const int k = 8 * nt + qr, l = 4 * ks + qc;
                    ga_k[nt][ks] = (want_a && k < K && l < L) ? static_cast<T>(g[k * L + l]) : T(0);
                }
#pragma unroll
            for (int ks = 0; ks < KSK; ks++) {
                const int k = 4 * ks + qc, l = 8 * warp + qr;
                gb_k[ks] = (want_b && k < K && l < L) ? static_cast<T>(g[k * L + l]) : T(0);
            }
        }
        __syncwarp();
        if (lane == 0) mbarrier_arrive(gfree + slot);
        if (warp == 0 && r + 2 < w.r1) {
            if (!mbarrier_wait(gfree + slot, phase)) {
                stalled = true;
                return;
            }
            issue_g(r + 2);
        }
    };

    // positions of entries below are relative to e_first (the block's range fits an int)
    int64_t row = w.r0;
    int e = static_cast<int>(w.e_begin - w.e_first);
    const int e_stop = static_cast<int>(w.e_last - w.e_first);
    int hi = static_cast<int>(row_end(row) - w.e_first);
    enter_row(row, hi > e);
    auto next_rows = [&] {
        while (row < w.r1 && e == hi && !stalled) {
            row++;
            if (row < w.r1) {
                hi = static_cast<int>(row_end(row) - w.e_first);
                enter_row(row, hi > e);
            }
        }
    };

    const int l_out = 8 * warp + 2 * qc; // the warp's columns of X: l_out, l_out + 1
    const bool l_ok = l_out < L, two = l_out + 1 < L;
    // Guards of the contraction dimensions: only the last k-step over K and the last two over
    // L can leave the arrays (K > 4 (KSK - 1), L > 8 (NW - 1)). The other dimension of a
    // fragment needs none: what lies behind a row only reaches elements that are not stored.
    const bool a_last = 4 * (KSK - 1) + qc < K;
    const bool l_last0 = 4 * (KSL - 2) + qc < L, l_last1 = 4 * (KSL - 1) + qc < L;
    const bool k_st0 = 8 * (NTK - 1) + 2 * qc < K, k_st1 = 8 * (NTK - 1) + 2 * qc + 1 < K;
    const bool do_w = gW != nullptr, do_b = gB != nullptr;
    int turn = 0; // whose turn the next tile's grad_A is
    int c_lo = 0;
    for (int c = 0; c < w.nchunks && !stalled; c++, c_lo += CH) {
        __syncthreads(); // every warp has left the other stage: refill it
        issue(c + 1);
        if (!mbarrier_wait(bars + (c & 1), (c >> 1) & 1)) {
            stalled = true;
            break;
        }
        const unsigned char* stage = pipe_smem + (c & 1) * lay.stage_bytes;
        const S* As = reinterpret_cast<const S*>(stage + lay.a_off) + qc;
        const S* Bs = reinterpret_cast<const S*>(stage + lay.b_off);
        const S* Ws = reinterpret_cast<const S*>(stage + lay.w_off);
        const int32_t* pws = reinterpret_cast<const int32_t*>(stage + lay.pw_off);
        const int c_hi = c_lo + CH < e_stop ? c_lo + CH : e_stop;
        while (true) {
            next_rows();
            if (stalled || row >= w.r1 || e >= c_hi) break;
            const int seg_end = hi < c_hi ? hi : c_hi;
            const int first = e - c_lo, last = seg_end - c_lo;
            // eight entries per tile, entry t0 + qr in this lane; running pointers to its rows
            const S* arow = As + (first + qr) * K;
            const S* brow = Bs + (first + qr) * LP;
            const S* wrow_s = Ws + (first + qr) * LP;
            const int64_t eg0 = w.e_first + c_lo + first + qr;
            S* ga_dst = want_a ? gA + eg0 * K + 2 * qc : nullptr;
            S* gb_dst = do_b ? gB + eg0 * L + l_out : nullptr;
            // whole tiles need no test per entry, the last one may
            auto tile = [&](int t0, auto ragged) {
                constexpr bool kRagged = decltype(ragged)::value;
                const bool valid = !kRagged || t0 + qr < last;
                if (want_a && turn == warp) {
                    // grad_A[entry qr][k = 8 nt + 2 qc + {0,1}] = sum_l (B*W)[entry][l] gO[k][l]
                    T bf[KSL];
                    const S* bp = brow + qc;
                    const S* wp = wrow_s + qc;
#pragma unroll
                    for (int ks = 0; ks < KSL; ks++) {
                        const bool in = valid && (ks < KSL - 2 || (ks == KSL - 2 ? l_last0 : l_last1));
                        bf[ks] = in ? static_cast<T>(bp[4 * ks]) * static_cast<T>(wp[4 * ks]) : T(0);
                    }
#pragma unroll
                    for (int nt = 0; nt < NTK; nt++) {
                        T cfrag[2];
                        dmma0(cfrag, bf[0], ga_k[nt][0]);
#pragma unroll
                        for (int ks = 1; ks < KSL; ks++) dmma(cfrag, bf[ks], ga_k[nt][ks]);
                        if (valid && (nt < NTK - 1 || k_st0)) ga_dst[8 * nt] = static_cast<S>(cfrag[0]);
                        if (valid && (nt < NTK - 1 || k_st1)) ga_dst[8 * nt + 1] = static_cast<S>(cfrag[1]);
                    }
                }
                turn = turn + 1 == NW ? 0 : turn + 1;
                if (want_b) {
                    // X[entry qr][l = 8 w + 2 qc + {0,1}] = sum_k A[entry][k] gO[k][l]
                    T af[KSK];
#pragma unroll
                    for (int ks = 0; ks < KSK; ks++) {
                        const bool in = valid && (ks < KSK - 1 || a_last);
                        af[ks] = in ? static_cast<T>(arow[4 * ks]) : T(0);
                    }
                    T cfrag[2];
                    dmma0(cfrag, af[0], gb_k[0]);
#pragma unroll
                    for (int ks = 1; ks < KSK; ks++) dmma(cfrag, af[ks], gb_k[ks]);
                    if (valid && l_ok) {
                        T w0, w1, b0, b1;
                        if (pair_ok) { // L even: both columns exist, aligned pairs
                            const S2 w2 = *reinterpret_cast<const S2*>(wrow_s + l_out);
                            const S2 b2 = *reinterpret_cast<const S2*>(brow + l_out);
                            w0 = w2.x, w1 = w2.y, b0 = b2.x, b1 = b2.y;
                        } else {
                            w0 = wrow_s[l_out], b0 = brow[l_out];
                            w1 = two ? static_cast<T>(wrow_s[l_out + 1]) : T(0);
                            b1 = two ? static_cast<T>(brow[l_out + 1]) : T(0);
                        }
                        if (do_w) {
                            S* gw = gW + static_cast<int64_t>(pws[t0 + qr]) * L + l_out;
                            red_add(gw, static_cast<S>(cfrag[0] * b0));
                            if (two) red_add(gw + 1, static_cast<S>(cfrag[1] * b1));
                        }
                        if (do_b) {
                            if (pair_ok) {
                                S2 v2;
                                v2.x = static_cast<S>(cfrag[0] * w0), v2.y = static_cast<S>(cfrag[1] * w1);
                                *reinterpret_cast<S2*>(gb_dst) = v2;
                            } else {
                                gb_dst[0] = static_cast<S>(cfrag[0] * w0);
                                if (two) gb_dst[1] = static_cast<S>(cfrag[1] * w1);
                            }
                        }
                    }
                }
                arow += 8 * K, brow += 8 * LP, wrow_s += 8 * LP;
                if (want_a) ga_dst += 8 * K;
                if (do_b) gb_dst += 8 * L;
            };
            int t0 = first;
            for (; t0 + 8 <= last; t0 += 8) tile(t0, std::false_type{});
            if (t0 < last) tile(t0, std::true_type{});
            e = seg_end;
        }
    }
    if (stalled) {
        if (lane == 0) report_stalled(st);
        return;
    }
    // Rows after the last entry have no gradients to produce, but their grad_output copies
    // may still be in flight into this block's shared memory: wait for them before leaving.
    next_rows();
}
