// Outer-product scatter-add (with and without weights), forward and VJP, as streaming kernels:
// the entries of a sorted scatter index are walked in order, their A and B slices (contiguous
// in memory), the gathered W rows and the grad_output rows arrive in shared memory through
// bulk asynchronous copies (bulk.cuh) several chunks ahead, and the per-row contractions run
// on the FP64 tensor-core instruction (f32 operands are widened on the way from shared memory
// to the fragments, so f32 results carry f64 products and sums).
//
// Why: the kernels in opsa.cu that load MMA fragments straight from global memory keep the
// data in flight in registers. A warp then has two or three steps (a few hundred bytes) in
// flight and restarts its pipeline at every output row, and the measured time was the sum of
// those exposed latencies, not the bytes moved. Here a warp owns a contiguous range of output
// rows, hence one contiguous range of entries, which it streams through a ring of
// shared-memory stages: one elected lane issues one copy per slice, the copy engine keeps tens
// of kilobytes per SM in flight, row boundaries do not interrupt the stream, and the
// instruction stream is almost only fragment reads and MMAs.
//
// Included by opsa.cu (inside its unnamed namespace).

struct PipeLayout {
    int K, L;     // widths of A and B
    int LP;       // row stride of B (and W) inside a stage: L when the B slice is copied as one
                  // piece, L + 4 when rows are copied one by one (weighted: conflict-free)
    int row_pieces;      // weighted: 16-byte pieces of one B / W row
    int row_pieces_log2; // its log2 when it is a power of two, else -1
    int ch;       // entries per chunk: a multiple of 4 (at most 32 with weights: a lane per entry)
    int stages;   // chunks in flight per warp + 1: a power of two
    int stages_log2;
    int a_off, b_off, w_off, pw_off; // byte offsets inside a stage (16-byte aligned)
    int stage_bytes;
    int g_off;    // grad_output ring (VJP): g_slots rows of g_bytes each; unused in the forward
    int g_bytes;
    int g_slots;  // 2, or 1 when rows are long (the next row's copy then has a whole row's time)
    int bar_off;  // mbarriers: one per stage, then two for the grad_output ring
    int warp_bytes;
};

constexpr int kPipeWarps = 4;

__host__ __device__ constexpr int round16(size_t n) { return static_cast<int>((n + 15) / 16 * 16); }

__host__ __device__ constexpr PipeLayout pipe_layout(size_t s, int K, int L, bool weighted, bool vjp, int ch,
                                                     int stages, int g_slots = 2) {
    PipeLayout p{};
    p.K = K, p.L = L;
    p.LP = weighted ? L + 4 : L;
    p.ch = ch;
    p.stages_log2 = stages >= 8 ? 3 : stages >= 4 ? 2 : 1;
    p.stages = 1 << p.stages_log2;
    p.row_pieces = static_cast<int>(L * s / 16);
    p.row_pieces_log2 = -1;
    for (int b = 0; b < 6; b++)
        if (p.row_pieces == (1 << b)) p.row_pieces_log2 = b;
    p.a_off = 0;
    p.b_off = round16(static_cast<size_t>(ch) * K * s);
    p.w_off = p.b_off + round16(static_cast<size_t>(ch) * p.LP * s);
    p.pw_off = weighted ? p.w_off + round16(static_cast<size_t>(ch) * p.LP * s) : p.w_off;
    p.stage_bytes = weighted ? p.pw_off + round16(static_cast<size_t>(ch) * 4) : p.pw_off;
    p.g_bytes = static_cast<int>(static_cast<size_t>(K) * L * s);
    p.g_off = p.stages * p.stage_bytes;
    p.g_slots = g_slots < 2 ? 1 : 2;
    p.bar_off = p.g_off + (vjp ? p.g_slots * round16(p.g_bytes) : 0);
    p.warp_bytes = (p.bar_off + 8 * (p.stages + 2) + 127) / 128 * 128;
    return p;
}

// Issues the copies of the chunk that starts at entry e0 into one stage. pw_lane: lane i holds
// the (range-checked) W row of entry e0 + i. All lanes call it.
template <typename S, bool WEIGHTED>
__device__ __forceinline__ void pipe_issue_chunk(const PipeLayout& lay, unsigned char* stage,
                                                 uint64_t* bar, const S* __restrict__ A,
                                                 const S* __restrict__ B, const S* __restrict__ W,
                                                 int64_t e0, int64_t J, int32_t pw_lane, int lane) {
    const int K = lay.K, L = lay.L;
    const int n = static_cast<int>(J - e0 < lay.ch ? J - e0 : lay.ch);
    S* As = reinterpret_cast<S*>(stage + lay.a_off);
    S* Bs = reinterpret_cast<S*>(stage + lay.b_off);
    const unsigned a_bytes = static_cast<unsigned>(n) * K * sizeof(S), a_bulk = a_bytes & ~15u;
    const unsigned b_bytes = static_cast<unsigned>(n) * L * sizeof(S);
    const unsigned b_bulk = WEIGHTED ? 0u : (b_bytes & ~15u);
    if (lane == 0) {
        mbarrier_arrive_expect(bar, a_bulk + b_bulk);
        if (a_bulk) bulk_copy_in(As, A + e0 * K, a_bulk, bar);
        if (b_bulk) bulk_copy_in(Bs, B + e0 * L, b_bulk, bar);
    }
    if (WEIGHTED) {
        // B rows and the gathered W rows go into padded rows, 16 bytes per lane copy; the
        // barrier counts every lane's arrival (made when that lane's copies are complete).
        S* Ws = reinterpret_cast<S*>(stage + lay.w_off);
        int32_t* pws = reinterpret_cast<int32_t*>(stage + lay.pw_off);
        if (lane < n) pws[lane] = pw_lane;
        __syncwarp();
        constexpr int kPer = 16 / static_cast<int>(sizeof(S)); // scalars per piece
        if (lay.row_pieces_log2 >= 0 && lay.row_pieces <= 32) {
            // a lane keeps its piece column and walks down the rows, 32 / row_pieces at a time
            const int per_round = 32 >> lay.row_pieces_log2;
            const int c = (lane & (lay.row_pieces - 1)) * kPer;
            int r = lane >> lay.row_pieces_log2;
            S* bd = Bs + r * lay.LP + c;
            S* wd = Ws + r * lay.LP + c;
            const S* bsrc = B + (e0 + r) * L + c;
            for (; r < n; r += per_round) {
                lane_copy16(bd, bsrc);
                lane_copy16(wd, W + static_cast<int64_t>(pws[r]) * L + c);
                bd += per_round * lay.LP, wd += per_round * lay.LP, bsrc += per_round * L;
            }
        } else {
            const int pieces = n * lay.row_pieces;
            for (int i = lane; i < pieces; i += 32) {
                const int r = i / lay.row_pieces;
                const int c = (i - r * lay.row_pieces) * kPer;
                lane_copy16(Bs + r * lay.LP + c, B + (e0 + r) * L + c);
                lane_copy16(Ws + r * lay.LP + c, W + static_cast<int64_t>(pws[r]) * L + c);
            }
        }
        lane_copies_arrive(bar);
    }
    // The slices end where the arrays end: the last few scalars (less than 16 bytes) of the
    // very last chunk are fetched with plain loads.
    if (a_bulk != a_bytes)
        for (int i = a_bulk / sizeof(S) + lane; i < n * K; i += 32) As[i] = A[e0 * K + i];
    if (!WEIGHTED && b_bulk != b_bytes)
        for (int i = b_bulk / sizeof(S) + lane; i < n * L; i += 32) Bs[i] = B[e0 * L + i];
}

// State shared by the two kernels: which rows and entries the warp owns, the ring, and the
// window of segment offsets (32 at a time, one per lane).
struct PipeWarp {
    int64_t r0, r1;           // output rows [r0, r1)
    int64_t e_begin, e_last;  // their entries
    int64_t e_first;          // e_begin rounded down to a multiple of four: 16-byte aligned slices
    int nchunks;
};

__device__ __forceinline__ PipeWarp pipe_partition(const int64_t* __restrict__ offsets, int64_t nO,
                                                   int ch, int warp) {
    PipeWarp w;
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(gridDim.x) * kPipeWarps;
    const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * kPipeWarps + warp;
    w.r0 = balanced_row_split(offsets, nO, gwarp, total, lane);
    w.r1 = balanced_row_split(offsets, nO, gwarp + 1, total, lane);
    w.e_begin = offsets[w.r0];
    w.e_last = offsets[w.r1];
    w.e_first = w.e_begin & ~static_cast<int64_t>(3);
    w.nchunks = w.e_last > w.e_begin ? static_cast<int>((w.e_last - w.e_first + ch - 1) / ch) : 0;
    return w;
}

// The VJP produces one gradient row per entry and sums nothing over the entries of an output
// row (grad_W goes through atomics anyway), so its warps split the ENTRIES evenly, in units
// of four so that every warp's first slice is 16-byte aligned: a warp may start and stop
// inside a row. One very long row, or fewer rows than warps, still occupies the whole GPU.
// r0 .. r1 are then the rows the warp's entries fall into (the first and the last one possibly
// shared with its neighbours).
__device__ __forceinline__ PipeWarp pipe_partition_entries(const int64_t* __restrict__ offsets,
                                                           int64_t nO, int ch, int warp) {
    PipeWarp w;
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(gridDim.x) * kPipeWarps;
    const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * kPipeWarps + warp;
    const int64_t J = offsets[nO], quads = (J + 3) / 4;
    const int64_t lo = quads / total * gwarp + quads % total * gwarp / total;
    const int64_t hi = quads / total * (gwarp + 1) + quads % total * (gwarp + 1) / total;
    w.e_begin = w.e_first = 4 * lo < J ? 4 * lo : J;
    w.e_last = 4 * hi < J ? 4 * hi : J;
    w.r0 = w.r1 = 0;
    w.nchunks = 0;
    if (w.e_last <= w.e_begin) return w;
    // the row that holds e_begin: the last one that starts at or before it (offsets[0] = 0 and
    // offsets[nO] = J > e_begin bracket it); likewise for the last entry
    w.r0 = warp_count_weighted_le(offsets, nO + 1, 0, w.e_begin, lane) - 1;
    w.r1 = warp_count_weighted_le(offsets, nO + 1, 0, w.e_last - 1, lane);
    w.nchunks = static_cast<int>((w.e_last - w.e_first + ch - 1) / ch);
    return w;
}

// ------------------------------------------------------------------------------- forward
// O[r] = A[seg]^T (B[seg] * W[PW[seg]]) with the entries as the MMA's k dimension, four per
// step. MT = ceil(K / 8), NT = ceil(L / 8).
//
// KC, LC > 0: K and L fixed at compile time (with the default ring: kFixedChunk entries per
// chunk, two stages): every offset inside a stage and every stride becomes a constant, which
// removes about a third of the instructions of the run-time-width kernel. The host picks such
// an instantiation when the shapes match one of the common ones and the run-time layout equals
// the fixed one; lay_rt is then ignored.
template <bool WEIGHTED> constexpr int kFixedChunk = WEIGHTED ? 8 : 32;

template <typename S, bool WEIGHTED, bool VJP, int KC, int LC>
__device__ __forceinline__ PipeLayout fixed_layout_or(const PipeLayout& run_time) {
    if constexpr (KC > 0) {
        constexpr PipeLayout fixed = pipe_layout(sizeof(S), KC, LC, WEIGHTED, VJP, kFixedChunk<WEIGHTED>, 2);
        PipeLayout lay = fixed;
        // the depth of the grad_output ring is the host's choice: it moves what lies behind it
        lay.g_slots = run_time.g_slots, lay.bar_off = run_time.bar_off, lay.warp_bytes = run_time.warp_bytes;
        return lay;
    } else {
        return run_time;
    }
}

template <typename S, int MT, int NT, bool WEIGHTED, int KC = 0, int LC = 0>
__global__ void __launch_bounds__(kPipeWarps * 32, (KC > 0 && WEIGHTED) ? 5 : 4)
opsa_fwd_pipe(S* __restrict__ O, const S* __restrict__ A, const S* __restrict__ B,
              const S* __restrict__ W, const int32_t* __restrict__ PW,
              const int64_t* __restrict__ offsets, int64_t J, int64_t nO, int64_t nW,
              PipeLayout lay_rt, Status st) {
    using T = double;
    const PipeLayout lay = fixed_layout_or<S, WEIGHTED, false, KC, LC>(lay_rt);
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    if (saw_unsorted(st)) return; // the atomic kernel of the same call does the work
    const int lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0); // uniform for the compiler
    const int qr = lane >> 2, qc = lane & 3;
    const int K = lay.K, L = lay.L, LP = lay.LP, CH = lay.ch, NS = lay.stages;
    unsigned char* area = pipe_smem + static_cast<size_t>(warp) * lay.warp_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(area + lay.bar_off);
    if (lane == 0) {
        for (int s = 0; s < NS; s++) mbarrier_init(bars + s, WEIGHTED ? 33 : 1);
        mbarrier_init_fence();
    }
    __syncwarp();
    const PipeWarp w = pipe_partition(offsets, nO, CH, warp);
    if (w.r0 >= w.r1) return;

    auto load_pw = [&](int c) -> int32_t {
        int32_t pw = 0;
        const int64_t e = w.e_first + static_cast<int64_t>(c) * CH + lane;
        if (WEIGHTED && lane < CH && e < J) {
            pw = __ldg(PW + e);
            if (clamp_index(pw, static_cast<int32_t>(nW))) report_bad_index(st, 1);
        }
        return pw;
    };
    int issued = 0;
    int32_t pw_reg = load_pw(0);
    auto issue_next = [&]() {
        if (issued < w.nchunks) {
            const int s = issued & (NS - 1);
            pipe_issue_chunk<S, WEIGHTED>(lay, area + s * lay.stage_bytes, bars + s, A, B, W,
                                          w.e_first + static_cast<int64_t>(issued) * CH, J, pw_reg,
                                          lane);
            issued++;
            if (WEIGHTED && issued < w.nchunks) pw_reg = load_pw(issued);
        }
    };
    for (int i = 0; i < NS - 1; i++) issue_next();

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

    T acc[MT][NT][2];
    auto clear = [&] {
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) acc[mt][nt][0] = acc[mt][nt][1] = T(0);
    };
    const int64_t rowsize = static_cast<int64_t>(K) * L;
    const bool pair_ok = L % 2 == 0 && reinterpret_cast<uintptr_t>(O) % (2 * sizeof(S)) == 0;
    // element (mt, nt, h) is O[r, k = 8 mt + qr, l = 8 nt + 2 qc + h]
    auto flush = [&](int64_t r) {
        S* dst = O + r * rowsize;
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const int k = 8 * mt + qr;
            if (k >= K) continue;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int l = 8 * nt + 2 * qc;
                if (l >= L) continue;
                S* d2 = dst + k * L + l;
                if (pair_ok) {
                    typename VecOf<S, 2>::type v2;
                    v2.x = static_cast<S>(acc[mt][nt][0]), v2.y = static_cast<S>(acc[mt][nt][1]);
                    *reinterpret_cast<typename VecOf<S, 2>::type*>(d2) = v2;
                } else {
                    d2[0] = static_cast<S>(acc[mt][nt][0]);
                    if (l + 1 < L) d2[1] = static_cast<S>(acc[mt][nt][1]);
                }
            }
        }
    };

    clear();
    // positions of entries below are relative to e_first (the warp's range fits an int)
    int64_t row = w.r0;
    int e = static_cast<int>(w.e_begin - w.e_first);
    const int e_stop = static_cast<int>(w.e_last - w.e_first);
    int hi = static_cast<int>(row_end(row) - w.e_first);
    // Rows whose last entry has been consumed (and rows without entries) are written out.
    auto finish_rows = [&] {
        while (row < w.r1 && e == hi) {
            flush(row);
            clear();
            row++;
            if (row < w.r1) hi = static_cast<int>(row_end(row) - w.e_first);
        }
    };
    // which fragment rows (k) and columns (l) of this lane exist
    bool ka[MT], la[NT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) ka[mt] = 8 * mt + qr < K;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) la[nt] = 8 * nt + qr < L;

    int c_lo = 0;
    for (int c = 0; c < w.nchunks; c++, c_lo += CH) {
        issue_next(); // into the stage that the previous iteration released
        const int s = c & (NS - 1);
        if (!mbarrier_wait(bars + s, (c >> lay.stages_log2) & 1)) {
            if (lane == 0) report_stalled(st);
            return;
        }
        __syncwarp();
        const unsigned char* stage = area + s * lay.stage_bytes;
        const S* As = reinterpret_cast<const S*>(stage + lay.a_off);
        const S* Bs = reinterpret_cast<const S*>(stage + lay.b_off);
        const S* Ws = reinterpret_cast<const S*>(stage + lay.w_off);
        const int c_hi = c_lo + CH < e_stop ? c_lo + CH : e_stop;
        while (true) {
            finish_rows();
            if (row >= w.r1 || e >= c_hi) break;
            const int seg_end = hi < c_hi ? hi : c_hi;
            // entries [e, seg_end) of the current row, four per MMA step: fragment
            // A^T[k = 8 mt + qr][entry qc], (B*W)[entry qc][l = 8 nt + qr]. Whole steps need no
            // test per entry, the last one of a segment may.
            const int first = e - c_lo, last = seg_end - c_lo;
            auto step = [&](int s0, auto ragged) {
                constexpr bool kRagged = decltype(ragged)::value;
                const int idx = s0 + qc;
                const bool valid = !kRagged || idx < last;
                const S* ap = As + idx * K + qr;
                const S* bp = Bs + idx * LP + qr;
                const S* wp = Ws + idx * LP + qr;
                T af[MT], bf[NT];
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
                    af[mt] = (valid && ka[mt]) ? static_cast<T>(ap[8 * mt]) : T(0);
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const bool in = valid && la[nt];
                    T v = in ? static_cast<T>(bp[8 * nt]) : T(0);
                    if (WEIGHTED && in) v *= static_cast<T>(wp[8 * nt]);
                    bf[nt] = v;
                }
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) dmma(acc[mt][nt], af[mt], bf[nt]);
            };
            int s0 = first;
#pragma unroll 2
            for (; s0 + 4 <= last; s0 += 4) step(s0, std::false_type{});
            if (s0 < last) step(s0, std::true_type{});
            e = seg_end;
        }
        __syncwarp(); // the stage may be refilled by the copies issued next
    }
    finish_rows();
}

// ----------------------------------------------------------------------------------- VJP
// For the entries of one output row, grad_A[seg] = (B*W)[seg] gO[r]^T and X = A[seg] gO[r]
// (grad_B = X * W, grad_W[PW] += X * B) with gO[r] as the common factor, kept in registers as
// MMA fragments while the row lasts; entries are the MMA's m dimension, eight per tile.
// KT = ceil(K / 4), LT8 = ceil(L / 8).
template <typename S, int KT, int LT8, bool WEIGHTED, int KC = 0, int LC = 0>
__global__ void __launch_bounds__(kPipeWarps * 32, (KC > 0 && WEIGHTED) ? 4 : 3)
opsa_vjp_pipe(S* __restrict__ gA, S* __restrict__ gB, S* __restrict__ gW,
              const S* __restrict__ gO, const S* __restrict__ A, const S* __restrict__ B,
              const S* __restrict__ W, const int32_t* __restrict__ PW,
              const int64_t* __restrict__ offsets, int64_t J, int64_t nO, int64_t nW,
              PipeLayout lay_rt, Status st) {
    using T = double;
    const PipeLayout lay = fixed_layout_or<S, WEIGHTED, true, KC, LC>(lay_rt);
    using S2 = typename VecOf<S, 2>::type;
    constexpr int NTK = (KT + 1) / 2; // 8-wide tiles over K
    constexpr int KSL = 2 * LT8;      // k-steps over L
    constexpr int NTL = LT8;          // 8-wide tiles over L
    constexpr int KSK = KT;           // k-steps over K
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    if (saw_unsorted(st)) return; // the entry-per-lane kernel of the same call does the work
    const int lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0);
    const int qr = lane >> 2, qc = lane & 3;
    const int K = lay.K, L = lay.L, LP = lay.LP, CH = lay.ch, NS = lay.stages;
    unsigned char* area = pipe_smem + static_cast<size_t>(warp) * lay.warp_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(area + lay.bar_off);
    uint64_t* gbars = bars + NS;
    if (lane == 0) {
        for (int s = 0; s < NS; s++) mbarrier_init(bars + s, WEIGHTED ? 33 : 1);
        mbarrier_init(gbars, 1);
        mbarrier_init(gbars + 1, 1);
        mbarrier_init_fence();
    }
    __syncwarp();
    const PipeWarp w = pipe_partition_entries(offsets, nO, CH, warp);
    if (w.r0 >= w.r1 || w.nchunks == 0) return; // gradients exist per entry only

    const bool want_a = gA != nullptr, want_b = gB != nullptr || (WEIGHTED && gW != nullptr);
    const bool pair_ok = L % 2 == 0 && (gB == nullptr || reinterpret_cast<uintptr_t>(gB) % (2 * sizeof(S)) == 0);
    const int64_t rowsize = static_cast<int64_t>(K) * L;
    const int g_slot_bytes = (lay.g_bytes + 15) / 16 * 16;

    auto load_pw = [&](int c) -> int32_t {
        int32_t pw = 0;
        const int64_t e = w.e_first + static_cast<int64_t>(c) * CH + lane;
        if (WEIGHTED && lane < CH && e < J) {
            pw = __ldg(PW + e);
            if (clamp_index(pw, static_cast<int32_t>(nW))) report_bad_index(st, 1);
        }
        return pw;
    };
    int issued = 0;
    int32_t pw_reg = load_pw(0);
    auto issue_next = [&]() {
        if (issued < w.nchunks) {
            const int s = issued & (NS - 1);
            pipe_issue_chunk<S, WEIGHTED>(lay, area + s * lay.stage_bytes, bars + s, A, B, W,
                                          w.e_first + static_cast<int64_t>(issued) * CH, J, pw_reg,
                                          lane);
            issued++;
            if (WEIGHTED && issued < w.nchunks) pw_reg = load_pw(issued);
        }
    };
    // grad_output rows r0, r0 + 1, ... go through a ring of two slots
    const bool two_slots = lay.g_slots == 2;
    auto issue_g = [&](int64_t r) {
        if (r < w.r1 && lane == 0) {
            const int slot = two_slots ? static_cast<int>(r - w.r0) & 1 : 0;
            mbarrier_arrive_expect(gbars + slot, static_cast<unsigned>(lay.g_bytes));
            bulk_copy_in(area + lay.g_off + slot * g_slot_bytes, gO + r * rowsize,
                         static_cast<unsigned>(lay.g_bytes), gbars + slot);
        }
    };
    issue_g(w.r0);
    if (two_slots) issue_g(w.r0 + 1);
    for (int i = 0; i < NS - 1; i++) issue_next();

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
    T gb_k[NTL][KSK]; // [k-step over k][n = l]: gO[k = 4 ks + qc][l = 8 nt + qr]
    bool stalled = false;
    // Waits for row r's grad_output, takes its fragments (if the row has entries) and hands
    // the slot to row r + 2.
    auto enter_row = [&](int64_t r, bool has_entries) {
        const int use = static_cast<int>(r - w.r0);
        const int slot = two_slots ? use & 1 : 0;
        if (!mbarrier_wait(gbars + slot, (two_slots ? use >> 1 : use) & 1)) {
            stalled = true;
            return;
        }
        if (has_entries) {
            const S* g = reinterpret_cast<const S*>(area + lay.g_off + slot * g_slot_bytes);
#pragma unroll
            for (int nt = 0; nt < NTK; nt++)
#pragma unroll
                for (int ks = 0; ks < KSL; ks++) {
                    const int k = 8 * nt + qr, l = 4 * ks + qc;
                    ga_k[nt][ks] = (want_a && k < K && l < L) ? static_cast<T>(g[k * L + l]) : T(0);
                }
#pragma unroll
            for (int nt = 0; nt < NTL; nt++)
#pragma unroll
                for (int ks = 0; ks < KSK; ks++) {
                    const int k = 4 * ks + qc, l = 8 * nt + qr;
                    gb_k[nt][ks] = (want_b && k < K && l < L) ? static_cast<T>(g[k * L + l]) : T(0);
                }
        }
        __syncwarp(); // every lane has its fragments: the slot can be refilled
        issue_g(r + (two_slots ? 2 : 1));
    };

    // positions of entries below are relative to e_first (the warp's range fits an int)
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

    int c_lo = 0;
    for (int c = 0; c < w.nchunks && !stalled; c++, c_lo += CH) {
        issue_next();
        const int s = c & (NS - 1);
        if (!mbarrier_wait(bars + s, (c >> lay.stages_log2) & 1)) {
            stalled = true;
            break;
        }
        __syncwarp();
        const unsigned char* stage = area + s * lay.stage_bytes;
        const S* As = reinterpret_cast<const S*>(stage + lay.a_off);
        const S* Bs = reinterpret_cast<const S*>(stage + lay.b_off);
        const S* Ws = reinterpret_cast<const S*>(stage + lay.w_off);
        const int32_t* pws = reinterpret_cast<const int32_t*>(stage + lay.pw_off);
        const int c_hi = c_lo + CH < e_stop ? c_lo + CH : e_stop;
        while (true) {
            next_rows();
            if (stalled || row >= w.r1 || e >= c_hi) break;
            const int seg_end = hi < c_hi ? hi : c_hi;
            const int first = e - c_lo, last = seg_end - c_lo;
            // eight entries per tile: whole tiles need no test per entry, the last one may
            auto tile = [&](int t0, auto ragged) {
                constexpr bool kRagged = decltype(ragged)::value;
                const int idx = t0 + qr; // this lane's entry of the tile, within the chunk
                const bool valid = !kRagged || idx < last;
                const int64_t eg = w.e_first + c_lo + idx;
                const S* brow = Bs + idx * LP;
                const S* wrow_s = Ws + idx * LP;
                if (want_a) {
                    // grad_A[entry qr][k = 8 nt + 2 qc + {0,1}] = sum_l (B*W)[entry][l] gO[k][l]
                    T bf[KSL];
                    const S* bp = brow + qc;
                    const S* wp = wrow_s + qc;
#pragma unroll
                    for (int ks = 0; ks < KSL; ks++) {
                        const bool in = valid && 4 * ks + qc < L;
                        T v = in ? static_cast<T>(bp[4 * ks]) : T(0);
                        if (WEIGHTED && in) v *= static_cast<T>(wp[4 * ks]);
                        bf[ks] = v;
                    }
                    S* dst = gA + eg * K + 2 * qc;
#pragma unroll
                    for (int nt = 0; nt < NTK; nt++) {
                        T cfrag[2];
                        dmma0(cfrag, bf[0], ga_k[nt][0]);
#pragma unroll
                        for (int ks = 1; ks < KSL; ks++) dmma(cfrag, bf[ks], ga_k[nt][ks]);
                        const int k = 8 * nt + 2 * qc;
                        if (valid && k < K) dst[8 * nt] = static_cast<S>(cfrag[0]);
                        if (valid && k + 1 < K) dst[8 * nt + 1] = static_cast<S>(cfrag[1]);
                    }
                }
                if (want_b) {
                    // X[entry qr][l = 8 nt + 2 qc + {0,1}] = sum_k A[entry][k] gO[k][l]
                    T af[KSK];
                    const S* ap = As + idx * K + qc;
#pragma unroll
                    for (int ks = 0; ks < KSK; ks++)
                        af[ks] = (valid && 4 * ks + qc < K) ? static_cast<T>(ap[4 * ks]) : T(0);
                    const int32_t wrow = (WEIGHTED && valid) ? pws[idx] : 0;
                    const S* wp = wrow_s + 2 * qc;
                    const S* bp = brow + 2 * qc;
                    S* gw = WEIGHTED && gW != nullptr ? gW + static_cast<int64_t>(wrow) * L + 2 * qc : nullptr;
                    S* dst = gB != nullptr ? gB + eg * L + 2 * qc : nullptr;
#pragma unroll
                    for (int nt = 0; nt < NTL; nt++) {
                        T cfrag[2];
                        dmma0(cfrag, af[0], gb_k[nt][0]);
#pragma unroll
                        for (int ks = 1; ks < KSK; ks++) dmma(cfrag, af[ks], gb_k[nt][ks]);
                        const int l = 8 * nt + 2 * qc;
                        if (!valid || l >= L) continue;
                        const bool two = l + 1 < L;
                        if (WEIGHTED) {
                            T w0, w1, b0, b1;
                            if (pair_ok) { // L even: both columns exist, 16-byte aligned pairs
                                const S2 w2 = *reinterpret_cast<const S2*>(wp + 8 * nt);
                                const S2 b2 = *reinterpret_cast<const S2*>(bp + 8 * nt);
                                w0 = w2.x, w1 = w2.y, b0 = b2.x, b1 = b2.y;
                            } else {
                                w0 = wp[8 * nt], b0 = bp[8 * nt];
                                w1 = two ? static_cast<T>(wp[8 * nt + 1]) : T(0);
                                b1 = two ? static_cast<T>(bp[8 * nt + 1]) : T(0);
                            }
                            if (gw != nullptr) {
                                red_add(gw + 8 * nt, static_cast<S>(cfrag[0] * b0));
                                if (two) red_add(gw + 8 * nt + 1, static_cast<S>(cfrag[1] * b1));
                            }
                            cfrag[0] *= w0;
                            cfrag[1] *= w1;
                        }
                        if (dst != nullptr) {
                            if (pair_ok) {
                                S2 v2;
                                v2.x = static_cast<S>(cfrag[0]), v2.y = static_cast<S>(cfrag[1]);
                                *reinterpret_cast<S2*>(dst + 8 * nt) = v2;
                            } else {
                                dst[8 * nt] = static_cast<S>(cfrag[0]);
                                if (two) dst[8 * nt + 1] = static_cast<S>(cfrag[1]);
                            }
                        }
                    }
                }
            };
            int t0 = first;
            for (; t0 + 8 <= last; t0 += 8) tile(t0, std::false_type{});
            if (t0 < last) tile(t0, std::true_type{});
            e = seg_end;
        }
        __syncwarp(); // the stage may be refilled by the copies issued next
    }
    if (stalled) {
        if (lane == 0) report_stalled(st);
        return;
    }
    // Rows after the last entry have no gradients to produce, but their grad_output copies
    // may still be in flight into this block's shared memory: wait for them before leaving.
    next_rows();
}

// ------------------------------------------------------------- f32 on the TF32 tensor path
// For f32 operands the FP64 MMA route above is bound by the FP64 tensor pipe (63 % busy at
// 57 % of the HBM peak): f32 moves half the bytes but needs the same number of FP64 MMAs. The
// kernels below run the same streaming structure on mma.sync m16n8k8 TF32 with the
// three-product split: every f32 operand x is taken as hi + lo with hi = the TF32 part of x,
// lo = the TF32 part of x - hi, and a product a*b as a_hi*b_hi + a_hi*b_lo + a_lo*b_hi (the
// dropped a_lo*b_lo is below 2^-20 |ab|), accumulated in f32. The result is f32-accurate (the parity tests hold
// it to 1e-5 of the largest output, like every f32 path). In the forward, where one output
// row sums over arbitrarily many entries, only the small correction products are chained
// through the tensor core's accumulator (which may round towards zero); the main products of
// every 8-entry step start from zero and are added to the running sums by ordinary f32
// additions.
__device__ __forceinline__ void tf32_split(float x, unsigned& hi, unsigned& lo) {
    // hi = the upper 19 bits of x (what the tensor core reads of an f32 register anyway), lo =
    // x - hi, exact in f32, of which the tensor core again reads the upper 19 bits. Dropping
    // bits instead of rounding (cvt.rna.tf32.f32, about five instructions here) leaves
    // |x - hi - lo'| < 2^-20 |x|, well inside the f32 tolerance, at two instructions.
    hi = __float_as_uint(x) & 0xffffe000u;
    lo = __float_as_uint(x - __uint_as_float(hi));
}

// d += a b for one m16n8k8 tile. Fragments (g = lane / 4, t = lane % 4):
// a0 (g, t) a1 (g + 8, t) a2 (g, t + 4) a3 (g + 8, t + 4); b0 (k = t, n = g) b1 (k = t + 4,
// n = g); d0 (g, 2 t) d1 (g, 2 t + 1) d2 (g + 8, 2 t) d3 (g + 8, 2 t + 1).
__device__ __forceinline__ void mma_tf32(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Forward, f32, K <= 16, L <= 32, no weights: O[r] = A[seg]^T B[seg], eight entries per step
// (the entries are the MMA's k dimension). NT = ceil(L / 8).
template <int NT>
__global__ void __launch_bounds__(kPipeWarps * 32, 4)
opsa_fwd_pipe_tf32(float* __restrict__ O, const float* __restrict__ A, const float* __restrict__ B,
                   const int64_t* __restrict__ offsets, int64_t J, int64_t nO, PipeLayout lay,
                   Status st) {
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    if (saw_unsorted(st)) return; // the atomic kernel of the same call does the work
    const int lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0);
    const int g = lane >> 2, t = lane & 3;
    const int K = lay.K, L = lay.L, CH = lay.ch, NS = lay.stages;
    unsigned char* area = pipe_smem + static_cast<size_t>(warp) * lay.warp_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(area + lay.bar_off);
    if (lane == 0) {
        for (int s = 0; s < NS; s++) mbarrier_init(bars + s, 1);
        mbarrier_init_fence();
    }
    __syncwarp();
    const PipeWarp w = pipe_partition(offsets, nO, CH, warp);
    if (w.r0 >= w.r1) return;

    int issued = 0;
    auto issue_next = [&]() {
        if (issued < w.nchunks) {
            const int s = issued & (NS - 1);
            pipe_issue_chunk<float, false>(lay, area + s * lay.stage_bytes, bars + s, A, B, nullptr,
                                           w.e_first + static_cast<int64_t>(issued) * CH, J, 0, lane);
            issued++;
        }
    };
    for (int i = 0; i < NS - 1; i++) issue_next();

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

    float sum[NT][4], corr[NT][4]; // running sums of the main products / chained corrections
    auto clear = [&] {
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) sum[nt][i] = corr[nt][i] = 0.0f;
    };
    const int64_t rowsize = static_cast<int64_t>(K) * L;
    const bool pair_ok = L % 2 == 0 && reinterpret_cast<uintptr_t>(O) % 8 == 0;
    const bool ka0 = g < K, ka1 = g + 8 < K; // which of the lane's two A^T rows exist
    // element (nt, 2 h + i) is O[r, k = g + 8 h, l = 8 nt + 2 t + i]
    auto flush = [&](int64_t r) {
        float* dst = O + r * rowsize;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int k = g + 8 * h;
            if (k >= K) continue;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int l = 8 * nt + 2 * t;
                if (l >= L) continue;
                const float v0 = sum[nt][2 * h] + corr[nt][2 * h];
                const float v1 = sum[nt][2 * h + 1] + corr[nt][2 * h + 1];
                float* d2 = dst + k * L + l;
                if (pair_ok) {
                    *reinterpret_cast<float2*>(d2) = make_float2(v0, v1);
                } else {
                    d2[0] = v0;
                    if (l + 1 < L) d2[1] = v1;
                }
            }
        }
    };

    clear();
    int64_t e = w.e_begin, row = w.r0;
    int64_t hi = row_end(row);
    auto finish_rows = [&] {
        while (row < w.r1 && e == hi) {
            flush(row);
            clear();
            row++;
            if (row < w.r1) hi = row_end(row);
        }
    };

    for (int c = 0; c < w.nchunks; c++) {
        issue_next();
        const int s = c & (NS - 1);
        if (!mbarrier_wait(bars + s, (c >> lay.stages_log2) & 1)) {
            if (lane == 0) report_stalled(st);
            return;
        }
        __syncwarp();
        const unsigned char* stage = area + s * lay.stage_bytes;
        const float* As = reinterpret_cast<const float*>(stage + lay.a_off);
        const float* Bs = reinterpret_cast<const float*>(stage + lay.b_off);
        const int64_t c_lo = w.e_first + static_cast<int64_t>(c) * CH;
        const int64_t c_hi = c_lo + CH < w.e_last ? c_lo + CH : w.e_last;
        while (true) {
            finish_rows();
            if (row >= w.r1 || e >= c_hi) break;
            const int64_t seg_end = hi < c_hi ? hi : c_hi;
            const int first = static_cast<int>(e - c_lo), last = static_cast<int>(seg_end - c_lo);
            // A^T fragment: (row k, column entry); B fragment: (row entry, column l). Whole
            // steps of eight entries need no per-entry test; the last, ragged one does.
            auto step = [&](int s0, auto ragged) {
                constexpr bool kRagged = decltype(ragged)::value;
                const int e0 = s0 + t, e1 = e0 + 4;
                const bool v0 = !kRagged || e0 < last, v1 = !kRagged || e1 < last;
                const float* a0 = As + e0 * K + g;
                const float* a1 = As + e1 * K + g;
                unsigned ah[4], al[4];
                tf32_split((v0 && ka0) ? a0[0] : 0.0f, ah[0], al[0]);
                tf32_split((v0 && ka1) ? a0[8] : 0.0f, ah[1], al[1]);
                tf32_split((v1 && ka0) ? a1[0] : 0.0f, ah[2], al[2]);
                tf32_split((v1 && ka1) ? a1[8] : 0.0f, ah[3], al[3]);
                const float* b0 = Bs + e0 * L + g;
                const float* b1 = Bs + e1 * L + g;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const bool lb = 8 * nt + g < L;
                    unsigned bh[2], bl[2];
                    tf32_split((v0 && lb) ? b0[8 * nt] : 0.0f, bh[0], bl[0]);
                    tf32_split((v1 && lb) ? b1[8 * nt] : 0.0f, bh[1], bl[1]);
                    float main_[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    mma_tf32(main_, ah, bh);
                    mma_tf32(corr[nt], ah, bl);
                    mma_tf32(corr[nt], al, bh);
#pragma unroll
                    for (int i = 0; i < 4; i++) sum[nt][i] += main_[i];
                }
            };
            int s0 = first;
            for (; s0 + 8 <= last; s0 += 8) step(s0, std::false_type{});
            if (s0 < last) step(s0, std::true_type{});
            e = seg_end;
        }
        __syncwarp();
    }
    finish_rows();
}

// VJP, f32, K <= 16, L <= 32, no weights: for the entries of one output row grad_A[seg] =
// B[seg] gO[r]^T and grad_B[seg] = A[seg] gO[r], sixteen entries per tile (the entries are the
// MMA's m dimension), gO[r] split once per row and kept in registers. KS = ceil(K / 8),
// LS = ceil(L / 8).
template <int KS, int LS>
__global__ void __launch_bounds__(kPipeWarps * 32, 3)
opsa_vjp_pipe_tf32(float* __restrict__ gA, float* __restrict__ gB, const float* __restrict__ gO,
                   const float* __restrict__ A, const float* __restrict__ B,
                   const int64_t* __restrict__ offsets, int64_t J, int64_t nO, PipeLayout lay,
                   Status st) {
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    if (saw_unsorted(st)) return; // the entry-per-lane kernel of the same call does the work
    const int lane = threadIdx.x & 31;
    const int warp = __shfl_sync(kFullMask, threadIdx.x >> 5, 0);
    const int g = lane >> 2, t = lane & 3;
    const int K = lay.K, L = lay.L, CH = lay.ch, NS = lay.stages;
    unsigned char* area = pipe_smem + static_cast<size_t>(warp) * lay.warp_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(area + lay.bar_off);
    uint64_t* gbars = bars + NS;
    if (lane == 0) {
        for (int s = 0; s < NS + 2; s++) mbarrier_init(bars + s, 1);
        mbarrier_init_fence();
    }
    __syncwarp();
    const PipeWarp w = pipe_partition_entries(offsets, nO, CH, warp);
    if (w.r0 >= w.r1 || w.nchunks == 0) return;
    const bool want_a = gA != nullptr, want_b = gB != nullptr;
    const int64_t rowsize = static_cast<int64_t>(K) * L;
    const int g_slot_bytes = (lay.g_bytes + 15) / 16 * 16;
    const bool pair_a = K % 2 == 0 && reinterpret_cast<uintptr_t>(gA) % 8 == 0;
    const bool pair_b = L % 2 == 0 && reinterpret_cast<uintptr_t>(gB) % 8 == 0;

    int issued = 0;
    auto issue_next = [&]() {
        if (issued < w.nchunks) {
            const int s = issued & (NS - 1);
            pipe_issue_chunk<float, false>(lay, area + s * lay.stage_bytes, bars + s, A, B, nullptr,
                                           w.e_first + static_cast<int64_t>(issued) * CH, J, 0, lane);
            issued++;
        }
    };
    auto issue_g = [&](int64_t r) {
        if (r < w.r1 && lane == 0) {
            const int slot = static_cast<int>(r - w.r0) & 1;
            mbarrier_arrive_expect(gbars + slot, static_cast<unsigned>(lay.g_bytes));
            bulk_copy_in(area + lay.g_off + slot * g_slot_bytes, gO + r * rowsize,
                         static_cast<unsigned>(lay.g_bytes), gbars + slot);
        }
    };
    issue_g(w.r0);
    issue_g(w.r0 + 1);
    for (int i = 0; i < NS - 1; i++) issue_next();

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

    // gO[r] as the B operand of both products, split into hi and lo:
    // ga: [k-step over l][tile over k]: b0 = gO[k = 8 nt + g][l = 8 ks + t], b1 = ... l + 4
    // gb: [k-step over k][tile over l]: b0 = gO[k = 8 ks + t][l = 8 nt + g], b1 = ... k + 4
    unsigned ga_h[LS][KS][2], ga_l[LS][KS][2], gb_h[KS][LS][2], gb_l[KS][LS][2];
    bool stalled = false;
    auto enter_row = [&](int64_t r, bool has_entries) {
        const int use = static_cast<int>(r - w.r0);
        if (!mbarrier_wait(gbars + (use & 1), (use >> 1) & 1)) {
            stalled = true;
            return;
        }
        if (has_entries) {
            const float* gs = reinterpret_cast<const float*>(area + lay.g_off + (use & 1) * g_slot_bytes);
#pragma unroll
            for (int ks = 0; ks < LS; ks++)
#pragma unroll
                for (int nt = 0; nt < KS; nt++)
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const int k = 8 * nt + g, l = 8 * ks + t + 4 * i;
                        tf32_split((want_a && k < K && l < L) ? gs[k * L + l] : 0.0f, ga_h[ks][nt][i],
                                   ga_l[ks][nt][i]);
                    }
#pragma unroll
            for (int ks = 0; ks < KS; ks++)
#pragma unroll
                for (int nt = 0; nt < LS; nt++)
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const int k = 8 * ks + t + 4 * i, l = 8 * nt + g;
                        tf32_split((want_b && k < K && l < L) ? gs[k * L + l] : 0.0f, gb_h[ks][nt][i],
                                   gb_l[ks][nt][i]);
                    }
        }
        __syncwarp();
        issue_g(r + 2);
    };

    int64_t e = w.e_begin, row = w.r0;
    int64_t hi = row_end(row);
    enter_row(row, hi > e);
    auto next_rows = [&] {
        while (row < w.r1 && e == hi && !stalled) {
            row++;
            if (row < w.r1) {
                hi = row_end(row);
                enter_row(row, hi > e);
            }
        }
    };

    for (int c = 0; c < w.nchunks && !stalled; c++) {
        issue_next();
        const int s = c & (NS - 1);
        if (!mbarrier_wait(bars + s, (c >> lay.stages_log2) & 1)) {
            stalled = true;
            break;
        }
        __syncwarp();
        const unsigned char* stage = area + s * lay.stage_bytes;
        const float* As = reinterpret_cast<const float*>(stage + lay.a_off);
        const float* Bs = reinterpret_cast<const float*>(stage + lay.b_off);
        const int64_t c_lo = w.e_first + static_cast<int64_t>(c) * CH;
        const int64_t c_hi = c_lo + CH < w.e_last ? c_lo + CH : w.e_last;
        while (true) {
            next_rows();
            if (stalled || row >= w.r1 || e >= c_hi) break;
            const int64_t seg_end = hi < c_hi ? hi : c_hi;
            const int first = static_cast<int>(e - c_lo), last = static_cast<int>(seg_end - c_lo);
            // sixteen entries per tile; whole tiles need no per-entry test, the last one does
            auto tile = [&](int t0, auto ragged) {
                constexpr bool kRagged = decltype(ragged)::value;
                const int i0 = t0 + g, i1 = i0 + 8; // this lane's two entries (fragment rows)
                const bool v0 = !kRagged || i0 < last, v1 = !kRagged || i1 < last;
                const int64_t eg0 = c_lo + i0;
                if (want_a) {
                    float acc[KS][4];
#pragma unroll
                    for (int nt = 0; nt < KS; nt++)
#pragma unroll
                        for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;
                    const float* b0 = Bs + i0 * L + t;
                    const float* b1 = b0 + 8 * L;
#pragma unroll
                    for (int ks = 0; ks < LS; ks++) {
                        const bool c0 = 8 * ks + t < L, c1 = 8 * ks + t + 4 < L;
                        unsigned bh[4], bl[4];
                        tf32_split((v0 && c0) ? b0[8 * ks] : 0.0f, bh[0], bl[0]);
                        tf32_split((v1 && c0) ? b1[8 * ks] : 0.0f, bh[1], bl[1]);
                        tf32_split((v0 && c1) ? b0[8 * ks + 4] : 0.0f, bh[2], bl[2]);
                        tf32_split((v1 && c1) ? b1[8 * ks + 4] : 0.0f, bh[3], bl[3]);
#pragma unroll
                        for (int nt = 0; nt < KS; nt++) {
                            mma_tf32(acc[nt], bl, ga_h[ks][nt]);
                            mma_tf32(acc[nt], bh, ga_l[ks][nt]);
                            mma_tf32(acc[nt], bh, ga_h[ks][nt]);
                        }
                    }
                    // acc[nt] = grad_A[entry g (+8)][k = 8 nt + 2 t (+1)]
                    float* dst = gA + eg0 * K + 2 * t;
#pragma unroll
                    for (int nt = 0; nt < KS; nt++) {
                        const int k = 8 * nt + 2 * t;
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (!(h ? v1 : v0) || k >= K) continue;
                            float* d2 = dst + h * 8 * K + 8 * nt;
                            if (pair_a) {
                                *reinterpret_cast<float2*>(d2) = make_float2(acc[nt][2 * h], acc[nt][2 * h + 1]);
                            } else {
                                d2[0] = acc[nt][2 * h];
                                if (k + 1 < K) d2[1] = acc[nt][2 * h + 1];
                            }
                        }
                    }
                }
                if (want_b) {
                    float acc[LS][4];
#pragma unroll
                    for (int nt = 0; nt < LS; nt++)
#pragma unroll
                        for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;
                    const float* a0 = As + i0 * K + t;
                    const float* a1 = a0 + 8 * K;
#pragma unroll
                    for (int ks = 0; ks < KS; ks++) {
                        const bool c0 = 8 * ks + t < K, c1 = 8 * ks + t + 4 < K;
                        unsigned ah[4], al[4];
                        tf32_split((v0 && c0) ? a0[8 * ks] : 0.0f, ah[0], al[0]);
                        tf32_split((v1 && c0) ? a1[8 * ks] : 0.0f, ah[1], al[1]);
                        tf32_split((v0 && c1) ? a0[8 * ks + 4] : 0.0f, ah[2], al[2]);
                        tf32_split((v1 && c1) ? a1[8 * ks + 4] : 0.0f, ah[3], al[3]);
#pragma unroll
                        for (int nt = 0; nt < LS; nt++) {
                            mma_tf32(acc[nt], al, gb_h[ks][nt]);
                            mma_tf32(acc[nt], ah, gb_l[ks][nt]);
                            mma_tf32(acc[nt], ah, gb_h[ks][nt]);
                        }
                    }
                    float* dst = gB + eg0 * L + 2 * t;
#pragma unroll
                    for (int nt = 0; nt < LS; nt++) {
                        const int l = 8 * nt + 2 * t;
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (!(h ? v1 : v0) || l >= L) continue;
                            float* d2 = dst + h * 8 * L + 8 * nt;
                            if (pair_b) {
                                *reinterpret_cast<float2*>(d2) = make_float2(acc[nt][2 * h], acc[nt][2 * h + 1]);
                            } else {
                                d2[0] = acc[nt][2 * h];
                                if (l + 1 < L) d2[1] = acc[nt][2 * h + 1];
                            }
                        }
                    }
                }
            };
            int t0 = first;
            for (; t0 + 16 <= last; t0 += 16) tile(t0, std::false_type{});
            if (t0 < last) tile(t0, std::true_type{});
            e = seg_end;
        }
        __syncwarp();
    }
    if (stalled) {
        if (lane == 0) report_stalled(st);
        return;
    }
    next_rows();
}
