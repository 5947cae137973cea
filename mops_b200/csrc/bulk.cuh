// Asynchronous bulk copies global -> shared memory (the copy engine of sm_90+/sm_100:
// `cp.async.bulk`, one instruction from one thread moves a whole contiguous slice, completion is
// counted in bytes on an mbarrier in shared memory) and the mbarrier operations that go with
// them. Used to stream the contiguous A / B slices of a run of entries, gathered W rows and
// grad_output rows into per-warp rings, so that the data in flight lives in shared memory
// instead of registers and costs no issue slots.
//
// Rules kept here: source and destination 16-byte aligned, size a multiple of 16 bytes; only
// this GPU's own global memory is ever a source; no cluster multicast; every wait is bounded
// (a kernel that gives up reports it through the status block and returns).
#ifndef MOPS_B200_BULK_CUH
#define MOPS_B200_BULK_CUH

#include <cstdint>

#include "device.cuh"

namespace mops_b200 {

__device__ __forceinline__ unsigned smem_address(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbarrier_init(uint64_t* bar, unsigned arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_address(bar)), "r"(arrivals)
                 : "memory");
}

// Makes freshly initialised barriers visible to the copy engine.
__device__ __forceinline__ void mbarrier_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}

// One arrival that also announces `bytes` of asynchronous copies for the current phase.
__device__ __forceinline__ void mbarrier_arrive_expect(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_address(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbarrier_try_wait(uint64_t* bar, unsigned parity) {
    unsigned done;
    asm volatile("{\n .reg .pred p;\n"
                 " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                 " selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done)
                 : "r"(smem_address(bar)), "r"(parity)
                 : "memory");
    return done != 0;
}

// Waits for the phase with the given parity, for about a second at most. Returns false when it
// gave up (the copies it waits for never arrived); the caller then reports and leaves.
__device__ __forceinline__ bool mbarrier_wait(uint64_t* bar, unsigned parity) {
    if (mbarrier_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!mbarrier_try_wait(bar, parity)) {
        if (clock64() - start > 2000000000LL) return false;
    }
    return true;
}

// Copies `bytes` (a multiple of 16) from global to this block's shared memory; completion is
// counted on `bar`. Both addresses 16-byte aligned.
__device__ __forceinline__ void bulk_copy_in(void* smem_dst, const void* global_src, unsigned bytes,
                                             uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
            "r"(smem_address(smem_dst)),
        "l"(global_src), "r"(bytes), "r"(smem_address(bar))
        : "memory");
}

// 16-byte asynchronous copy global -> shared by the calling lane (LDGSTS, around L1), for rows
// that are gathered one by one: the copy engine's bulk copies are slow for pieces of a few
// hundred bytes, sixteen lanes moving one 256-byte row are not.
__device__ __forceinline__ void lane_copy16(void* smem_dst, const void* global_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_address(smem_dst)),
                 "l"(global_src)
                 : "memory");
}

// The calling lane arrives on `bar` once all the lane copies it has issued so far are complete.
// The barrier's arrival count must include this arrival (it does not raise the pending count).
__device__ __forceinline__ void lane_copies_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(smem_address(bar))
                 : "memory");
}

// A kernel stopped waiting for its own copies (never expected; reported as an internal error).
__device__ __forceinline__ void report_stalled(const Status& st) {
    st.dev[kStalled] = st.epoch;
    st.host[kStalled] = st.epoch;
    __threadfence_system();
}

} // namespace mops_b200

#endif
