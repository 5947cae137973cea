// Host-side execution context shared by the five operations: which stream a call runs on,
// whether it returns only when the results are complete, and the small status block through
// which kernels report what they found in the index arrays.
//
// Replaces the reference's CUDA_CHECK_ERROR, which prints and calls exit()
// (mops/src/internal/cuda_utils.cuh:11-24): here every CUDA failure becomes a
// std::runtime_error, which the C API turns into status 1 and a stored message.
#ifndef MOPS_B200_RUNTIME_HPP
#define MOPS_B200_RUNTIME_HPP

#include <cstdint>
#include <stdexcept>
#include <string>

#include <cuda_runtime.h>

#include "mops.hpp"

namespace mops_b200 {

// Words of the status block. Kernels write the device copy (read by later kernels of the
// same call) and the host-mapped copy (read by the host after the stream has drained).
// Every word holds the epoch (call number) of the last call that raised it; plain stores,
// no atomics, so the host-mapped copy needs nothing special from the interconnect.
enum StatusWord : int {
    kUnsortedEpoch = 0, // a scatter index was not in ascending order
    kBadIndex0 = 1,     // words 1..6: index array 0..5 of the op held an out-of-range value
    kMaxIndexArrays = 6,
    kStalled = 7,       // a kernel gave up waiting for one of its own asynchronous copies
    kStatusWords = 8
};

struct Status {
    uint32_t* dev;  // device memory
    uint32_t* host; // host-mapped pinned memory, same layout (device-visible address)
    uint32_t epoch; // identifies this call; never 0
};

struct Call {
    cudaStream_t stream;
    bool wait; // true: results complete when the entry point returns
    Status status;
    int device;
};

[[noreturn]] void throw_cuda(cudaError_t err, const char* what, const char* file, int line);

#define MOPS_CUDA_OK(expr)                                                                         \
    do {                                                                                           \
        cudaError_t mops_err__ = (expr);                                                           \
        if (mops_err__ != cudaSuccess)                                                             \
            ::mops_b200::throw_cuda(mops_err__, #expr, __FILE__, __LINE__);                        \
    } while (0)

// Starts a call on the calling thread's stream (default: the legacy default stream, like the
// reference) for the current device; allocates that thread's status block for this
// (device, stream) on first use.
Call begin_call();

// Which main kernels the calling thread's current call dispatched to, with their template
// arguments ("hpe_vjp_rows<f64,K=4,R=4>"), so that a measurement can be paired with the
// profile of the same instantiation. Cleared by begin_call.
void note_kernel(const std::string& name);
void note_kernel_f(const char* format, ...); // printf-style
const char* last_kernels();
template <typename T> inline const char* scalar_name() { return sizeof(T) == 8 ? "f64" : "f32"; }

// True when the call found its scatter index unsorted (host view; only meaningful after the
// stream has been synchronised).
bool host_saw_unsorted(const Call& call);

// Ends a call: checks the launch status, waits when `call.wait`, then turns index errors
// reported by the kernels into exceptions. `index_names` lists the op's index arrays in the
// bit order the kernels use.
void end_call(const Call& call, const char* operation, const char* const* index_names,
              int n_index_names);

// Waits for the stream of `call` (used between the main and the fallback kernels when the
// call is synchronous anyway).
void wait_stream(const Call& call);

// Per-thread settings (extensions to the reference API, which has no stream argument).
void set_stream(void* stream); // cudaStream_t; nullptr = legacy default stream
void* get_stream();
void set_wait(bool wait); // false: entry points return after enqueueing (used by the torch ops)
bool get_wait();

// Scratch memory for one call, ordered on the call's stream.
void* scratch_alloc(const Call& call, size_t bytes);
void scratch_free(const Call& call, void* ptr);

// ---- reusable device tables ("plans")
// Every operation first turns its index (and coefficient) arrays into a device table: the
// segment offsets of a scatter index, HPE's packed monomial records, SAP's sorted triplets,
// SASAW's grouped coupling table. Without a plan these tables are call-scoped scratch and are
// rebuilt by every call (as the reference rebuilds its first-occurrence table,
// mops/src/internal/cuda_first_occurences.cu:82-117). With a plan bound to the calling thread
// a table is built by the first call that needs it and kept: later calls with the same arrays
// (same addresses and sizes: the caller promises not to change their contents) reuse it, so the
// forward and the VJP of one graph share one segment table, nothing is rebuilt, and a scatter
// call knows without asking the device that its index is sorted.
enum TableKind : int {
    kSegmentTable = 1,
    kSasawCouplingTable = 2,
    kHpeTable = 3,
    kSapTable = 4,
    kSapSmallTable = 5
};

struct TableKey {
    int kind;
    int scalar_bytes;
    const void* ptr[5]; // the arrays the table is derived from
    int64_t n[10];      // their sizes and the layout parameters of the table
};

struct TableRef {
    void* ptr;          // device memory of `bytes` bytes
    bool fresh;         // the caller must fill it (launch the builder), then commit_table()
    bool owned_by_plan; // kept by the bound plan (else call-scoped scratch: release_table frees)
    bool sorted;        // segment tables from a plan: the index is known to be sorted
    int slot;           // position in the plan
};

class TablePlan;
TablePlan* plan_create();
void plan_destroy(TablePlan* plan);
void plan_bind(TablePlan* plan); // nullptr unbinds; per thread
TablePlan* plan_bound();
int plan_table_count(const TablePlan* plan);

// Unbinds the calling thread's plan for the lifetime of the object (for internal calls whose
// index arrays are temporaries).
struct PlanSuspended {
    TablePlan* saved;
    PlanSuspended() : saved(plan_bound()) { plan_bind(nullptr); }
    ~PlanSuspended() { plan_bind(saved); }
    PlanSuspended(const PlanSuspended&) = delete;
    PlanSuspended& operator=(const PlanSuspended&) = delete;
};

// Looks `key` up in the bound plan; without a plan (or when the plan knows that this index is
// not sorted or held bad values) returns call-scoped scratch that the caller fills as before.
TableRef acquire_table(const Call& call, const TableKey& key, size_t bytes);
// To be called once the builder of a fresh table is enqueued. For a plan-owned table this
// waits for the stream (once per table) and records whether the builder found the scatter
// index sorted; a table whose builder reported bad indices is not kept.
void commit_table(const Call& call, TableRef& ref);
void release_table(const Call& call, const TableRef& ref);

int sm_count(int device);
int max_optin_smem(int device);

} // namespace mops_b200

#endif
