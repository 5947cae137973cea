#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <vector>
#include <map>
#include <mutex>
#include <unordered_map>
#include <utility>

#include "runtime.hpp"

namespace mops_b200 {

[[noreturn]] void throw_cuda(cudaError_t err, const char* what, const char* file, int line) {
    // Clear the (non-sticky) error so that the next call starts clean.
    (void)cudaGetLastError();
    throw std::runtime_error(
        std::string("CUDA error: ") + cudaGetErrorString(err) + " in `" + what + "` at " + file +
        ":" + std::to_string(line));
}

namespace {

struct ThreadState {
    cudaStream_t stream = nullptr;
    bool wait = true;
    uint32_t epoch = 0;
    // One status block per (device, stream) this thread has used: calls on one stream run in
    // order, so a call's words cannot be overwritten before its own kernels have read them,
    // and calls on different streams (which may overlap) never share a block. The blocks are
    // a few bytes and live until the process exits.
    std::map<std::pair<int, cudaStream_t>, Status> blocks;
    std::string kernels; // main kernels dispatched by the current / last call
};

thread_local ThreadState g_thread;

struct DeviceInfo {
    int sms = 0;
    int smem = 0;
};
std::mutex g_info_mutex;
std::unordered_map<int, DeviceInfo> g_info;

const DeviceInfo& device_info(int device) {
    std::lock_guard<std::mutex> lock(g_info_mutex);
    auto it = g_info.find(device);
    if (it == g_info.end()) {
        DeviceInfo info;
        MOPS_CUDA_OK(cudaDeviceGetAttribute(&info.sms, cudaDevAttrMultiProcessorCount, device));
        MOPS_CUDA_OK(
            cudaDeviceGetAttribute(&info.smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
        it = g_info.emplace(device, info).first;
    }
    return it->second;
}

} // namespace

int sm_count(int device) { return device_info(device).sms; }
int max_optin_smem(int device) { return device_info(device).smem; }

void set_stream(void* stream) { g_thread.stream = static_cast<cudaStream_t>(stream); }
void* get_stream() { return g_thread.stream; }
void set_wait(bool wait) { g_thread.wait = wait; }
bool get_wait() { return g_thread.wait; }

Call begin_call() {
    Call call;
    MOPS_CUDA_OK(cudaGetDevice(&call.device));
    call.stream = g_thread.stream;
    call.wait = g_thread.wait;

    g_thread.kernels.clear();
    const auto key = std::make_pair(call.device, call.stream);
    auto it = g_thread.blocks.find(key);
    if (it == g_thread.blocks.end()) {
        Status block{};
        void* host = nullptr;
        MOPS_CUDA_OK(cudaHostAlloc(&host, kStatusWords * sizeof(uint32_t),
                                   cudaHostAllocMapped | cudaHostAllocPortable));
        for (int i = 0; i < kStatusWords; i++) static_cast<volatile uint32_t*>(host)[i] = 0;
        void* host_dev = nullptr;
        MOPS_CUDA_OK(cudaHostGetDevicePointer(&host_dev, host, 0));
        (void)host_dev; // with unified addressing the host pointer is the device-visible one
        block.host = static_cast<uint32_t*>(host);
        MOPS_CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&block.dev),
                                kStatusWords * sizeof(uint32_t)));
        MOPS_CUDA_OK(cudaMemset(block.dev, 0, kStatusWords * sizeof(uint32_t)));
        it = g_thread.blocks.emplace(key, block).first;
    }
    call.status = it->second;
    g_thread.epoch += 1;
    if (g_thread.epoch == 0) g_thread.epoch = 1;
    call.status.epoch = g_thread.epoch;
    return call;
}

void note_kernel(const std::string& name) {
    if (!g_thread.kernels.empty()) g_thread.kernels += "; ";
    g_thread.kernels += name;
}
void note_kernel_f(const char* format, ...) {
    char text[160];
    va_list args;
    va_start(args, format);
    vsnprintf(text, sizeof(text), format, args);
    va_end(args);
    note_kernel(text);
}
const char* last_kernels() { return g_thread.kernels.c_str(); }

void wait_stream(const Call& call) { MOPS_CUDA_OK(cudaStreamSynchronize(call.stream)); }

bool host_saw_unsorted(const Call& call) {
    return static_cast<volatile uint32_t*>(call.status.host)[kUnsortedEpoch] == call.status.epoch;
}

void end_call(const Call& call, const char* operation, const char* const* index_names,
              int n_index_names) {
    MOPS_CUDA_OK(cudaGetLastError());
    if (!call.wait) return;
    MOPS_CUDA_OK(cudaStreamSynchronize(call.stream));
    volatile uint32_t* host = call.status.host;
    if (host[kStalled] == call.status.epoch)
        throw std::runtime_error(std::string("internal error in operation ") + operation +
                                 ": a kernel gave up waiting for an asynchronous copy; the "
                                 "results of this call are incomplete");
    std::string names;
    for (int i = 0; i < n_index_names && i < kMaxIndexArrays; i++) {
        if (host[kBadIndex0 + i] == call.status.epoch) {
            if (!names.empty()) names += ", ";
            names += index_names[i];
        }
    }
    if (!names.empty()) {
        throw std::runtime_error(
            "Index array " + names + " in operation " + operation +
            " contains negative or too large elements; this would cause out-of-bounds accesses");
    }
}

namespace {
// One stream-ordered pool per device that keeps freed blocks instead of returning them to the
// driver at the next synchronisation (the default pool's behaviour, which would make every
// call pay for mapping its scratch memory again).
std::mutex g_pool_mutex;
std::unordered_map<int, cudaMemPool_t> g_pools;

cudaMemPool_t scratch_pool(int device) {
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    auto it = g_pools.find(device);
    if (it == g_pools.end()) {
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = device;
        cudaMemPool_t pool = nullptr;
        MOPS_CUDA_OK(cudaMemPoolCreate(&pool, &props));
        uint64_t keep = UINT64_MAX;
        MOPS_CUDA_OK(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
        it = g_pools.emplace(device, pool).first;
    }
    return it->second;
}
} // namespace

// ---- plans
class TablePlan {
  public:
    struct Entry {
        TableKey key;
        int device;
        void* ptr;
        size_t bytes;
        bool ready;  // built and committed
        bool usable; // false: the index was unsorted or held bad values (rebuild per call)
    };
    std::mutex mutex;
    std::vector<Entry> entries;
};

namespace {
thread_local TablePlan* g_bound_plan = nullptr;
bool same_key(const TableKey& a, const TableKey& b) { return std::memcmp(&a, &b, sizeof(TableKey)) == 0; }
} // namespace

TablePlan* plan_create() { return new TablePlan(); }

void plan_destroy(TablePlan* plan) {
    if (plan == nullptr) return;
    if (g_bound_plan == plan) g_bound_plan = nullptr;
    for (auto& e : plan->entries) {
        if (e.ptr != nullptr) {
            int previous = 0;
            if (cudaGetDevice(&previous) == cudaSuccess && cudaSetDevice(e.device) == cudaSuccess) {
                (void)cudaFree(e.ptr);
                (void)cudaSetDevice(previous);
            }
        }
    }
    delete plan;
}

void plan_bind(TablePlan* plan) { g_bound_plan = plan; }
TablePlan* plan_bound() { return g_bound_plan; }

int plan_table_count(const TablePlan* plan) {
    if (plan == nullptr) return 0;
    std::lock_guard<std::mutex> lock(const_cast<TablePlan*>(plan)->mutex);
    int n = 0;
    for (const auto& e : plan->entries) n += e.ready && e.usable ? 1 : 0;
    return n;
}

TableRef acquire_table(const Call& call, const TableKey& key_in, size_t bytes) {
    TableRef ref{nullptr, true, false, false, -1};
    TablePlan* plan = g_bound_plan;
    if (plan != nullptr) {
        TableKey key;
        std::memset(&key, 0, sizeof(key)); // padding bytes take part in the comparison
        key.kind = key_in.kind;
        key.scalar_bytes = key_in.scalar_bytes;
        for (int i = 0; i < 5; i++) key.ptr[i] = key_in.ptr[i];
        for (int i = 0; i < 10; i++) key.n[i] = key_in.n[i];
        std::lock_guard<std::mutex> lock(plan->mutex);
        for (size_t i = 0; i < plan->entries.size(); i++) {
            TablePlan::Entry& e = plan->entries[i];
            if (e.device != call.device || !same_key(e.key, key)) continue;
            if (e.ready && e.usable) {
                ref.ptr = e.ptr;
                ref.fresh = false;
                ref.owned_by_plan = true;
                ref.sorted = true;
                ref.slot = static_cast<int>(i);
                return ref;
            }
            // known to be unusable (or being built by another thread): per-call scratch
            ref.ptr = scratch_alloc(call, bytes);
            return ref;
        }
        TablePlan::Entry e{};
        e.key = key;
        e.device = call.device;
        e.bytes = bytes;
        e.ready = false;
        e.usable = false;
        // plain cudaMalloc: the table outlives the call and is used from any stream
        MOPS_CUDA_OK(cudaMalloc(&e.ptr, bytes > 0 ? bytes : 1));
        plan->entries.push_back(e);
        ref.ptr = e.ptr;
        ref.owned_by_plan = true;
        ref.slot = static_cast<int>(plan->entries.size() - 1);
        return ref;
    }
    ref.ptr = scratch_alloc(call, bytes);
    return ref;
}

void commit_table(const Call& call, TableRef& ref) {
    if (!ref.owned_by_plan || !ref.fresh) return;
    TablePlan* plan = g_bound_plan;
    // The table must be complete before another stream may use it, and what its builder
    // reported decides whether it can be kept.
    MOPS_CUDA_OK(cudaStreamSynchronize(call.stream));
    volatile uint32_t* host = call.status.host;
    bool clean = true;
    for (int w = 0; w < kStatusWords; w++) clean = clean && host[w] != call.status.epoch;
    ref.sorted = clean;
    if (plan == nullptr) return;
    std::lock_guard<std::mutex> lock(plan->mutex);
    if (ref.slot >= 0 && ref.slot < static_cast<int>(plan->entries.size())) {
        plan->entries[ref.slot].ready = true;
        plan->entries[ref.slot].usable = clean;
    }
}

void release_table(const Call& call, const TableRef& ref) {
    if (!ref.owned_by_plan) scratch_free(call, ref.ptr);
}

void* scratch_alloc(const Call& call, size_t bytes) {
    void* ptr = nullptr;
    MOPS_CUDA_OK(cudaMallocFromPoolAsync(&ptr, bytes, scratch_pool(call.device), call.stream));
    return ptr;
}

void scratch_free(const Call& call, void* ptr) {
    if (ptr != nullptr) MOPS_CUDA_OK(cudaFreeAsync(ptr, call.stream));
}

} // namespace mops_b200
