// The plug-in's own C entry points that are not the graph-pass tools (those sit beside the pass): allocator counters
// and hooks, graph-replay counters, page-locked memory for Mats.  Declared in include/tnn_b200_plugin.h.
#include <cstring>
#include <string>

#include "b200_cuda_context.h"
#include "b200_cuda_device.h"
#include "tnn_b200_plugin.h"

using namespace TNN_NS;

extern "C" {

void tnnb200_arena_stats(int device_id, uint64_t out[8]) {
    const B200ArenaStats s = B200CudaDevice::Stats(device_id);
    out[0] = s.driver_allocations;
    out[1] = s.driver_frees;
    out[2] = s.bytes_reserved;
    out[3] = s.bytes_in_use;
    out[4] = s.live_blocks;
    out[5] = s.requests;
    out[6] = s.pinned_allocations;
    out[7] = s.pinned_bytes_reserved;
}

uint64_t tnnb200_release_cached_memory(int device_id) { return B200CudaDevice::ReleaseCachedMemory(device_id); }

void tnnb200_inject_allocation_failure(int skip, int count) { B200CudaDevice::InjectAllocationFailure(skip, count); }

int tnnb200_selftest_range_arena(unsigned seed, int steps, int pooled, char* err, int err_cap) {
    std::string why;
    const int rc = B200CudaDevice::SelfTestRangeArena(seed, steps, pooled, &why);
    if (err && err_cap > 0) {
        std::strncpy(err, why.c_str(), static_cast<size_t>(err_cap) - 1);
        err[err_cap - 1] = 0;
    }
    return rc;
}

int tnnb200_graph_counters(void* command_queue, uint64_t out[4]) {
    B200CudaContext* ctx = B200CudaContext::FromCommandQueue(command_queue);
    if (!ctx) return -1;
    ctx->GraphCounters(out);
    return 0;
}

void* tnnb200_host_alloc(size_t bytes) {
    void* p = nullptr;
    return B200CudaDevice::AllocateHost(&p, bytes) == TNN_OK ? p : nullptr;
}

void tnnb200_host_free(void* ptr) { B200CudaDevice::FreeHost(ptr); }

}  // extern "C"
