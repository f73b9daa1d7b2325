#include "b200_cuda_device.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "b200_cuda_context.h"
#include "b200_range_arena.h"
#include "tnn/utils/blob_memory_size_utils.h"
#include "tnn/utils/data_type_utils.h"
#include "tnn/utils/dims_utils.h"

namespace TNN_NS {

namespace {

std::atomic<int> g_fail_skip{0};    // allocations still to let through before the injected failures
std::atomic<int> g_fail_count{0};   // injected failures still to deliver

constexpr int kMaxGpus = 64;
constexpr size_t kAlign = 256;
inline size_t RoundUp(size_t n, size_t a) { return (n + a - 1) / a * a; }

// ---------------------------------------------------------------------------------------------------- device arena
// One RangeArena per GPU (the sub-allocation logic, b200_range_arena.h) over cudaMalloc'ed slabs, plus a cache of pinned
// host blocks.
size_t SlabBytes() {
    static const size_t v = []() -> size_t {
        const char* e = std::getenv("TNN_B200_ARENA_SLAB_MB");
        long mb       = e ? std::atol(e) : 64;
        if (mb < 1) mb = 1;
        return static_cast<size_t>(mb) << 20;
    }();
    return v;
}

// TNN_B200_ARENA=0: every block is its own cudaMalloc (the reference's behaviour), for comparison and debugging.
bool ArenaEnabled() {
    static const bool on = []() {
        const char* e = std::getenv("TNN_B200_ARENA");
        return !(e != nullptr && e[0] == '0');
    }();
    return on;
}

struct Arena {
    std::mutex mu;
    tnn_b200::RangeArena* ranges[kMaxGpus];
    B200ArenaStats stats[kMaxGpus];
    // pinned host blocks that were released and wait for the next request they fit
    std::vector<std::pair<void*, size_t>> pinned_free;
    std::unordered_map<void*, size_t> pinned_live;
    uint64_t pinned_allocations = 0;
    uint64_t pinned_bytes       = 0;
    Arena() {
        for (auto& s : stats) s = B200ArenaStats();
        for (auto& r : ranges) r = nullptr;
    }
    tnn_b200::RangeArena& Ranges(int dev) {
        if (!ranges[dev]) ranges[dev] = new tnn_b200::RangeArena(SlabBytes(), kAlign, ArenaEnabled());
        return *ranges[dev];
    }
};

Arena& TheArena() {
    static Arena* a = new Arena();   // never destroyed: blocks may be freed from static destructors of the host
    return *a;
}

void* CudaSlabAlloc(size_t bytes) {
    void* base = nullptr;
    if (cudaMalloc(&base, bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return base;
}

void CudaSlabFree(void* base) { cudaFree(base); }   // the pointer identifies its GPU: no device switch needed

}  // namespace

B200CudaDevice::B200CudaDevice(DeviceType device_type) : AbstractDevice(device_type) {}
B200CudaDevice::~B200CudaDevice() {}

void B200CudaDevice::InjectAllocationFailure(int skip, int count) {
    g_fail_skip.store(skip > 0 ? skip : 0);
    g_fail_count.store(count > 0 ? count : 0);
}

BlobMemorySizeInfo B200CudaDevice::Calculate(BlobDesc& desc) {
    BlobMemorySizeInfo info = Calculate1DMemorySize(desc);
    if (DimsVectorUtils::Count(info.dims) == 0) info.dims[0] = 1;
    return info;
}

static size_t BytesOf(const BlobMemorySizeInfo& info) {
    size_t count = 1;
    for (int d : info.dims) count *= static_cast<size_t>(d > 0 ? d : 1);
    return count * static_cast<size_t>(DataTypeUtils::GetBytesSize(info.data_type));
}

Status B200CudaDevice::Allocate(void** handle, MatType mat_type, DimsVector dims) {
    BlobDesc desc;
    desc.dims        = dims;
    desc.device_type = DEVICE_CUDA;
    desc.data_format = DATA_FORMAT_NCHW;
    desc.data_type   = mat_type == NCHW_FLOAT ? DATA_TYPE_FLOAT
                       : mat_type == NC_INT32 ? DATA_TYPE_INT32
                       : (mat_type == RESERVED_FP16_TEST || mat_type == RESERVED_BFP16_TEST) ? DATA_TYPE_HALF
                                                                                             : DATA_TYPE_INT8;
    auto info = Calculate(desc);
    return Allocate(handle, info);
}

Status B200CudaDevice::Allocate(void** handle, BlobMemorySizeInfo& size_info) { return Allocate(handle, BytesOf(size_info)); }

Status B200CudaDevice::Allocate(void** handle, size_t bytes) {
    if (!handle) return Status(TNNERR_NULL_PARAM, "null handle");
    if (g_fail_count.load() > 0) {
        if (g_fail_skip.load() > 0) {
            g_fail_skip.fetch_sub(1);
        } else {
            g_fail_count.fetch_sub(1);
            return Status(TNNERR_OUTOFMEMORY, "cuda alloc failed (injected)");
        }
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxGpus) {
        cudaGetLastError();
        return Status(TNNERR_DEVICE_NOT_SUPPORT, "no current CUDA device");
    }
    // 256-byte granularity: more than the TMA descriptors need (16), and vector loads of a trailing partial group
    // stay inside the block.
    Arena& a = TheArena();
    std::lock_guard<std::mutex> lock(a.mu);
    B200ArenaStats& st = a.stats[dev];
    ++st.requests;
    const tnn_b200::RangeArena::TakeResult r = a.Ranges(dev).Take(bytes, CudaSlabAlloc);
    if (!r.ptr) return Status(TNNERR_OUTOFMEMORY, "cuda alloc failed");
    if (r.new_slab) {
        ++st.driver_allocations;
        st.bytes_reserved += r.new_slab;
    }
    st.bytes_in_use += r.length;
    ++st.live_blocks;
    *handle = r.ptr;
    return TNN_OK;
}

Status B200CudaDevice::Free(void* handle) {
    if (!handle) return TNN_OK;
    Arena& a = TheArena();
    std::lock_guard<std::mutex> lock(a.mu);
    for (int dev = 0; dev < kMaxGpus; ++dev) {
        if (!a.ranges[dev] || !a.ranges[dev]->Owns(handle)) continue;
        const tnn_b200::RangeArena::GiveResult r = a.ranges[dev]->Give(handle, CudaSlabFree);
        B200ArenaStats& st = a.stats[dev];
        st.bytes_in_use -= r.length;
        --st.live_blocks;
        if (r.freed_slab) {
            ++st.driver_frees;
            st.bytes_reserved -= r.freed_slab;
        }
        return TNN_OK;
    }
    return Status(TNNERR_COMMON_ERROR, "cuda free: block does not belong to this device");
}

uint64_t B200CudaDevice::ReleaseCachedMemory(int device_id) {
    Arena& a = TheArena();
    std::lock_guard<std::mutex> lock(a.mu);
    uint64_t released = 0;
    for (int dev = 0; dev < kMaxGpus; ++dev) {
        if ((device_id >= 0 && dev != device_id) || !a.ranges[dev]) continue;
        size_t slabs      = 0;
        const size_t freed = a.ranges[dev]->ReleaseEmpty(CudaSlabFree, &slabs);
        a.stats[dev].driver_frees += slabs;
        a.stats[dev].bytes_reserved -= freed;
        released += freed;
    }
    for (auto& b : a.pinned_free) {
        cudaFreeHost(b.first);
        a.pinned_bytes -= b.second;
        released += b.second;
    }
    a.pinned_free.clear();
    cudaGetLastError();
    return released;
}

// Host-only exercise of the sub-allocation logic: a seeded random sequence of requests and releases against a fake
// backing store (address ranges that are never touched), with the structural invariants checked after every step.
// Returns 0, or the number of the step at which an invariant broke (message in `why`).
int B200CudaDevice::SelfTestRangeArena(unsigned seed, int steps, int pooled, std::string* why) {
    struct Backing {
        uintptr_t next = 1u << 20;
        std::map<uintptr_t, size_t> slabs;
        size_t allocated = 0, freed = 0;
    } backing;
    auto alloc = [&](size_t bytes) -> void* {
        const uintptr_t base = backing.next;
        backing.next += (bytes + 4095) / 4096 * 4096 + 4096;   // a hole between slabs: blocks must not merge across them
        backing.slabs[base] = bytes;
        ++backing.allocated;
        return reinterpret_cast<void*>(base);
    };
    auto release = [&](void* p) {
        backing.slabs.erase(reinterpret_cast<uintptr_t>(p));
        ++backing.freed;
    };
    const size_t slab = 1u << 20, align = 256;
    tnn_b200::RangeArena arena(slab, align, pooled != 0);
    std::vector<std::pair<void*, size_t>> held;
    uint64_t state = seed * 2654435761u + 12345u;
    auto rnd = [&]() -> uint32_t {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        return static_cast<uint32_t>(state >> 33);
    };
    auto fail = [&](int step, const std::string& msg) {
        if (why) *why = msg;
        return step;
    };
    for (int step = 1; step <= steps; ++step) {
        const bool take = held.empty() || (rnd() % 100) < (held.size() < 200 ? 60u : 35u);
        if (take) {
            const uint32_t kind = rnd() % 10;
            const size_t bytes = kind == 0 ? 0 : kind < 6 ? 1 + rnd() % 5000 : kind < 9 ? 1 + rnd() % 300000
                                                                                          : slab / 2 + rnd() % (2 * slab);
            const auto r = arena.Take(bytes, alloc);
            if (!r.ptr) return fail(step, "Take failed although the backing store never refuses");
            if (r.length < bytes || r.length % align || r.length >= bytes + align + (bytes ? 0 : 1))
                return fail(step, "wrong rounded length");
            // the block lies inside one slab of the backing store
            const uintptr_t p = reinterpret_cast<uintptr_t>(r.ptr);
            auto it = backing.slabs.upper_bound(p);
            if (it == backing.slabs.begin()) return fail(step, "block below every slab");
            --it;
            if (p + r.length > it->first + it->second) return fail(step, "block reaches past its slab");
            for (const auto& h : held) {
                const uintptr_t q = reinterpret_cast<uintptr_t>(h.first);
                if (p < q + h.second && q < p + r.length) return fail(step, "two live blocks overlap");
            }
            held.push_back(std::make_pair(r.ptr, r.length));
        } else {
            const size_t i = rnd() % held.size();
            const auto r = arena.Give(held[i].first, release);
            if (!r.found || r.length != held[i].second) return fail(step, "Give did not recognise a live block");
            if (arena.Give(held[i].first, release).found) return fail(step, "a block could be given back twice");
            held.erase(held.begin() + i);
        }
        const std::string bad = arena.CheckInvariants();
        if (!bad.empty()) return fail(step, bad);
        if (arena.live_blocks() != held.size()) return fail(step, "live block count");
        size_t bytes_held = 0;
        for (const auto& h : held) bytes_held += h.second;
        if (arena.bytes_in_use() != bytes_held) return fail(step, "bytes in use");
        if (!pooled && arena.slab_count() != held.size()) return fail(step, "unpooled: one slab per block");
    }
    for (const auto& h : held)
        if (!arena.Give(h.first, release).found) return fail(steps + 1, "final release");
    const std::string bad = arena.CheckInvariants();
    if (!bad.empty()) return fail(steps + 1, bad);
    if (arena.bytes_in_use() != 0 || arena.live_blocks() != 0) return fail(steps + 1, "not empty after releasing all");
    const size_t reserved = arena.bytes_reserved();
    if (arena.ReleaseEmpty(release) != reserved || arena.slab_count() != 0 || !backing.slabs.empty() ||
        backing.allocated != backing.freed)
        return fail(steps + 2, "slabs left behind after ReleaseEmpty");
    return 0;
}

B200ArenaStats B200CudaDevice::Stats(int device_id) {
    Arena& a = TheArena();
    std::lock_guard<std::mutex> lock(a.mu);
    B200ArenaStats s = (device_id >= 0 && device_id < kMaxGpus) ? a.stats[device_id] : B200ArenaStats();
    s.pinned_allocations    = a.pinned_allocations;
    s.pinned_bytes_reserved = a.pinned_bytes;
    return s;
}

Status B200CudaDevice::AllocateHost(void** ptr, size_t bytes) {
    if (!ptr) return Status(TNNERR_NULL_PARAM, "null pointer");
    const size_t rounded = RoundUp(bytes ? bytes : 1, 4096);
    Arena& a = TheArena();
    std::lock_guard<std::mutex> lock(a.mu);
    size_t best = a.pinned_free.size();
    for (size_t i = 0; i < a.pinned_free.size(); ++i) {
        const size_t len = a.pinned_free[i].second;
        if (len >= rounded && len <= 2 * rounded && (best == a.pinned_free.size() || len < a.pinned_free[best].second))
            best = i;
    }
    if (best != a.pinned_free.size()) {
        *ptr = a.pinned_free[best].first;
        a.pinned_live[*ptr] = a.pinned_free[best].second;
        a.pinned_free.erase(a.pinned_free.begin() + best);
        return TNN_OK;
    }
    void* p = nullptr;
    // portable: the same staging serves whichever GPU the instance runs on
    if (cudaHostAlloc(&p, rounded, cudaHostAllocPortable) != cudaSuccess || p == nullptr) {
        cudaGetLastError();
        return Status(TNNERR_OUTOFMEMORY, "pinned host alloc failed");
    }
    ++a.pinned_allocations;
    a.pinned_bytes += rounded;
    a.pinned_live[p] = rounded;
    *ptr = p;
    return TNN_OK;
}

void B200CudaDevice::FreeHost(void* ptr) {
    if (!ptr) return;
    Arena& a = TheArena();
    std::lock_guard<std::mutex> lock(a.mu);
    auto it = a.pinned_live.find(ptr);
    if (it == a.pinned_live.end()) return;
    a.pinned_free.push_back(std::make_pair(ptr, it->second));
    a.pinned_live.erase(it);
}

Status B200CudaDevice::CopyToDevice(BlobHandle* dst, const BlobHandle* src, BlobDesc& desc, void* command_queue) {
    cudaStream_t stream = static_cast<cudaStream_t>(command_queue);
    const size_t bytes = BytesOf(Calculate(desc));
    if (cudaMemcpyAsync(static_cast<char*>(dst->base) + dst->bytes_offset,
                        static_cast<const char*>(src->base) + src->bytes_offset, bytes, cudaMemcpyHostToDevice,
                        stream) != cudaSuccess)
        return Status(TNNERR_CUDA_MEMCPY_ERROR, "H2D copy failed");
    if (cudaStreamSynchronize(stream) != cudaSuccess) return Status(TNNERR_CUDA_SYNC_ERROR, "stream sync failed");
    return TNN_OK;
}

Status B200CudaDevice::CopyFromDevice(BlobHandle* dst, const BlobHandle* src, BlobDesc& desc, void* command_queue) {
    cudaStream_t stream = static_cast<cudaStream_t>(command_queue);
    const size_t bytes = BytesOf(Calculate(desc));
    if (cudaMemcpyAsync(static_cast<char*>(dst->base) + dst->bytes_offset,
                        static_cast<const char*>(src->base) + src->bytes_offset, bytes, cudaMemcpyDeviceToHost,
                        stream) != cudaSuccess)
        return Status(TNNERR_CUDA_MEMCPY_ERROR, "D2H copy failed");
    if (cudaStreamSynchronize(stream) != cudaSuccess) return Status(TNNERR_CUDA_SYNC_ERROR, "stream sync failed");
    return TNN_OK;
}

AbstractLayerAcc* B200CudaDevice::CreateLayerAcc(LayerType type) {
    auto& m = GetLayerCreatorMap();
    auto it = m.find(type);
    // No acc registered => nullptr => BaseLayer::Init fails with "layer acc is nil": there is no CPU fallback.
    return it == m.end() ? nullptr : it->second->CreateLayerAcc(type);
}

Context* B200CudaDevice::CreateContext(int device_id) {
    auto* ctx = new B200CudaContext();
    if (ctx->Setup(device_id) != TNN_OK) {
        delete ctx;
        return nullptr;
    }
    return ctx;
}

NetworkType B200CudaDevice::ConvertAutoNetworkType() { return NETWORK_TYPE_DEFAULT; }

Status B200CudaDevice::RegisterLayerAccCreator(LayerType type, LayerAccCreator* creator) {
    GetLayerCreatorMap()[type] = std::shared_ptr<LayerAccCreator>(creator);
    return TNN_OK;
}

bool B200CudaDevice::HasLayerAcc(LayerType type) { return GetLayerCreatorMap().count(type) > 0; }

std::map<LayerType, std::shared_ptr<LayerAccCreator>>& B200CudaDevice::GetLayerCreatorMap() {
    static std::map<LayerType, std::shared_ptr<LayerAccCreator>> m;
    return m;
}

TypeDeviceRegister<B200CudaDevice> g_b200_cuda_device_register(DEVICE_CUDA);

}  // namespace TNN_NS
