#include "b200_cuda_device.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "b200_cuda_context.h"
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
// One slab = one cudaMalloc.  Free ranges are kept by offset so that neighbours merge in O(log n).
struct Slab {
    char* base;
    size_t size;
    size_t in_use;
    std::map<size_t, size_t> free_ranges;   // offset -> length
};

struct Live {
    int device;
    Slab* slab;
    size_t length;
};

struct Arena {
    std::mutex mu;
    std::vector<Slab*> slabs[kMaxGpus];
    std::unordered_map<void*, Live> live;
    B200ArenaStats stats[kMaxGpus];
    // pinned host blocks that were released and wait for the next request they fit
    std::vector<std::pair<void*, size_t>> pinned_free;
    std::unordered_map<void*, size_t> pinned_live;
    uint64_t pinned_allocations = 0;
    uint64_t pinned_bytes       = 0;
    Arena() {
        for (auto& s : stats) s = B200ArenaStats();
    }
};

Arena& TheArena() {
    static Arena* a = new Arena();   // never destroyed: blocks may be freed from static destructors of the host
    return *a;
}

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

void* TakeFrom(Slab* s, std::map<size_t, size_t>::iterator it, size_t bytes) {
    const size_t off = it->first, len = it->second;
    s->free_ranges.erase(it);
    if (len > bytes) s->free_ranges[off + bytes] = len - bytes;
    s->in_use += bytes;
    return s->base + off;
}

void GiveBack(Slab* s, size_t off, size_t len) {
    s->in_use -= len;
    auto next = s->free_ranges.lower_bound(off);
    if (next != s->free_ranges.end() && off + len == next->first) {
        len += next->second;
        next = s->free_ranges.erase(next);
    }
    if (next != s->free_ranges.begin()) {
        auto prev = std::prev(next);
        if (prev->first + prev->second == off) {
            prev->second += len;
            return;
        }
    }
    s->free_ranges[off] = len;
}

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
    const size_t rounded = RoundUp(bytes ? bytes : 1, kAlign);
    Arena& a = TheArena();
    std::lock_guard<std::mutex> lock(a.mu);
    B200ArenaStats& st = a.stats[dev];
    ++st.requests;

    Slab* best_slab = nullptr;
    std::map<size_t, size_t>::iterator best_it;
    if (ArenaEnabled()) {
        size_t best_len = ~static_cast<size_t>(0);
        for (Slab* s : a.slabs[dev]) {
            for (auto it = s->free_ranges.begin(); it != s->free_ranges.end(); ++it) {
                if (it->second >= rounded && it->second < best_len) {
                    best_len  = it->second;
                    best_slab = s;
                    best_it   = it;
                }
            }
        }
    }
    if (!best_slab) {
        const size_t slab_bytes = ArenaEnabled() ? (rounded > SlabBytes() / 2 ? rounded : SlabBytes()) : rounded;
        void* base = nullptr;
        if (cudaMalloc(&base, slab_bytes) != cudaSuccess || base == nullptr) {
            cudaGetLastError();
            return Status(TNNERR_OUTOFMEMORY, "cuda alloc failed");
        }
        ++st.driver_allocations;
        st.bytes_reserved += slab_bytes;
        Slab* s = new Slab();
        s->base   = static_cast<char*>(base);
        s->size   = slab_bytes;
        s->in_use = 0;
        s->free_ranges[0] = slab_bytes;
        a.slabs[dev].push_back(s);
        best_slab = s;
        best_it   = s->free_ranges.begin();
    }
    void* p = TakeFrom(best_slab, best_it, rounded);
    a.live[p] = Live{dev, best_slab, rounded};
    st.bytes_in_use += rounded;
    ++st.live_blocks;
    *handle = p;
    return TNN_OK;
}

Status B200CudaDevice::Free(void* handle) {
    if (!handle) return TNN_OK;
    Arena& a = TheArena();
    std::lock_guard<std::mutex> lock(a.mu);
    auto it = a.live.find(handle);
    if (it == a.live.end()) return Status(TNNERR_COMMON_ERROR, "cuda free: block does not belong to this device");
    const Live l = it->second;
    a.live.erase(it);
    B200ArenaStats& st = a.stats[l.device];
    st.bytes_in_use -= l.length;
    --st.live_blocks;
    GiveBack(l.slab, static_cast<size_t>(static_cast<char*>(handle) - l.slab->base), l.length);
    if (!ArenaEnabled() && l.slab->in_use == 0) {
        auto& v = a.slabs[l.device];
        for (size_t i = 0; i < v.size(); ++i) {
            if (v[i] == l.slab) {
                v.erase(v.begin() + i);
                break;
            }
        }
        cudaFree(l.slab->base);
        ++st.driver_frees;
        st.bytes_reserved -= l.slab->size;
        delete l.slab;
    }
    return TNN_OK;
}

uint64_t B200CudaDevice::ReleaseCachedMemory(int device_id) {
    Arena& a = TheArena();
    std::lock_guard<std::mutex> lock(a.mu);
    uint64_t released = 0;
    for (int dev = 0; dev < kMaxGpus; ++dev) {
        if (device_id >= 0 && dev != device_id) continue;
        auto& v = a.slabs[dev];
        for (size_t i = 0; i < v.size();) {
            if (v[i]->in_use == 0) {
                cudaFree(v[i]->base);   // the pointer identifies its GPU: no device switch needed
                ++a.stats[dev].driver_frees;
                a.stats[dev].bytes_reserved -= v[i]->size;
                released += v[i]->size;
                delete v[i];
                v.erase(v.begin() + i);
            } else {
                ++i;
            }
        }
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
