// Host-side runtime of the kernel library: the per-device status word, the tensor-map cache, the launch counter and
// the small housekeeping entry points of the C ABI.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"

namespace b200 {

__device__ unsigned int g_device_status = 0;

// Self-test of the bounded-wait convention (b200_selftest_bounded_wait): one warp waits on an mbarrier that nobody ever
// arrives at, with a small poll limit, gives up, records it in the status word and returns normally.
__global__ void bounded_wait_selftest_kernel(unsigned int* status, uint32_t poll_limit) {
    __shared__ uint64_t bar;
    __shared__ uint32_t gave_up;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        gave_up = 0;
        mbar_fence_init();
    }
    __syncwarp();
    bool arrived = false;
    for (uint32_t i = 0; i < poll_limit && !arrived; ++i) arrived = mbar_try_wait(&bar, 0);
    if (!arrived) gave_up = 1u;
    __syncwarp();
    if (threadIdx.x == 0 && gave_up != 0 && status != nullptr) atomicOr(status, 1u);
}

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

bool pdl_enabled() {
    static const bool on = []() {
        const char* e = std::getenv("TNN_B200_PDL");
        return !(e != nullptr && e[0] == '0');
    }();
    return on;
}

static unsigned int* g_status_addr[kMaxDevices] = {nullptr};
static std::mutex g_status_mutex;

unsigned int* device_status_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    unsigned int* p = g_status_addr[dev];
    if (p) return p;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status_addr[dev]) {
        void* addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_device_status) != cudaSuccess) return nullptr;
        g_status_addr[dev] = static_cast<unsigned int*>(addr);
    }
    return g_status_addr[dev];
}

// ---------------------------------------------------------------- tensor-map cache
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Self-test hook (b200_selftest_tensor_map_cache): a stand-in encoder, so that the cache can be exercised on a machine
// without a driver.  Null in normal operation.
static std::atomic<EncodeTiledFn> g_encode_override{nullptr};

static EncodeTiledFn resolve_encode() {
    if (EncodeTiledFn o = g_encode_override.load(std::memory_order_acquire)) return o;
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        // The driver is reached through the runtime so that the library links against cudart only.
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
        if (q != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

struct MapKey {
    uint64_t v[12];
    bool operator==(const MapKey& o) const { return std::memcmp(v, o.v, sizeof(v)) == 0; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = 1469598103934665603ull;
        for (uint64_t x : k.v) {
            h ^= x;
            h *= 1099511628211ull;
        }
        return static_cast<size_t>(h);
    }
};
static std::mutex g_map_mutex;
static std::atomic<size_t> g_max_cached_maps{65536};
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

bool get_tensor_map(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box, int swizzle_bytes) {
    if (!out || rank < 2 || rank > 3) return false;
    if (swizzle_bytes != 128 && swizzle_bytes != 64) return false;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        dev = 0;
    }
    MapKey key;
    std::memset(&key, 0, sizeof(key));
    key.v[0] = reinterpret_cast<uint64_t>(base);
    key.v[1] = static_cast<uint64_t>(rank) | (static_cast<uint64_t>(dev) << 8) | (static_cast<uint64_t>(swizzle_bytes) << 16);
    for (int i = 0; i < rank; ++i) {
        key.v[2 + i] = dims[i];
        key.v[8 + i] = box[i];
    }
    for (int i = 0; i + 1 < rank; ++i) key.v[5 + i] = strides_bytes[i];

    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
        *out = it->second;
        return true;
    }
    if (!encode_tensor_map(out, base, rank, dims, strides_bytes, box, swizzle_bytes)) return false;
    // Bound the cache: a caller that streams fresh pointers forever must not leak.  Entries are values, and callers
    // hold copies, so dropping them all is safe whoever is launching at this moment.
    if (g_maps.size() >= g_max_cached_maps.load(std::memory_order_relaxed)) g_maps.clear();
    g_maps.emplace(key, *out);
    return true;
}

// Encodes a tensor map into caller-provided storage (no cache, no allocation).  Same conventions as get_tensor_map.
bool encode_tensor_map(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                       const uint32_t* box, int swizzle_bytes) {
    if (!out || rank < 2 || rank > 3 || (swizzle_bytes != 128 && swizzle_bytes != 64)) return false;
    EncodeTiledFn encode = resolve_encode();
    if (!encode) return false;
    cuuint64_t gdims[3] = {1, 1, 1};
    cuuint64_t gstrides[2] = {0, 0};
    cuuint32_t gbox[3] = {1, 1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
    }
    for (int i = 0; i + 1 < rank; ++i) gstrides[i] = strides_bytes[i];
    return encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims,
                  gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace b200

extern "C" {

const char* b200_status_string(int status) {
    switch (status) {
        case B200_OK: return "ok";
        case B200_ERR_PARAM: return "bad parameter (null pointer, dtype, alignment or leading dimension)";
        case B200_ERR_UNSUPPORTED: return "shape not supported by this kernel";
        case B200_ERR_LAUNCH: return "CUDA launch error";
        case B200_ERR_DRIVER: return "tensor-map encode failed (driver entry point missing or descriptor refused)";
        case B200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case B200_ERR_NOT_SM100: return "current device is not an sm_100 GPU";
        case B200_ERR_STATIC_LIMIT: return "size exceeds the fixed capacity of the library's static device scratch";
        case B200_ERR_INDEX: return "an embedding index was outside its table";
        default: return "unknown status";
    }
}

int b200_device_status(void) {
    unsigned int* p = b200::device_status_ptr();
    if (!p) return B200_ERR_LAUNCH;
    unsigned int v = 0;
    if (cudaMemcpy(&v, p, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return B200_ERR_LAUNCH;
    if (v != 0) {
        unsigned int zero = 0;
        cudaMemcpy(p, &zero, sizeof(zero), cudaMemcpyHostToDevice);
        return b200_decode_status_word(v);
    }
    return B200_OK;
}

int b200_selftest_bounded_wait(b200_stream_t stream) {
    unsigned int* p = b200::device_status_ptr();
    if (!p) return B200_ERR_LAUNCH;
    b200::bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p, 1024u);
    b200::count_launch();
    return b200::check_launch();
}

int b200_device_status_async(unsigned int* host_word, b200_stream_t stream) {
    if (!host_word) return B200_ERR_PARAM;
    unsigned int* p = b200::device_status_ptr();
    if (!p) return B200_ERR_LAUNCH;
    if (cudaMemcpyAsync(host_word, p, sizeof(unsigned int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)) !=
        cudaSuccess) {
        cudaGetLastError();
        return B200_ERR_LAUNCH;
    }
    return B200_OK;
}

int b200_decode_status_word(unsigned int word) {
    if (word == 0) return B200_OK;
    return (word & ~8u) != 0 ? B200_ERR_DEVICE_TIMEOUT : B200_ERR_INDEX;   // bit 3: index out of range
}

// Hammers the tensor-map cache from `threads` host threads with a stand-in encoder and a cache capacity of `capacity`
// entries, so that evictions happen all the time while other threads are reading.  Every returned map is compared
// with what the stand-in writes for its key.  Returns the number of wrong maps (0 = pass), negative on bad arguments.
// Needs no GPU and no driver.
int b200_selftest_tensor_map_cache(int threads, int maps_per_thread, int capacity) {
    using namespace b200;
    if (threads <= 0 || threads > 64 || maps_per_thread <= 0 || capacity <= 0) return B200_ERR_PARAM;
    struct Stub {
        static CUresult encode(CUtensorMap* map, CUtensorMapDataType, cuuint32_t rank, void* base, const cuuint64_t* dims,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) {
            uint64_t* w = reinterpret_cast<uint64_t*>(map);
            for (size_t i = 0; i < sizeof(CUtensorMap) / 8; ++i)
                w[i] = reinterpret_cast<uint64_t>(base) * 0x9E3779B97F4A7C15ull + dims[1] * 31 + i + rank;
            return CUDA_SUCCESS;
        }
    };
    const size_t old_cap = g_max_cached_maps.exchange(static_cast<size_t>(capacity));
    g_encode_override.store(&Stub::encode, std::memory_order_release);
    std::atomic<int> bad{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) {
        pool.emplace_back([&, t]() {
            for (int round = 0; round < 4; ++round) {
                for (int i = 0; i < maps_per_thread; ++i) {
                    // half of the keys are shared between threads (hits and evictions race), half are private
                    const uint64_t id = (i & 1) ? static_cast<uint64_t>(i) : (static_cast<uint64_t>(t) << 32) + i;
                    void* base = reinterpret_cast<void*>((id + 1) << 8);
                    const uint64_t dims[2] = {64, 128 + (id & 7)};
                    const uint64_t strides[1] = {128};
                    const uint32_t box[2] = {64, 128};
                    CUtensorMap got, want;
                    if (!get_tensor_map(&got, base, 2, dims, strides, box) ||
                        Stub::encode(&want, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base, dims, nullptr, nullptr, nullptr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
                        std::memcmp(&got, &want, sizeof(CUtensorMap)) != 0)
                        bad.fetch_add(1);
                }
            }
        });
    }
    for (auto& th : pool) th.join();
    g_encode_override.store(nullptr, std::memory_order_release);
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        g_maps.clear();   // the stand-in's entries must not outlive the test
    }
    g_max_cached_maps.store(old_cap);
    return bad.load();
}

uint64_t b200_launch_count(void) { return b200::g_launches.load(std::memory_order_relaxed); }

const char* b200_version(void) { return "tnn_b200 0.1 (sm_100a)"; }

}  // extern "C"
