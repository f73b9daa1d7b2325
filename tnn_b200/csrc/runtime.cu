// Host-side runtime of the kernel library: the per-device status word, the tensor-map cache, the launch counter and
// the small housekeeping entry points of the C ABI.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

#include "common.cuh"

namespace b200 {

__device__ unsigned int g_device_status = 0;

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

bool pdl_enabled() {
    static const bool on = []() {
        const char* e = std::getenv("TNN_B200_PDL");
        return !(e != nullptr && e[0] == '0');
    }();
    return on;
}

static constexpr int kMaxDevices = 64;
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

static EncodeTiledFn resolve_encode() {
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
static std::unordered_map<MapKey, CUtensorMap*, MapKeyHash> g_maps;

const CUtensorMap* get_tensor_map(const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                                  const uint32_t* box, int swizzle_bytes) {
    if (rank < 2 || rank > 3) return nullptr;
    if (swizzle_bytes != 128 && swizzle_bytes != 64) return nullptr;
    int dev = 0;
    cudaGetDevice(&dev);
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
    if (it != g_maps.end()) return it->second;

    EncodeTiledFn encode = resolve_encode();
    if (!encode) return nullptr;
    // cudaMallocHost is not needed: the map is copied into the kernel's parameter space at launch.
    CUtensorMap* map = new CUtensorMap;
    cuuint64_t gdims[3] = {1, 1, 1};
    cuuint64_t gstrides[2] = {0, 0};
    cuuint32_t gbox[3] = {1, 1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
    }
    for (int i = 0; i + 1 < rank; ++i) gstrides[i] = strides_bytes[i];
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                        gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        delete map;
        return nullptr;
    }
    if (g_maps.size() > 65536) {  // bound the cache: a caller that streams fresh pointers forever must not leak
        for (auto& kv : g_maps) delete kv.second;
        g_maps.clear();
    }
    g_maps.emplace(key, map);
    return map;
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
        return (v & ~8u) != 0 ? B200_ERR_DEVICE_TIMEOUT : B200_ERR_INDEX;   // bit 3: index out of range
    }
    return B200_OK;
}

uint64_t b200_launch_count(void) { return b200::g_launches.load(std::memory_order_relaxed); }

const char* b200_version(void) { return "tnn_b200 0.1 (sm_100a)"; }

}  // extern "C"
