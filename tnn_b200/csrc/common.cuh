// Shared host/device helpers of the tnn_b200 kernel library: dtype tags, packed conversions, the per-device status
// word that bounded waits report through, the launch counter and the tensor-map (TMA descriptor) cache.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>
#include <utility>

#include "../../include/tnn_b200.h"

namespace b200 {

// ---------------------------------------------------------------- device status word
// Bit 0: a bounded wait ran out in a GEMM CTA; bit 1: in an attention CTA; bit 2: misaligned dynamic shared memory
// (attention); bit 3: an embedding index outside its table.  The word itself is a __device__ variable
// of runtime.cu; kernels receive its address as a parameter (no relocatable device code needed).
unsigned int* device_status_ptr();  // address of the word on the current device (looked up once per device)

void count_launch(int n = 1);

// ---------------------------------------------------------------- dtype helpers (device)
template <int DT> struct Elem;
template <> struct Elem<B200_F16> { using type = __half; using type2 = __half2; };
template <> struct Elem<B200_BF16> { using type = __nv_bfloat16; using type2 = __nv_bfloat162; };

__device__ __forceinline__ uint32_t pack2(float a, float b, int dtype) {
    if (dtype == B200_F16) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
}
// Compile-time variant: with the dtype as a run-time value the compiler emits both conversions and a select.
template <int DT>
__device__ __forceinline__ uint32_t pack2t(float a, float b) {
    if (DT == B200_F16) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
}
__device__ __forceinline__ float2 unpack2(uint32_t u, int dtype) {
    if (dtype == B200_F16) {
        return __half22float2(*reinterpret_cast<__half2*>(&u));
    } else {
        return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
    }
}

inline size_t dtype_size(int dt) { return dt == B200_F32 ? 4 : 2; }
inline bool is_half_dtype(int dt) { return dt == B200_F16 || dt == B200_BF16; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------- tensor maps
// 2-D or 3-D tiled map over a 2-byte-element tensor whose innermost dimension is contiguous, 128- or 64-byte
// swizzle, inner box = 64 or 32 elements.  dims/strides are innermost first; strides[i] is the byte stride of dim i+1.
// Maps are cached per device by their full key; encoding takes about a microsecond and the same activations and
// weights come back every Forward.  The 128-byte map is copied into `*out` under the cache's lock, so that no caller
// ever holds a pointer into the cache (another thread may evict entries at any time).  Returns false if the driver
// entry point is missing or refuses the descriptor.
// swizzle_bytes: 128 (box inner extent 64 elements) or 64 (inner extent 32 elements).
bool get_tensor_map(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box, int swizzle_bytes = 128);

// The same encoding into caller-provided storage: no cache entry, no allocation of any kind.
bool encode_tensor_map(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                       const uint32_t* box, int swizzle_bytes = 128);

// One-time set-up per device (kernel attributes, symbol addresses, occupancy queries) that several host threads — one
// per GPU, or several instances on one GPU — may reach at the same moment: double-checked under a mutex.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
    std::atomic<bool> done[kMaxDevices];
    std::mutex mu;
    PerDeviceOnce() {
        for (auto& d : done) d.store(false, std::memory_order_relaxed);
    }
    // Runs `fn` (returning bool: success) once for `dev`; false if it failed (it is retried on the next call).
    template <typename F>
    bool ensure(int dev, F&& fn) {
        if (dev < 0 || dev >= kMaxDevices) return false;
        if (done[dev].load(std::memory_order_acquire)) return true;
        std::lock_guard<std::mutex> lock(mu);
        if (done[dev].load(std::memory_order_relaxed)) return true;
        if (!fn()) return false;
        done[dev].store(true, std::memory_order_release);
        return true;
    }
};

inline int check_launch() { return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH; }

// ---------------------------------------------------------------- launches
// Every kernel of the library is launched with programmatic stream serialization allowed: its CTAs may be placed while
// the previous kernel of the stream drains, run their set-up, and block in griddepcontrol.wait until that kernel has
// completed (each kernel calls it before its first access to global memory other than constants).  This hides launch
// latency and prologues between the seven short kernels of an encoder layer.  TNN_B200_PDL=0 in the environment
// turns the attribute off (plain stream order), for comparison.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace b200
