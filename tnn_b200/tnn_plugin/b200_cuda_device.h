// DEVICE_CUDA for TNN's DefaultNetwork, B200 build.  Replaces the reference's CudaDevice
// (source/tnn/device/cuda/cuda_device.{h,cc}), which routes DEVICE_CUDA to TensorRT
// (ConvertAutoNetworkType() == NETWORK_TYPE_TENSORRT, cuda_device.cc:159-161), allocates with `int` byte counts
// and one cudaMalloc per blob (cuda_device.cc:53-64, called once per pooled blob by
// source/tnn/memory_manager/blob_memory_pool.cc:47-121) and aborts on CUDA errors.  This one serves
// NETWORK_TYPE_DEFAULT, uses 64-bit sizes, returns Status codes, and sub-allocates every block — blobs, packed weights,
// acc buffers, converter staging — from an arena of large slabs per GPU:
//
//   * a request is rounded to 256 bytes and served best-fit from the free ranges of the GPU's slabs; only when none
//     fits is a new slab taken from the driver (64 MiB, or the request itself when that is larger);
//   * freed ranges merge with their neighbours and stay in the arena, so an instance that is destroyed and created
//     again, or reshaped, takes no memory from the driver at all, and nothing is ever allocated while a Forward runs;
//   * ReleaseCachedMemory() returns slabs that are entirely free to the driver.
//
// TNN's device interface hands over one blob at a time without saying which instance asks, so the arena belongs to the
// GPU, not to an instance; instances on one GPU share it (under a mutex: allocation happens at Init / Reshape only).
#ifndef TNN_B200_CUDA_DEVICE_H_
#define TNN_B200_CUDA_DEVICE_H_

#include <cstdint>
#include <map>
#include <string>
#include <memory>

#include "tnn/core/abstract_device.h"

namespace TNN_NS {

// Counters of one GPU's arena (all monotonic except bytes_in_use / bytes_reserved / live_blocks).
struct B200ArenaStats {
    uint64_t driver_allocations;   // cudaMalloc calls made so far
    uint64_t driver_frees;         // cudaFree calls made so far
    uint64_t bytes_reserved;       // held from the driver now
    uint64_t bytes_in_use;         // handed out now
    uint64_t live_blocks;          // blocks handed out now
    uint64_t requests;             // Allocate calls served so far
    uint64_t pinned_allocations;   // cudaHostAlloc calls made so far (host staging of the blob converters)
    uint64_t pinned_bytes_reserved;
};

class B200CudaDevice : public AbstractDevice {
public:
    explicit B200CudaDevice(DeviceType device_type);
    ~B200CudaDevice();

    virtual BlobMemorySizeInfo Calculate(BlobDesc& desc);
    virtual Status Allocate(void** handle, MatType mat_type, DimsVector dims);
    virtual Status Allocate(void** handle, BlobMemorySizeInfo& size_info);
    // `bytes` of device memory of the CURRENT device, 256-byte aligned, from that GPU's arena.
    Status Allocate(void** handle, size_t bytes);
    virtual Status Free(void* handle);
    virtual Status CopyToDevice(BlobHandle* dst, const BlobHandle* src, BlobDesc& desc, void* command_queue);
    virtual Status CopyFromDevice(BlobHandle* dst, const BlobHandle* src, BlobDesc& desc, void* command_queue);
    virtual AbstractLayerAcc* CreateLayerAcc(LayerType type);
    virtual Context* CreateContext(int device_id);
    virtual NetworkType ConvertAutoNetworkType();

    static Status RegisterLayerAccCreator(LayerType type, LayerAccCreator* creator);
    static bool HasLayerAcc(LayerType type);

    // Page-locked host memory for the blob converters' staging (cached like device memory: a released block is kept
    // and handed to the next request it fits).
    static Status AllocateHost(void** ptr, size_t bytes);
    static void FreeHost(void* ptr);

    static B200ArenaStats Stats(int device_id);
    // Returns every slab of `device_id` (-1: all GPUs) that holds no live block, and every cached pinned block, to the
    // driver.  Returns the number of bytes released.
    static uint64_t ReleaseCachedMemory(int device_id);

    // Test hook: after `skip` more successful device allocations, the next `count` fail with TNNERR_OUTOFMEMORY
    // (host-side fault injection; no GPU fault is provoked).  count = 0 switches it off.
    static void InjectAllocationFailure(int skip, int count);

    // Host-only self-test of the arena's sub-allocation logic (no CUDA call): `steps` seeded random requests and
    // releases against a fake backing store with the structural invariants checked after each; pooled = 0 tests the
    // one-allocation-per-block mode.  Returns 0, or the step at which an invariant broke (message in `why`).
    static int SelfTestRangeArena(unsigned seed, int steps, int pooled, std::string* why);

private:
    static std::map<LayerType, std::shared_ptr<LayerAccCreator>>& GetLayerCreatorMap();
};

template <typename T>
class B200CudaLayerAccRegister {
public:
    explicit B200CudaLayerAccRegister(LayerType type) { B200CudaDevice::RegisterLayerAccCreator(type, new T()); }
};

}  // namespace TNN_NS
#endif
