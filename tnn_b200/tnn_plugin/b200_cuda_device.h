// DEVICE_CUDA for TNN's DefaultNetwork, B200 build.  Replaces the reference's CudaDevice
// (source/tnn/device/cuda/cuda_device.{h,cc}), which routes DEVICE_CUDA to TensorRT
// (ConvertAutoNetworkType() == NETWORK_TYPE_TENSORRT, cuda_device.cc:159-161), allocates with `int` byte counts
// (cuda_device.cc:53-64) and aborts on CUDA errors.  This one serves NETWORK_TYPE_DEFAULT, uses 64-bit sizes,
// hands out 256-byte aligned blocks and returns Status codes.
#ifndef TNN_B200_CUDA_DEVICE_H_
#define TNN_B200_CUDA_DEVICE_H_

#include <map>
#include <memory>

#include "tnn/core/abstract_device.h"

namespace TNN_NS {

class B200CudaDevice : public AbstractDevice {
public:
    explicit B200CudaDevice(DeviceType device_type);
    ~B200CudaDevice();

    virtual BlobMemorySizeInfo Calculate(BlobDesc& desc);
    virtual Status Allocate(void** handle, MatType mat_type, DimsVector dims);
    virtual Status Allocate(void** handle, BlobMemorySizeInfo& size_info);
    Status Allocate(void** handle, size_t bytes);
    virtual Status Free(void* handle);
    virtual Status CopyToDevice(BlobHandle* dst, const BlobHandle* src, BlobDesc& desc, void* command_queue);
    virtual Status CopyFromDevice(BlobHandle* dst, const BlobHandle* src, BlobDesc& desc, void* command_queue);
    virtual AbstractLayerAcc* CreateLayerAcc(LayerType type);
    virtual Context* CreateContext(int device_id);
    virtual NetworkType ConvertAutoNetworkType();

    static Status RegisterLayerAccCreator(LayerType type, LayerAccCreator* creator);

    // Test hook: the next `n` allocations fail with TNNERR_OUTOFMEMORY (host-side fault injection; no GPU fault).
    static void FailNextAllocations(int n);

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
