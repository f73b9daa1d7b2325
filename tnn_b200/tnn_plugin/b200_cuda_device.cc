#include "b200_cuda_device.h"

#include <cuda_runtime.h>

#include <atomic>

#include "b200_cuda_context.h"
#include "tnn/utils/blob_memory_size_utils.h"
#include "tnn/utils/data_type_utils.h"
#include "tnn/utils/dims_utils.h"

namespace TNN_NS {

static std::atomic<int> g_fail_allocations{0};

B200CudaDevice::B200CudaDevice(DeviceType device_type) : AbstractDevice(device_type) {}
B200CudaDevice::~B200CudaDevice() {}

void B200CudaDevice::FailNextAllocations(int n) { g_fail_allocations.store(n); }

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
    if (g_fail_allocations.load() > 0) {
        g_fail_allocations.fetch_sub(1);
        return Status(TNNERR_OUTOFMEMORY, "cuda alloc failed (injected)");
    }
    // cudaMalloc returns at least 256-byte aligned blocks, which is what the TMA descriptors need (16) with room to
    // spare; sizes are rounded up so that vector loads of a trailing partial group stay inside the block.
    const size_t rounded = (bytes + 255) & ~static_cast<size_t>(255);
    void* ptr = nullptr;
    cudaError_t st = cudaMalloc(&ptr, rounded ? rounded : 256);
    if (st != cudaSuccess || ptr == nullptr) {
        cudaGetLastError();
        return Status(TNNERR_OUTOFMEMORY, "cuda alloc failed");
    }
    *handle = ptr;
    return TNN_OK;
}

Status B200CudaDevice::Free(void* handle) {
    if (cudaFree(handle) != cudaSuccess) {
        cudaGetLastError();
        return Status(TNNERR_COMMON_ERROR, "cuda free failed");
    }
    return TNN_OK;
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

std::map<LayerType, std::shared_ptr<LayerAccCreator>>& B200CudaDevice::GetLayerCreatorMap() {
    static std::map<LayerType, std::shared_ptr<LayerAccCreator>> m;
    return m;
}

TypeDeviceRegister<B200CudaDevice> g_b200_cuda_device_register(DEVICE_CUDA);

}  // namespace TNN_NS
