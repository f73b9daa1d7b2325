#include "b200_cuda_context.h"

#include "b200_plugin_common.h"

namespace TNN_NS {

B200CudaContext::~B200CudaContext() {
    cudaSetDevice(device_id_);
    if (workspace_) cudaFree(workspace_);
    if (kv_len_buf_) cudaFree(kv_len_buf_);
    if (own_stream_ && stream_) cudaStreamDestroy(stream_);
}

Status B200CudaContext::Setup(int device_id) {
    device_id_ = device_id;
    if (cudaSetDevice(device_id) != cudaSuccess) {
        cudaGetLastError();
        return Status(TNNERR_DEVICE_NOT_SUPPORT, "cudaSetDevice failed");
    }
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device_id);
    if (major != 10) return Status(TNNERR_DEVICE_NOT_SUPPORT, "tnn_b200 needs a compute-capability 10.x GPU");
    if (cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        return Status(TNNERR_DEVICE_NOT_SUPPORT, "cudaStreamCreate failed");
    }
    own_stream_ = true;
    return TNN_OK;
}

Status B200CudaContext::LoadLibrary(std::vector<std::string> path) { return TNN_OK; }

Status B200CudaContext::GetCommandQueue(void** command_queue) {
    cudaSetDevice(device_id_);   // the caller's thread may have switched devices (several replicas per process)
    *command_queue = stream_;
    return TNN_OK;
}

Status B200CudaContext::ShareCommandQueue(Context* context) {
    auto* other = dynamic_cast<B200CudaContext*>(context);
    if (!other) return Status(TNNERR_DEVICE_LIBRARY_LOAD, "inpute context is not B200CudaContext");
    if (own_stream_ && stream_) cudaStreamDestroy(stream_);
    own_stream_ = false;
    stream_     = other->stream_;
    return TNN_OK;
}

Status B200CudaContext::OnInstanceForwardBegin() {
    cudaSetDevice(device_id_);
    ++forward_id_;
    return TNN_OK;
}

Status B200CudaContext::OnInstanceForwardEnd() { return TNN_OK; }

Status B200CudaContext::Synchronize() {
    if (cudaStreamSynchronize(stream_) != cudaSuccess) {
        cudaGetLastError();
        return Status(TNNERR_CUDA_SYNC_ERROR, "stream synchronize failed");
    }
    // A bounded device-side wait that ran out is reported here, after the stream has drained.
    const int rc = b200_device_status();
    if (rc != B200_OK) return B200ToStatus(rc, "device status");
    return TNN_OK;
}

Status B200CudaContext::ReserveWorkspace(size_t bytes) {
    if (bytes <= workspace_size_) return TNN_OK;
    cudaSetDevice(device_id_);
    cudaStreamSynchronize(stream_);   // Init/Reshape time only: nothing of this instance may still use the old block
    void* p = nullptr;
    const size_t rounded = (bytes + 255) & ~static_cast<size_t>(255);
    if (cudaMalloc(&p, rounded) != cudaSuccess) {
        cudaGetLastError();
        return Status(TNNERR_OUTOFMEMORY, "workspace alloc failed");
    }
    if (workspace_) cudaFree(workspace_);
    workspace_      = p;
    workspace_size_ = rounded;
    return TNN_OK;
}

const int* B200CudaContext::GetKvLen(const float* mask, int batch, int seq, float exclude_below, Status* status) {
    *status = TNN_OK;
    if (kv_forward_id_ == forward_id_ && kv_mask_ == mask && kv_batch_ == batch && kv_seq_ == seq) return kv_len_buf_;
    if (batch > kv_len_capacity_) {
        // Grows only on the first Forward with a larger batch than any seen before.
        cudaStreamSynchronize(stream_);
        if (kv_len_buf_) cudaFree(kv_len_buf_);
        kv_len_buf_ = nullptr;
        if (cudaMalloc(reinterpret_cast<void**>(&kv_len_buf_), sizeof(int) * static_cast<size_t>(batch)) != cudaSuccess) {
            cudaGetLastError();
            kv_len_capacity_ = 0;
            *status = Status(TNNERR_OUTOFMEMORY, "kv_len alloc failed");
            return nullptr;
        }
        kv_len_capacity_ = batch;
    }
    const int rc = b200_mask_to_kv_len(mask, batch, seq, exclude_below, kv_len_buf_, stream_);
    if (rc != B200_OK) {
        *status = B200ToStatus(rc, "b200_mask_to_kv_len");
        return nullptr;
    }
    kv_forward_id_ = forward_id_;
    kv_mask_       = mask;
    kv_batch_      = batch;
    kv_seq_        = seq;
    return kv_len_buf_;
}

}  // namespace TNN_NS
