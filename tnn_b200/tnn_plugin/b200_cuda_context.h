// Per-instance CUDA context: one stream on `device_id` plus a workspace arena.  Replaces the reference's CudaContext
// (source/tnn/device/cuda/cuda_context.{h,cc}) without its cuDNN / cuBLAS handles and without re-allocating the
// workspace inside Forward (cuda_context.cc:137-145): accs state their need in Init/Reshape through ReserveWorkspace,
// sub-allocate 256-byte aligned slices from it and nothing is allocated while a Forward is in flight.
#ifndef TNN_B200_CUDA_CONTEXT_H_
#define TNN_B200_CUDA_CONTEXT_H_

#include <cuda_runtime.h>

#include <map>
#include <string>
#include <vector>

#include "tnn/core/context.h"

namespace TNN_NS {

class B200CudaContext : public Context {
public:
    ~B200CudaContext();
    Status Setup(int device_id);

    virtual Status LoadLibrary(std::vector<std::string> path) override;
    virtual Status GetCommandQueue(void** command_queue) override;
    virtual Status ShareCommandQueue(Context* context) override;
    virtual Status OnInstanceForwardBegin() override;
    virtual Status OnInstanceForwardEnd() override;
    virtual Status Synchronize() override;

    cudaStream_t GetStream() const { return stream_; }
    int GetDeviceId() const { return device_id_; }

    // Shared scratch used by one layer at a time (layers of an instance run in order on one stream).  Grows only
    // here, i.e. at Init/Reshape time; returns TNNERR_OUTOFMEMORY instead of aborting.
    Status ReserveWorkspace(size_t bytes);
    void* GetWorkspace() const { return workspace_; }
    size_t GetWorkspaceSize() const { return workspace_size_; }

    // kv_len of an attention mask, computed once per Forward and shared by the attention layers of the instance.
    // Returns a device pointer to B int32 values (nullptr on failure).
    const int* GetKvLen(const float* mask, int batch, int seq, float exclude_below, Status* status);

private:
    cudaStream_t stream_ = nullptr;
    bool own_stream_     = false;
    int device_id_       = 0;
    void* workspace_     = nullptr;
    size_t workspace_size_ = 0;

    int* kv_len_buf_        = nullptr;
    int kv_len_capacity_    = 0;
    const float* kv_mask_   = nullptr;   // mask the cached kv_len belongs to (valid for the current Forward only)
    int kv_batch_ = 0, kv_seq_ = 0;
    unsigned long long forward_id_ = 0, kv_forward_id_ = ~0ull;
};

}  // namespace TNN_NS
#endif
