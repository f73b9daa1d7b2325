#include "b200_cuda_layer_acc.h"

#include "tnn/utils/blob_transfer_utils.h"

namespace TNN_NS {

B200CudaLayerAcc::~B200CudaLayerAcc() {
    for (void* p : owned_)
        if (p && device_) device_->Free(p);
}

Status B200CudaLayerAcc::Init(Context* context, LayerParam* param, LayerResource* resource,
                              const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    AbstractLayerAcc::Init(context, param, resource, inputs, outputs);   // format resolution; 3-D blobs stay AUTO
    device_   = dynamic_cast<B200CudaDevice*>(GetDevice(DEVICE_CUDA));
    context_  = dynamic_cast<B200CudaContext*>(context);
    param_    = param;
    resource_ = resource;
    if (!device_ || !context_) return Status(TNNERR_DEVICE_NOT_SUPPORT, "DEVICE_CUDA is not served by tnn_b200");
    return ReloadConstantBlobs(inputs, false);
}

Status B200CudaLayerAcc::ReloadConstantBlobs(const std::vector<Blob*>& inputs, bool only_reload_shape_differ_blob) {
    void* command_queue = nullptr;
    context_->GetCommandQueue(&command_queue);
    for (auto* blob : inputs) {
        const std::string name = blob->GetBlobDesc().name;
        if (const_resource_ == nullptr || const_resource_->find(name) == const_resource_->end()) continue;
        if (only_reload_shape_differ_blob && const_resource_flag_ &&
            const_resource_flag_->find(name) == const_resource_flag_->end())
            continue;
        auto buffer = (*const_resource_)[name];
        if (buffer->GetBytesSize() == 0) continue;
        std::shared_ptr<Blob> host_blob = nullptr;
        RETURN_ON_NEQ(RawBuffer2Blob(buffer.get(), host_blob), TNN_OK);
        BlobDesc desc    = host_blob->GetBlobDesc();
        desc.device_type = DEVICE_CUDA;
        auto cuda_blob   = std::make_shared<Blob>(desc, true);
        RETURN_ON_NEQ(CopyToDevice(cuda_blob.get(), host_blob.get(), command_queue), TNN_OK);
        cuda_blob->SetFlag(DATA_FLAG_CHANGE_NEVER);
        const_blob_map_[name] = cuda_blob;
        blob->SetHandle(cuda_blob->GetHandle());
    }
    return TNN_OK;
}

Status B200CudaLayerAcc::Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) { return TNN_OK; }
Status B200CudaLayerAcc::DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) { return TNN_OK; }

Status B200CudaLayerAcc::Forward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    if (context_->Replaying()) return TNN_OK;   // the instance's graph stands for this layer's launches
    context_->RecordCall(this, inputs, outputs);
#if TNN_PROFILE
    if (context_->profile_layer) {
        auto pdata = std::make_shared<ProfilingData>();
        UpdateProfilingData(pdata.get(), param_, inputs[0]->GetBlobDesc().dims, outputs[0]->GetBlobDesc().dims);
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, context_->GetStream());
        Status st = DoForward(inputs, outputs);
        cudaEventRecord(e1, context_->GetStream());
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        pdata->kernel_time = ms;
        context_->AddProfilingData(pdata);
        return st;
    }
#endif
    return DoForward(inputs, outputs);
}

Status B200CudaLayerAcc::EnsureBuffer(void** ptr, size_t* capacity, size_t bytes) {
    if (bytes <= *capacity && *ptr) return TNN_OK;
    void* p = nullptr;
    RETURN_ON_NEQ(device_->Allocate(&p, bytes), TNN_OK);
    if (*ptr) {
        cudaStreamSynchronize(context_->GetStream());
        for (auto& o : owned_)
            if (o == *ptr) o = nullptr;
        device_->Free(*ptr);
    }
    owned_.push_back(p);
    *ptr      = p;
    *capacity = bytes;
    return TNN_OK;
}

std::vector<DataFormat> B200CudaLayerAcc::SupportDataFormat(DataType data_type, int dims_size, BlobType blob_type) {
    std::vector<DataFormat> list;
    if (dims_size == 4) list.push_back(DATA_FORMAT_NCHW);
    return list;
}

}  // namespace TNN_NS
