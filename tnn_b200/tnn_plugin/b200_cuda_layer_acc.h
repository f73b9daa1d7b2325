// Base class of the plug-in's DEVICE_CUDA layer accs: the AbstractLayerAcc surface
// (Init / Reshape / Forward over TNN Blobs, source/tnn/core/abstract_layer_acc.h:39-127) with the stream, the device
// and the upload of constant input blobs, as the reference's CudaLayerAcc provides
// (source/tnn/device/cuda/acc/cuda_layer_acc.{h,cc}: Init :31-45, ReloadConstantBlobs :47-85, SupportDataFormat
// :96-102 — the constant upload and the format list follow that file because AbstractLayerAcc's protected members
// dictate them).  Differences: device pointers honour BlobHandle.bytes_offset, acc-private buffers are sized in
// Init/Reshape (never in Forward), errors come back as Status, and Forward is a wrapper: the subclasses implement
// DoForward, and Forward skips it while the context replays a captured CUDA graph of the whole instance
// (b200_cuda_context.h).  Built with TNN_PROFILE, Forward brackets DoForward with CUDA events and feeds the layer's
// device time to the context's profile, as the reference's CPU accs do with host timers
// (source/tnn/device/x86/acc/x86_layer_acc.cc:55-73).
#ifndef TNN_B200_CUDA_LAYER_ACC_H_
#define TNN_B200_CUDA_LAYER_ACC_H_

#include <vector>

#include "b200_cuda_context.h"
#include "b200_cuda_device.h"
#include "b200_plugin_common.h"
#include "tnn/core/abstract_layer_acc.h"
#include "tnn/core/blob.h"

namespace TNN_NS {

class B200CudaLayerAcc : public AbstractLayerAcc {
public:
    virtual ~B200CudaLayerAcc();
    virtual Status Init(Context* context, LayerParam* param, LayerResource* resource, const std::vector<Blob*>& inputs,
                        const std::vector<Blob*>& outputs);
    virtual Status Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs);
    virtual Status Forward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) final;
    // The layer's launches on the context's stream.  Also called by the context itself when a graph capture has to
    // be re-run eagerly.
    virtual Status DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs);
    virtual Status ReloadConstantBlobs(const std::vector<Blob*>& inputs, bool only_reload_shape_differ_blob = false);

protected:
    static void* DevicePtr(Blob* blob) {
        BlobHandle h = blob->GetHandle();
        return static_cast<char*>(h.base) + h.bytes_offset;
    }
    // Acc-owned device buffer (freed in the destructor); (re)allocated only when it has to grow.
    Status EnsureBuffer(void** ptr, size_t* capacity, size_t bytes);

    B200CudaDevice* device_   = nullptr;
    B200CudaContext* context_ = nullptr;
    LayerParam* param_        = nullptr;
    LayerResource* resource_  = nullptr;
    std::vector<void*> owned_;

private:
    virtual std::vector<DataFormat> SupportDataFormat(DataType data_type, int dims_size, BlobType blob_type);
};

#define B200_DECLARE_CUDA_ACC(type_string)                                                                             \
    class B200Cuda##type_string##LayerAcc : public B200CudaLayerAcc {                                                  \
    public:                                                                                                            \
        virtual Status Init(Context* context, LayerParam* param, LayerResource* resource,                              \
                            const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs);                      \
        virtual ~B200Cuda##type_string##LayerAcc() {}                                                                  \
        virtual Status Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs);                   \
        virtual Status DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs);                 \
                                                                                                                       \
    private:

#define B200_REGISTER_CUDA_ACC(type_string, layer_type)                                                                \
    B200CudaLayerAccRegister<TypeLayerAccCreator<B200Cuda##type_string##LayerAcc>> g_b200_cuda_##type_string##_acc(    \
        layer_type);

}  // namespace TNN_NS
#endif
