// Mat <-> Blob conversion for DEVICE_CUDA blobs (the I/O edge of the encoder).  Replaces the reference's
// CudaBlobConverterAcc (source/tnn/device/cuda/cuda_blob_converter.cc:36-194) for the Mat types this path uses:
// NCHW_FLOAT, NC_INT32 and the half-precision RESERVED_FP16_TEST / RESERVED_BFP16_TEST, host or device Mats.
// Differences: BlobHandle.bytes_offset is honoured (the reference ignores it, :133), half / bfloat16 blobs convert
// through the library's conversion kernel (the fused region's outputs are half precision), non-identity scale/bias
// (image preprocessing) is refused rather than mis-applied to a [B,S,H] activation, and host Mats move like this:
//
//   * a Mat whose memory is page-locked (cudaHostAlloc / cudaHostRegister by the caller; found with
//     cudaPointerGetAttributes) is the source / target of the DMA itself: one cudaMemcpyAsync, nothing else;
//   * a pageable Mat goes through the converter's own page-locked staging buffer in 8 MiB chunks, the host copy of one
//     chunk (several threads) running while the previous chunk is on the bus; the reference hands the pageable
//     pointer to cudaMemcpyAsync, which stages it inside the driver at a fraction of the bus rate;
//   * ConvertFromMatAsync returns when the caller's Mat has been read (it may be reused at once);
//     ConvertToMatAsync enqueues the device-to-host copy and, for a pageable Mat, a host function behind it that
//     fills the Mat: the Mat is complete once the command queue has been synchronised, as the interface says.
//
// The staging buffers (page-locked host memory, and device memory when Mat and blob types differ) are sized on the
// first conversion of a blob and kept; later conversions allocate nothing.  One converter serves one conversion at a
// time (TNN creates one per input / output blob); a second call waits until the first one's staging is free.
#include <cuda_runtime.h>
#include <omp.h>

#include <cstring>
#include <vector>

#include "b200_cuda_context.h"
#include "b200_cuda_device.h"
#include "b200_plugin_common.h"
#include "tnn/core/blob.h"
#include "tnn/core/mat.h"
#include "tnn/utils/blob_converter_internal.h"
#include "tnn/utils/dims_utils.h"

namespace TNN_NS {

namespace {

constexpr size_t kChunkBytes = 8u << 20;

// memcpy with a few threads: one thread moves ~10 GB/s, a PCIe 5 x16 link 50+.
void ParallelCopy(void* dst, const void* src, size_t bytes) {
    const size_t piece = 1u << 20;
    const long pieces  = static_cast<long>((bytes + piece - 1) / piece);
    int threads        = omp_get_max_threads();
    if (threads > 8) threads = 8;
    if (pieces < 4 || threads < 2) {
        std::memcpy(dst, src, bytes);
        return;
    }
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long i = 0; i < pieces; ++i) {
        const size_t off = static_cast<size_t>(i) * piece;
        const size_t n   = off + piece <= bytes ? piece : bytes - off;
        std::memcpy(static_cast<char*>(dst) + off, static_cast<const char*>(src) + off, n);
    }
}

bool IsPageLocked(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeHost;
}

struct HostCopyJob {
    void* dst;
    const void* src;
    size_t bytes;
};
void CUDART_CB RunHostCopy(void* arg) {
    auto* j = static_cast<HostCopyJob*>(arg);
    std::memcpy(j->dst, j->src, j->bytes);   // a stream callback must stay off the CUDA API and off OpenMP teams
}

}  // namespace

class B200CudaBlobConverterAcc : public BlobConverterAcc {
public:
    explicit B200CudaBlobConverterAcc(Blob* blob) : BlobConverterAcc(blob) {}
    virtual ~B200CudaBlobConverterAcc() {
        if (stage_free_) {
            cudaEventSynchronize(stage_free_);
            cudaEventDestroy(stage_free_);
        }
        for (cudaEvent_t e : chunk_done_) cudaEventDestroy(e);
        if (dev_stage_) {
            auto* dev = dynamic_cast<B200CudaDevice*>(GetDevice(DEVICE_CUDA));
            if (dev) dev->Free(dev_stage_);
        }
        if (pinned_) B200CudaDevice::FreeHost(pinned_);
        cudaGetLastError();
    }

    virtual Status ConvertToMat(Mat& image, MatConvertParam param, void* command_queue = NULL) {
        return Convert(image, param, command_queue, /*to_mat=*/true, /*blocking=*/true);
    }
    virtual Status ConvertFromMat(Mat& image, MatConvertParam param, void* command_queue = NULL) {
        return Convert(image, param, command_queue, /*to_mat=*/false, /*blocking=*/true);
    }
    virtual Status ConvertToMatAsync(Mat& image, MatConvertParam param, void* command_queue = NULL) {
        return Convert(image, param, command_queue, /*to_mat=*/true, /*blocking=*/false);
    }
    virtual Status ConvertFromMatAsync(Mat& image, MatConvertParam param, void* command_queue = NULL) {
        return Convert(image, param, command_queue, /*to_mat=*/false, /*blocking=*/false);
    }

private:
    Status Convert(Mat& image, const MatConvertParam& param, void* command_queue, bool to_mat, bool blocking) {
        cudaStream_t stream = static_cast<cudaStream_t>(command_queue);
        if (!blob_) return Status(TNNERR_NULL_PARAM, "blob is null");
        if (NeedDoScaleBias(param) || param.reverse_channel)
            return Status(TNNERR_PARAM_ERR, "tnn_b200 blob converter: scale/bias/reverse_channel are not supported");
        const BlobDesc& desc = blob_->GetBlobDesc();
        const int64_t count  = DimsVectorUtils::Count(desc.dims);
        if (count != DimsVectorUtils::Count(image.GetDims()))
            return Status(TNNERR_PARAM_ERR, "Mat and Blob element counts differ");
        BlobHandle h   = blob_->GetHandle();
        char* blob_ptr = static_cast<char*>(h.base) + h.bytes_offset;
        const MatType mt = image.GetMatType();
        const bool mat_on_device = image.GetDeviceType() == DEVICE_CUDA;

        // Mat element type (as a kernel-library dtype; int32 moves as raw 4-byte words) and blob element type
        int mdt = -1, bdt = -1;
        size_t mes = 0;
        if (mt == NC_INT32) {
            if (desc.data_type != DATA_TYPE_INT32) return Status(TNNERR_PARAM_ERR, "NC_INT32 Mat needs an int32 blob");
            mdt = bdt = B200_F32;   // same type on both sides: plain copy
            mes = 4;
        } else {
            // Float Mats: NCHW_FLOAT, or half precision / bfloat16 host data (RESERVED_FP16_TEST / RESERVED_BFP16_TEST,
            // the Mat types the reference's default converter accepts for them,
            // source/tnn/utils/blob_converter_default.cc:323-331): with a blob of the same type the copy is the whole
            // conversion, which halves the bytes over PCIe.
            mdt = mt == NCHW_FLOAT ? B200_F32 : (mt == RESERVED_FP16_TEST ? B200_F16 : (mt == RESERVED_BFP16_TEST ? B200_BF16 : -1));
            if (mdt < 0) return Status(TNNERR_PARAM_ERR, "tnn_b200 blob converter: Mat type not supported");
            bdt = B200DataType(desc.data_type);
            if (bdt < 0) return Status(TNNERR_PARAM_ERR, "blob data type not supported");
            mes = mdt == B200_F32 ? 4 : 2;
        }
        const size_t bytes      = static_cast<size_t>(count) * mes;
        const bool need_convert = mdt != bdt;

        // The Mat-typed image of the data on the device: the blob itself, or the staging buffer next to it.
        char* dev_side = blob_ptr;
        if (mat_on_device) {
            dev_side = static_cast<char*>(image.GetData());
        } else if (need_convert) {
            RETURN_ON_NEQ(EnsureDeviceStage(bytes, stream), TNN_OK);
            dev_side = static_cast<char*>(dev_stage_);
        }

        Status st = TNN_OK;
        if (to_mat) {
            if (need_convert)
                RETURN_ON_NEQ(B200ToStatus(b200_convert(blob_ptr, bdt, dev_side, mdt, count, stream), "b200_convert"), TNN_OK);
            if (mat_on_device) {
                if (!need_convert) st = Copy(dev_side, blob_ptr, bytes, cudaMemcpyDeviceToDevice, stream);
            } else {
                st = ToHost(image.GetData(), dev_side, bytes, stream, blocking);
            }
        } else {
            if (mat_on_device) {
                if (!need_convert) st = Copy(blob_ptr, dev_side, bytes, cudaMemcpyDeviceToDevice, stream);
            } else {
                st = FromHost(dev_side, image.GetData(), bytes, stream);
            }
            if (st == TNN_OK && need_convert)
                st = B200ToStatus(b200_convert(dev_side, mdt, blob_ptr, bdt, count, stream), "b200_convert");
        }
        RETURN_ON_NEQ(st, TNN_OK);
        if (blocking) {
            if (cudaStreamSynchronize(stream) != cudaSuccess) {
                cudaGetLastError();
                return Status(TNNERR_CUDA_SYNC_ERROR, "stream sync failed");
            }
            // The stream has drained, so the instance's status word (copied to the host behind the last Forward) is
            // in: a Forward whose device-side wait ran out is reported with its output, not one call later.
            if (to_mat) {
                if (B200CudaContext* ctx = B200CudaContext::FromCommandQueue(command_queue))
                    RETURN_ON_NEQ(ctx->CheckStatusAfterSync(), TNN_OK);
            }
        }
        return TNN_OK;
    }

    // host Mat -> device.  Returns when the Mat has been read.
    Status FromHost(char* dst_dev, const void* src, size_t bytes, cudaStream_t stream) {
        if (IsPageLocked(src)) return Copy(dst_dev, src, bytes, cudaMemcpyHostToDevice, stream);
        RETURN_ON_NEQ(EnsurePinned(bytes), TNN_OK);
        WaitStageFree();
        for (size_t off = 0; off < bytes; off += kChunkBytes) {
            const size_t n = off + kChunkBytes <= bytes ? kChunkBytes : bytes - off;
            ParallelCopy(static_cast<char*>(pinned_) + off, static_cast<const char*>(src) + off, n);
            RETURN_ON_NEQ(Copy(dst_dev + off, static_cast<char*>(pinned_) + off, n, cudaMemcpyHostToDevice, stream), TNN_OK);
        }
        return MarkStageBusy(stream);
    }

    // device -> host Mat.
    Status ToHost(void* dst, const char* src_dev, size_t bytes, cudaStream_t stream, bool blocking) {
        if (IsPageLocked(dst)) return Copy(dst, src_dev, bytes, cudaMemcpyDeviceToHost, stream);
        RETURN_ON_NEQ(EnsurePinned(bytes), TNN_OK);
        WaitStageFree();
        if (!blocking) {
            RETURN_ON_NEQ(Copy(pinned_, src_dev, bytes, cudaMemcpyDeviceToHost, stream), TNN_OK);
            job_.dst   = dst;
            job_.src   = pinned_;
            job_.bytes = bytes;
            if (cudaLaunchHostFunc(stream, RunHostCopy, &job_) != cudaSuccess) {
                cudaGetLastError();
                return Status(TNNERR_CUDA_MEMCPY_ERROR, "cudaLaunchHostFunc failed");
            }
            return MarkStageBusy(stream);
        }
        // Blocking: every chunk is copied out of the staging buffer as soon as it has landed there.
        const size_t chunks = (bytes + kChunkBytes - 1) / kChunkBytes;
        while (chunk_done_.size() < chunks) {
            cudaEvent_t e = nullptr;
            if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) {
                cudaGetLastError();
                return Status(TNNERR_CUDA_SYNC_ERROR, "cudaEventCreate failed");
            }
            chunk_done_.push_back(e);
        }
        for (size_t c = 0; c < chunks; ++c) {
            const size_t off = c * kChunkBytes;
            const size_t n   = off + kChunkBytes <= bytes ? kChunkBytes : bytes - off;
            RETURN_ON_NEQ(Copy(static_cast<char*>(pinned_) + off, src_dev + off, n, cudaMemcpyDeviceToHost, stream), TNN_OK);
            cudaEventRecord(chunk_done_[c], stream);
        }
        for (size_t c = 0; c < chunks; ++c) {
            const size_t off = c * kChunkBytes;
            const size_t n   = off + kChunkBytes <= bytes ? kChunkBytes : bytes - off;
            if (cudaEventSynchronize(chunk_done_[c]) != cudaSuccess) {
                cudaGetLastError();
                return Status(TNNERR_CUDA_SYNC_ERROR, "event sync failed");
            }
            ParallelCopy(static_cast<char*>(dst) + off, static_cast<char*>(pinned_) + off, n);
        }
        return TNN_OK;
    }

    Status EnsurePinned(size_t bytes) {
        if (bytes <= pinned_bytes_ && pinned_) return TNN_OK;
        WaitStageFree();
        if (pinned_) B200CudaDevice::FreeHost(pinned_);
        pinned_       = nullptr;
        pinned_bytes_ = 0;
        RETURN_ON_NEQ(B200CudaDevice::AllocateHost(&pinned_, bytes), TNN_OK);
        pinned_bytes_ = bytes;
        return TNN_OK;
    }

    Status EnsureDeviceStage(size_t bytes, cudaStream_t stream) {
        if (bytes <= dev_stage_bytes_ && dev_stage_) return TNN_OK;
        auto* dev = dynamic_cast<B200CudaDevice*>(GetDevice(DEVICE_CUDA));
        if (!dev) return Status(TNNERR_DEVICE_NOT_SUPPORT, "DEVICE_CUDA is not served by tnn_b200");
        if (dev_stage_) {
            cudaStreamSynchronize(stream);   // a conversion still in flight may use the old block
            dev->Free(dev_stage_);
            dev_stage_       = nullptr;
            dev_stage_bytes_ = 0;
        }
        RETURN_ON_NEQ(dev->Allocate(&dev_stage_, bytes), TNN_OK);
        dev_stage_bytes_ = bytes;
        return TNN_OK;
    }

    // The page-locked staging buffer is in use until the copies (and the host function) enqueued on it have run.
    void WaitStageFree() {
        if (stage_free_ && stage_busy_) {
            cudaEventSynchronize(stage_free_);
            stage_busy_ = false;
        }
    }
    Status MarkStageBusy(cudaStream_t stream) {
        if (!stage_free_ && cudaEventCreateWithFlags(&stage_free_, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            stage_free_ = nullptr;
            // without an event the only safe answer is to wait here
            cudaStreamSynchronize(stream);
            return TNN_OK;
        }
        cudaEventRecord(stage_free_, stream);
        stage_busy_ = true;
        return TNN_OK;
    }

    static Status Copy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, cudaStream_t stream) {
        if (cudaMemcpyAsync(dst, src, bytes, kind, stream) != cudaSuccess) {
            cudaGetLastError();
            return Status(TNNERR_CUDA_MEMCPY_ERROR, "cudaMemcpyAsync failed");
        }
        return TNN_OK;
    }

    void* dev_stage_        = nullptr;   // Mat-typed image of the blob on the device (only when the types differ)
    size_t dev_stage_bytes_ = 0;
    void* pinned_           = nullptr;   // page-locked host staging for pageable Mats
    size_t pinned_bytes_    = 0;
    cudaEvent_t stage_free_ = nullptr;
    bool stage_busy_        = false;
    std::vector<cudaEvent_t> chunk_done_;
    HostCopyJob job_{nullptr, nullptr, 0};
};

DECLARE_BLOB_CONVERTER_CREATER(B200Cuda);
REGISTER_BLOB_CONVERTER(B200Cuda, DEVICE_CUDA);

}  // namespace TNN_NS
