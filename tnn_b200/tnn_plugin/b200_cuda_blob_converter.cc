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

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <vector>
#if defined(__x86_64__)
#include <immintrin.h>
#endif

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

// Worker threads for the host-side copies and conversions: what OpenMP allows this process (OMP_NUM_THREADS), at most
// 8.  A launcher that runs one rank per GPU on a host with few cores per GPU sets that to 1 (torchrun does by
// default), and it has to be respected: eight ranks with eight workers each on a 16-core host ran the pageable route
// four times slower than with one worker per rank.
int HostThreads() {
    int n = omp_get_max_threads();
    return n > 8 ? 8 : (n < 1 ? 1 : n);
}

// memcpy with a few threads: one thread moves ~10 GB/s, a PCIe 5 x16 link 50+.
void ParallelCopy(void* dst, const void* src, size_t bytes) {
    const size_t piece = 1u << 20;
    const long pieces  = static_cast<long>((bytes + piece - 1) / piece);
    const int threads  = HostThreads();
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

// ---- fp32 <-> half precision on the host cores (round to nearest even, as the device's conversion kernel does)
inline uint16_t FloatToHalfBits(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return static_cast<uint16_t>(sign | (x > 0x7f800000u ? 0x7e00u : 0x7c00u));   // NaN / inf
    if (x >= 0x477ff000u) return static_cast<uint16_t>(sign | 0x7c00u);                                  // rounds to inf
    if (x < 0x33000001u) return static_cast<uint16_t>(sign);                                            // rounds to zero
    if (x < 0x38800000u) {                                                                               // subnormal half
        const int shift   = 126 - static_cast<int>(x >> 23);          // 14 ... 24
        const uint32_t m  = (x & 0x7fffffu) | 0x800000u;
        const uint32_t q  = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
        return static_cast<uint16_t>(sign | (q + ((rem > half || (rem == half && (q & 1u))) ? 1u : 0u)));
    }
    const uint32_t r = x + 0xfffu + ((x >> 13) & 1u);                  // normal: round the 13 dropped bits to even
    return static_cast<uint16_t>(sign | ((r - 0x38000000u) >> 13));
}
inline float HalfBitsToFloat(uint16_t h) {
    const uint32_t sign = (static_cast<uint32_t>(h) & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu, x;
    if (e == 0) {
        if (m == 0) {
            x = sign;
        } else {
            int s = 0;
            while (!(m & 0x400u)) { m <<= 1; ++s; }
            x = sign | (static_cast<uint32_t>(113 - s) << 23) | ((m & 0x3ffu) << 13);
        }
    } else if (e == 31) {
        x = sign | 0x7f800000u | (m << 13);
    } else {
        x = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}
inline uint16_t FloatToBf16Bits(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((x >> 16) | 0x40u);   // NaN stays NaN
    return static_cast<uint16_t>((x + 0x7fffu + ((x >> 16) & 1u)) >> 16);
}

#if defined(__x86_64__)
__attribute__((target("avx2,f16c"))) void FloatToHalfRun(uint16_t* dst, const float* src, size_t n) {
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        _mm_storeu_si128(reinterpret_cast<__m128i*>(dst + i),
                         _mm256_cvtps_ph(_mm256_loadu_ps(src + i), _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
    for (; i < n; ++i) dst[i] = FloatToHalfBits(src[i]);
}
__attribute__((target("avx2,f16c"))) void HalfToFloatRun(float* dst, const uint16_t* src, size_t n) {
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        _mm256_storeu_ps(dst + i, _mm256_cvtph_ps(_mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i))));
    for (; i < n; ++i) dst[i] = HalfBitsToFloat(src[i]);
}
bool HaveF16C() {
    static const bool have = __builtin_cpu_supports("f16c") && __builtin_cpu_supports("avx2");
    return have;
}
#else
bool HaveF16C() { return false; }
void FloatToHalfRun(uint16_t*, const float*, size_t) {}
void HalfToFloatRun(float*, const uint16_t*, size_t) {}
#endif

// `half_dtype`: B200_F16 or B200_BF16.  A few threads each take whole pieces.
void ParallelToHalf(uint16_t* dst, const float* src, size_t n, int half_dtype) {
    const size_t piece = 1u << 18;
    const long pieces  = static_cast<long>((n + piece - 1) / piece);
    const int threads  = pieces < 4 ? 1 : HostThreads();
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long i = 0; i < pieces; ++i) {
        const size_t off = static_cast<size_t>(i) * piece;
        const size_t m   = off + piece <= n ? piece : n - off;
        if (half_dtype == B200_F16) {
            if (HaveF16C()) FloatToHalfRun(dst + off, src + off, m);
            else for (size_t k = 0; k < m; ++k) dst[off + k] = FloatToHalfBits(src[off + k]);
        } else {
            for (size_t k = 0; k < m; ++k) dst[off + k] = FloatToBf16Bits(src[off + k]);
        }
    }
}
void ParallelToFloat(float* dst, const uint16_t* src, size_t n, int half_dtype) {
    const size_t piece = 1u << 18;
    const long pieces  = static_cast<long>((n + piece - 1) / piece);
    const int threads  = pieces < 4 ? 1 : HostThreads();
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long i = 0; i < pieces; ++i) {
        const size_t off = static_cast<size_t>(i) * piece;
        const size_t m   = off + piece <= n ? piece : n - off;
        if (half_dtype == B200_F16) {
            if (HaveF16C()) HalfToFloatRun(dst + off, src + off, m);
            else for (size_t k = 0; k < m; ++k) dst[off + k] = HalfBitsToFloat(src[off + k]);
        } else {
            for (size_t k = 0; k < m; ++k) {
                const uint32_t x = static_cast<uint32_t>(src[off + k]) << 16;
                std::memcpy(dst + off + k, &x, 4);
            }
        }
    }
}

// TNN_B200_HOST_CONVERT=1: fp32 host Mats of half-precision blobs are converted on the host cores, so that only half
// the bytes cross the bus (several GPUs share the host's DMA path; with one GPU the plain copy is as fast and costs
// no host time).  Read at every conversion.
std::atomic<uint64_t> g_host_conversions{0};   // conversions that took the host-side route (for tests)

bool HostConvertWanted() {
    const char* e = std::getenv("TNN_B200_HOST_CONVERT");
    return e != nullptr && e[0] != 0 && e[0] != '0';
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

        // fp32 host Mat <-> half-precision blob, converted on the host cores (opt-in): half the bytes on the bus, no
        // device staging, no conversion launch.  ConvertToMatAsync keeps the device route (its tail runs in a stream
        // callback, which must stay off thread teams).
        if (!mat_on_device && need_convert && mdt == B200_F32 && (bdt == B200_F16 || bdt == B200_BF16) &&
            (!to_mat || blocking) && HostConvertWanted()) {
            RETURN_ON_NEQ(to_mat ? ToHostAsFloat(static_cast<float*>(image.GetData()), blob_ptr, count, bdt, stream)
                                 : FromHostAsHalf(blob_ptr, static_cast<const float*>(image.GetData()), count, bdt, stream),
                          TNN_OK);
            if (blocking) {
                if (cudaStreamSynchronize(stream) != cudaSuccess) {
                    cudaGetLastError();
                    return Status(TNNERR_CUDA_SYNC_ERROR, "stream sync failed");
                }
                if (to_mat) {
                    if (B200CudaContext* ctx = B200CudaContext::FromCommandQueue(command_queue))
                        RETURN_ON_NEQ(ctx->CheckStatusAfterSync(), TNN_OK);
                }
            }
            return TNN_OK;
        }

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

    // fp32 host Mat -> half-precision blob: chunks are converted into the page-locked staging buffer by the host cores
    // and copied from there, one chunk's conversion running while the previous chunk is on the bus.
    Status FromHostAsHalf(char* blob_ptr, const float* src, int64_t count, int half_dtype, cudaStream_t stream) {
        const size_t n = static_cast<size_t>(count);
        ++g_host_conversions;
        RETURN_ON_NEQ(EnsurePinned(n * 2), TNN_OK);
        WaitStageFree();
        const size_t chunk = kChunkBytes / 4;   // elements
        uint16_t* stage    = static_cast<uint16_t*>(pinned_);
        for (size_t off = 0; off < n; off += chunk) {
            const size_t m = off + chunk <= n ? chunk : n - off;
            ParallelToHalf(stage + off, src + off, m, half_dtype);
            RETURN_ON_NEQ(Copy(blob_ptr + off * 2, stage + off, m * 2, cudaMemcpyHostToDevice, stream), TNN_OK);
        }
        return MarkStageBusy(stream);
    }

    // half-precision blob -> fp32 host Mat (blocking): every chunk is converted out of the staging buffer as soon as it
    // has landed there.
    Status ToHostAsFloat(float* dst, const char* blob_ptr, int64_t count, int half_dtype, cudaStream_t stream) {
        const size_t n = static_cast<size_t>(count);
        ++g_host_conversions;
        RETURN_ON_NEQ(EnsurePinned(n * 2), TNN_OK);
        WaitStageFree();
        const size_t chunk  = kChunkBytes / 4;   // elements
        const size_t chunks = (n + chunk - 1) / chunk;
        while (chunk_done_.size() < chunks) {
            cudaEvent_t e = nullptr;
            if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) {
                cudaGetLastError();
                return Status(TNNERR_CUDA_SYNC_ERROR, "cudaEventCreate failed");
            }
            chunk_done_.push_back(e);
        }
        uint16_t* stage = static_cast<uint16_t*>(pinned_);
        for (size_t c = 0; c < chunks; ++c) {
            const size_t off = c * chunk;
            const size_t m   = off + chunk <= n ? chunk : n - off;
            RETURN_ON_NEQ(Copy(stage + off, blob_ptr + off * 2, m * 2, cudaMemcpyDeviceToHost, stream), TNN_OK);
            cudaEventRecord(chunk_done_[c], stream);
        }
        for (size_t c = 0; c < chunks; ++c) {
            const size_t off = c * chunk;
            const size_t m   = off + chunk <= n ? chunk : n - off;
            if (cudaEventSynchronize(chunk_done_[c]) != cudaSuccess) {
                cudaGetLastError();
                return Status(TNNERR_CUDA_SYNC_ERROR, "event sync failed");
            }
            ParallelToFloat(dst + off, stage + off, m, half_dtype);
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

}  // namespace TNN_NS

// The converter's host-side fp32 <-> half conversion, callable without a GPU (declared in include/tnn_b200_plugin.h).
extern "C" __attribute__((visibility("default"))) int tnnb200_host_convert(const float* src, uint64_t n, int half_dtype,
                                                                            int force_scalar, uint16_t* half_out,
                                                                            float* back_out) {
    using namespace TNN_NS;
    if (!src || !half_out || (half_dtype != B200_F16 && half_dtype != B200_BF16)) return -1;
    if (force_scalar) {
        for (uint64_t i = 0; i < n; ++i)
            half_out[i] = half_dtype == B200_F16 ? FloatToHalfBits(src[i]) : FloatToBf16Bits(src[i]);
        if (back_out) {
            for (uint64_t i = 0; i < n; ++i) {
                if (half_dtype == B200_F16) {
                    back_out[i] = HalfBitsToFloat(half_out[i]);
                } else {
                    const uint32_t x = static_cast<uint32_t>(half_out[i]) << 16;
                    std::memcpy(back_out + i, &x, 4);
                }
            }
        }
        return 0;
    }
    ParallelToHalf(half_out, src, static_cast<size_t>(n), half_dtype);
    if (back_out) ParallelToFloat(back_out, half_out, static_cast<size_t>(n), half_dtype);
    return HaveF16C() ? 1 : 0;
}

extern "C" __attribute__((visibility("default"))) uint64_t tnnb200_host_conversions() {
    return TNN_NS::g_host_conversions.load();
}

namespace TNN_NS {

DECLARE_BLOB_CONVERTER_CREATER(B200Cuda);
REGISTER_BLOB_CONVERTER(B200Cuda, DEVICE_CUDA);

}  // namespace TNN_NS
