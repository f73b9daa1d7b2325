// C ABI over TNN's public C++ API (TNN::Init / CreateInst / Instance::Forward, include/tnn/core/tnn.h:34-67,
// include/tnn/core/instance.h:42-144) so that a host without C++ bindings — the Python tests and the benchmark — can
// drive a TNN instance on any registered device: DEVICE_NAIVE / DEVICE_X86 (the reference's CPU implementations) or
// DEVICE_CUDA (served by the tnn_b200 plug-in once it has been loaded into the process).
// Only public TNN headers are used.  Nothing here computes.
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "tnn/core/common.h"
#include "tnn/core/instance.h"
#include "tnn/core/mat.h"
#include "tnn/core/tnn.h"
#include "tnn/utils/blob_converter.h"
#include "tnn/utils/dims_vector_utils.h"

using namespace TNN_NS;

namespace {

struct Handle {
    TNN net;
    std::shared_ptr<Instance> inst;
    DeviceType device;
    std::string last_error;
    // The caller-driven conversion path (BlobConverter on an input / output blob, as TNNTest drives it,
    // test/test.cc:99-152): converters and Mats are created once per blob and reused.
    std::map<std::string, std::shared_ptr<BlobConverter>> converters;
    std::map<std::string, std::shared_ptr<Mat>> mats;
};

bool read_file(const char* path, std::string* out) {
    std::ifstream f(path, std::ios::binary);
    if (!f) return false;
    std::stringstream ss;
    ss << f.rdbuf();
    *out = ss.str();
    return true;
}

void set_err(char* err, int errlen, const std::string& msg) {
    if (err && errlen > 0) {
        std::snprintf(err, static_cast<size_t>(errlen), "%s", msg.c_str());
    }
}

int64_t count(const DimsVector& d) {
    int64_t n = 1;
    for (int x : d) n *= x;
    return n;
}

// `kind` of the C interface -> MatType: 0 = NCHW_FLOAT, 1 = RESERVED_FP16_TEST, 2 = RESERVED_BFP16_TEST, 3 = NC_INT32.
bool mat_type_of(int kind, MatType* mt) {
    switch (kind) {
        case 0: *mt = NCHW_FLOAT; return true;
        case 1: *mt = RESERVED_FP16_TEST; return true;
        case 2: *mt = RESERVED_BFP16_TEST; return true;
        case 3: *mt = NC_INT32; return true;
        default: return false;
    }
}

}  // namespace

extern "C" {

#define TNNC_API __attribute__((visibility("default")))

// device: 0 = DEVICE_NAIVE, 1 = DEVICE_X86, 2 = DEVICE_CUDA.  precision: -1 auto, 0 normal, 1 high, 2 low.
// Returns an opaque handle or NULL (message in err).
// share_memory_mode: 0 = every instance allocates its blob memory, 1 = instances created by one thread share it
// (SHARE_MEMORY_MODE_SHARE_ONE_THREAD), 2 = the caller provides it (SHARE_MEMORY_MODE_SET_FROM_EXTERNAL: ask
// tnnc_forward_memory_size, then tnnc_set_forward_memory before the first Forward).
TNNC_API void* tnnc_create_ex(const char* proto_path, const char* model_path, int device, int device_id, int precision,
                              int cpu_threads, int share_memory_mode, char* err, int errlen) {
    std::unique_ptr<Handle> h(new Handle);
    ModelConfig mc;
    mc.model_type = MODEL_TYPE_TNN;
    std::string proto, model;
    if (!read_file(proto_path, &proto) || !read_file(model_path, &model)) {
        set_err(err, errlen, "cannot read proto/model file");
        return nullptr;
    }
    mc.params = {proto, model};
    Status st = h->net.Init(mc);
    if (st != TNN_OK) {
        set_err(err, errlen, "TNN::Init: " + st.description());
        return nullptr;
    }
    NetworkConfig nc;
    nc.device_type = device == 0 ? DEVICE_NAIVE : (device == 1 ? DEVICE_X86 : DEVICE_CUDA);
    nc.device_id = device_id;
    nc.network_type = NETWORK_TYPE_DEFAULT;
    nc.precision = static_cast<Precision>(precision);
    nc.share_memory_mode = static_cast<ShareMemoryMode>(share_memory_mode);
    h->device = nc.device_type;
    h->inst = h->net.CreateInst(nc, st);
    if (st != TNN_OK || !h->inst) {
        set_err(err, errlen, "CreateInst: " + st.description());
        return nullptr;
    }
    if (cpu_threads > 0) h->inst->SetCpuNumThreads(cpu_threads);
    return h.release();
}

TNNC_API void* tnnc_create(const char* proto_path, const char* model_path, int device, int device_id, int precision,
                           int cpu_threads, char* err, int errlen) {
    return tnnc_create_ex(proto_path, model_path, device, device_id, precision, cpu_threads, 0, err, errlen);
}

TNNC_API void tnnc_destroy(void* handle) { delete static_cast<Handle*>(handle); }

// Instance::GetForwardMemorySize / SetForwardMemory (include/tnn/core/instance.h): bytes of blob memory the instance
// needs, and the caller's block of that size on the instance's device.
TNNC_API int64_t tnnc_forward_memory_size(void* handle) {
    Handle* h = static_cast<Handle*>(handle);
    int bytes = 0;   // the reference's interface counts in int: blob memory above 2 GiB cannot be set from outside
    Status st = h->inst->GetForwardMemorySize(bytes);
    if (st != TNN_OK) { h->last_error = st.description(); return -1; }
    return static_cast<int64_t>(bytes);
}

TNNC_API int tnnc_set_forward_memory(void* handle, void* memory) {
    Handle* h = static_cast<Handle*>(handle);
    Status st = h->inst->SetForwardMemory(memory);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st ? (int)st : -1; }
    return 0;
}

// Instance::ShareCommandQueue: `handle` enqueues on `other`'s command queue from now on.
TNNC_API int tnnc_share_command_queue(void* handle, void* other) {
    Handle* h = static_cast<Handle*>(handle);
    Status st = h->inst->ShareCommandQueue(static_cast<Handle*>(other)->inst.get());
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st ? (int)st : -1; }
    return 0;
}

TNNC_API const char* tnnc_last_error(void* handle) { return static_cast<Handle*>(handle)->last_error.c_str(); }

// Copies `n` floats into the named input blob (host blobs: plain copy; CUDA blobs: through the blob converter, as
// TNNTest does, test/test.cc:125-152).  Returns 0 or a TNN status code.
TNNC_API int tnnc_set_input(void* handle, const char* name, const float* data, int64_t n) {
    Handle* h = static_cast<Handle*>(handle);
    BlobMap blobs;
    Status st = h->inst->GetAllInputBlobs(blobs);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st; }
    auto it = blobs.find(name);
    if (it == blobs.end()) { h->last_error = std::string("no input named ") + name; return -1; }
    Blob* blob = it->second;
    const DimsVector dims = blob->GetBlobDesc().dims;
    if (count(dims) != n) { h->last_error = "input element count mismatch"; return -2; }
    if (h->device == DEVICE_CUDA) {
        auto mat = std::make_shared<Mat>(DEVICE_NAIVE, NCHW_FLOAT, dims, const_cast<float*>(data));
        MatConvertParam param;
        st = h->inst->SetInputMat(mat, param, name);
        if (st != TNN_OK) { h->last_error = st.description(); return (int)st; }
    } else {
        BlobHandle bh = blob->GetHandle();
        std::memcpy(static_cast<char*>(bh.base) + bh.bytes_offset, data, static_cast<size_t>(n) * sizeof(float));
    }
    return 0;
}

// The same for an int32 input blob (token ids, segment ids, 0/1 masks: typed graph inputs).
TNNC_API int tnnc_set_input_i32(void* handle, const char* name, const int32_t* data, int64_t n) {
    Handle* h = static_cast<Handle*>(handle);
    BlobMap blobs;
    Status st = h->inst->GetAllInputBlobs(blobs);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st; }
    auto it = blobs.find(name);
    if (it == blobs.end()) { h->last_error = std::string("no input named ") + name; return -1; }
    Blob* blob = it->second;
    const DimsVector dims = blob->GetBlobDesc().dims;
    if (count(dims) != n) { h->last_error = "input element count mismatch"; return -2; }
    if (blob->GetBlobDesc().data_type != DATA_TYPE_INT32) { h->last_error = "input blob is not int32"; return -3; }
    if (h->device == DEVICE_CUDA) {
        auto mat = std::make_shared<Mat>(DEVICE_NAIVE, NC_INT32, dims, const_cast<int32_t*>(data));
        MatConvertParam param;
        st = h->inst->SetInputMat(mat, param, name);
        if (st != TNN_OK) { h->last_error = st.description(); return (int)st; }
    } else {
        BlobHandle bh = blob->GetHandle();
        std::memcpy(static_cast<char*>(bh.base) + bh.bytes_offset, data, static_cast<size_t>(n) * sizeof(int32_t));
    }
    return 0;
}

// Half-precision host data (fp16 bit patterns, or bfloat16 when bf16 != 0) into the named input blob, as a
// RESERVED_FP16_TEST / RESERVED_BFP16_TEST Mat through SetInputMat (every device's converter accepts these).
TNNC_API int tnnc_set_input_half(void* handle, const char* name, const uint16_t* data, int64_t n, int bf16) {
    Handle* h = static_cast<Handle*>(handle);
    BlobMap blobs;
    Status st = h->inst->GetAllInputBlobs(blobs);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st; }
    auto it = blobs.find(name);
    if (it == blobs.end()) { h->last_error = std::string("no input named ") + name; return -1; }
    const DimsVector dims = it->second->GetBlobDesc().dims;
    if (count(dims) != n) { h->last_error = "input element count mismatch"; return -2; }
    auto mat = std::make_shared<Mat>(DEVICE_NAIVE, bf16 ? RESERVED_BFP16_TEST : RESERVED_FP16_TEST, dims,
                                     const_cast<uint16_t*>(data));
    MatConvertParam param;
    st = h->inst->SetInputMat(mat, param, name);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st; }
    return 0;
}

// Output blob -> half-precision host data through GetOutputMat.  Returns the element count or a negative error.
TNNC_API int64_t tnnc_get_output_half(void* handle, const char* name, uint16_t* dst, int64_t capacity, int bf16) {
    Handle* h = static_cast<Handle*>(handle);
    BlobMap blobs;
    Status st = h->inst->GetAllOutputBlobs(blobs);
    if (st != TNN_OK) { h->last_error = st.description(); return -1; }
    auto it = (name && name[0]) ? blobs.find(name) : blobs.begin();
    if (it == blobs.end()) { h->last_error = "no such output"; return -1; }
    const int64_t n = count(it->second->GetBlobDesc().dims);
    if (!dst) return n;
    if (capacity < n) { h->last_error = "output buffer too small"; return -2; }
    std::shared_ptr<Mat> mat;
    MatConvertParam param;
    st = h->inst->GetOutputMat(mat, param, it->first, DEVICE_NAIVE, bf16 ? RESERVED_BFP16_TEST : RESERVED_FP16_TEST);
    if (st != TNN_OK || !mat) { h->last_error = st.description(); return -3; }
    std::memcpy(dst, mat->GetData(), static_cast<size_t>(n) * sizeof(uint16_t));
    return n;
}

// Device-resident Mats (zero host copies): `kind` 0 = NCHW_FLOAT, 1 = RESERVED_FP16_TEST, 2 = RESERVED_BFP16_TEST,
// 3 = NC_INT32.  The pointer is device memory of the instance's GPU; the converter's branch for
// image.GetDeviceType() == DEVICE_CUDA (reference: source/tnn/device/cuda/cuda_blob_converter.cc:140-149) copies or
// converts device to device on the instance's stream.
TNNC_API int tnnc_set_input_device(void* handle, const char* name, void* device_ptr, int64_t n, int kind) {
    Handle* h = static_cast<Handle*>(handle);
    MatType mt;
    if (h->device != DEVICE_CUDA || !mat_type_of(kind, &mt)) { h->last_error = "device Mats need DEVICE_CUDA and a valid kind"; return -4; }
    BlobMap blobs;
    Status st = h->inst->GetAllInputBlobs(blobs);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st; }
    auto it = blobs.find(name);
    if (it == blobs.end()) { h->last_error = std::string("no input named ") + name; return -1; }
    const DimsVector dims = it->second->GetBlobDesc().dims;
    if (count(dims) != n) { h->last_error = "input element count mismatch"; return -2; }
    auto mat = std::make_shared<Mat>(DEVICE_CUDA, mt, dims, device_ptr);
    MatConvertParam param;
    st = h->inst->SetInputMat(mat, param, name);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st; }
    return 0;
}

// The named output as a device Mat of the requested kind.  *device_ptr receives the Mat's device pointer, owned by the
// instance and valid until the next call for this output; returns the element count or a negative error.
TNNC_API int64_t tnnc_get_output_device(void* handle, const char* name, int kind, void** device_ptr) {
    Handle* h = static_cast<Handle*>(handle);
    MatType mt;
    if (h->device != DEVICE_CUDA || !mat_type_of(kind, &mt) || !device_ptr) { h->last_error = "device Mats need DEVICE_CUDA and a valid kind"; return -4; }
    BlobMap blobs;
    Status st = h->inst->GetAllOutputBlobs(blobs);
    if (st != TNN_OK) { h->last_error = st.description(); return -1; }
    auto it = (name && name[0]) ? blobs.find(name) : blobs.begin();
    if (it == blobs.end()) { h->last_error = "no such output"; return -1; }
    const int64_t n = count(it->second->GetBlobDesc().dims);
    std::shared_ptr<Mat> mat;
    MatConvertParam param;
    st = h->inst->GetOutputMat(mat, param, it->first, DEVICE_CUDA, mt);
    if (st != TNN_OK || !mat) { h->last_error = st.description(); return -3; }
    *device_ptr = mat->GetData();
    return n;
}



// ---- the reference benchmark's own loop, piece by piece (test/test.cc:125-152): BlobConverter::ConvertFromMatAsync on
// the input blobs, Instance::ForwardAsync, BlobConverter::ConvertToMat on the output blobs, all on the instance's
// command queue.  `kind`: 0 = NCHW_FLOAT, 1 = RESERVED_FP16_TEST, 2 = RESERVED_BFP16_TEST, 3 = NC_INT32.  `host` is the
// caller's buffer (pageable or page-locked); it is wrapped in a Mat, never copied by the shim.
static Status io_objects(Handle* h, const char* name, bool input, void* host, int64_t n, int kind,
                         std::shared_ptr<BlobConverter>* conv, std::shared_ptr<Mat>* mat) {
    MatType mt;
    if (!mat_type_of(kind, &mt)) return Status(TNNERR_PARAM_ERR, "bad Mat kind");
    BlobMap blobs;
    Status st = input ? h->inst->GetAllInputBlobs(blobs) : h->inst->GetAllOutputBlobs(blobs);
    if (st != TNN_OK) return st;
    auto it = (name && name[0]) ? blobs.find(name) : blobs.begin();
    if (it == blobs.end()) return Status(TNNERR_PARAM_ERR, std::string("no blob named ") + (name ? name : ""));
    const DimsVector dims = it->second->GetBlobDesc().dims;
    if (count(dims) != n) return Status(TNNERR_PARAM_ERR, "element count mismatch");
    const std::string key = std::string(input ? "i:" : "o:") + it->first;
    auto c = h->converters.find(key);
    if (c == h->converters.end()) c = h->converters.emplace(key, std::make_shared<BlobConverter>(it->second)).first;
    *conv = c->second;
    auto m = h->mats.find(key);
    if (m == h->mats.end() || m->second->GetData() != host || m->second->GetMatType() != mt ||
        !DimsVectorUtils::Equal(m->second->GetDims(), dims)) {
        h->mats[key] = std::make_shared<Mat>(DEVICE_NAIVE, mt, dims, host);
        m = h->mats.find(key);
    }
    *mat = m->second;
    return TNN_OK;
}

TNNC_API int tnnc_from_mat_async(void* handle, const char* name, void* host, int64_t n, int kind) {
    Handle* h = static_cast<Handle*>(handle);
    std::shared_ptr<BlobConverter> conv;
    std::shared_ptr<Mat> mat;
    Status st = io_objects(h, name, true, host, n, kind, &conv, &mat);
    void* q = nullptr;
    if (st == TNN_OK) st = h->inst->GetCommandQueue(&q);
    if (st == TNN_OK) st = conv->ConvertFromMatAsync(*mat, MatConvertParam(), q);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st ? (int)st : -1; }
    return 0;
}

TNNC_API int tnnc_to_mat(void* handle, const char* name, void* host, int64_t n, int kind, int blocking) {
    Handle* h = static_cast<Handle*>(handle);
    std::shared_ptr<BlobConverter> conv;
    std::shared_ptr<Mat> mat;
    Status st = io_objects(h, name, false, host, n, kind, &conv, &mat);
    void* q = nullptr;
    if (st == TNN_OK) st = h->inst->GetCommandQueue(&q);
    if (st == TNN_OK) st = blocking ? conv->ConvertToMat(*mat, MatConvertParam(), q)
                                    : conv->ConvertToMatAsync(*mat, MatConvertParam(), q);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st ? (int)st : -1; }
    return 0;
}

TNNC_API int tnnc_forward_async(void* handle) {
    Handle* h = static_cast<Handle*>(handle);
    Status st = h->inst->ForwardAsync(nullptr);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st; }
    return 0;
}

TNNC_API void* tnnc_command_queue(void* handle) {
    Handle* h = static_cast<Handle*>(handle);
    void* q = nullptr;
    return h->inst->GetCommandQueue(&q) == TNN_OK ? q : nullptr;
}

// The whole loop, natively, over `n_handles` instances taken round-robin (1 = exactly the reference benchmark's loop;
// 2 = the usual serving arrangement, two instances of one model on one GPU, so that one instance's copies run while
// the other computes).  Per step: every input of the instance whose turn it is goes ConvertFromMatAsync, then
// ForwardAsync; the instance that was issued n_handles - 1 steps earlier is drained with a blocking ConvertToMat of
// every output.  inputs / outputs: n_handles x n_in (n_out) records, instance-major.  Runs `warmup` untimed steps, then
// `steps` timed ones (drained to the last); returns the wall time of the timed steps in milliseconds, negative on error.
struct TnncIo {
    const char* name;
    void* host;
    int64_t n;
    int32_t kind;
    int32_t reserved_;
};

TNNC_API double tnnc_run_pipeline(void** handles, int n_handles, const TnncIo* inputs, int n_in, const TnncIo* outputs,
                                  int n_out, int warmup, int steps) {
    if (!handles || n_handles <= 0 || n_in <= 0 || n_out <= 0 || steps <= 0) return -1.0;
    std::vector<Handle*> hs(n_handles);
    for (int k = 0; k < n_handles; ++k) hs[k] = static_cast<Handle*>(handles[k]);
    struct Bound { std::shared_ptr<BlobConverter> conv; std::shared_ptr<Mat> mat; };
    std::vector<std::vector<Bound>> in(n_handles), out(n_handles);
    std::vector<void*> queue(n_handles, nullptr);
    for (int k = 0; k < n_handles; ++k) {
        if (hs[k]->inst->GetCommandQueue(&queue[k]) != TNN_OK) return -2.0;
        for (int i = 0; i < n_in; ++i) {
            const TnncIo& io = inputs[k * n_in + i];
            Bound b;
            Status st = io_objects(hs[k], io.name, true, io.host, io.n, io.kind, &b.conv, &b.mat);
            if (st != TNN_OK) { hs[k]->last_error = st.description(); return -3.0; }
            in[k].push_back(b);
        }
        for (int i = 0; i < n_out; ++i) {
            const TnncIo& io = outputs[k * n_out + i];
            Bound b;
            Status st = io_objects(hs[k], io.name, false, io.host, io.n, io.kind, &b.conv, &b.mat);
            if (st != TNN_OK) { hs[k]->last_error = st.description(); return -3.0; }
            out[k].push_back(b);
        }
    }
    MatConvertParam param;
    auto issue = [&](int k) -> bool {
        for (auto& b : in[k])
            if (b.conv->ConvertFromMatAsync(*b.mat, param, queue[k]) != TNN_OK) return false;
        Status st = hs[k]->inst->ForwardAsync(nullptr);
        if (st != TNN_OK) { hs[k]->last_error = st.description(); return false; }
        return true;
    };
    auto drain = [&](int k) -> bool {
        for (auto& b : out[k]) {
            Status st = b.conv->ConvertToMat(*b.mat, param, queue[k]);
            if (st != TNN_OK) { hs[k]->last_error = st.description(); return false; }
        }
        return true;
    };
    auto run = [&](int count) -> bool {
        for (int s = 0; s < count; ++s) {
            if (!issue(s % n_handles)) return false;
            if (s >= n_handles - 1 && !drain((s - (n_handles - 1)) % n_handles)) return false;
        }
        for (int s = count > n_handles - 1 ? count - (n_handles - 1) : 0; s < count; ++s)
            if (!drain(s % n_handles)) return false;
        return true;
    };
    if (warmup > 0 && !run(warmup)) return -4.0;
    auto t0 = std::chrono::steady_clock::now();
    if (!run(steps)) return -5.0;
    auto t1 = std::chrono::steady_clock::now();
    return std::chrono::duration<double, std::milli>(t1 - t0).count();
}

// Instance::Reshape: new dims for `n_inputs` named input blobs at once (dims_flat holds them back to back, nds[i] dims
// each).  The shapes must stay within those the instance was created with (TNN sizes blob memory at Init).
TNNC_API int tnnc_reshape(void* handle, int n_inputs, const char* const* names, const int* dims_flat, const int* nds) {
    Handle* h = static_cast<Handle*>(handle);
    if (!names || !dims_flat || !nds || n_inputs <= 0) { h->last_error = "bad arguments"; return -1; }
    InputShapesMap shapes;
    const int* p = dims_flat;
    for (int i = 0; i < n_inputs; ++i) {
        shapes[names[i]] = DimsVector(p, p + nds[i]);
        p += nds[i];
    }
    Status st = h->inst->Reshape(shapes);
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st ? (int)st : -1; }
    return 0;
}

// Instance::StartProfile / FinishProfile (include/tnn/core/instance.h:103-109), which exist only in a TNN_PROFILE
// build of the host framework.  tnnc_finish_profile copies the per-layer table into `buf` and returns its length;
// both return -1 in a build without the switch.
TNNC_API int tnnc_start_profile(void* handle) {
#if TNN_PROFILE
    static_cast<Handle*>(handle)->inst->StartProfile();
    return 0;
#else
    (void)handle;
    return -1;
#endif
}

TNNC_API int64_t tnnc_finish_profile(void* handle, char* buf, int64_t cap) {
#if TNN_PROFILE
    const std::string s = static_cast<Handle*>(handle)->inst->FinishProfile(false);
    if (buf && cap > 0) {
        const size_t n = s.size() < static_cast<size_t>(cap - 1) ? s.size() : static_cast<size_t>(cap - 1);
        std::memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    return static_cast<int64_t>(s.size());
#else
    (void)handle; (void)buf; (void)cap;
    return -1;
#endif
}

TNNC_API int tnnc_forward(void* handle) {
    Handle* h = static_cast<Handle*>(handle);
    Status st = h->inst->Forward();
    if (st != TNN_OK) { h->last_error = st.description(); return (int)st; }
    return 0;
}

// Runs Forward `iters` times and returns the mean wall time per call in milliseconds (negative on error).
TNNC_API double tnnc_time_forward(void* handle, int warmup, int iters) {
    Handle* h = static_cast<Handle*>(handle);
    for (int i = 0; i < warmup; ++i)
        if (h->inst->Forward() != TNN_OK) return -1.0;
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < iters; ++i)
        if (h->inst->Forward() != TNN_OK) return -1.0;
    auto t1 = std::chrono::steady_clock::now();
    return std::chrono::duration<double, std::milli>(t1 - t0).count() / (iters > 0 ? iters : 1);
}

// Output blob -> host floats.  dims_out receives up to 8 dims; returns the element count, or a negative error.
TNNC_API int64_t tnnc_get_output(void* handle, const char* name, float* dst, int64_t capacity, int* dims_out,
                                 int* ndims_out) {
    Handle* h = static_cast<Handle*>(handle);
    BlobMap blobs;
    Status st = h->inst->GetAllOutputBlobs(blobs);
    if (st != TNN_OK) { h->last_error = st.description(); return -1; }
    auto it = (name && name[0]) ? blobs.find(name) : blobs.begin();
    if (it == blobs.end()) { h->last_error = "no such output"; return -1; }
    Blob* blob = it->second;
    const DimsVector dims = blob->GetBlobDesc().dims;
    const int64_t n = count(dims);
    if (ndims_out) *ndims_out = static_cast<int>(dims.size());
    if (dims_out)
        for (size_t i = 0; i < dims.size() && i < 8; ++i) dims_out[i] = dims[i];
    if (!dst) return n;
    if (capacity < n) { h->last_error = "output buffer too small"; return -2; }
    if (h->device == DEVICE_CUDA) {
        std::shared_ptr<Mat> mat;
        MatConvertParam param;
        st = h->inst->GetOutputMat(mat, param, it->first, DEVICE_NAIVE, NCHW_FLOAT);
        if (st != TNN_OK || !mat) { h->last_error = st.description(); return -3; }
        std::memcpy(dst, mat->GetData(), static_cast<size_t>(n) * sizeof(float));
    } else {
        BlobHandle bh = blob->GetHandle();
        std::memcpy(dst, static_cast<char*>(bh.base) + bh.bytes_offset, static_cast<size_t>(n) * sizeof(float));
    }
    return n;
}

}  // extern "C"
