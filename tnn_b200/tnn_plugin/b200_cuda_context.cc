#include "b200_cuda_context.h"

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "b200_cuda_device.h"
#include "b200_cuda_layer_acc.h"
#include "b200_plugin_common.h"

namespace TNN_NS {

namespace {
std::mutex g_ctx_mutex;
std::unordered_map<void*, B200CudaContext*>& ContextsByStream() {
    static auto* m = new std::unordered_map<void*, B200CudaContext*>();
    return *m;
}
void* DevicePtrOf(Blob* b) {
    BlobHandle h = b->GetHandle();
    return static_cast<char*>(h.base) + h.bytes_offset;
}
}  // namespace

B200CudaContext* B200CudaContext::FromCommandQueue(void* command_queue) {
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    auto& m = ContextsByStream();
    auto it = m.find(command_queue);
    return it == m.end() ? nullptr : it->second;
}

B200CudaContext::~B200CudaContext() {
    cudaSetDevice(device_id_);
    AbortCapture();
    if (stream_) cudaStreamSynchronize(stream_);
    DropGraph();
    {
        std::lock_guard<std::mutex> lock(g_ctx_mutex);
        auto& m = ContextsByStream();
        auto it = m.find(stream_);
        if (it != m.end() && it->second == this) m.erase(it);
    }
    auto* dev = dynamic_cast<B200CudaDevice*>(GetDevice(DEVICE_CUDA));
    if (dev) {
        if (workspace_) dev->Free(workspace_);
        if (kv_len_buf_) dev->Free(kv_len_buf_);
    }
    if (host_status_) B200CudaDevice::FreeHost(host_status_);
    if (own_stream_ && stream_) cudaStreamDestroy(stream_);
    cudaGetLastError();
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
    auto* dev = dynamic_cast<B200CudaDevice*>(GetDevice(DEVICE_CUDA));
    if (!dev) return Status(TNNERR_DEVICE_NOT_SUPPORT, "DEVICE_CUDA is not served by tnn_b200");
    void* p = nullptr;
    RETURN_ON_NEQ(dev->Allocate(&p, sizeof(int) * static_cast<size_t>(kKvLenCapacity)), TNN_OK);
    kv_len_buf_ = static_cast<int*>(p);
    void* hs = nullptr;
    RETURN_ON_NEQ(B200CudaDevice::AllocateHost(&hs, 64), TNN_OK);
    host_status_  = static_cast<unsigned int*>(hs);
    *host_status_ = 0;
    const char* e  = std::getenv("TNN_B200_GRAPH");
    graph_enabled_ = !(e != nullptr && e[0] == '0');
    {
        std::lock_guard<std::mutex> lock(g_ctx_mutex);
        ContextsByStream()[stream_] = this;
    }
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
    AbortCapture();
    DropGraph();
    {
        std::lock_guard<std::mutex> lock(g_ctx_mutex);
        auto& m = ContextsByStream();
        auto it = m.find(stream_);
        if (it != m.end() && it->second == this) m.erase(it);
    }
    if (own_stream_ && stream_) cudaStreamDestroy(stream_);
    own_stream_ = false;
    stream_     = other->stream_;
    // Two instances now enqueue on one stream; a capture by one would swallow the other's work, so this context
    // keeps launching eagerly (the owner of the stream may still replay: a graph launch is an ordinary stream item).
    graph_enabled_ = false;
    return TNN_OK;
}

// ------------------------------------------------------------------------------------------------ graph replay
void B200CudaContext::AbortCapture() {
    if (mode_ != kCapture) return;
    cudaGraph_t g = nullptr;
    cudaStreamEndCapture(stream_, &g);
    if (g) cudaGraphDestroy(g);
    cudaGetLastError();
    mode_ = kEager;
    calls_.clear();
}

void B200CudaContext::DropGraph() {
    if (graph_exec_) {
        cudaGraphExecDestroy(graph_exec_);
        graph_exec_ = nullptr;
    }
    graph_calls_.clear();
    eager_since_change_ = 0;
}

bool B200CudaContext::SignatureMatches() const {
    for (const Call& c : graph_calls_) {
        size_t i = 0;
        for (Blob* b : c.inputs)
            if (DevicePtrOf(b) != c.handles[i++]) return false;
        for (Blob* b : c.outputs)
            if (DevicePtrOf(b) != c.handles[i++]) return false;
    }
    return true;
}

void B200CudaContext::RecordCall(B200CudaLayerAcc* acc, const std::vector<Blob*>& inputs,
                                 const std::vector<Blob*>& outputs) {
    if (!graph_enabled_) return;
    Call c;
    c.acc     = acc;
    c.inputs  = inputs;
    c.outputs = outputs;
    for (Blob* b : inputs) c.handles.push_back(DevicePtrOf(b));
    for (Blob* b : outputs) c.handles.push_back(DevicePtrOf(b));
    calls_.push_back(std::move(c));
}

Status B200CudaContext::RunCallsEagerly() {
    // `calls_` holds what the executor asked for during this Forward, in order.  What the accs cached for this Forward
    // (kv_len, converted inputs) was recorded into the failed capture, never executed: a new id voids those caches.
    ++forward_id_;
    std::vector<Call> todo;
    todo.swap(calls_);
    for (Call& c : todo) RETURN_ON_NEQ(c.acc->DoForward(c.inputs, c.outputs), TNN_OK);
    return TNN_OK;
}

Status B200CudaContext::OnInstanceForwardBegin() {
    cudaSetDevice(device_id_);
    AbortCapture();   // a Forward that failed half-way never reached OnInstanceForwardEnd
    ++forward_id_;
    if (sticky_error_ != TNN_OK) {
        Status st     = sticky_error_;
        sticky_error_ = TNN_OK;
        return st;
    }
    mode_ = kEager;
    calls_.clear();
    bool profiling = false;
#if TNN_PROFILE
    profiling = profile_layer;
#endif
    if (!graph_enabled_ || profiling) return TNN_OK;
    if (graph_exec_) {
        if (SignatureMatches()) {
            mode_ = kReplay;
            return TNN_OK;
        }
        DropGraph();
    }
    if (eager_since_change_ >= 1 && capture_failures_ < 2) {
        if (cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
            mode_ = kCapture;
        } else {
            cudaGetLastError();
            ++capture_failures_;
            ++n_failures_;
        }
    }
    return TNN_OK;
}

Status B200CudaContext::OnInstanceForwardEnd() {
    Status st = TNN_OK;
    if (mode_ == kCapture) {
        cudaGraph_t graph    = nullptr;
        cudaGraphExec_t exec = nullptr;
        const bool ended     = cudaStreamEndCapture(stream_, &graph) == cudaSuccess && graph != nullptr;
        mode_                = kEager;
        bool launched        = false;
        if (ended && cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess && exec != nullptr) {
            if (cudaGraphLaunch(exec, stream_) == cudaSuccess) {
                launched    = true;
                graph_exec_ = exec;
                graph_calls_.swap(calls_);
                calls_.clear();
                ++n_captures_;
                ++n_launches_;
            } else {
                cudaGraphExecDestroy(exec);
            }
        }
        if (graph) cudaGraphDestroy(graph);
        if (!launched) {
            cudaGetLastError();
            ++capture_failures_;
            ++n_failures_;
            st = RunCallsEagerly();   // the capture swallowed this Forward's launches: issue them for real
            ++n_eager_;
        }
    } else if (mode_ == kReplay) {
        mode_ = kEager;
        if (cudaGraphLaunch(graph_exec_, stream_) == cudaSuccess) {
            ++n_launches_;
        } else {
            cudaGetLastError();
            ++n_failures_;
            calls_ = graph_calls_;
            DropGraph();
            st = RunCallsEagerly();
            ++n_eager_;
        }
    } else {
        ++n_eager_;
        ++eager_since_change_;
        calls_.clear();
    }
    // The device status word follows the Forward down the stream into pinned memory; whoever synchronises the stream
    // next (Synchronize, a blocking blob conversion) looks at it without another round trip.
    if (host_status_) b200_device_status_async(host_status_, stream_);
    return st;
}

Status B200CudaContext::OnInstanceReshapeBegin() {
    cudaSetDevice(device_id_);
    AbortCapture();
    // blob dims and handles are about to change: whatever was captured is void
    if (stream_) cudaStreamSynchronize(stream_);
    DropGraph();
    capture_failures_ = 0;
    return TNN_OK;
}

void B200CudaContext::GraphCounters(uint64_t out[4]) const {
    out[0] = n_eager_;
    out[1] = n_captures_;
    out[2] = n_launches_;
    out[3] = n_failures_;
}

Status B200CudaContext::CheckStatusAfterSync() {
    if (!host_status_ || *host_status_ == 0) return TNN_OK;
    *host_status_ = 0;
    cudaSetDevice(device_id_);
    const int rc = b200_device_status();   // reads and clears the device word (blocking; error path only)
    return B200ToStatus(rc != B200_OK ? rc : B200_ERR_DEVICE_TIMEOUT, "device status");
}

Status B200CudaContext::Synchronize() {
    AbortCapture();
    if (cudaStreamSynchronize(stream_) != cudaSuccess) {
        cudaGetLastError();
        sticky_error_ = Status(TNNERR_CUDA_SYNC_ERROR, "stream synchronize failed");
        return sticky_error_;
    }
    // A bounded device-side wait that ran out is reported here, after the stream has drained.  DefaultNetwork::Forward
    // drops this return value (source/tnn/core/default_network.cc:632-633), so the error is also kept for the next
    // OnInstanceForwardBegin, whose status Forward does return.
    Status st = CheckStatusAfterSync();
    if (st != TNN_OK) sticky_error_ = st;
    return st;
}

const void* B200CudaContext::FindConverted(const void* src, int dtype, int64_t count) const {
    for (const Converted& c : converted_)
        if (c.forward_id == forward_id_ && c.src == src && c.dtype == dtype && c.count == count && c.dst) return c.dst;
    return nullptr;
}

void B200CudaContext::NoteConverted(const void* src, int dtype, int64_t count, const void* dst) {
    converted_[converted_next_] = Converted{src, dst, count, dtype, forward_id_};
    converted_next_             = (converted_next_ + 1) % 4;
}

Status B200CudaContext::ReserveWorkspace(size_t bytes) {
    if (bytes <= workspace_size_) return TNN_OK;
    cudaSetDevice(device_id_);
    cudaStreamSynchronize(stream_);   // Init/Reshape time only: nothing of this instance may still use the old block
    auto* dev = dynamic_cast<B200CudaDevice*>(GetDevice(DEVICE_CUDA));
    if (!dev) return Status(TNNERR_DEVICE_NOT_SUPPORT, "DEVICE_CUDA is not served by tnn_b200");
    void* p = nullptr;
    RETURN_ON_NEQ(dev->Allocate(&p, bytes), TNN_OK);
    if (workspace_) dev->Free(workspace_);
    workspace_      = p;
    workspace_size_ = bytes;
    return TNN_OK;
}

const int* B200CudaContext::GetKvLen(const float* mask, int batch, int seq, float exclude_below, Status* status) {
    *status = TNN_OK;
    if (kv_forward_id_ == forward_id_ && kv_mask_ == mask && kv_batch_ == batch && kv_seq_ == seq) return kv_len_buf_;
    if (batch > kKvLenCapacity || kv_len_buf_ == nullptr) {
        *status = Status(TNNERR_PARAM_ERR, "attention batch exceeds the kv_len array reserved at set-up");
        return nullptr;
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
