// Per-instance CUDA context: one stream on `device_id`, a workspace, and the replay of a Forward as a CUDA graph.
// Replaces the reference's CudaContext (source/tnn/device/cuda/cuda_context.{h,cc}) without its cuDNN / cuBLAS handles
// and without re-allocating the workspace inside Forward (cuda_context.cc:137-145): accs state their need in
// Init/Reshape through ReserveWorkspace, the kv_len array of the attention layers is reserved at Setup, and nothing is
// allocated while a Forward is in flight.
//
// CUDA-graph replay.  TNN's executor calls every layer acc once per Forward (source/tnn/core/default_network.cc:
// 558-635); a fused BERT-base encoder is 86 launches of 10-40 us kernels, which a host thread cannot enqueue as fast as
// the GPU runs them.  The context therefore turns a Forward into one graph launch:
//   Forward 1 after Init / Reshape  runs eagerly (first launches set kernel attributes and load modules);
//   Forward 2                       runs with the stream in capture: the accs launch as usual, the context records
//                                   which acc ran on which blobs, ends the capture in OnInstanceForwardEnd, instantiates
//                                   the graph and launches it;
//   Forward 3, 4, ...               the accs' Forward returns at once and OnInstanceForwardEnd launches the graph —
//                                   as long as every blob the accs touched still has the handle it had at capture
//                                   (checked each Forward; a Reshape, or a caller that re-binds a blob, drops the graph
//                                   and the sequence starts over).
// If the capture or a graph launch fails, the recorded acc calls are run eagerly in its place: a Forward never loses
// its work to the graph path.  TNN_B200_GRAPH=0 in the environment turns the replay off.
#ifndef TNN_B200_CUDA_CONTEXT_H_
#define TNN_B200_CUDA_CONTEXT_H_

#include <cuda_runtime.h>

#include <map>
#include <string>
#include <vector>

#include "tnn/core/blob.h"
#include "tnn/core/context.h"

namespace TNN_NS {

class B200CudaLayerAcc;

class B200CudaContext : public Context {
public:
    ~B200CudaContext();
    Status Setup(int device_id);

    virtual Status LoadLibrary(std::vector<std::string> path) override;
    virtual Status GetCommandQueue(void** command_queue) override;
    virtual Status ShareCommandQueue(Context* context) override;
    virtual Status OnInstanceForwardBegin() override;
    virtual Status OnInstanceForwardEnd() override;
    virtual Status OnInstanceReshapeBegin() override;
    virtual Status Synchronize() override;

    cudaStream_t GetStream() const { return stream_; }
    int GetDeviceId() const { return device_id_; }

    // The context that owns `command_queue` (a cudaStream_t handed out by GetCommandQueue), or nullptr.  The blob
    // converters only receive the command queue; this is how they reach the instance's status word.
    static B200CudaContext* FromCommandQueue(void* command_queue);

    // Shared scratch used by one layer at a time (layers of an instance run in order on one stream).  Grows only
    // here, i.e. at Init/Reshape time; returns TNNERR_OUTOFMEMORY instead of aborting.
    Status ReserveWorkspace(size_t bytes);
    void* GetWorkspace() const { return workspace_; }
    size_t GetWorkspaceSize() const { return workspace_size_; }

    // kv_len of an attention mask, computed once per Forward and shared by the attention layers of the instance.
    // Returns a device pointer to B int32 values (nullptr on failure).  The array is reserved at Setup
    // (kKvLenCapacity entries, the attention kernels' own batch limit), never in Forward.
    static const int kKvLenCapacity = 65536;
    const int* GetKvLen(const float* mask, int batch, int seq, float exclude_below, Status* status);

    // Half-precision copies of fp32 blobs made during the current Forward (the graph input feeds the first layer's
    // projection and, as the residual, its output projection): the second layer that needs one reuses the first's.
    const void* FindConverted(const void* src, int dtype, int64_t count) const;
    void NoteConverted(const void* src, int dtype, int64_t count, const void* dst);

    // ---- graph replay, driven by B200CudaLayerAcc::Forward
    // True while a captured graph stands in for the accs' launches: the acc returns without launching.
    bool Replaying() const { return mode_ == kReplay; }
    // Called by every acc before it launches (eager and capture mode): remembers the call for the signature check and
    // for the eager re-run.
    void RecordCall(B200CudaLayerAcc* acc, const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs);
    // Counters for tests and the benchmark: {eager Forwards, captures, graph launches, capture failures}.
    void GraphCounters(uint64_t out[4]) const;

    // After the stream has been synchronised by the caller: the device status word of the last Forward (a bounded
    // device-side wait that ran out, an embedding index outside its table) as a Status; clears it.
    Status CheckStatusAfterSync();

private:
    enum Mode { kEager, kCapture, kReplay };
    struct Call {
        B200CudaLayerAcc* acc;
        std::vector<Blob*> inputs, outputs;
        std::vector<void*> handles;   // device pointers of inputs then outputs at record time
    };
    void AbortCapture();
    void DropGraph();
    bool SignatureMatches() const;
    Status RunCallsEagerly();

    cudaStream_t stream_ = nullptr;
    bool own_stream_     = false;
    int device_id_       = 0;
    void* workspace_     = nullptr;
    size_t workspace_size_ = 0;

    int* kv_len_buf_        = nullptr;
    const float* kv_mask_   = nullptr;   // mask the cached kv_len belongs to (valid for the current Forward only)
    int kv_batch_ = 0, kv_seq_ = 0;
    unsigned long long forward_id_ = 0, kv_forward_id_ = ~0ull;

    struct Converted {
        const void* src;
        const void* dst;
        int64_t count;
        int dtype;
        unsigned long long forward_id;
    };
    Converted converted_[4] = {};
    int converted_next_ = 0;

    unsigned int* host_status_ = nullptr;   // pinned; receives the device status word at the end of every Forward
    Status sticky_error_       = TNN_OK;    // reported by the next OnInstanceForwardBegin (Forward drops Synchronize's)

    bool graph_enabled_ = true;
    Mode mode_          = kEager;
    std::vector<Call> calls_;               // the acc calls of the Forward being recorded / captured
    std::vector<Call> graph_calls_;         // the acc calls the instantiated graph stands for
    cudaGraphExec_t graph_exec_ = nullptr;
    int eager_since_change_     = 0;        // eager Forwards since Init / Reshape / a dropped graph
    int capture_failures_       = 0;
    uint64_t n_eager_ = 0, n_captures_ = 0, n_launches_ = 0, n_failures_ = 0;
};

}  // namespace TNN_NS
#endif
