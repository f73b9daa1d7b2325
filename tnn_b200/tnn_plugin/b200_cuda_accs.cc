// DEVICE_CUDA layer accs of the fused encoder graph: FusedLinear, FusedAttention and LayerNorm.  Each DoForward is one
// launch through the kernel library's C ABI on the context's stream (plus a conversion launch where an fp32 blob
// enters the half-precision region).  Registered in the device's acc registry like the reference's accs
// (REGISTER_CUDA_ACC, source/tnn/device/cuda/acc/cuda_layer_acc.h:105-107).
#include <cstring>

#include "b200_cuda_layer_acc.h"
#include "tnn/utils/data_type_utils.h"
#include "tnn/utils/dims_utils.h"

namespace TNN_NS {

namespace {

int64_t Rows(const DimsVector& dims) {
    int64_t n = 1;
    for (size_t i = 0; i + 1 < dims.size(); ++i) n *= dims[i];
    return n;
}

}  // namespace

// ================================================================= FusedLinear
B200_DECLARE_CUDA_ACC(FusedLinear)
    // `src` as a half-precision [rows, cols] device pointer: the blob itself when it already has the compute dtype,
    // otherwise a conversion into the acc's staging buffer.
    Status AsCompute(Blob* src, void* staging, int64_t count, const void** out);

    void* w_packed_   = nullptr;   // [N, K] compute dtype
    float* bias_      = nullptr;   // [N] fp32
    void* x_staging_  = nullptr;   // conversion buffers for fp32 inputs (first layer of the graph)
    size_t x_cap_     = 0;
    void* r_staging_  = nullptr;
    size_t r_cap_     = 0;
    int64_t K_ = 0, N_ = 0;
};

Status B200CudaFusedLinearLayerAcc::Init(Context* context, LayerParam* param, LayerResource* resource,
                                         const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    RETURN_ON_NEQ(B200CudaLayerAcc::Init(context, param, resource, inputs, outputs), TNN_OK);
    auto* p = dynamic_cast<FusedLinearLayerParam*>(param);
    auto* r = dynamic_cast<FusedLinearLayerResource*>(resource);
    if (!p || !r || r->weights.empty() || r->weights.size() != r->biases.size())
        return Status(TNNERR_PARAM_ERR, "FusedLinear: param/resource missing");
    K_ = p->in_features;
    N_ = p->out_features;
    cudaStream_t stream = context_->GetStream();
    const size_t es = 2;
    size_t cap = 0;
    RETURN_ON_NEQ(EnsureBuffer(&w_packed_, &cap, static_cast<size_t>(N_) * K_ * es), TNN_OK);
    cap = 0;
    void* bias = nullptr;
    RETURN_ON_NEQ(EnsureBuffer(&bias, &cap, static_cast<size_t>(N_) * sizeof(float)), TNN_OK);
    bias_ = static_cast<float*>(bias);

    // Upload each fp32 [K, N_i] weight and pack it to [N_i, K] half precision at row offset n0 of the merged operand.
    // The host RawBuffers are only read: they are shared with every other instance of the model.
    int64_t n0 = 0;
    for (size_t i = 0; i < r->weights.size(); ++i) {
        RawBuffer& w = r->weights[i];
        RawBuffer& b = r->biases[i];
        const DimsVector wd = w.GetBufferDims();
        if (w.GetDataType() != DATA_TYPE_FLOAT || wd.size() != 2 || wd[0] != K_)
            return Status(TNNERR_PARAM_ERR, "FusedLinear: weight must be fp32 [K, N]");
        const int64_t Ni = wd[1];
        if (b.GetDataType() != DATA_TYPE_FLOAT || b.GetDataCount() != Ni)
            return Status(TNNERR_PARAM_ERR, "FusedLinear: bias must be fp32 [N]");
        void* tmp = nullptr;
        RETURN_ON_NEQ(device_->Allocate(&tmp, static_cast<size_t>(K_) * Ni * sizeof(float)), TNN_OK);
        Status st = TNN_OK;
        if (cudaMemcpyAsync(tmp, w.force_to<float*>(), static_cast<size_t>(K_) * Ni * sizeof(float),
                            cudaMemcpyHostToDevice, stream) != cudaSuccess ||
            cudaMemcpyAsync(bias_ + n0, b.force_to<float*>(), static_cast<size_t>(Ni) * sizeof(float),
                            cudaMemcpyHostToDevice, stream) != cudaSuccess) {
            cudaGetLastError();
            st = Status(TNNERR_CUDA_MEMCPY_ERROR, "FusedLinear: weight upload failed");
        }
        if (st == TNN_OK)
            st = B200ToStatus(b200_pack_weight(static_cast<const float*>(tmp), K_, Ni, Ni,
                                               static_cast<char*>(w_packed_) + n0 * K_ * es, K_, p->compute_dtype, stream),
                              "b200_pack_weight");
        cudaStreamSynchronize(stream);   // Init time: the staging copy is released right away
        device_->Free(tmp);
        RETURN_ON_NEQ(st, TNN_OK);
        n0 += Ni;
    }
    if (n0 != N_) return Status(TNNERR_PARAM_ERR, "FusedLinear: merged weight widths do not add up to out_features");
    return Reshape(inputs, outputs);
}

Status B200CudaFusedLinearLayerAcc::Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    auto* p = dynamic_cast<FusedLinearLayerParam*>(param_);
    const int64_t rows = Rows(inputs[0]->GetBlobDesc().dims);
    // Staging for inputs that are not in the compute dtype yet (sized here, never in Forward).
    if (B200DataType(inputs[0]->GetBlobDesc().data_type) != p->compute_dtype)
        RETURN_ON_NEQ(EnsureBuffer(&x_staging_, &x_cap_, static_cast<size_t>(rows) * K_ * 2), TNN_OK);
    if (inputs.size() > 1 && B200DataType(inputs[1]->GetBlobDesc().data_type) != p->compute_dtype)
        RETURN_ON_NEQ(EnsureBuffer(&r_staging_, &r_cap_, static_cast<size_t>(rows) * N_ * 2), TNN_OK);
    return TNN_OK;
}

Status B200CudaFusedLinearLayerAcc::AsCompute(Blob* src, void* staging, int64_t count, const void** out) {
    auto* p = dynamic_cast<FusedLinearLayerParam*>(param_);
    const int sdt = B200DataType(src->GetBlobDesc().data_type);
    if (sdt == p->compute_dtype) {
        *out = DevicePtr(src);
        return TNN_OK;
    }
    if (sdt < 0 || !staging) return Status(TNNERR_PARAM_ERR, "FusedLinear: unsupported input data type");
    // another layer of this Forward may already have converted this blob (the graph input is both the first
    // projection's operand and the first residual)
    if (const void* done = context_->FindConverted(DevicePtr(src), p->compute_dtype, count)) {
        *out = done;
        return TNN_OK;
    }
    *out = staging;
    RETURN_ON_NEQ(B200ToStatus(b200_convert(DevicePtr(src), sdt, staging, p->compute_dtype, count, context_->GetStream()),
                               "b200_convert"),
                  TNN_OK);
    context_->NoteConverted(DevicePtr(src), p->compute_dtype, count, staging);
    return TNN_OK;
}

Status B200CudaFusedLinearLayerAcc::DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    auto* p = dynamic_cast<FusedLinearLayerParam*>(param_);
    const int64_t rows = Rows(inputs[0]->GetBlobDesc().dims);
    B200LinearDesc d;
    std::memset(&d, 0, sizeof(d));
    RETURN_ON_NEQ(AsCompute(inputs[0], x_staging_, rows * K_, &d.x), TNN_OK);
    if (p->epilogue == B200_EPI_BIAS_RESIDUAL)
        RETURN_ON_NEQ(AsCompute(inputs[1], r_staging_, rows * N_, &d.residual), TNN_OK);
    d.w_nk = w_packed_;
    d.bias = bias_;
    d.y    = DevicePtr(outputs[0]);
    d.M = rows; d.N = N_; d.K = K_;
    d.ldx = K_; d.ldw = K_; d.ldr = N_; d.ldy = N_;
    d.dtype     = p->compute_dtype;
    d.out_dtype = B200DataType(outputs[0]->GetBlobDesc().data_type);
    d.epilogue  = p->epilogue;
    d.block_n   = 0;
    return B200ToStatus(b200_linear_fwd(&d, context_->GetStream()), "b200_linear_fwd");
}
B200_REGISTER_CUDA_ACC(FusedLinear, LAYER_B200_FUSED_LINEAR)

// ================================================================= FusedAttention
B200_DECLARE_CUDA_ACC(FusedAttention)
};

Status B200CudaFusedAttentionLayerAcc::Init(Context* context, LayerParam* param, LayerResource* resource,
                                            const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    RETURN_ON_NEQ(B200CudaLayerAcc::Init(context, param, resource, inputs, outputs), TNN_OK);
    auto* p = dynamic_cast<FusedAttentionLayerParam*>(param);
    if (!p) return Status(TNNERR_PARAM_ERR, "FusedAttention: param missing");
    if (p->head_dim != 64) return Status(TNNERR_PARAM_ERR, "FusedAttention: only head_dim 64 is implemented");
    if (B200DataType(inputs[0]->GetBlobDesc().data_type) != p->compute_dtype)
        return Status(TNNERR_PARAM_ERR, "FusedAttention: qkv input must already be in the compute dtype");
    if (inputs.size() > 1 && inputs[1]->GetBlobDesc().data_type != DATA_TYPE_FLOAT)
        return Status(TNNERR_PARAM_ERR, "FusedAttention: mask must be fp32");
    return Reshape(inputs, outputs);
}

Status B200CudaFusedAttentionLayerAcc::Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    return TNN_OK;
}

Status B200CudaFusedAttentionLayerAcc::DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    auto* p = dynamic_cast<FusedAttentionLayerParam*>(param_);
    const DimsVector dims = inputs[0]->GetBlobDesc().dims;
    const int64_t B = dims[0], S = dims[1];
    const int64_t H = static_cast<int64_t>(p->heads) * p->head_dim;
    B200AttentionDesc d;
    std::memset(&d, 0, sizeof(d));
    char* qkv = static_cast<char*>(DevicePtr(inputs[0]));
    d.q = qkv; d.k = qkv + H * 2; d.v = qkv + 2 * H * 2;
    d.ldq = d.ldk = d.ldv = 3 * H;
    d.out = DevicePtr(outputs[0]);
    d.ldo = H;
    if (inputs.size() > 1) {
        d.mask_add = static_cast<const float*>(DevicePtr(inputs[1]));
        Status st = TNN_OK;
        d.kv_len = context_->GetKvLen(d.mask_add, static_cast<int>(B), static_cast<int>(S), p->mask_exclude_below, &st);
        RETURN_ON_NEQ(st, TNN_OK);
    }
    d.B = B; d.S = S;
    d.heads = p->heads; d.head_dim = p->head_dim;
    d.dtype = p->compute_dtype;
    d.scale = p->scale;
    d.mask_exclude_below = p->mask_exclude_below;
    return B200ToStatus(b200_attention_fwd(&d, context_->GetStream()), "b200_attention_fwd");
}
B200_REGISTER_CUDA_ACC(FusedAttention, LAYER_B200_FUSED_ATTENTION)

// ================================================================= FusedEmbedding
B200_DECLARE_CUDA_ACC(FusedEmbedding)
    Status Upload(RawBuffer& table, int64_t rows, int64_t H, int dtype, void** out);

    void* word_ = nullptr;   // [vocab, H] compute dtype
    void* type_ = nullptr;   // [type_vocab, H]
    void* pos_  = nullptr;   // [S, H]
    int64_t vocab_ = 0, type_vocab_ = 0, pos_rows_ = 0;
};

// fp32 host table -> device, converted to the compute dtype (tables are read once per token: half the bytes)
Status B200CudaFusedEmbeddingLayerAcc::Upload(RawBuffer& table, int64_t rows, int64_t H, int dtype, void** out) {
    if (table.GetDataType() != DATA_TYPE_FLOAT || table.GetDataCount() != rows * H)
        return Status(TNNERR_PARAM_ERR, "FusedEmbedding: tables must be fp32 [rows, H]");
    cudaStream_t stream = context_->GetStream();
    size_t cap = 0;
    RETURN_ON_NEQ(EnsureBuffer(out, &cap, static_cast<size_t>(rows) * H * 2), TNN_OK);
    void* tmp = nullptr;
    RETURN_ON_NEQ(device_->Allocate(&tmp, static_cast<size_t>(rows) * H * sizeof(float)), TNN_OK);
    Status st = TNN_OK;
    if (cudaMemcpyAsync(tmp, table.force_to<float*>(), static_cast<size_t>(rows) * H * sizeof(float),
                        cudaMemcpyHostToDevice, stream) != cudaSuccess) {
        cudaGetLastError();
        st = Status(TNNERR_CUDA_MEMCPY_ERROR, "FusedEmbedding: table upload failed");
    }
    if (st == TNN_OK) st = B200ToStatus(b200_convert(tmp, B200_F32, *out, dtype, rows * H, stream), "b200_convert");
    cudaStreamSynchronize(stream);   // Init time: the staging copy is released right away
    device_->Free(tmp);
    return st;
}

Status B200CudaFusedEmbeddingLayerAcc::Init(Context* context, LayerParam* param, LayerResource* resource,
                                            const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    RETURN_ON_NEQ(B200CudaLayerAcc::Init(context, param, resource, inputs, outputs), TNN_OK);
    auto* p = dynamic_cast<FusedEmbeddingLayerParam*>(param);
    auto* r = dynamic_cast<FusedEmbeddingLayerResource*>(resource);
    if (!p || !r || p->hidden <= 0) return Status(TNNERR_PARAM_ERR, "FusedEmbedding: param/resource missing");
    if (inputs.size() != 4 || inputs[0]->GetBlobDesc().data_type != DATA_TYPE_INT32 ||
        inputs[1]->GetBlobDesc().data_type != DATA_TYPE_INT32)
        return Status(TNNERR_PARAM_ERR, "FusedEmbedding: ids and segment ids must be int32 blobs");
    if (inputs[2]->GetBlobDesc().data_type != DATA_TYPE_FLOAT || inputs[3]->GetBlobDesc().data_type != DATA_TYPE_FLOAT)
        return Status(TNNERR_PARAM_ERR, "FusedEmbedding: scale and bias must be fp32");
    const int64_t H = p->hidden;
    vocab_      = r->word.GetDataCount() / H;
    type_vocab_ = r->type.GetDataCount() / H;
    pos_rows_   = r->position.GetDataCount() / H;
    RETURN_ON_NEQ(Upload(r->word, vocab_, H, p->compute_dtype, &word_), TNN_OK);
    RETURN_ON_NEQ(Upload(r->type, type_vocab_, H, p->compute_dtype, &type_), TNN_OK);
    RETURN_ON_NEQ(Upload(r->position, pos_rows_, H, p->compute_dtype, &pos_), TNN_OK);
    return Reshape(inputs, outputs);
}

Status B200CudaFusedEmbeddingLayerAcc::Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    const DimsVector dims = inputs[0]->GetBlobDesc().dims;
    if (dims.size() != 2 || dims[1] > pos_rows_)
        return Status(TNNERR_PARAM_ERR, "FusedEmbedding: sequence longer than the position table of the graph");
    return TNN_OK;
}

Status B200CudaFusedEmbeddingLayerAcc::DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    auto* p = dynamic_cast<FusedEmbeddingLayerParam*>(param_);
    const DimsVector dims = inputs[0]->GetBlobDesc().dims;
    B200EmbeddingDesc d;
    std::memset(&d, 0, sizeof(d));
    d.input_ids   = static_cast<const int32_t*>(DevicePtr(inputs[0]));
    d.segment_ids = static_cast<const int32_t*>(DevicePtr(inputs[1]));
    d.word_emb = word_; d.type_emb = type_; d.pos_emb = pos_;
    d.gamma = static_cast<const float*>(DevicePtr(inputs[2]));
    d.beta  = static_cast<const float*>(DevicePtr(inputs[3]));
    d.out = DevicePtr(outputs[0]);
    d.B = dims[0]; d.S = dims[1]; d.H = p->hidden;
    d.vocab = vocab_; d.type_vocab = type_vocab_;
    d.ld_table = p->hidden; d.ld_out = p->hidden;
    d.table_dtype = p->compute_dtype;
    d.out_dtype   = B200DataType(outputs[0]->GetBlobDesc().data_type);
    d.eps = p->eps;
    if (d.out_dtype < 0) return Status(TNNERR_PARAM_ERR, "FusedEmbedding: unsupported output data type");
    return B200ToStatus(b200_embedding_layernorm_fwd(&d, context_->GetStream()), "b200_embedding_layernorm_fwd");
}
B200_REGISTER_CUDA_ACC(FusedEmbedding, LAYER_B200_FUSED_EMBEDDING)

// ================================================================= FusedMask
B200_DECLARE_CUDA_ACC(FusedMask)
};

Status B200CudaFusedMaskLayerAcc::Init(Context* context, LayerParam* param, LayerResource* resource,
                                       const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    RETURN_ON_NEQ(B200CudaLayerAcc::Init(context, param, resource, inputs, outputs), TNN_OK);
    if (!dynamic_cast<FusedMaskLayerParam*>(param)) return Status(TNNERR_PARAM_ERR, "FusedMask: param missing");
    if (inputs[0]->GetBlobDesc().data_type != DATA_TYPE_INT32 || outputs[0]->GetBlobDesc().data_type != DATA_TYPE_FLOAT)
        return Status(TNNERR_PARAM_ERR, "FusedMask: int32 in, fp32 out");
    return Reshape(inputs, outputs);
}

Status B200CudaFusedMaskLayerAcc::Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    return TNN_OK;
}

Status B200CudaFusedMaskLayerAcc::DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    auto* p = dynamic_cast<FusedMaskLayerParam*>(param_);
    const DimsVector dims = inputs[0]->GetBlobDesc().dims;
    return B200ToStatus(b200_mask_from_input_mask(static_cast<const int32_t*>(DevicePtr(inputs[0])), dims[0], dims[1],
                                                  p->masked_value, -5000.0f, static_cast<float*>(DevicePtr(outputs[0])),
                                                  nullptr, context_->GetStream()),
                        "b200_mask_from_input_mask");
}
B200_REGISTER_CUDA_ACC(FusedMask, LAYER_B200_FUSED_MASK)

// ================================================================= FusedQAHead
B200_DECLARE_CUDA_ACC(FusedQAHead)
    float* weight_ = nullptr;    // fp32 [H, outputs]
    float* bias_   = nullptr;    // fp32 [outputs]
};

Status B200CudaFusedQAHeadLayerAcc::Init(Context* context, LayerParam* param, LayerResource* resource,
                                         const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    RETURN_ON_NEQ(B200CudaLayerAcc::Init(context, param, resource, inputs, outputs), TNN_OK);
    auto* p = dynamic_cast<FusedQAHeadLayerParam*>(param);
    auto* r = dynamic_cast<FusedQAHeadLayerResource*>(resource);
    if (!p || !r || p->hidden <= 0 || p->outputs <= 0) return Status(TNNERR_PARAM_ERR, "FusedQAHead: param/resource missing");
    if (r->weight.GetDataType() != DATA_TYPE_FLOAT || r->weight.GetDataCount() != p->hidden * p->outputs ||
        r->bias.GetDataType() != DATA_TYPE_FLOAT || r->bias.GetDataCount() != p->outputs)
        return Status(TNNERR_PARAM_ERR, "FusedQAHead: weight must be fp32 [H, outputs], bias fp32 [outputs]");
    if (static_cast<int>(outputs.size()) != p->outputs) return Status(TNNERR_PARAM_ERR, "FusedQAHead: output count");
    for (auto* o : outputs)
        if (o->GetBlobDesc().data_type != DATA_TYPE_FLOAT) return Status(TNNERR_PARAM_ERR, "FusedQAHead: fp32 outputs");
    if (B200DataType(inputs[0]->GetBlobDesc().data_type) != B200_F16 && B200DataType(inputs[0]->GetBlobDesc().data_type) != B200_BF16)
        return Status(TNNERR_PARAM_ERR, "FusedQAHead: the input must be a half-precision activation of the fused region");
    size_t cap = 0;
    void* w = nullptr;
    RETURN_ON_NEQ(EnsureBuffer(&w, &cap, static_cast<size_t>(p->hidden) * p->outputs * sizeof(float)), TNN_OK);
    weight_ = static_cast<float*>(w);
    cap = 0;
    void* b = nullptr;
    RETURN_ON_NEQ(EnsureBuffer(&b, &cap, static_cast<size_t>(p->outputs) * sizeof(float)), TNN_OK);
    bias_ = static_cast<float*>(b);
    cudaStream_t stream = context_->GetStream();
    if (cudaMemcpyAsync(weight_, r->weight.force_to<float*>(), static_cast<size_t>(p->hidden) * p->outputs * sizeof(float),
                        cudaMemcpyHostToDevice, stream) != cudaSuccess ||
        cudaMemcpyAsync(bias_, r->bias.force_to<float*>(), static_cast<size_t>(p->outputs) * sizeof(float),
                        cudaMemcpyHostToDevice, stream) != cudaSuccess) {
        cudaGetLastError();
        return Status(TNNERR_CUDA_MEMCPY_ERROR, "FusedQAHead: weight upload failed");
    }
    cudaStreamSynchronize(stream);
    return Reshape(inputs, outputs);
}

Status B200CudaFusedQAHeadLayerAcc::Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    return TNN_OK;
}

Status B200CudaFusedQAHeadLayerAcc::DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    auto* p = dynamic_cast<FusedQAHeadLayerParam*>(param_);
    const DimsVector dims = inputs[0]->GetBlobDesc().dims;
    B200QAHeadDesc d;
    std::memset(&d, 0, sizeof(d));
    d.x = DevicePtr(inputs[0]);
    d.weight = weight_;
    d.bias = bias_;
    d.M = Rows(dims);
    d.H = p->hidden;
    d.ldx = d.H;
    d.N = p->outputs;
    d.x_dtype = B200DataType(inputs[0]->GetBlobDesc().data_type);
    // every output straight into its own blob (the graph's "unstack"): no copy behind the kernel
    if (p->outputs > 4) return Status(TNNERR_PARAM_ERR, "FusedQAHead: at most 4 outputs");
    for (int n = 0; n < p->outputs; ++n) d.out_n[n] = static_cast<float*>(DevicePtr(outputs[n]));
    return B200ToStatus(b200_qa_head_fwd(&d, context_->GetStream()), "b200_qa_head_fwd");
}
B200_REGISTER_CUDA_ACC(FusedQAHead, LAYER_B200_FUSED_QA_HEAD)

// ================================================================= Squeeze / Unsqueeze
// Shape-only layers: the element order does not change, the acc copies the blob (the reference's CUDA accs do the
// same, source/tnn/device/cuda/acc/cuda_squeeze_layer_acc.cu and cuda_unsqueeze_layer_acc.cu).
static Status CopyBlob(Blob* in, Blob* out, void* src, void* dst, cudaStream_t stream) {
    const BlobDesc& a = in->GetBlobDesc();
    const BlobDesc& b = out->GetBlobDesc();
    const int64_t n = DimsVectorUtils::Count(a.dims);
    if (n != DimsVectorUtils::Count(b.dims) || a.data_type != b.data_type)
        return Status(TNNERR_PARAM_ERR, "shape-only layer: element counts or types differ");
    if (cudaMemcpyAsync(dst, src, static_cast<size_t>(n) * DataTypeUtils::GetBytesSize(a.data_type), cudaMemcpyDeviceToDevice,
                        stream) != cudaSuccess) {
        cudaGetLastError();
        return Status(TNNERR_CUDA_MEMCPY_ERROR, "shape-only layer: copy failed");
    }
    return TNN_OK;
}

B200_DECLARE_CUDA_ACC(Squeeze)
};
Status B200CudaSqueezeLayerAcc::Init(Context* context, LayerParam* param, LayerResource* resource,
                                     const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    return B200CudaLayerAcc::Init(context, param, resource, inputs, outputs);
}
Status B200CudaSqueezeLayerAcc::Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    return TNN_OK;
}
Status B200CudaSqueezeLayerAcc::DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    return CopyBlob(inputs[0], outputs[0], DevicePtr(inputs[0]), DevicePtr(outputs[0]), context_->GetStream());
}
B200_REGISTER_CUDA_ACC(Squeeze, LAYER_SQUEEZE)

B200_DECLARE_CUDA_ACC(Unsqueeze)
};
Status B200CudaUnsqueezeLayerAcc::Init(Context* context, LayerParam* param, LayerResource* resource,
                                       const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    return B200CudaLayerAcc::Init(context, param, resource, inputs, outputs);
}
Status B200CudaUnsqueezeLayerAcc::Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    return TNN_OK;
}
Status B200CudaUnsqueezeLayerAcc::DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    return CopyBlob(inputs[0], outputs[0], DevicePtr(inputs[0]), DevicePtr(outputs[0]), context_->GetStream());
}
B200_REGISTER_CUDA_ACC(Unsqueeze, LAYER_UNSQUEEZE)

// ================================================================= LayerNorm
// The graph's own LayerNorm layer (gamma, beta = input blobs 1 and 2, uploaded by ReloadConstantBlobs).  The reference's
// CUDA acc (source/tnn/device/cuda/acc/cuda_layer_norm_layer_acc.cu:28-146) reads gamma/beta in the activation's
// type; here they stay fp32 whatever the activation type is.
B200_DECLARE_CUDA_ACC(LayerNorm)
};

Status B200CudaLayerNormLayerAcc::Init(Context* context, LayerParam* param, LayerResource* resource,
                                       const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    RETURN_ON_NEQ(B200CudaLayerAcc::Init(context, param, resource, inputs, outputs), TNN_OK);
    auto* p = dynamic_cast<LayerNormLayerParam*>(param);
    if (!p || inputs.size() < 3) return Status(TNNERR_PARAM_ERR, "LayerNorm: needs x, scale and bias inputs");
    if (p->reduce_dims_size != 1)
        return Status(TNNERR_PARAM_ERR, "LayerNorm: only normalisation over the last dimension is implemented");
    if (inputs[1]->GetBlobDesc().data_type != DATA_TYPE_FLOAT || inputs[2]->GetBlobDesc().data_type != DATA_TYPE_FLOAT)
        return Status(TNNERR_PARAM_ERR, "LayerNorm: scale and bias must be fp32");
    return Reshape(inputs, outputs);
}

Status B200CudaLayerNormLayerAcc::Reshape(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    return TNN_OK;
}

Status B200CudaLayerNormLayerAcc::DoForward(const std::vector<Blob*>& inputs, const std::vector<Blob*>& outputs) {
    auto* p = dynamic_cast<LayerNormLayerParam*>(param_);
    const DimsVector dims = inputs[0]->GetBlobDesc().dims;
    B200LayerNormDesc d;
    std::memset(&d, 0, sizeof(d));
    d.x = DevicePtr(inputs[0]);
    d.gamma = static_cast<const float*>(DevicePtr(inputs[1]));
    d.beta  = static_cast<const float*>(DevicePtr(inputs[2]));
    d.y = DevicePtr(outputs[0]);
    d.rows = Rows(dims);
    d.H = dims.back();
    d.ldx = d.ldy = d.H;
    d.in_dtype  = B200DataType(inputs[0]->GetBlobDesc().data_type);
    d.out_dtype = B200DataType(outputs[0]->GetBlobDesc().data_type);
    d.eps = p->eps;
    if (d.in_dtype < 0 || d.out_dtype < 0) return Status(TNNERR_PARAM_ERR, "LayerNorm: unsupported data type");
    return B200ToStatus(b200_add_layernorm_fwd(&d, context_->GetStream()), "b200_add_layernorm_fwd");
}
B200_REGISTER_CUDA_ACC(LayerNorm, LAYER_LAYER_NORM)

}  // namespace TNN_NS
