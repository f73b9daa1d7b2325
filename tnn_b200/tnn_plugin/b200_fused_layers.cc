// Shape / data-type inference of the two fused layer types, and their registration (layer factory + type names).
// Modelled on how the reference adds a CUDA-only fused layer (source/tnn/layer/cbam_fused_reduce_layer.cc).
#include <map>
#include <string>

#include "b200_plugin_common.h"
#include "tnn/layer/base_layer.h"

namespace TNN_NS {

// ---------------------------------------------------------------- type names
// global_layer_type_map is a file-static of layer_type.cc that is only reachable through a const accessor
// (source/tnn/core/layer_type.cc:261-263); a build inside the TNN tree would add the two strings there instead.
struct B200LayerTypeNames {
    B200LayerTypeNames() {
        auto& m = const_cast<std::map<std::string, LayerType>&>(GetGlobalLayerTypeMap());
        m[kFusedLinearTypeName]    = LAYER_B200_FUSED_LINEAR;
        m[kFusedAttentionTypeName] = LAYER_B200_FUSED_ATTENTION;
        m[kFusedEmbeddingTypeName] = LAYER_B200_FUSED_EMBEDDING;
        m[kFusedMaskTypeName]      = LAYER_B200_FUSED_MASK;
        m[kFusedQAHeadTypeName]    = LAYER_B200_FUSED_QA_HEAD;
    }
};
static B200LayerTypeNames g_b200_layer_type_names;

// ---------------------------------------------------------------- FusedLinear
DECLARE_LAYER(B200FusedLinear, LAYER_B200_FUSED_LINEAR);

Status B200FusedLinearLayer::InferOutputDataType() {
    BaseLayer::InferOutputDataType();
    auto* p = dynamic_cast<FusedLinearLayerParam*>(param_);
    CHECK_PARAM_NULL(p);
    for (auto* b : output_blobs_) b->GetBlobDesc().data_type = TnnDataType(p->compute_dtype);
    return TNN_OK;
}

// Output dims = input dims with the last one replaced by N (the MatMul rule for a 2-D weight,
// source/tnn/layer/mat_mul_layer.cc:42-148).
Status B200FusedLinearLayer::InferOutputShape(bool ignore_error) {
    BaseLayer::InferOutputShape(ignore_error);
    auto* p = dynamic_cast<FusedLinearLayerParam*>(param_);
    CHECK_PARAM_NULL(p);
    DimsVector dims = input_blobs_[0]->GetBlobDesc().dims;
    if (dims.size() < 2 || dims.back() != p->in_features) {
        LOGE_IF(!ignore_error, "FusedLinear: input feature dim does not match the weight\n");
        return Status(TNNERR_PARAM_ERR, "FusedLinear: input feature dim does not match the weight");
    }
    if (p->epilogue == B200_EPI_BIAS_RESIDUAL) {
        if (input_blobs_.size() < 2) return Status(TNNERR_PARAM_ERR, "FusedLinear: residual input missing");
        DimsVector r = input_blobs_[1]->GetBlobDesc().dims;
        DimsVector want = dims;
        want.back() = p->out_features;
        if (r != want) return Status(TNNERR_PARAM_ERR, "FusedLinear: residual dims differ from the output dims");
    }
    dims.back() = p->out_features;
    output_blobs_[0]->GetBlobDesc().dims = dims;
    return TNN_OK;
}
REGISTER_LAYER(B200FusedLinear, LAYER_B200_FUSED_LINEAR);

// ---------------------------------------------------------------- FusedAttention
DECLARE_LAYER(B200FusedAttention, LAYER_B200_FUSED_ATTENTION);

Status B200FusedAttentionLayer::InferOutputDataType() {
    BaseLayer::InferOutputDataType();
    auto* p = dynamic_cast<FusedAttentionLayerParam*>(param_);
    CHECK_PARAM_NULL(p);
    for (auto* b : output_blobs_) b->GetBlobDesc().data_type = TnnDataType(p->compute_dtype);
    return TNN_OK;
}

// qkv [B, S, 3*heads*head_dim] -> context [B, S, heads*head_dim]
Status B200FusedAttentionLayer::InferOutputShape(bool ignore_error) {
    BaseLayer::InferOutputShape(ignore_error);
    auto* p = dynamic_cast<FusedAttentionLayerParam*>(param_);
    CHECK_PARAM_NULL(p);
    DimsVector dims = input_blobs_[0]->GetBlobDesc().dims;
    const int hidden = p->heads * p->head_dim;
    if (dims.size() != 3 || dims[2] != 3 * hidden) {
        LOGE_IF(!ignore_error, "FusedAttention: qkv input must be [B, S, 3*heads*head_dim]\n");
        return Status(TNNERR_PARAM_ERR, "FusedAttention: qkv input must be [B, S, 3*heads*head_dim]");
    }
    if (input_blobs_.size() > 1) {
        const DimsVector m = input_blobs_[1]->GetBlobDesc().dims;
        int64_t n = 1;
        for (int d : m) n *= d;
        if (m.empty() || m[0] != dims[0] || m.back() != dims[1] || n != static_cast<int64_t>(dims[0]) * dims[1])
            return Status(TNNERR_PARAM_ERR, "FusedAttention: mask must be [B,1,1,S]");
    }
    dims[2] = hidden;
    output_blobs_[0]->GetBlobDesc().dims = dims;
    return TNN_OK;
}
REGISTER_LAYER(B200FusedAttention, LAYER_B200_FUSED_ATTENTION);

// ---------------------------------------------------------------- FusedEmbedding
DECLARE_LAYER(B200FusedEmbedding, LAYER_B200_FUSED_EMBEDDING);

Status B200FusedEmbeddingLayer::InferOutputDataType() {
    BaseLayer::InferOutputDataType();
    auto* p = dynamic_cast<FusedEmbeddingLayerParam*>(param_);
    CHECK_PARAM_NULL(p);
    for (auto* b : output_blobs_) b->GetBlobDesc().data_type = TnnDataType(p->compute_dtype);
    return TNN_OK;
}

// ids [B, S] -> [B, S, H] (the Gather rule: index dims followed by the table's trailing dims,
// source/tnn/layer/gather_layer.cc:49-90)
Status B200FusedEmbeddingLayer::InferOutputShape(bool ignore_error) {
    BaseLayer::InferOutputShape(ignore_error);
    auto* p = dynamic_cast<FusedEmbeddingLayerParam*>(param_);
    CHECK_PARAM_NULL(p);
    if (input_blobs_.size() != 4) return Status(TNNERR_PARAM_ERR, "FusedEmbedding: needs ids, segments, gamma, beta");
    DimsVector dims = input_blobs_[0]->GetBlobDesc().dims;
    if (dims.size() != 2 || input_blobs_[1]->GetBlobDesc().dims != dims) {
        LOGE_IF(!ignore_error, "FusedEmbedding: ids and segment ids must both be [B, S]\n");
        return Status(TNNERR_PARAM_ERR, "FusedEmbedding: ids and segment ids must both be [B, S]");
    }
    dims.push_back(p->hidden);
    output_blobs_[0]->GetBlobDesc().dims = dims;
    return TNN_OK;
}
REGISTER_LAYER(B200FusedEmbedding, LAYER_B200_FUSED_EMBEDDING);

// ---------------------------------------------------------------- FusedMask
DECLARE_LAYER(B200FusedMask, LAYER_B200_FUSED_MASK);

Status B200FusedMaskLayer::InferOutputDataType() {
    BaseLayer::InferOutputDataType();
    for (auto* b : output_blobs_) b->GetBlobDesc().data_type = DATA_TYPE_FLOAT;
    return TNN_OK;
}

// [B, S] -> [B, 1, 1, S] (Unsqueeze at axes 1 and 2)
Status B200FusedMaskLayer::InferOutputShape(bool ignore_error) {
    BaseLayer::InferOutputShape(ignore_error);
    const DimsVector dims = input_blobs_[0]->GetBlobDesc().dims;
    if (dims.size() != 2) {
        LOGE_IF(!ignore_error, "FusedMask: input mask must be [B, S]\n");
        return Status(TNNERR_PARAM_ERR, "FusedMask: input mask must be [B, S]");
    }
    output_blobs_[0]->GetBlobDesc().dims = {dims[0], 1, 1, dims[1]};
    return TNN_OK;
}
REGISTER_LAYER(B200FusedMask, LAYER_B200_FUSED_MASK);

// ---------------------------------------------------------------- FusedQAHead
DECLARE_LAYER(B200FusedQAHead, LAYER_B200_FUSED_QA_HEAD);

Status B200FusedQAHeadLayer::InferOutputDataType() {
    BaseLayer::InferOutputDataType();
    for (auto* b : output_blobs_) b->GetBlobDesc().data_type = DATA_TYPE_FLOAT;
    return TNN_OK;
}

// x [B, S, H] -> `outputs` blobs [B, S, 1] (MatMul to [B, S, outputs], SplitV of the last axis into slices of 1)
Status B200FusedQAHeadLayer::InferOutputShape(bool ignore_error) {
    BaseLayer::InferOutputShape(ignore_error);
    auto* p = dynamic_cast<FusedQAHeadLayerParam*>(param_);
    CHECK_PARAM_NULL(p);
    DimsVector dims = input_blobs_[0]->GetBlobDesc().dims;
    if (dims.size() < 2 || dims.back() != p->hidden || static_cast<int>(output_blobs_.size()) != p->outputs) {
        LOGE_IF(!ignore_error, "FusedQAHead: input feature dim or output count does not match the weight\n");
        return Status(TNNERR_PARAM_ERR, "FusedQAHead: input feature dim or output count does not match the weight");
    }
    dims.back() = 1;
    for (auto* b : output_blobs_) b->GetBlobDesc().dims = dims;
    return TNN_OK;
}
REGISTER_LAYER(B200FusedQAHead, LAYER_B200_FUSED_QA_HEAD);

}  // namespace TNN_NS
