// Shared declarations of the tnn_b200 DEVICE_CUDA plug-in for TNN: the two fused layer types the graph pass emits,
// their param / resource structs, and the mapping from the kernel library's status codes to TNN `Status`.
//
// In-tree these would be two new entries of the LayerType enum (source/tnn/core/layer_type.h) with their strings in
// global_layer_type_map (source/tnn/core/layer_type.cc:173-252).  Built out of tree against an unmodified TNN, the
// enum values are taken from an unused range and the strings are added to the map when the plug-in is loaded.
#ifndef TNN_B200_PLUGIN_COMMON_H_
#define TNN_B200_PLUGIN_COMMON_H_

#include <string>
#include <vector>

#include "tnn/core/common.h"
#include "tnn/core/layer_type.h"
#include "tnn/core/status.h"
#include "tnn/interpreter/layer_param.h"
#include "tnn/interpreter/layer_resource.h"
#include "tnn/interpreter/raw_buffer.h"

#include "tnn_b200.h"

namespace TNN_NS {

// Free slots between LAYER_CBAM_FUSED_POOLING (801) and LAYER_DUMMY_TYPE (1000).
static const LayerType LAYER_B200_FUSED_LINEAR    = static_cast<LayerType>(810);
static const LayerType LAYER_B200_FUSED_ATTENTION = static_cast<LayerType>(811);
static const LayerType LAYER_B200_FUSED_EMBEDDING = static_cast<LayerType>(812);
static const LayerType LAYER_B200_FUSED_MASK      = static_cast<LayerType>(813);
static const LayerType LAYER_B200_FUSED_QA_HEAD   = static_cast<LayerType>(814);
static const char* const kFusedLinearTypeName     = "FusedLinear";
static const char* const kFusedAttentionTypeName  = "FusedAttention";
static const char* const kFusedEmbeddingTypeName  = "FusedEmbedding";
static const char* const kFusedMaskTypeName       = "FusedMask";
static const char* const kFusedQAHeadTypeName     = "FusedQAHead";

// y = epilogue(x . W + bias (+ residual)); replaces MatMul -> Add(bias) [-> GELU | -> Add(residual)].
// Inputs: x [, residual].  Several matched MatMul+Add pairs that share x (Q, K, V) are merged: their weights are kept
// as separate read-only RawBuffers (the storage is shared with the matched layers' resources, which other instances
// of the same model also point at) and concatenated along N when the acc packs them.
struct FusedLinearLayerParam : public LayerParam {
    int epilogue      = B200_EPI_BIAS;  // B200_EPI_*
    int compute_dtype = B200_F16;       // B200_F16 or B200_BF16: operand and output type of the fused region
    int in_features   = 0;              // K
    int out_features  = 0;              // N (sum over merged weights)
    PARAM_COPY(FusedLinearLayerParam)
};

struct FusedLinearLayerResource : public LayerResource {
    std::vector<RawBuffer> weights;  // each fp32 [K, N_i], TNN MatMul layout (y = x.W)
    std::vector<RawBuffer> biases;   // each fp32 [N_i]
};

// context = softmax(scale * Q K^T + mask) V over a packed QKV activation; replaces
// Reshape/Permute x3 -> MatMul -> Mul(scale) -> Add(mask) -> Softmax -> MatMul -> Permute -> Reshape.
// Inputs: qkv [B,S,3H] [, mask [B,1,1,S]].
struct FusedAttentionLayerParam : public LayerParam {
    int heads                = 0;
    int head_dim             = 0;
    float scale              = 1.0f;
    float mask_exclude_below = -5000.0f;  // mask values at or below this drop the key exactly
    int compute_dtype        = B200_F16;
    PARAM_COPY(FusedAttentionLayerParam)
};

// out = LayerNorm(word_emb[ids] + type_emb[segments] + pos_emb[position]); replaces
// Gather(word) + Gather(segment) -> Add -> Add(position slice) -> LayerNorm in front of the first encoder layer.
// Inputs: input_ids [B,S] int32, segment_ids [B,S] int32, gamma [H], beta [H] (the LayerNorm's constant inputs).
struct FusedEmbeddingLayerParam : public LayerParam {
    int hidden        = 0;
    float eps         = 1e-12f;
    int compute_dtype = B200_F16;   // table and output type
    PARAM_COPY(FusedEmbeddingLayerParam)
};

struct FusedEmbeddingLayerResource : public LayerResource {
    RawBuffer word;       // fp32 [vocab, H]       (storage shared with the matched Gather's resource)
    RawBuffer type;       // fp32 [type_vocab, H]
    RawBuffer position;   // fp32 [1, S, H] or [S, H]: the position rows 0..S-1
};

// mask_add = (1 - input_mask) * masked_value as fp32 [B,1,1,S]; replaces Unsqueeze -> Cast -> Sub -> Mul.
// Input: input_mask [B,S] int32.
struct FusedMaskLayerParam : public LayerParam {
    float masked_value = -10000.0f;
    PARAM_COPY(FusedMaskLayerParam)
};

// Span-extraction head: logits = x . W + b with W [H, outputs], one fp32 [B, S, 1] output blob per logit; replaces
// MatMul -> Add(bias) -> SplitV(last axis, sizes 1).  Input: x [B, S, H].
struct FusedQAHeadLayerParam : public LayerParam {
    int hidden  = 0;
    int outputs = 0;
    PARAM_COPY(FusedQAHeadLayerParam)
};

struct FusedQAHeadLayerResource : public LayerResource {
    RawBuffer weight;   // fp32 [H, outputs] (storage shared with the matched MatMul's resource)
    RawBuffer bias;     // fp32 [outputs]
};

inline DataType TnnDataType(int b200_dtype) {
    return b200_dtype == B200_BF16 ? DATA_TYPE_BFP16 : (b200_dtype == B200_F16 ? DATA_TYPE_HALF : DATA_TYPE_FLOAT);
}
inline int B200DataType(DataType t) {
    return t == DATA_TYPE_BFP16 ? B200_BF16 : (t == DATA_TYPE_HALF ? B200_F16 : (t == DATA_TYPE_FLOAT ? B200_F32 : -1));
}

// Kernel-library status -> TNN Status.  The reference's CUDA_CHECK aborts the process
// (source/tnn/device/cuda/cuda_macro.h:24-40); these accs return instead.
inline Status B200ToStatus(int rc, const char* where) {
    if (rc == B200_OK) return TNN_OK;
    std::string msg = std::string(where) + ": " + b200_status_string(rc);
    switch (rc) {
        case B200_ERR_PARAM:
        case B200_ERR_UNSUPPORTED:
            return Status(TNNERR_PARAM_ERR, msg);
        case B200_ERR_NOT_SM100:
            return Status(TNNERR_DEVICE_NOT_SUPPORT, msg);
        default:
            return Status(TNNERR_CUDA_KERNEL_LAUNCH_ERROR, msg);
    }
}

}  // namespace TNN_NS

#endif  // TNN_B200_PLUGIN_COMMON_H_
