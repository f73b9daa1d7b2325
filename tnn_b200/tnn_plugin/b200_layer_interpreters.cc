// tnnproto / tnnmodel (de)serialisation of the fused layer types, so that a model optimised by the pass can be saved
// with the reference's ModelPacker (source/tnn/interpreter/tnn/model_packer.cc:70-248) and loaded again without
// running the matcher.  Registered like every layer interpreter of the reference
// (source/tnn/interpreter/tnn/layer_interpreter/layer_interpreter_macro.h:20-30).
//
// Proto parameters (after the layer's input / output names):
//   FusedLinear     epilogue compute_dtype in_features out_features weight_count
//   FusedAttention  heads head_dim scale mask_exclude_below compute_dtype
//   FusedEmbedding  hidden eps compute_dtype
//   FusedMask       masked_value
//   FusedQAHead     hidden outputs
// Resources: FusedLinear = weight_count, then (weight fp32 [K,N_i], bias fp32 [N_i]) per merged weight;
//            FusedEmbedding = word, segment and position tables;  FusedQAHead = weight fp32 [H, outputs], bias.
#include <fstream>

#include "b200_plugin_common.h"
#include "tnn/interpreter/tnn/layer_interpreter/abstract_layer_interpreter.h"
#include "tnn/interpreter/tnn/layer_interpreter/layer_interpreter_macro.h"

namespace TNN_NS {

// ---------------------------------------------------------------- FusedLinear
DECLARE_LAYER_INTERPRETER(B200FusedLinear, LAYER_B200_FUSED_LINEAR);

Status B200FusedLinearLayerInterpreter::InterpretProto(str_arr layer_cfg_arr, int index, LayerParam** param) {
    auto p = CreateLayerParam<FusedLinearLayerParam>(param);
    GET_INT_1_OR_DEFAULT(p->epilogue, B200_EPI_BIAS);
    GET_INT_1_OR_DEFAULT(p->compute_dtype, B200_F16);
    GET_INT_1(p->in_features);
    GET_INT_1(p->out_features);
    return TNN_OK;
}

Status B200FusedLinearLayerInterpreter::InterpretResource(Deserializer& deserializer, LayerResource** resource) {
    auto r      = CreateLayerRes<FusedLinearLayerResource>(resource);
    const int n = deserializer.GetInt();
    if (n <= 0 || n > 16) return Status(TNNERR_INVALID_MODEL, "FusedLinear: bad weight count");
    for (int i = 0; i < n; ++i) {
        RawBuffer w, b;
        deserializer.GetRaw(w);
        deserializer.GetRaw(b);
        r->weights.push_back(w);
        r->biases.push_back(b);
    }
    return TNN_OK;
}

Status B200FusedLinearLayerInterpreter::SaveProto(std::ofstream& output_stream, LayerParam* param) {
    auto p = dynamic_cast<FusedLinearLayerParam*>(param);
    if (!p) return Status(TNNERR_NULL_PARAM, "invalid layer param to save");
    output_stream << p->epilogue << " " << p->compute_dtype << " " << p->in_features << " " << p->out_features << " ";
    return TNN_OK;
}

Status B200FusedLinearLayerInterpreter::SaveResource(Serializer& serializer, LayerParam* param, LayerResource* resource) {
    auto r = dynamic_cast<FusedLinearLayerResource*>(resource);
    if (!r || r->weights.size() != r->biases.size()) return Status(TNNERR_NULL_PARAM, "invalid layer resource to save");
    serializer.PutInt(static_cast<int>(r->weights.size()));
    for (size_t i = 0; i < r->weights.size(); ++i) {
        serializer.PutRaw(r->weights[i]);
        serializer.PutRaw(r->biases[i]);
    }
    return TNN_OK;
}
REGISTER_LAYER_INTERPRETER(B200FusedLinear, LAYER_B200_FUSED_LINEAR);

// ---------------------------------------------------------------- FusedAttention
DECLARE_LAYER_INTERPRETER(B200FusedAttention, LAYER_B200_FUSED_ATTENTION);

Status B200FusedAttentionLayerInterpreter::InterpretProto(str_arr layer_cfg_arr, int index, LayerParam** param) {
    auto p = CreateLayerParam<FusedAttentionLayerParam>(param);
    GET_INT_1(p->heads);
    GET_INT_1(p->head_dim);
    GET_FLOAT_1_OR_DEFAULT(p->scale, 1.0f);
    GET_FLOAT_1_OR_DEFAULT(p->mask_exclude_below, -5000.0f);
    GET_INT_1_OR_DEFAULT(p->compute_dtype, B200_F16);
    return TNN_OK;
}
Status B200FusedAttentionLayerInterpreter::InterpretResource(Deserializer& deserializer, LayerResource** resource) {
    return TNN_OK;
}
Status B200FusedAttentionLayerInterpreter::SaveProto(std::ofstream& output_stream, LayerParam* param) {
    auto p = dynamic_cast<FusedAttentionLayerParam*>(param);
    if (!p) return Status(TNNERR_NULL_PARAM, "invalid layer param to save");
    output_stream.precision(9);   // a float survives the text round trip
    output_stream << p->heads << " " << p->head_dim << " " << p->scale << " " << p->mask_exclude_below << " "
                  << p->compute_dtype << " ";
    return TNN_OK;
}
Status B200FusedAttentionLayerInterpreter::SaveResource(Serializer& serializer, LayerParam* param,
                                                        LayerResource* resource) {
    return TNN_OK;
}
REGISTER_LAYER_INTERPRETER(B200FusedAttention, LAYER_B200_FUSED_ATTENTION);

// ---------------------------------------------------------------- FusedEmbedding
DECLARE_LAYER_INTERPRETER(B200FusedEmbedding, LAYER_B200_FUSED_EMBEDDING);

Status B200FusedEmbeddingLayerInterpreter::InterpretProto(str_arr layer_cfg_arr, int index, LayerParam** param) {
    auto p = CreateLayerParam<FusedEmbeddingLayerParam>(param);
    GET_INT_1(p->hidden);
    GET_FLOAT_1_OR_DEFAULT(p->eps, 1e-12f);
    GET_INT_1_OR_DEFAULT(p->compute_dtype, B200_F16);
    return TNN_OK;
}
Status B200FusedEmbeddingLayerInterpreter::InterpretResource(Deserializer& deserializer, LayerResource** resource) {
    auto r = CreateLayerRes<FusedEmbeddingLayerResource>(resource);
    GET_BUFFER_FOR_ATTR(r, word, deserializer);
    GET_BUFFER_FOR_ATTR(r, type, deserializer);
    GET_BUFFER_FOR_ATTR(r, position, deserializer);
    return TNN_OK;
}
Status B200FusedEmbeddingLayerInterpreter::SaveProto(std::ofstream& output_stream, LayerParam* param) {
    auto p = dynamic_cast<FusedEmbeddingLayerParam*>(param);
    if (!p) return Status(TNNERR_NULL_PARAM, "invalid layer param to save");
    output_stream.precision(9);
    output_stream << p->hidden << " " << p->eps << " " << p->compute_dtype << " ";
    return TNN_OK;
}
Status B200FusedEmbeddingLayerInterpreter::SaveResource(Serializer& serializer, LayerParam* param,
                                                        LayerResource* resource) {
    auto r = dynamic_cast<FusedEmbeddingLayerResource*>(resource);
    if (!r) return Status(TNNERR_NULL_PARAM, "invalid layer resource to save");
    serializer.PutRaw(r->word);
    serializer.PutRaw(r->type);
    serializer.PutRaw(r->position);
    return TNN_OK;
}
REGISTER_LAYER_INTERPRETER(B200FusedEmbedding, LAYER_B200_FUSED_EMBEDDING);

// ---------------------------------------------------------------- FusedMask
DECLARE_LAYER_INTERPRETER(B200FusedMask, LAYER_B200_FUSED_MASK);

Status B200FusedMaskLayerInterpreter::InterpretProto(str_arr layer_cfg_arr, int index, LayerParam** param) {
    auto p = CreateLayerParam<FusedMaskLayerParam>(param);
    GET_FLOAT_1_OR_DEFAULT(p->masked_value, -10000.0f);
    return TNN_OK;
}
Status B200FusedMaskLayerInterpreter::InterpretResource(Deserializer& deserializer, LayerResource** resource) {
    return TNN_OK;
}
Status B200FusedMaskLayerInterpreter::SaveProto(std::ofstream& output_stream, LayerParam* param) {
    auto p = dynamic_cast<FusedMaskLayerParam*>(param);
    if (!p) return Status(TNNERR_NULL_PARAM, "invalid layer param to save");
    output_stream.precision(9);
    output_stream << p->masked_value << " ";
    return TNN_OK;
}
Status B200FusedMaskLayerInterpreter::SaveResource(Serializer& serializer, LayerParam* param, LayerResource* resource) {
    return TNN_OK;
}
REGISTER_LAYER_INTERPRETER(B200FusedMask, LAYER_B200_FUSED_MASK);

// ---------------------------------------------------------------- FusedQAHead
DECLARE_LAYER_INTERPRETER(B200FusedQAHead, LAYER_B200_FUSED_QA_HEAD);

Status B200FusedQAHeadLayerInterpreter::InterpretProto(str_arr layer_cfg_arr, int index, LayerParam** param) {
    auto p = CreateLayerParam<FusedQAHeadLayerParam>(param);
    GET_INT_1(p->hidden);
    GET_INT_1(p->outputs);
    return TNN_OK;
}
Status B200FusedQAHeadLayerInterpreter::InterpretResource(Deserializer& deserializer, LayerResource** resource) {
    auto r = CreateLayerRes<FusedQAHeadLayerResource>(resource);
    GET_BUFFER_FOR_ATTR(r, weight, deserializer);
    GET_BUFFER_FOR_ATTR(r, bias, deserializer);
    return TNN_OK;
}
Status B200FusedQAHeadLayerInterpreter::SaveProto(std::ofstream& output_stream, LayerParam* param) {
    auto p = dynamic_cast<FusedQAHeadLayerParam*>(param);
    if (!p) return Status(TNNERR_NULL_PARAM, "invalid layer param to save");
    output_stream << p->hidden << " " << p->outputs << " ";
    return TNN_OK;
}
Status B200FusedQAHeadLayerInterpreter::SaveResource(Serializer& serializer, LayerParam* param, LayerResource* resource) {
    auto r = dynamic_cast<FusedQAHeadLayerResource*>(resource);
    if (!r) return Status(TNNERR_NULL_PARAM, "invalid layer resource to save");
    serializer.PutRaw(r->weight);
    serializer.PutRaw(r->bias);
    return TNN_OK;
}
REGISTER_LAYER_INTERPRETER(B200FusedQAHead, LAYER_B200_FUSED_QA_HEAD);

}  // namespace TNN_NS
