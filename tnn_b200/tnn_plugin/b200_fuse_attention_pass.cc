// Graph-optimizer pass "net_optimizer_b200_fuse_attention": collapses the unfused transformer-encoder subgraphs of a
// TNN model into the fused layers the B200 accs implement.  Written against the reference's pass registry
// (NetOptimizerRegister, source/tnn/optimizer/net_optimizer_manager.h:46-66) and its graph matcher
// (Graph::fromInterpreted / GraphParser / Graph::rewrite, source/tnn/optimizer/graph_matcher/), with
// source/tnn/optimizer/net_optimizer_convert_matmul_to_conv.cc as the model for how a pass uses them.
//
//   1. attention block (with or without the additive mask):
//        MatMul+Add x3 (Q, K, V on the same input) -> Reshape -> Permute -> MatMul(QK^T) -> Mul(scale) [-> Add(mask)]
//        -> Softmax(axis 3) -> MatMul(PV) -> Permute -> Reshape
//      becomes  FusedLinear(x; Wq|Wk|Wv) -> FusedAttention(qkv [, mask])
//   2. MatMul -> Add(bias) -> GELU            becomes FusedLinear(epilogue GELU); -> Tanh (the pooler head) likewise
//   7. MatMul [H,2] -> Add -> SplitV(last axis, 1 + 1)   becomes FusedQAHead (two [B,S,1] outputs; the Squeeze layers
//      behind it stay and run on the device's shape-only acc)
//   3. MatMul -> Add(bias) -> Add(residual)   becomes FusedLinear(epilogue residual), either operand order of the Add
//   4. MatMul -> Add(bias)                    becomes FusedLinear
//   5. the embedding front-end  Gather(word) + Gather(segment) -> Add -> Add(position slice) -> LayerNorm
//                                              becomes FusedEmbedding(ids, segments, gamma, beta)
//   6. the mask builder  Unsqueeze(1,2) -> Cast(float) -> Sub(1 - m) -> Mul(c)   becomes FusedMask(input_mask)
// Other LayerNorm layers stay as they are (the device has an acc for them).
//
// The matcher compares layer types, input/output counts and topology only, so everything else — permute orders,
// reshape targets, softmax axis, weight positions, bias shapes — is validated in the generator, which declines
// (returns nullptr) when a subgraph is not the attention computation it looks like.  Matched weight buffers are
// never modified: every instance created from one TNN object shares them.
#include <cmath>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <tuple>
#include <vector>

#include "b200_cuda_device.h"
#include "b200_plugin_common.h"
#include "tnn/interpreter/layer_param.h"
#include "tnn/interpreter/layer_resource.h"
#include "tnn/optimizer/graph_matcher/graph_matcher.h"
#include "tnn/optimizer/graph_matcher/graph_parser.h"
#include "tnn/optimizer/graph_matcher/ir.h"
#include "tnn/optimizer/graph_matcher/logger.h"
#include "tnn/optimizer/net_optimizer.h"
#include "tnn/optimizer/net_optimizer_manager.h"

namespace TNN_NS {
namespace optimizer {

class NetOptimizerB200FuseAttention : public NetOptimizer {
public:
    virtual std::string Strategy() { return "net_optimizer_b200_fuse_attention"; }
    virtual bool IsSupported(const NetworkConfig& net_config);
    virtual Status Optimize(NetStructure* structure, NetResource* resource);

private:
    // The rewriting itself, on working copies (see Optimize).  `keep_reshape`: two-input Reshape layers to leave in
    // their two-input form; `survivors`: Reshape layers that were given a static shape and were not fused afterwards.
    Status Fuse(NetStructure* structure, NetResource* resource, int dtype, const std::set<std::string>& keep_reshape,
                std::vector<std::string>* survivors);
    Precision precision_ = PRECISION_AUTO;
};

NetOptimizerRegister<NetOptimizerB200FuseAttention> g_net_optimizer_b200_fuse_attention(OptPriority::P1);

bool NetOptimizerB200FuseAttention::IsSupported(const NetworkConfig& net_config) {
    // DefaultNetwork driving DEVICE_CUDA accs directly; called by the manager right before Optimize under the
    // optimizer mutex (source/tnn/core/default_network.cc:109-114), so the precision can be handed over in a member.
    precision_ = net_config.precision;
    return net_config.device_type == DEVICE_CUDA &&
           (net_config.network_type == NETWORK_TYPE_DEFAULT || net_config.network_type == NETWORK_TYPE_AUTO);
}

namespace {

struct LinearParts {
    RawBuffer weight;   // fp32 [K, N]; shares storage with the matched layer's resource
    RawBuffer bias;     // fp32 [N]
    int K = 0, N = 0;
};

// MatMul(weight as layer resource, [K,N]) followed by Add(bias as layer resource, [N]).
bool ExtractLinear(const std::shared_ptr<Node>& mm, const std::shared_ptr<Node>& add, NetResource* resource,
                   LinearParts* out) {
    if (!mm || !add) return false;
    auto mm_param = std::dynamic_pointer_cast<MatMulLayerParam>(mm->info->param);
    if (!mm_param || mm_param->weight_position != 1 || mm->info->inputs.size() != 1) return false;
    auto it = resource->resource_map.find(mm->info->name);
    if (it == resource->resource_map.end()) return false;
    auto mm_res = std::dynamic_pointer_cast<MatMulLayerResource>(it->second);
    if (!mm_res) return false;
    const DimsVector wd = mm_res->weight.GetBufferDims();
    if (wd.size() != 2 || mm_res->weight.GetDataType() != DATA_TYPE_FLOAT) return false;

    auto add_param = std::dynamic_pointer_cast<MultidirBroadcastLayerParam>(add->info->param);
    if (!add_param || add->info->inputs.size() != 1 || add_param->weight_input_index != 1) return false;
    auto jt = resource->resource_map.find(add->info->name);
    if (jt == resource->resource_map.end()) return false;
    auto add_res = std::dynamic_pointer_cast<EltwiseLayerResource>(jt->second);
    if (!add_res || add_res->element_handle.GetDataType() != DATA_TYPE_FLOAT) return false;
    if (add_res->element_handle.GetDataCount() != wd[1]) return false;

    out->weight = mm_res->weight;           // RawBuffer copy = shared storage, no data copy
    out->bias   = add_res->element_handle;
    out->K      = wd[0];
    out->N      = wd[1];
    return true;
}

bool PermuteIs(const std::shared_ptr<Node>& n, const std::vector<int>& want) {
    if (!n) return false;
    auto p = std::dynamic_pointer_cast<PermuteLayerParam>(n->info->param);
    return p && p->orders == want;
}

// Reshape [B,S,H] -> [B,S,heads,head_dim]: shape {., ., heads, head_dim}, one of the two possibly written as -1
// ("whatever is left": exporters do, and the reference's CPU Reshape rewrites its parameter that way when the constant
// folder has run, source/tnn/device/cpu/acc/cpu_reshape_layer_acc.cc:56-89); `width` = heads * head_dim.
bool SplitHeads(const std::shared_ptr<Node>& n, int width, int* heads, int* head_dim) {
    if (!n || n->info->inputs.size() != 1) return false;
    auto p = std::dynamic_pointer_cast<ReshapeLayerParam>(n->info->param);
    if (!p || p->shape.size() != 4 || p->axis != 0) return false;
    int h = p->shape[2], d = p->shape[3];
    if (h == -1 && d > 0 && width % d == 0) h = width / d;
    if (d == -1 && h > 0 && width % h == 0) d = width / h;
    if (h <= 0 || d <= 0) return false;
    *heads    = h;
    *head_dim = d;
    return true;
}

std::shared_ptr<Graph> ParsePattern(const std::string& text) {
    GraphRegistry registry;
    GraphParser parser(&registry);
    if (!parser.parseFromString(text)) return nullptr;
    return parser.getGraph();
}

Status AddFusedLinear(const std::shared_ptr<Graph>& g, const std::vector<std::string>& ins, const std::string& out,
                      const std::vector<LinearParts>& parts, int epilogue, int dtype) {
    RETURN_ON_NEQ(g->createNode(LAYER_B200_FUSED_LINEAR, ins, {out}), TNN_OK);
    auto node = g->getNodeByTensorName(out);
    if (!node) return Status(TNNERR_NET_ERR, "fused node not created");
    RETURN_ON_NEQ(node->createParam<FusedLinearLayerParam>(), TNN_OK);
    auto p           = node->param<FusedLinearLayerParam>();
    p->type          = kFusedLinearTypeName;
    p->name          = out;
    p->epilogue      = epilogue;
    p->compute_dtype = dtype;
    p->in_features   = parts[0].K;
    p->out_features  = 0;
    RETURN_ON_NEQ(node->createResource<FusedLinearLayerResource>(), TNN_OK);
    auto r  = node->resource<FusedLinearLayerResource>();
    r->name = out;
    for (const auto& lp : parts) {
        r->weights.push_back(lp.weight);
        r->biases.push_back(lp.bias);
        p->out_features += lp.N;
    }
    return TNN_OK;
}

// Converter exports differ in where constants live and how the scale is written; the patterns below know one form.
// This step rewrites the other forms into it, layer by layer, before matching:
//   * MatMul(x, W) with W a 2-D fp32 entry of the constant map (weight_position -1, two inputs) becomes MatMul(x) with
//     W as the layer's resource (weight_position 1) — both forms are handled by the reference's own pass,
//     source/tnn/optimizer/net_optimizer_convert_matmul_to_conv.cc:112-146;
//   * Add(x, c) / Add(c, x) / Mul(x, c) / Div(x, c) with c an fp32 entry of the constant map becomes the one-input
//     form with c as the layer's resource (weight_input_index 1; for Div only Div(x, c));
//   * Div by a one-element constant becomes Mul by its reciprocal (the attention scale written as / sqrt(d)).
// Shared objects are never modified: every new resource is a new object whose RawBuffer shares the constant's storage
// (or, for the reciprocal, owns four new bytes); the resource map is shared by the instances of a model, and a second
// instance's pass finds the entries of the first and replaces them with equal ones.
void Canonicalize(NetStructure* structure, NetResource* resource, const std::set<std::string>& keep_reshape,
                  std::vector<std::string>* static_reshapes) {
    auto constant = [&](const std::string& name) -> std::shared_ptr<RawBuffer> {
        auto it = resource->constant_map.find(name);
        if (it == resource->constant_map.end() || !it->second || it->second->GetDataType() != DATA_TYPE_FLOAT) return nullptr;
        return it->second;
    };
    std::vector<std::string> absorbed;   // constants that became layer resources
    for (auto& l : structure->layers) {
        if (l->type == LAYER_MATMUL && l->inputs.size() == 2) {
            auto p = std::dynamic_pointer_cast<MatMulLayerParam>(l->param);
            auto w = constant(l->inputs[1]);
            if (!p || !w || w->GetBufferDims().size() != 2 || constant(l->inputs[0])) continue;
            auto r    = std::make_shared<MatMulLayerResource>();
            r->name   = l->name;
            r->weight = *w;
            resource->resource_map[l->name] = r;
            p->weight_position = 1;
            absorbed.push_back(l->inputs[1]);
            l->inputs.pop_back();
        } else if ((l->type == LAYER_ADD || l->type == LAYER_MUL || l->type == LAYER_DIV) && l->inputs.size() == 2) {
            auto p = std::dynamic_pointer_cast<MultidirBroadcastLayerParam>(l->param);
            if (!p) continue;
            auto c1 = constant(l->inputs[1]);
            auto c0 = constant(l->inputs[0]);
            if (c1 && !c0) {
                absorbed.push_back(l->inputs[1]);
                l->inputs.pop_back();
            } else if (c0 && !c1 && l->type != LAYER_DIV) {
                absorbed.push_back(l->inputs[0]);
                l->inputs.erase(l->inputs.begin());
                c1 = c0;
            } else {
                continue;
            }
            auto r            = std::make_shared<EltwiseLayerResource>();
            r->name           = l->name;
            r->element_handle = *c1;
            r->element_shape  = c1->GetBufferDims();
            resource->resource_map[l->name] = r;
            p->weight_input_index = 1;
        }
        if (l->type == LAYER_DIV && l->inputs.size() == 1) {
            auto it = resource->resource_map.find(l->name);
            auto r  = it == resource->resource_map.end() ? nullptr : std::dynamic_pointer_cast<EltwiseLayerResource>(it->second);
            auto p  = std::dynamic_pointer_cast<MultidirBroadcastLayerParam>(l->param);
            if (!r || !p || p->weight_input_index != 1 || r->element_handle.GetDataCount() != 1 ||
                r->element_handle.GetDataType() != DATA_TYPE_FLOAT)
                continue;
            const float c = r->element_handle.force_to<float*>()[0];
            if (c == 0.f) continue;
            const float inv = 1.0f / c;
            auto m            = std::make_shared<EltwiseLayerResource>();
            m->name           = l->name;
            m->element_handle = RawBuffer(sizeof(float), reinterpret_cast<char*>(const_cast<float*>(&inv)), r->element_handle.GetBufferDims());
            m->element_handle.SetDataType(DATA_TYPE_FLOAT);
            m->element_shape  = r->element_shape;
            resource->resource_map[l->name] = m;
            l->type     = LAYER_MUL;
            l->type_str = "Mul";
            p->type     = "Mul";
        }
    }
    // Reshape(x, target) with the target shape an int32 constant — either a plain constant of the model or the result
    // of a Shape -> Gather -> Concat subgraph that the constant folder has evaluated (its value then sits in the
    // constant map under the blob's name) — becomes the one-input Reshape with that shape as its parameter, which is
    // what the reference's own Reshape layer does with such an input at Init
    // (ReshapeLayer::FillLayerParamWithConstantResource, source/tnn/layer/reshape_layer.cc:72-91).  Meant for the
    // Reshape layers that disappear in the attention pattern; the caller repeats the pass without this step for any
    // that does not (`keep_reshape`).
    bool any_reshape = false;
    for (auto& l : structure->layers) {
        if (l->type != LAYER_RESHAPE || l->inputs.size() != 2 || keep_reshape.count(l->name)) continue;
        auto it = resource->constant_map.find(l->inputs[1]);
        if (it == resource->constant_map.end() || !it->second || it->second->GetDataType() != DATA_TYPE_INT32) continue;
        auto p = std::dynamic_pointer_cast<ReshapeLayerParam>(l->param);
        const int n = it->second->GetDataCount();
        if (!p || n < 1 || n > 6) continue;
        const int* dims = it->second->force_to<int*>();
        p->shape.assign(dims, dims + n);
        p->axis     = 0;
        p->num_axes = n;
        absorbed.push_back(l->inputs[1]);
        l->inputs.pop_back();
        static_reshapes->push_back(l->name);
        any_reshape = true;
    }
    // Constant layers whose outputs nothing reads any more (the shape arithmetic behind such a Reshape) leave the
    // structure together with their folded values.
    for (bool again = any_reshape; again;) {
        again = false;
        for (size_t i = 0; i < structure->layers.size(); ++i) {
            auto l = structure->layers[i];
            if (!resource->constant_layers.count(l->name)) continue;
            bool used = false;
            for (auto& o : l->outputs) {
                used = used || structure->outputs.count(o) > 0;
                for (auto& m : structure->layers)
                    for (auto& in : m->inputs) used = used || in == o;
            }
            if (used) continue;
            for (auto& o : l->outputs) {
                resource->constant_map.erase(o);
                resource->constant_blob_flags.erase(o);
                structure->blobs.erase(o);
            }
            for (auto& in : l->inputs) absorbed.push_back(in);
            resource->constant_layers.erase(l->name);
            resource->shape_differ_layers.erase(l->name);
            resource->resource_map.erase(l->name);
            structure->layers.erase(structure->layers.begin() + i);
            again = true;
            break;
        }
    }
    // A constant nothing reads any more leaves this instance's constant map (the map is the instance's own copy; its
    // entries are shared): the graph matcher turns every entry into a node and refuses a graph with loose nodes.
    for (const auto& name : absorbed) {
        bool used = false;
        for (auto& l : structure->layers)
            for (auto& in : l->inputs) used = used || in == name;
        if (used) continue;
        resource->constant_map.erase(name);
        structure->blobs.erase(name);
    }
}

const char* kAttentionMasked = R"(
    graph(%x, %mask):
        %q_mm = MatMul(%x)
        %q_b  = Add(%q_mm)
        %q_r  = Reshape(%q_b)
        %q_p  = Permute(%q_r)
        %k_mm = MatMul(%x)
        %k_b  = Add(%k_mm)
        %k_r  = Reshape(%k_b)
        %k_p  = Permute(%k_r)
        %v_mm = MatMul(%x)
        %v_b  = Add(%v_mm)
        %v_r  = Reshape(%v_b)
        %v_p  = Permute(%v_r)
        %qk   = MatMul(%q_p, %k_p)
        %qk_s = Mul(%qk)
        %qk_m = Add(%qk_s, %mask)
        %sm   = Softmax(%qk_m)
        %ctx  = MatMul(%sm, %v_p)
        %ctx_p = Permute(%ctx)
        %ctx_r = Reshape(%ctx_p)
        return (%ctx_r)
)";

const char* kAttentionUnmasked = R"(
    graph(%x):
        %q_mm = MatMul(%x)
        %q_b  = Add(%q_mm)
        %q_r  = Reshape(%q_b)
        %q_p  = Permute(%q_r)
        %k_mm = MatMul(%x)
        %k_b  = Add(%k_mm)
        %k_r  = Reshape(%k_b)
        %k_p  = Permute(%k_r)
        %v_mm = MatMul(%x)
        %v_b  = Add(%v_mm)
        %v_r  = Reshape(%v_b)
        %v_p  = Permute(%v_r)
        %qk   = MatMul(%q_p, %k_p)
        %qk_s = Mul(%qk)
        %sm   = Softmax(%qk_s)
        %ctx  = MatMul(%sm, %v_p)
        %ctx_p = Permute(%ctx)
        %ctx_r = Reshape(%ctx_p)
        return (%ctx_r)
)";

}  // namespace

// All or nothing.  Instance::Init for DEVICE_CUDA tries the network twice (source/tnn/core/instance.cc:86-124): if the
// first DefaultNetwork::Init fails, the constant folder runs the graph's shape arithmetic on DEVICE_NAIVE — over the very
// NetStructure this pass has been given — and the network is initialised again.  A graph left half fused by a first
// attempt that then fails (fused layers have no CPU implementation) would break that retry.  So the pass works on
// copies and commits them only if every layer of the result can run: it has a DEVICE_CUDA acc, or the constant folder
// has evaluated it (constant layers are not instantiated, source/tnn/core/default_network.cc:255-259).  Otherwise the
// graph is left exactly as it was and the Status names the layers that stand in the way; on the first attempt TNN
// discards it and retries with the constants folded, on the second it is what the caller sees.
Status NetOptimizerB200FuseAttention::Optimize(NetStructure* structure, NetResource* resource) {
    if (!structure || !resource) return Status(TNNERR_NET_ERR, "Error: empty NetStructure or NetResource");
    if (precision_ == PRECISION_HIGH)
        return Status(TNNERR_PARAM_ERR,
                      "tnn_b200: PRECISION_HIGH (fp32) is not offered on DEVICE_CUDA; use AUTO/NORMAL (fp16) or LOW (bf16)");
    const int dtype = precision_ == PRECISION_LOW ? B200_BF16 : B200_F16;

    // Already fused (the pass must be idempotent: Instance::Init may run the optimizers twice on one structure).
    for (auto& l : structure->layers)
        if (l->type == LAYER_B200_FUSED_LINEAR || l->type == LAYER_B200_FUSED_ATTENTION ||
            l->type == LAYER_B200_FUSED_EMBEDDING || l->type == LAYER_B200_FUSED_MASK ||
            l->type == LAYER_B200_FUSED_QA_HEAD)
            return TNN_OK;

    // A two-input Reshape whose target shape is a folded constant is given that shape as a parameter so that the
    // attention pattern can see through it; one that does not end up inside a fused attention must keep its two-input
    // form (its shape follows the inputs when the instance is reshaped), so the attempt is repeated without touching it.
    std::shared_ptr<NetStructure> work_structure;
    NetResource work_resource;
    std::set<std::string> keep_reshape;
    for (int attempt = 0; attempt < 3; ++attempt) {
        work_structure = structure->Copy();   // layer infos and their params are copied
        if (!work_structure) return Status(TNNERR_OUTOFMEMORY, "tnn_b200: cannot copy the NetStructure");
        work_resource = *resource;            // maps of shared objects; the pass replaces entries, never edits them
        std::vector<std::string> survivors;
        RETURN_ON_NEQ(Fuse(work_structure.get(), &work_resource, dtype, keep_reshape, &survivors), TNN_OK);
        if (survivors.empty()) break;
        if (attempt == 2) return Status(TNNERR_NET_ERR, "tnn_b200: the fusion pass did not settle");
        keep_reshape.insert(survivors.begin(), survivors.end());
    }

    std::string missing;
    int n_missing = 0;
    for (auto& l : work_structure->layers) {
        if (work_resource.constant_layers.count(l->name)) continue;
        if (B200CudaDevice::HasLayerAcc(l->type)) continue;
        if (++n_missing <= 8) missing += (missing.empty() ? "" : ", ") + l->type_str + " '" + l->name + "'";
    }
    if (n_missing > 0) {
        if (n_missing > 8) missing += ", ... (" + std::to_string(n_missing) + " in all)";
        return Status(TNNERR_LAYER_ERR,
                      "tnn_b200: DEVICE_CUDA cannot run this graph: no CUDA implementation for " + missing +
                          " (after fusing the encoder subgraphs; layers the constant folder evaluates are exempt). "
                          "The graph was left unfused; there is no CPU fallback.");
    }
    *structure = *work_structure;
    *resource  = work_resource;
    return TNN_OK;
}

Status NetOptimizerB200FuseAttention::Fuse(NetStructure* structure, NetResource* resource, int dtype,
                                           const std::set<std::string>& keep_reshape,
                                           std::vector<std::string>* survivors) {
    std::vector<std::string> static_reshapes;
    Canonicalize(structure, resource, keep_reshape, &static_reshapes);

    std::shared_ptr<Graph> graph = std::make_shared<Graph>();
    Status status = graph->fromInterpreted(structure, resource);
    if (status != TNN_OK) {
        LOGE("%s", status.description().c_str());
        return TNN_OK;   // leave the graph alone, as the reference's passes do
    }

    // ---------------------------------------------------------------- 5. embedding front-end
    {
        std::shared_ptr<Graph> pattern = ParsePattern(R"(
            graph(%ids, %seg, %g, %be):
                %w   = Gather(%ids)
                %t   = Gather(%seg)
                %wt  = Add(%w, %t)
                %wtp = Add(%wt)
                %ln  = LayerNorm(%wtp, %g, %be)
                return (%ln)
        )");
        if (!pattern) return Status(TNNERR_PARAM_ERR, "invalid pattern syntax");
        auto gen = [&](std::shared_ptr<AnchorGraph> in) -> std::shared_ptr<Graph> {
            if (in->inputs().size() != 4 || in->outputs().size() != 1) return nullptr;
            auto node = [&](const char* n) { return in->getNodeByTensorName(std::string("@") + n); };
            // table rows gathered along axis 0 by a blob of indices; the table is the layer's resource
            auto table = [&](const std::shared_ptr<Node>& n, RawBuffer* out) {
                if (!n || n->info->inputs.size() != 1) return false;
                auto gp = std::dynamic_pointer_cast<GatherLayerParam>(n->info->param);
                if (!gp || gp->axis != 0 || !gp->data_in_resource || gp->indices_in_resource) return false;
                auto it = resource->resource_map.find(n->info->name);
                if (it == resource->resource_map.end()) return false;
                auto gr = std::dynamic_pointer_cast<GatherLayerResource>(it->second);
                if (!gr || gr->data.GetDataType() != DATA_TYPE_FLOAT || gr->data.GetBufferDims().size() != 2) return false;
                *out = gr->data;
                return true;
            };
            RawBuffer word, type;
            if (!table(node("w"), &word) || !table(node("t"), &type)) return nullptr;
            const int H = word.GetBufferDims()[1];
            if (type.GetBufferDims()[1] != H || H <= 0 || (H % 8) != 0 || H > 1024) return nullptr;
            auto wt = std::dynamic_pointer_cast<MultidirBroadcastLayerParam>(node("wt")->info->param);
            if (!wt || wt->weight_input_index != -1 || node("wt")->info->inputs.size() != 2) return nullptr;
            // position rows: a constant [1, S, H] (or [S, H]) added to every sequence
            auto wtp = node("wtp");
            auto wtp_param = std::dynamic_pointer_cast<MultidirBroadcastLayerParam>(wtp->info->param);
            if (!wtp_param || wtp->info->inputs.size() != 1) return nullptr;
            auto pr = resource->resource_map.find(wtp->info->name);
            if (pr == resource->resource_map.end()) return nullptr;
            auto pos_res = std::dynamic_pointer_cast<EltwiseLayerResource>(pr->second);
            if (!pos_res || pos_res->element_handle.GetDataType() != DATA_TYPE_FLOAT) return nullptr;
            const DimsVector pd = pos_res->element_handle.GetBufferDims();
            if (pd.size() < 2 || pd.back() != H || pos_res->element_handle.GetDataCount() % H != 0) return nullptr;
            if (pd.size() == 3 && pd[0] != 1) return nullptr;
            if (pd.size() > 3) return nullptr;
            auto ln = std::dynamic_pointer_cast<LayerNormLayerParam>(node("ln")->info->param);
            if (!ln || ln->reduce_dims_size != 1) return nullptr;

            auto g = std::make_shared<Graph>();
            const std::vector<std::string> ins = {"in_0", "in_1", "in_2", "in_3"};
            for (auto& n : ins) g->getNodeOrCreatePlaceHolder(n);
            const std::string out = node("ln")->info->name + "_b200_emb";
            if (g->createNode(LAYER_B200_FUSED_EMBEDDING, ins, {out}) != TNN_OK) return nullptr;
            auto fused = g->getNodeByTensorName(out);
            if (!fused || fused->createParam<FusedEmbeddingLayerParam>() != TNN_OK) return nullptr;
            auto fp           = fused->param<FusedEmbeddingLayerParam>();
            fp->type          = kFusedEmbeddingTypeName;
            fp->name          = out;
            fp->hidden        = H;
            fp->eps           = ln->eps;
            fp->compute_dtype = dtype;
            if (fused->createResource<FusedEmbeddingLayerResource>() != TNN_OK) return nullptr;
            auto fr      = fused->resource<FusedEmbeddingLayerResource>();
            fr->name     = out;
            fr->word     = word;
            fr->type     = type;
            fr->position = pos_res->element_handle;
            if (g->setInputsOrder(ins) != TNN_OK) return nullptr;
            return g;
        };
        RETURN_ON_FAIL(graph->rewrite(pattern, gen));
    }

    // ---------------------------------------------------------------- 6. mask builder
    {
        std::shared_ptr<Graph> pattern = ParsePattern(R"(
            graph(%m):
                %u = Unsqueeze(%m)
                %f = Cast(%u)
                %s = Sub(%f)
                %o = Mul(%s)
                return (%o)
        )");
        if (!pattern) return Status(TNNERR_PARAM_ERR, "invalid pattern syntax");
        auto gen = [&](std::shared_ptr<AnchorGraph> in) -> std::shared_ptr<Graph> {
            if (in->inputs().size() != 1 || in->outputs().size() != 1) return nullptr;
            auto node = [&](const char* n) { return in->getNodeByTensorName(std::string("@") + n); };
            auto up = std::dynamic_pointer_cast<UnsqueezeLayerParam>(node("u")->info->param);
            if (!up || up->axes != std::vector<int>({1, 2})) return nullptr;
            auto cp = std::dynamic_pointer_cast<CastLayerParam>(node("f")->info->param);
            if (!cp || cp->to != DATA_TYPE_FLOAT) return nullptr;
            auto scalar = [&](const std::shared_ptr<Node>& n, int want_index, float* value) {
                auto bp = std::dynamic_pointer_cast<MultidirBroadcastLayerParam>(n->info->param);
                if (!bp || n->info->inputs.size() != 1) return false;
                if (want_index >= 0 && bp->weight_input_index != want_index) return false;
                auto it = resource->resource_map.find(n->info->name);
                if (it == resource->resource_map.end()) return false;
                auto er = std::dynamic_pointer_cast<EltwiseLayerResource>(it->second);
                if (!er || er->element_handle.GetDataCount() != 1 || er->element_handle.GetDataType() != DATA_TYPE_FLOAT)
                    return false;
                *value = er->element_handle.force_to<float*>()[0];
                return true;
            };
            float one = 0.f, masked_value = 0.f;
            if (!scalar(node("s"), 0, &one) || one != 1.0f) return nullptr;    // the constant is the minuend: 1 - m
            if (!scalar(node("o"), -1, &masked_value)) return nullptr;         // multiplication commutes
            auto g = std::make_shared<Graph>();
            g->getNodeOrCreatePlaceHolder("in_0");
            const std::string out = node("o")->info->name + "_b200_mask";
            if (g->createNode(LAYER_B200_FUSED_MASK, {"in_0"}, {out}) != TNN_OK) return nullptr;
            auto fused = g->getNodeByTensorName(out);
            if (!fused || fused->createParam<FusedMaskLayerParam>() != TNN_OK) return nullptr;
            auto fp          = fused->param<FusedMaskLayerParam>();
            fp->type         = kFusedMaskTypeName;
            fp->name         = out;
            fp->masked_value = masked_value;
            return g;
        };
        RETURN_ON_FAIL(graph->rewrite(pattern, gen));
    }

    // ---------------------------------------------------------------- 1. attention
    for (int masked = 1; masked >= 0; --masked) {
        std::shared_ptr<Graph> pattern = ParsePattern(masked ? kAttentionMasked : kAttentionUnmasked);
        if (!pattern) return Status(TNNERR_PARAM_ERR, "invalid attention pattern syntax");

        auto gen = [&](std::shared_ptr<AnchorGraph> in) -> std::shared_ptr<Graph> {
            if (in->inputs().size() != static_cast<size_t>(masked ? 2 : 1) || in->outputs().size() != 1) return nullptr;
            auto node = [&](const char* n) { return in->getNodeByTensorName(std::string("@") + n); };
            LinearParts q, k, v;
            if (!ExtractLinear(node("q_mm"), node("q_b"), resource, &q) ||
                !ExtractLinear(node("k_mm"), node("k_b"), resource, &k) ||
                !ExtractLinear(node("v_mm"), node("v_b"), resource, &v))
                return nullptr;
            if (q.K != k.K || q.K != v.K || q.N != k.N || q.N != v.N) return nullptr;
            int heads = 0, head_dim = 0, h2 = 0, d2 = 0, h3 = 0, d3 = 0;
            if (!SplitHeads(node("q_r"), q.N, &heads, &head_dim) || !SplitHeads(node("k_r"), q.N, &h2, &d2) ||
                !SplitHeads(node("v_r"), q.N, &h3, &d3))
                return nullptr;
            if (heads != h2 || heads != h3 || head_dim != d2 || head_dim != d3 || heads * head_dim != q.N) return nullptr;
            if (!PermuteIs(node("q_p"), {0, 2, 1, 3}) || !PermuteIs(node("k_p"), {0, 2, 3, 1}) ||
                !PermuteIs(node("v_p"), {0, 2, 1, 3}) || !PermuteIs(node("ctx_p"), {0, 2, 1, 3}))
                return nullptr;
            for (const char* n : {"qk", "ctx"}) {
                auto p = std::dynamic_pointer_cast<MatMulLayerParam>(node(n)->info->param);
                if (!p || p->weight_position != -1) return nullptr;
            }
            auto sm = std::dynamic_pointer_cast<SoftmaxLayerParam>(node("sm")->info->param);
            if (!sm || (sm->axis != 3 && sm->axis != -1)) return nullptr;
            // merged heads: Reshape back to [B, S, H]
            auto ctx_r = std::dynamic_pointer_cast<ReshapeLayerParam>(node("ctx_r")->info->param);
            if (!ctx_r || ctx_r->shape.size() != 3 || (ctx_r->shape[2] != q.N && ctx_r->shape[2] != -1)) return nullptr;
            // scale: Mul by a one-element constant held as the layer's resource
            auto mul = node("qk_s");
            auto mul_param = std::dynamic_pointer_cast<MultidirBroadcastLayerParam>(mul->info->param);
            if (!mul_param || mul->info->inputs.size() != 1) return nullptr;
            auto mr = resource->resource_map.find(mul->info->name);
            if (mr == resource->resource_map.end()) return nullptr;
            auto mul_res = std::dynamic_pointer_cast<EltwiseLayerResource>(mr->second);
            if (!mul_res || mul_res->element_handle.GetDataCount() != 1 ||
                mul_res->element_handle.GetDataType() != DATA_TYPE_FLOAT)
                return nullptr;
            const float scale = mul_res->element_handle.force_to<float*>()[0];
            if (masked) {
                auto add = std::dynamic_pointer_cast<MultidirBroadcastLayerParam>(node("qk_m")->info->param);
                if (!add || add->weight_input_index != -1 || node("qk_m")->info->inputs.size() != 2) return nullptr;
            }

            const std::string prefix = node("q_mm")->info->name + "_b200_";
            auto g = std::make_shared<Graph>();
            const std::string in_x = "in_0", in_mask = "in_1";
            g->getNodeOrCreatePlaceHolder(in_x);
            if (masked) g->getNodeOrCreatePlaceHolder(in_mask);
            const std::string qkv_name = prefix + "qkv", ctx_name = prefix + "ctx";
            if (AddFusedLinear(g, {in_x}, qkv_name, {q, k, v}, B200_EPI_BIAS, dtype) != TNN_OK) return nullptr;
            std::vector<std::string> attn_in = {qkv_name};
            if (masked) attn_in.push_back(in_mask);
            if (g->createNode(LAYER_B200_FUSED_ATTENTION, attn_in, {ctx_name}) != TNN_OK) return nullptr;
            auto attn = g->getNodeByTensorName(ctx_name);
            if (!attn || attn->createParam<FusedAttentionLayerParam>() != TNN_OK) return nullptr;
            auto ap           = attn->param<FusedAttentionLayerParam>();
            ap->type          = kFusedAttentionTypeName;
            ap->name          = ctx_name;
            ap->heads         = heads;
            ap->head_dim      = head_dim;
            ap->scale         = scale;
            ap->compute_dtype = dtype;
            if (masked && g->setInputsOrder({in_x, in_mask}) != TNN_OK) return nullptr;
            return g;
        };
        RETURN_ON_FAIL(graph->rewrite(pattern, gen));
    }

    // ---------------------------------------------------------------- 2. MatMul -> Add -> GELU
    {
        std::shared_ptr<Graph> pattern = ParsePattern(R"(
            graph(%x):
                %mm  = MatMul(%x)
                %b   = Add(%mm)
                %act = GELU(%b)
                return (%act)
        )");
        if (!pattern) return Status(TNNERR_PARAM_ERR, "invalid pattern syntax");
        auto gen = [&](std::shared_ptr<AnchorGraph> in) -> std::shared_ptr<Graph> {
            if (in->inputs().size() != 1 || in->outputs().size() != 1) return nullptr;
            LinearParts lp;
            auto mm = in->getNodeByTensorName(std::string("@mm"));
            if (!ExtractLinear(mm, in->getNodeByTensorName(std::string("@b")), resource, &lp)) return nullptr;
            auto g = std::make_shared<Graph>();
            g->getNodeOrCreatePlaceHolder("in_0");
            if (AddFusedLinear(g, {"in_0"}, mm->info->name + "_b200_gelu", {lp}, B200_EPI_BIAS_GELU, dtype) != TNN_OK)
                return nullptr;
            return g;
        };
        RETURN_ON_FAIL(graph->rewrite(pattern, gen));
    }

    // ---------------------------------------------------------------- 2b. MatMul -> Add -> Tanh (the pooler head)
    {
        std::shared_ptr<Graph> pattern = ParsePattern(R"(
            graph(%x):
                %mm  = MatMul(%x)
                %b   = Add(%mm)
                %act = Tanh(%b)
                return (%act)
        )");
        if (!pattern) return Status(TNNERR_PARAM_ERR, "invalid pattern syntax");
        auto gen = [&](std::shared_ptr<AnchorGraph> in) -> std::shared_ptr<Graph> {
            if (in->inputs().size() != 1 || in->outputs().size() != 1) return nullptr;
            LinearParts lp;
            auto mm = in->getNodeByTensorName(std::string("@mm"));
            if (!ExtractLinear(mm, in->getNodeByTensorName(std::string("@b")), resource, &lp)) return nullptr;
            auto g = std::make_shared<Graph>();
            g->getNodeOrCreatePlaceHolder("in_0");
            if (AddFusedLinear(g, {"in_0"}, mm->info->name + "_b200_tanh", {lp}, B200_EPI_BIAS_TANH, dtype) != TNN_OK)
                return nullptr;
            return g;
        };
        RETURN_ON_FAIL(graph->rewrite(pattern, gen));
    }

    // ---------------------------------------------------------------- 3. MatMul -> Add -> Add(residual)
    for (int order = 0; order < 2; ++order) {
        std::shared_ptr<Graph> pattern = ParsePattern(order == 0 ? R"(
            graph(%x, %r):
                %mm = MatMul(%x)
                %b  = Add(%mm)
                %o  = Add(%b, %r)
                return (%o)
        )" : R"(
            graph(%x, %r):
                %mm = MatMul(%x)
                %b  = Add(%mm)
                %o  = Add(%r, %b)
                return (%o)
        )");
        if (!pattern) return Status(TNNERR_PARAM_ERR, "invalid pattern syntax");
        auto gen = [&](std::shared_ptr<AnchorGraph> in) -> std::shared_ptr<Graph> {
            if (in->inputs().size() != 2 || in->outputs().size() != 1) return nullptr;
            LinearParts lp;
            auto mm = in->getNodeByTensorName(std::string("@mm"));
            if (!ExtractLinear(mm, in->getNodeByTensorName(std::string("@b")), resource, &lp)) return nullptr;
            auto res_add = in->getNodeByTensorName(std::string("@o"));
            auto rp = std::dynamic_pointer_cast<MultidirBroadcastLayerParam>(res_add->info->param);
            if (!rp || rp->weight_input_index != -1 || res_add->info->inputs.size() != 2) return nullptr;
            // the residual must be an activation, not a constant of the model
            const std::string r_name = res_add->info->inputs[order == 0 ? 1 : 0];
            if (resource->constant_map.count(r_name) > 0) return nullptr;
            auto g = std::make_shared<Graph>();
            g->getNodeOrCreatePlaceHolder("in_0");
            g->getNodeOrCreatePlaceHolder("in_1");
            if (AddFusedLinear(g, {"in_0", "in_1"}, mm->info->name + "_b200_res", {lp}, B200_EPI_BIAS_RESIDUAL, dtype) !=
                TNN_OK)
                return nullptr;
            if (g->setInputsOrder({"in_0", "in_1"}) != TNN_OK) return nullptr;
            return g;
        };
        RETURN_ON_FAIL(graph->rewrite(pattern, gen));
    }

    // ---------------------------------------------------------------- 7. span-extraction head (before the plain linear)
    // MatMul [H, 2] -> Add(bias) -> SplitV(last axis, sizes 1, 1); the graph goes on with one Squeeze(last axis) per
    // slice to the two [B, S] outputs the reading-comprehension demo reads
    // (examples/linux/src/BertReadingComprehension/BertReadingComprehension.cc:109).  The Squeeze layers stay in the
    // graph (the device has an acc for them): a pattern that includes both is symmetric in them, the matcher finds it
    // twice with the outputs swapped and drops overlapping matches.
    {
        std::shared_ptr<Graph> pattern = ParsePattern(R"(
            graph(%x):
                %mm      = MatMul(%x)
                %b       = Add(%mm)
                %s0, %s1 = SplitV(%b)
                return (%s0, %s1)
        )");
        if (!pattern) return Status(TNNERR_PARAM_ERR, "invalid pattern syntax");
        auto gen = [&](std::shared_ptr<AnchorGraph> in) -> std::shared_ptr<Graph> {
            if (in->inputs().size() != 1 || in->outputs().size() != 2) return nullptr;
            LinearParts lp;
            auto mm = in->getNodeByTensorName(std::string("@mm"));
            if (!ExtractLinear(mm, in->getNodeByTensorName(std::string("@b")), resource, &lp)) return nullptr;
            if (lp.N != 2) return nullptr;
            auto split = in->getNodeByTensorName(std::string("@s0"));
            auto sp    = split ? std::dynamic_pointer_cast<SplitVLayerParam>(split->info->param) : nullptr;
            if (!sp || (sp->axis != 2 && sp->axis != -1) || sp->slices != std::vector<int>({1, 1})) return nullptr;
            auto g = std::make_shared<Graph>();
            g->getNodeOrCreatePlaceHolder("in_0");
            const std::string o0 = mm->info->name + "_b200_qa0", o1 = mm->info->name + "_b200_qa1";
            if (g->createNode(LAYER_B200_FUSED_QA_HEAD, {"in_0"}, {o0, o1}) != TNN_OK) return nullptr;
            auto node = g->getNodeByTensorName(o0);
            if (!node || node->createParam<FusedQAHeadLayerParam>() != TNN_OK) return nullptr;
            auto p     = node->param<FusedQAHeadLayerParam>();
            p->type    = kFusedQAHeadTypeName;
            p->name    = o0;
            p->hidden  = lp.K;
            p->outputs = lp.N;
            if (node->createResource<FusedQAHeadLayerResource>() != TNN_OK) return nullptr;
            auto r    = node->resource<FusedQAHeadLayerResource>();
            r->weight = lp.weight;
            r->bias   = lp.bias;
            return g;
        };
        RETURN_ON_FAIL(graph->rewrite(pattern, gen));
    }

    // ---------------------------------------------------------------- 4. MatMul -> Add
    {
        std::shared_ptr<Graph> pattern = ParsePattern(R"(
            graph(%x):
                %mm = MatMul(%x)
                %b  = Add(%mm)
                return (%b)
        )");
        if (!pattern) return Status(TNNERR_PARAM_ERR, "invalid pattern syntax");
        auto gen = [&](std::shared_ptr<AnchorGraph> in) -> std::shared_ptr<Graph> {
            if (in->inputs().size() != 1 || in->outputs().size() != 1) return nullptr;
            LinearParts lp;
            auto mm = in->getNodeByTensorName(std::string("@mm"));
            if (!ExtractLinear(mm, in->getNodeByTensorName(std::string("@b")), resource, &lp)) return nullptr;
            auto g = std::make_shared<Graph>();
            g->getNodeOrCreatePlaceHolder("in_0");
            if (AddFusedLinear(g, {"in_0"}, mm->info->name + "_b200_lin", {lp}, B200_EPI_BIAS, dtype) != TNN_OK)
                return nullptr;
            return g;
        };
        RETURN_ON_FAIL(graph->rewrite(pattern, gen));
    }
    for (const auto& name : static_reshapes)
        for (auto& l : structure->layers)
            if (l->name == name) survivors->push_back(name);
    return TNN_OK;
}

}  // namespace optimizer
}  // namespace TNN_NS

// ---------------------------------------------------------------------------------------------------------------
// Host-only hook for tests: run the pass on a model and describe the resulting layer list
// ("<type> <name> <inputs> -> <outputs>" per line).  Needs no GPU.
#include "tnn/interpreter/abstract_model_interpreter.h"
#include <cstdio>

#include "tnn/core/const_folder.h"
#include "tnn/interpreter/default_model_interpreter.h"

// What Instance::Init does around the pass for DEVICE_CUDA (source/tnn/core/instance.cc:86-124), without a device: the
// pass on the interpreted model; if it refuses and `fold_constants` is set, the reference's constant folder on
// DEVICE_NAIVE over the same structure, then the pass again.  `err` receives the last refusal's text.
static int RunPassLikeInstanceInit(TNN_NS::DefaultModelInterpreter* interp, int precision, int fold_constants, char* err,
                                   size_t err_cap) {
    using namespace TNN_NS;
    auto note = [&](const std::string& m) {
        if (err && err_cap > 0) std::snprintf(err, err_cap, "%s", m.c_str());
    };
    note("");
    optimizer::NetOptimizerB200FuseAttention pass;
    NetworkConfig cfg;
    cfg.device_type  = DEVICE_CUDA;
    cfg.network_type = NETWORK_TYPE_DEFAULT;
    cfg.precision    = static_cast<Precision>(precision);
    if (!pass.IsSupported(cfg)) return -3;
    Status st = pass.Optimize(interp->GetNetStructure(), interp->GetNetResource());
    if (st != TNN_OK && fold_constants) {
        note(st.description());
        auto folder = std::make_shared<ConstFolder>();
        ModelConfig mc;
        mc.model_type = MODEL_TYPE_TNN;
        NetworkConfig fc = cfg;
        InputShapesMap none;
        Status fs = folder->Init(fc, mc, interp, none, none);
        if (fs != TNN_OK) {
            note("constant folder: " + fs.description());
            return -7;
        }
        st = pass.Optimize(interp->GetNetStructure(), interp->GetNetResource());
    }
    if (st != TNN_OK) {
        note(st.description());
        return -4;
    }
    // run it again: must be a no-op
    if (pass.Optimize(interp->GetNetStructure(), interp->GetNetResource()) != TNN_OK) return -5;
    return 0;
}

extern "C" __attribute__((visibility("default"))) int tnnb200_test_fuse_ex(const char* proto, size_t proto_len,
                                                                            const char* model, size_t model_len,
                                                                            int precision, int fold_constants, char* out,
                                                                            size_t out_cap, char* err, size_t err_cap) {
    using namespace TNN_NS;
    auto* interp = dynamic_cast<DefaultModelInterpreter*>(CreateModelInterpreter(MODEL_TYPE_TNN));
    if (!interp) return -1;
    std::unique_ptr<DefaultModelInterpreter> guard(interp);
    std::vector<std::string> params = {std::string(proto, proto_len), std::string(model, model_len)};
    if (interp->Interpret(params) != TNN_OK) return -2;
    const int rc = RunPassLikeInstanceInit(interp, precision, fold_constants, err, err_cap);
    if (rc != 0) return rc;
    std::string text;
    for (auto& l : interp->GetNetStructure()->layers) {
        if (interp->GetNetResource()->constant_layers.count(l->name)) continue;   // folded: never instantiated
        text += l->type_str + " " + l->name;
        for (auto& i : l->inputs) text += " " + i;
        text += " ->";
        for (auto& o : l->outputs) text += " " + o;
        text += "\n";
    }
    if (text.size() + 1 > out_cap) return -6;
    std::memcpy(out, text.c_str(), text.size() + 1);
    return static_cast<int>(interp->GetNetStructure()->layers.size());
}

extern "C" __attribute__((visibility("default"))) int tnnb200_test_fuse(const char* proto, size_t proto_len,
                                                                         const char* model, size_t model_len,
                                                                         int precision, char* out, size_t out_cap) {
    return tnnb200_test_fuse_ex(proto, proto_len, model, model_len, precision, 0, out, out_cap, nullptr, 0);
}

// Host-only: run the pass on a model and save the optimised model with the reference's ModelPacker.  The saved pair
// loads through the fused layers' interpreters (b200_layer_interpreters.cc); the pass then finds nothing to do.
#include "tnn/interpreter/tnn/model_packer.h"

extern "C" __attribute__((visibility("default"))) int tnnb200_fuse_and_pack(const char* proto, size_t proto_len,
                                                                             const char* model, size_t model_len,
                                                                             int precision, const char* out_proto,
                                                                             const char* out_model) {
    using namespace TNN_NS;
    auto* interp = dynamic_cast<DefaultModelInterpreter*>(CreateModelInterpreter(MODEL_TYPE_TNN));
    if (!interp) return -1;
    std::unique_ptr<DefaultModelInterpreter> guard(interp);
    std::vector<std::string> params = {std::string(proto, proto_len), std::string(model, model_len)};
    if (interp->Interpret(params) != TNN_OK) return -2;
    optimizer::NetOptimizerB200FuseAttention pass;
    NetworkConfig cfg;
    cfg.device_type  = DEVICE_CUDA;
    cfg.network_type = NETWORK_TYPE_DEFAULT;
    cfg.precision    = static_cast<Precision>(precision);
    if (!pass.IsSupported(cfg)) return -3;
    if (pass.Optimize(interp->GetNetStructure(), interp->GetNetResource()) != TNN_OK) return -4;
    ModelPacker packer(interp->GetNetStructure(), interp->GetNetResource());
    if (packer.Pack(out_proto, out_model) != TNN_OK) return -5;
    return static_cast<int>(interp->GetNetStructure()->layers.size());
}
