"""CPU: the graph pass of the TNN plug-in (no GPU needed: the pass only rewrites the interpreted model)."""
import os
import tempfile

import pytest

from tnn_b200 import model_synth as ms
from tnn_b200 import tnn_runtime as rt

pytestmark = pytest.mark.skipif(not rt.available(), reason="TNN host framework / plug-in not built here")


def _fuse(wl, precision=rt.PRECISION_AUTO):
    d = tempfile.mkdtemp(prefix="fuse_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model)
    n_before = sum(1 for ln in open(proto).read().split("\n")[5:] if ln.strip())
    return n_before, rt.fuse_report(proto, model, precision)


def test_encoder_layers_collapse_to_seven_fused_layers():
    wl = ms.make_workload(ms.BERT_BASE, 2, 128, seed=1, num_layers=3)
    n_before, lines = _fuse(wl)
    assert n_before == 3 * 30
    types = [ln.split()[0] for ln in lines]
    assert types == ["FusedLinear", "FusedAttention", "FusedLinear", "LayerNorm",
                     "FusedLinear", "FusedLinear", "LayerNorm"] * 3
    # the attention layer consumes the packed QKV projection and the graph's mask input
    attn = [ln for ln in lines if ln.startswith("FusedAttention")][0].split()
    assert attn[3] == "mask"
    # layer names stay unique across encoder layers
    names = [ln.split()[1] for ln in lines]
    assert len(set(names)) == len(names)
    # the graph output keeps its name
    assert lines[-1].split()[-1] == "l2_ln2"


def test_attention_block_only_and_large_geometry():
    n_before, lines = _fuse(ms.config_workload(1))
    assert n_before == 23
    assert [ln.split()[0] for ln in lines] == ["FusedLinear", "FusedAttention", "FusedLinear", "LayerNorm"]
    wl = ms.make_workload(ms.BERT_LARGE, 1, 64, seed=2, num_layers=1)
    _, lines = _fuse(wl, rt.PRECISION_LOW)
    assert [ln.split()[0] for ln in lines].count("FusedLinear") == 4


def test_bert_graph_with_frontend_fuses_embedding_and_mask():
    """int32 inputs -> Gather x2 + Add x2 + LayerNorm and Unsqueeze/Cast/Sub/Mul in front of the encoder layers."""
    cfg = ms.EncoderConfig(1, 256, 4, 1024)
    wl = ms.make_workload(cfg, 2, 16, seed=1)
    fw = ms.make_frontend_workload(256, 2, 16, vocab=100, max_pos=32, seed=2)
    d = tempfile.mkdtemp(prefix="fuse_bert_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    out = ms.write_tnn_bert_model(fw, wl, proto, model)
    lines = rt.fuse_report(proto, model)
    types = [ln.split()[0] for ln in lines]
    assert types == ["FusedEmbedding", "FusedMask", "FusedLinear", "FusedAttention", "FusedLinear", "LayerNorm",
                     "FusedLinear", "FusedLinear", "LayerNorm"]
    emb, mask = lines[0].split(), lines[1].split()
    assert emb[2:6] == ["input_ids", "segment_ids", "emb_g", "emb_be"] and mask[2] == "input_mask"
    # the encoder consumes the fused front-end's outputs, and the graph output keeps its name
    assert lines[2].split()[2] == emb[-1] and lines[3].split()[3] == mask[-1]
    assert lines[-1].split()[-1] == out


def test_fused_model_round_trips_through_model_packer():
    """Pass -> ModelPacker -> files -> interpreters of the fused layers: the saved model lists the same layers and the
    pass has nothing left to do on it."""
    cfg = ms.EncoderConfig(2, 256, 4, 1024)
    wl = ms.make_workload(cfg, 2, 16, seed=3, randomize_affine=True)
    fw = ms.make_frontend_workload(256, 2, 16, vocab=100, max_pos=32, seed=4)
    d = tempfile.mkdtemp(prefix="fuse_pack_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_bert_model(fw, wl, proto, model)
    proto2, model2 = os.path.join(d, "f.tnnproto"), os.path.join(d, "f.tnnmodel")
    n = rt.fuse_and_pack(proto, model, proto2, model2)
    first = rt.fuse_report(proto, model)
    again = rt.fuse_report(proto2, model2)
    assert n == len(first) == 2 + 7 * 2
    assert again == first
    text = open(proto2).read()
    assert "FusedEmbedding" in text and "MatMul" not in text and "Gather" not in text


def test_export_style_graph_fuses_like_the_resource_style():
    """Weights and biases as constant-map inputs (MatMul weight_position -1, bias on either side of the Add) and the
    scale written as Div(sqrt(d)): the pass brings them to the form its patterns know and fuses the same layers; two
    instances of one model (a shared resource object, one private structure each) both fuse."""
    wl = ms.make_workload(ms.BERT_BASE, 2, 32, seed=2, num_layers=2)
    d = tempfile.mkdtemp(prefix="fuse_export_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model, style="export")
    text = open(proto).read()
    assert "Div" in text and " -1," in text
    lines = rt.fuse_report(proto, model)
    assert [ln.split()[0] for ln in lines] == ["FusedLinear", "FusedAttention", "FusedLinear", "LayerNorm",
                                               "FusedLinear", "FusedLinear", "LayerNorm"] * 2
    assert rt.fuse_report(proto, model) == lines
    # the fused model can be saved and reloaded
    proto2, model2 = os.path.join(d, "f.tnnproto"), os.path.join(d, "f.tnnmodel")
    assert rt.fuse_and_pack(proto, model, proto2, model2) == len(lines)
    assert rt.fuse_report(proto2, model2) == lines


def test_shape_subgraph_export_fuses_after_constant_folding():
    """Reshape layers whose target shape is computed in the graph (Shape -> Gather -> Concat -> two-input Reshape).  On
    its own the pass cannot see through them and must leave the WHOLE graph alone (a half-fused graph would break the
    constant folder's run on the CPU device that TNN starts next), saying which layers stand in the way; once the
    reference's constant folder has evaluated the shape arithmetic, the pass fuses the graph to the same seven layers
    per encoder layer, and the folded layers are gone from what is instantiated."""
    wl = ms.make_workload(ms.BERT_BASE, 2, 32, seed=2, num_layers=2)
    d = tempfile.mkdtemp(prefix="fuse_shapes_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model, style="export_shapes")
    with pytest.raises(rt.FuseRefused) as e:
        rt.fuse_report(proto, model)
    msg = str(e.value)
    assert "no CUDA implementation" in msg and "Shape 'l0_q_r_shape'" in msg and "left unfused" in msg
    lines = rt.fuse_report(proto, model, fold_constants=True)
    assert [ln.split()[0] for ln in lines] == ["FusedLinear", "FusedAttention", "FusedLinear", "LayerNorm",
                                               "FusedLinear", "FusedLinear", "LayerNorm"] * 2
    ref_lines = None
    proto0, model0 = os.path.join(d, "r.tnnproto"), os.path.join(d, "r.tnnmodel")
    ms.write_tnn_model(wl, proto0, model0, style="export")
    ref_lines = rt.fuse_report(proto0, model0)
    assert [ln.split()[0] for ln in ref_lines] == [ln.split()[0] for ln in lines]


def test_graph_with_a_layer_the_device_cannot_run_is_refused_whole():
    """An encoder followed by a layer without a CUDA implementation (Sigmoid): nothing is fused — not even the parts
    the pass knows — and the refusal names the layer, with and without constant folding.  Instance::Init then fails
    with this text instead of stumbling over fused layers on the CPU device."""
    wl = ms.make_workload(ms.EncoderConfig(1, 256, 4, 1024), 2, 16, seed=7)
    d = tempfile.mkdtemp(prefix="fuse_refuse_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    out = ms.write_tnn_model(wl, proto, model)
    text = open(proto).read().split("\n")
    # append Sigmoid(out) -> sig and make it the graph's output
    n_layers = int(text[4].strip('", '))
    text[4] = '" %d ,"' % (n_layers + 1)
    text[3] = '"sig ,"'
    text[2] = text[2].replace(' ,"', ' sig ,"')
    while text and not text[-1].strip():
        text.pop()
    text.append('"Sigmoid sig 1 1 %s sig ,"' % out)
    open(proto, "w").write("\n".join(text) + "\n")
    for fold in (False, True):
        with pytest.raises(rt.FuseRefused) as e:
            rt.fuse_report(proto, model, fold_constants=fold)
        assert "Sigmoid 'sig'" in str(e.value) and "no CPU fallback" in str(e.value)


def test_qa_head_fuses_to_one_layer_with_two_named_outputs():
    """MatMul [H, 2] -> Add -> SplitV becomes one FusedQAHead; the two Squeeze layers behind it keep the graph's
    output names; the fused model survives the ModelPacker round trip."""
    cfg = ms.EncoderConfig(1, 256, 4, 1024)
    wl = ms.make_workload(cfg, 2, 16, seed=5)
    d = tempfile.mkdtemp(prefix="fuse_qa_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    outs = ms.write_tnn_model(wl, proto, model, qa=ms.make_qa_head(256, 1))
    lines = rt.fuse_report(proto, model)
    types = [ln.split()[0] for ln in lines]
    assert types[-3:] == ["FusedQAHead", "Squeeze", "Squeeze"] and types.count("FusedQAHead") == 1
    assert not {"MatMul", "SplitV", "Add"} & set(types)
    assert [ln.split()[-1] for ln in lines[-2:]] == list(outs) == list(ms.QA_OUTPUTS)
    assert [ln.split()[2] for ln in lines[-2:]] == lines[-3].split()[-2:]     # each Squeeze reads one head output
    proto2, model2 = os.path.join(d, "f.tnnproto"), os.path.join(d, "f.tnnmodel")
    assert rt.fuse_and_pack(proto, model, proto2, model2) == len(lines)
    assert rt.fuse_report(proto2, model2) == lines


def test_precision_high_is_refused():
    with pytest.raises(RuntimeError):
        _fuse(ms.config_workload(1), rt.PRECISION_HIGH)
