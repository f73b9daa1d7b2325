"""CPU: the numpy restatement against outputs of the reference itself (tests/golden, made by oracle/make_golden.py)."""
import os
import sys

import numpy as np
import pytest

from util import cosine, max_abs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

from oracle import bert_oracle  # noqa: E402
from oracle.make_golden import CASES, FRONTEND_CASES, GOLDEN, POOLER_CASES, QA_CASES, golden_workload  # noqa: E402
from tnn_b200 import model_synth  # noqa: E402


@pytest.mark.parametrize("name", sorted(CASES))
def test_restatement_matches_reference_x86(name):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    wl = golden_workload(**CASES[name])
    assert np.array_equal(g["lengths"], wl.lengths)
    y = bert_oracle.encoder_forward(wl)
    ref = g["x86"]
    assert y.shape == ref.shape
    # fp32 against fp32: only summation order differs (the x86 acc blocks K by 256 and uses FMA)
    assert max_abs(y, ref) < 5e-5
    assert cosine(y, ref) > 1 - 1e-9
    # the reference's two CPU devices agreed with each other when the fixture was made
    assert float(g["x86_vs_naive_max_abs"]) < 5e-5


@pytest.mark.parametrize("name", sorted(FRONTEND_CASES))
def test_frontend_restatement_matches_reference_x86(name):
    """Embedding gathers + adds + LayerNorm and the mask builder against the reference's own run of that graph."""
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    fw = model_synth.make_frontend_workload(**FRONTEND_CASES[name])
    emb, mask = bert_oracle.embedding_frontend(fw)
    assert emb.shape == g["emb_x86"].shape and mask.shape == g["mask_x86"].shape
    assert max_abs(emb, g["emb_x86"]) < 5e-6
    assert np.array_equal(mask, g["mask_x86"])           # (1 - m) * -10000 is exact in fp32
    assert float(g["x86_vs_naive_max_abs"]) < 5e-6


@pytest.mark.parametrize("name", sorted(POOLER_CASES))
def test_pooler_restatement_matches_reference_x86(name):
    """Encoder + pooler head (MatMul -> Add -> Tanh) against the reference's own run."""
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    kw = dict(POOLER_CASES[name])
    pooler = model_synth.make_pooler(768 if kw["geometry"] == "base" else 1024, kw.pop("pooler_seed"))
    wl = golden_workload(**kw)
    y = bert_oracle.linear(bert_oracle.encoder_forward(wl), pooler[0], pooler[1], act="tanh")
    assert max_abs(y, g["x86"]) < 5e-5
    assert float(g["x86_vs_naive_max_abs"]) < 5e-5


@pytest.mark.parametrize("name", sorted(QA_CASES))
def test_qa_head_restatement_matches_reference_x86(name):
    """Encoder + span-extraction head (MatMul [H, 2] -> Add -> SplitV -> Squeeze x 2) against the reference's own run:
    its two outputs `unstack:0` / `unstack:1`."""
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    kw = dict(QA_CASES[name])
    qa = model_synth.make_qa_head(768 if kw["geometry"] == "base" else 1024, kw.pop("qa_seed"))
    wl = golden_workload(**kw)
    start, end = bert_oracle.qa_head(bert_oracle.encoder_forward(wl), qa[0], qa[1])
    assert start.shape == g["start_x86"].shape == wl.x.shape[:2]
    assert max_abs(start, g["start_x86"]) < 5e-5 and max_abs(end, g["end_x86"]) < 5e-5
    assert float(g["x86_vs_naive_max_abs"]) < 5e-5


def test_export_style_graph_gives_the_fixture_on_the_reference():
    """The same weights written the way a plain converter export does (constant-map weights, Div scale) run on the
    reference's DEVICE_X86 to the committed fixture of the resource-style graph: the two forms are one computation."""
    import tempfile
    from oracle import tnn_ref
    if not tnn_ref.available():
        pytest.skip("the reference build is not here")
    name = "base_2layer_ragged"
    wl = golden_workload(**CASES[name])
    d = tempfile.mkdtemp(prefix="export_style_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    model_synth.write_tnn_model(wl, proto, model, style="export")
    inst = tnn_ref.TnnInstance(proto, model, device=tnn_ref.DEVICE_X86)
    inst.set_input("x", wl.x)
    inst.set_input("mask", wl.mask_add)
    inst.forward()
    y = inst.get_output().reshape(wl.x.shape)
    inst.close()
    assert max_abs(y, np.load(os.path.join(GOLDEN, name + ".npz"))["x86"]) < 2e-5


def test_shape_subgraph_export_gives_the_fixture_on_the_reference():
    """The export form whose head-split / head-merge Reshape layers take their target shape from a Shape -> Gather ->
    Concat subgraph in the graph: the reference folds the subgraph at Init and runs to the same committed fixture."""
    import tempfile
    from oracle import tnn_ref
    if not tnn_ref.available():
        pytest.skip("the reference build is not here")
    name = "base_2layer_ragged"
    wl = golden_workload(**CASES[name])
    d = tempfile.mkdtemp(prefix="export_shapes_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    model_synth.write_tnn_model(wl, proto, model, style="export_shapes")
    text = open(proto).read()
    assert "Shape " in text and "Gather " in text and "Concat " in text and "Reshape l0_q_r 2 1" in text
    for device in (tnn_ref.DEVICE_X86, tnn_ref.DEVICE_NAIVE):
        inst = tnn_ref.TnnInstance(proto, model, device=device)
        inst.set_input("x", wl.x)
        inst.set_input("mask", wl.mask_add)
        inst.forward()
        y = inst.get_output().reshape(wl.x.shape)
        inst.close()
        assert max_abs(y, np.load(os.path.join(GOLDEN, name + ".npz"))["x86"]) < 2e-5


def test_gather_out_of_range_is_an_error():
    with pytest.raises(IndexError):
        bert_oracle.gather_rows(np.zeros((4, 2), np.float32), np.array([0, 4]))


def test_softmax_masked_keys_underflow_to_zero():
    # -10000 on a key underflows exp() to exactly 0 in fp32: the reference's padded keys carry no weight.
    x = np.zeros((1, 1, 2, 8), np.float32)
    x[..., 5:] = -10000.0
    p = bert_oracle.softmax_last(x)
    assert np.all(p[..., 5:] == 0.0)
    assert np.allclose(p[..., :5], 0.2)


def test_layer_norm_constant_row_is_finite():
    x = np.full((2, 16), 3.0, np.float32)
    y = bert_oracle.layer_norm(x, np.ones(16, np.float32), np.zeros(16, np.float32), 1e-12)
    assert np.all(np.isfinite(y))


def test_gelu_erf_form():
    x = np.array([-3.0, -1.0, 0.0, 0.5, 2.0], np.float32)
    import math
    want = np.array([0.5 * v * (1 + math.erf(v / math.sqrt(2))) for v in x], np.float32)
    assert np.allclose(bert_oracle.gelu(x), want, atol=1e-6)


def test_reference_build_matches_fixture_when_present():
    """Where the compiled reference is present, re-run config 1 and compare with the committed fixture."""
    from oracle import tnn_ref
    if not tnn_ref.available():
        pytest.skip("oracle/_ref not built here")
    wl = golden_workload(**CASES["c1_attention_block"])
    out, _ = tnn_ref.run_workload(wl, tnn_ref.DEVICE_X86)
    g = np.load(os.path.join(GOLDEN, "c1_attention_block.npz"))
    assert max_abs(out, g["x86"]) < 1e-5
