"""GPU: the drop-in path — TNN's own Instance::Forward on DEVICE_CUDA (served by the plug-in: fusion pass + fused
accs) against TNN's DEVICE_X86 on the same model files and inputs, in the same process.  This is the reference's
differential test idea (test/unit_test/layer_test/layer_test.cc) one level up."""
import os
import tempfile

import numpy as np
import pytest

from oracle.make_golden import CASES, GOLDEN, POOLER_CASES, QA_CASES, golden_workload
from tnn_b200 import model_synth as ms
from tnn_b200 import tnn_runtime as rt
from util import COS_TOL, MAX_ABS_TOL, cosine, max_abs, tolerances, valid_rows

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not rt.available(), reason="TNN host framework / plug-in missing")]


def _files(wl):
    d = tempfile.mkdtemp(prefix="plug_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model)
    return proto, model


def _run(proto, model, wl, device, precision=rt.PRECISION_AUTO):
    inst = rt.Instance(proto, model, device=device, precision=precision)
    inst.set_input("x", wl.x)
    inst.set_input("mask", wl.mask_add)
    inst.forward()
    out = inst.get_output()
    inst.close()
    return out


@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_instance_matches_x86_instance(cuda_device, name):
    wl = golden_workload(**CASES[name])
    proto, model = _files(wl)
    y = _run(proto, model, wl, rt.DEVICE_CUDA)
    ref = _run(proto, model, wl, rt.DEVICE_X86, rt.PRECISION_HIGH)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    assert max_abs(ref, g["x86"]) < 1e-5            # the x86 instance in this process is the committed fixture
    assert y.shape == ref.shape
    assert max_abs(y, ref) <= MAX_ABS_TOL
    assert cosine(y, ref) >= COS_TOL
    assert max_abs(valid_rows(y, wl.lengths), valid_rows(ref, wl.lengths)) <= MAX_ABS_TOL


def test_bf16_precision_low(cuda_device):
    wl = golden_workload(**CASES["base_2layer_ragged"])
    proto, model = _files(wl)
    y = _run(proto, model, wl, rt.DEVICE_CUDA, rt.PRECISION_LOW)
    ref = np.load(os.path.join(GOLDEN, "base_2layer_ragged.npz"))["x86"]
    tol, cos_tol = tolerances("bfloat16")
    assert max_abs(y, ref) <= tol
    assert cosine(y, ref) >= cos_tol


def test_plugin_path_equals_c_abi_path(cuda_device):
    """The accs launch the same kernels as the host mirror: bit-identical outputs."""
    import torch
    from tnn_b200.encoder import Encoder
    wl = golden_workload(**CASES["base_2layer_ragged"])
    proto, model = _files(wl)
    y = _run(proto, model, wl, rt.DEVICE_CUDA)
    enc = Encoder.from_workload(wl, torch.float16, fold_layernorm=False)   # the plug-in keeps LayerNorm layers
    z = enc.forward(torch.from_numpy(wl.x).cuda(), torch.from_numpy(wl.mask_add).cuda()).cpu().numpy()
    assert np.array_equal(y, z)


def test_two_instances_share_weights_and_repeat(cuda_device):
    """Two instances from the same files (shared host weights, private packed copies), forward twice each."""
    wl = golden_workload(**CASES["c1_attention_block"])
    proto, model = _files(wl)
    a = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    b = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    outs = []
    for inst in (a, b, a, b):
        inst.set_input("x", wl.x)
        inst.set_input("mask", wl.mask_add)
        inst.forward()
        outs.append(inst.get_output())
    for o in outs[1:]:
        assert np.array_equal(outs[0], o)
    ref = np.load(os.path.join(GOLDEN, "c1_attention_block.npz"))["x86"]
    assert max_abs(outs[0], ref) <= MAX_ABS_TOL


def test_unfusable_graph_fails_loudly(cuda_device):
    """PRECISION_HIGH has no CUDA path here: instance creation must fail, not fall back to a CPU device."""
    wl = golden_workload(**CASES["c1_attention_block"])
    proto, model = _files(wl)
    with pytest.raises(RuntimeError):
        rt.Instance(proto, model, device=rt.DEVICE_CUDA, precision=rt.PRECISION_HIGH)


def test_bert_graph_with_frontend_matches_x86_instance(cuda_device):
    """A converted-BERT-shaped graph: int32 input_ids / segment_ids / input_mask -> embedding gathers + LayerNorm and the
    mask builder -> two encoder layers.  DEVICE_CUDA (FusedEmbedding, FusedMask, fused encoder) against DEVICE_X86."""
    from oracle import bert_oracle
    cfg = ms.EncoderConfig(2, 768, 12, 3072)
    wl = ms.make_workload(cfg, 4, 128, seed=11, randomize_affine=True)
    fw = ms.make_frontend_workload(768, 4, 128, vocab=5000, type_vocab=2, max_pos=512, seed=12, length_range=(9, 128))
    d = tempfile.mkdtemp(prefix="plug_bert_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    out_name = ms.write_tnn_bert_model(fw, wl, proto, model)
    lines = rt.fuse_report(proto, model)
    types = [ln.split()[0] for ln in lines]
    assert types[:2] == ["FusedEmbedding", "FusedMask"] and "Gather" not in types and "Cast" not in types

    def run(device, precision):
        inst = rt.Instance(proto, model, device=device, precision=precision)
        inst.set_input_i32("input_ids", fw.input_ids)
        inst.set_input_i32("segment_ids", fw.segment_ids)
        inst.set_input_i32("input_mask", fw.input_mask)
        inst.forward()
        y = inst.get_output(out_name)
        inst.close()
        return y

    y = run(rt.DEVICE_CUDA, rt.PRECISION_AUTO)
    ref = run(rt.DEVICE_X86, rt.PRECISION_HIGH)
    emb, mask_add = bert_oracle.embedding_frontend(fw)
    want = bert_oracle.encoder_forward(wl, x=emb, mask_add=mask_add)
    assert max_abs(ref, want) < 5e-5                 # the reference and the restatement agree on the composed graph
    assert y.shape == ref.shape
    assert max_abs(y, ref) <= MAX_ABS_TOL
    assert cosine(y, ref) >= COS_TOL
    assert max_abs(valid_rows(y, fw.lengths), valid_rows(ref, fw.lengths)) <= MAX_ABS_TOL


def test_pooler_head_matches_x86_fixture(cuda_device):
    """Encoder layer + pooler head MatMul -> Add -> Tanh: fused into a FusedLinear with the tanh epilogue."""
    name = "base_1layer_pooler"
    kw = dict(POOLER_CASES[name])
    pooler = ms.make_pooler(768, kw.pop("pooler_seed"))
    wl = golden_workload(**kw)
    d = tempfile.mkdtemp(prefix="plug_pool_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model, pooler=pooler)
    lines = rt.fuse_report(proto, model)
    assert [ln.split()[0] for ln in lines][-1] == "FusedLinear" and "Tanh" not in [ln.split()[0] for ln in lines]
    y = _run(proto, model, wl, rt.DEVICE_CUDA)
    ref = np.load(os.path.join(GOLDEN, name + ".npz"))["x86"]
    assert y.shape == ref.shape
    assert max_abs(y, ref) <= MAX_ABS_TOL
    assert cosine(y, ref) >= COS_TOL


def test_export_style_graph_matches_x86_fixture(cuda_device):
    """Constant-map weights and biases, Div scale (a plain converter export): fused after canonicalisation, equal to the
    resource-style graph's result bit for bit."""
    name = "base_2layer_ragged"
    wl = golden_workload(**CASES[name])
    d = tempfile.mkdtemp(prefix="plug_export_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model, style="export")
    y = _run(proto, model, wl, rt.DEVICE_CUDA)
    proto0, model0 = _files(wl)
    assert np.array_equal(y, _run(proto0, model0, wl, rt.DEVICE_CUDA))
    ref = np.load(os.path.join(GOLDEN, name + ".npz"))["x86"]
    assert max_abs(y.reshape(ref.shape), ref) <= MAX_ABS_TOL


def test_shape_subgraph_export_runs_through_instance_init(cuda_device):
    """Target shapes computed in the graph (Shape -> Gather -> Concat -> two-input Reshape).  Instance::Init's own
    sequence for DEVICE_CUDA — a first attempt the pass refuses as a whole, the constant folder on the CPU device, a
    second attempt in which the pass fuses the folded graph — ends in the same fused layers and the same bits as the
    resource-style graph."""
    name = "base_2layer_ragged"
    wl = golden_workload(**CASES[name])
    d = tempfile.mkdtemp(prefix="plug_shapes_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model, style="export_shapes")
    y = _run(proto, model, wl, rt.DEVICE_CUDA)
    proto0, model0 = _files(wl)
    assert np.array_equal(y, _run(proto0, model0, wl, rt.DEVICE_CUDA))
    ref = np.load(os.path.join(GOLDEN, name + ".npz"))["x86"]
    assert max_abs(y.reshape(ref.shape), ref) <= MAX_ABS_TOL


def test_unsupported_layer_fails_with_the_pass_explanation(cuda_device):
    """A graph the device cannot run whole (an encoder followed by Sigmoid): instance creation fails, and the message
    is the pass's — which layer has no CUDA implementation — not a complaint about fused layers on the CPU device."""
    wl = ms.make_workload(ms.EncoderConfig(1, 256, 4, 1024), 2, 16, seed=7)
    d = tempfile.mkdtemp(prefix="plug_refuse_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    out = ms.write_tnn_model(wl, proto, model)
    text = open(proto).read().split("\n")
    n_layers = int(text[4].strip('", '))
    text[4] = '" %d ,"' % (n_layers + 1)
    text[3] = '"sig ,"'
    text[2] = text[2].replace(' ,"', ' sig ,"')
    while text and not text[-1].strip():
        text.pop()
    text.append('"Sigmoid sig 1 1 %s sig ,"' % out)
    open(proto, "w").write("\n".join(text) + "\n")
    with pytest.raises(RuntimeError) as e:
        rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    assert "Sigmoid 'sig'" in str(e.value) and "no CUDA implementation" in str(e.value)


def test_qa_head_matches_x86_fixture(cuda_device):
    """Encoder layer + span-extraction head: one FusedQAHead, outputs `unstack:0` / `unstack:1` as the demo reads them."""
    name = "base_1layer_qa"
    kw = dict(QA_CASES[name])
    qa = ms.make_qa_head(768, kw.pop("qa_seed"))
    wl = golden_workload(**kw)
    d = tempfile.mkdtemp(prefix="plug_qa_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    outs = ms.write_tnn_model(wl, proto, model, qa=qa)
    inst = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    inst.set_input("x", wl.x)
    inst.set_input("mask", wl.mask_add)
    inst.forward()
    start, end = inst.get_output(outs[0]), inst.get_output(outs[1])
    inst.close()
    ref = np.load(os.path.join(GOLDEN, name + ".npz"))
    assert start.size == ref["start_x86"].size == wl.x.shape[0] * wl.x.shape[1]
    for got, want in ((start, ref["start_x86"]), (end, ref["end_x86"])):
        got = valid_rows(got.reshape(want.shape)[..., None], wl.lengths)     # logits of the real tokens
        want = valid_rows(want[..., None], wl.lengths)
        assert max_abs(got, want) <= MAX_ABS_TOL
        assert cosine(got, want) >= COS_TOL


def test_half_precision_mats_in_and_out(cuda_device):
    """A model whose activation input is declared half precision: RESERVED_FP16_TEST Mats go to / come from the device
    as plain copies (half the PCIe bytes), and the result equals the fp32-Mat route bit for bit."""
    wl = golden_workload(**CASES["base_2layer_ragged"])
    d = tempfile.mkdtemp(prefix="plug_half_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model, input_dtype="half")
    inst = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    inst.set_input_half("x", wl.x.astype(np.float16))
    inst.set_input("mask", wl.mask_add)
    inst.forward()
    y16 = inst.get_output_half().astype(np.float32).reshape(wl.x.shape)
    inst.close()
    # (Instance caches one output Mat per blob, so the other Mat type gets an instance of its own.)
    inst = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    inst.set_input("x", wl.x)                       # an fp32 Mat into the half blob: converted on the device
    inst.set_input("mask", wl.mask_add)
    inst.forward()
    y32 = inst.get_output()                         # the half-precision output blob, up-converted on the device
    inst.close()
    assert np.array_equal(y16, y32)
    proto32, model32 = _files(wl)                   # the untyped (fp32 input) model
    assert np.array_equal(_run(proto32, model32, wl, rt.DEVICE_CUDA), y32)
    ref = np.load(os.path.join(GOLDEN, "base_2layer_ragged.npz"))["x86"]
    assert max_abs(y32, ref) <= MAX_ABS_TOL


class _DevView:
    """A zero-copy view of device memory for torch.as_tensor (the CUDA array interface)."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


def test_device_mats_in_and_out(cuda_device):
    """DEVICE_CUDA Mats (the converter's device branch): the input comes from a torch tensor on the GPU, the output Mat
    stays on the GPU; equal to the host-Mat route bit for bit, for fp16 Mats (plain copies) and fp32 Mats (converted)."""
    import torch
    wl = golden_workload(**CASES["base_2layer_ragged"])
    d = tempfile.mkdtemp(prefix="plug_dev_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model, input_dtype="half")
    ref = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    ref.set_input_half("x", wl.x.astype(np.float16))
    ref.set_input("mask", wl.mask_add)
    ref.forward()
    want = ref.get_output_half()
    ref.close()

    for kind, dt, typestr in ((rt.Instance.MAT_F16, torch.float16, "<f2"), (rt.Instance.MAT_F32, torch.float32, "<f4")):
        inst = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
        x = torch.from_numpy(wl.x.astype(np.float16)).to("cuda").to(dt).contiguous()
        m = torch.from_numpy(np.ascontiguousarray(wl.mask_add, dtype=np.float32)).to("cuda").contiguous()
        torch.cuda.synchronize()
        inst.set_input_device("x", x.data_ptr(), x.numel(), kind)
        inst.set_input_device("mask", m.data_ptr(), m.numel(), rt.Instance.MAT_F32)
        inst.forward()
        ptr, n = inst.get_output_device("", kind)
        assert n == want.size and ptr
        y = torch.as_tensor(_DevView(ptr, n, typestr), device="cuda").to(torch.float16).cpu().numpy()
        np.testing.assert_array_equal(y.view(np.uint16), want.view(np.uint16))
        inst.close()


def test_saved_fused_model_runs_identically(cuda_device):
    """The optimised model saved by ModelPacker (fused layer types in the files) gives the same bits as the original."""
    wl = golden_workload(**CASES["base_2layer_ragged"])
    proto, model = _files(wl)
    d = tempfile.mkdtemp(prefix="plug_pack_")
    proto2, model2 = os.path.join(d, "f.tnnproto"), os.path.join(d, "f.tnnmodel")
    rt.fuse_and_pack(proto, model, proto2, model2)
    a = _run(proto, model, wl, rt.DEVICE_CUDA)
    b = _run(proto2, model2, wl, rt.DEVICE_CUDA)
    assert np.array_equal(a, b)


def test_instance_reshape_within_the_created_shapes(cuda_device):
    """Instance::Reshape (source/tnn/core/instance.cc:143-152, default_network.cc:456-500): smaller batch and sequence
    length, then back to the created shape, on the same instances.  DEVICE_CUDA must follow DEVICE_X86 at every shape
    (the replayed graph of the previous shape must not be used), take nothing from the driver on the way, and return
    to the first result bit for bit."""
    wl = golden_workload(**CASES["base_2layer_ragged"])
    proto, model = _files(wl)
    B, S, H = wl.x.shape
    cuda = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    x86 = rt.Instance(proto, model, device=rt.DEVICE_X86, precision=rt.PRECISION_HIGH)

    def run(inst, x, mask):
        inst.set_input("x", x)
        inst.set_input("mask", mask)
        inst.forward()
        inst.forward()          # the second Forward of a shape is the captured one, the third a replay
        inst.forward()
        return inst.get_output()

    first = run(cuda, wl.x, wl.mask_add)
    before = rt.arena_stats(0)
    captures = cuda.graph_counters()["captures"]
    for b, s in ((1, 96), (B, 64), (1, 1), (B, S - 8), (B, S)):
        x = np.ascontiguousarray(wl.x[:b, :s])
        mask = np.ascontiguousarray(wl.mask_add[:b, :, :, :s])
        for inst in (cuda, x86):
            inst.reshape({"x": [b, s, H], "mask": [b, 1, 1, s]})
        y, ref = run(cuda, x, mask), run(x86, x, mask)
        assert y.shape == ref.shape == (b, s, H)
        lengths = np.minimum(wl.lengths[:b], s)
        assert max_abs(valid_rows(y, lengths), valid_rows(ref, lengths)) <= MAX_ABS_TOL, (b, s)
        assert cosine(y, ref) >= COS_TOL, (b, s)
    assert np.array_equal(y, first)
    after = rt.arena_stats(0)
    assert after["driver_allocations"] == before["driver_allocations"]
    counters = cuda.graph_counters()
    assert counters["captures"] > captures and counters["failures"] == 0
    cuda.close()
    x86.close()


def test_share_memory_modes_and_shared_command_queue(cuda_device):
    """NetworkConfig.share_memory_mode and Instance::ShareCommandQueue on DEVICE_CUDA (include/tnn/core/common.h:117-125,
    source/tnn/core/blob_manager.cc:230-262,314-330, source/tnn/device/cuda/cuda_context.cc ShareCommandQueue): blob
    memory provided by the caller (handles = base + bytes_offset), blob memory shared by the instances of one thread,
    and two instances on one command queue all give the result of a default instance, bit for bit."""
    import torch
    wl = golden_workload(**CASES["base_2layer_ragged"])
    proto, model = _files(wl)
    x2 = np.ascontiguousarray(wl.x * np.float32(0.5))

    def run(inst, x):
        inst.set_input("x", x)
        inst.set_input("mask", wl.mask_add)
        inst.forward()
        inst.forward()
        return inst.get_output()

    plain = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    want1, want2 = run(plain, wl.x), run(plain, x2)
    assert not np.array_equal(want1, want2)

    ext = rt.Instance(proto, model, device=rt.DEVICE_CUDA, share_memory_mode=rt.SHARE_MEMORY_FROM_EXTERNAL)
    size = ext.forward_memory_size()
    assert size > wl.x.nbytes
    block = torch.full((size + 512,), 0x5A, dtype=torch.uint8, device=cuda_device)
    ext.set_forward_memory(block.data_ptr())
    assert np.array_equal(run(ext, wl.x), want1)
    assert np.array_equal(run(ext, x2), want2)
    torch.cuda.synchronize()
    assert bool((block[size:] == 0x5A).all())          # nothing was written behind the block
    ext.close()

    a = rt.Instance(proto, model, device=rt.DEVICE_CUDA, share_memory_mode=rt.SHARE_MEMORY_ONE_THREAD)
    b = rt.Instance(proto, model, device=rt.DEVICE_CUDA, share_memory_mode=rt.SHARE_MEMORY_ONE_THREAD)
    for _ in range(2):                                  # the instances take turns on the shared blob memory
        assert np.array_equal(run(a, wl.x), want1)
        assert np.array_equal(run(b, x2), want2)
    a.close()
    b.close()

    c = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    c.share_command_queue(plain)
    assert c.command_queue() == plain.command_queue()
    for _ in range(2):
        assert np.array_equal(run(c, x2), want2)
        assert np.array_equal(run(plain, wl.x), want1)
    c.close()
    plain.close()
