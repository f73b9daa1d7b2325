"""Synthetic BERT-style encoder models in TNN's own formats, and the seeded weights/inputs of the benchmark configs.

The reference's BERT model files are download-only, so every workload here is synthetic: weights ~ N(0, 0.02),
biases 0, LayerNorm gamma 1 / beta 0 / eps 1e-12, activations ~ N(0, 1), drawn from numpy `default_rng(seed)` in a
fixed order (per layer Wq, Wk, Wv, Wo, W1, W2; then activations; then lengths).  `randomize_affine=True` additionally
draws non-trivial biases / gamma / beta so that tests exercise those terms.

`write_tnn_model` emits the UNFUSED graph exactly as a converter would (MatMul, Add, Reshape, Permute, Mul, Softmax,
LayerNorm, GELU layers) as `.tnnproto` text + `.tnnmodel` binary:
  * proto grammar: source/tnn/interpreter/tnn/model_interpreter.cc:174-398 (header line, inputs, blobs, outputs, layers)
  * model binary : source/tnn/interpreter/tnn/model_interpreter.cc:400-476, source/tnn/interpreter/tnn/objseri.h:57-167
    (magic, layer count, per-layer {type enum, type string, name, RawBuffer}, then the constant map)
so that the very same files run on the reference's DEVICE_X86 and on DEVICE_CUDA through the fusion pass.
"""
import struct
from dataclasses import dataclass, field

import numpy as np

MAGIC = 0x0FABC0002   # untyped-input proto / model magic (source/tnn/interpreter/tnn/objseri.h:29-30)
MAGIC_RAW = 0x0FABC0004
# LayerType enum values used in the binary (source/tnn/core/layer_type.h); the parser keys on the type string.
_TYPE_ID = {"MatMul": 105, "Add": 38, "Mul": 42, "Gather": 104, "Sub": 108, "Div": 175}


@dataclass
class EncoderConfig:
    layers: int = 12
    hidden: int = 768
    heads: int = 12
    ffn: int = 3072
    ln_eps: float = 1e-12
    with_ffn: bool = True      # False: attention block + residual + LayerNorm only (config 1)

    @property
    def head_dim(self):
        return self.hidden // self.heads


BERT_BASE = EncoderConfig(12, 768, 12, 3072)
BERT_LARGE = EncoderConfig(24, 1024, 16, 4096)


@dataclass
class LayerWeights:
    wq: np.ndarray
    wk: np.ndarray
    wv: np.ndarray
    wo: np.ndarray
    bq: np.ndarray
    bk: np.ndarray
    bv: np.ndarray
    bo: np.ndarray
    ln1_g: np.ndarray
    ln1_b: np.ndarray
    w1: np.ndarray = None
    b1: np.ndarray = None
    w2: np.ndarray = None
    b2: np.ndarray = None
    ln2_g: np.ndarray = None
    ln2_b: np.ndarray = None


@dataclass
class Workload:
    cfg: EncoderConfig
    weights: list
    x: np.ndarray            # [B, S, H] fp32
    lengths: np.ndarray      # [B] int
    mask_add: np.ndarray     # [B, 1, 1, S] fp32: 0 valid, -10000 padded
    meta: dict = field(default_factory=dict)


def make_workload(cfg, batch, seq, seed=0, length_range=None, randomize_affine=False, num_layers=None):
    """Seeded weights + inputs.  `length_range=(lo, hi)` draws integer lengths ~ Uniform[lo, hi]; None = all full."""
    rng = np.random.default_rng(seed)
    H, F = cfg.hidden, cfg.ffn
    L = cfg.layers if num_layers is None else num_layers
    ws = []
    for _ in range(L):
        def w(k, n):
            return rng.normal(0.0, 0.02, (k, n)).astype(np.float32)
        wq, wk, wv, wo = w(H, H), w(H, H), w(H, H), w(H, H)
        w1 = w(H, F) if cfg.with_ffn else None
        w2 = w(F, H) if cfg.with_ffn else None
        z = lambda n: np.zeros((n,), np.float32)  # noqa: E731
        o = lambda n: np.ones((n,), np.float32)   # noqa: E731
        lw = LayerWeights(wq, wk, wv, wo, z(H), z(H), z(H), z(H), o(H), z(H))
        if cfg.with_ffn:
            lw.w1, lw.b1, lw.w2, lw.b2, lw.ln2_g, lw.ln2_b = w1, z(F), w2, z(H), o(H), z(H)
        ws.append(lw)
    x = rng.normal(0.0, 1.0, (batch, seq, H)).astype(np.float32)
    if length_range is None:
        lengths = np.full((batch,), seq, np.int64)
    else:
        lengths = rng.integers(length_range[0], length_range[1] + 1, size=(batch,))
    if randomize_affine:
        r2 = np.random.default_rng(seed + 7919)
        for lw in ws:
            for name in ("bq", "bk", "bv", "bo", "b1", "b2"):
                a = getattr(lw, name)
                if a is not None:
                    setattr(lw, name, r2.normal(0, 0.1, a.shape).astype(np.float32))
            for name in ("ln1_g", "ln2_g"):
                a = getattr(lw, name)
                if a is not None:
                    setattr(lw, name, (1.0 + r2.normal(0, 0.1, a.shape)).astype(np.float32))
            for name in ("ln1_b", "ln2_b"):
                a = getattr(lw, name)
                if a is not None:
                    setattr(lw, name, r2.normal(0, 0.1, a.shape).astype(np.float32))
    mask = np.zeros((batch, 1, 1, seq), np.float32)
    for b in range(batch):
        mask[b, 0, 0, int(lengths[b]):] = -10000.0
    return Workload(cfg, ws, x, np.asarray(lengths, np.int64), mask,
                    {"batch": batch, "seq": seq, "seed": seed, "layers": L})


# The five benchmark configurations (sizes only; `scale` shrinks batch for tests that must finish in seconds).
def config_workload(index, batch=None, num_layers=None, dtype_note=None):
    if index == 1:
        cfg = EncoderConfig(1, 768, 12, 3072, with_ffn=False)
        return make_workload(cfg, batch or 1, 128, seed=0)
    if index == 2:
        return make_workload(BERT_BASE, batch or 64, 128, seed=0, num_layers=num_layers)
    if index == 3:
        return make_workload(BERT_BASE, batch or 32, 256, seed=0, length_range=(16, 256), num_layers=num_layers)
    if index == 4:
        return make_workload(BERT_LARGE, batch or 64, 384, seed=0, length_range=(128, 384), num_layers=num_layers)
    if index == 5:
        return make_workload(BERT_BASE, batch or 1024, 128, seed=0, num_layers=num_layers)
    raise ValueError("config index 1..5")


# --------------------------------------------------------------------------------------------- TNN file writers
def _pstr(s):
    b = s.encode()
    return struct.pack("<i", len(b)) + b


def _raw(a):
    """A RawBuffer record: fp32 (data type 0) unless the array is int32 (data type 3, include/tnn/core/common.h:31-49)."""
    a = np.asarray(a)
    if a.dtype == np.int32:
        a, code = np.ascontiguousarray(a), 3
    else:
        a, code = np.ascontiguousarray(a, dtype=np.float32), 0
    dims = a.shape
    return (struct.pack("<Iii", MAGIC_RAW, code, a.nbytes) + struct.pack("<i", len(dims)) +
            b"".join(struct.pack("<i", d) for d in dims) + a.tobytes())


def _encoder_graph(wl, input_name, mask_name, style="resource"):
    """Layer lines, resource records and constants of the unfused encoder graph; returns them with the output name.
    `style` "resource": weights and biases are layer resources and the scale is Mul(1/sqrt(d)), the form the TNN
    converters write after constant folding; "export": weights and biases are entries of the constant map consumed as
    second inputs (MatMul weight_position -1; every second bias written as Add(bias, x)) and the scale is
    Div(sqrt(d)), the form of a plain converter export; "export_shapes": the export form whose head-split and
    head-merge Reshape layers take their target shape as a second input computed in the graph — Shape(x) ->
    Gather(index 0), Gather(index 1) -> Concat with the constant head count and head size — as exporters write a
    reshape whose batch and sequence dimensions are dynamic (source/tnn/layer/reshape_layer.cc:72-91 fills the
    Reshape's shape from that input once the constant folder has evaluated it)."""
    cfg = wl.cfg
    B, S, H = wl.x.shape
    NH, D, F = cfg.heads, cfg.head_dim, cfg.ffn
    layers, res, consts = [], [], {}

    def layer(t, name, ins, outs, params=""):
        layers.append('"%s %s %d %d %s %s %s,"' % (t, name, len(ins), len(outs), " ".join(ins), " ".join(outs), params))

    def resource(t, name, arr):
        res.append(struct.pack("<i", _TYPE_ID[t]) + _pstr(t) + _pstr(name) + _raw(arr))

    n_linear = [0]

    def gather_resource(name, index):
        # GatherLayerResource: no data, indices = int32 [1] (gather_layer_interpreter.cc:29-43)
        res.append(struct.pack("<i", _TYPE_ID["Gather"]) + _pstr("Gather") + _pstr(name) + struct.pack("<i", 0) +
                   struct.pack("<i", 1) + _raw(np.array([index], np.int32)))

    def reshape(name, x, tail, static_params):
        """Reshape of [B, S, ...] to [B, S] + tail: static parameters, or (export_shapes) a shape computed in the graph."""
        if style != "export_shapes":
            layer("Reshape", name, [x], [name], static_params)
            return name
        layer("Shape", name + "_shape", [x], [name + "_shape"])
        parts = []
        for i in (0, 1):
            g = "%s_dim%d" % (name, i)
            layer("Gather", g, [name + "_shape"], [g], "0 0 1")
            gather_resource(g, i)
            parts.append(g)
        for j, v in enumerate(tail):
            c = "%s_c%d" % (name, j)
            consts[c] = np.array([v], np.int32)
            parts.append(c)
        layer("Concat", name + "_target", parts, [name + "_target"], "0")
        layer("Reshape", name, [x, name + "_target"], [name], "0 0 0 0")
        return name

    def linear(name, x, w, b):
        if style in ("export", "export_shapes"):
            n_linear[0] += 1
            consts[name + "_w"] = w
            consts[name + "_bias"] = b.reshape(-1)
            layer("MatMul", name + "_mm", [x, name + "_w"], [name + "_mm"], "-1")
            ins = [name + "_mm", name + "_bias"] if n_linear[0] % 2 else [name + "_bias", name + "_mm"]
            layer("Add", name + "_b", ins, [name + "_b"], "-1")
            return name + "_b"
        layer("MatMul", name + "_mm", [x], [name + "_mm"], "1")
        resource("MatMul", name + "_mm", w)
        layer("Add", name + "_b", [name + "_mm"], [name + "_b"], "1")
        resource("Add", name + "_b", b.reshape(-1))   # explicit [N] dims: see MultidirBroadcastLayer's guess rule
        return name + "_b"

    def lnorm(name, x, g, be):
        consts[name + "_g"] = g
        consts[name + "_be"] = be
        layer("LayerNorm", name, [x, name + "_g", name + "_be"], [name], "1 %.1e" % cfg.ln_eps)
        return name

    x = input_name
    for li, lw in enumerate(wl.weights):
        p = "l%d_" % li
        for n, w, b, perm in (("q", lw.wq, lw.bq, "0 2 1 3"), ("k", lw.wk, lw.bk, "0 2 3 1"),
                              ("v", lw.wv, lw.bv, "0 2 1 3")):
            o = linear(p + n, x, w, b)
            reshape(p + n + "_r", o, (NH, D), "0 4 4 0 0 %d %d 0" % (NH, D))
            layer("Permute", p + n + "_p", [p + n + "_r"], [p + n + "_p"], "4 " + perm)
        layer("MatMul", p + "qk", [p + "q_p", p + "k_p"], [p + "qk"], "-1")
        if style in ("export", "export_shapes"):
            layer("Div", p + "qk_s", [p + "qk"], [p + "qk_s"], "1")
            resource("Div", p + "qk_s", np.array([np.sqrt(D)], np.float32))
        else:
            layer("Mul", p + "qk_s", [p + "qk"], [p + "qk_s"], "1")
            resource("Mul", p + "qk_s", np.array([1.0 / np.sqrt(D)], np.float32))
        layer("Add", p + "qk_m", [p + "qk_s", mask_name], [p + "qk_m"], "-1")
        layer("Softmax", p + "sm", [p + "qk_m"], [p + "sm"], "3")
        layer("MatMul", p + "ctx", [p + "sm", p + "v_p"], [p + "ctx"], "-1")
        layer("Permute", p + "ctx_p", [p + "ctx"], [p + "ctx_p"], "4 0 2 1 3")
        reshape(p + "ctx_r", p + "ctx_p", (H,), "0 3 3 0 0 %d 0" % H)
        o = linear(p + "o", p + "ctx_r", lw.wo, lw.bo)
        layer("Add", p + "res1", [o, x], [p + "res1"], "-1")
        a = lnorm(p + "ln1", p + "res1", lw.ln1_g, lw.ln1_b)
        if cfg.with_ffn:
            f1 = linear(p + "f1", a, lw.w1, lw.b1)
            layer("GELU", p + "gelu", [f1], [p + "gelu"])
            f2 = linear(p + "f2", p + "gelu", lw.w2, lw.b2)
            layer("Add", p + "res2", [f2, a], [p + "res2"], "-1")
            x = lnorm(p + "ln2", p + "res2", lw.ln2_g, lw.ln2_b)
        else:
            x = a
    return layers, res, consts, x


def _write_files(proto_path, model_path, magic, inputs_line, outputs, layers, res, consts):
    blobs = set()
    for ln in layers:
        t = ln.strip('",').split()
        ni, no = int(t[2]), int(t[3])
        blobs.update(t[4:4 + ni + no])
    proto = ['"1 %d 1 %d ,"' % (len(blobs), magic),
             '"%s ,"' % inputs_line,
             '" ' + " ".join(sorted(blobs)) + ' ,"',
             '"%s ,"' % " ".join(outputs),
             '" %d ,"' % len(layers)] + layers
    with open(proto_path, "w") as fh:
        fh.write("\n".join(proto) + "\n")
    m = struct.pack("<I", MAGIC) + struct.pack("<i", len(res)) + b"".join(res)
    m += struct.pack("<Ii", MAGIC, len(consts)) + b"".join(_pstr(k) + _raw(v) for k, v in consts.items())
    with open(model_path, "wb") as fh:
        fh.write(m)


def make_pooler(hidden, seed=0):
    """Weights of the BERT pooler head, tanh(x . Wp + bp): (Wp [H, H] fp32, bp [H])."""
    rng = np.random.default_rng(seed + 104729)
    return (rng.normal(0.0, 0.02, (hidden, hidden)).astype(np.float32), rng.normal(0.0, 0.1, hidden).astype(np.float32))


def _pooler_graph(x, pooler):
    """MatMul -> Add(bias) -> Tanh over every token row of `x` (a converter's graph first slices the [CLS] row; the
    slice is a strided view for the kernel and is left out here).  Type ids: Tanh has no resource."""
    wp, bp = pooler
    layers, res = [], []
    layers.append('"MatMul pool_mm 1 1 %s pool_mm 1,"' % x)
    res.append(struct.pack("<i", _TYPE_ID["MatMul"]) + _pstr("MatMul") + _pstr("pool_mm") + _raw(wp))
    layers.append('"Add pool_b 1 1 pool_mm pool_b 1,"')
    res.append(struct.pack("<i", _TYPE_ID["Add"]) + _pstr("Add") + _pstr("pool_b") + _raw(bp.reshape(-1)))
    layers.append('"Tanh pooled 1 1 pool_b pooled ,"')
    return layers, res, "pooled"


def make_qa_head(hidden, seed=0, outputs=2):
    """Weights of the span-extraction head, x . Wq + bq: (Wq [H, outputs] fp32, bq [outputs])."""
    rng = np.random.default_rng(seed + 15485863)
    return (rng.normal(0.0, 0.05, (hidden, outputs)).astype(np.float32), rng.normal(0.0, 0.1, outputs).astype(np.float32))


QA_OUTPUTS = ("unstack:0", "unstack:1")   # the names the reading-comprehension demo reads
                                          # (examples/linux/src/BertReadingComprehension/BertReadingComprehension.cc:109)


def _qa_graph(x, qa):
    """MatMul [H, 2] -> Add(bias) -> SplitV(axis 2, sizes 1, 1) -> Squeeze(axis 2) x 2: start / end logits [B, S].
    SplitV parameters: axis, slice count, slices (splitv_layer_interpreter.cc); Squeeze: axis count, axes."""
    wq, bq = qa
    assert wq.shape[1] == 2
    layers, res = [], []
    layers.append('"MatMul qa_mm 1 1 %s qa_mm 1,"' % x)
    res.append(struct.pack("<i", _TYPE_ID["MatMul"]) + _pstr("MatMul") + _pstr("qa_mm") + _raw(wq))
    layers.append('"Add qa_b 1 1 qa_mm qa_b 1,"')
    res.append(struct.pack("<i", _TYPE_ID["Add"]) + _pstr("Add") + _pstr("qa_b") + _raw(bq.reshape(-1)))
    layers.append('"SplitV qa_split 1 2 qa_b qa_s0 qa_s1 2 2 1 1 ,"')
    layers.append('"Squeeze qa_sq0 1 1 qa_s0 %s 1 2 ,"' % QA_OUTPUTS[0])
    layers.append('"Squeeze qa_sq1 1 1 qa_s1 %s 1 2 ,"' % QA_OUTPUTS[1])
    return layers, res, list(QA_OUTPUTS)


def write_tnn_model(wl, proto_path, model_path, input_name="x", mask_name="mask", pooler=None, input_dtype=None,
                    qa=None, style="resource"):
    """Write the unfused encoder graph of `wl` as tnnproto + tnnmodel.  Returns the output blob name (a list of two
    names with `qa`).  `pooler` (from make_pooler) appends the pooler head MatMul -> Add -> Tanh to the last layer's
    output; `qa` (from make_qa_head) appends the span-extraction head with its two unstacked outputs.  `input_dtype`
    "half" / "bf16" declares the activation input as a typed (v2) half-precision blob (include/tnn/core/common.h
    DataType: 1 = half, 4 = bfp16), so that a half-precision Mat reaches the device without conversion."""
    B, S, H = wl.x.shape
    layers, res, consts, out = _encoder_graph(wl, input_name, mask_name, style)
    if pooler is not None:
        l2, r2, out = _pooler_graph(out, pooler)
        layers, res = layers + l2, res + r2
    outs = [out]
    if qa is not None:
        l2, r2, outs = _qa_graph(out, qa)
        layers, res = layers + l2, res + r2
        out = outs
    if input_dtype is not None:
        code = {"half": 1, "bf16": 4}[input_dtype]
        _write_files(proto_path, model_path, MAGIC_RAW,
                     "%s 4 %d 1 1 %d 0 : %s 3 %d %d %d %d" % (mask_name, B, S, input_name, B, S, H, code),
                     outs, layers, res, consts)
        return out
    _write_files(proto_path, model_path, MAGIC, "%s %d 1 1 %d : %s %d %d %d" % (mask_name, B, S, input_name, B, S, H),
                 outs, layers, res, consts)
    return out


# --------------------------------------------------------------------------------------------- embedding front-end
@dataclass
class FrontendWorkload:
    """The step before the encoder path: token / segment / position embeddings + LayerNorm, and the additive key mask
    built from the 0/1 input mask (int32 graph inputs as in examples/base/bert_tokenizer.cc:351-355)."""
    hidden: int
    word_emb: np.ndarray      # [vocab, H] fp32
    type_emb: np.ndarray      # [type_vocab, H]
    pos_emb: np.ndarray       # [max_pos, H]
    gamma: np.ndarray
    beta: np.ndarray
    eps: float
    input_ids: np.ndarray     # [B, S] int32
    segment_ids: np.ndarray   # [B, S] int32
    input_mask: np.ndarray    # [B, S] int32, 1 = token, 0 = padding
    lengths: np.ndarray


def make_frontend_workload(hidden, batch, seq, vocab=30522, type_vocab=2, max_pos=512, seed=0, length_range=None,
                           eps=1e-12):
    rng = np.random.default_rng(seed)
    n = lambda *shape: rng.normal(0.0, 0.02, shape).astype(np.float32)   # noqa: E731
    word, typ, pos = n(vocab, hidden), n(type_vocab, hidden), n(max_pos, hidden)
    gamma = (1.0 + rng.normal(0, 0.1, hidden)).astype(np.float32)
    beta = rng.normal(0, 0.1, hidden).astype(np.float32)
    ids = rng.integers(0, vocab, size=(batch, seq)).astype(np.int32)
    seg = rng.integers(0, type_vocab, size=(batch, seq)).astype(np.int32)
    if length_range is None:
        lengths = np.full((batch,), seq, np.int64)
    else:
        lengths = rng.integers(length_range[0], length_range[1] + 1, size=(batch,))
    mask = (np.arange(seq)[None, :] < lengths[:, None]).astype(np.int32)
    return FrontendWorkload(hidden, word, typ, pos, gamma, beta, eps, ids, seg, mask, np.asarray(lengths, np.int64))


def write_tnn_frontend_model(fw, proto_path, model_path):
    """The unfused front-end graph as a converter emits it: Gather(word) + Gather(segment) -> Add -> Add(position
    slice, a constant) -> LayerNorm = `emb_out`; Unsqueeze(1,2) -> Cast(float) -> Sub(1 - m) -> Mul(-10000) =
    `mask_add`.  Typed (v2) inputs: input_ids, segment_ids, input_mask int32 [B, S].
    Grammar: Gather source/tnn/interpreter/tnn/layer_interpreter/gather_layer_interpreter.cc:23-47, Unsqueeze
    unsqueeze_layer_interpreter.cc:20-30, Cast cast_layer_interpreter.cc:21-25, Sub sub_layer_interpreter.cc:23-47."""
    layers, res, consts = _frontend_graph(fw)
    _write_files(proto_path, model_path, MAGIC_RAW, _frontend_inputs(fw), ["emb_out", "mask_add"], layers, res, consts)
    return "emb_out", "mask_add"


def _frontend_inputs(fw):
    B, S = fw.input_ids.shape
    return " : ".join("%s 2 %d %d 3" % (n, B, S) for n in ("input_ids", "segment_ids", "input_mask"))


def _frontend_graph(fw):
    B, S = fw.input_ids.shape
    H = fw.hidden
    layers, res, consts = [], [], {}

    def layer(t, name, ins, outs, params=""):
        layers.append('"%s %s %d %d %s %s %s,"' % (t, name, len(ins), len(outs), " ".join(ins), " ".join(outs), params))

    def head(t, name):
        return struct.pack("<i", _TYPE_ID[t]) + _pstr(t) + _pstr(name)

    layer("Gather", "word_e", ["input_ids"], ["word_e"], "0 1 0")
    res.append(head("Gather", "word_e") + struct.pack("<i", 1) + _raw(fw.word_emb) + struct.pack("<i", 0))
    layer("Gather", "type_e", ["segment_ids"], ["type_e"], "0 1 0")
    res.append(head("Gather", "type_e") + struct.pack("<i", 1) + _raw(fw.type_emb) + struct.pack("<i", 0))
    layer("Add", "wt_e", ["word_e", "type_e"], ["wt_e"], "-1")
    layer("Add", "wtp_e", ["wt_e"], ["wtp_e"], "1")
    res.append(head("Add", "wtp_e") + _raw(fw.pos_emb[:S].reshape(1, S, H)))
    consts["emb_g"], consts["emb_be"] = fw.gamma, fw.beta
    layer("LayerNorm", "emb_out", ["wtp_e", "emb_g", "emb_be"], ["emb_out"], "1 %.1e" % fw.eps)
    layer("Unsqueeze", "mask_u", ["input_mask"], ["mask_u"], "2 1 2")
    layer("Cast", "mask_f", ["mask_u"], ["mask_f"], "0")
    layer("Sub", "mask_inv", ["mask_f"], ["mask_inv"], "0")
    res.append(head("Sub", "mask_inv") + _raw(np.array([1.0], np.float32)))
    layer("Mul", "mask_add", ["mask_inv"], ["mask_add"], "1")
    res.append(head("Mul", "mask_add") + _raw(np.array([-10000.0], np.float32)))
    return layers, res, consts


def write_tnn_bert_model(fw, wl, proto_path, model_path):
    """Front-end + encoder as one graph, the shape of a converted BERT: int32 inputs input_ids / segment_ids /
    input_mask [B, S]; `emb_out` feeds the first encoder layer, `mask_add` every attention block.  Returns the output
    blob name.  (`wl.x` and `wl.mask_add` are not used: the graph computes them.)"""
    assert fw.hidden == wl.cfg.hidden and fw.input_ids.shape == wl.x.shape[:2]
    l1, r1, c1 = _frontend_graph(fw)
    l2, r2, c2, out = _encoder_graph(wl, "emb_out", "mask_add")
    c1.update(c2)
    _write_files(proto_path, model_path, MAGIC_RAW, _frontend_inputs(fw), [out], l1 + l2, r1 + r2, c1)
    return out


# --------------------------------------------------------------------------------------------- FLOP accounting
def layer_flops(seq_len, hidden, ffn=None, with_ffn=True):
    """Algorithmic FLOPs of one encoder layer for one sequence of `seq_len` tokens (2 per MAC; GEMMs + QK^T + PV)."""
    ffn = 4 * hidden if ffn is None else ffn
    f = 8 * seq_len * hidden * hidden + 4 * seq_len * seq_len * hidden
    if with_ffn:
        f += 4 * seq_len * hidden * ffn
    return f


def workload_flops(wl, effective=True):
    cfg = wl.cfg
    S = wl.x.shape[1]
    L = len(wl.weights)
    lens = wl.lengths if effective else np.full_like(wl.lengths, S)
    return int(sum(L * layer_flops(int(n), cfg.hidden, cfg.ffn, cfg.with_ffn) for n in lens))
