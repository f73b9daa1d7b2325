"""CPU restatement (numpy, fp32) of the reference's arithmetic for the transformer-encoder attention path.

TEST INFRASTRUCTURE ONLY — this module is the checker for tests/, smoke() and bench.py's cpu_baseline leg.  No product
code imports it; the product path is the CUDA library and fails loudly without it.

Parity pin: `oracle/make_golden.py` runs the reference's own DEVICE_X86 and DEVICE_NAIVE implementations (built
unmodified from the reference sources by oracle/build_ref.py) on seeded models and commits their outputs under
tests/golden/; tests/test_oracle.py checks this restatement against those files.

Each function follows the unfused TNN layer it restates:
  matmul      X86MatMulLayerAcc::DoForward  source/tnn/device/x86/acc/x86_mat_mul_layer_acc.cc:49-114 (fp32 sgemm,
              batch broadcast); the naive acc accumulates in double, source/tnn/device/cpu/acc/cpu_mat_mul_layer_acc.cc:102-111
  add / mul   X86BinaryOpLayerAcc (numpy-style broadcasting) source/tnn/device/x86/acc/x86_binary_op_layer_acc.cc:536-805
  softmax     X86SoftMaxLayerAcc  source/tnn/device/x86/acc/x86_softmax_layer_acc.cc:28-83,153-187
              (row max, exp(x - max), sum, multiply by the reciprocal of the sum)
  layer_norm  X86LayerNormLayerAcc  source/tnn/device/x86/acc/x86_layer_norm_layer_acc.cc:26-86
              (one pass: sum x, sum x^2; var = max(E[x^2] - mean^2, 0); 1/sqrt(var + eps);
               y = x*(rstd*gamma) + (beta - mean*rstd*gamma))
  gelu        0.5*x*(1+erf(x*0.707106793288165))  source/tnn/device/x86/acc/x86_gelu_layer_acc.cc:22-62 (its vector
              path evaluates erf by a rational-exponential fit with |error| ~1.2e-7; exact erf is used here)
  reshape / permute   source/tnn/layer/reshape_layer.cc:40-91, source/tnn/layer/permute_layer.cc:28-63
"""
import numpy as np

try:
    from scipy.special import erf as _erf
except Exception:  # pragma: no cover - scipy is present in this image
    import math
    _erf = np.vectorize(math.erf, otypes=[np.float64])

F32 = np.float32


def matmul(a, b):
    return np.matmul(a.astype(F32, copy=False), b.astype(F32, copy=False)).astype(F32)


def softmax_last(x):
    m = np.max(x, axis=-1, keepdims=True)
    e = np.exp((x - m).astype(F32)).astype(F32)
    s = np.sum(e, axis=-1, keepdims=True, dtype=F32)
    return (e * (F32(1.0) / s)).astype(F32)


def layer_norm(x, gamma, beta, eps):
    n = F32(x.shape[-1])
    sum_x = np.sum(x, axis=-1, keepdims=True, dtype=F32)
    sum_x2 = np.sum(x * x, axis=-1, keepdims=True, dtype=F32)
    mean = sum_x / n
    var = np.maximum(sum_x2 / n - mean * mean, F32(0))
    rstd = (F32(1.0) / np.sqrt((var + F32(eps)).astype(F32))).astype(F32)
    scale = rstd * gamma.astype(F32)
    return (x * scale + (beta.astype(F32) - scale * mean)).astype(F32)


def gelu(x):
    return (F32(0.5) * x * (F32(1.0) + _erf(x.astype(np.float64) * 0.707106793288165).astype(F32))).astype(F32)


def attention_block(x, mask_add, lw, heads, eps):
    """MatMul+Add x3 -> Reshape/Permute -> MatMul -> Mul(1/sqrt d) -> Add(mask) -> Softmax -> MatMul -> Permute/Reshape
    -> MatMul+Add -> Add(residual) -> LayerNorm."""
    B, S, H = x.shape
    D = H // heads
    q = matmul(x, lw.wq) + lw.bq
    k = matmul(x, lw.wk) + lw.bk
    v = matmul(x, lw.wv) + lw.bv
    q = q.reshape(B, S, heads, D).transpose(0, 2, 1, 3)
    k = k.reshape(B, S, heads, D).transpose(0, 2, 3, 1)
    v = v.reshape(B, S, heads, D).transpose(0, 2, 1, 3)
    scores = matmul(q, k) * F32(1.0 / np.sqrt(D))
    if mask_add is not None:
        scores = scores + mask_add.reshape(B, 1, 1, S).astype(F32)
    p = softmax_last(scores.astype(F32))
    ctx = matmul(p, v).transpose(0, 2, 1, 3).reshape(B, S, H)
    o = matmul(ctx, lw.wo) + lw.bo
    return layer_norm((o + x).astype(F32), lw.ln1_g, lw.ln1_b, eps)


def encoder_layer(x, mask_add, lw, cfg):
    a = attention_block(x, mask_add, lw, cfg.heads, cfg.ln_eps)
    if not cfg.with_ffn:
        return a
    f1 = gelu((matmul(a, lw.w1) + lw.b1).astype(F32))
    f2 = matmul(f1, lw.w2) + lw.b2
    return layer_norm((f2 + a).astype(F32), lw.ln2_g, lw.ln2_b, cfg.ln_eps)


def encoder_forward(wl, x=None, mask_add=None, upto_layer=None):
    """Whole stack on a Workload (tnn_b200.model_synth.Workload); returns fp32 [B, S, H]."""
    h = (wl.x if x is None else x).astype(F32)
    m = wl.mask_add if mask_add is None else mask_add
    for i, lw in enumerate(wl.weights):
        if upto_layer is not None and i >= upto_layer:
            break
        h = encoder_layer(h, m, lw, wl.cfg)
    return h


# ---- stand-alone pieces used by the per-kernel parity tests
def linear(x, w_kn, bias=None, residual=None, act=None):
    y = matmul(x, w_kn)
    if bias is not None:
        y = y + bias.astype(F32)
    if act == "gelu":
        y = gelu(y.astype(F32))
    if act == "tanh":   # source/tnn/device/x86/acc/x86_tanh_layer_acc.cc:19-31
        y = np.tanh(y.astype(F32))
    if residual is not None:
        y = y + residual.astype(F32)
    return y.astype(F32)


def qa_head(x, w_kn, bias):
    """Span-extraction head: logits = x . W + b with W [H, N], then one [B, S] array per output ("unstack": SplitV along
    the last axis, source/tnn/device/x86/acc/x86_splitv_layer_acc.cc:23, + Squeeze of that axis)."""
    y = linear(x, w_kn, bias)
    return tuple(np.ascontiguousarray(y[..., n]) for n in range(y.shape[-1]))


def attention_core(q, k, v, mask_add, scale):
    """q, k, v: [B, heads, S, D] fp32; mask_add: [B, S] or None.  Returns [B, heads, S, D]."""
    scores = matmul(q, k.transpose(0, 1, 3, 2)) * F32(scale)
    if mask_add is not None:
        B, S = mask_add.shape
        scores = scores + mask_add.reshape(B, 1, 1, S).astype(F32)
    return matmul(softmax_last(scores.astype(F32)), v)


# --------------------------------------------------------------------------------------------- embedding front-end
def gather_rows(table, indices):
    """Gather along axis 0 with a resource table: out[i...] = table[indices[i...]]
    (source/tnn/device/x86/acc/x86_gather_layer_acc.cc:23-76: a memcpy per index; an index outside [0, rows) is an
    error there, TNNERR_MODEL_ERR)."""
    idx = np.asarray(indices)
    if idx.size and (idx.min() < 0 or idx.max() >= table.shape[0]):
        raise IndexError("gather index out of range")
    return table[idx]


def embedding_frontend(fw):
    """word + segment + position embeddings, LayerNorm; the additive key mask (1 - m) * -10000 as [B,1,1,S].
    Gather as above; Add: source/tnn/device/x86/acc/x86_add_layer_acc.cc:66-92 (the position slice [1,S,H] is
    broadcast over the batch); LayerNorm: x86_layer_norm_layer_acc.cc:26-86; Unsqueeze / Cast(int32 -> float) move no
    values; Sub with the constant as input 0 (weight_input_index 0) computes 1 - m, Mul scales by -10000
    (source/tnn/device/x86/acc/x86_binary_op_layer_acc.cc:536-805)."""
    B, S = fw.input_ids.shape
    e = gather_rows(fw.word_emb, fw.input_ids) + gather_rows(fw.type_emb, fw.segment_ids)
    e = e + fw.pos_emb[:S].reshape(1, S, -1)
    out = layer_norm(e.astype(np.float32), fw.gamma, fw.beta, fw.eps)
    mask_add = ((np.float32(1.0) - fw.input_mask.astype(np.float32)) * np.float32(-10000.0)).reshape(B, 1, 1, S)
    return out.astype(np.float32), mask_add.astype(np.float32)
