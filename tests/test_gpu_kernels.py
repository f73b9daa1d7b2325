"""GPU: each kernel of the path through the C ABI against the CPU oracle on the same seeded inputs."""
import numpy as np
import pytest
import torch

from oracle import bert_oracle
from tnn_b200 import capi, ops
from util import cosine, max_abs

pytestmark = pytest.mark.gpu

DT = {"f16": torch.float16, "bf16": torch.bfloat16}
# one half-precision rounding of an O(1) value: 2^-11 (fp16) / 2^-8 (bf16); sums of K products stay fp32
ATOL = {"f16": 4e-3, "bf16": 3e-2}


def _np(t):
    return t.detach().float().cpu().numpy()


def _rounded(a, dt):
    """numpy fp32 -> rounded through the half dtype (what the kernel's operands hold) -> fp32."""
    return torch.from_numpy(a).to(dt).float().numpy()


@pytest.fixture(autouse=True)
def _status_clean(cuda_device):
    yield
    torch.cuda.synchronize()
    assert capi.device_status() == capi.OK


@pytest.mark.parametrize("dt", ["f16", "bf16"])
# bn > 0: tile width on CTA-pair tiles (256 x bn) when M > 128; bn < 0: single-CTA tiles (128 x -bn); 0: auto
@pytest.mark.parametrize("M,N,K,bn", [
    (128, 128, 64, 128), (128, 256, 128, 256), (256, 64, 64, 64),
    (512, 768, 768, 0), (300, 2304, 768, 0), (1, 8, 8, 0), (129, 136, 72, 128),
    (1024, 3072, 768, 256), (640, 768, 3072, 128),
    (256, 256, 64, 256), (257, 392, 200, 192), (1000, 768, 768, 192), (8192, 768, 768, 0),
    (900, 2304, 768, -256), (384, 200, 136, -128), (512, 72, 64, -64), (700, 1024, 1024, 64),
])
def test_linear_bias(cuda_device, dt, M, N, K, bn):
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    x = rng.normal(0, 1, (M, K)).astype(np.float32)
    w = rng.normal(0, 0.05, (K, N)).astype(np.float32)
    b = rng.normal(0, 0.5, (N,)).astype(np.float32)
    xd = torch.from_numpy(x).to(cuda_device).to(DT[dt])
    wd = ops.pack_weight(torch.from_numpy(w).to(cuda_device), DT[dt])
    assert np.array_equal(_np(wd), _rounded(w, DT[dt]).T)          # the pre-pack is exact rounding + transpose
    y = ops.linear(xd, wd, torch.from_numpy(b).to(cuda_device), out_dtype=torch.float32, block_n=bn)
    want = bert_oracle.linear(_rounded(x, DT[dt]), _rounded(w, DT[dt]), b)
    assert max_abs(_np(y), want) < 2e-3 * max(1.0, np.sqrt(K / 64))
    y16 = ops.linear(xd, wd, torch.from_numpy(b).to(cuda_device), block_n=bn)
    assert max_abs(_np(y16), want) < ATOL[dt] * max(1.0, float(np.abs(want).max()))


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("epi", ["gelu", "residual"])
def test_linear_epilogues(cuda_device, dt, epi):
    M, N, K = 384, 1024, 256
    rng = np.random.default_rng(5)
    x = rng.normal(0, 1, (M, K)).astype(np.float32)
    w = rng.normal(0, 0.08, (K, N)).astype(np.float32)
    b = rng.normal(0, 0.5, (N,)).astype(np.float32)
    r = rng.normal(0, 1, (M, N)).astype(np.float32)
    xd = torch.from_numpy(x).to(cuda_device).to(DT[dt])
    wd = ops.pack_weight(torch.from_numpy(w).to(cuda_device), DT[dt])
    bd = torch.from_numpy(b).to(cuda_device)
    xr, wr = _rounded(x, DT[dt]), _rounded(w, DT[dt])
    if epi == "gelu":
        y = ops.linear(xd, wd, bd, epilogue=ops.EPI_BIAS_GELU, out_dtype=torch.float32)
        want = bert_oracle.linear(xr, wr, b, act="gelu")
    else:
        rd = torch.from_numpy(r).to(cuda_device).to(DT[dt])
        y = ops.linear(xd, wd, bd, residual=rd, epilogue=ops.EPI_BIAS_RESIDUAL, out_dtype=torch.float32)
        want = bert_oracle.linear(xr, wr, b, residual=_rounded(r, DT[dt]))
    assert max_abs(_np(y), want) < 4e-3


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K,bn", [(512, 768, 768, 0), (300, 1024, 256, 192), (130, 96, 64, -64), (1000, 3072, 768, 256)])
def test_linear_layernorm_folding(cuda_device, dt, M, N, K, bn):
    """out_stats, folded input LayerNorm and folded residual LayerNorm against the unfused oracle."""
    rng = np.random.default_rng(M + N)
    eps = 1e-12
    t = rng.normal(0.2, 1.5, (M, K)).astype(np.float32)            # a pre-LayerNorm activation
    g = (1 + rng.normal(0, 0.2, (K,))).astype(np.float32)
    be = rng.normal(0, 0.2, (K,)).astype(np.float32)
    w = rng.normal(0, 0.05, (K, N)).astype(np.float32)
    b = rng.normal(0, 0.3, (N,)).astype(np.float32)
    dev = cuda_device
    td = torch.from_numpy(t).to(dev).to(DT[dt])
    tr = _rounded(t, DT[dt])
    # (1) producer: y = x.I-like GEMM writing statistics of its output rows
    w0 = rng.normal(0, 0.05, (K, K)).astype(np.float32)
    st = ops.stats_buffer(M, K, dev)
    y0 = ops.linear(td, ops.pack_weight(torch.from_numpy(w0).to(dev), DT[dt]), None, out_stats=st, block_n=bn)
    y0f = _np(y0).astype(np.float64)
    s = _np(st).astype(np.float64).sum(axis=0)
    # the statistics are taken before the output is rounded to half precision: the sums differ by rounding noise
    atol = 0.15 if dt == "f16" else 1.2
    assert np.allclose(s[:, 0], y0f.sum(axis=1), rtol=0, atol=atol)
    assert np.allclose(s[:, 1], (y0f ** 2).sum(axis=1), rtol=1e-2, atol=atol)
    # (2) consumer with the input LayerNorm folded: LN(y0).W + b
    wf, c1, c2 = ops.fold_layernorm_weight(torch.from_numpy(w).to(dev), torch.from_numpy(g).to(dev),
                                           torch.from_numpy(be).to(dev), torch.from_numpy(b).to(dev), DT[dt])
    out = ops.linear(y0, wf, None, ln_in=(st, c1, c2), ln_eps=eps, out_dtype=torch.float32, block_n=bn)
    ln = bert_oracle.layer_norm(_np(y0), g, be, eps)
    want = bert_oracle.linear(ln, w, b)
    tol = 2e-2 if dt == "f16" else 1.2e-1
    assert max_abs(_np(out), want) < tol
    assert cosine(_np(out), want) > (0.9999 if dt == "f16" else 0.999)
    # (3) residual through a folded LayerNorm: x.W + b + LN(r) with r of width N
    r = rng.normal(-0.1, 2.0, (M, N)).astype(np.float32)
    gr = (1 + rng.normal(0, 0.2, (N,))).astype(np.float32)
    br = rng.normal(0, 0.2, (N,)).astype(np.float32)
    rd = torch.from_numpy(r).to(dev).to(DT[dt])
    # statistics of r from an identity-free route: a GEMM that reproduces r is overkill; compute them with torch ops
    rf = rd.float()
    chunks = (N + 31) // 32
    pad = chunks * 32 - N
    rp = torch.nn.functional.pad(rf, (0, pad)).reshape(M, chunks, 32)
    str_ = torch.stack([rp.sum(-1), (rp * rp).sum(-1)], dim=-1).permute(1, 0, 2).contiguous()
    out2 = ops.linear(td, ops.pack_weight(torch.from_numpy(w).to(dev), DT[dt]), torch.from_numpy(b).to(dev),
                      residual=rd, epilogue=ops.EPI_BIAS_RESIDUAL, out_dtype=torch.float32, block_n=bn,
                      res_ln=(str_, torch.from_numpy(gr).to(dev), torch.from_numpy(br).to(dev)), ln_eps=eps)
    want2 = bert_oracle.linear(tr, _rounded(w, DT[dt]), b) + bert_oracle.layer_norm(_np(rd), gr, br, eps)
    assert max_abs(_np(out2), want2) < 6e-3 * max(1.0, np.sqrt(K / 64))


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("H,rows", [(768, 1000), (1024, 77), (8, 3), (4096, 9), (1536, 64)])
@pytest.mark.parametrize("with_res", [False, True])
def test_add_layernorm(cuda_device, dt, H, rows, with_res):
    rng = np.random.default_rng(H + rows)
    x = rng.normal(0.3, 2.0, (rows, H)).astype(np.float32)
    r = rng.normal(0, 1.0, (rows, H)).astype(np.float32)
    g = (1 + rng.normal(0, 0.2, (H,))).astype(np.float32)
    be = rng.normal(0, 0.2, (H,)).astype(np.float32)
    xd = torch.from_numpy(x).to(cuda_device).to(DT[dt])
    rd = torch.from_numpy(r).to(cuda_device).to(DT[dt]) if with_res else None
    y = ops.add_layernorm(xd, torch.from_numpy(g).to(cuda_device), torch.from_numpy(be).to(cuda_device), 1e-12,
                          residual=rd, out_dtype=torch.float32)
    xin = _rounded(x, DT[dt]) + (_rounded(r, DT[dt]) if with_res else 0)
    want = bert_oracle.layer_norm(xin.astype(np.float32), g, be, 1e-12)
    assert max_abs(_np(y), want) < 2e-4
    # fp32 in / fp32 out: the un-fused LayerNorm layer of the graph
    y32 = ops.add_layernorm(torch.from_numpy(x).to(cuda_device), torch.from_numpy(g).to(cuda_device),
                            torch.from_numpy(be).to(cuda_device), 1e-12)
    assert max_abs(_np(y32), bert_oracle.layer_norm(x, g, be, 1e-12)) < 2e-4


def test_convert_roundtrip_and_tail(cuda_device):
    for n in (1, 7, 8, 1000, 4099):
        a = torch.randn(n, device=cuda_device)
        h = ops.convert(a, torch.float16)
        assert torch.equal(h, a.to(torch.float16))
        assert torch.equal(ops.convert(h, torch.float32), h.float())
        b = ops.convert(a, torch.bfloat16)
        assert torch.equal(b, a.to(torch.bfloat16))


def test_mask_to_kv_len(cuda_device):
    B, S = 7, 300
    m = np.full((B, S), -10000.0, np.float32)
    lens = [0, 1, 128, 129, 300, 17, 256]
    for b, n in enumerate(lens):
        m[b, :n] = 0
    m[5, 40] = 0          # a hole beyond the prefix: kv_len follows the last valid key
    out = ops.mask_to_kv_len(torch.from_numpy(m).to(cuda_device)).cpu().numpy()
    want = np.array(lens)
    want[5] = 41
    assert np.array_equal(out, want)


def _attention_case(cuda_device, dt, B, S, heads, lengths, seed=0, holes=False):
    H = heads * 64
    rng = np.random.default_rng(seed)
    qkv = rng.normal(0, 1, (B, S, 3 * H)).astype(np.float32)
    mask = np.zeros((B, S), np.float32)
    for b, n in enumerate(lengths):
        mask[b, n:] = -10000.0
    if holes:
        mask[:, 1::5] = -10000.0
    qd = torch.from_numpy(qkv).to(cuda_device).to(DT[dt])
    md = torch.from_numpy(mask).to(cuda_device)
    kv = ops.mask_to_kv_len(md)
    out = ops.attention(qd, heads, md, kv)
    r = _rounded(qkv, DT[dt]).reshape(B, S, 3, heads, 64)
    q, k, v = (r[:, :, i].transpose(0, 2, 1, 3) for i in range(3))
    want = bert_oracle.attention_core(q, k, v, mask, 0.125).transpose(0, 2, 1, 3).reshape(B, S, H)
    return _np(out), want, qd, md, kv


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("B,S,heads,lengths", [
    (2, 128, 12, [128, 128]), (3, 128, 2, [1, 17, 100]), (2, 96, 4, [96, 5]), (2, 200, 3, [200, 131]),
    (2, 256, 2, [16, 256]), (1, 384, 16, [300]), (1, 1, 1, [1]), (2, 512, 2, [512, 129]), (1, 130, 1, [130]),
    # the persistent long-sequence kernel's last length and the one-item kernel's first
    (3, 1024, 2, [1024, 700, 130]), (2, 1152, 1, [1152, 600]),
])
def test_attention(cuda_device, dt, B, S, heads, lengths):
    got, want, *_ = _attention_case(cuda_device, dt, B, S, heads, lengths, seed=S + B)
    tol = 6e-3 if dt == "f16" else 3e-2
    for b, n in enumerate(lengths):
        # every query row, padded ones included, is computed like the reference computes it
        assert max_abs(got[b], want[b]) < tol
    assert cosine(got, want) > 0.9995


@pytest.mark.parametrize("S", [384, 200, 640])
def test_attention_many_items_per_persistent_cta(cuda_device, S):
    """More items than resident CTAs, ragged lengths: every CTA of the persistent long-sequence kernel walks several
    items with different numbers of key tiles; at S = 384 and 640 every second item has one query tile only (the second
    UMMA-issuing warp and the second softmax warpgroup sit those out), at S = 200 the second tile is partly empty."""
    B, heads = 50, 4
    rng = np.random.default_rng(S)
    lengths = [int(x) for x in rng.integers(1, S + 1, B)]
    lengths[0], lengths[1] = S, 1
    got, want, *_ = _attention_case(cuda_device, "f16", B, S, heads, lengths, seed=S)
    for b in range(B):
        assert max_abs(got[b], want[b]) < 6e-3, (b, lengths[b])
    assert cosine(got, want) > 0.9995


def test_attention_mask_with_holes_and_no_mask(cuda_device):
    got, want, *_ = _attention_case(cuda_device, "f16", 2, 256, 2, [256, 200], seed=3, holes=True)
    assert max_abs(got, want) < 6e-3
    # no mask at all
    rng = np.random.default_rng(9)
    qkv = rng.normal(0, 1, (1, 128, 3 * 128)).astype(np.float32)
    qd = torch.from_numpy(qkv).cuda().half()
    out = ops.attention(qd, 2)
    r = _rounded(qkv, torch.float16).reshape(1, 128, 3, 2, 64)
    q, k, v = (r[:, :, i].transpose(0, 2, 1, 3) for i in range(3))
    want = bert_oracle.attention_core(q, k, v, None, 0.125).transpose(0, 2, 1, 3).reshape(1, 128, 128)
    assert max_abs(_np(out), want) < 6e-3


@pytest.mark.parametrize("S,lengths", [(256, [77, 200]), (128, [5, 100]), (96, [33, 96])])
def test_attention_padded_keys_have_exactly_zero_weight(cuda_device, S, lengths):
    """Perturbing K/V rows of padded keys must leave every output bit-identical."""
    B, heads = 2, 4
    H = heads * 64
    got, _, qd, md, kv = _attention_case(cuda_device, "f16", B, S, heads, lengths, seed=11)
    q2 = qd.clone()
    for b, n in enumerate(lengths):
        q2[b, n:, H:] = torch.randn_like(q2[b, n:, H:]) * 50.0      # K and V of padded keys
    out2 = ops.attention(q2, heads, md, kv)
    out1 = ops.attention(qd, heads, md, kv)
    for b, n in enumerate(lengths):
        assert torch.equal(out1[b, :n], out2[b, :n])


def test_attention_all_keys_masked_follows_reference(cuda_device):
    """A sequence with no valid key: the reference's softmax sees a constant shift and weighs all keys uniformly."""
    got, want, *_ = _attention_case(cuda_device, "f16", 2, 128, 2, [0, 64], seed=5)
    assert max_abs(got, want) < 6e-3


def test_bad_arguments_on_gpu(cuda_device):
    x = torch.zeros(16, 24, dtype=torch.float16, device=cuda_device)
    w = torch.zeros(8, 24, dtype=torch.float16, device=cuda_device)
    with pytest.raises(capi.B200Error) as e:
        ops.linear(x[:, :20], w[:, :20])       # K = 20 is not a multiple of 8
    assert e.value.code == capi.ERR_PARAM
    with pytest.raises(capi.B200Error):
        ops.linear(x, w, block_n=96)


@pytest.mark.parametrize("M,N,K", [(64, 768, 768), (8192, 768, 768), (300, 1024, 1024)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_linear_tanh_epilogue_against_oracle(M, N, K, dtype):
    """The pooler head: y = tanh(x . W + b); also over a strided view of the activation (every S-th row = [CLS])."""
    g = torch.Generator(device="cuda").manual_seed(M + N)
    S = 4
    full = torch.randn(M * S, K, device="cuda", generator=g).to(dtype)
    x = full.view(M, S * K)[:, :K]                 # row stride S*K: the first token of each sequence
    w_kn = (torch.randn(K, N, device="cuda", generator=g) * 0.05)
    b = torch.randn(N, device="cuda", generator=g) * 0.1
    w_nk = ops.pack_weight(w_kn, dtype)
    y = ops.linear(x, w_nk, b, epilogue=ops.EPI_BIAS_TANH)
    torch.cuda.synchronize()
    assert capi.device_status() == capi.OK
    want = bert_oracle.linear(x.float().cpu().numpy(), w_nk.float().t().cpu().numpy(), b.cpu().numpy(), act="tanh")
    tol = 2e-3 if dtype == torch.float16 else 1.2e-2       # half-precision output rounding of values in (-1, 1)
    assert np.abs(y.float().cpu().numpy() - want).max() < tol


@pytest.mark.parametrize("M,K,N", [(128, 768, 2), (8192, 768, 2), (300, 1024, 2), (77, 768, 1), (64, 768, 4), (0, 768, 2)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_qa_head_against_oracle(M, K, N, dtype):
    """The span-extraction head: fp32 logits = x . W + b, output n of every token as its own row (`unstack:n`)."""
    g = torch.Generator(device="cuda").manual_seed(M + K + N)
    x = torch.randn(max(M, 1), K, device="cuda", generator=g).to(dtype)[:M]
    w = (torch.randn(K, N, device="cuda", generator=g) * 0.05).contiguous()
    b = torch.randn(N, device="cuda", generator=g) * 0.1
    out = ops.qa_head(x, w, b)
    torch.cuda.synchronize()
    assert capi.device_status() == capi.OK and out.shape == (N, M) and out.dtype == torch.float32
    if M == 0:
        return
    want = bert_oracle.qa_head(_np(x.float()), _np(w), _np(b))
    for n in range(N):
        assert np.abs(_np(out[n]) - want[n]).max() < 2e-4      # fp32 accumulation, another summation order
    # no bias; a strided activation (row stride 2K)
    wide = torch.randn(M, 2 * K, device="cuda", generator=g).to(dtype)
    out2 = ops.qa_head(wide[:, :K], w)
    want2 = bert_oracle.qa_head(_np(wide[:, :K].float()), _np(w), np.zeros(N, np.float32))
    torch.cuda.synchronize()
    for n in range(N):
        assert np.abs(_np(out2[n]) - want2[n]).max() < 2e-4


def test_qa_head_rejects_bad_arguments():
    x = torch.zeros(8, 768, device="cuda", dtype=torch.float16)
    with pytest.raises(capi.B200Error):
        ops.qa_head(x, torch.zeros(768, 5, device="cuda"))          # more outputs than the kernel holds
    with pytest.raises(capi.B200Error):
        ops.qa_head(x[:, :762], torch.zeros(762, 2, device="cuda"))  # H not a multiple of 8


# ------------------------------------------------------------------------------------------------ launch ordering
def test_attention_reads_kv_len_behind_the_dependency_wait():
    """A kernel launched with programmatic stream serialization may start before its predecessor has finished; it must
    not read what the predecessor writes until its dependency wait.  b200_mask_from_input_mask writes mask and kv_len,
    the long-sequence attention kernel (S = 256) launched right behind it on the same stream reads both.  Fifty rounds
    with a new mask each, the same buffers every time (a stale kv_len from the previous round would change the
    result), compared bit for bit with the same two launches separated by a device synchronise."""
    dev = torch.device("cuda")
    B, S, heads = 8, 256, 4
    g = torch.Generator(device="cpu").manual_seed(5)
    qkv = torch.randn(B, S, 3 * heads * 64, generator=g).to(dev).half()
    mask_a, kv_a = torch.empty(B, S, device=dev), torch.empty(B, dtype=torch.int32, device=dev)
    mask_b, kv_b = torch.empty(B, S, device=dev), torch.empty(B, dtype=torch.int32, device=dev)
    out_a = torch.empty(B, S, heads * 64, dtype=torch.float16, device=dev)
    out_b = torch.empty_like(out_a)
    rng = np.random.default_rng(7)
    for r in range(50):
        lengths = rng.integers(1, S + 1, size=B)
        im = torch.from_numpy((np.arange(S)[None, :] < lengths[:, None]).astype(np.int32)).to(dev)
        torch.cuda.synchronize()
        # back to back
        ops.mask_from_input_mask(im, out_mask=mask_a, out_kv_len=kv_a)
        ops.attention(qkv, heads, mask_a, kv_a, out=out_a)
        torch.cuda.synchronize()
        # synchronised
        ops.mask_from_input_mask(im, out_mask=mask_b, out_kv_len=kv_b)
        torch.cuda.synchronize()
        ops.attention(qkv, heads, mask_b, kv_b, out=out_b)
        torch.cuda.synchronize()
        assert torch.equal(kv_a, kv_b)
        assert torch.equal(out_a, out_b), r
    assert capi.device_status() == capi.OK


def test_bounded_wait_expires_cleanly_and_the_device_carries_on():
    """The convention every device-side wait follows, shown on a kernel made for it: a warp waits on a barrier nobody
    arrives at, gives up after its poll limit, flags the status word and returns.  The host sees
    B200_ERR_DEVICE_TIMEOUT once, the word is clear again, and the next GEMM runs and is correct."""
    lib = capi.lib()
    assert capi.device_status() == capi.OK
    assert lib.b200_selftest_bounded_wait(capi.stream_ptr()) == capi.OK
    torch.cuda.synchronize()
    assert capi.device_status() == capi.ERR_DEVICE_TIMEOUT
    assert capi.device_status() == capi.OK
    # the asynchronous read of the same word
    word = torch.zeros(1, dtype=torch.int32).pin_memory()
    assert lib.b200_selftest_bounded_wait(capi.stream_ptr()) == capi.OK
    assert lib.b200_device_status_async(word.data_ptr(), capi.stream_ptr()) == capi.OK
    torch.cuda.synchronize()
    assert lib.b200_decode_status_word(int(word[0])) == capi.ERR_DEVICE_TIMEOUT
    assert capi.device_status() == capi.ERR_DEVICE_TIMEOUT   # the asynchronous read does not clear
    assert capi.device_status() == capi.OK
    x = torch.randn(512, 256, device="cuda").half()
    w = (torch.randn(128, 256, device="cuda") * 0.05).half()
    y = ops.linear(x, w)
    torch.cuda.synchronize()
    assert capi.device_status() == capi.OK
    assert (y.float() - x.float() @ w.float().t()).abs().max().item() < 2e-2

