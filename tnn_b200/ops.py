"""Host-side operator wrappers over the C ABI: one function per fused layer of the path.

Names and argument meaning follow the fused TNN layers (FusedLinear, FusedAttention, LayerNorm) that the graph pass
emits; tensors are torch CUDA tensors used as device buffers.  Every function launches through `extern "C"` entry
points of libtnn_b200.so on the current torch stream; nothing here computes with torch.
"""
import ctypes

import torch

from . import capi
from .capi import EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL, EPI_BIAS_TANH  # noqa: F401


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("tnn_b200 operators take CUDA tensors only (there is no CPU path)")


def pack_weight(w_kn, dtype=torch.float16, out=None):
    """fp32 `[K, N]` (TNN MatMul weight layout, y = x.W) -> `dtype` `[N, K]` on the device."""
    _require_cuda(w_kn)
    assert w_kn.dtype == torch.float32 and w_kn.dim() == 2 and w_kn.stride(1) == 1
    K, N = w_kn.shape
    if out is None:
        out = torch.empty((N, K), dtype=dtype, device=w_kn.device)
    assert out.shape[0] == N and out.shape[1] == K and out.stride(1) == 1
    rc = capi.lib().b200_pack_weight(w_kn.data_ptr(), K, N, w_kn.stride(0), out.data_ptr(), out.stride(0),
                                     capi.dtype_code(out.dtype), capi.stream_ptr())
    capi.check(rc, "b200_pack_weight")
    return out


def fold_layernorm_weight(w_kn, gamma, beta, bias=None, dtype=torch.float16, out=None):
    """For y = LayerNorm(x; gamma, beta).W + bias: returns (w_nk with gamma folded in, c1, c2), see include/tnn_b200.h."""
    _require_cuda(w_kn, gamma, beta, bias)
    K, N = w_kn.shape
    if out is None:
        out = torch.empty((N, K), dtype=dtype, device=w_kn.device)
    c1 = torch.empty((N,), dtype=torch.float32, device=w_kn.device)
    c2 = torch.empty((N,), dtype=torch.float32, device=w_kn.device)
    rc = capi.lib().b200_fold_layernorm_weight(w_kn.data_ptr(), K, N, w_kn.stride(0), gamma.data_ptr(),
                                               beta.data_ptr(), capi.ptr(bias), out.data_ptr(), out.stride(0),
                                               capi.dtype_code(out.dtype), c1.data_ptr(), c2.data_ptr(),
                                               capi.stream_ptr())
    capi.check(rc, "b200_fold_layernorm_weight")
    return out, c1, c2


def stats_buffer(rows, width, device):
    """Row-statistics buffer of a `[rows, width]` activation: `[ceil(width/32), rows, 2]` fp32."""
    return torch.empty(((width + 31) // 32, rows, 2), dtype=torch.float32, device=device)


def convert(src, dtype, out=None):
    _require_cuda(src)
    assert src.is_contiguous()
    if out is None:
        out = torch.empty(src.shape, dtype=dtype, device=src.device)
    assert out.is_contiguous() and out.numel() == src.numel()
    rc = capi.lib().b200_convert(src.data_ptr(), capi.dtype_code(src.dtype), out.data_ptr(),
                                 capi.dtype_code(out.dtype), src.numel(), capi.stream_ptr())
    capi.check(rc, "b200_convert")
    return out


def _linear_desc(x, w_nk, bias, residual, epilogue, out_dtype, out, block_n, out_stats=None, ln_in=None, res_ln=None,
                 ln_eps=1e-12):
    _require_cuda(x, w_nk, bias, residual, out)
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    M = x2.shape[0]
    N = w_nk.shape[0]
    assert w_nk.shape[1] == K and x2.stride(1) == 1 and w_nk.stride(1) == 1
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty(x.shape[:-1] + (N,), dtype=out_dtype, device=x.device)
    y2 = out.reshape(-1, N)
    d = capi.LinearDesc()
    d.x, d.w_nk, d.bias, d.y = x2.data_ptr(), w_nk.data_ptr(), capi.ptr(bias), y2.data_ptr()
    d.M, d.N, d.K = M, N, K
    d.ldx, d.ldw, d.ldy = x2.stride(0), w_nk.stride(0), y2.stride(0)
    if residual is not None:
        r2 = residual.reshape(-1, N)
        assert r2.dtype == x.dtype and r2.stride(1) == 1
        d.residual, d.ldr = r2.data_ptr(), r2.stride(0)
    d.dtype, d.out_dtype = capi.dtype_code(x.dtype), capi.dtype_code(out.dtype)
    d.epilogue, d.block_n = epilogue, block_n
    # LayerNorm folding: ln_in = (stats of x, c1, c2); res_ln = (stats of residual, gamma, beta)
    d.ln_eps = float(ln_eps)
    if out_stats is not None:
        d.out_stats = out_stats.data_ptr()
    if ln_in is not None:
        d.ln_in_stats, d.ln_c1, d.ln_c2 = (t.data_ptr() for t in ln_in)
    if res_ln is not None:
        d.res_ln_stats, d.res_ln_gamma, d.res_ln_beta = (t.data_ptr() for t in res_ln)
    return d, out


def linear(x, w_nk, bias=None, residual=None, epilogue=EPI_BIAS, out_dtype=None, out=None, block_n=0,
           out_stats=None, ln_in=None, res_ln=None, ln_eps=1e-12):
    """y[M,N] = epilogue(x[M,K] . w_nk[N,K]^T + bias (+ residual)); x may be `[..., K]`."""
    d, out = _linear_desc(x, w_nk, bias, residual, epilogue, out_dtype, out, block_n, out_stats, ln_in, res_ln, ln_eps)
    rc = capi.lib().b200_linear_fwd(ctypes.byref(d), capi.stream_ptr())
    capi.check(rc, "b200_linear_fwd")
    return out


def mask_to_kv_len(mask_add, exclude_below=-5000.0, out=None):
    """mask_add fp32 `[B, S]` (or `[B,1,1,S]`) -> int32 `[B]`."""
    _require_cuda(mask_add)
    S = mask_add.shape[-1]
    m2 = mask_add.reshape(-1, S)
    assert m2.is_contiguous() and m2.dtype == torch.float32
    if out is None:
        out = torch.empty((m2.shape[0],), dtype=torch.int32, device=mask_add.device)
    rc = capi.lib().b200_mask_to_kv_len(m2.data_ptr(), m2.shape[0], S, exclude_below, out.data_ptr(),
                                        capi.stream_ptr())
    capi.check(rc, "b200_mask_to_kv_len")
    return out


def attention(qkv, heads, mask_add=None, kv_len=None, scale=None, exclude_below=-5000.0, out=None):
    """qkv `[B, S, 3*heads*64]` packed (Q | K | V along the last axis) -> context `[B, S, heads*64]`."""
    _require_cuda(qkv, mask_add, kv_len, out)
    B, S, W = qkv.shape
    H = heads * 64
    assert W == 3 * H and qkv.stride(2) == 1 and qkv.stride(0) == S * qkv.stride(1)
    if out is None:
        out = torch.empty((B, S, H), dtype=qkv.dtype, device=qkv.device)
    es = qkv.element_size()
    d = capi.AttentionDesc()
    d.q, d.k, d.v = qkv.data_ptr(), qkv.data_ptr() + H * es, qkv.data_ptr() + 2 * H * es
    d.ldq = d.ldk = d.ldv = qkv.stride(1)
    d.out, d.ldo = out.data_ptr(), out.stride(1)
    if mask_add is not None:
        m2 = mask_add.reshape(B, S)
        assert m2.is_contiguous() and m2.dtype == torch.float32
        d.mask_add = m2.data_ptr()
    if kv_len is not None:
        assert kv_len.dtype == torch.int32 and kv_len.numel() == B
        d.kv_len = kv_len.data_ptr()
    d.B, d.S, d.heads, d.head_dim = B, S, heads, 64
    d.dtype = capi.dtype_code(qkv.dtype)
    d.scale = float(scale if scale is not None else 0.125)
    d.mask_exclude_below = float(exclude_below)
    rc = capi.lib().b200_attention_fwd(ctypes.byref(d), capi.stream_ptr())
    capi.check(rc, "b200_attention_fwd")
    return out


def _layernorm_desc(x, gamma, beta, eps, residual, out_dtype, out):
    _require_cuda(x, gamma, beta, residual, out)
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    assert x2.stride(1) == 1 and gamma.dtype == torch.float32 and beta.dtype == torch.float32
    if out is None:
        out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    y2 = out.reshape(-1, H)
    d = capi.LayerNormDesc()
    d.x, d.gamma, d.beta, d.y = x2.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y2.data_ptr()
    d.rows, d.H, d.ldx, d.ldy = x2.shape[0], H, x2.stride(0), y2.stride(0)
    if residual is not None:
        r2 = residual.reshape(-1, H)
        assert r2.dtype == x.dtype
        d.residual, d.ldr = r2.data_ptr(), r2.stride(0)
    d.in_dtype, d.out_dtype, d.eps = capi.dtype_code(x.dtype), capi.dtype_code(out.dtype), float(eps)
    return d, out


def add_layernorm(x, gamma, beta, eps, residual=None, out_dtype=None, out=None):
    d, out = _layernorm_desc(x, gamma, beta, eps, residual, out_dtype, out)
    rc = capi.lib().b200_add_layernorm_fwd(ctypes.byref(d), capi.stream_ptr())
    capi.check(rc, "b200_add_layernorm_fwd")
    return out


def embedding_layernorm(input_ids, segment_ids, word_emb, type_emb, pos_emb, gamma, beta, eps, out_dtype=torch.float16,
                        out=None):
    """`[B,S]` int32 ids (+ segment ids or None) -> LayerNorm(word + segment + position embeddings) `[B,S,H]`."""
    _require_cuda(input_ids, segment_ids, word_emb, type_emb, pos_emb, gamma, beta, out)
    B, S = input_ids.shape
    H = word_emb.shape[1]
    assert input_ids.dtype == torch.int32 and input_ids.is_contiguous()
    assert word_emb.stride(1) == 1 and pos_emb.dtype == word_emb.dtype and pos_emb.shape[0] >= S
    assert pos_emb.stride(0) == word_emb.stride(0)
    if out is None:
        out = torch.empty((B, S, H), dtype=out_dtype, device=input_ids.device)
    d = capi.EmbeddingDesc()
    d.input_ids, d.word_emb, d.pos_emb = input_ids.data_ptr(), word_emb.data_ptr(), pos_emb.data_ptr()
    if segment_ids is not None:
        assert segment_ids.dtype == torch.int32 and segment_ids.is_contiguous() and type_emb is not None
        assert type_emb.dtype == word_emb.dtype and type_emb.stride(0) == word_emb.stride(0)
        d.segment_ids, d.type_emb, d.type_vocab = segment_ids.data_ptr(), type_emb.data_ptr(), type_emb.shape[0]
    d.gamma, d.beta, d.out = gamma.data_ptr(), beta.data_ptr(), out.data_ptr()
    d.B, d.S, d.H, d.vocab = B, S, H, word_emb.shape[0]
    d.ld_table, d.ld_out = word_emb.stride(0), out.reshape(-1, H).stride(0)
    d.table_dtype, d.out_dtype, d.eps = capi.dtype_code(word_emb.dtype), capi.dtype_code(out.dtype), float(eps)
    rc = capi.lib().b200_embedding_layernorm_fwd(ctypes.byref(d), capi.stream_ptr())
    capi.check(rc, "b200_embedding_layernorm_fwd")
    return out


def mask_from_input_mask(input_mask, masked_value=-10000.0, exclude_below=-5000.0, out_mask=None, out_kv_len=None):
    """int32 0/1 `[B,S]` -> (additive fp32 mask `[B,S]`, int32 kv_len `[B]`), into the given buffers if any."""
    _require_cuda(input_mask, out_mask, out_kv_len)
    B, S = input_mask.shape
    assert input_mask.dtype == torch.int32 and input_mask.is_contiguous()
    mask_add = out_mask if out_mask is not None else torch.empty((B, S), dtype=torch.float32, device=input_mask.device)
    kv_len = out_kv_len if out_kv_len is not None else torch.empty((B,), dtype=torch.int32, device=input_mask.device)
    assert mask_add.dtype == torch.float32 and mask_add.is_contiguous() and mask_add.numel() == B * S
    assert kv_len.dtype == torch.int32 and kv_len.numel() == B
    rc = capi.lib().b200_mask_from_input_mask(input_mask.data_ptr(), B, S, masked_value, exclude_below,
                                              mask_add.data_ptr(), kv_len.data_ptr(), capi.stream_ptr())
    capi.check(rc, "b200_mask_from_input_mask")
    return mask_add, kv_len


def qa_head(x, weight, bias=None, out=None):
    """Span-extraction head: `x` `[..., H]` half precision, `weight` fp32 `[H, N]` (N <= 4), `bias` fp32 `[N]` or None
    -> fp32 `[N, M]` (M = tokens): row n is output n of every token (the graph's `unstack:n`)."""
    _require_cuda(x, weight, bias, out)
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    M, N = x2.shape[0], weight.shape[1]
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape[0] == H and x2.stride(1) == 1
    if out is None:
        out = torch.empty((N, M), dtype=torch.float32, device=x.device)
    d = capi.QAHeadDesc()
    d.x, d.weight, d.out = x2.data_ptr(), weight.data_ptr(), out.data_ptr()
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
        d.bias = bias.data_ptr()
    d.M, d.H, d.N = M, H, N
    d.ldx, d.ld_out, d.x_dtype = x2.stride(0), out.stride(0), capi.dtype_code(x.dtype)
    rc = capi.lib().b200_qa_head_fwd(ctypes.byref(d), capi.stream_ptr())
    capi.check(rc, "b200_qa_head_fwd")
    return out
