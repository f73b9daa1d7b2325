"""GPU: the allocation-free masked-attention entry point against the regular one.

Some hosts of this library may not allocate device memory when they call it — an operator whose Forward must not
allocate and that was given no workspace, a process living inside a memory budget fixed at start-up, a plug-in in
someone else's server.  For them `b200_attention_masked_fwd_static` keeps its only temporary (the per-sequence
kv_len array derived from the mask) in a fixed array inside the library image instead of in caller memory.  This
test calls it through the C ABI twice in a row, with different batches and masks so that stale scratch contents from
the first call would show up in the second, and compares each result with `b200_mask_to_kv_len` +
`b200_attention_fwd`, which use a caller-provided kv_len buffer.  It also checks the size limit.

Collected last (file name) so that a run that stops at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

from tnn_b200 import capi, ops

pytestmark = pytest.mark.gpu

TOL = 6e-3   # the fp16 tolerance the attention parity tests use; the two paths run the same kernels


def _desc(qkv, heads, mask2d, out):
    B, S, W = qkv.shape
    H = heads * 64
    es = qkv.element_size()
    d = capi.AttentionDesc()
    d.q, d.k, d.v = qkv.data_ptr(), qkv.data_ptr() + H * es, qkv.data_ptr() + 2 * H * es
    d.ldq = d.ldk = d.ldv = qkv.stride(1)
    d.out, d.ldo = out.data_ptr(), out.stride(1)
    d.mask_add = mask2d.data_ptr()
    d.B, d.S, d.heads, d.head_dim = B, S, heads, 64
    d.dtype = capi.dtype_code(qkv.dtype)
    d.scale = 0.125
    d.mask_exclude_below = -5000.0
    return d


def _case(device, B, S, heads, lengths, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    qkv = torch.randn(B, S, 3 * heads * 64, generator=g).to(device).half()
    mask = torch.zeros(B, S)
    for b, n in enumerate(lengths):
        mask[b, n:] = -10000.0
    return qkv, mask.to(device)


def test_static_scratch_entry_point_matches_regular_one_twice_in_a_row(cuda_device):
    lib = capi.lib()
    stream = capi.stream_ptr()
    # second call: smaller batch, different lengths, longer sequences (the multi-tile kernel)
    cases = [(6, 128, 4, [128, 1, 77, 128, 30, 101], 1), (3, 200, 2, [200, 17, 140], 2)]
    for B, S, heads, lengths, seed in cases:
        qkv, mask = _case(cuda_device, B, S, heads, lengths, seed)
        want = ops.attention(qkv, heads, mask, ops.mask_to_kv_len(mask))      # caller-owned kv_len buffer
        got = torch.empty_like(want)
        d = _desc(qkv, heads, mask, got)
        rc = lib.b200_attention_masked_fwd_static(ctypes.byref(d), stream)
        assert rc == capi.OK, lib.b200_status_string(rc)
        torch.cuda.synchronize()
        assert capi.device_status() == capi.OK
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= TOL, diff
        assert torch.equal(got, want)     # same kernels, same inputs: identical bits


def test_static_scratch_limit_and_required_mask(cuda_device):
    lib = capi.lib()
    qkv, mask = _case(cuda_device, 2, 128, 1, [128, 64], 3)
    out = torch.empty(2, 128, 64, dtype=torch.float16, device=cuda_device)
    d = _desc(qkv, 1, mask, out)
    d.B = capi.STATIC_MAX_BATCH + 1                    # rejected before anything is launched or read
    assert lib.b200_attention_masked_fwd_static(ctypes.byref(d), capi.stream_ptr()) == capi.ERR_STATIC_LIMIT
    assert b"static" in lib.b200_status_string(capi.ERR_STATIC_LIMIT)
    d.B = 2
    d.mask_add = None                                   # this entry point exists for the masked case only
    assert lib.b200_attention_masked_fwd_static(ctypes.byref(d), capi.stream_ptr()) == capi.ERR_PARAM
