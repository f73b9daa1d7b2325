"""GPU: the allocation-free masked-attention entry point against the regular one.

Some hosts of this library may not allocate device memory when they call it — an operator whose Forward must not
allocate and that was given no workspace, a process living inside a memory budget fixed at start-up, a plug-in in
someone else's server.  For them `b200_attention_masked_fwd_static` keeps its only temporary (the per-sequence
kv_len array derived from the mask) in a fixed array inside the library image instead of in caller memory.  This
test calls it through the C ABI twice in a row, with different batches and masks so that stale scratch contents from
the first call would show up in the second, and compares each result with `b200_mask_to_kv_len` +
`b200_attention_fwd`, which use a caller-provided kv_len buffer, and with the CPU oracle.  The second call is
bracketed by reads of the device's free memory (cudaMemGetInfo) and of torch's allocator counters: neither may move,
which is the property the entry point is named for.  (The first call on a device is its documented warm-up: it looks
the scratch array's address up, sets kernel attributes and may make the driver load the kernels' module.)  It also
checks the size limit.

Collected last (file name) so that a run that stops at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import bert_oracle
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


def _oracle(qkv, mask, heads):
    B, S, _ = qkv.shape
    x = qkv.float().cpu().numpy().reshape(B, S, 3, heads, 64)
    q, k, v = (np.ascontiguousarray(x[:, :, i].transpose(0, 2, 1, 3)) for i in range(3))
    o = bert_oracle.attention_core(q, k, v, mask.cpu().numpy(), 0.125)        # [B, heads, S, 64]
    return o.transpose(0, 2, 1, 3).reshape(B, S, heads * 64)


def test_static_scratch_entry_point_matches_regular_one_twice_in_a_row(cuda_device):
    lib = capi.lib()
    stream = capi.stream_ptr()
    # second call: smaller batch, different lengths, longer sequences (the multi-tile kernel)
    cases = [(6, 128, 4, [128, 1, 77, 128, 30, 101], 1), (3, 200, 2, [200, 17, 140], 2)]
    # warm-up of both kernels of the entry point on this device (S <= 128 and S > 128), outside the bracket below
    for B, S, heads, lengths, seed in cases:
        qkv, mask = _case(cuda_device, B, S, heads, lengths, seed + 10)
        d = _desc(qkv, heads, mask, torch.empty(B, S, heads * 64, dtype=torch.float16, device=cuda_device))
        assert lib.b200_attention_masked_fwd_static(ctypes.byref(d), stream) == capi.OK
    torch.cuda.synchronize()
    for i, (B, S, heads, lengths, seed) in enumerate(cases):
        qkv, mask = _case(cuda_device, B, S, heads, lengths, seed)
        want = ops.attention(qkv, heads, mask, ops.mask_to_kv_len(mask))      # caller-owned kv_len buffer
        got = torch.empty_like(want)
        d = _desc(qkv, heads, mask, got)
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info(cuda_device)                       # cudaMemGetInfo
        reserved0, allocated0 = torch.cuda.memory_reserved(cuda_device), torch.cuda.memory_allocated(cuda_device)
        rc = lib.b200_attention_masked_fwd_static(ctypes.byref(d), stream)
        assert rc == capi.OK, lib.b200_status_string(rc)
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info(cuda_device)
        assert free1 == free0, (free0, free1)                                  # no device memory taken or returned
        assert torch.cuda.memory_reserved(cuda_device) == reserved0
        assert torch.cuda.memory_allocated(cuda_device) == allocated0
        assert capi.device_status() == capi.OK
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= TOL, diff
        assert torch.equal(got, want)     # same kernels, same inputs: identical bits
        # and against the CPU oracle, on the valid query rows
        ref = _oracle(qkv, mask, heads)
        g = got.float().cpu().numpy()
        for b, n in enumerate(lengths):
            assert np.abs(g[b, :n] - ref[b, :n]).max() <= TOL


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
