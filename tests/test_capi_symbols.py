"""CPU: the C-ABI library loads and exports every symbol include/tnn_b200.h declares; argument checks that need no
GPU return the documented error codes."""
import ctypes
import os
import re

from tnn_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tnn_b200.h")).read()
    return sorted(set(re.findall(r"B200_API[^;(]*?\b(b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 10
    lib = ctypes.CDLL(capi.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(capi.SYMBOLS), (set(names) ^ set(capi.SYMBOLS))


def test_status_strings_and_version():
    l = capi.lib()
    assert l.b200_status_string(0) == b"ok"
    for code in range(-6, 0):
        assert len(l.b200_status_string(code)) > 0
    assert b"sm_100a" in l.b200_version()


def test_null_and_bad_descriptors_are_rejected_without_a_gpu():
    l = capi.lib()
    assert l.b200_linear_fwd(None, None) == capi.ERR_PARAM
    assert l.b200_attention_fwd(None, None) == capi.ERR_PARAM
    assert l.b200_add_layernorm_fwd(None, None) == capi.ERR_PARAM
    assert l.b200_encoder_fwd(None, None) == capi.ERR_PARAM
    d = capi.LinearDesc()
    d.x = d.w_nk = d.y = 256
    d.M, d.N, d.K = 128, 64, 12          # K not a multiple of 8
    d.ldx = d.ldw = 16
    d.ldy = 64
    assert l.b200_linear_fwd(ctypes.byref(d), None) == capi.ERR_PARAM
    a = capi.AttentionDesc()
    a.q = a.k = a.v = a.out = 256
    a.B, a.S, a.heads, a.head_dim = 1, 128, 12, 32   # only head_dim 64 exists
    a.ldq = a.ldk = a.ldv = a.ldo = 768
    assert l.b200_attention_fwd(ctypes.byref(a), None) == capi.ERR_UNSUPPORTED
    assert l.b200_encoder_workspace_bytes(0, 768, 3072, 0) == 0
    n = l.b200_encoder_workspace_bytes(128, 768, 3072, 0)
    assert n >= 128 * (3 * 768 + 3 * 768 + 3072) * 2 and n % 256 == 0


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    from tnn_b200 import ops
    with pytest.raises(ValueError):
        ops.linear(torch.zeros(8, 8, dtype=torch.float16), torch.zeros(8, 8, dtype=torch.float16))
