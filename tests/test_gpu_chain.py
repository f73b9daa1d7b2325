"""b200_chain_fwd: several dependent GEMMs / LayerNorms of an encoder layer in one launch.  The chain performs the same
arithmetic in the same order as the separate launches with 256 x 192 tiles, so results must be bit-identical to them;
the separate launches are themselves checked against the oracle in test_gpu_kernels.py."""
import pytest
import torch

from tnn_b200 import capi, ops

pytestmark = pytest.mark.gpu


def _w(n, k, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(n, k, device="cuda", generator=g) * 0.03).to(dtype)


def _v(n, seed, scale=0.1, shift=0.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(n, device="cuda", generator=g) * scale + shift


@pytest.mark.parametrize("M", [8192, 1000, 130, 256])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_ffn_chain_equals_separate_launches(M, dtype):
    H, F = 768, 3072
    g = torch.Generator(device="cuda").manual_seed(M)
    a = torch.randn(M, H, device="cuda", generator=g).to(dtype)
    w1, b1 = _w(F, H, dtype, 1), _v(F, 2)
    w2, b2 = _w(H, F, dtype, 3), _v(H, 4)
    f_ref = ops.linear(a, w1, b1, epilogue=ops.EPI_BIAS_GELU, block_n=192)
    t_ref = ops.linear(f_ref, w2, b2, residual=a, epilogue=ops.EPI_BIAS_RESIDUAL, block_n=192)
    c = ops.Chain()
    f = c.linear(a, w1, b1, epilogue=ops.EPI_BIAS_GELU)
    t = c.linear(f, w2, b2, residual=a, epilogue=ops.EPI_BIAS_RESIDUAL)
    c.run()
    torch.cuda.synchronize()
    assert capi.device_status() == capi.OK
    assert torch.equal(f, f_ref)
    assert torch.equal(t, t_ref)


@pytest.mark.parametrize("M,H,F", [(8192, 768, 3072), (900, 768, 3072), (384, 1024, 4096), (200, 256, 512)])
def test_layer_tail_chain_equals_separate_launches(M, H, F):
    """out-proj + residual -> LayerNorm -> FFN1 + GELU -> FFN2 + residual -> LayerNorm -> next layer's QKV."""
    dtype = torch.float16
    g = torch.Generator(device="cuda").manual_seed(M + H)
    ctx = torch.randn(M, H, device="cuda", generator=g).to(dtype)
    h = torch.randn(M, H, device="cuda", generator=g).to(dtype)
    wo, bo = _w(H, H, dtype, 1), _v(H, 2)
    w1, b1 = _w(F, H, dtype, 3), _v(F, 4)
    w2, b2 = _w(H, F, dtype, 5), _v(H, 6)
    wq, bq = _w(3 * H, H, dtype, 7), _v(3 * H, 8)
    g1, be1 = _v(H, 9, 0.2, 1.0), _v(H, 10)
    g2, be2 = _v(H, 11, 0.2, 1.0), _v(H, 12)
    eps = 1e-12
    t_ref = ops.linear(ctx, wo, bo, residual=h, epilogue=ops.EPI_BIAS_RESIDUAL, block_n=192)
    a_ref = ops.add_layernorm(t_ref, g1, be1, eps)
    f_ref = ops.linear(a_ref, w1, b1, epilogue=ops.EPI_BIAS_GELU, block_n=192)
    t2_ref = ops.linear(f_ref, w2, b2, residual=a_ref, epilogue=ops.EPI_BIAS_RESIDUAL, block_n=192)
    h2_ref = ops.add_layernorm(t2_ref, g2, be2, eps)
    q_ref = ops.linear(h2_ref, wq, bq, block_n=192)

    c = ops.Chain()
    t = c.linear(ctx, wo, bo, residual=h, epilogue=ops.EPI_BIAS_RESIDUAL)
    a = c.add_layernorm(t, g1, be1, eps)
    f = c.linear(a, w1, b1, epilogue=ops.EPI_BIAS_GELU)
    t2 = c.linear(f, w2, b2, residual=a, epilogue=ops.EPI_BIAS_RESIDUAL)
    h2 = c.add_layernorm(t2, g2, be2, eps)
    q = c.linear(h2, wq, bq)
    sync = torch.empty(4096, dtype=torch.int32, device="cuda")
    for _ in range(2):                      # the second run reuses the (re-zeroed) counters and every buffer
        c.run(sync)
    torch.cuda.synchronize()
    assert capi.device_status() == capi.OK
    for got, ref in [(t, t_ref), (a, a_ref), (f, f_ref), (t2, t2_ref), (h2, h2_ref), (q, q_ref)]:
        assert torch.equal(got, ref)


def test_chain_rejects_bad_arguments():
    dtype = torch.float16
    a = torch.zeros(256, 768, device="cuda", dtype=dtype)
    w = torch.zeros(768, 768, device="cuda", dtype=dtype)
    c = ops.Chain()
    c.linear(a, w)
    arr = (capi.ChainPhase * 1)(*c.phases)
    lib = capi.lib()
    assert lib.b200_chain_fwd(arr, 1, None, capi.stream_ptr()) == capi.ERR_PARAM
    assert lib.b200_chain_fwd(arr, 0, a.data_ptr(), capi.stream_ptr()) == capi.ERR_PARAM
    assert lib.b200_chain_fwd(arr, 9, a.data_ptr(), capi.stream_ptr()) == capi.ERR_PARAM
    # phases with different row counts
    c2 = ops.Chain()
    c2.linear(a, w)
    c2.rows = None
    c2.linear(torch.zeros(128, 768, device="cuda", dtype=dtype), w)
    arr2 = (capi.ChainPhase * 2)(*c2.phases)
    sync = torch.zeros(64, dtype=torch.int32, device="cuda")
    assert lib.b200_chain_fwd(arr2, 2, sync.data_ptr(), capi.stream_ptr()) == capi.ERR_PARAM
    assert lib.b200_chain_sync_bytes(8192, 6) == 32 * 6 * 4
