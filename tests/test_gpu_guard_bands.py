"""GPU: no kernel of the path writes outside the output it was given, and none modifies its inputs.

Every output is a window into a larger buffer that was filled with a bit pattern: guard bands in front and behind, and
(where the entry point takes a leading dimension) the columns between a row's end and the next row's start.  After the
call every element outside the window must still hold the pattern, bit for bit, and the inputs must be unchanged.
Shapes are the ragged ones: rows and columns that end inside a tile, sequence lengths inside a key tile, element counts
that are not a multiple of the vector width.
"""
import numpy as np
import pytest
import torch

from tnn_b200 import capi, ops

pytestmark = pytest.mark.gpu

GUARD = 4096            # elements in front and behind; a multiple of 16 bytes for every dtype used
PATTERN16 = 0x7B7B


class Guarded:
    """A `[rows, cols]` window with leading dimension `ld` inside a pattern-filled buffer."""

    def __init__(self, rows, cols, dtype, device, ld=None):
        ld = ld or cols
        self.rows, self.cols, self.ld = rows, cols, ld
        n = GUARD + rows * ld + GUARD
        self.backing = torch.empty(n, dtype=dtype, device=device)
        self.bits().fill_(PATTERN16)
        self.window = self.backing[GUARD:GUARD + rows * ld].view(rows, ld)[:, :cols]
        inside = torch.zeros(n, dtype=torch.bool, device=device)
        inside[GUARD:GUARD + rows * ld].view(rows, ld)[:, :cols] = True
        self.outside = ~inside

    def bits(self):
        return self.backing.view(torch.int16)

    def assert_intact(self):
        per = self.backing.element_size() // 2
        b = self.bits().view(-1, per)
        touched = (b != PATTERN16).any(dim=1) & self.outside
        assert not bool(touched.any()), "elements outside the output were written at %s" % \
            touched.nonzero().flatten()[:8].tolist()
        written = (b != PATTERN16).any(dim=1) & ~self.outside
        # the window itself must have been produced (the pattern is not a value these kernels emit for these inputs)
        assert int(written.sum()) >= int((~self.outside).sum()) * 0.99


@pytest.fixture(autouse=True)
def _status_clean(cuda_device):
    yield
    torch.cuda.synchronize()
    assert capi.device_status() == capi.OK


def _unchanged(pairs):
    for t, copy in pairs:
        assert torch.equal(t, copy)


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("epi", ["bias", "gelu", "residual"])
@pytest.mark.parametrize("M,N,K,bn,pad", [
    (257, 392, 200, 192, 8), (300, 2304, 768, 0, 16), (129, 136, 72, 128, 8), (900, 776, 264, -256, 24),
    (1, 8, 8, 0, 8), (513, 264, 136, 256, 8), (384, 200, 136, -128, 8), (255, 72, 64, 64, 40), (128, 768, 768, 0, 0),
])
def test_linear_stays_inside_its_output(cuda_device, M, N, K, bn, pad, epi, out_dtype):
    g = torch.Generator(device="cpu").manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(cuda_device).half()
    w = (torch.randn(N, K, generator=g) * 0.05).to(cuda_device).half()
    b = torch.randn(N, generator=g).to(cuda_device)
    r = torch.randn(M, N, generator=g).to(cuda_device).half() if epi == "residual" else None
    keep = [(t, t.clone()) for t in (x, w, b) + ((r,) if r is not None else ())]
    out = Guarded(M, N, out_dtype, cuda_device, ld=N + pad)
    code = {"bias": ops.EPI_BIAS, "gelu": ops.EPI_BIAS_GELU, "residual": ops.EPI_BIAS_RESIDUAL}[epi]
    ops.linear(x, w, b, residual=r, epilogue=code, out=out.window, block_n=bn)
    torch.cuda.synchronize()
    out.assert_intact()
    _unchanged(keep)
    want = ops.linear(x, w, b, residual=r, epilogue=code, out_dtype=out_dtype, block_n=bn)
    assert torch.equal(out.window, want)        # the strided call computes what the contiguous call computes


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,S,heads,pad", [(3, 96, 2, 8), (2, 128, 12, 0), (3, 130, 2, 64), (2, 200, 3, 8),
                                           (2, 384, 2, 16), (1, 1, 1, 8), (5, 33, 1, 8)])
def test_attention_stays_inside_its_output(cuda_device, B, S, heads, pad, dt):
    H = heads * 64
    g = torch.Generator(device="cpu").manual_seed(B * 1000 + S)
    qkv = torch.randn(B, S, 3 * H, generator=g).to(cuda_device).to(dt)
    lengths = torch.randint(1, S + 1, (B,), generator=g)
    lengths[0] = S
    mask = torch.zeros(B, S)
    for i, n in enumerate(lengths.tolist()):
        mask[i, n:] = -10000.0
    mask = mask.to(cuda_device)
    kv = ops.mask_to_kv_len(mask)
    keep = [(t, t.clone()) for t in (qkv, mask, kv)]
    out = Guarded(B * S, H, dt, cuda_device, ld=H + pad)
    view = out.window.unflatten(0, (B, S))
    assert view.data_ptr() == out.window.data_ptr()
    ops.attention(qkv, heads, mask, kv, out=view)
    torch.cuda.synchronize()
    out.assert_intact()
    _unchanged(keep)
    want = ops.attention(qkv, heads, mask, kv)
    assert torch.equal(view, want)


@pytest.mark.parametrize("rows,H,pad,resid", [(37, 768, 8, False), (37, 768, 8, True), (5000, 768, 0, False),
                                              (19, 1024, 16, True), (7, 2048, 8, False), (3, 4096, 8, True),
                                              (1, 8, 8, False), (300, 256, 24, False)])
def test_layernorm_stays_inside_its_output(cuda_device, rows, H, pad, resid):
    g = torch.Generator(device="cpu").manual_seed(rows + H)
    x = torch.randn(rows, H, generator=g).to(cuda_device).half()
    r = torch.randn(rows, H, generator=g).to(cuda_device).half() if resid else None
    gamma = torch.randn(H, generator=g).to(cuda_device)
    beta = torch.randn(H, generator=g).to(cuda_device)
    keep = [(t, t.clone()) for t in (x, gamma, beta) + ((r,) if resid else ())]
    out = Guarded(rows, H, torch.float16, cuda_device, ld=H + pad)
    ops.add_layernorm(x, gamma, beta, 1e-12, residual=r, out=out.window)
    torch.cuda.synchronize()
    out.assert_intact()
    _unchanged(keep)
    assert torch.equal(out.window, ops.add_layernorm(x, gamma, beta, 1e-12, residual=r))


@pytest.mark.parametrize("n", [1, 7, 8, 1003, 65537])
@pytest.mark.parametrize("src,dst", [(torch.float32, torch.float16), (torch.float16, torch.float32),
                                     (torch.float32, torch.bfloat16)])
def test_convert_stays_inside_its_output(cuda_device, n, src, dst):
    x = torch.randn(n).to(cuda_device).to(src)
    keep = x.clone()
    out = Guarded(1, n, dst, cuda_device)
    ops.convert(x, dst, out=out.window.view(-1))
    torch.cuda.synchronize()
    out.assert_intact()
    assert torch.equal(x, keep)
    assert torch.equal(out.window.view(-1), x.to(dst))


@pytest.mark.parametrize("K,N", [(72, 40), (768, 2304), (33 * 8, 31 * 8)])
def test_pack_weight_stays_inside_its_output(cuda_device, K, N):
    w = torch.randn(K, N).to(cuda_device)
    keep = w.clone()
    out = Guarded(N, K, torch.float16, cuda_device)
    ops.pack_weight(w, torch.float16, out=out.window)
    torch.cuda.synchronize()
    out.assert_intact()
    assert torch.equal(w, keep)
    assert torch.equal(out.window, w.t().half())


def test_front_end_and_head_stay_inside_their_outputs(cuda_device):
    B, S, H, vocab = 3, 50, 768, 1000
    g = torch.Generator(device="cpu").manual_seed(11)
    ids = torch.randint(0, vocab, (B, S), generator=g, dtype=torch.int32).to(cuda_device)
    seg = torch.randint(0, 2, (B, S), generator=g, dtype=torch.int32).to(cuda_device)
    word = torch.randn(vocab, H, generator=g).to(cuda_device).half()
    typ = torch.randn(2, H, generator=g).to(cuda_device).half()
    pos = torch.randn(512, H, generator=g).to(cuda_device).half()
    gamma, beta = torch.randn(H, generator=g).to(cuda_device), torch.randn(H, generator=g).to(cuda_device)
    out = Guarded(B * S, H, torch.float16, cuda_device)
    ops.embedding_layernorm(ids, seg, word, typ, pos, gamma, beta, 1e-12, out=out.window.unflatten(0, (B, S)))
    torch.cuda.synchronize()
    out.assert_intact()

    im = torch.ones(B, S, dtype=torch.int32)
    im[1, 20:] = 0
    im[2, 1:] = 0
    im = im.to(cuda_device)
    m = Guarded(B, S, torch.float32, cuda_device)
    kv = Guarded(1, B, torch.int32, cuda_device)
    # the additive mask of a valid key is 0.0, whose bits differ from the pattern; kv_len values are 50, 20, 1
    ops.mask_from_input_mask(im, out_mask=m.window, out_kv_len=kv.window.view(-1))
    torch.cuda.synchronize()
    m.assert_intact()
    kv.assert_intact()
    assert kv.window.view(-1).tolist() == [50, 20, 1]

    x = out.window
    wq = (torch.randn(H, 2, generator=g) * 0.05).to(cuda_device).contiguous()
    bq = torch.randn(2, generator=g).to(cuda_device)
    q = Guarded(2, B * S, torch.float32, cuda_device)
    ops.qa_head(x, wq, bq, out=q.window)
    torch.cuda.synchronize()
    q.assert_intact()
    want = (x.float() @ wq + bq).t()
    assert float((q.window - want).abs().max()) < 2e-3
