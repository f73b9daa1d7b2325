"""CPU: the blob converter's host-side fp32 <-> half conversion (TNN_B200_HOST_CONVERT) rounds exactly like the
device's conversion kernel: to nearest even, subnormal halves included, overflow to infinity, NaN kept.  numpy's float16
conversion and torch's bfloat16 conversion are the yardsticks; both the F16C path and the portable scalar path run."""
import numpy as np
import pytest
import torch

from tnn_b200 import tnn_runtime as rt

pytestmark = pytest.mark.skipif(not rt.available(), reason="the plug-in is not built")


def _values():
    rng = np.random.default_rng(0)
    parts = [rng.normal(0, 1, 300000).astype(np.float32),
             (rng.normal(0, 1, 100000) * 1e-5).astype(np.float32),           # subnormal halves
             (rng.normal(0, 1, 50000) * 3e4).astype(np.float32),             # around the largest half
             np.array([0.0, -0.0, 1.0, -1.0, 65504.0, 65519.9, 65520.0, -65520.0, 1e9, -1e9, np.inf, -np.inf, np.nan,
                       5.9604645e-8, 2.9802322e-8, 2.9802326e-8, 8.940697e-8, 6.1035156e-5, 6.0975552e-5,
                       1.0009765625, 1.00048828125, 1.00146484375, 2049.0, 2051.0, 1e-40, -1e-40], np.float32)]
    # exact ties between two neighbouring halves, in every binade of the normal range
    mant = rng.integers(0, 1024, 20000).astype(np.uint32)
    expo = rng.integers(113, 142, 20000).astype(np.uint32)
    ties = ((expo << 23) | (mant << 13) | 0x1000).view(np.float32)
    parts.append(ties)
    parts.append(-ties)
    return np.concatenate(parts)


@pytest.mark.parametrize("force_scalar", [False, True])
def test_fp16_matches_numpy(force_scalar):
    x = _values()
    half, back, _ = rt.host_convert(x, bf16=False, force_scalar=force_scalar)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16)
    nan = np.isnan(x)
    assert np.array_equal(half[~nan], want.view(np.uint16)[~nan])
    assert np.isnan(half.view(np.float16)[nan]).all()
    assert np.array_equal(back[~nan], want.astype(np.float32)[~nan])


@pytest.mark.parametrize("force_scalar", [False, True])
def test_bf16_matches_torch(force_scalar):
    x = _values()
    half, back, _ = rt.host_convert(x, bf16=True, force_scalar=force_scalar)
    want = torch.from_numpy(x).to(torch.bfloat16)
    want_bits = want.view(torch.int16).numpy().view(np.uint16)
    nan = np.isnan(x)
    assert np.array_equal(half[~nan], want_bits[~nan])
    assert np.isnan(back[nan]).all()
    assert np.array_equal(back[~nan], want.float().numpy()[~nan])
