"""GPU: the fused encoder through the C ABI against (a) outputs of the reference's DEVICE_X86 committed under
tests/golden and (b) the CPU oracle, at the benchmark's tolerances."""
import os

import numpy as np
import pytest
import torch

from oracle import bert_oracle
from oracle.make_golden import CASES, GOLDEN, golden_workload
from tnn_b200 import capi, model_synth
from tnn_b200.encoder import Encoder
from util import COS_TOL, MAX_ABS_TOL, cosine, max_abs, valid_rows

pytestmark = pytest.mark.gpu


def _run(wl, dtype, single_call=True, fold=True, layernorm_in_gemm=False):
    enc = Encoder.from_workload(wl, dtype, fold_layernorm=fold)
    enc.layernorm_in_gemm = layernorm_in_gemm
    x = torch.from_numpy(wl.x).cuda()
    m = torch.from_numpy(wl.mask_add).cuda()
    y = enc.forward(x, m) if single_call else enc.forward_ops(x, m)
    torch.cuda.synchronize()
    assert capi.device_status() == capi.OK
    return y.cpu().numpy()


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fold", [True, False])   # LayerNorms folded into the GEMMs (5 launches/layer) or kept (7)
def test_against_reference_x86_fixture(cuda_device, name, dtype, fold):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    wl = golden_workload(**CASES[name])
    y = _run(wl, dtype, fold=fold)
    ref = g["x86"]
    # full tensor: padded query rows are computed like any other row, as the reference does
    tol = MAX_ABS_TOL if dtype == torch.float16 else 4 * MAX_ABS_TOL   # bf16 carries 3 fewer mantissa bits
    assert max_abs(y, ref) <= tol
    assert cosine(y, ref) >= (COS_TOL if dtype == torch.float16 else 0.999)
    assert max_abs(valid_rows(y, wl.lengths), valid_rows(ref, wl.lengths)) <= tol


@pytest.mark.parametrize("fold", [True, False])
def test_single_call_equals_layer_by_layer(cuda_device, fold):
    wl = golden_workload(**CASES["base_2layer_ragged"])
    a = _run(wl, torch.float16, single_call=True, fold=fold)
    b = _run(wl, torch.float16, single_call=False, fold=fold)
    assert np.array_equal(a, b)


def test_layernorm_in_gemm_launch_equals_separate_launches(cuda_device):
    """b200_encoder_fwd with the LayerNorms inside the producing GEMM launches (5 launches per layer) against the
    same stack with separate LayerNorm launches (7): the arithmetic is the same, so is every bit."""
    for case in ("base_2layer_ragged", "large_1layer_s96"):
        wl = golden_workload(**CASES[case])
        a = _run(wl, torch.float16, fold=False)
        b = _run(wl, torch.float16, fold=False, layernorm_in_gemm=True)
        assert np.array_equal(a, b)
    wl = model_synth.config_workload(2, batch=16, num_layers=2)
    a = _run(wl, torch.float16, fold=False)
    b = _run(wl, torch.float16, fold=False, layernorm_in_gemm=True)
    assert np.array_equal(a, b)


def test_config2_shape_subset_against_oracle(cuda_device):
    """Config 2 geometry (12 layers, S=128, full length) on the first 4 sequences of the seeded batch."""
    wl = model_synth.config_workload(2, batch=4)
    y = _run(wl, torch.float16)
    want = bert_oracle.encoder_forward(wl)
    assert max_abs(y, want) <= MAX_ABS_TOL
    assert cosine(y, want) >= COS_TOL


def test_config3_ragged_against_oracle(cuda_device):
    """Config 3 geometry: S=256, lengths ~ U[16,256], 12 layers, first 4 sequences."""
    wl = model_synth.config_workload(3, batch=4)
    y = _run(wl, torch.float16)
    want = bert_oracle.encoder_forward(wl)
    assert max_abs(valid_rows(y, wl.lengths), valid_rows(want, wl.lengths)) <= MAX_ABS_TOL
    assert cosine(valid_rows(y, wl.lengths), valid_rows(want, wl.lengths)) >= COS_TOL


def test_sequences_are_independent_at_full_batch(cuda_device):
    """Size-independent property at config 2's full batch: a sequence's output does not depend on its batch-mates
    (run B=64, then the first 4 alone: bit-identical)."""
    wl = model_synth.config_workload(2, batch=64, num_layers=2)
    y = _run(wl, torch.float16)
    sub = model_synth.Workload(wl.cfg, wl.weights, wl.x[:4], wl.lengths[:4], wl.mask_add[:4], wl.meta)
    y4 = _run(sub, torch.float16)
    assert np.array_equal(y[:4], y4)


def test_config4_geometry_bf16_and_f16_against_oracle(cuda_device):
    """Config 4 geometry: BERT-large (H=1024, 16 heads, FFN 4096), S=384, lengths ~ U[128,384]; first 2 sequences of the
    seeded batch and the first 4 of the 24 layers (sequences are independent; the oracle needs ~10 s per layer here)."""
    wl = model_synth.config_workload(4, batch=2, num_layers=4)
    want = bert_oracle.encoder_forward(wl)
    vw = valid_rows(want, wl.lengths)
    y = _run(wl, torch.float16, fold=False)
    assert max_abs(valid_rows(y, wl.lengths), vw) <= MAX_ABS_TOL
    assert cosine(valid_rows(y, wl.lengths), vw) >= COS_TOL
    yb = _run(wl, torch.bfloat16, fold=False)
    assert max_abs(valid_rows(yb, wl.lengths), vw) <= 4 * MAX_ABS_TOL
    assert cosine(valid_rows(yb, wl.lengths), vw) >= 0.999


def test_config5_batch_shard_is_a_slice_of_the_full_batch(cuda_device):
    """Config 5 shards one batch over GPUs: a rank's shard must give what the same rows give in the full batch
    (128 sequences = the per-GPU shard at 8 GPUs, against its first and last 16-sequence slices; 2 layers)."""
    wl = model_synth.config_workload(5, batch=128, num_layers=2)
    y = _run(wl, torch.float16, fold=False)
    for lo in (0, 112):
        sub = model_synth.Workload(wl.cfg, wl.weights, wl.x[lo:lo + 16], wl.lengths[lo:lo + 16],
                                   wl.mask_add[lo:lo + 16], wl.meta)
        assert np.array_equal(y[lo:lo + 16], _run(sub, torch.float16, fold=False))
