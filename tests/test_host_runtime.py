"""CPU: the host framework's instance API as the Python mirror drives it (tnn_b200/tnn_runtime.py over the C shim), on
the reference's DEVICE_X86: Reshape within the created shapes and the share_memory_mode settings.  The GPU tests run the
same calls on DEVICE_CUDA; these pin what the calls mean."""
import os
import tempfile

import numpy as np
import pytest

from oracle import bert_oracle
from oracle.make_golden import CASES, golden_workload
from tnn_b200 import model_synth as ms
from tnn_b200 import tnn_runtime as rt

pytestmark = pytest.mark.skipif(not rt.available(), reason="the host framework is not built")


@pytest.fixture(scope="module")
def model_files():
    wl = golden_workload(**CASES["base_2layer_ragged"])
    d = tempfile.mkdtemp(prefix="host_rt_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model)
    return wl, proto, model


def _run(inst, x, mask):
    inst.set_input("x", x)
    inst.set_input("mask", mask)
    inst.forward()
    return inst.get_output()


def test_reshape_follows_the_oracle_at_every_shape(model_files):
    wl, proto, model = model_files
    B, S, H = wl.x.shape
    inst = rt.Instance(proto, model, device=rt.DEVICE_X86, precision=rt.PRECISION_HIGH)
    for b, s in ((1, 96), (B, 64), (B, S)):
        x = np.ascontiguousarray(wl.x[:b, :s])
        mask = np.ascontiguousarray(wl.mask_add[:b, :, :, :s])
        inst.reshape({"x": [b, s, H], "mask": [b, 1, 1, s]})
        y = _run(inst, x, mask)
        sub = ms.Workload(wl.cfg, wl.weights, x, np.minimum(wl.lengths[:b], s), mask, wl.meta)
        assert y.shape == (b, s, H)
        assert float(np.abs(y - bert_oracle.encoder_forward(sub)).max()) < 5e-5
    inst.close()


def test_share_memory_modes_give_the_default_result(model_files):
    wl, proto, model = model_files
    plain = rt.Instance(proto, model, device=rt.DEVICE_X86, precision=rt.PRECISION_HIGH)
    want = _run(plain, wl.x, wl.mask_add)
    ext = rt.Instance(proto, model, device=rt.DEVICE_X86, precision=rt.PRECISION_HIGH,
                      share_memory_mode=rt.SHARE_MEMORY_FROM_EXTERNAL)
    size = ext.forward_memory_size()
    block = np.full(size + 64, 0x5A, np.uint8)
    ext.set_forward_memory(block.ctypes.data)
    assert np.array_equal(_run(ext, wl.x, wl.mask_add), want)
    assert (block[size:] == 0x5A).all()
    one = [rt.Instance(proto, model, device=rt.DEVICE_X86, precision=rt.PRECISION_HIGH,
                       share_memory_mode=rt.SHARE_MEMORY_ONE_THREAD) for _ in range(2)]
    for inst in one:
        assert np.array_equal(_run(inst, wl.x, wl.mask_add), want)
    for inst in one + [ext, plain]:
        inst.close()
