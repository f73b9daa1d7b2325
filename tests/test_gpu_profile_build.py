"""GPU: the reference's per-layer profiling (TNN_PROFILE builds: Instance::StartProfile / FinishProfile,
source/tnn/core/profile.h, source/tnn/device/x86/acc/x86_layer_acc.cc:55-73 for the CPU accs) served by the plug-in's
accs on DEVICE_CUDA.  TNN_PROFILE adds members to TNN's classes, so host framework, shim and plug-in are a build of
their own (oracle/build_ref.py --profile --out oracle/_ref_profile; tnn_plugin/build_plugin.py --profile) and run in a
process of their own; the test is skipped where that build is absent."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NEEDED = [os.path.join(ROOT, "tnn_b200", "host_profile", "libTNN.so"),
          os.path.join(ROOT, "tnn_b200", "host_profile", "libtnn_capi.so"),
          os.path.join(ROOT, "tnn_b200", "lib_profile", "libtnn_b200_plugin.so")]

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not all(os.path.exists(p) for p in NEEDED), reason="no TNN_PROFILE build present")]

SCRIPT = r"""
import os, sys, tempfile
import numpy as np
sys.path.insert(0, %(root)r)
sys.path.insert(0, os.path.join(%(root)r, "tests"))
from oracle.make_golden import CASES, golden_workload
from tnn_b200 import model_synth as ms, tnn_runtime as rt
wl = golden_workload(**CASES["base_2layer_ragged"])
d = tempfile.mkdtemp()
proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
ms.write_tnn_model(wl, proto, model)
inst = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
inst.set_input("x", wl.x)
inst.set_input("mask", wl.mask_add)
inst.forward()
inst.forward()
inst.forward()                       # by now the instance replays a captured graph
plain = inst.get_output()
inst.start_profile()
inst.forward()
inst.forward()
table = inst.finish_profile()
profiled = inst.get_output()
inst.forward()                       # and replays again once the profile is closed
after = inst.get_output()
counters = inst.graph_counters()
print("EQUAL", bool(np.array_equal(plain, profiled)), bool(np.array_equal(plain, after)))
print("COUNTERS", counters)
print("TABLE-BEGIN")
print(table)
print("TABLE-END")
"""


def test_per_layer_profile_of_the_fused_accs():
    env = dict(os.environ, TNN_B200_PROFILE_BUILD="1")
    out = subprocess.run([sys.executable, "-c", SCRIPT % {"root": ROOT}], env=env, capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    text = out.stdout
    assert "EQUAL True True" in text                      # profiling changes nothing but the way layers are launched
    table = text.split("TABLE-BEGIN", 1)[1].split("TABLE-END", 1)[0]
    rows = [[c.strip() for c in line.strip().strip("|").split("|")] for line in table.splitlines()
            if line.startswith("|") and "Op Type" not in line]
    per_layer = [r for r in rows if len(r) >= 5]
    types = {r[1] for r in per_layer}
    assert {"FusedLinear", "FusedAttention", "LayerNorm"} <= types, types
    # 2 encoder layers = 2 x (QKV, attention, out-proj, LayerNorm, FFN1, FFN2, LayerNorm), each with a device time
    fused = [r for r in per_layer if r[1] in ("FusedLinear", "FusedAttention", "LayerNorm")]
    assert len(fused) >= 14
    assert all(float(r[2]) > 0.0 for r in fused), fused[:3]
    assert "kernel runtime total" in table
