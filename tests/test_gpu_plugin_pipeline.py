"""GPU: the serving path inside the plug-in — CUDA-graph replay of Instance::Forward, the blob converter's page-locked
staging and asynchronous conversions, pipelined Forwards over one and two instances, and the device's memory arena
(no driver allocation in steady state, injected allocation failure).  Everything goes through TNN's own API
(Instance / BlobConverter) via the C shim; results are compared with a plain blocking Forward and the x86 fixture."""
import os
import tempfile

import numpy as np
import pytest

from oracle.make_golden import CASES, GOLDEN, golden_workload
from tnn_b200 import model_synth as ms
from tnn_b200 import tnn_runtime as rt
from util import MAX_ABS_TOL, max_abs

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not rt.available(), reason="TNN host framework / plug-in missing")]


def _files(wl):
    d = tempfile.mkdtemp(prefix="plug_pipe_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model)
    return proto, model


def _blocking(inst, x, mask):
    inst.set_input("x", x)
    inst.set_input("mask", mask)
    inst.forward()
    return inst.get_output()


def test_graph_replay_equals_layer_by_layer_launches(cuda_device):
    """Forward 1 launches layer by layer, Forward 2 is captured, Forward 3+ replay the graph: same bits every time, also
    when the input changes between Forwards (the graph reads the blobs, not a snapshot of them)."""
    wl = golden_workload(**CASES["base_2layer_ragged"])
    proto, model = _files(wl)
    inst = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    first = _blocking(inst, wl.x, wl.mask_add)
    assert inst.graph_counters() == {"eager": 1, "captures": 0, "launches": 0, "failures": 0}
    outs = [_blocking(inst, wl.x, wl.mask_add) for _ in range(3)]
    c = inst.graph_counters()
    assert c["captures"] == 1 and c["launches"] == 3 and c["failures"] == 0 and c["eager"] == 1, c
    for o in outs:
        assert np.array_equal(first, o)
    ref = np.load(os.path.join(GOLDEN, "base_2layer_ragged.npz"))["x86"]
    assert max_abs(first, ref) <= MAX_ABS_TOL
    # another input through the replayed graph against a fresh instance that launches it layer by layer
    x2 = np.ascontiguousarray(wl.x[::-1])
    m2 = np.ascontiguousarray(wl.mask_add[::-1])
    y2 = _blocking(inst, x2, m2)
    assert inst.graph_counters()["launches"] == 4
    fresh = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    assert np.array_equal(y2, _blocking(fresh, x2, m2))
    assert not np.array_equal(y2, first)
    inst.close()
    fresh.close()


def test_graph_replay_can_be_switched_off(cuda_device, monkeypatch):
    wl = golden_workload(**CASES["c1_attention_block"])
    proto, model = _files(wl)
    monkeypatch.setenv("TNN_B200_GRAPH", "0")
    inst = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    a = _blocking(inst, wl.x, wl.mask_add)
    b = _blocking(inst, wl.x, wl.mask_add)
    b = _blocking(inst, wl.x, wl.mask_add)
    assert inst.graph_counters() == {"eager": 3, "captures": 0, "launches": 0, "failures": 0}
    assert np.array_equal(a, b)
    inst.close()


@pytest.mark.parametrize("pinned", [False, True])
def test_back_to_back_pipelined_forwards_return_each_inputs_own_result(cuda_device, pinned):
    """ConvertFromMatAsync -> ForwardAsync -> ConvertToMatAsync twice in a row with different inputs and no
    synchronisation in between, then one blocking conversion: each output buffer holds its own input's result."""
    wl = golden_workload(**CASES["base_2layer_ragged"])
    proto, model = _files(wl)
    inst = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    xs = [wl.x, np.ascontiguousarray(wl.x[::-1] * np.float32(0.5))]
    masks = [wl.mask_add, np.ascontiguousarray(wl.mask_add[::-1])]
    want = [_blocking(inst, x, m) for x, m in zip(xs, masks)]      # also warms the graph up
    keep = []

    def buf(a):
        if not pinned:
            return np.array(a, copy=True)
        p = rt.PinnedArray(a.shape, a.dtype)
        p.array[...] = a
        keep.append(p)
        return p.array

    ins = [(buf(x), buf(m)) for x, m in zip(xs, masks)]
    outs = [buf(np.zeros_like(want[0])) for _ in range(2)]
    probe = buf(np.zeros_like(want[0]))
    for i in range(2):
        inst.from_mat_async("x", ins[i][0])
        inst.from_mat_async("mask", ins[i][1])
        if not pinned:
            ins[i][0][...] = 7.0        # the Mat has been read when ConvertFromMatAsync returns: scribbling is harmless
        inst.forward_async()
        inst.to_mat("", outs[i], blocking=False)
    inst.to_mat("", probe, blocking=True)                               # drains the queue
    assert np.array_equal(outs[0], want[0])
    assert np.array_equal(outs[1], want[1])
    assert np.array_equal(probe, want[1])
    inst.close()
    for p in keep:
        p.free()


@pytest.mark.parametrize("n_inst", [1, 2, 3])
def test_native_pipeline_loop_over_instances(cuda_device, n_inst):
    """tnnc_run_pipeline (the reference benchmark's loop, over one instance or two taken in turn): after the loop every
    instance's output buffer holds the result of the input it was given."""
    wl = golden_workload(**CASES["base_2layer_ragged"])
    proto, model = _files(wl)
    insts = [rt.Instance(proto, model, device=rt.DEVICE_CUDA) for _ in range(n_inst)]
    xs = [np.ascontiguousarray(wl.x * np.float32(1.0 - 0.25 * k)) for k in range(n_inst)]
    want = [_blocking(insts[k], xs[k], wl.mask_add) for k in range(n_inst)]
    outs = [np.zeros_like(want[0]) for _ in range(n_inst)]
    inputs = [[("x", xs[k]), ("mask", wl.mask_add)] for k in range(n_inst)]
    outputs = [[("", outs[k])] for k in range(n_inst)]
    secs = rt.run_pipeline(insts, inputs, outputs, warmup=3, steps=7)
    assert secs > 0
    for k in range(n_inst):
        assert np.array_equal(outs[k], want[k]), k
        assert insts[k].graph_counters()["failures"] == 0
    for i in insts:
        i.close()


def test_steady_state_takes_no_memory_from_the_driver(cuda_device):
    """The first SetInputMat / Forward / GetOutputMat of an instance sizes its staging; after that neither Forward nor
    the conversions allocate (device or page-locked host memory), and an instance that is destroyed and created again
    is served from the arena without a single cudaMalloc."""
    wl = golden_workload(**CASES["base_2layer_ragged"])
    proto, model = _files(wl)
    inst = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    y0 = _blocking(inst, wl.x, wl.mask_add)
    s0 = rt.arena_stats(0)
    assert s0["driver_allocations"] >= 1 and s0["bytes_in_use"] > 0 and s0["bytes_reserved"] >= s0["bytes_in_use"]
    for _ in range(3):
        assert np.array_equal(_blocking(inst, wl.x, wl.mask_add), y0)
    s1 = rt.arena_stats(0)
    for k in ("driver_allocations", "pinned_allocations", "requests", "live_blocks", "bytes_in_use"):
        assert s1[k] == s0[k], (k, s0, s1)
    inst.close()
    s2 = rt.arena_stats(0)
    assert s2["bytes_reserved"] == s1["bytes_reserved"] and s2["bytes_in_use"] < s1["bytes_in_use"]
    again = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    assert np.array_equal(_blocking(again, wl.x, wl.mask_add), y0)
    s3 = rt.arena_stats(0)
    assert s3["driver_allocations"] == s1["driver_allocations"], (s1, s3)
    assert s3["pinned_allocations"] == s1["pinned_allocations"], (s1, s3)
    again.close()
    live = rt.arena_stats(0)["live_blocks"]
    assert rt.release_cached_memory(0) >= 0
    assert rt.arena_stats(0)["live_blocks"] == live


def test_injected_allocation_failure_is_reported_and_leaks_nothing(cuda_device):
    """Host-side fault injection: allocations that fail during CreateInst come back as an error status (instance
    creation raises, nothing aborts), the blocks taken before the failure are returned, and the next creation works.
    Instance::Init tries a DEVICE_CUDA network twice (source/tnn/core/instance.cc:86-124), so the injection stays on
    until both attempts have failed: the first one `skip` allocations into its Init, the second at its first."""
    wl = golden_workload(**CASES["c1_attention_block"])
    proto, model = _files(wl)
    warm = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    want = _blocking(warm, wl.x, wl.mask_add)
    warm.close()
    before = rt.arena_stats(0)
    for skip in (0, 2, 7):            # the first allocation (context set-up), an early one, one in the middle of Init
        rt.inject_allocation_failure(skip, 1 << 30)
        try:
            with pytest.raises(RuntimeError):
                rt.Instance(proto, model, device=rt.DEVICE_CUDA)
        finally:
            rt.inject_allocation_failure(0, 0)
        after = rt.arena_stats(0)
        assert after["live_blocks"] == before["live_blocks"], (skip, before, after)
        assert after["bytes_in_use"] == before["bytes_in_use"]
    ok = rt.Instance(proto, model, device=rt.DEVICE_CUDA)
    assert np.array_equal(_blocking(ok, wl.x, wl.mask_add), want)
    ok.close()


@pytest.mark.parametrize("input_dtype,precision", [("half", rt.PRECISION_AUTO), ("bf16", rt.PRECISION_LOW)])
def test_host_side_half_conversion_changes_no_bit(cuda_device, monkeypatch, input_dtype, precision):
    """TNN_B200_HOST_CONVERT=1: fp32 host Mats of half-precision blobs (a model whose activation input is declared half
    or bfloat16) are converted on the host cores, so that half the bytes cross the bus.  Same bits as the device-side
    conversion, through the blocking calls and through the pipelined loop, with pageable and page-locked Mats."""
    wl = golden_workload(**CASES["base_2layer_ragged"])
    d = tempfile.mkdtemp(prefix="plug_hostconv_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model, input_dtype=input_dtype)
    insts = [rt.Instance(proto, model, device=rt.DEVICE_CUDA, precision=precision) for _ in range(2)]
    monkeypatch.delenv("TNN_B200_HOST_CONVERT", raising=False)
    want = _blocking(insts[0], wl.x, wl.mask_add)
    n0 = rt.host_conversions()
    monkeypatch.setenv("TNN_B200_HOST_CONVERT", "1")
    assert np.array_equal(_blocking(insts[0], wl.x, wl.mask_add), want)
    assert rt.host_conversions() == n0 + 2        # the activation in, the result out; the fp32 mask blob is a plain copy
    keep = []
    for pin in (False, True):
        ins, outs = [], []
        for _ in insts:
            if pin:
                px, pm, po = (rt.PinnedArray(a.shape, np.float32) for a in (wl.x, wl.mask_add, want))
                px.array[...] = wl.x
                pm.array[...] = wl.mask_add
                po.array[...] = 0
                keep += [px, pm, po]
                ins.append([("x", px.array), ("mask", pm.array)])
                outs.append([("", po.array)])
            else:
                ins.append([("x", np.array(wl.x, copy=True)), ("mask", np.array(wl.mask_add, copy=True))])
                outs.append([("", np.zeros_like(want))])
        assert rt.run_pipeline(insts, ins, outs, warmup=2, steps=5) > 0
        for o in outs:
            assert np.array_equal(o[0][1], want), pin
    assert rt.host_conversions() == n0 + 2 + 2 * 2 * (2 + 5)   # two rounds of 7 steps, in and out
    for p in keep:
        p.free()
    for i in insts:
        i.close()
