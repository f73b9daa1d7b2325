"""Run the reference's own CPU implementation (DEVICE_X86 / DEVICE_NAIVE of oracle/_ref/libTNN.so) from Python.

TEST INFRASTRUCTURE ONLY: used by oracle/make_golden.py, tests/ and bench.py's CPU-baseline / reference arm.
"""
import ctypes
import os
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
CAPI = os.path.join(REF_DIR, "libtnn_capi.so")
LIBTNN = os.path.join(REF_DIR, "libTNN.so")

DEVICE_NAIVE, DEVICE_X86, DEVICE_CUDA = 0, 1, 2
PRECISION_AUTO, PRECISION_NORMAL, PRECISION_HIGH, PRECISION_LOW = -1, 0, 1, 2


def available():
    return os.path.exists(CAPI) and os.path.exists(LIBTNN)


_lib = None


def _loaded_libtnn():
    """Path of a libTNN.so this process has already mapped, or None.  A process must hold ONE copy of the framework:
    its registries (devices, layers, accs, passes) are static objects, and a second copy would own a second set."""
    try:
        with open("/proc/self/maps") as fh:
            for line in fh:
                path = line.rstrip("\n").rsplit(" ", 1)[-1]
                if path.endswith("/libTNN.so"):
                    return path
    except OSError:
        pass
    return None


def capi():
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError("reference build missing: run `python oracle/build_ref.py` where the reference "
                               "sources are present")
        ctypes.CDLL(_loaded_libtnn() or LIBTNN, mode=ctypes.RTLD_GLOBAL)
        l = ctypes.CDLL(CAPI)
        l.tnnc_create.restype = ctypes.c_void_p
        l.tnnc_create.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                  ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
        l.tnnc_destroy.argtypes = [ctypes.c_void_p]
        l.tnnc_last_error.restype = ctypes.c_char_p
        l.tnnc_last_error.argtypes = [ctypes.c_void_p]
        l.tnnc_set_input.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64]
        l.tnnc_set_input_i32.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64]
        l.tnnc_forward.argtypes = [ctypes.c_void_p]
        l.tnnc_time_forward.restype = ctypes.c_double
        l.tnnc_time_forward.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        l.tnnc_get_output.restype = ctypes.c_int64
        l.tnnc_get_output.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64,
                                      ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        _lib = l
    return _lib


class TnnInstance:
    """One TNN instance created from tnnproto/tnnmodel files on the given device."""

    def __init__(self, proto_path, model_path, device=DEVICE_X86, device_id=0, precision=PRECISION_HIGH, threads=1):
        self.l = capi()
        err = ctypes.create_string_buffer(512)
        self.h = self.l.tnnc_create(proto_path.encode(), model_path.encode(), device, device_id, precision, threads,
                                    err, 512)
        if not self.h:
            raise RuntimeError("tnnc_create failed: %s" % err.value.decode())

    def close(self):
        if self.h:
            self.l.tnnc_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError("%s failed: %d %s" % (what, rc, self.l.tnnc_last_error(self.h).decode()))

    def set_input(self, name, arr):
        a = np.ascontiguousarray(arr, dtype=np.float32)
        self._check(self.l.tnnc_set_input(self.h, name.encode(), a.ctypes.data, a.size), "set_input(%s)" % name)

    def set_input_i32(self, name, arr):
        a = np.ascontiguousarray(arr, dtype=np.int32)
        self._check(self.l.tnnc_set_input_i32(self.h, name.encode(), a.ctypes.data, a.size), "set_input_i32(%s)" % name)

    def forward(self):
        self._check(self.l.tnnc_forward(self.h), "forward")

    def time_forward(self, warmup, iters):
        ms = self.l.tnnc_time_forward(self.h, warmup, iters)
        if ms < 0:
            raise RuntimeError("forward failed while timing")
        return ms

    def get_output(self, name=""):
        dims = (ctypes.c_int * 8)()
        nd = ctypes.c_int(0)
        n = self.l.tnnc_get_output(self.h, name.encode(), None, 0, dims, ctypes.byref(nd))
        if n < 0:
            raise RuntimeError("get_output: %s" % self.l.tnnc_last_error(self.h).decode())
        out = np.empty((n,), np.float32)
        n2 = self.l.tnnc_get_output(self.h, name.encode(), out.ctypes.data, n, dims, ctypes.byref(nd))
        if n2 != n:
            raise RuntimeError("get_output: %s" % self.l.tnnc_last_error(self.h).decode())
        return out.reshape([dims[i] for i in range(nd.value)])


def run_workload(wl, device=DEVICE_X86, threads=1, time_iters=0, warmup=1, workdir=None, pooler=None, qa=None):
    """Write `wl` as TNN files, run it on the reference CPU device; returns (output, ms_per_forward or None); with `qa`
    the output is the pair (start logits, end logits)."""
    from tnn_b200 import model_synth
    d = workdir or tempfile.mkdtemp(prefix="tnnref_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    names = model_synth.write_tnn_model(wl, proto, model, pooler=pooler, qa=qa)
    inst = TnnInstance(proto, model, device=device, threads=threads)
    inst.set_input("x", wl.x)
    inst.set_input("mask", wl.mask_add)
    ms = None
    if time_iters > 0:
        ms = inst.time_forward(warmup, time_iters)
    else:
        inst.forward()
    out = tuple(inst.get_output(n) for n in names) if qa is not None else inst.get_output()
    inst.close()
    return out, ms
