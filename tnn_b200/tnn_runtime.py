"""Drive a TNN instance whose DEVICE_CUDA is served by the tnn_b200 plug-in (the drop-in path).

Loads, in this order, the host framework (libTNN.so built from the unmodified TNN sources), the CUDA kernel library
and the plug-in (whose static constructors register the device, the accs, the fused layers and the graph pass), then
exposes the C shim over TNN's public API (tnn_plugin/tnn_capi.cc).
"""
import ctypes
import os

import numpy as np

from . import capi

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
LIBTNN = os.environ.get("TNN_B200_LIBTNN", os.path.join(_HERE, "host", "libTNN.so"))
SHIM = os.environ.get("TNN_B200_SHIM", os.path.join(_HERE, "host", "libtnn_capi.so"))
PLUGIN = os.path.join(_HERE, "lib", "libtnn_b200_plugin.so")

DEVICE_NAIVE, DEVICE_X86, DEVICE_CUDA = 0, 1, 2
PRECISION_AUTO, PRECISION_NORMAL, PRECISION_HIGH, PRECISION_LOW = -1, 0, 1, 2

_state = {}


def available():
    return all(os.path.exists(p) for p in (LIBTNN, SHIM, PLUGIN, capi.LIB_PATH))


def load():
    """Returns (shim, plugin) ctypes handles; raises if a piece is missing (there is no fallback)."""
    if "shim" not in _state:
        for p in (LIBTNN, capi.LIB_PATH, PLUGIN, SHIM):
            if not os.path.exists(p):
                raise RuntimeError("missing %s (build with tnn_b200/tnn_plugin/build_plugin.py)" % p)
        ctypes.CDLL(LIBTNN, mode=ctypes.RTLD_GLOBAL)
        ctypes.CDLL(capi.LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        plugin = ctypes.CDLL(PLUGIN, mode=ctypes.RTLD_GLOBAL)
        shim = ctypes.CDLL(SHIM)
        shim.tnnc_create.restype = ctypes.c_void_p
        shim.tnnc_create.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
        shim.tnnc_destroy.argtypes = [ctypes.c_void_p]
        shim.tnnc_last_error.restype = ctypes.c_char_p
        shim.tnnc_last_error.argtypes = [ctypes.c_void_p]
        shim.tnnc_set_input.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64]
        shim.tnnc_set_input_i32.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64]
        shim.tnnc_set_input_half.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        shim.tnnc_get_output_half.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        shim.tnnc_get_output_half.restype = ctypes.c_int64
        shim.tnnc_set_input_device.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        shim.tnnc_get_output_device.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int,
                                                ctypes.POINTER(ctypes.c_void_p)]
        shim.tnnc_get_output_device.restype = ctypes.c_int64
        shim.tnnc_forward.argtypes = [ctypes.c_void_p]
        shim.tnnc_time_forward.restype = ctypes.c_double
        shim.tnnc_time_forward.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        shim.tnnc_get_output.restype = ctypes.c_int64
        shim.tnnc_get_output.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64,
                                         ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        plugin.tnnb200_fuse_and_pack.restype = ctypes.c_int
        plugin.tnnb200_fuse_and_pack.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t,
                                                 ctypes.c_int, ctypes.c_char_p, ctypes.c_char_p]
        plugin.tnnb200_test_fuse.restype = ctypes.c_int
        plugin.tnnb200_test_fuse.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t,
                                             ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t]
        _state["shim"], _state["plugin"] = shim, plugin
    return _state["shim"], _state["plugin"]


def fuse_report(proto_path, model_path, precision=PRECISION_AUTO):
    """Run only the graph pass on a model (no GPU needed); returns the fused layer list as text lines."""
    _, plugin = load()
    proto = open(proto_path, "rb").read()
    model = open(model_path, "rb").read()
    buf = ctypes.create_string_buffer(1 << 22)
    n = plugin.tnnb200_test_fuse(proto, len(proto), model, len(model), precision, buf, len(buf))
    if n < 0:
        raise RuntimeError("tnnb200_test_fuse failed: %d" % n)
    return buf.value.decode().strip().split("\n")


def fuse_and_pack(proto_path, model_path, out_proto_path, out_model_path, precision=PRECISION_AUTO):
    """Run the graph pass on a model and save the optimised model (fused layers) with the reference's ModelPacker.
    Needs no GPU.  Returns the number of layers of the saved model."""
    _, plugin = load()
    proto = open(proto_path, "rb").read()
    model = open(model_path, "rb").read()
    n = plugin.tnnb200_fuse_and_pack(proto, len(proto), model, len(model), precision, out_proto_path.encode(),
                                     out_model_path.encode())
    if n < 0:
        raise RuntimeError("tnnb200_fuse_and_pack failed: %d" % n)
    return n


class Instance:
    """TNN::Init + CreateInst on a device; set_input / forward / get_output move fp32 host arrays."""

    def __init__(self, proto_path, model_path, device=DEVICE_CUDA, device_id=0, precision=PRECISION_AUTO, threads=1):
        self.shim, _ = load()
        err = ctypes.create_string_buffer(1024)
        self.h = self.shim.tnnc_create(proto_path.encode(), model_path.encode(), device, device_id, precision,
                                       threads, err, 1024)
        if not self.h:
            raise RuntimeError("TNN instance creation failed: %s" % err.value.decode())

    def close(self):
        if getattr(self, "h", None):
            self.shim.tnnc_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError("%s failed: 0x%X %s" % (what, rc & 0xFFFFFFFF,
                                                       self.shim.tnnc_last_error(self.h).decode()))

    def set_input(self, name, arr):
        a = np.ascontiguousarray(arr, dtype=np.float32)
        self._check(self.shim.tnnc_set_input(self.h, name.encode(), a.ctypes.data, a.size), "set_input(%s)" % name)

    def set_input_i32(self, name, arr):
        a = np.ascontiguousarray(arr, dtype=np.int32)
        self._check(self.shim.tnnc_set_input_i32(self.h, name.encode(), a.ctypes.data, a.size),
                    "set_input_i32(%s)" % name)

    def set_input_half(self, name, arr):
        """`arr`: numpy float16 (or uint16 bfloat16 bit patterns with bf16=True via set_input_bits)."""
        a = np.ascontiguousarray(arr, dtype=np.float16)
        self._check(self.shim.tnnc_set_input_half(self.h, name.encode(), a.ctypes.data, a.size, 0),
                    "set_input_half(%s)" % name)

    def get_output_half(self, name=""):
        n = self.shim.tnnc_get_output_half(self.h, name.encode(), None, 0, 0)
        if n < 0:
            raise RuntimeError("get_output_half: %s" % self.shim.tnnc_last_error(self.h).decode())
        out = np.empty((n,), np.float16)
        if self.shim.tnnc_get_output_half(self.h, name.encode(), out.ctypes.data, n, 0) != n:
            raise RuntimeError("get_output_half: %s" % self.shim.tnnc_last_error(self.h).decode())
        return out

    # Device-resident Mats: kind 0 fp32, 1 fp16, 2 bf16 bit patterns, 3 int32.
    MAT_F32, MAT_F16, MAT_BF16, MAT_I32 = 0, 1, 2, 3

    def set_input_device(self, name, device_ptr, count, kind):
        """Input from device memory of the instance's GPU (a DEVICE_CUDA Mat): no host copy.  The caller orders the
        producer of that memory before this call (the converter works on the instance's own stream)."""
        self._check(self.shim.tnnc_set_input_device(self.h, name.encode(), ctypes.c_void_p(device_ptr), count, kind),
                    "set_input_device(%s)" % name)

    def get_output_device(self, name="", kind=1):
        """(device pointer, element count) of the output as a DEVICE_CUDA Mat owned by the instance."""
        ptr = ctypes.c_void_p()
        n = self.shim.tnnc_get_output_device(self.h, name.encode(), kind, ctypes.byref(ptr))
        if n < 0:
            raise RuntimeError("get_output_device: %s" % self.shim.tnnc_last_error(self.h).decode())
        return ptr.value, n

    def forward(self):
        self._check(self.shim.tnnc_forward(self.h), "Forward")

    def time_forward(self, warmup, iters):
        ms = self.shim.tnnc_time_forward(self.h, warmup, iters)
        if ms < 0:
            raise RuntimeError("Forward failed while timing: %s" % self.shim.tnnc_last_error(self.h).decode())
        return ms

    def get_output(self, name=""):
        dims = (ctypes.c_int * 8)()
        nd = ctypes.c_int(0)
        n = self.shim.tnnc_get_output(self.h, name.encode(), None, 0, dims, ctypes.byref(nd))
        if n < 0:
            raise RuntimeError("get_output: %s" % self.shim.tnnc_last_error(self.h).decode())
        out = np.empty((n,), np.float32)
        n2 = self.shim.tnnc_get_output(self.h, name.encode(), out.ctypes.data, n, dims, ctypes.byref(nd))
        if n2 != n:
            raise RuntimeError("get_output: %s" % self.shim.tnnc_last_error(self.h).decode())
        return out.reshape([dims[i] for i in range(nd.value)])
