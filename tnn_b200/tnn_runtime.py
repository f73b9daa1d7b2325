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
# TNN_B200_PROFILE_BUILD=1 selects the TNN_PROFILE build of host framework, shim and plug-in (build_plugin.py --profile):
# the switch changes the layout of TNN's classes, so the three must come from the same build and a process uses one.
_SUFFIX = "_profile" if os.environ.get("TNN_B200_PROFILE_BUILD", "0") not in ("", "0") else ""
LIBTNN = os.environ.get("TNN_B200_LIBTNN", os.path.join(_HERE, "host" + _SUFFIX, "libTNN.so"))
SHIM = os.environ.get("TNN_B200_SHIM", os.path.join(_HERE, "host" + _SUFFIX, "libtnn_capi.so"))
PLUGIN = os.path.join(_HERE, "lib" + _SUFFIX, "libtnn_b200_plugin.so")

DEVICE_NAIVE, DEVICE_X86, DEVICE_CUDA = 0, 1, 2
PRECISION_AUTO, PRECISION_NORMAL, PRECISION_HIGH, PRECISION_LOW = -1, 0, 1, 2

_state = {}

MAT_F32, MAT_F16, MAT_BF16, MAT_I32 = 0, 1, 2, 3
_KIND_OF = {np.dtype(np.float32): MAT_F32, np.dtype(np.float16): MAT_F16, np.dtype(np.int32): MAT_I32}


class TnncIo(ctypes.Structure):
    """One input or output of tnnc_run_pipeline: blob name, host buffer, element count, Mat kind."""
    _fields_ = [("name", ctypes.c_char_p), ("host", ctypes.c_void_p), ("n", ctypes.c_int64), ("kind", ctypes.c_int32),
                ("reserved_", ctypes.c_int32)]


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


def available():
    return all(os.path.exists(p) for p in (LIBTNN, SHIM, PLUGIN, capi.LIB_PATH))


def load():
    """Returns (shim, plugin) ctypes handles; raises if a piece is missing (there is no fallback)."""
    if "shim" not in _state:
        for p in (LIBTNN, capi.LIB_PATH, PLUGIN, SHIM):
            if not os.path.exists(p):
                raise RuntimeError("missing %s (build with tnn_b200/tnn_plugin/build_plugin.py)" % p)
        ctypes.CDLL(_loaded_libtnn() or LIBTNN, mode=ctypes.RTLD_GLOBAL)
        ctypes.CDLL(capi.LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        plugin = ctypes.CDLL(PLUGIN, mode=ctypes.RTLD_GLOBAL)
        shim = ctypes.CDLL(SHIM)
        shim.tnnc_create.restype = ctypes.c_void_p
        shim.tnnc_create.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
        shim.tnnc_create_ex.restype = ctypes.c_void_p
        shim.tnnc_create_ex.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
        shim.tnnc_forward_memory_size.restype = ctypes.c_int64
        shim.tnnc_forward_memory_size.argtypes = [ctypes.c_void_p]
        shim.tnnc_set_forward_memory.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        shim.tnnc_share_command_queue.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
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
        shim.tnnc_start_profile.argtypes = [ctypes.c_void_p]
        shim.tnnc_finish_profile.restype = ctypes.c_int64
        shim.tnnc_finish_profile.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int64]
        shim.tnnc_reshape.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_char_p),
                                      ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        shim.tnnc_time_forward.restype = ctypes.c_double
        shim.tnnc_time_forward.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        shim.tnnc_get_output.restype = ctypes.c_int64
        shim.tnnc_get_output.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64,
                                         ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        shim.tnnc_from_mat_async.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        shim.tnnc_to_mat.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                     ctypes.c_int]
        shim.tnnc_forward_async.argtypes = [ctypes.c_void_p]
        shim.tnnc_command_queue.restype = ctypes.c_void_p
        shim.tnnc_command_queue.argtypes = [ctypes.c_void_p]
        shim.tnnc_run_pipeline.restype = ctypes.c_double
        shim.tnnc_run_pipeline.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.POINTER(TnncIo),
                                           ctypes.c_int, ctypes.POINTER(TnncIo), ctypes.c_int, ctypes.c_int, ctypes.c_int]
        plugin.tnnb200_arena_stats.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_uint64)]
        plugin.tnnb200_release_cached_memory.restype = ctypes.c_uint64
        plugin.tnnb200_release_cached_memory.argtypes = [ctypes.c_int]
        plugin.tnnb200_inject_allocation_failure.argtypes = [ctypes.c_int, ctypes.c_int]
        plugin.tnnb200_selftest_range_arena.restype = ctypes.c_int
        plugin.tnnb200_selftest_range_arena.argtypes = [ctypes.c_uint, ctypes.c_int, ctypes.c_int, ctypes.c_char_p,
                                                        ctypes.c_int]
        plugin.tnnb200_host_conversions.restype = ctypes.c_uint64
        plugin.tnnb200_host_convert.restype = ctypes.c_int
        plugin.tnnb200_host_convert.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_int,
                                                ctypes.c_void_p, ctypes.c_void_p]
        plugin.tnnb200_graph_counters.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint64)]
        plugin.tnnb200_host_alloc.restype = ctypes.c_void_p
        plugin.tnnb200_host_alloc.argtypes = [ctypes.c_size_t]
        plugin.tnnb200_host_free.argtypes = [ctypes.c_void_p]
        plugin.tnnb200_fuse_and_pack.restype = ctypes.c_int
        plugin.tnnb200_fuse_and_pack.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t,
                                                 ctypes.c_int, ctypes.c_char_p, ctypes.c_char_p]
        plugin.tnnb200_test_fuse_ex.restype = ctypes.c_int
        plugin.tnnb200_test_fuse_ex.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t,
                                                ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t,
                                                ctypes.c_char_p, ctypes.c_size_t]
        plugin.tnnb200_test_fuse.restype = ctypes.c_int
        plugin.tnnb200_test_fuse.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t,
                                             ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t]
        _state["shim"], _state["plugin"] = shim, plugin
    return _state["shim"], _state["plugin"]


class FuseRefused(RuntimeError):
    """The graph pass left the model unfused; `.args[0]` is its explanation."""


def fuse_report(proto_path, model_path, precision=PRECISION_AUTO, fold_constants=False):
    """Run only the graph pass on a model (no GPU needed); returns the fused layer list as text lines.
    fold_constants: if the pass refuses the graph, run the reference's constant folder on it (as Instance::Init does for
    DEVICE_CUDA) and try again.  Raises FuseRefused with the pass's explanation if the graph stays unfused."""
    _, plugin = load()
    proto = open(proto_path, "rb").read()
    model = open(model_path, "rb").read()
    buf = ctypes.create_string_buffer(1 << 22)
    err = ctypes.create_string_buffer(4096)
    n = plugin.tnnb200_test_fuse_ex(proto, len(proto), model, len(model), precision, 1 if fold_constants else 0,
                                    buf, len(buf), err, len(err))
    if n == -4:
        raise FuseRefused(err.value.decode())
    if n < 0:
        raise RuntimeError("tnnb200_test_fuse_ex failed: %d %s" % (n, err.value.decode()))
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


ARENA_KEYS = ("driver_allocations", "driver_frees", "bytes_reserved", "bytes_in_use", "live_blocks", "requests",
              "pinned_allocations", "pinned_bytes_reserved")


def arena_stats(device_id=0):
    """Counters of the plug-in's device-memory arena on one GPU (tnnb200_arena_stats) as a dict."""
    _, plugin = load()
    out = (ctypes.c_uint64 * 8)()
    plugin.tnnb200_arena_stats(device_id, out)
    return dict(zip(ARENA_KEYS, (int(v) for v in out)))


def release_cached_memory(device_id=-1):
    _, plugin = load()
    return int(plugin.tnnb200_release_cached_memory(device_id))


def inject_allocation_failure(skip, count):
    """Host-side fault injection: after `skip` more successful device allocations of the plug-in, the next `count`
    report out-of-memory (count = 0 switches it off)."""
    _, plugin = load()
    plugin.tnnb200_inject_allocation_failure(int(skip), int(count))


def selftest_range_arena(seed, steps, pooled=True):
    """Runs the arena's host-only self-test (no CUDA call); returns (failing step or 0, message)."""
    _, plugin = load()
    err = ctypes.create_string_buffer(256)
    rc = plugin.tnnb200_selftest_range_arena(int(seed), int(steps), 1 if pooled else 0, err, len(err))
    return int(rc), err.value.decode()


def host_conversions():
    """Mat <-> blob conversions of this process that took the converter's host-side route."""
    _, plugin = load()
    return int(plugin.tnnb200_host_conversions())


def host_convert(src, bf16=False, force_scalar=False):
    """The blob converter's host-side fp32 -> half conversion and back: (uint16 bit patterns, fp32 round trip, vector
    path used)."""
    _, plugin = load()
    a = np.ascontiguousarray(src, dtype=np.float32).ravel()
    half = np.empty(a.shape, np.uint16)
    back = np.empty(a.shape, np.float32)
    rc = plugin.tnnb200_host_convert(a.ctypes.data, a.size, 1 if bf16 else 0, 1 if force_scalar else 0,
                                     half.ctypes.data, back.ctypes.data)
    if rc < 0:
        raise RuntimeError("tnnb200_host_convert failed")
    return half, back, bool(rc)


class PinnedArray:
    """A numpy array over page-locked host memory from the plug-in (tnnb200_host_alloc): Mats that wrap it are copied
    by DMA directly, without a staging copy on the host."""

    def __init__(self, shape, dtype):
        _, self._plugin = load()
        self.nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        self.ptr = self._plugin.tnnb200_host_alloc(max(self.nbytes, 1))
        if not self.ptr:
            raise MemoryError("tnnb200_host_alloc(%d) failed" % self.nbytes)
        buf = (ctypes.c_char * self.nbytes).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=dtype).reshape(shape)

    def free(self):
        if getattr(self, "ptr", None):
            self.array = None
            self._plugin.tnnb200_host_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def run_pipeline(instances, inputs, outputs, warmup, steps):
    """The reference benchmark's loop (ConvertFromMatAsync of every input -> ForwardAsync -> blocking ConvertToMat of
    every output, test/test.cc:125-152) run natively over `instances` taken round-robin (tnnc_run_pipeline).
    inputs / outputs: per instance a list of (blob name, numpy array); the arrays are the host buffers themselves
    (pageable numpy memory or PinnedArray.array).  Returns the wall time of the `steps` timed steps in seconds."""
    shim, _ = load()
    n = len(instances)
    assert len(inputs) == n and len(outputs) == n
    n_in, n_out = len(inputs[0]), len(outputs[0])
    keep = []

    def records(per_inst, width):
        arr = (TnncIo * (n * width))()
        for k, ios in enumerate(per_inst):
            assert len(ios) == width
            for i, (name, a) in enumerate(ios):
                assert a.flags["C_CONTIGUOUS"]
                nm = name.encode()
                keep.append(nm)
                r = arr[k * width + i]
                r.name, r.host, r.n, r.kind = nm, a.ctypes.data, a.size, _KIND_OF[a.dtype]
        return arr

    ins, outs = records(inputs, n_in), records(outputs, n_out)
    hs = (ctypes.c_void_p * n)(*[inst.h for inst in instances])
    ms = shim.tnnc_run_pipeline(hs, n, ins, n_in, outs, n_out, int(warmup), int(steps))
    if ms < 0:
        raise RuntimeError("tnnc_run_pipeline failed (%g): %s" % (
            ms, "; ".join(shim.tnnc_last_error(i.h).decode() for i in instances)))
    return ms / 1e3


SHARE_MEMORY_DEFAULT, SHARE_MEMORY_ONE_THREAD, SHARE_MEMORY_FROM_EXTERNAL = 0, 1, 2


class Instance:
    """TNN::Init + CreateInst on a device; set_input / forward / get_output move fp32 host arrays."""

    def __init__(self, proto_path, model_path, device=DEVICE_CUDA, device_id=0, precision=PRECISION_AUTO, threads=1,
                 share_memory_mode=SHARE_MEMORY_DEFAULT):
        self.shim, _ = load()
        err = ctypes.create_string_buffer(1024)
        self.h = self.shim.tnnc_create_ex(proto_path.encode(), model_path.encode(), device, device_id, precision,
                                          threads, share_memory_mode, err, 1024)
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

    def forward_memory_size(self):
        """Instance::GetForwardMemorySize: bytes of blob memory the instance needs."""
        n = self.shim.tnnc_forward_memory_size(self.h)
        if n < 0:
            raise RuntimeError("GetForwardMemorySize: %s" % self.shim.tnnc_last_error(self.h).decode())
        return int(n)

    def set_forward_memory(self, device_pointer):
        """Instance::SetForwardMemory (share_memory_mode SET_FROM_EXTERNAL): the caller's block on the device."""
        self._check(self.shim.tnnc_set_forward_memory(self.h, ctypes.c_void_p(device_pointer)), "SetForwardMemory")

    def share_command_queue(self, other):
        """Instance::ShareCommandQueue: this instance enqueues on `other`'s command queue from now on."""
        self._check(self.shim.tnnc_share_command_queue(self.h, other.h), "ShareCommandQueue")

    def start_profile(self):
        """Instance::StartProfile (TNN_PROFILE builds only): per-layer timing of the Forwards that follow."""
        if self.shim.tnnc_start_profile(self.h) != 0:
            raise RuntimeError("not a TNN_PROFILE build of the host framework")

    def finish_profile(self):
        """Instance::FinishProfile: the per-layer table as text."""
        buf = ctypes.create_string_buffer(1 << 20)
        n = self.shim.tnnc_finish_profile(self.h, buf, len(buf))
        if n < 0:
            raise RuntimeError("not a TNN_PROFILE build of the host framework")
        return buf.value.decode(errors="replace")

    def reshape(self, shapes):
        """Instance::Reshape with `{input name: dims}`; the shapes must stay within those of the model file."""
        names = (ctypes.c_char_p * len(shapes))(*[k.encode() for k in shapes])
        flat = [int(d) for v in shapes.values() for d in v]
        dims = (ctypes.c_int * len(flat))(*flat)
        nds = (ctypes.c_int * len(shapes))(*[len(v) for v in shapes.values()])
        self._check(self.shim.tnnc_reshape(self.h, len(shapes), names, dims, nds), "Reshape")

    # ---- the caller-driven conversion path (BlobConverter + ForwardAsync, as the reference's benchmark uses them)
    def from_mat_async(self, name, arr):
        """ConvertFromMatAsync of a host array (float32 / float16 / int32; the array itself is the Mat's memory)."""
        assert arr.flags["C_CONTIGUOUS"]
        self._check(self.shim.tnnc_from_mat_async(self.h, name.encode(), arr.ctypes.data, arr.size, _KIND_OF[arr.dtype]),
                    "ConvertFromMatAsync(%s)" % name)

    def forward_async(self):
        self._check(self.shim.tnnc_forward_async(self.h), "ForwardAsync")

    def to_mat(self, name, arr, blocking=True):
        """ConvertToMat (blocking) or ConvertToMatAsync into a host array; with blocking=False the array is complete
        once the instance's command queue has been synchronised (a later blocking conversion does that)."""
        assert arr.flags["C_CONTIGUOUS"] and arr.flags["WRITEABLE"]
        self._check(self.shim.tnnc_to_mat(self.h, name.encode(), arr.ctypes.data, arr.size, _KIND_OF[arr.dtype],
                                          1 if blocking else 0), "ConvertToMat(%s)" % name)

    def command_queue(self):
        return self.shim.tnnc_command_queue(self.h)

    def graph_counters(self):
        """{eager, captures, launches, failures} of the plug-in's CUDA-graph replay for this instance."""
        _, plugin = load()
        out = (ctypes.c_uint64 * 4)()
        if plugin.tnnb200_graph_counters(ctypes.c_void_p(self.command_queue()), out) != 0:
            raise RuntimeError("instance is not served by the tnn_b200 plug-in")
        return dict(zip(("eager", "captures", "launches", "failures"), (int(v) for v in out)))

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
