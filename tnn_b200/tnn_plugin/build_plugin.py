"""Build the pieces that compile against TNN's headers: the DEVICE_CUDA plug-in and the C shim over TNN's public API
(tnn_capi.cc).  Needs a TNN checkout (headers) and a host framework library, libTNN.so, built from the unmodified TNN
sources.

    python tnn_b200/tnn_plugin/build_plugin.py [--reference /path/to/TNN] [--libtnn /path/to/libTNN.so]

Products:
    tnn_b200/lib/libtnn_b200_plugin.so   the plug-in (device, context, blob converter, fused layers, accs, graph pass)
    tnn_b200/host/libTNN.so              the host framework the plug-in is loaded into (a copy of --libtnn)
    tnn_b200/host/libtnn_capi.so         the C shim the Python harness drives TNN through

With --profile the same three are built with -DTNN_PROFILE against a host framework built the same way
(oracle/build_ref.py --profile --out oracle/_ref_profile) into tnn_b200/lib_profile/ and tnn_b200/host_profile/:
TNN_PROFILE adds members to TNN's classes, so a profiling plug-in and a plain host (or the reverse) do not mix.
"""
import argparse
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
HOST = os.path.join(ROOT, "tnn_b200", "host")


def default_reference():
    """The TNN checkout: $TNN_REFERENCE, else a directory named `reference` beside this repository."""
    return os.environ.get("TNN_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference())
    ap.add_argument("--libtnn", default=os.environ.get("TNN_B200_LIBTNN_SRC",
                                                       os.path.join(ROOT, "oracle", "_ref", "libTNN.so")),
                    help="a libTNN.so built from the unmodified TNN sources with visible symbols "
                         "(the test tree's oracle/build_ref.py produces one)")
    ap.add_argument("--profile", action="store_true", help="build the TNN_PROFILE variant (see above)")
    a = ap.parse_args()
    global HOST
    suffix = "_profile" if a.profile else ""
    if a.profile:
        HOST = os.path.join(ROOT, "tnn_b200", "host_profile")
        if a.libtnn == os.path.join(ROOT, "oracle", "_ref", "libTNN.so"):
            a.libtnn = os.path.join(ROOT, "oracle", "_ref_profile", "libTNN.so")
    ref = a.reference
    if not os.path.isdir(os.path.join(ref, "include", "tnn")):
        print("TNN headers not found at %s; nothing built" % ref)
        return 0
    if not os.path.exists(a.libtnn):
        print("host framework %s not found; nothing built" % a.libtnn)
        return 0
    os.makedirs(HOST, exist_ok=True)
    host_lib = os.path.join(HOST, "libTNN.so")
    if not os.path.exists(host_lib) or os.path.getmtime(host_lib) < os.path.getmtime(a.libtnn):
        shutil.copy2(a.libtnn, host_lib)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    common = [cxx, "-std=gnu++11", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-fopenmp", "-include", "cstdint",
              "-I%s/include" % ref, "-I%s/source" % ref] + (["-DTNN_PROFILE=1"] if a.profile else [])
    subprocess.check_call(common + [os.path.join(HERE, "tnn_capi.cc"), "-o", os.path.join(HOST, "libtnn_capi.so"),
                                    "-L" + HOST, "-lTNN", "-ldl", "-Wl,-rpath,$ORIGIN"])

    # The DEVICE_CUDA plug-in.  Loaded into a process next to libTNN.so (dlopen / LD_PRELOAD / link), its static
    # constructors register everything.
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    libdir = os.path.join(ROOT, "tnn_b200", "lib")
    srcs = sorted(glob.glob(os.path.join(HERE, "b200_*.cc")))
    outdir = os.path.join(ROOT, "tnn_b200", "lib" + suffix)
    os.makedirs(outdir, exist_ok=True)
    out = os.path.join(outdir, "libtnn_b200_plugin.so")
    cmd = (common + ["-I%s/include" % cuda, "-I%s/include" % ROOT, "-I%s/third_party/xbyak" % ref] + srcs +
           ["-o", out, "-L" + libdir, "-ltnn_b200", "-L" + HOST, "-lTNN",
            "-L%s/lib64" % cuda, "-lcudart_static", "-ldl", "-lrt", "-lpthread", "-fopenmp",
            "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../lib", "-Wl,-rpath,$ORIGIN/../host" + suffix])
    subprocess.check_call(cmd)
    return 0


if __name__ == "__main__":
    sys.exit(main())
