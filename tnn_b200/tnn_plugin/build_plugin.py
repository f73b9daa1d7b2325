"""Build the pieces that compile against TNN's headers: the C shim over TNN's public API (tnn_capi.cc) and, once
present, the DEVICE_CUDA plug-in.  Needs the reference checkout (headers) and oracle/_ref/libTNN.so (host framework).

    python tnn_b200/tnn_plugin/build_plugin.py [--reference /path/to/TNN]
"""
import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF_OUT = os.path.join(ROOT, "oracle", "_ref")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TNN_REFERENCE", "/root/reference"))
    a = ap.parse_args()
    ref = a.reference
    if not os.path.isdir(os.path.join(ref, "include", "tnn")):
        print("TNN headers not found at %s; nothing built" % ref)
        return 0
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    common = [cxx, "-std=gnu++11", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-include", "cstdint",
              "-I%s/include" % ref, "-I%s/source" % ref]
    link = ["-L" + REF_OUT, "-lTNN", "-Wl,-rpath,$ORIGIN"]
    subprocess.check_call(common + [os.path.join(HERE, "tnn_capi.cc"), "-o", os.path.join(REF_OUT, "libtnn_capi.so")]
                          + link)

    # The DEVICE_CUDA plug-in: device, context, blob converter, fused layers, accs and the graph pass.  Loaded into
    # a process next to libTNN.so (dlopen / LD_PRELOAD / link), its static constructors register everything.
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    libdir = os.path.join(ROOT, "tnn_b200", "lib")
    srcs = sorted(glob.glob(os.path.join(HERE, "b200_*.cc")))
    out = os.path.join(libdir, "libtnn_b200_plugin.so")
    cmd = (common + ["-I%s/include" % cuda, "-I%s/include" % ROOT, "-I%s/third_party/xbyak" % ref] + srcs +
           ["-o", out, "-L" + libdir, "-ltnn_b200", "-L" + REF_OUT, "-lTNN",
            "-L%s/lib64" % cuda, "-lcudart_static", "-ldl", "-lrt", "-lpthread",
            "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../../oracle/_ref"])
    subprocess.check_call(cmd)
    return 0


if __name__ == "__main__":
    sys.exit(main())
