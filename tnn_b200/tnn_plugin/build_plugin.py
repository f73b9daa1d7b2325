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
    return 0


if __name__ == "__main__":
    sys.exit(main())
