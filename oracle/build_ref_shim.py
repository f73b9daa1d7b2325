#!/usr/bin/env python3
"""Build oracle/_ref/libtnn_capi.so: the C shim (tnn_b200/tnn_plugin/tnn_capi.cc, public TNN API only) linked against
the reference build in oracle/_ref, through which oracle/tnn_ref.py drives the reference's DEVICE_X86 / DEVICE_NAIVE.

TEST INFRASTRUCTURE ONLY.  Usage: python oracle/build_ref_shim.py [--reference /path/to/TNN]
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from build_ref import OUT, default_reference  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference())
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(a.reference, "include", "tnn")) or not os.path.exists(os.path.join(OUT, "libTNN.so")):
        print("reference headers or oracle/_ref/libTNN.so missing; nothing built")
        return 0
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    src = os.path.join(os.path.dirname(HERE), "tnn_b200", "tnn_plugin", "tnn_capi.cc")
    return subprocess.call([cxx, "-std=gnu++11", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-include", "cstdint",
                            "-I%s/include" % a.reference, "-I%s/source" % a.reference, src, "-o",
                            os.path.join(OUT, "libtnn_capi.so"), "-L" + OUT, "-lTNN", "-ldl", "-Wl,-rpath,$ORIGIN"])


if __name__ == "__main__":
    sys.exit(main())
