#!/usr/bin/env python3
"""Build the reference's own CPU implementation (DEVICE_NAIVE + DEVICE_X86) into oracle/_ref/libTNN.so.

TEST INFRASTRUCTURE ONLY.  The library produced here is the parity checker and the timed CPU baseline; no product
code path computes through it.

The sources are compiled where they lie in the reference checkout (nothing is copied).  The reference's own CMake
project is not run; this script restates its source selection and flags for the CPU + x86 configuration:

* common sources: core, layer, utils, interpreter, optimizer, extern_wrapper, memory_manager (CMakeLists.txt:283-296)
* device/cpu: every .cc (source/tnn/device/cpu/CMakeLists.txt:1-3)
* device/x86: every .cc; the files directly inside acc/, acc/compute/, acc/convolution/, acc/deconvolution/ get
  -mavx -mavx2 -mfma -ffast-math (except acc/x86_unary2_layer_register.cc, which is compiled with the plain
  flags), everything gets -msse4.2 (source/tnn/device/x86/CMakeLists.txt:1-27)
* -std=c++11 -O3 -DNDEBUG -fPIC -fopenmp -pthread -D_GLIBCXX_USE_CXX11_ABI=1 -D_SOURCE_DIR_LEN=<len>
  (CMakeLists.txt:186-223,301-302); symbols are left visible (as the reference's unit-test build does,
  CMakeLists.txt:127-130) so that a device plug-in can link against the host framework.
* `-include cstdint -include algorithm`: gcc 13 no longer pulls these in transitively
  (source/tnn/utils/data_type_utils.cc:61 uses uint64_t, source/tnn/core/profile.cc:146 uses std::sort).

Usage:  python oracle/build_ref.py [--reference /path/to/TNN] [--jobs N] [--profile --out oracle/_ref_profile]
"""
import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def default_reference():
    """The TNN checkout: $TNN_REFERENCE, else a directory named `reference` beside this repository."""
    return os.environ.get("TNN_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def rglob(root, sub):
    return sorted(glob.glob(os.path.join(root, sub, "**", "*.cc"), recursive=True))


def collect(ref):
    src = os.path.join(ref, "source", "tnn")
    common = []
    for d in ("core", "layer", "utils", "interpreter", "optimizer", "extern_wrapper", "memory_manager"):
        common += rglob(src, d)
    cpu = rglob(src, "device/cpu")
    x86_all = rglob(src, "device/x86")
    x86dir = os.path.join(src, "device", "x86")
    acc = []
    for d in ("acc", "acc/compute", "acc/convolution", "acc/deconvolution"):
        acc += sorted(glob.glob(os.path.join(x86dir, d, "*.cc")))
    exclude = os.path.join(x86dir, "acc", "x86_unary2_layer_register.cc")
    acc = [f for f in acc if f != exclude]
    accset = set(acc)
    x86 = [f for f in x86_all if f not in accset]  # includes `exclude`, built without the AVX flags
    return common, cpu, x86, acc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference())
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--profile", action="store_true", help="also define TNN_PROFILE (per-layer host timers)")
    ap.add_argument("--out", default=None, help="output directory (default oracle/_ref; a TNN_PROFILE build changes "
                                                 "class layouts and needs a directory of its own, e.g. oracle/_ref_profile)")
    ap.add_argument("--cxx", default="/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
    args = ap.parse_args()
    global OUT
    if args.out:
        OUT = os.path.abspath(args.out)
    ref = os.path.abspath(args.reference)
    if not os.path.isdir(os.path.join(ref, "source", "tnn")):
        print("reference sources not found at %s; nothing built" % ref)
        return 0 if os.path.exists(os.path.join(OUT, "libTNN.so")) else 1

    common, cpu, x86, acc = collect(ref)
    objdir = os.path.join(OUT, "obj")
    os.makedirs(objdir, exist_ok=True)
    base = ("-std=gnu++11 -O3 -DNDEBUG -fPIC -fopenmp -pthread -D_GLIBCXX_USE_CXX11_ABI=1 "
            "-D_SOURCE_DIR_LEN=%d -include cstdint -include algorithm -w "
            "-I%s/include -I%s/source -I%s/third_party/xbyak" % (len(ref), ref, ref, ref))
    if args.profile:
        base += " -DTNN_PROFILE"
    lines = [
        "cxx = %s" % args.cxx,
        "base = %s" % base,
        "rule cc",
        "  command = $cxx $base $extra -MMD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = CXX $in",
        "rule link",
        "  command = $cxx -shared -fopenmp -pthread -o $out @$out.rsp -ldl -lrt",
        "  rspfile = $out.rsp",
        "  rspfile_content = $in",
        "  description = LINK $out",
        "",
    ]
    objs = []

    def add(files, extra):
        for f in files:
            rel = os.path.relpath(f, ref).replace("/", "_").replace(" ", "_")
            o = os.path.join(objdir, rel[:-3] + ".o")
            objs.append(o)
            # one reference file name contains a space; ninja wants "$ " and the shell wants quotes
            lines.append("build %s: cc %s" % (o, f.replace(" ", "$ ")))
            if extra:
                lines.append("  extra = %s" % extra)

    add(common, "")
    add(cpu, "")
    add(x86, "-msse4.2")
    add(acc, "-msse4.2 -mavx -ffast-math -mavx2 -mfma")
    lib = os.path.join(OUT, "libTNN.so")
    lines.append("build %s: link %s" % (lib, " ".join(objs)))
    lines.append("default %s" % lib)
    ninja_file = os.path.join(OUT, "build.ninja")
    with open(ninja_file, "w") as fh:
        fh.write("\n".join(lines) + "\n")
    # -C: ninja keeps its own state files (.ninja_log, .ninja_deps) in the directory it runs in
    return subprocess.call(["ninja", "-C", OUT, "-f", ninja_file, "-j", str(args.jobs)])


if __name__ == "__main__":
    sys.exit(main())
