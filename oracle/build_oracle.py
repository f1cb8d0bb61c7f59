"""Build recipe for the two CPU checkers (TEST INFRASTRUCTURE ONLY).

1. ``oracle/libmcn_oracle.so`` -- the plain-C restatement ``mcn_oracle.c``.
   Always buildable (needs only gcc).
2. ``oracle/_ref/libmcn_ref.so`` -- the reference's own CPU backend, compiled
   from its sources where they lie (never copied): ``matlab/src/bits/*.cpp``
   plus ``impl/im2row_cpu.cpp`` and ``impl/copy_cpu.cpp``, together with
   ``ref_capi.cpp`` (C entry points) and ``ref_blas.cpp`` (the BLAS the
   reference expects from MATLAB).  Built only where the reference checkout
   is present; elsewhere the prebuilt file is used as it is.

Flags: ``-O2 -DENABLE_DOUBLE -DNDEBUG -ffp-contract=off`` and no
``-ffast-math`` (the reference Makefile:130 passes it; leaving it out keeps
the arithmetic plain IEEE and reproducible).  ``nnpooling.cpp`` needs
``-include limits`` because nnpooling.cu:38 uses std::numeric_limits without
including the header.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: MCN_REFERENCE_ROOT, else a directory "reference" beside this repository
REF_ROOT = os.environ.get("MCN_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
REF_BITS = os.path.join(REF_ROOT, "matlab", "src", "bits")
REF_OUT = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_OUT, "libmcn_ref.so")
ORACLE_SO = os.path.join(HERE, "libmcn_oracle.so")

REF_SOURCES = [
    "data.cpp", "nnconv.cpp", "nnbias.cpp", "nnfullyconnected.cpp", "nnsubsample.cpp",
    "nnpooling.cpp", "nnbnorm.cpp", "nnbilinearsampler.cpp", "nnroipooling.cpp", "nnnormalize.cpp",
    "impl/im2row_cpu.cpp", "impl/copy_cpu.cpp",
]
CXXFLAGS = ["-std=c++11", "-O2", "-fPIC", "-DENABLE_DOUBLE", "-DNDEBUG", "-ffp-contract=off", "-w"]


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.exists(s) and os.path.getmtime(s) <= t for s in sources)


def build_restatement(force=False):
    srcs = [os.path.join(HERE, "mcn_oracle.c"), os.path.join(HERE, "mcn_oracle_impl.h")]
    if not force and _newer(ORACLE_SO, srcs):
        return ORACLE_SO
    cmd = ["gcc", "-std=c99", "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-o", ORACLE_SO, srcs[0], "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def reference_available():
    return os.path.isfile(os.path.join(REF_BITS, "nnconv.cpp"))


def build_reference(force=False):
    """Compile the reference CPU backend; returns the .so path or None when the
    reference checkout is absent and no prebuilt library exists."""
    if not reference_available():
        return REF_SO if os.path.exists(REF_SO) else None
    own = [os.path.join(HERE, "ref_capi.cpp"), os.path.join(HERE, "ref_blas.cpp"),
           os.path.join(HERE, "ref_shim", "blas.h")]
    if not force and _newer(REF_SO, own + [os.path.abspath(__file__)]):
        return REF_SO
    os.makedirs(REF_OUT, exist_ok=True)
    inc = ["-I", os.path.join(HERE, "ref_shim"), "-I", REF_BITS]
    objs = []
    for s in REF_SOURCES:
        o = os.path.join(REF_OUT, s.replace("/", "_").replace(".cpp", ".o"))
        extra = ["-include", "limits"] if s == "nnpooling.cpp" else []
        subprocess.check_call(["g++"] + CXXFLAGS + extra + inc + ["-c", os.path.join(REF_BITS, s), "-o", o])
        objs.append(o)
    for s in ("ref_capi.cpp", "ref_blas.cpp"):
        o = os.path.join(REF_OUT, s.replace(".cpp", ".o"))
        subprocess.check_call(["g++"] + CXXFLAGS + inc + ["-c", os.path.join(HERE, s), "-o", o])
        objs.append(o)
    subprocess.check_call(["g++", "-shared", "-o", REF_SO] + objs + ["-ldl"])
    return REF_SO


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_restatement(force))
    print(build_reference(force))
