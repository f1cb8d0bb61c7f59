"""Builds the MEX gateway test double (TEST INFRASTRUCTURE ONLY).

The reference's MEX gateways (matlab/src/vl_nnconv.cu, vl_nnbnorm.cu, vl_nnpool.cu, vl_nnroipool.cu,
vl_nnbilinearsampler.cu) and its data layer (matlab/src/bits/data.cu, datacu.cu, datamex.cu, impl/copy_*.c*) are
compiled UNMODIFIED, from where they lie in the reference checkout, against

  * include/ here: a stand-in for MATLAB's mex.h / matrix.h / gpu/mxGPUArray.h (mxdouble.cpp implements it), and
  * vlb_functors.cpp: the reference's operator classes (its own bits/nn*.hpp declarations) defined over the vlb C ABI,
    in place of the reference's bits/nn*.cu.

Result, in _build/ (kept out of the history, shipped with the tree like every other built library):
libmexdouble.so (stand-in + data layer + operator classes, linked to libvlb.so) and one vl_nn*.so per gateway, each
exporting mexFunction.  Nothing of the reference is copied: without the checkout nothing is built and the prebuilt
libraries are used as they are.
"""
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build")
GATEWAYS = ["vl_nnconv", "vl_nnbnorm", "vl_nnpool", "vl_nnroipool", "vl_nnbilinearsampler"]
DATA_LAYER = ["bits/datamex.cu", "bits/data.cu", "bits/datacu.cu", "bits/impl/copy_gpu.cu", "bits/impl/copy_cpu.cpp"]
OWN = ["mxdouble.cpp", "vlb_functors.cpp"]


def reference_src():
    root = os.environ.get("MCN_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
    src = os.path.join(root, "matlab", "src")
    return src if os.path.exists(os.path.join(src, "vl_nnconv.cu")) else None


def _nvcc():
    cand = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _run(cmd):
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError("build of the MEX test double failed:\n%s\n%s\n%s" % (" ".join(cmd), p.stdout, p.stderr))


def _newer(target, deps):
    return os.path.exists(target) and all(os.path.getmtime(target) >= os.path.getmtime(d) for d in deps)


def libraries():
    """Paths of the built libraries, or None when they are not there."""
    paths = [os.path.join(OUT, "libmexdouble.so")] + [os.path.join(OUT, g + ".so") for g in GATEWAYS]
    return paths if all(os.path.exists(p) for p in paths) else None


def build():
    """Compiles everything where the reference checkout exists; returns libraries()."""
    src = reference_src()
    if src is None:
        return libraries()
    from matconvnet_b200 import build as engine
    libvlb = engine.build()
    os.makedirs(OUT, exist_ok=True)
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++14", "-Xcompiler", "-fPIC", "-w",
             "-DENABLE_GPU", "-I", os.path.join(HERE, "include"), "-I", src, "-I", os.path.join(ROOT, "include"),
             # the reference's BLAS helper header wants MATLAB's blas.h; the checker's stand-in declares the same routines
             "-I", os.path.join(ROOT, "oracle", "ref_shim")]
    headers = [os.path.join(dp, f) for dp, _, fs in os.walk(os.path.join(HERE, "include")) for f in fs]
    headers.append(os.path.join(ROOT, "include", "vlb.h"))

    def compile_one(job):
        path, obj = job
        if not _newer(obj, [path] + headers):
            _run([_nvcc()] + flags + ["-c", path, "-o", obj])
        return obj

    jobs = [(os.path.join(src, f), os.path.join(OUT, "ref_" + os.path.basename(f).split(".")[0] + ".o")) for f in DATA_LAYER]
    jobs += [(os.path.join(HERE, f), os.path.join(OUT, f.split(".")[0] + ".o")) for f in OWN]
    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, jobs))
    common = os.path.join(OUT, "libmexdouble.so")
    if not _newer(common, objs + [libvlb]):
        _run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", common] + objs +
             ["-L", os.path.dirname(libvlb), "-lvlb", "-lcublas", "-lcudart", "-Xlinker", "--no-undefined",
              "-Xlinker", "-rpath=$ORIGIN/../../../matconvnet_b200"])

    def gateway(name):
        out = os.path.join(OUT, name + ".so")
        path = os.path.join(src, name + ".cu")
        if not _newer(out, [path, common] + headers):
            _run([_nvcc()] + flags + ["-shared", path, "-o", out, "-L", OUT, "-lmexdouble", "-lcudart", "-Xlinker", "--no-undefined",
                                      "-Xlinker", "-rpath=$ORIGIN"])
        return out

    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(gateway, GATEWAYS))
    return libraries()


if __name__ == "__main__":
    import sys
    sys.path.insert(0, ROOT)
    print("\n".join(build() or ["reference checkout not found and no prebuilt libraries"]))
