"""The header-only C++ mirror of the reference's operator classes (include/vlb/*.hpp): it compiles
and links against libvlb.so with a plain host compiler (no GPU needed), and on a B200 the compiled
program drives every operator through vl::nn::* objects on vl::Tensor views and checks the results
against the CPU checker."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "test_classes")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build_program():
    from matconvnet_b200 import build
    lib = build.build()
    libdir = os.path.dirname(lib)
    src = os.path.join(ROOT, "tests", "cpp", "test_classes.cpp")
    if not os.path.exists(EXE) or os.path.getmtime(EXE) < max(os.path.getmtime(src), os.path.getmtime(lib)):
        cmd = ["g++", "-std=c++11", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
               src, "-o", EXE, "-L", libdir, "-lvlb", "-L", os.path.join(CUDA, "lib64"), "-lcudart", "-ldl",
               "-Wl,-rpath," + libdir, "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
        subprocess.check_call(cmd)
    return EXE


def test_headers_compile_and_link():
    assert os.path.exists(build_program())


@pytest.mark.gpu
def test_operator_classes_on_gpu():
    import sys
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as O
    O.restatement()
    exe = build_program()
    p = subprocess.run([exe, os.path.join(ROOT, "oracle", "libmcn_oracle.so")], capture_output=True, text=True, timeout=300)
    print(p.stdout, p.stderr)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "all checks passed" in p.stdout
