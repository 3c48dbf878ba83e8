"""Build the C++ layer: lib/libmlxr_primitives.so (MLXR's Primitive classes and free functions
and the graph layers RMSNorm / Linear / RotaryEmbedding / MLP over the C ABI, compiled against
the MLX stand-in in cpp/mlx) and its test program
lib/primitives_test.  Plain g++; the CUDA runtime is needed for managed memory and streams.

    python -m mlxr_b200.build_cpp
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CPP = os.path.join(HERE, "cpp")
OUT = os.path.join(HERE, "lib")
LIB = os.path.join(OUT, "libmlxr_primitives.so")
TEST = os.path.join(OUT, "primitives_test")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wno-unused-function", f"-I{CPP}", f"-I{CUDA}/include"]


def _run(cmd):
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + p.stdout + p.stderr)
        raise RuntimeError("C++ build failed")
    return p.stdout + p.stderr


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _tree(root):
    out = []
    for d, _, fs in os.walk(root):
        out += [os.path.join(d, f) for f in fs if f.endswith((".h", ".cpp"))]
    return out


def build(force: bool = False):
    from . import build as cuda_build
    core = cuda_build.build()
    os.makedirs(OUT, exist_ok=True)
    srcs = [os.path.join(CPP, "mlx_shim.cpp"), os.path.join(CPP, "primitives", "mlxr_kernels.cpp"),
            os.path.join(CPP, "graph", "layers.cpp")]
    deps = _tree(CPP) + [os.path.join(os.path.dirname(HERE), "include", "mlxr_b200.h"), core]
    link = [f"-L{OUT}", "-lmlxr_b200", f"-L{CUDA}/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{CUDA}/lib64"]
    if force or _newer(LIB, deps):
        _run(["g++", *FLAGS, "-shared", "-o", LIB, *srcs, *link])
    test_src = os.path.join(CPP, "tests", "primitives_test.cpp")
    if force or _newer(TEST, deps + [test_src, LIB]):
        _run(["g++", *FLAGS, f"-I{os.path.join(CPP, 'primitives')}", "-o", TEST, test_src, "-lmlxr_primitives", *link])
    return LIB, TEST


if __name__ == "__main__":
    print(*build("--force" in sys.argv), sep="\n")
