"""Build recipe: compiles the CUDA sources under csrc/ for sm_100a with nvcc and links
them in-tree into lib/libmlxr_b200.so (the C ABI of include/mlxr_b200.h).

    python -m mlxr_b200.build            # build what is out of date
    python -m mlxr_b200.build --force    # rebuild everything
    python -m mlxr_b200.build --verbose  # keep ptxas -v resource usage in lib/build.log

nvcc cross-compiles without a GPU.  No CMake: one nvcc call per .cu file (in parallel) and
one link.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "lib")
OBJ = os.path.join(OUT, "obj")
LIB = os.path.join(OUT, "libmlxr_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
    "-Xptxas", "-v",
    "-I", os.path.join(ROOT, "include"),
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build mlxr_b200")
    return exe


def _deps_mtime() -> float:
    """Newest mtime over headers every object depends on."""
    t = 0.0
    for d in (CSRC, os.path.join(ROOT, "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh", ".inc")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    # MLXR_TUNING=1 in the environment keeps the tuning probes (environment overrides read by the
    # launchers); the default build has none.  A change of flags rebuilds everything.
    flags = list(NVCC_FLAGS) + (["-DMLXR_TUNING"] if os.environ.get("MLXR_TUNING") == "1" else [])
    stamp = os.path.join(OBJ, "flags.txt")
    old = open(stamp).read() if os.path.exists(stamp) else None
    if old != " ".join(flags):
        force = True
        with open(stamp, "w") as f:
            f.write(" ".join(flags))
    hdr_t = _deps_mtime()
    jobs = []
    objs = []
    for src in sources():
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_t):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [nvcc, *flags, "-c", s, "-o", o]
        p = subprocess.run(cmd, capture_output=True, text=True)
        return s, p.returncode, p.stdout + p.stderr

    log_lines = []
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for s, rc, out in ex.map(compile_one, jobs):
                log_lines.append(f"==== {os.path.basename(s)}\n{out}")
                if rc != 0:
                    sys.stderr.write(out)
                    raise RuntimeError(f"nvcc failed on {s}")
                warn = [ln for ln in out.splitlines() if "warning" in ln.lower() or "spill" in ln and " 0 bytes spill" not in ln]
                if verbose:
                    print(out)
                elif warn:
                    print(f"[{os.path.basename(s)}]", *warn[:20], sep="\n  ")
        with open(os.path.join(OUT, "build.log"), "a" if not force else "w") as f:
            f.write("\n".join(log_lines) + "\n")
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xlinker", "--no-undefined", "-ldl"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
