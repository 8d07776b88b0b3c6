"""Builds oracle/_ref/libcgadimpl_ref.so: the REFERENCE's own sources for the RMSNorm path, compiled
from where they lie in the reference checkout (nothing is copied; location: $CGADIMPL_REFERENCE), over the CPU stand-in for its absent
tensor library in oracle/ref_shim/.  Test infrastructure; needs the reference tree, so it runs in
the development container only -- the built library travels with the repository snapshot.

    python oracle/build_ref.py [--force]

Reference files compiled, unmodified:
    cgadimpl/src/core/{graph,schema,autodiff}.cpp
    cgadimpl/src/ops/{normalization,arithmetic,reduction}.cpp
    cgadimpl/src/autodiff/{autodiff_vjp_ops,autodiff_jvp_ops}.cpp
    cgadimpl/src/optimizer/optim.cpp
The reference's own build (CMake + OwnTensor + MLIR + Nova) is not used and cannot run here.
autodiff.cpp is compiled without -fopenmp: it carries a stray `#pragma omp parallel for` in front of
a function definition (src/core/autodiff.cpp:32), which is an error once OpenMP is enabled.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# The reference checkout's cgadimpl/ directory: $CGADIMPL_REFERENCE, else a checkout named "reference" beside
# this repository; neither = not available (the prebuilt library, if any, is used as it is).
REF = os.environ.get("CGADIMPL_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference", "cgadimpl")
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libcgadimpl_ref.so")
SHIM = os.path.join(HERE, "ref_shim")
CUDA_INC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"

REF_SOURCES = [
    ("src/core/graph.cpp", True), ("src/core/schema.cpp", True), ("src/core/autodiff.cpp", False),
    ("src/ops/normalization.cpp", True), ("src/ops/arithmetic.cpp", True), ("src/ops/reduction.cpp", True),
    ("src/autodiff/autodiff_vjp_ops.cpp", True), ("src/autodiff/autodiff_jvp_ops.cpp", True),
    ("src/optimizer/optim.cpp", True),
]
SHIM_SOURCES = ["owntensor_shim.cpp", "ref_driver.cpp"]
FLAGS = ["-std=c++20", "-O2", "-ffp-contract=off", "-fPIC", "-w", "-pthread"]
INCLUDES = ["-I", SHIM, "-I", os.path.join(REF, "include"), "-I", CUDA_INC]


def available() -> bool:
    return bool(REF) and os.path.isdir(os.path.join(REF, "src"))


def build(force: bool = False) -> str:
    if not available():
        if os.path.exists(OUT):
            return OUT
        raise RuntimeError(f"reference tree not found at {REF}")
    srcs = [os.path.join(REF, s) for s, _ in REF_SOURCES] + [os.path.join(SHIM, s) for s in SHIM_SOURCES]
    deps = srcs + [os.path.join(SHIM, "TensorLib.h"), os.path.abspath(__file__)]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps):
        return OUT
    obj_dir = os.path.join(OUT_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    objs = []
    jobs = [(os.path.join(REF, s), omp) for s, omp in REF_SOURCES] + [(os.path.join(SHIM, s), True) for s in SHIM_SOURCES]
    for src, omp in jobs:
        obj = os.path.join(obj_dir, os.path.basename(src)[:-4] + ".o")
        cmd = [CXX] + FLAGS + (["-fopenmp"] if omp else []) + INCLUDES + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("compile failed:\n" + " ".join(cmd) + "\n" + r.stderr[-4000:])
        objs.append(obj)
    cmd = [CXX, "-shared", "-fopenmp", "-o", OUT] + objs + ["-Wl,--no-undefined", "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + " ".join(cmd) + "\n" + r.stderr[-6000:])
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
