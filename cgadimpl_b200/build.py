"""Compiles the CUDA library for sm_100a with nvcc (cross-compiles without a GPU).

    python -m cgadimpl_b200.build [--force] [--verbose]

Output: cgadimpl_b200/libagb_cuda.so and, next to it, libagb_cuda.ptxas.log with ptxas' resource usage
of every kernel (registers, spills, shared memory); both in-tree and git-ignored.
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libagb_cuda.so")
PTXAS_LOG = os.path.join(PKG, "libagb_cuda.ptxas.log")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # No implicit multiply-add contraction: the kernels keep the reference's rounding points.  (This does
    # not cover the packed __fmul2_rn -> __fadd2_rn pair; see the caution in rmsnorm_staged.cuh.)
    "--fmad=false",
    "--shared", "-Xcompiler", "-fPIC",
]


def _nvcc():
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _sources():
    out = []
    for d in (CSRC, os.path.join(ROOT, "include", "agb")):
        for f in sorted(os.listdir(d)):
            if f.endswith((".cu", ".cuh", ".h")):
                out.append(os.path.join(d, f))
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = _sources()
    if not force and os.path.exists(LIB) and os.path.exists(PTXAS_LOG) and \
            all(os.path.getmtime(LIB) >= os.path.getmtime(s) for s in srcs):
        return LIB
    tmp = LIB + ".new"     # written beside the target and renamed: a reader never sees a half-written library
    cmd = [_nvcc()] + NVCC_FLAGS + ["-Xptxas", "-v", "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-o", tmp,
                                    os.path.join(CSRC, "agb_cuda.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(r.stderr)
    if r.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    os.replace(tmp, LIB)
    with open(PTXAS_LOG, "w") as f:
        f.write(r.stderr)
    return LIB


def kernel_resources():
    """{mangled kernel name: {"registers": n, "spill_stores": bytes, "spill_loads": bytes}} from the last build."""
    import re

    build()
    out, name = {}, None
    for line in open(PTXAS_LOG):
        m = re.search(r"Compiling entry function '(\S+)'", line)
        if m:
            name = m.group(1)
            out[name] = {}
            continue
        if name is None:
            continue
        m = re.search(r"(\d+) bytes spill stores, (\d+) bytes spill loads", line)
        if m:
            out[name]["spill_stores"], out[name]["spill_loads"] = int(m.group(1)), int(m.group(2))
        m = re.search(r"Used (\d+) registers", line)
        if m:
            out[name]["registers"] = int(m.group(1))
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
