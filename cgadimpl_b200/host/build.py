"""Builds the C++ host layer (the `ag::` graph API over libagb_cuda.so) and its test programs.

    python -m cgadimpl_b200.host.build [--force]

Outputs (git-ignored): cgadimpl_b200/host/libagb_host.so and cgadimpl_b200/host/build/<test programs>.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
LIB = os.path.join(HERE, "libagb_host.so")
BIN = os.path.join(HERE, "build")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")

CXXFLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter", "-pthread"]
INCLUDES = ["-I", os.path.join(HERE, "include"), "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "oracle"),
            "-I", os.path.join(CUDA, "include")]


def _cxx():
    for c in ("/usr/bin/g++", shutil.which("g++"), os.environ.get("CXX")):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("no C++ compiler found")


def _newer(target, deps):
    return os.path.exists(target) and all(os.path.getmtime(target) >= os.path.getmtime(d) for d in deps)


def _all_headers():
    out = []
    for base in (os.path.join(HERE, "include"), os.path.join(ROOT, "include")):
        for d, _, files in os.walk(base):
            out += [os.path.join(d, f) for f in files]
    return out


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build(force: bool = False) -> str:
    from cgadimpl_b200 import build as cuda_build

    cuda_lib = cuda_build.build()
    srcs = sorted(os.path.join(HERE, "src", f) for f in os.listdir(os.path.join(HERE, "src")) if f.endswith(".cpp"))
    deps = srcs + _all_headers() + [cuda_lib, os.path.abspath(__file__)]
    link = ["-L", PKG, "-lagb_cuda", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
            "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    if force or not _newer(LIB, deps):
        _run([_cxx()] + CXXFLAGS + INCLUDES + ["-shared", "-o", LIB + ".new"] + srcs + link)
        os.replace(LIB + ".new", LIB)   # renamed into place: a reader never sees a half-written library
    os.makedirs(BIN, exist_ok=True)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import build_oracle

    oracle = build_oracle.build()
    tdir = os.path.join(HERE, "tests")
    for f in sorted(os.listdir(tdir)):
        if not f.endswith(".cpp"):
            continue
        exe = os.path.join(BIN, f[:-4])
        src = os.path.join(tdir, f)
        if force or not _newer(exe, [src, LIB, oracle] + _all_headers()):
            # the timing programs (bench_*.cpp) are product-side: they neither include nor link the CPU checker
            checker = [] if f.startswith("bench_") else ["-L", os.path.dirname(oracle), "-l:liboracle.so",
                                                         "-Wl,-rpath," + os.path.dirname(oracle)]
            _run([_cxx()] + CXXFLAGS + INCLUDES + ["-o", exe + ".new", src, "-L", HERE, "-lagb_host"] + checker + link +
                 ["-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath,$ORIGIN/../.."])
            os.replace(exe + ".new", exe)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
