"""Build recipe for the CPU checker (test infrastructure, never part of the shipped library).

    python oracle/build_oracle.py        ->  oracle/liboracle.so

-ffp-contract=off keeps every fp32 rounding point where agb_oracle.c puts it.  OpenMP is
used when the compiler has it (some gcc installs lack libgomp); the arithmetic does not
depend on the thread count except where agb_oracle.c says so.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "agb_oracle.c")
OUT = os.path.join(HERE, "liboracle.so")
BASE = ["-O2", "-ffp-contract=off", "-fPIC", "-shared", "-std=c11", "-Wall", "-Wextra"]


def _candidates():
    seen = []
    for c in ("/usr/bin/gcc", shutil.which("gcc"), shutil.which("cc"), os.environ.get("CC")):
        if c and os.path.exists(c) and c not in seen:
            seen.append(c)
    return seen


def build(force: bool = False) -> str:
    deps = [SRC, os.path.join(HERE, "agb_oracle.h"), os.path.abspath(__file__)]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps):
        return OUT
    errors = []
    for omp in (["-fopenmp"], []):
        for cc in _candidates():
            cmd = [cc] + BASE + omp + ["-o", OUT, SRC, "-lm"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode == 0:
                return OUT
            errors.append(" ".join(cmd) + "\n" + r.stderr)
    raise RuntimeError("could not build liboracle.so:\n" + "\n".join(errors))


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
