"""Build the CPU oracle shared libraries (test infrastructure).

``python oracle/build_oracle.py`` compiles ``corr_oracle.c`` twice with gcc:
``_build/liboracle_f32.so`` (REAL=float, the CorrMM float32 path) and
``_build/liboracle_f64.so`` (REAL=double, used as a high-precision yardstick).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")


def lib_path(real):
    return os.path.join(OUT, "liboracle_%s.so" % ("f32" if real == "float" else "f64"))


def build(force=False, verbose=False):
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(HERE, "corr_oracle.c")
    for real in ("float", "double"):
        dst = lib_path(real)
        if not force and os.path.exists(dst) and os.path.getmtime(dst) >= os.path.getmtime(src):
            continue
        cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-std=c99",
               "-DREAL=" + real, src, "-o", dst, "-lm"]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
