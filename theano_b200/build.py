"""Build ``libb200conv.so`` in-tree with nvcc for sm_100a.

    python -m theano_b200.build [--force] [--verbose] [--debug]

``--debug`` builds ``libb200conv_debug.so`` instead: the same sources with ``-DB200CONV_DEBUG``,
in which every global store, tiled TMA store and gradient-slab index of the tensor-core kernels
is range-checked (a violation is recorded in the status word and the access skipped).  Select it
at run time with ``B200CONV_LIB=<path>``.

The library is plain CUDA C++ behind a C ABI (``include/b200conv.h``); it links
only the CUDA runtime.  NCCL and the driver entry point for tensor maps are
looked up at run time, so the build needs no GPU and no extra libraries.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200conv.so")
DEBUG_LIB = os.path.join(HERE, "libb200conv_debug.so")
SOURCES = ["api.cu", "conv_umma.cu", "conv_slab.cu", "wgrad_umma.cu", "wgrad_group.cu", "conv_direct.cu", "layout.cu", "selftest.cu", "elementwise.cu", "gemm_pair.cu", "wgrad_pair.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(lib):
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "b200conv.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, debug=False):
    """Compile every CUDA source and link the shared library; returns its path."""
    lib = DEBUG_LIB if debug else LIB
    if not force and not _stale(lib):
        return lib
    objdir = os.path.join(HERE, "build", "debug" if debug else "release")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    flags = NVCC_FLAGS + (["-DB200CONV_DEBUG"] if debug else [])
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            print(" ".join(cmd))
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    objs = []
    for src, obj, p in procs:
        out = p.communicate()[0].decode()
        if p.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s" % (src, out))
        if verbose and out.strip():
            print(out)
        objs.append(obj)
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib] + objs + ["-ldl"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, debug="--debug" in sys.argv))
