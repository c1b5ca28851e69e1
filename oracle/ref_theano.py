"""Import the unmodified reference Theano from its source tree (checker glue only: used by the
tests, the golden-vector generators and the reference arm of bench.py, never by the product).

The reference predates numpy 2 / Python 3.12.  This module patches a few
removed names *at run time* (no reference file is edited), sets the flags the
C code generator needs and then imports ``theano``.  It is used to generate the
golden fixtures and by the CPU-side tests of the Theano ops; it is skipped when
the reference tree is absent.
"""
import configparser
import os
import sys
import tempfile
import types

import numpy as np

# the reference's source tree (a directory "reference" beside the repository), else an installed
# copy that travels with the repository (``pip install --target baseline/_ref <reference>``; not
# under version control)
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SOURCE = os.path.join(os.path.dirname(_REPO), "reference")
_INSTALLED = os.path.join(_REPO, "baseline", "_ref")
REF_ROOT = os.environ.get("THEANO_REF_ROOT") or (
    _SOURCE if os.path.isdir(os.path.join(_SOURCE, "theano")) else _INSTALLED)


def available():
    return os.path.isdir(os.path.join(REF_ROOT, "theano"))


def _find_openblas():
    import glob
    for sp in sys.path:
        hits = glob.glob(os.path.join(sp, "opencv_python_headless.libs", "libopenblasp-*.so"))
        if hits:
            return hits[0]
    return None


def import_theano(openmp=True):
    """Return the reference ``theano`` module (imports it on first call)."""
    if "theano" in sys.modules:
        return sys.modules["theano"]
    if not available():
        raise ImportError("reference tree not found at %s" % REF_ROOT)

    nd = types.ModuleType("numpy.distutils")
    mu = types.ModuleType("numpy.distutils.misc_util")
    mu.get_numpy_include_dirs = lambda: [np.get_include()]
    si = types.ModuleType("numpy.distutils.system_info")

    class _SystemInfo(object):
        verbosity = 0

    si.system_info = _SystemInfo
    si.get_info = lambda *a, **k: {}
    cfg = types.ModuleType("numpy.distutils.__config__")
    nd.misc_util, nd.system_info, nd.__config__ = mu, si, cfg
    sys.modules.update({"numpy.distutils": nd, "numpy.distutils.misc_util": mu,
                        "numpy.distutils.system_info": si, "numpy.distutils.__config__": cfg})
    np.distutils = nd
    if not hasattr(configparser, "SafeConfigParser"):
        configparser.SafeConfigParser = configparser.ConfigParser
    for name, val in (("complex", complex), ("bool", bool), ("float", float), ("int", int),
                      ("object", object)):
        if not hasattr(np, name):
            setattr(np, name, val)
    if not hasattr(np, "ComplexWarning"):
        np.ComplexWarning = np.exceptions.ComplexWarning
    if not hasattr(np, "product"):
        np.product = np.prod
    if not hasattr(np, "sctype2char"):      # theano/tensor/elemwise.py:700 (constant folding in python)
        np.sctype2char = lambda t: np.dtype(t).char

    compiledir = os.environ.get("THEANO_REF_COMPILEDIR",
                                os.path.join(tempfile.gettempdir(), "theano_ref_compiledir"))
    os.makedirs(compiledir, exist_ok=True)
    cxxflags = ("-DNPY_PY3K=1 -DPyInt_AsLong=PyLong_AsLong -DPyInt_FromLong=PyLong_FromLong "
                "-DPyInt_Check=PyLong_Check -DPyInt_AS_LONG=PyLong_AsLong "
                "-DPyString_FromString=PyUnicode_FromString -fpermissive")
    flags = ["base_compiledir=" + compiledir, "device=cpu", "floatX=float32",
             "gcc.cxxflags=" + cxxflags]
    blas = _find_openblas()
    if blas and openmp:
        d, f = os.path.split(blas)
        flags += ["blas.ldflags=-L%s -l:%s -Wl\\,-rpath\\,%s" % (d, f, d), "openmp=True"]
    else:
        flags += ["blas.ldflags=", "openmp=False"]
    os.environ["THEANO_FLAGS"] = ",".join(flags)
    os.environ.setdefault("OMP_NUM_THREADS", str(os.cpu_count() or 1))

    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    import warnings
    warnings.filterwarnings("ignore")
    import theano
    from theano.gof.utils import MethodNotDefined
    from theano.tensor.elemwise import DimShuffle

    def _no_c(self, *a, **k):
        raise MethodNotDefined("c_code disabled: needs PyArray_Descr.elsize")

    DimShuffle.c_code = _no_c
    return theano
