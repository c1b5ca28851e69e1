"""CPU-side checks of the C-ABI library: it loads without a GPU, exports every function the
public header declares, and refuses to compute when no B200 is present."""
import ctypes
import os
import re

import numpy as np
import pytest

from theano_b200 import build, shim

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "b200conv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200conv_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_header_symbols():
    build.build()
    lib = ctypes.CDLL(shim.LIB_PATH)
    names = header_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), "missing symbol " + n
    # the ctypes signatures cover exactly the header
    assert sorted(shim.SIGNATURES) == names


def test_desc_struct_matches_header():
    text = open(os.path.join(ROOT, "include", "b200conv.h")).read()
    body = text[text.index("typedef struct b200conv_desc {"):text.index("} b200conv_desc;")]
    fields = []
    for line in body.splitlines()[1:]:
        line = line.split("/*")[0].strip()
        if line.startswith("int32_t"):
            fields += [f.strip() for f in line[len("int32_t"):].rstrip(";").split(",")]
    assert fields == [f[0] for f in shim.Desc._fields_]
    assert ctypes.sizeof(shim.Desc) == 4 * len(fields)


def test_flag_and_error_constants_match_header():
    """The binding's flag bits and error codes are the header's enumerators."""
    text = open(os.path.join(ROOT, "include", "b200conv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    flags = {m.group(1): 1 << int(m.group(2)) for m in re.finditer(r"B200CONV_([A-Z0-9_]+)\s*=\s*1\s*<<\s*(\d+)", text)}
    assert len(flags) >= 12
    for name, bit in flags.items():
        assert getattr(shim, name) == bit, name
    errors = {m.group(1): int(m.group(2)) for m in re.finditer(r"B200CONV_(E_[A-Z]+)\s*=\s*(-\d+)", text)}
    assert len(errors) >= 6
    for name, code in errors.items():
        assert getattr(shim, name) == code, name


def test_no_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(shim.B200Error):
        shim.Context(0)
    with pytest.raises(shim.B200Error):
        shim.conv2d_forward(np.zeros((1, 1, 4, 4), np.float32), np.zeros((1, 1, 3, 3), np.float32))


def test_product_does_not_import_oracle():
    """The package must never reach for the CPU oracle (it is test infrastructure)."""
    pkg = os.path.join(ROOT, "theano_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read().lower()
                assert "oracle" not in src, (f, "mentions the oracle")
