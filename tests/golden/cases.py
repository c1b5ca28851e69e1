"""Case list and seeded input generator shared by the golden-fixture script and the tests.

The small-shape matrix follows the reference's own conv test matrix
(theano/tensor/nnet/tests/test_abstract_conv.py:584-599 shapes, subsamples,
dilations, border modes, flips; :1490-1495 groups; :1961-1964 asymmetric
padding); the ``cfg*`` cases are scaled-down versions of the benchmark
configurations, and ``cfg1`` is the first one at full size.
"""
import zlib

import numpy as np

REF_INPUTS = [(8, 1, 6, 6), (8, 1, 8, 8), (2, 1, 7, 7), (6, 1, 10, 11), (2, 1, 6, 5), (1, 5, 9, 9),
              (0, 1, 6, 6), (1, 0, 6, 6), (1, 1, 6, 6)]
REF_FILTERS = [(5, 1, 2, 2), (4, 1, 3, 3), (2, 1, 3, 3), (1, 1, 2, 3), (4, 1, 1, 3), (4, 5, 3, 2),
               (1, 1, 2, 2), (1, 0, 2, 2), (0, 1, 2, 2)]
SUBSAMPLES = [(1, 1), (2, 2), (2, 4)]
DILATIONS = [(1, 1), (1, 2), (2, 1)]
BORDER_MODES = ["valid", "half", "full", (0, 0), (1, 1), (5, 5), (5, 2)]


def _case(name, x, w, border="valid", sub=(1, 1), dil=(1, 1), groups=1, flip=True, dist="uniform",
          sample=1):
    return dict(name=name, x=tuple(x), w=tuple(w), border=border, sub=tuple(sub), dil=tuple(dil),
                groups=groups, flip=flip, dist=dist, sample=sample)


def out_hw(c):
    """Output height/width of a case, or None if the geometry is impossible."""
    res = []
    for a in range(2):
        k = (c["w"][2 + a] - 1) * c["dil"][a] + 1
        b = c["border"]
        if b == "valid":
            pl = pr = 0
        elif b == "half":
            pl = pr = k // 2
        elif b == "full":
            pl = pr = k - 1
        else:
            m = b[a] if isinstance(b, tuple) else b
            pl, pr = m if isinstance(m, tuple) else (m, m)
        o = (c["x"][2 + a] + pl + pr - k) // c["sub"][a] + 1
        if o <= 0:
            return None
        res.append(o)
    return tuple(res)


def all_cases():
    cases = []
    for i, (xs, ws) in enumerate(zip(REF_INPUTS, REF_FILTERS)):
        cases.append(_case("ref%d" % i, xs, ws))
    n = 0
    for sub in SUBSAMPLES:
        for bm in BORDER_MODES:
            for dil in DILATIONS:
                for flip in (True, False):
                    c = _case("mat%03d" % n, REF_INPUTS[3], REF_FILTERS[3], bm, sub, dil, 1, flip)
                    n += 1
                    if out_hw(c) is not None:
                        cases.append(c)
    n = 0
    for sub in SUBSAMPLES:
        for bm in BORDER_MODES:
            c = _case("multi%02d" % n, REF_INPUTS[5], REF_FILTERS[5], bm, sub)
            n += 1
            if out_hw(c) is not None:
                cases.append(c)
    grp = [((5, 6, 5, 5), (6, 2, 3, 3), 3), ((4, 4, 7, 5), (6, 2, 5, 3), 2),
           ((3, 8, 5, 3), (4, 2, 3, 3), 4), ((2, 4, 7, 7), (4, 1, 3, 5), 4)]
    for i, (xs, ws, g) in enumerate(grp):
        cases.append(_case("group%d" % i, xs, ws, groups=g))
        cases.append(_case("group%d_s2" % i, xs, ws, border="half", sub=(2, 1), groups=g, flip=False))
    asym = [((2, 2, 4, 4), (4, 2, 2, 2), ((1, 2), (2, 1))), ((3, 2, 4, 2), (2, 2, 4, 2), ((1, 1), (0, 3))),
            ((3, 3, 5, 3), (2, 3, 3, 3), ((2, 1), (0, 0)))]
    for i, (xs, ws, bm) in enumerate(asym):
        cases.append(_case("asym%d" % i, xs, ws, border=bm))
    # benchmark configurations, scaled down where the full size would bloat the fixture
    cases.append(_case("cfg1", (16, 3, 32, 32), (64, 3, 3, 3), "half", dist="cfg1", sample=53))
    cases.append(_case("cfg2_small", (4, 64, 14, 14), (64, 64, 3, 3), (1, 1), dist="he", sample=7))
    cases.append(_case("cfg4a_small", (2, 64, 28, 28), (16, 64, 1, 1), dist="he", sample=5))
    cases.append(_case("cfg4b_small", (2, 16, 28, 28), (32, 16, 3, 3), (1, 1), sub=(2, 2), dist="he", sample=5))
    cases.append(_case("cfg4c_small", (2, 32, 14, 14), (32, 32, 3, 3), (2, 2), dil=(2, 2), dist="he", sample=5))
    cases.append(_case("cfg4d_small", (2, 64, 14, 14), (64, 8, 3, 3), (1, 1), groups=8, dist="he", sample=5))
    cases.append(_case("stem7x7", (2, 3, 32, 32), (16, 3, 7, 7), (3, 3), sub=(2, 2), dist="he", sample=5))
    cases.append(_case("proj1x1s2", (2, 32, 14, 14), (64, 32, 1, 1), sub=(2, 2), dist="he", sample=3))
    cases.append(_case("skewed", (1, 64, 3, 256), (4, 64, 1, 1), dist="he", sample=3))
    cases.append(_case("depthwise", (2, 8, 9, 9), (8, 1, 3, 3), "half", groups=8, dist="he"))
    return cases


def make_inputs(c, dtype=np.float32):
    """Seeded x, w, dy for a case (seed derived from its name)."""
    rs = np.random.RandomState(zlib.crc32(c["name"].encode()) & 0x7FFFFFFF)
    hw = out_hw(c)
    yshape = (c["x"][0], c["w"][0]) + hw
    if c["dist"] == "uniform":       # reference tests: np.random.random, test_abstract_conv.py:377-382
        x = rs.random_sample(c["x"])
        w = rs.random_sample(c["w"])
        dy = rs.random_sample(yshape)
    else:
        fan = max(1, c["w"][1] * c["w"][2] * c["w"][3])
        x = rs.standard_normal(c["x"])
        std = np.sqrt(1.0 / 27) if c["dist"] == "cfg1" else np.sqrt(2.0 / fan)
        w = rs.standard_normal(c["w"]) * std
        dy = rs.standard_normal(yshape)
    return x.astype(dtype), w.astype(dtype), dy.astype(dtype)


def sampled(a, step):
    return np.ascontiguousarray(a.ravel()[::step]) if step > 1 else a
