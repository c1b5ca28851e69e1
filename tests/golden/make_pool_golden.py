"""Generate ``tests/golden/pool_golden.npz`` by running the reference's pooling ops.

Run where the reference source tree is present:

    python tests/golden/make_pool_golden.py

For a few seeded inputs (even and odd image sizes, values with ties inside windows) it compiles
``pool_2d(x, (2, 2), ignore_border=True)`` and its gradient with the reference's default optimizer
(asserting that the graph holds ``Pool`` and ``MaxPoolGrad``, theano/tensor/signal/pool.py:271,
1091), runs them and stores x, y, gy, gx.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import ref_theano  # noqa: E402

CASES = {                       # name -> (shape, seed, quantised values => ties)
    "even": ((3, 5, 8, 12), 11, False),
    "odd": ((2, 4, 9, 7), 12, False),
    "ties": ((2, 3, 6, 6), 13, True),
    "wide": ((1, 40, 14, 14), 14, False),
}


def inputs(name):
    shape, seed, ties = CASES[name]
    rs = np.random.RandomState(seed)
    x = rs.standard_normal(shape).astype(np.float32)
    if ties:
        x = np.round(x)                     # few distinct values: several maxima per window
    gy = rs.standard_normal((shape[0], shape[1], shape[2] // 2, shape[3] // 2)).astype(np.float32)
    return x, gy


def main():
    theano = ref_theano.import_theano()
    import theano.tensor as T
    from theano.tensor.signal.pool import MaxPoolGrad, Pool, pool_2d

    xs, gs = T.ftensor4("x"), T.ftensor4("gy")
    y = pool_2d(xs, (2, 2), ignore_border=True, mode="max")
    gx = theano.grad((y * gs).sum(), xs)
    f = theano.function([xs, gs], [y, gx])
    ops = [type(n.op) for n in f.maker.fgraph.toposort()]
    assert Pool in ops and MaxPoolGrad in ops, ops      # the reference's compiled C implementations
    store = {}
    for name in CASES:
        x, gy = inputs(name)
        yv, gxv = f(x, gy)
        store[name + "/x"], store[name + "/y"], store[name + "/gy"], store[name + "/gx"] = x, yv, gy, gxv
    path = os.path.join(HERE, "pool_golden.npz")
    np.savez_compressed(path, **store)
    print("wrote", path, len(store), "arrays")


if __name__ == "__main__":
    main()
