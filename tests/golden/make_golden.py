"""Generate ``tests/golden/corrmm_golden.npz`` by running the reference itself.

Run where the reference source tree is present:

    python tests/golden/make_golden.py

For every case in ``cases.py`` it builds the *abstract* graph
(``theano.tensor.nnet.conv2d`` and ``theano.grad`` of it), compiles it with the
reference's default optimizer so that it is lowered to ``CorrMM`` /
``CorrMM_gradInputs`` / ``CorrMM_gradWeights`` (asserted), runs it on the seeded
inputs and stores y, dx, dw (strided samples for the larger cases).  It also
stores a fused bias+ReLU forward, a 2x2 max-pool, and the literal
input/kernel/output triple that the reference's ``TestCausalConv`` holds
(read out of the reference test file with ``ast``, not retyped).
"""
import ast
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

import cases as C  # noqa: E402
import ref_theano  # noqa: E402


def causal_triple():
    path = os.path.join(ref_theano.REF_ROOT, "theano/tensor/nnet/tests/test_abstract_conv.py")
    tree = ast.parse(open(path).read())
    out = {}
    for node in tree.body:
        if isinstance(node, ast.ClassDef) and node.name == "TestCausalConv":
            for st in node.body:
                if isinstance(st, ast.Assign) and st.targets[0].id in ("img", "kern", "precomp_top", "dilation"):
                    val = st.value
                    if st.targets[0].id != "dilation":
                        val = val.func.value.args[0]      # np.array(<literal>).astype(...)
                    out[st.targets[0].id] = np.asarray(ast.literal_eval(val), dtype=np.float32)
    assert set(out) == {"img", "kern", "precomp_top", "dilation"}
    return out


def main():
    theano = ref_theano.import_theano()
    import theano.tensor as T
    from theano.tensor.nnet import corr
    from theano.tensor.signal.pool import pool_2d

    store = {}
    for c in C.all_cases():
        x, w, dy = C.make_inputs(c)
        xs, ws, gs = T.ftensor4("x"), T.ftensor4("w"), T.ftensor4("dy")
        y = T.nnet.conv2d(xs, ws, border_mode=c["border"], subsample=c["sub"],
                          filter_flip=c["flip"], filter_dilation=c["dil"], num_groups=c["groups"])
        dx, dw = theano.grad((y * gs).sum(), [xs, ws])
        f = theano.function([xs, ws, gs], [y, dx, dw])
        ops = [type(n.op) for n in f.maker.fgraph.toposort()]
        if min(c["x"]) > 0 and min(c["w"]) > 0:
            assert corr.CorrMM in ops and corr.CorrMM_gradInputs in ops and corr.CorrMM_gradWeights in ops, ops
        yv, dxv, dwv = f(x, w, dy)
        assert yv.shape[2:] == C.out_hw(c), (c, yv.shape)
        s = c["sample"]
        store[c["name"] + "/y"] = C.sampled(yv, s)
        store[c["name"] + "/dx"] = C.sampled(dxv, s)
        store[c["name"] + "/dw"] = dwv
        print("%-14s y%s dx%s dw%s" % (c["name"], yv.shape, dxv.shape, dwv.shape))

    # fused epilogue + pool on one case: relu(conv + b) then 2x2 max pool
    c = [k for k in C.all_cases() if k["name"] == "cfg2_small"][0]
    x, w, _ = C.make_inputs(c)
    b = np.random.RandomState(7).standard_normal(c["w"][0]).astype(np.float32)
    xs, ws, bs = T.ftensor4("x"), T.ftensor4("w"), T.fvector("b")
    act = T.nnet.relu(T.nnet.conv2d(xs, ws, border_mode=c["border"]) + bs.dimshuffle("x", 0, "x", "x"))
    f = theano.function([xs, ws, bs], [act, pool_2d(act, (2, 2), ignore_border=True)])
    a, p = f(x, w, b)
    store["epilogue/bias"] = b
    store["epilogue/act"] = C.sampled(a, c["sample"])
    store["epilogue/pool"] = p

    for k, v in causal_triple().items():
        store["causal/" + k] = v

    out = os.path.join(HERE, "corrmm_golden.npz")
    np.savez_compressed(out, **store)
    print("wrote", out, os.path.getsize(out), "bytes;", len(store), "arrays")


if __name__ == "__main__":
    main()
