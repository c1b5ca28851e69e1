"""Layer shapes of the benchmark configurations and seeded synthetic tensors for them.

The network names only supply layer shapes (architecture hyper-parameters); no dataset, labels
or trained weights are involved.  Distributions follow the benchmark description: images ~ N(0, 1)
(U(0, 1) for the VGG input), filters He-normal N(0, 2 / ((C/g) kH kW)), upstream gradients
N(0, 1) in float32 and N(0, 1e-2) (sigma 0.1) in float16; float16 tensors are rounded before
they are fed to either implementation.
"""
import numpy as np


def L(c, k, ks, stride, pad, h, count=1, dil=1, groups=1, pool=False):
    return dict(C=c, K=k, k=ks, s=stride, p=pad, H=h, n=count, d=dil, g=groups, pool=pool)


def layer_name(lay):
    return "%d->%d %dx%d s%d d%d g%d @%d%s" % (lay["C"], lay["K"], lay["k"], lay["k"], lay["s"], lay["d"],
                                              lay["g"], lay["H"], " +pool" if lay.get("pool") else "")


def out_size(lay):
    keff = (lay["k"] - 1) * lay["d"] + 1
    return (lay["H"] + 2 * lay["p"] - keff) // lay["s"] + 1


def conv_kwargs(lay):
    return dict(border_mode=(lay["p"], lay["p"]), subsample=(lay["s"], lay["s"]),
                filter_dilation=(lay["d"], lay["d"]), num_groups=lay["g"], filter_flip=True)


def shapes(lay, batch):
    """(x, w, y) shapes of a layer in the reference's NCHW / OIHW order."""
    ho = out_size(lay)
    return ((batch, lay["C"], lay["H"], lay["H"]), (lay["K"], lay["C"] // lay["g"], lay["k"], lay["k"]),
            (batch, lay["K"], ho, ho))


def flops(lay, batch):
    """One pass (forward, gradInputs or gradWeights): 2 N K (C/g) kH kW Ho Wo
    (theano/tensor/nnet/abstract_conv.py:2163-2177)."""
    ho = out_size(lay)
    return 2.0 * batch * lay["K"] * (lay["C"] // lay["g"]) * lay["k"] * lay["k"] * ho * ho


def algorithmic_bytes(lay, batch, itemsize):
    """|X| + |W| + |Y|, each tensor touched once; a 2x2 max pooling fused into the layer writes a quarter of |Y|."""
    xs, ws, ys = shapes(lay, batch)
    ny = np.prod(ys, dtype=np.float64) / (4.0 if lay.get("pool") else 1.0)
    return float(itemsize) * (np.prod(xs, dtype=np.float64) + np.prod(ws, dtype=np.float64) + ny)


# 13 convolutions of VGG-16 (3x3, pad 1) with the 2x2 max pooling after layers 2, 4, 7, 10 and 13 as part of
# those layers (it runs in their epilogue)
VGG16 = [L(3, 64, 3, 1, 1, 224), L(64, 64, 3, 1, 1, 224, pool=True), L(64, 128, 3, 1, 1, 112),
         L(128, 128, 3, 1, 1, 112, pool=True), L(128, 256, 3, 1, 1, 56), L(256, 256, 3, 1, 1, 56),
         L(256, 256, 3, 1, 1, 56, pool=True), L(256, 512, 3, 1, 1, 28), L(512, 512, 3, 1, 1, 28),
         L(512, 512, 3, 1, 1, 28, pool=True), L(512, 512, 3, 1, 1, 14, 2), L(512, 512, 3, 1, 1, 14, pool=True)]
# the 23 distinct shapes among the 53 convolutions of ResNet-50 (stride 2 on the 3x3 of the
# down-sampling bottlenecks), with their number of occurrences
RESNET50 = [L(3, 64, 7, 2, 3, 224), L(64, 64, 1, 1, 0, 56), L(64, 256, 1, 1, 0, 56, 4), L(64, 64, 3, 1, 1, 56, 3),
            L(256, 64, 1, 1, 0, 56, 2), L(256, 512, 1, 2, 0, 56), L(256, 128, 1, 1, 0, 56),
            L(128, 128, 3, 2, 1, 56), L(128, 512, 1, 1, 0, 28, 4), L(512, 128, 1, 1, 0, 28, 3),
            L(128, 128, 3, 1, 1, 28, 3), L(512, 1024, 1, 2, 0, 28), L(512, 256, 1, 1, 0, 28),
            L(256, 256, 3, 2, 1, 28), L(256, 1024, 1, 1, 0, 14, 6), L(1024, 256, 1, 1, 0, 14, 5),
            L(256, 256, 3, 1, 1, 14, 5), L(1024, 2048, 1, 2, 0, 14), L(1024, 512, 1, 1, 0, 14),
            L(512, 512, 3, 2, 1, 14), L(512, 2048, 1, 1, 0, 7, 3), L(2048, 512, 1, 1, 0, 7, 2),
            L(512, 512, 3, 1, 1, 7, 2)]
SWEEP = [L(256, 64, 1, 1, 0, 56), L(64, 128, 3, 2, 1, 56), L(128, 128, 3, 1, 2, 28, dil=2),
         L(256, 256, 3, 1, 1, 28, groups=32)]
CONFIGS = {
    "cfg1": dict(layers=[L(3, 64, 3, 1, 1, 32)], batch=16, dtype=np.float32, dirs=("fwd",), relu=False),
    "cfg2": dict(layers=[L(256, 256, 3, 1, 1, 14)], batch=128, dtype=np.float32, dirs=("fwd", "dgrad", "wgrad"), relu=False),
    "vgg16": dict(layers=VGG16, batch=64, dtype=np.float32, dirs=("fwd",), relu=True),
    "sweep": dict(layers=SWEEP, batch=256, dtype=np.float32, dirs=("fwd", "dgrad", "wgrad"), relu=False),
    "resnet50": dict(layers=RESNET50, batch=256, dtype=np.float16, dirs=("fwd", "dgrad", "wgrad"), relu=False),
}


def resnet50_network():
    """The 53 convolutions in network order (forward order), each a layer dict with n = 1."""
    def one(c, k, ks, s, p, h):
        return L(c, k, ks, s, p, h)
    net = [one(3, 64, 7, 2, 3, 224)]
    h, cin = 56, 64
    for width, blocks, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
        for b in range(blocks):
            s = stride if b == 0 else 1
            net.append(one(cin, width, 1, 1, 0, h))                 # reduce
            net.append(one(width, width, 3, s, 1, h))               # 3x3 (carries the stride)
            ho = h // s
            net.append(one(width, 4 * width, 1, 1, 0, ho))          # expand
            if b == 0:
                net.append(one(cin, 4 * width, 1, s, 0, h))         # projection shortcut
            cin, h = 4 * width, ho
    assert len(net) == 53
    return net


def random_tensor(seed, shape, dtype, scale=1.0, dist="normal"):
    """Seeded tensor; beyond 4 M elements a 4 M block is repeated (host time only: the block
    length is no multiple of any image size here, so images still differ)."""
    n = int(np.prod(shape))
    block = min(n, (1 << 22) + 17)
    rng = np.random.default_rng(seed)
    if dist == "uniform":
        a = rng.random(block, dtype=np.float32)
    else:
        a = rng.standard_normal(block, dtype=np.float32)
    if scale != 1.0:
        a *= np.float32(scale)
    a = a.astype(dtype, copy=False)
    if block < n:
        out = np.empty(n, a.dtype)
        for i in range(0, n, block):
            m = min(block, n - i)
            out[i:i + m] = a[:m]
        a = out
    return a.reshape(shape)


def layer_tensors(lay, batch, dtype, seed, x_dist="normal"):
    """(x, w, dy) for one layer, drawn in that order from one seed."""
    xs, ws, ys = shapes(lay, batch)
    x = random_tensor(seed, xs, dtype, dist=x_dist)
    w = random_tensor(seed + 100003, ws, dtype, np.sqrt(2.0 / ((lay["C"] // lay["g"]) * lay["k"] * lay["k"])))
    dy = random_tensor(seed + 200003, ys, dtype, 0.1 if np.dtype(dtype) == np.float16 else 1.0)
    return x, w, dy
