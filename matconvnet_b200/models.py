"""Layer lists of the networks the reference's examples build, with seeded random weights.

Shapes follow the reference's model builders: LeNet (examples/mnist/cnn_mnist_init.m:10-39),
the CIFAR-10 net (examples/cifar/cnn_cifar_init.m:8-65) and VGG-VD-16
(examples/imagenet/cnn_imagenet_init.m:336-400, dropout left out).  Weights are generated
on the host from a numpy seed -- so that every rank of a data-parallel run starts from the same
replica -- and uploaded as MATLAB-order device tensors.
"""
import numpy as np

from . import mat


def _conv(rng, fh, fw, cin, cout, stride=1, pad=0, init="he", scale=0.01, device="cuda"):
    if init == "he":          # dagnn.Conv.initParams (matlab/+dagnn/Conv.m:38-46)
        sc = np.sqrt(2.0 / (fh * fw * cin))
    else:
        sc = scale
    f = (rng.standard_normal((fh, fw, cin, cout)) * sc).astype(np.float32)
    b = np.zeros((1, cout), np.float32)
    return {"type": "conv", "weights": [mat.from_numpy(f, device), mat.from_numpy(b, device)],
            "stride": stride, "pad": pad, "dilate": 1}


def _relu():
    return {"type": "relu"}


def _pool(method, pool, stride, pad=0):
    return {"type": "pool", "method": method, "pool": [pool, pool], "stride": stride, "pad": pad}


def vgg16(seed=0, device="cuda", classes=1000):
    rng = np.random.default_rng(seed)
    layers = []
    cin = 3
    for block, (cout, reps) in enumerate([(64, 2), (128, 2), (256, 3), (512, 3), (512, 3)]):
        for _ in range(reps):
            layers += [_conv(rng, 3, 3, cin, cout, 1, 1, device=device), _relu()]
            cin = cout
        layers.append(_pool("max", 2, 2))
    layers += [_conv(rng, 7, 7, 512, 4096, device=device), _relu(),
               _conv(rng, 1, 1, 4096, 4096, device=device), _relu(),
               _conv(rng, 1, 1, 4096, classes, device=device),
               {"type": "softmaxloss", "class": None}]
    return {"layers": layers, "input": (224, 224, 3)}


def lenet_block(seed=0, device="cuda"):
    """conv 5x5x1x20 -> maxpool 2 -> conv 5x5x20x50 -> maxpool 2 (the first four layers of LeNet)."""
    rng = np.random.default_rng(seed)
    layers = [_conv(rng, 5, 5, 1, 20, init="gauss", device=device), _pool("max", 2, 2),
              _conv(rng, 5, 5, 20, 50, init="gauss", device=device), _pool("max", 2, 2)]
    return {"layers": layers, "input": (28, 28, 1)}


def cifar(seed=0, device="cuda"):
    rng = np.random.default_rng(seed)
    g = dict(init="gauss", device=device)
    layers = [_conv(rng, 5, 5, 3, 32, 1, 2, **g), _pool("max", 3, 2, [0, 1, 0, 1]), _relu(),
              _conv(rng, 5, 5, 32, 32, 1, 2, **g), _relu(), _pool("avg", 3, 2, [0, 1, 0, 1]),
              _conv(rng, 5, 5, 32, 64, 1, 2, **g), _relu(), _pool("avg", 3, 2, [0, 1, 0, 1]),
              _conv(rng, 4, 4, 64, 64, 1, 0, **g), _relu(),
              _conv(rng, 1, 1, 64, 10, 1, 0, **g),
              {"type": "softmaxloss", "class": None}]
    return {"layers": layers, "input": (32, 32, 3)}


def parameter_count(net):
    return sum(int(w.numel()) for l in net["layers"] if "weights" in l for w in l["weights"] if w is not None)


def conv_flops(net, batch):
    """Algorithmic multiply-add flops (2*M*N*K) of one forward pass of every convolution, per layer."""
    h, w, _ = net["input"]
    out = []
    for l in net["layers"]:
        if l["type"] == "conv":
            fh, fw, fc, k = [int(v) for v in l["weights"][0].shape]
            pad = l["pad"] if isinstance(l["pad"], (list, tuple)) else [l["pad"]] * 4
            s = l["stride"] if isinstance(l["stride"], (list, tuple)) else [l["stride"]] * 2
            ho = (h + pad[0] + pad[1] - fh) // s[0] + 1
            wo = (w + pad[2] + pad[3] - fw) // s[1] + 1
            out.append(2.0 * batch * ho * wo * k * fh * fw * fc)
            h, w = ho, wo
        elif l["type"] == "pool":
            pad = l["pad"] if isinstance(l["pad"], (list, tuple)) else [l["pad"]] * 4
            h = (h + pad[0] + pad[1] - l["pool"][0]) // l["stride"] + 1
            w = (w + pad[2] + pad[3] - l["pool"][1]) // l["stride"] + 1
    return out
