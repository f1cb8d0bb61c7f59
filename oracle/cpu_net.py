"""Linear-chain forward/backward on the CPU checkers (TEST INFRASTRUCTURE ONLY).

The same schedule as the reference's vl_simplenn (matlab/simplenn/vl_simplenn.m:294-524)
over numpy arrays, each block computed by a CpuBackend of oracle.py: the compiled reference
where it exists (conv, bnorm, pool), the C restatement for the blocks the reference has only
in MATLAB (ReLU, softmax-loss).  Used by the full-network parity tests and by the timed CPU
baseline of the benchmark; never by the library.
"""
import numpy as np


def _pair(v):
    v = np.atleast_1d(v).astype(int).ravel()
    return (int(v[0]), int(v[0])) if v.size == 1 else (int(v[0]), int(v[1]))


def _quad(v):
    v = np.atleast_1d(v).astype(int).ravel()
    return (int(v[0]),) * 4 if v.size == 1 else tuple(int(i) for i in v)


def _is_fc(l, xi):
    """The gateway's test for the fully connected shortcut (matlab/src/vl_nnconv.cu:351-361): the filters cover the
    whole input, no padding, unit stride and dilation, one filter group."""
    f = l["weights"][0]
    return (tuple(f.shape[:3]) == tuple(xi.shape[:3]) and _pair(l.get("stride", 1)) == (1, 1)
            and _quad(l.get("pad", 0)) == (0, 0, 0, 0) and _pair(l.get("dilate", 1)) == (1, 1))


def layer_forward(backend, glue, l, xi):
    """Output of one layer on input xi."""
    t = l["type"]
    if t == "conv":
        bias = None if l["weights"][1] is None else np.asarray(l["weights"][1]).ravel()
        if _is_fc(l, xi):
            return backend.fc_forward(xi, l["weights"][0], bias)
        return backend.conv_forward(xi, l["weights"][0], bias, _pair(l.get("stride", 1)), _quad(l.get("pad", 0)),
                                    _pair(l.get("dilate", 1)))
    if t == "relu":
        return glue.relu_forward(xi)
    if t == "pool":
        return backend.pool_forward(xi, _pair(l["pool"]), _pair(l.get("stride", 1)), _quad(l.get("pad", 0)),
                                    l.get("method", "max"))
    if t == "bnorm":
        return backend.bnorm_forward(xi, l["weights"][0], l["weights"][1], l.get("epsilon", 1e-4))[0]
    if t == "softmaxloss":
        return glue.softmaxloss_forward(xi, l["class"])
    if t == "normalize":
        return glue.lrn_forward(xi, l["param"])
    if t == "softmax":
        return glue.softmax(xi)
    raise ValueError(t)


def layer_backward(backend, glue, l, xi, d):
    """(dzdx, dzdw or None) of one layer from its input xi and the derivative d of its output."""
    t = l["type"]
    if t == "conv" and _is_fc(l, xi):
        dx, df, db = backend.fc_backward(xi, l["weights"][0], d)
        return dx, [df, db if l["weights"][1] is not None else None]
    if t == "conv":
        dx, df, db = backend.conv_backward(xi, l["weights"][0], d, _pair(l.get("stride", 1)), _quad(l.get("pad", 0)),
                                           _pair(l.get("dilate", 1)))
        return dx, [df, db if l["weights"][1] is not None else None]
    if t == "relu":
        return glue.relu_backward(xi, d), None
    if t == "pool":
        return backend.pool_backward(xi, d, _pair(l["pool"]), _pair(l.get("stride", 1)), _quad(l.get("pad", 0)),
                                     l.get("method", "max")), None
    if t == "bnorm":
        dx, dg, db, mom = backend.bnorm_backward(xi, l["weights"][0], l["weights"][1], d, l.get("epsilon", 1e-4))
        return dx, [dg, db, mom]
    if t == "softmaxloss":
        return glue.softmaxloss_backward(xi, l["class"], float(d)), None
    if t == "normalize":
        return glue.lrn_backward(xi, l["param"], d), None
    if t == "softmax":
        return glue.softmax(xi, d), None
    raise ValueError(t)


def simplenn(backend, glue, layers, x, dzdy=None, conserve_memory=False):
    """layers: dicts like matconvnet_b200.simplenn's, with numpy weights.
    Returns res: list of dicts with x, dzdx, dzdw (MATLAB-order numpy arrays)."""
    n = len(layers)
    res = [dict(x=None, dzdx=None, dzdw=None) for _ in range(n + 1)]
    res[0]["x"] = x
    for i, l in enumerate(layers):
        res[i + 1]["x"] = layer_forward(backend, glue, l, res[i]["x"])
    if dzdy is None:
        return res
    res[n]["dzdx"] = dzdy
    for i in range(n - 1, -1, -1):
        res[i]["dzdx"], res[i]["dzdw"] = layer_backward(backend, glue, layers[i], res[i]["x"], res[i + 1]["dzdx"])
        if conserve_memory and i + 1 < n:
            res[i + 1]["dzdx"] = None
    return res
