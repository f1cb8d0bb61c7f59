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


def simplenn(backend, glue, layers, x, dzdy=None):
    """layers: dicts like matconvnet_b200.simplenn's, with numpy weights.
    Returns res: list of dicts with x, dzdx, dzdw (MATLAB-order numpy arrays)."""
    n = len(layers)
    res = [dict(x=None, dzdx=None, dzdw=None) for _ in range(n + 1)]
    res[0]["x"] = x
    for i, l in enumerate(layers):
        t, xi = l["type"], res[i]["x"]
        if t == "conv":
            res[i + 1]["x"] = backend.conv_forward(xi, l["weights"][0], np.asarray(l["weights"][1]).ravel(),
                                                   _pair(l.get("stride", 1)), _quad(l.get("pad", 0)),
                                                   _pair(l.get("dilate", 1)))
        elif t == "relu":
            res[i + 1]["x"] = glue.relu_forward(xi)
        elif t == "pool":
            res[i + 1]["x"] = backend.pool_forward(xi, _pair(l["pool"]), _pair(l.get("stride", 1)),
                                                   _quad(l.get("pad", 0)), l.get("method", "max"))
        elif t == "bnorm":
            res[i + 1]["x"], _ = backend.bnorm_forward(xi, l["weights"][0], l["weights"][1], l.get("epsilon", 1e-4))
        elif t == "softmaxloss":
            res[i + 1]["x"] = glue.softmaxloss_forward(xi, l["class"])
        else:
            raise ValueError(t)
    if dzdy is None:
        return res
    res[n]["dzdx"] = dzdy
    for i in range(n - 1, -1, -1):
        l = layers[i]
        t, xi, d = l["type"], res[i]["x"], res[i + 1]["dzdx"]
        if t == "conv":
            dx, df, db = backend.conv_backward(xi, l["weights"][0], d, _pair(l.get("stride", 1)),
                                               _quad(l.get("pad", 0)), _pair(l.get("dilate", 1)))
            res[i]["dzdx"], res[i]["dzdw"] = dx, [df, db]
        elif t == "relu":
            res[i]["dzdx"] = glue.relu_backward(xi, d)
        elif t == "pool":
            res[i]["dzdx"] = backend.pool_backward(xi, d, _pair(l["pool"]), _pair(l.get("stride", 1)),
                                                   _quad(l.get("pad", 0)), l.get("method", "max"))
        elif t == "bnorm":
            dx, dg, db, mom = backend.bnorm_backward(xi, l["weights"][0], l["weights"][1], d, l.get("epsilon", 1e-4))
            res[i]["dzdx"], res[i]["dzdw"] = dx, [dg, db, mom]
        elif t == "softmaxloss":
            res[i]["dzdx"] = glue.softmaxloss_backward(xi, l["class"], float(d))
        if i + 1 < n:
            res[i + 1]["dzdx"] = None
    return res
