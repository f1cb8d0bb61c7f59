"""Linear-chain forward/backward in the reference's schedule (matlab/simplenn/vl_simplenn.m).

A network is ``{'layers': [layer, ...]}`` with layers shaped like the reference's structs:
  {'type': 'conv', 'weights': [f, b], 'stride': s, 'pad': p, 'dilate': d}
  {'type': 'relu'}   {'type': 'pool', 'method': 'max'|'avg', 'pool': [ph pw], 'stride': s, 'pad': p}
  {'type': 'bnorm', 'weights': [g, b, moments], 'epsilon': e}   {'type': 'softmaxloss', 'class': c}
  {'type': 'normalize', 'param': [N kappa alpha beta]}   {'type': 'softmax'}
  {'type': 'dropout', 'rate': r}  (training mode: a new mask per forward pass, kept in res[i]['aux'] for the backward pass)
``vl_simplenn(net, x, dzdy)`` runs the forward pass storing every intermediate (res[i]['x'],
vl_simplenn.m:294-398) and, when dzdy is given, the backward pass in reverse order
(vl_simplenn.m:404-524), leaving res[i]['dzdx'] and, for parametrised layers, res[i]['dzdw'].
As in the reference, each layer's parameter derivatives are handed to the gradient exchange
as soon as they exist (vl_simplenn.m:504-509): ``on_dzdw(i, j, tensor)`` is called right
after layer i's backward, which is what lets the all-reduce overlap the remaining layers.
``grad_out`` maps (i, j) to a tensor the derivative of parameter j of layer i is written into (views
into the gradient exchange's buckets, ``dataparallel.GradientExchange.plan``) instead of a new one.
Every block is a call into the C ABI; nothing is computed on the host.
"""
from . import nn


def grad_name(i, j):
    """The name under which the derivative of parameter j of layer i is handed to the gradient exchange."""
    return "l%d_%d" % (i, j)


def gradient_specs(net):
    """[(name, MATLAB shape)] of the parameter derivatives of conv and bnorm layers in the order the backward pass
    produces them (last layer first, filters before biases): the input of GradientExchange.plan."""
    specs = []
    for i in range(len(net["layers"]) - 1, -1, -1):
        l = net["layers"][i]
        if l["type"] in ("conv", "bnorm"):
            for j, w in enumerate(l["weights"][:2]):
                if w is not None:
                    specs.append((grad_name(i, j), tuple(int(v) for v in w.shape)))
    return specs


def _get(l, key, default):
    return l[key] if key in l and l[key] is not None else default


def vl_simplenn(net, x, dzdy=None, res=None, on_dzdw=None, ctx=None, skip_forward=False,
                back_prop_depth=None, conserve_memory=False, fuse_relu=False, grad_out=None):
    layers = net["layers"]
    n = len(layers)
    if res is None:
        res = [dict(x=None, dzdx=None, dzdw=None, aux=None) for _ in range(n + 1)]
    if not skip_forward:
        res[0]["x"] = x
        fused = False
        for i, l in enumerate(layers):
            t = l["type"]
            xi = res[i]["x"]
            if t == "conv":
                # fuse_relu: a ReLU that follows is applied by the convolution's own kernels; the ReLU's input is never
                # stored, as when the reference drops it to conserve memory (vl_simplenn.m:386)
                fused = fuse_relu and i + 1 < n and layers[i + 1]["type"] == "relu"
                y = nn.vl_nnconv(xi, l["weights"][0], l["weights"][1], stride=_get(l, "stride", 1),
                                 pad=_get(l, "pad", 0), dilate=_get(l, "dilate", 1), relu=fused, ctx=ctx)
                if fused:
                    res[i + 1]["x"], res[i + 2]["x"] = None, y
                else:
                    res[i + 1]["x"] = y
            elif t == "relu":
                if fused:
                    fused = False          # done by the convolution before
                else:
                    res[i + 1]["x"] = nn.vl_nnrelu(xi, ctx=ctx)
            elif t == "pool":
                res[i + 1]["x"] = nn.vl_nnpool(xi, l["pool"], stride=_get(l, "stride", 1), pad=_get(l, "pad", 0),
                                               method=_get(l, "method", "max"), ctx=ctx)
            elif t == "bnorm":
                # training mode: moments from the batch (vl_simplenn.m:345-351); a ReLU that follows is applied by the
                # same kernel under fuse_relu, as after a convolution
                fused = fuse_relu and i + 1 < n and layers[i + 1]["type"] == "relu"
                y, res[i]["aux"] = nn.vl_nnbnorm(xi, l["weights"][0], l["weights"][1], epsilon=_get(l, "epsilon", 1e-4),
                                                 relu=fused, ctx=ctx)
                if fused:
                    res[i + 1]["x"], res[i + 2]["x"] = None, y
                else:
                    res[i + 1]["x"] = y
            elif t == "softmaxloss":
                res[i + 1]["x"] = nn.vl_nnsoftmaxloss(xi, l["class"], ctx=ctx)
            elif t == "normalize":
                res[i + 1]["x"] = nn.vl_nnnormalize(xi, l["param"], ctx=ctx)
            elif t == "softmax":
                res[i + 1]["x"] = nn.vl_nnsoftmax(xi, ctx=ctx)
            elif t == "dropout":
                # vl_simplenn.m:352-360 (training mode); 'seed' makes the mask reproducible, the layer index separates layers
                res[i + 1]["x"], res[i]["aux"] = nn.vl_nndropout(xi, rate=_get(l, "rate", 0.5),
                                                                 seed=(int(_get(l, "seed", 0)) << 16) + i, ctx=ctx)
            else:
                raise ValueError("Unknown layer type '%s'." % t)
    if dzdy is None:
        return res
    res[n]["dzdx"] = dzdy
    grad_out = grad_out or {}
    first = 0 if back_prop_depth is None else max(0, n - back_prop_depth)
    masked = False
    for i in range(n - 1, first - 1, -1):
        l = layers[i]
        t = l["type"]
        xi, d = res[i]["x"], res[i + 1]["dzdx"]
        # fuse_relu: the backward pass of a ReLU directly before a convolution or pooling layer is done by that layer's
        # own data-gradient kernel, which zeroes the derivative where its input (the ReLU's output) is not positive; the
        # derivative between the two layers is never stored, as when the reference conserves memory (vl_simplenn.m:512-514)
        through = fuse_relu and t in ("conv", "pool") and i - 1 >= first and layers[i - 1]["type"] == "relu"
        if t == "conv":
            dx, df, db = nn.vl_nnconv(xi, l["weights"][0], l["weights"][1], d, stride=_get(l, "stride", 1),
                                      pad=_get(l, "pad", 0), dilate=_get(l, "dilate", 1), through_relu=through,
                                      der_out=(grad_out.get((i, 0)), grad_out.get((i, 1))), ctx=ctx)
            res[i]["dzdw"] = [df, db]
            res[i]["dzdx"], res[i - 1 if through else i]["dzdx"] = None, dx
        elif t == "relu":
            if masked:
                pass                       # done by the layer after
            else:
                # an input that was not kept: the mask comes from the output, which is positive exactly where the input
                # is (vl_simplenn.m:448-455)
                res[i]["dzdx"] = nn.vl_nnrelu(xi if xi is not None else res[i + 1]["x"], d, ctx=ctx)
        elif t == "pool":
            dx = nn.vl_nnpool(xi, l["pool"], d, stride=_get(l, "stride", 1), pad=_get(l, "pad", 0),
                              method=_get(l, "method", "max"), through_relu=through, ctx=ctx)
            res[i]["dzdx"], res[i - 1 if through else i]["dzdx"] = None, dx
        elif t == "bnorm":
            dx, dg, db, mom = nn.vl_nnbnorm(xi, l["weights"][0], l["weights"][1], d, epsilon=_get(l, "epsilon", 1e-4),
                                            der_out=(grad_out.get((i, 0)), grad_out.get((i, 1))), ctx=ctx)
            res[i]["dzdx"], res[i]["dzdw"] = dx, [dg, db, mom]
        elif t == "softmaxloss":
            res[i]["dzdx"] = nn.vl_nnsoftmaxloss(xi, l["class"], d, ctx=ctx)
        elif t == "normalize":
            res[i]["dzdx"] = nn.vl_nnnormalize(xi, l["param"], d, ctx=ctx)
        elif t == "softmax":
            res[i]["dzdx"] = nn.vl_nnsoftmax(xi, d, ctx=ctx)
        elif t == "dropout":
            res[i]["dzdx"], _ = nn.vl_nndropout(xi, d, mask=res[i]["aux"], ctx=ctx)      # vl_simplenn.m:466-473
        else:
            raise ValueError("Unknown layer type '%s'." % t)
        if on_dzdw is not None and res[i]["dzdw"] is not None:
            for j, w in enumerate(res[i]["dzdw"]):
                if w is not None:
                    on_dzdw(i, j, w)
        masked = through
        if conserve_memory and i + 1 < n:
            res[i + 1]["dzdx"] = None      # opts.conserveMemory (vl_simplenn.m:512-514)
    return res
