"""The parameter update of the reference's trainer, after the gradient exchange (examples/cnn_train.m:451-500,
accumulateGradients): for every parameter of every layer, pull the summed derivative, normalise it by the number of
workers, add weight decay, update the momentum and the parameter -- or, for the third parameter of a bnorm layer (its
moments), move the stored moments towards the batch's (cnn_train.m:468-476).

``params``: dict with learning_rate, weight_decay, momentum, nesterov_update (cnn_train.m:17-45 defaults: 0.001, 0.0005,
0.9, False) and optionally solver ('adagrad', 'adadelta', 'adam' or 'rmsprop': examples/+solver/*.m, called at
cnn_train.m:503-507 instead of the momentum step) with solver_opts (the solver's own defaults otherwise).  A layer may carry 'learningRate' / 'weightDecay' lists (per parameter multipliers, default 1;
vl_simplenn_tidy).  ``state`` maps (layer index, parameter index) to the momentum tensor, created as zeros on first use
(cnn_train.m:292-301).  Every tensor operation is a call into the C ABI.
"""
import torch

from . import nn


def default_params():
    return dict(learning_rate=0.001, weight_decay=0.0005, momentum=0.9, nesterov_update=False)


def accumulate_gradients(net, res, state, params, num_workers=1, pulled=None, ctx=None):
    """net, res as in vl_simplenn; pulled: {(l, j): tensor} of derivatives SUMMED over the workers -- what
    GradientExchange.pull_all() returns by default and ParameterServer.pull returns in the reference -- else
    res[l]['dzdw'][j] is used as it is (cnn_train.m:459-464).  This function is the one place that divides by
    num_workers (cnn_train.m:455,482), so an exchange built with average=True must not be combined with num_workers > 1."""
    layers = net["layers"]
    for l in range(len(layers) - 1, -1, -1):
        dzdw = res[l]["dzdw"]
        if dzdw is None:
            continue
        layer = layers[l]
        for j in range(len(dzdw) - 1, -1, -1):
            der = pulled[(l, j)] if pulled is not None and (l, j) in pulled else dzdw[j]
            if der is None:
                continue
            w = layer["weights"][j]
            lr_mult = layer.get("learningRate", [1.0] * len(dzdw))[j]
            wd_mult = layer.get("weightDecay", [1.0] * len(dzdw))[j]
            if j == 2 and layer["type"] == "bnorm":
                # moments: w = (1 - lr) * w + lr / numWorkers * der   (cnn_train.m:468-476)
                nn.vl_taccum(1.0 - lr_mult, w, lr_mult / num_workers, der, out=w, ctx=ctx)
                continue
            decay = params["weight_decay"] * wd_mult
            lr = params["learning_rate"] * lr_mult
            if lr > 0 or decay > 0:
                key = (l, j)
                if params.get("solver"):
                    nn.solver_update_(params["solver"], w, state.setdefault(key, {}), der, 1.0 / num_workers, decay, lr,
                                      params.get("solver_opts"), ctx=ctx)
                    continue
                if key not in state:
                    state[key] = torch.zeros_like(w)
                nn.sgd_update_(w, state[key], der, 1.0 / num_workers, decay, params["momentum"], lr,
                               params.get("nesterov_update", False), ctx=ctx)
    return state
