"""vl_taccum and the fused SGD step against the reference trainer's arithmetic (examples/cnn_train.m:451-500)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _taccum_np(alpha, a, beta, b):
    # a scaled in single precision, then an axpy with one rounding (matlab/src/vl_taccummex.cu:50-76)
    t = (np.float32(alpha) * a).astype(np.float32)
    return (np.float64(np.float32(beta)) * b.astype(np.float64) + t.astype(np.float64)).astype(np.float32)


@pytest.mark.parametrize("n", [1, 7, 4096, 100003])
def test_taccum_matches_the_two_blas_calls(gpu, n):
    import torch
    nn, mat, ctx = gpu
    g = torch.Generator(device="cuda").manual_seed(n)
    a = torch.randn(n, device="cuda", generator=g)
    b = torch.randn(n, device="cuda", generator=g)
    want = _taccum_np(0.9, a.cpu().numpy(), -0.37, b.cpu().numpy())
    got = nn.vl_taccum(0.9, a, -0.37, b).cpu().numpy()
    # the double rounding of the emulation can differ from the fused multiply-add in the last place
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30)) <= 2.5e-7
    a2 = a.clone()
    nn.vl_taccum(0.9, a2, -0.37, b, out=a2)
    assert torch.equal(a2.cpu(), torch.from_numpy(got))
    # unaligned views take the scalar path and agree bit for bit
    if n > 8:
        assert torch.equal(nn.vl_taccum(0.9, a[1:], -0.37, b[1:]), torch.from_numpy(got).cuda()[1:])


@pytest.mark.parametrize("nesterov", [False, True])
def test_sgd_update_is_the_four_taccum_passes(gpu, nesterov):
    import torch
    nn, mat, ctx = gpu
    g = torch.Generator(device="cuda").manual_seed(11)
    n = 70001
    w = torch.randn(n, device="cuda", generator=g)
    m = torch.randn(n, device="cuda", generator=g) * 0.01
    der = torch.randn(n, device="cuda", generator=g)
    workers, decay, momentum, lr = 4, 0.0005, 0.9, 0.01
    # the reference's sequence (cnn_train.m:478-499)
    par = nn.vl_taccum(1.0 / workers, der, decay, w)
    m_ref = nn.vl_taccum(momentum, m, -1.0, par)
    delta = (momentum * m_ref - par) if nesterov else m_ref
    w_ref = nn.vl_taccum(1.0, w, lr, delta)
    w2, m2, der0 = w.clone(), m.clone(), der.clone()
    nn.sgd_update_(w2, m2, der, 1.0 / workers, decay, momentum, lr, nesterov)
    assert torch.equal(m2, m_ref) and torch.equal(w2, w_ref) and torch.equal(der, der0)
    # and the closed form in double precision
    wd, md, gd = w.double(), m.double(), der.double()
    pd = gd / workers + decay * wd
    md2 = momentum * md - pd
    dd = momentum * md2 - pd if nesterov else md2
    assert float((w2.double() - (wd + lr * dd)).abs().max()) < 1e-6
    assert float((m2.double() - md2).abs().max()) < 1e-6


def test_accumulate_gradients_follows_the_trainer(gpu):
    """One training step of a small network with a bnorm layer: forward/backward, then the update; the parameters move as
    the trainer's formulas say, the bnorm moments by the moving average, a layer with learning rate 0 and no decay stays."""
    import torch
    from matconvnet_b200 import models, simplenn, train
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    rng = np.random.default_rng(2)
    g = torch.Generator(device="cuda").manual_seed(2)
    C = 8
    layers = [models._conv(rng, 3, 3, 3, C, 1, 1),
              {"type": "bnorm", "weights": [mat.from_numpy(np.ones((C, 1), np.float32)), mat.from_numpy(np.zeros((C, 1), np.float32)),
                                            mat.from_numpy(np.zeros((C, 2), np.float32))], "epsilon": 1e-4,
               "learningRate": [2.0, 1.0, 0.1], "weightDecay": [0.0, 0.0, 0.0]},
              models._relu(), models._pool("max", 2, 2),
              models._conv(rng, 4, 4, C, 5, 1, 0),
              {"type": "softmaxloss", "class": torch.randint(1, 6, (6,), device="cuda", generator=g).float()}]
    layers[4]["learningRate"] = [0.0, 1.0]
    layers[4]["weightDecay"] = [0.0, 1.0]
    net = {"layers": layers}
    x = mat.as_mat(torch.randn(8, 8, 3, 6, device="cuda", generator=g))
    res = simplenn.vl_simplenn(net, x, 1.0, ctx=ctx)
    before = {(l, j): w.clone() for l, lay in enumerate(layers) if "weights" in lay for j, w in enumerate(lay["weights"])}
    params = dict(learning_rate=0.05, weight_decay=0.001, momentum=0.9, nesterov_update=False)
    state = {}
    workers = 2
    train.accumulate_gradients(net, res, state, params, num_workers=workers, ctx=ctx)
    for (l, j), w0 in before.items():
        lay = layers[l]
        w1, der = lay["weights"][j], res[l]["dzdw"][j]
        lrm = lay.get("learningRate", [1.0] * 3)[j]
        wdm = lay.get("weightDecay", [1.0] * 3)[j]
        if lay["type"] == "bnorm" and j == 2:
            want = (1 - lrm) * w0.double() + lrm / workers * der.double()
        elif lrm == 0 and wdm == 0:
            assert torch.equal(w1, w0) and (l, j) not in state
            continue
        else:
            par = der.double() / workers + params["weight_decay"] * wdm * w0.double()
            want = w0.double() + params["learning_rate"] * lrm * (-par)           # the momentum starts at zero
            assert float((state[(l, j)].double() + par).abs().max()) < 1e-6
        assert float((w1.double() - want).abs().max()) < 1e-6, (l, j)
    # a second step uses the stored momentum
    res = simplenn.vl_simplenn(net, x, 1.0, ctx=ctx)
    m0 = state[(0, 0)].clone()
    w0 = layers[0]["weights"][0].clone()
    train.accumulate_gradients(net, res, state, params, num_workers=workers, ctx=ctx)
    par = res[0]["dzdw"][0].double() / workers + params["weight_decay"] * w0.double()
    m1 = params["momentum"] * m0.double() - par
    assert float((layers[0]["weights"][0].double() - (w0.double() + params["learning_rate"] * m1)).abs().max()) < 1e-6


def test_exchanged_sums_are_normalised_exactly_once(gpu, monkeypatch):
    """pull_all returns sums (ParameterServer.pull); accumulate_gradients divides by the number of workers
    (cnn_train.m:455,482).  Four workers with identical shards -- the collective is faked as "multiply by four" -- must
    therefore move the parameters exactly as one worker alone does.  The derivatives are written straight into the
    exchange's buckets."""
    import copy
    import torch
    import torch.distributed as dist
    from matconvnet_b200 import dataparallel, models, simplenn, train
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    world = 4

    class _Done:
        def wait(self, *a):
            return True

    def fake_all_reduce(t, op=None, async_op=False):
        assert op == dist.ReduceOp.SUM
        t.mul_(world)
        return _Done()

    monkeypatch.setattr(dist, "all_reduce", fake_all_reduce)
    g = torch.Generator(device="cuda").manual_seed(5)

    def make():
        rng = np.random.default_rng(9)
        layers = [models._conv(rng, 3, 3, 3, 8, 1, 1), models._relu(), models._pool("max", 2, 2),
                  models._conv(rng, 4, 4, 8, 5, 1, 0),
                  {"type": "softmaxloss", "class": torch.tensor([1, 5, 2, 3, 4, 1], device="cuda").float()}]
        return {"layers": layers}

    x = mat.as_mat(torch.randn(8, 8, 3, 6, device="cuda", generator=g))
    params = dict(learning_rate=0.05, weight_decay=0.001, momentum=0.9, nesterov_update=False)

    alone = make()
    res = simplenn.vl_simplenn(alone, x, 1.0, ctx=ctx)
    train.accumulate_gradients(alone, res, {}, params, num_workers=1, ctx=ctx)

    net = make()
    ex = dataparallel.GradientExchange(world, bucket_bytes=1 << 12)
    views = ex.plan(simplenn.gradient_specs(net), "cuda")
    key = {simplenn.grad_name(i, j): (i, j) for i in range(len(net["layers"])) for j in range(2)}
    grad_out = {key[n]: v for n, v in views.items()}
    res = simplenn.vl_simplenn(net, x, 1.0, ctx=ctx, grad_out=grad_out,
                               on_dzdw=lambda i, j, w: ex.push(simplenn.grad_name(i, j), w))
    assert res[0]["dzdw"][0].data_ptr() == views[simplenn.grad_name(0, 0)].data_ptr()
    torch.cuda.synchronize()
    pulled = {key[n]: t for n, t in ex.pull_all().items()}
    assert ex.collectives < len(pulled)                      # bucketed: fewer collectives than tensors
    train.accumulate_gradients(net, res, {}, params, num_workers=world, pulled=pulled, ctx=ctx)
    for la, lb in zip(alone["layers"], net["layers"]):
        for wa, wb in zip(la.get("weights", []), lb.get("weights", [])):
            assert float((wa.double() - wb.double()).abs().max()) < 1e-6


def _solver_np(solver, w, s1, s2, g0, grad_mult, decay, lr, o, t):
    """examples/+solver/*.m on float32 arrays, one rounding per MATLAB operation, after the trainer's normalisation pass."""
    f = np.float32
    g = _taccum_np(grad_mult, g0, decay, w)
    gg = g * g
    if solver == "adagrad":
        s1 = s1 * f(o["rho"]) + gg
        w = w - (f(lr) * g) / (np.sqrt(s1) + f(o["epsilon"]))
    elif solver == "rmsprop":
        s1 = s1 * f(o["rho"]) + gg * f(1.0 - o["rho"])
        w = w - (f(lr) * g) / (np.sqrt(s1) + f(o["epsilon"]))
    elif solver == "adadelta":
        s1 = s1 * f(o["rho"]) + gg * f(1.0 - o["rho"])
        nd = -np.sqrt((s2 + f(o["epsilon"])) / (s1 + f(o["epsilon"]))) * g
        s2 = s2 * f(o["rho"]) + (nd * nd) * f(1.0 - o["rho"])
        w = w + nd
    else:
        s1 = f(o["beta1"]) * s1 + f(1.0 - o["beta1"]) * g
        s2 = f(o["beta2"]) * s2 + f(1.0 - o["beta2"]) * gg
        lr_t = f(lr * (np.sqrt(1.0 - o["beta2"] ** t) / (1.0 - o["beta1"] ** t)))
        w = w - (lr_t * s1) / (np.sqrt(s2) + f(o["epsilon"]))
    return w.astype(f), s1.astype(f), None if s2 is None else s2.astype(f)


@pytest.mark.parametrize("solver", ["adagrad", "adadelta", "adam", "rmsprop"])
def test_solver_update_follows_the_matlab_expressions(gpu, solver):
    """Three steps of each solver of examples/+solver on one tensor: bit for bit a float32 evaluation of the MATLAB
    expressions operation by operation (the taccum pass before it to its last-place tolerance), and within 1e-6 of the
    same formulas in double precision."""
    import torch
    from matconvnet_b200 import capi
    nn, mat, ctx = gpu
    g = torch.Generator(device="cuda").manual_seed(31)
    n = 50003
    w = torch.randn(n, device="cuda", generator=g)
    o = capi.SOLVER_DEFAULTS[solver]
    two = solver in ("adadelta", "adam")
    wn = w.cpu().numpy().copy()
    s1n, s2n = np.zeros(n, np.float32), (np.zeros(n, np.float32) if two else None)
    wd, s1d, s2d = wn.astype(np.float64), np.zeros(n), np.zeros(n)
    state = {}
    workers, decay, lr = 4, 0.0005, 0.01
    for t in range(1, 4):
        der = torch.randn(n, device="cuda", generator=g)
        der0 = der.clone()
        nn.solver_update_(solver, w, state, der, 1.0 / workers, decay, lr, ctx=ctx)
        assert torch.equal(der, der0) and state["t"] == t
        wn, s1n, s2n = _solver_np(solver, wn, s1n, s2n, der.cpu().numpy(), 1.0 / workers, decay, lr, o, t)
        # double-precision closed form
        gd = der.cpu().numpy().astype(np.float64) / workers + decay * wd
        if solver == "adagrad":
            s1d = s1d * o["rho"] + gd ** 2
            wd = wd - lr * gd / (np.sqrt(s1d) + o["epsilon"])
        elif solver == "rmsprop":
            s1d = s1d * o["rho"] + gd ** 2 * (1 - o["rho"])
            wd = wd - lr * gd / (np.sqrt(s1d) + o["epsilon"])
        elif solver == "adadelta":
            s1d = s1d * o["rho"] + gd ** 2 * (1 - o["rho"])
            nd = -np.sqrt((s2d + o["epsilon"]) / (s1d + o["epsilon"])) * gd
            s2d = s2d * o["rho"] + nd ** 2 * (1 - o["rho"])
            wd = wd + nd
        else:
            s1d = o["beta1"] * s1d + (1 - o["beta1"]) * gd
            s2d = o["beta2"] * s2d + (1 - o["beta2"]) * gd ** 2
            wd = wd - lr * (np.sqrt(1 - o["beta2"] ** t) / (1 - o["beta1"] ** t)) * s1d / (np.sqrt(s2d) + o["epsilon"])
    got = w.cpu().numpy()
    assert np.max(np.abs(got - wd)) < 2e-6
    # the emulated taccum pass rounds twice where the kernel's fused multiply-add rounds once: last-place differences
    assert np.max(np.abs(got - wn) / np.maximum(np.abs(wn), 1e-3)) < 2e-6
    assert np.max(np.abs(state["s1"].cpu().numpy() - s1n) / np.maximum(np.abs(s1n), 1e-6)) < 1e-5


def test_accumulate_gradients_with_a_solver(gpu):
    """train.accumulate_gradients(params['solver']='adam') moves a network's parameters as nn.solver_update_ does tensor
    by tensor (the call site examples/cnn_train.m:503-507)."""
    import torch
    from matconvnet_b200 import models, simplenn, train
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    rng = np.random.default_rng(4)
    g = torch.Generator(device="cuda").manual_seed(4)
    layers = [models._conv(rng, 3, 3, 3, 8, 1, 1), models._relu(), models._conv(rng, 8, 8, 8, 5, 1, 0),
              {"type": "softmaxloss", "class": torch.tensor([1, 2, 3, 4], device="cuda").float()}]
    net = {"layers": layers}
    x = mat.as_mat(torch.randn(8, 8, 3, 4, device="cuda", generator=g))
    res = simplenn.vl_simplenn(net, x, 1.0, ctx=ctx)
    want = {}
    for l in (0, 2):
        for j in (0, 1):
            w = layers[l]["weights"][j].clone()
            nn.solver_update_("adam", w, {}, res[l]["dzdw"][j], 0.5, 0.0005, 0.001, ctx=ctx)
            want[(l, j)] = w
    state = {}
    train.accumulate_gradients(net, res, state, dict(learning_rate=0.001, weight_decay=0.0005, momentum=0.9, solver="adam"),
                               num_workers=2, ctx=ctx)
    for (l, j), w in want.items():
        assert torch.equal(layers[l]["weights"][j], w) and state[(l, j)]["t"] == 1
