"""Optimizers and LR schedulers on CPU: closed-form steps and agreement with torch.optim where the rules coincide."""
import math

import pytest
import torch

from prometorch_b200 import optim as O


def _problem(seed=0):
    torch.manual_seed(seed)
    w = torch.nn.Parameter(torch.randn(6, 5))
    b = torch.nn.Parameter(torch.randn(5))
    x, y = torch.randn(32, 6), torch.randn(32, 5)
    return [w, b], lambda: ((x @ w + b - y) ** 2).mean()


def _run(opt_cls, steps=5, **kw):
    ps, loss = _problem()
    opt = opt_cls(ps, **kw)
    for _ in range(steps):
        opt.zero_grad()
        loss().backward()
        opt.step()
    return [p.detach().clone() for p in ps]


@pytest.mark.parametrize("ours,theirs,kw", [
    (O.SGD, torch.optim.SGD, dict(lr=0.1, momentum=0.9, nesterov=True, weight_decay=0.01)),
    (O.Adam, torch.optim.Adam, dict(lr=1e-2, weight_decay=0.1)),
    (O.Adam, torch.optim.Adam, dict(lr=1e-2, amsgrad=True)),
    (O.AdamW, torch.optim.AdamW, dict(lr=1e-2, weight_decay=0.1)),
    (O.RMSprop, torch.optim.RMSprop, dict(lr=1e-2, momentum=0.5, centered=True)),
    (O.NAdam, torch.optim.NAdam, dict(lr=2e-3)),
    (O.RAdam, torch.optim.RAdam, dict(lr=1e-2)),
    (O.Adagrad, torch.optim.Adagrad, dict(lr=0.05, lr_decay=0.1)),
    (O.Adadelta, torch.optim.Adadelta, dict(lr=1.0)),
    (O.Adamax, torch.optim.Adamax, dict(lr=2e-3)),
])
def test_matches_torch(ours, theirs, kw):
    a = _run(ours, steps=8, **kw)
    b = _run(theirs, steps=8, **kw)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, atol=2e-6, rtol=1e-5), (x - y).abs().max()


def test_lion_closed_form():
    p = torch.nn.Parameter(torch.tensor([1.0, -2.0]))
    opt = O.Lion([p], lr=0.1, betas=(0.9, 0.99), weight_decay=0.1)
    p.grad = torch.tensor([0.5, -0.25])
    opt.step()
    exp = torch.tensor([1.0, -2.0]) * (1 - 0.1 * 0.1) - 0.1 * torch.sign(torch.tensor([0.05, -0.025]))
    assert torch.allclose(p.detach(), exp)
    assert torch.allclose(opt.state[p]["exp_avg"], torch.tensor([0.005, -0.0025]))


def test_sophia_clip():
    p = torch.nn.Parameter(torch.zeros(3))
    opt = O.SophiaG([p], lr=1.0, rho=0.04)
    p.grad = torch.tensor([1.0, -1.0, 1e-9])
    opt.step()
    assert torch.allclose(p.detach()[:2], torch.tensor([-0.04, 0.04]))


@pytest.mark.parametrize("cls,kw", [(O.LAMB, {}), (O.Adafactor, {}), (O.AdamKiller, {}), (O.ASGD, dict(lr=0.05)),
                                     (O.Lion, dict(lr=1e-2)), (O.SophiaG, dict(lr=1e-2))])
def test_loss_decreases(cls, kw):
    ps, loss = _problem(1)
    opt = cls(ps, **kw)
    l0 = float(loss())
    for _ in range(60):
        opt.zero_grad()
        loss().backward()
        opt.step()
    assert float(loss()) < l0


def test_lbfgs_closure():
    ps, loss = _problem(2)
    opt = O.LBFGS(ps, lr=0.5)
    l0 = float(loss())

    def closure():
        opt.zero_grad()
        l = loss()
        l.backward()
        return l
    for _ in range(3):
        opt.step(closure)
    assert float(loss()) < 0.5 * l0


def test_param_groups_and_state_dict_roundtrip():
    ps, loss = _problem(3)
    opt = O.AdamW([O.ParamGroup([ps[0]], lr=1e-2), O.ParamGroup([ps[1]], weight_decay=0.0)], lr=1e-3)
    assert opt.param_groups[0]["lr"] == 1e-2 and opt.param_groups[1]["lr"] == 1e-3
    assert opt.param_groups[1]["weight_decay"] == 0.0 and opt.param_groups[0]["weight_decay"] == 0.01
    for _ in range(3):
        opt.zero_grad(); loss().backward(); opt.step()
    import copy
    sd = copy.deepcopy(opt.state_dict())      # state_dict() hands out live tensors
    flat = opt.flat_state_dict()
    assert set(k.split(".", 2)[2] for k in flat) == {"step", "exp_avg", "exp_avg_sq"} and float(flat["state.0.step"]) == 3
    ps2, loss2 = _problem(3)
    for a, b in zip(ps2, ps):
        a.data.copy_(b.data)
    opt2 = O.AdamW([O.ParamGroup([ps2[0]], lr=1e-2), O.ParamGroup([ps2[1]], weight_decay=0.0)], lr=1e-3)
    opt2.load_state_dict(sd)
    for o, l in ((opt, loss), (opt2, loss2)):
        o.zero_grad(); l().backward(); o.step()
    for a, b in zip(ps, ps2):
        assert torch.allclose(a, b, atol=1e-7)


@pytest.mark.parametrize("make", [lambda ps: O.Adam(ps, lr=1e-2), lambda ps: O.SGD(ps, lr=1e-2, momentum=0.9),
                                  lambda ps: O.RAdam(ps, lr=1e-2)])
def test_flat_state_resume_continues_the_run(make):
    """save -> load_flat_state_dict -> step must equal the uninterrupted run (bias correction, momentum buffer)."""
    import copy
    ps, loss = _problem(3)
    opt = make(ps)
    for _ in range(5):
        opt.zero_grad(); loss().backward(); opt.step()
    flat = copy.deepcopy(opt.flat_state_dict())
    ps2, loss2 = _problem(3)
    for a, b in zip(ps2, ps):
        a.data.copy_(b.data)
    opt2 = make(ps2)
    opt2.load_flat_state_dict(flat)
    for o, l in ((opt, loss), (opt2, loss2)):
        o.zero_grad(); l().backward(); o.step()
    for a, b in zip(ps, ps2):
        assert torch.allclose(a, b, atol=1e-7)


def test_ema():
    p = torch.nn.Parameter(torch.ones(2))
    e = O.EMA([p], decay=0.9)
    p.data.fill_(2.0)
    e.update()
    assert torch.allclose(e.shadow[0], torch.full((2,), 1.1))
    e.apply_shadow()
    assert torch.allclose(p.detach(), torch.full((2,), 1.1))
    e.restore()
    assert torch.allclose(p.detach(), torch.full((2,), 2.0))
    with pytest.raises(ValueError):
        O.EMA([p], decay=1.0)


def _lrs(sched, n, opt, arg=None):
    out = []
    for _ in range(n):
        sched.step() if arg is None else sched.step(arg)
        out.append(opt.param_groups[0]["lr"])
    return out


def _opt(lr=1.0):
    return O.SGD([torch.nn.Parameter(torch.zeros(1))], lr=lr)


def test_schedulers_closed_forms():
    o = _opt(); assert _lrs(O.StepLR(o, 2, 0.5), 5, o) == [1.0, 1.0, 0.5, 0.5, 0.25]
    o = _opt(); assert _lrs(O.MultiStepLR(o, [1, 3], 0.1), 4, o) == pytest.approx([1.0, 0.1, 0.1, 0.01])
    o = _opt(); assert _lrs(O.ExponentialLR(o, 0.5), 3, o) == [1.0, 0.5, 0.25]
    o = _opt(); assert _lrs(O.CosineAnnealingLR(o, 4), 5, o) == pytest.approx([1.0, (1 + math.cos(math.pi / 4)) / 2, 0.5, (1 + math.cos(3 * math.pi / 4)) / 2, 0.0], abs=1e-12)
    o = _opt(); assert _lrs(O.LinearLR(o, 0.5, 1.0, 2), 4, o) == pytest.approx([0.5, 0.75, 1.0, 1.0])
    o = _opt(); assert _lrs(O.ConstantLR(o, 0.25, 2), 3, o) == [0.25, 0.25, 1.0]
    o = _opt(); assert _lrs(O.WarmupCosineAnnealingLR(o, 2, 6), 7, o) == pytest.approx([0.5, 1.0, 1.0, (1 + math.cos(math.pi / 4)) / 2, 0.5, (1 + math.cos(3 * math.pi / 4)) / 2, 0.0], abs=1e-12)
    o = _opt(); assert _lrs(O.PolynomialLR(o, 4, 2.0), 5, o) == pytest.approx([1.0, 0.5625, 0.25, 0.0625, 0.0])
    o = _opt(); assert _lrs(O.LambdaLR(o, lambda e: 1 / (e + 1)), 3, o) == pytest.approx([1.0, 0.5, 1 / 3])
    o = _opt(); assert _lrs(O.MultiplicativeLR(o, lambda e: 0.5), 3, o) == [1.0, 0.5, 0.25]
    o = _opt(); assert _lrs(O.CosineAnnealingWarmRestarts(o, 2), 4, o) == pytest.approx([0.5, 1.0, 0.5, 1.0])
    o = _opt(); assert _lrs(O.CyclicLR(o, 0.1, 1.1, 2), 5, o) == pytest.approx([0.1, 0.6, 1.1, 0.6, 0.1])


def test_onecycle_plateau_sequential_chained():
    o = _opt()
    s = O.OneCycleLR(o, max_lr=1.0, total_steps=10, pct_start=0.3, div_factor=10, final_div_factor=10)
    assert o.param_groups[0]["lr"] == pytest.approx(0.1)
    lrs = _lrs(s, 10, o)
    assert lrs[2] == pytest.approx(1.0) and lrs[-1] == pytest.approx(0.01) and max(lrs) == pytest.approx(1.0)
    o = _opt()
    s = O.ReduceLROnPlateau(o, "min", factor=0.5, patience=1)
    for m in [1.0, 1.0, 1.0]:
        s.step(m)
    assert o.param_groups[0]["lr"] == 0.5
    o = _opt()
    s = O.SequentialLR(o, [O.ConstantLR(o, 0.1, 100), O.ExponentialLR(o, 0.5)], [2])
    assert _lrs(s, 4, o) == pytest.approx([0.1, 0.1, 1.0, 0.5])
    o = _opt()
    s = O.ChainedScheduler(o, [O.ExponentialLR(o, 0.5), O.ConstantLR(o, 0.1, 2)])
    assert _lrs(s, 3, o) == pytest.approx([0.1, 0.05, 0.25])
    with pytest.raises(ValueError):
        O.SequentialLR(o, [O.ExponentialLR(o, 0.5)], [1])


def test_clip_grad_norm_cpu():
    p = torch.nn.Parameter(torch.zeros(4))
    p.grad = torch.tensor([3.0, 4.0, 0.0, 0.0])
    n = O.clip_grad_norm_([p], 1.0)
    assert float(n) == pytest.approx(5.0) and float(p.grad.norm()) == pytest.approx(1.0, abs=1e-5)
    O.clip_grad_value_([p], 0.1)
    assert float(p.grad.abs().max()) <= 0.1 + 1e-7


def test_option_defaults_are_the_reference_table():
    """The default of every optimizer option and scheduler argument, pinned (the reference's option structs, torch/optim/*.h)."""
    import inspect
    from prometorch_b200 import optim as O
    want = {
        "SGD": dict(lr=0.01, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False),
        "Adam": dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, amsgrad=False),
        "AdamW": dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, amsgrad=False),
        "RMSprop": dict(lr=0.01, alpha=0.99, eps=1e-8, weight_decay=0.0, momentum=0.0, centered=False),
        "Lion": dict(lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0),
        "SophiaG": dict(lr=1e-4, betas=(0.965, 0.99), eps=1e-12, weight_decay=0.0, rho=0.04, hessian_update_interval=10),
        "LAMB": dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01, bias_correction=True),
        "Adafactor": dict(lr=0.0, eps1=1e-30, eps2=1e-3, clip_threshold=1.0, decay_rate=-0.8, beta1=0.0, weight_decay=0.0, scale_parameter=True,
                          relative_step=True, warmup_init=False),
        "NAdam": dict(lr=2e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, momentum_decay=0.004),
        "RAdam": dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0),
        "Adagrad": dict(lr=0.01, lr_decay=0.0, weight_decay=0.0, eps=1e-10, initial_accumulator_value=0.0),
        "Adadelta": dict(lr=1.0, rho=0.9, eps=1e-6, weight_decay=0.0),
        "Adamax": dict(lr=2e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0),
        "AdamKiller": dict(lr=1e-3, beta1_min=0.7, beta1_max=0.95, beta2=0.999, eps=1e-8, weight_decay=0.01, use_adaptive_momentum=True),
        "ASGD": dict(lr=0.01, lambd=1e-4, alpha=0.75, t0=1e6, weight_decay=0.0),
        "LBFGS": dict(lr=1.0, max_iter=20, max_eval=25, tolerance_grad=1e-7, tolerance_change=1e-9, history_size=100),
        "StepLR": dict(gamma=0.1), "MultiStepLR": dict(gamma=0.1), "CosineAnnealingLR": dict(eta_min=0.0),
        "LinearLR": dict(start_factor=1 / 3, end_factor=1.0, total_iters=5), "ConstantLR": dict(factor=1 / 3, total_iters=5),
        "ReduceLROnPlateau": dict(mode="min", factor=0.1, patience=10, threshold=1e-4, min_lr=0.0),
        "WarmupCosineAnnealingLR": dict(eta_min=0.0), "OneCycleLR": dict(pct_start=0.3, div_factor=25.0, final_div_factor=1e4),
        "CosineAnnealingWarmRestarts": dict(T_mult=1, eta_min=0.0), "CyclicLR": dict(step_size_up=2000, step_size_down=-1, mode="triangular", gamma=1.0),
        "PolynomialLR": dict(power=1.0),
    }
    bad = {}
    for name, defaults in want.items():
        sig = inspect.signature(getattr(O, name).__init__).parameters
        for k, v in defaults.items():
            got = sig[k].default if k in sig else "<missing>"
            same = (got == pytest.approx(v)) if isinstance(v, float) else (tuple(got) == v if isinstance(v, tuple) and got != "<missing>" else got == v)
            if not same:
                bad[f"{name}.{k}"] = (got, v)
    assert not bad, bad
    ema = O.EMA([torch.nn.Parameter(torch.ones(2))])
    assert ema.decay == 0.999 and all(hasattr(ema, m) for m in ("update", "apply_shadow", "restore", "set_decay"))
