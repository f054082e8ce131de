"""Fused multi-tensor optimizer kernels against the tensor-op form of the same rules."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from prometorch_b200 import optim as O

CASES = [
    (O.SGD, dict(lr=0.1, momentum=0.9, nesterov=True, weight_decay=0.01)),
    (O.SGD, dict(lr=0.1)),
    (O.Adam, dict(lr=1e-2, weight_decay=0.1, amsgrad=True)),
    (O.AdamW, dict(lr=1e-2, weight_decay=0.1)),
    (O.RMSprop, dict(lr=1e-2, momentum=0.5, centered=True)),
    (O.Lion, dict(lr=1e-3, weight_decay=0.1)),
    (O.SophiaG, dict(lr=1e-2, weight_decay=0.1)),
    (O.NAdam, dict(lr=2e-3, weight_decay=0.01)),
    (O.RAdam, dict(lr=1e-2)),
    (O.Adagrad, dict(lr=0.05, lr_decay=0.1)),
    (O.Adadelta, dict(lr=1.0, weight_decay=0.01)),
    (O.Adamax, dict(lr=2e-3)),
    (O.ASGD, dict(lr=0.05, t0=2)),
    (O.LAMB, dict(lr=1e-2, weight_decay=0.05)),
    (O.AdamKiller, dict(lr=1e-2, weight_decay=0.02, use_warm_restarts=True, restart_period=3)),
    (O.AdamKiller, dict(lr=5e-3, use_gradient_prediction=False, use_per_layer_lr=False, max_grad_norm=100.0)),
    (O.Adafactor, dict()),
    (O.Adafactor, dict(lr=1e-2, relative_step=False, scale_parameter=False, beta1=0.9, weight_decay=0.01, clip_threshold=0.5)),
]


def _params(dev, seed=0):
    g = torch.Generator().manual_seed(seed)
    shapes = [(300, 70), (70,), (5, 3, 7), (70001,), (1,)]
    return [torch.nn.Parameter(torch.randn(*s, generator=g).to(dev)) for s in shapes]


@pytest.mark.parametrize("cls,kw", CASES)
@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_fused_matches_tensor_ops(cls, kw, gdtype):
    a, b = _params("cuda"), _params("cuda")
    oa, ob = cls(a, fused=True, **kw), cls(b, fused=False, **kw)
    gen = torch.Generator().manual_seed(1)
    for step in range(7 if cls is not O.RAdam else 9):
        for p, q in zip(a, b):
            g = torch.randn(p.shape, generator=gen).to("cuda").to(gdtype)
            if gdtype == torch.float32:
                p.grad, q.grad = g.clone(), g.clone()
            else:       # .grad must have the parameter's dtype: bf16 gradients are registered on the side
                oa.set_grad_source(p, g.clone()); ob.set_grad_source(q, g.clone())
        oa.step(); ob.step()
    torch.cuda.synchronize()
    for p, q in zip(a, b):
        assert torch.allclose(p, q, atol=3e-6, rtol=2e-5), (cls.__name__, (p - q).abs().max())
    for p, q in zip(a, b):
        for k in oa.state[p]:
            if k not in ("step", "lamb_update", "ak_scratch", "af_scalars"):
                assert torch.allclose(oa.state[p][k], ob.state[q][k], atol=3e-6, rtol=2e-5), (cls.__name__, k)


def test_lowp_shadow_grad_scale_and_skip():
    a = _params("cuda")
    opt = O.AdamW(a, lr=1e-2, fused=True)
    shadows = [torch.zeros_like(p, dtype=torch.bfloat16) for p in a]
    for p, s in zip(a, shadows):
        opt.attach_lowp(p, s)
    opt.grad_scale = torch.tensor(0.5, device="cuda")
    opt.skip_flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = _params("cuda")
    oref = O.AdamW(ref, lr=1e-2, fused=False)
    for p, q in zip(a, ref):
        g = torch.randn_like(p)
        p.grad, q.grad = g.clone(), g * 0.5
    opt.step(); oref.step()
    for p, q, s in zip(a, ref, shadows):
        assert torch.allclose(p, q, atol=1e-6)
        assert torch.equal(s, p.detach().to(torch.bfloat16))
    before = [p.detach().clone() for p in a]
    opt.skip_flag.fill_(1)
    opt.step()
    for p, q in zip(a, before):
        assert torch.equal(p.detach(), q)


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_grad_norm_clip_and_inf(gdtype):
    ps = _params("cuda")
    if gdtype == torch.float32:
        for p in ps:
            p.grad = torch.randn_like(p)
    else:
        from prometorch_b200.optim.grad_utils import grads_as_params
        ps = grads_as_params([torch.randn_like(p).to(gdtype) for p in ps])
    ref = torch.linalg.vector_norm(torch.cat([p.grad.float().reshape(-1) for p in ps]))
    before = [p.grad.float().clone() for p in ps]
    n = O.clip_grad_norm_(ps, 1.0)
    assert torch.allclose(n, ref, rtol=1e-5)
    for p, g in zip(ps, before):
        tol = 1e-6 if gdtype == torch.float32 else 2e-2
        assert torch.allclose(p.grad.float(), g / (ref + 1e-6), atol=tol, rtol=tol)
    c = O.GradNormClipper(ps, 1.0)
    ps[2].grad[0, 0, 0] = float("inf")
    c.compute()
    assert int(c.found_inf) == 1
