"""Table-driven checks of the operator wrappers' plain-math paths (what answers for CPU tensors and what the GPU tests use as
their oracle): every op x shape x dtype x memory layout against an independent formulation, and gradients by numeric
differentiation in float64.  The reference generates such tests from a table of op specs (test/cpp/ops_spec.h)."""
import itertools
import math

import pytest
import torch
import torch.nn.functional as F

from prometorch_b200.ops import attention as A
from prometorch_b200.ops import fused_ops as O
from prometorch_b200.ops import gemm as G

TOL = {torch.float64: 1e-10, torch.float32: 2e-5, torch.bfloat16: 3e-2}


def rope_tables(T, D, base=10000.0):
    inv = base ** (-torch.arange(0, D // 2, dtype=torch.float64) / (D // 2))
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None]
    return ang.cos().float(), ang.sin().float()


def layouts(x):
    """The same values contiguous, as a transposed view made contiguous-in-values, and as a strided slice of a wider buffer."""
    yield "contiguous", x.contiguous()
    wide = torch.zeros(*x.shape[:-1], x.shape[-1] * 2, dtype=x.dtype)
    wide[..., ::2] = x
    yield "strided", wide[..., ::2]
    if x.dim() >= 2:
        yield "transposed", x.transpose(0, 1).contiguous().transpose(0, 1)


# ---------------------------------------------------------------------------------------------------------- references
def ref_rms(x, w, eps):
    x64 = x.double()
    return x64 / torch.sqrt((x64 * x64).mean(-1, keepdim=True) + eps) * w.double()


def ref_rope(x, cos, sin, neox, off):
    """Rotation written with complex numbers: pair (a, b) -> (a + ib) e^{i angle}."""
    B, T, H, D = x.shape
    x64 = x.double()
    ang = torch.atan2(sin[off:off + T].double(), cos[off:off + T].double())[None, :, None, :]
    if neox:
        z = torch.complex(x64[..., :D // 2], x64[..., D // 2:]) * torch.polar(torch.ones_like(ang), ang)
        return torch.cat([z.real, z.imag], -1)
    z = torch.complex(x64[..., 0::2], x64[..., 1::2]) * torch.polar(torch.ones_like(ang), ang)
    return torch.stack([z.real, z.imag], -1).flatten(-2)


def ref_attention(q, k, v, causal, q_offset, scale):
    B, Tq, H, D = q.shape
    Hk = k.shape[2]
    out = torch.zeros(B, Tq, H, D, dtype=torch.float64)
    for b, h in itertools.product(range(B), range(H)):
        kh = h // (H // Hk)
        for t in range(Tq):
            n = min(k.shape[1], t + q_offset + 1) if causal else k.shape[1]
            s = (k[b, :n, kh].double() @ q[b, t, h].double()) * scale
            out[b, t, h] = torch.softmax(s, 0) @ v[b, :n, kh].double()
    return out


SHAPES_2D = [(1, 8), (3, 64), (17, 96), (2, 5, 48), (4, 1, 256)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64], ids=str)
@pytest.mark.parametrize("shape", SHAPES_2D, ids=str)
def test_rms_norm_and_fused_add(shape, dtype):
    g = torch.Generator().manual_seed(len(shape) * 100 + shape[-1])
    x, r = torch.randn(*shape, generator=g).to(dtype), torch.randn(*shape, generator=g).to(dtype)
    w = torch.rand(shape[-1], generator=g).to(dtype) + 0.5
    for name, xv in layouts(x):
        y = O.rms_norm(xv, w, 1e-6)
        assert y.dtype == dtype and torch.allclose(y.double(), ref_rms(xv, w, 1e-6), atol=TOL[dtype], rtol=TOL[dtype]), name
        yn, h = O.add_rms_norm(xv, r, w, 1e-5)
        assert torch.allclose(h.double(), (xv + r).double(), atol=TOL[dtype]) and torch.allclose(yn.double(), ref_rms(xv + r, w, 1e-5), atol=TOL[dtype], rtol=TOL[dtype]), name


@pytest.mark.parametrize("neox", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=str)
@pytest.mark.parametrize("shape,off", [((1, 1, 1, 8), 0), ((2, 7, 3, 16), 0), ((1, 5, 2, 64), 11), ((3, 4, 1, 128), 2)], ids=str)
def test_rope_and_qkv_split(shape, off, dtype, neox):
    B, T, H, D = shape
    g = torch.Generator().manual_seed(D + T)
    cos, sin = rope_tables(T + off + 3, D)
    x = torch.randn(*shape, generator=g).to(dtype)
    for name, xv in layouts(x):
        y = O.rope(xv, cos, sin, neox, off)
        assert y.shape == x.shape and torch.allclose(y.double(), ref_rope(xv, cos, sin, neox, off), atol=4 * TOL[dtype], rtol=TOL[dtype]), name
    # a rotation keeps the length of every pair, and position 0 is the identity
    y = O.rope(x.float(), cos, sin, neox, 0)
    assert torch.allclose(y.pow(2).sum(-1), x.float().pow(2).sum(-1), rtol=1e-4, atol=1e-4) and torch.allclose(y[:, 0], x.float()[:, 0], atol=1e-6)
    Hk = max(1, H // 2)
    qkv = torch.randn(B, T, (H + 2 * Hk) * D, generator=g).to(dtype)
    q, k, v = O.qkv_rope_split(qkv, H, Hk, D, cos, sin, neox, off)
    parts = qkv.view(B, T, H + 2 * Hk, D)
    assert torch.allclose(q.double(), ref_rope(parts[:, :, :H], cos, sin, neox, off), atol=4 * TOL[dtype], rtol=TOL[dtype])
    assert torch.allclose(k.double(), ref_rope(parts[:, :, H:H + Hk], cos, sin, neox, off), atol=4 * TOL[dtype], rtol=TOL[dtype])
    assert torch.equal(v, parts[:, :, H + Hk:])


@pytest.mark.parametrize("gelu", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=str)
@pytest.mark.parametrize("shape", [(1, 2), (5, 32), (3, 7, 64), (2, 2, 2, 16)], ids=str)
def test_gated_activation(shape, dtype, gelu):
    g = torch.Generator().manual_seed(sum(shape))
    gu = (torch.randn(*shape, generator=g) * 2).to(dtype)
    a, b = gu.double()[..., :shape[-1] // 2], gu.double()[..., shape[-1] // 2:]
    want = (0.5 * a * (1 + torch.tanh(math.sqrt(2 / math.pi) * (a + 0.044715 * a ** 3))) if gelu else a / (1 + torch.exp(-a))) * b
    for name, v in layouts(gu):
        y = O.swiglu(v, gelu)
        assert y.shape == (*shape[:-1], shape[-1] // 2) and torch.allclose(y.double(), want, atol=4 * TOL[dtype], rtol=2 * TOL[dtype]), name


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=str)
@pytest.mark.parametrize("rows,vocab,ignored", [(1, 2, 0), (7, 33, 2), (64, 1000, 10), (5, 50257, 1)], ids=str)
def test_cross_entropy(rows, vocab, ignored, dtype):
    g = torch.Generator().manual_seed(rows + vocab)
    logits = (torch.randn(rows, vocab, generator=g) * 3).to(dtype)
    target = torch.randint(0, vocab, (rows,), generator=g)
    target[:ignored] = -100
    if ignored == rows:
        return
    keep = target != -100
    l64 = logits.double()
    want = (torch.logsumexp(l64[keep], -1) - l64[keep].gather(1, target[keep][:, None])[:, 0]).mean()
    got = O.cross_entropy(logits, target)
    assert abs(float(got) - float(want)) < 10 * TOL[torch.float32] * max(1.0, abs(float(want)))
    got3 = O.cross_entropy(logits.view(1, rows, vocab), target.view(1, rows))           # leading dimensions are flattened
    assert abs(float(got3) - float(got)) < 1e-6


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,Tq,Tk,H,Hk,D,off", [(1, 1, 1, 1, 1, 8, 0), (2, 5, 5, 4, 2, 16, 0), (1, 3, 9, 6, 1, 32, 6), (1, 8, 8, 2, 2, 64, 0)], ids=str)
def test_attention_reference_path(B, Tq, Tk, H, Hk, D, off, causal):
    g = torch.Generator().manual_seed(Tq * 31 + Tk)
    q, k, v = torch.randn(B, Tq, H, D, generator=g), torch.randn(B, Tk, Hk, D, generator=g), torch.randn(B, Tk, Hk, D, generator=g)
    scale = 1.0 / math.sqrt(D)
    o, lse = A.flash_attention(q, k, v, causal=causal, q_offset=off, return_lse=True)
    assert torch.allclose(o.double(), ref_attention(q, k, v, causal, off, scale), atol=1e-5)
    # the log-sum-exp is what a split-KV or ring merge needs: recombining two halves of the keys gives the same output
    if Tk >= 2 and not causal:
        h = Tk // 2
        o1, l1 = A.flash_attention(q, k[:, :h], v[:, :h], causal=False, return_lse=True)
        o2, l2 = A.flash_attention(q, k[:, h:], v[:, h:], causal=False, return_lse=True)
        w1, w2 = torch.exp(l1 - lse).permute(0, 2, 1)[..., None], torch.exp(l2 - lse).permute(0, 2, 1)[..., None]
        assert torch.allclose(o1 * w1 + o2 * w2, o, atol=1e-5)


@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (3, 16, 8), (2 * 5, 64, 24), (33, 130, 7)], ids=str)
def test_linear_family(m, k, n, bias):
    g = torch.Generator().manual_seed(m + k + n)
    x, w = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g)
    b = torch.randn(n, generator=g) if bias else None
    want = x.double() @ w.double().t() + (b.double() if bias else 0)
    for name, xv in layouts(x):
        assert torch.allclose(G.linear(xv, w, b).double(), want, atol=1e-4, rtol=1e-4), name
    assert torch.allclose(G.linear(x.view(1, m, k), w, b)[0].double(), want, atol=1e-4, rtol=1e-4)
    if n % 2 == 0:
        y = G.linear_swiglu(x, w)
        z = x.double() @ w.double().t()
        assert torch.allclose(y.double(), F.silu(z[:, :n // 2]) * z[:, n // 2:], atol=1e-4, rtol=1e-4)
    r, nw = torch.randn(m, n, generator=g), torch.rand(n, generator=g) + 0.5
    yn, h = G.linear_add_rms_norm(x, w, r, nw, 1e-6)
    hh = x.double() @ w.double().t() + r.double()
    assert torch.allclose(h.double(), hh, atol=1e-4, rtol=1e-4) and torch.allclose(yn.double(), ref_rms(hh, nw, 1e-6), atol=1e-4, rtol=1e-4)


def test_gradients_by_numeric_differentiation():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 8, dtype=torch.float64, generator=g, requires_grad=True)
    w = (torch.rand(8, dtype=torch.float64, generator=g) + 0.5).requires_grad_(True)
    assert torch.autograd.gradcheck(lambda a, b: O.rms_norm(a, b, 1e-6), (x, w), atol=1e-6)
    r = torch.randn(3, 8, dtype=torch.float64, generator=g, requires_grad=True)
    assert torch.autograd.gradcheck(lambda a, b, c: O.add_rms_norm(a, b, c, 1e-6), (x, r, w), atol=1e-6)
    cos, sin = rope_tables(6, 8)
    xr = torch.randn(2, 4, 2, 8, dtype=torch.float64, generator=g, requires_grad=True)
    for neox in (True, False):
        assert torch.autograd.gradcheck(lambda a: O.rope(a, cos.double(), sin.double(), neox, 1).double(), (xr,), atol=1e-5)
    gu = torch.randn(4, 10, dtype=torch.float64, generator=g, requires_grad=True)
    assert torch.autograd.gradcheck(lambda a: O.swiglu(a, False), (gu,), atol=1e-6) and torch.autograd.gradcheck(lambda a: O.swiglu(a, True), (gu,), atol=1e-6)
    q, k, v = (torch.randn(1, 4, 2, 8, dtype=torch.float64, generator=g, requires_grad=True) for _ in range(3))
    assert torch.autograd.gradcheck(lambda a, b, c: A.flash_attention(a, b, c, causal=True).double(), (q, k, v), atol=1e-4, eps=1e-4)
