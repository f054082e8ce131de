"""GPU numerics of the training kernels (GEMM, RMSNorm, RoPE, gated activation, cross-entropy) vs PyTorch fp32."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (300, 200, 136), (4096, 2048, 2048), (64, 96, 1000), (1000, 32000, 512)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_bf16(M, N, K, a_mn, b_mn):
    from prometorch_b200.ops.gemm import check_status, gemm_bf16
    if (a_mn and M % 8) or (b_mn and N % 8) or K % 8:
        pytest.skip("pitch must be a multiple of 8 elements")
    if M * N > 4e6 and (a_mn or b_mn):
        pytest.skip("large case covered in the K-major layout")
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    ref = A.float() @ B.float().t()
    out = gemm_bf16(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    check_status()
    assert out.shape == (M, N)
    assert _rel(out, ref) < 5e-3, _rel(out, ref)
    out32 = gemm_bf16(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert _rel(out32, ref) < 1e-4, _rel(out32, ref)


def test_gemm_epilogues():
    from prometorch_b200.ops.gemm import gemm_bf16
    A = torch.randn(200, 320, device="cuda").bfloat16()
    B = torch.randn(264, 320, device="cuda").bfloat16()
    bias = torch.randn(264, device="cuda")
    ref = A.float() @ B.float().t()
    assert _rel(gemm_bf16(A, B, bias=bias, out_dtype=torch.float32), ref + bias) < 1e-4
    acc = torch.ones(200, 264, device="cuda")
    gemm_bf16(A, B, out=acc, accumulate=True)
    assert _rel(acc, ref + 1) < 1e-4
    assert _rel(gemm_bf16(A, B, gelu=True, out_dtype=torch.float32), F.gelu(ref, approximate="tanh")) < 1e-3


def test_linear_autograd():
    from prometorch_b200.ops.gemm import linear
    x = torch.randn(4, 96, 256, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(512, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    b = torch.randn(512, device="cuda").bfloat16().requires_grad_()
    y = linear(x, w, b)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr, wr, br = x.detach().float().requires_grad_(), w.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    yr = F.linear(xr, wr, br)
    yr.backward(gy.float())
    assert _rel(y, yr) < 5e-3 and _rel(x.grad, xr.grad) < 5e-3 and _rel(w.grad, wr.grad) < 5e-3 and _rel(b.grad, br.grad) < 5e-3


@pytest.mark.parametrize("M,N,K", [(1, 2048, 2048), (3, 3072, 2048), (32, 2048, 5632), (64, 11264, 2048), (128, 512, 4096), (8, 32000, 2048),
                                   (33, 1000, 520), (17, 136, 64), (100, 2048, 2048)])
def test_gemm_skinny_split_k(M, N, K):
    """Decode-sized batches: the K dimension is split over the idle SMs and reduced by a second launch."""
    from prometorch_b200 import _native as NL
    from prometorch_b200.ops.gemm import check_status, gemm_bf16
    g = torch.Generator(device="cuda").manual_seed(M * 3 + N + K)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    bias = torch.randn(N, device="cuda", generator=g)
    ref = A.float() @ B.float().t()
    out = gemm_bf16(A, B)
    torch.cuda.synchronize()
    check_status()
    assert _rel(out, ref) < 5e-3, _rel(out, ref)
    assert _rel(gemm_bf16(A, B, bias=bias), ref + bias) < 5e-3
    assert _rel(gemm_bf16(A, B, bias=bias, gelu=True), F.gelu(ref + bias, approximate="tanh")) < 8e-3
    splits = NL.lib().ptb_gemm_pick_splits(M, N, K, 148)
    assert 0 <= splits <= 16
    if M <= 64:
        assert splits >= 1                      # decode-sized batches always take the swapped-operand path


@pytest.mark.parametrize("M,N,K", [(1, 2048, 2048), (32, 2048, 5632), (8, 4096, 4096), (128, 512, 1024)])
def test_skinny_linear_add_rms_norm(M, N, K):
    from prometorch_b200.ops.gemm import check_status, linear_add_rms_norm
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * K ** -0.5).bfloat16()
    resid = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    nw = (1 + 0.1 * torch.randn(N, device="cuda", generator=g)).bfloat16()
    with torch.no_grad():
        y, h = linear_add_rms_norm(x, w, resid, nw, 1e-5)
    torch.cuda.synchronize()
    check_status()
    h_ref = x.float() @ w.float().t() + resid.float()
    y_ref = h_ref * torch.rsqrt(h_ref.pow(2).mean(-1, keepdim=True) + 1e-5) * nw.float()
    assert _rel(h, h_ref) < 5e-3 and _rel(y, y_ref) < 8e-3, (_rel(h, h_ref), _rel(y, y_ref))


@pytest.mark.parametrize("M,I,K,gelu", [(1, 5632, 2048, False), (32, 5632, 2048, False), (16, 1024, 512, True), (128, 11008, 4096, False)])
def test_skinny_linear_swiglu(M, I, K, gelu):
    from prometorch_b200.ops.gemm import check_status, linear_swiglu
    g = torch.Generator(device="cuda").manual_seed(M + I + K)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(2 * I, K, device="cuda", generator=g) * K ** -0.5).bfloat16()
    with torch.no_grad():
        out = linear_swiglu(x, w, gelu)
    torch.cuda.synchronize()
    check_status()
    gu = x.float() @ w.float().t()
    act = F.gelu(gu[:, :I], approximate="tanh") if gelu else F.silu(gu[:, :I])
    assert out.shape == (M, I) and _rel(out, act * gu[:, I:]) < 8e-3, _rel(out, act * gu[:, I:])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("H", [384, 2048, 2560, 4096])
def test_rmsnorm(dtype, H):
    from prometorch_b200.ops.fused_ops import add_rms_norm, rms_norm
    x = torch.randn(3, 37, H, device="cuda").to(dtype).requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(dtype).requires_grad_()
    y = rms_norm(x, w, 1e-6)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    yr.backward(gy.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert _rel(y, yr) < tol and _rel(x.grad, xr.grad) < tol and _rel(w.grad, wr.grad) < tol
    # fused residual add
    r = torch.randn_like(x).detach().requires_grad_()
    x2 = x.detach().clone().requires_grad_()
    yn, h = add_rms_norm(x2, r, w.detach(), 1e-6)
    (yn.float().sum() + 2 * h.float().sum()).backward()
    xr2, rr = x2.detach().float().requires_grad_(), r.detach().float().requires_grad_()
    hr = xr2 + rr
    ynr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * w.detach().float()
    (ynr.sum() + 2 * hr.sum()).backward()
    assert _rel(h, hr) < tol and _rel(yn, ynr) < tol and _rel(x2.grad, xr2.grad) < tol and _rel(r.grad, rr.grad) < tol


@pytest.mark.parametrize("neox", [True, False])
def test_rope(neox):
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.models.gguf_oracle import apply_rope, rope_tables
    from prometorch_b200.ops.fused_ops import rope
    cos, sin = rope_tables(tiny_qwen3_config(), 64, "cuda")
    x = torch.randn(2, 48, 6, 128, device="cuda").bfloat16().requires_grad_()
    y = rope(x, cos, sin, neox)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr = x.detach().float().requires_grad_()
    yr = torch.stack([apply_rope(xr[b], cos[:48], sin[:48], neox) for b in range(2)])
    yr.backward(gy.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2


@pytest.mark.parametrize("neox,H,Hk,D,off", [(True, 8, 2, 128, 0), (False, 6, 6, 64, 3), (True, 4, 1, 64, 5)])
def test_qkv_rope_split(neox, H, Hk, D, off):
    """The fused split + rotary kernel against rope() on the three slices, forward and backward."""
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.models.gguf_oracle import apply_rope, rope_tables
    from prometorch_b200.ops.fused_ops import qkv_rope_split
    cfg = tiny_qwen3_config(head_dim=D)
    cos, sin = rope_tables(cfg, 64, "cuda")
    B, T = 2, 40
    qkv = torch.randn(B, T, (H + 2 * Hk) * D, device="cuda").bfloat16().requires_grad_()
    q, k, v = qkv_rope_split(qkv, H, Hk, D, cos, sin, neox, off)
    gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    r = qkv.detach().float().requires_grad_()
    x = r.view(B, T, H + 2 * Hk, D)
    c, s_ = cos[off:off + T], sin[off:off + T]
    qr = torch.stack([apply_rope(x[b, :, :H], c, s_, neox) for b in range(B)])
    kr = torch.stack([apply_rope(x[b, :, H:H + Hk], c, s_, neox) for b in range(B)])
    vr = x[:, :, H + Hk:]
    torch.autograd.backward([qr, kr, vr], [gq.float(), gk.float(), gv.float()])
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    assert _rel(q, qr) < 1e-2 and _rel(k, kr) < 1e-2 and torch.equal(v.float(), vr.detach().to(torch.bfloat16).float())
    assert _rel(qkv.grad, r.grad) < 1e-2


@pytest.mark.parametrize("gelu", [False, True])
def test_swiglu(gelu):
    from prometorch_b200.ops.fused_ops import swiglu
    gu = torch.randn(5, 33, 2 * 1408, device="cuda").bfloat16().requires_grad_()
    y = swiglu(gu, gelu)
    gy = torch.randn_like(y)
    y.backward(gy)
    r = gu.detach().float().requires_grad_()
    g, u = r.chunk(2, -1)
    yr = (F.gelu(g, approximate="tanh") if gelu else F.silu(g)) * u
    yr.backward(gy.float())
    assert _rel(y, yr) < 1e-2 and _rel(gu.grad, r.grad) < 1.5e-2


@pytest.mark.parametrize("V,dtype", [(65, torch.float32), (32000, torch.bfloat16), (1000, torch.float32), (151936, torch.bfloat16)])
def test_cross_entropy(V, dtype):
    from prometorch_b200.ops.fused_ops import cross_entropy
    rows = 64
    Vp = (V + 7) // 8 * 8
    buf = torch.randn(rows, Vp, device="cuda").to(dtype) * 3
    logits = buf[:, :V].detach().requires_grad_()
    tgt = torch.randint(0, V, (rows,), device="cuda")
    tgt[5] = -100
    loss = cross_entropy(logits, tgt)
    loss.backward()
    lr = logits.detach().float().requires_grad_()
    ref = F.cross_entropy(lr, tgt, ignore_index=-100)
    ref.backward()
    assert abs(float(loss) - float(ref)) < (2e-2 if dtype == torch.bfloat16 else 1e-4) * max(1.0, abs(float(ref)))
    assert _rel(logits.grad, lr.grad) < (2e-2 if dtype == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("B,T,H,Hk,D,causal", [(2, 256, 6, 6, 64, True), (1, 300, 8, 2, 128, True), (2, 128, 4, 1, 128, False),
                                               (1, 1000, 4, 4, 64, True), (1, 64, 32, 4, 64, True)])
def test_flash_attention(B, T, H, Hk, D, causal):
    from prometorch_b200.ops.attention import attention_reference, flash_attention
    g = torch.Generator(device="cuda").manual_seed(T + H)
    q = torch.randn(B, T, H, D, device="cuda", generator=g).bfloat16().requires_grad_()
    k = torch.randn(B, T, Hk, D, device="cuda", generator=g).bfloat16().requires_grad_()
    v = torch.randn(B, T, Hk, D, device="cuda", generator=g).bfloat16().requires_grad_()
    o, lse = flash_attention(q, k, v, causal=causal, return_lse=True)
    go = torch.randn_like(o)
    o.backward(go)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf, lser = attention_reference(qr, kr, vr, causal)
    orf.backward(go.float())
    assert _rel(o, orf) < 1e-2, _rel(o, orf)
    assert torch.allclose(lse, lser, atol=2e-2, rtol=1e-3)
    assert _rel(q.grad, qr.grad) < 2e-2, _rel(q.grad, qr.grad)
    assert _rel(k.grad, kr.grad) < 2e-2, _rel(k.grad, kr.grad)
    assert _rel(v.grad, vr.grad) < 2e-2, _rel(v.grad, vr.grad)


def test_llama_tiny_forward_backward():
    from prometorch_b200.models.llama import Llama, LlamaConfig
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(hidden_size=256, num_heads=4, num_kv_heads=2, intermediate_size=512, vocab_size=1024, max_seq=256)
    m = Llama(cfg).cuda().bfloat16()
    ref = Llama(cfg).float()
    ref.load_state_dict({k: v.float().cpu() for k, v in m.state_dict().items()})
    tok = torch.randint(0, 1024, (2, 129))
    loss = m(tok[:, :-1].cuda(), tok[:, 1:].cuda())
    loss.backward()
    lr = ref(tok[:, :-1], tok[:, 1:])
    lr.backward()
    assert abs(float(loss) - float(lr)) < 0.05 * float(lr)
    gm, gr = m.blocks[0].mlp.down.weight.grad.float().cpu(), ref.blocks[0].mlp.down.weight.grad
    assert _rel(gm, gr) < 0.1, _rel(gm, gr)


@pytest.mark.parametrize("B,T,D,dtype", [(2, 300, 96, torch.float32), (1, 4096, 256, torch.float32), (3, 64, 130, torch.bfloat16),
                                         (2, 1000, 512, torch.bfloat16), (4, 1, 32, torch.float32)])
def test_linear_scan_fwd_bwd(B, T, D, dtype):
    """Chunked gated linear recurrence on the GPU against the step-by-step fp32 loop, forward and both gradients."""
    from prometorch_b200.ops.scan import linear_scan, linear_scan_reference
    g0 = torch.Generator(device="cuda").manual_seed(B * 7 + T + D)
    g = (0.5 + 0.5 * torch.rand(B, T, D, device="cuda", generator=g0)).to(dtype)
    x = torch.randn(B, T, D, device="cuda", generator=g0).to(dtype)
    w = torch.randn(B, T, D, device="cuda", generator=g0)
    ga, xa = g.clone().requires_grad_(), x.clone().requires_grad_()
    h = linear_scan(ga, xa)
    (h.float() * w).sum().backward()
    gr, xr = g.float().clone().requires_grad_(), x.float().clone().requires_grad_()
    hr = linear_scan_reference(gr, xr)
    (hr * w).sum().backward()
    torch.cuda.synchronize()
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-4
    assert h.dtype == dtype and _rel(h, hr) < tol, _rel(h, hr)
    assert _rel(xa.grad, xr.grad) < tol and _rel(ga.grad, gr.grad) < tol, (_rel(xa.grad, xr.grad), _rel(ga.grad, gr.grad))
