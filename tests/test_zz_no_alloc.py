"""The allocation-free RMSNorm backward entry point (static device scratch) against the regular one.

Collected last on purpose (file name): it must pass on a device that other tests have already used,
and on its own."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from prometorch_b200 import _native as N
    from prometorch_b200.ops import fused_ops  # noqa: F401  (registers ptb_rmsnorm_bwd's prototype)
    L = N.lib()
    vp, ci, ll = C.c_void_p, C.c_int, C.c_longlong
    L.ptb_rmsnorm_bwd_static.argtypes = [vp, vp, vp, vp, vp, vp, ci, ll, ci, vp, ci, vp]
    L.ptb_rmsnorm_bwd_static.restype = ci
    return N, L


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_matches_regular_entry_point(dtype):
    N, L = _lib()
    dev = torch.device("cuda", 0)
    rows, H, n_ctas = 1000, 2560, 296
    st = torch.cuda.current_stream(dev).cuda_stream
    bf16 = int(dtype == torch.bfloat16)
    for call in range(2):                                   # two calls in a row share the static array
        g = torch.Generator(device="cpu").manual_seed(10 + call)
        x = torch.randn(rows, H, generator=g).to(dev, dtype)
        w = (1 + 0.1 * torch.randn(H, generator=g)).to(dev, dtype)
        dy = torch.randn(rows, H, generator=g).to(dev, dtype)
        dres = torch.randn(rows, H, generator=g).to(dev, dtype) if call else None
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
        dx_a, dw_a = torch.empty_like(x), torch.empty_like(w)
        dx_b, dw_b = torch.empty_like(x), torch.empty_like(w)
        part = torch.empty(n_ctas, H, dtype=torch.float32, device=dev)
        dres_p = dres.data_ptr() if dres is not None else None
        N.check(L.ptb_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx_a.data_ptr(), dw_a.data_ptr(),
                                  part.data_ptr(), n_ctas, rows, H, dres_p, bf16, st), "rmsnorm_bwd")
        N.check(L.ptb_rmsnorm_bwd_static(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx_b.data_ptr(), dw_b.data_ptr(),
                                         n_ctas, rows, H, dres_p, bf16, st), "rmsnorm_bwd_static")
        torch.cuda.synchronize()
        assert torch.equal(dx_a, dx_b) and torch.equal(dw_a, dw_b)
        # and both agree with plain fp32 math
        xf, wf, gf = x.float(), w.float(), dy.float()
        r = rstd[:, None]
        ref_dx = r * gf * wf - xf * (r ** 3) * (gf * wf * xf).sum(-1, keepdim=True) / H
        if dres is not None:
            ref_dx = ref_dx + dres.float()
        ref_dw = (gf * xf * r).sum(0)
        tol = 3e-2 if bf16 else 1e-4
        assert (dx_b.float() - ref_dx).abs().max() <= tol * ref_dx.abs().max()
        assert (dw_b.float() - ref_dw).abs().max() <= tol * ref_dw.abs().max()


def test_static_scratch_rejects_oversize():
    N, L = _lib()
    rc = L.ptb_rmsnorm_bwd_static(None, None, None, None, None, None, 1024, 4096, 2048, None, 1, None)   # 2 Mi floats > 1 Mi
    assert rc == -1
    assert b"exceeds the static scratch" in N.lib().ptb_last_error()
