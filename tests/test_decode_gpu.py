"""GPU numerics of the decode kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from prometorch_b200.io import gguf_quant as Q
from prometorch_b200.io.config import tiny_qwen3_config
from prometorch_b200.io.synthetic import write_synthetic_gguf


def _packed(rows, cols, qt, seed=0, layout=None):
    from prometorch_b200.io.gguf_model import pack_weight
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(rows, cols, device="cuda", generator=g) * 0.02
    raw = Q.quantize(w, qt)
    wd = Q.dequantize(raw, qt, cols)
    return pack_weight(raw, qt, cols, "cuda", layout=layout), wd


def _rel(a, b):
    return float((a - b).norm() / b.norm())


@pytest.mark.parametrize("layout", [0, 1], ids=["segment-dp4a", "tile16-mma"])
@pytest.mark.parametrize("qt", [Q.GGMLType.Q4_K, Q.GGMLType.Q6_K])
@pytest.mark.parametrize("rows,cols", [(4096, 2560), (2560, 9728), (1024, 2560), (2560, 4096), (300, 512), (7, 256)])
def test_gemv_matches_fp32(qt, rows, cols, layout):
    from prometorch_b200.ops.quant_gemv import quant_gemv
    pw, wd = _packed(rows, cols, qt, seed=rows + cols, layout=layout)
    x = torch.randn(cols, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rows * 7 + cols))
    y = quant_gemv(pw, x)
    torch.cuda.synchronize()
    ref_q8 = wd @ Q.quantize_activation_q8(x)        # same activation rounding as the kernel
    ref = wd @ x
    # one int8 step on a single activation (x * (127 / amax) against x / (amax / 127) at a rounding boundary) moves the
    # result by ~3e-4 of its norm at these sizes; anything systematic is orders of magnitude above that
    assert _rel(y, ref_q8) < 8e-4, _rel(y, ref_q8)
    assert _rel(y, ref) < 2e-2, _rel(y, ref)


@pytest.mark.parametrize("qt", [Q.GGMLType.Q5_K, Q.GGMLType.Q8_0, Q.GGMLType.F16], ids=["q5_k", "q8_0", "f16"])
@pytest.mark.parametrize("rows,cols", [(4096, 2560), (2560, 9728), (300, 512), (7, 256)])
def test_gemv_native_q5k_q8_0_f16(qt, rows, cols):
    """Q5_K, Q8_0 and fp16 matrices are streamed as they are (16-row tile layout), not transcoded."""
    from prometorch_b200.io.gguf_model import QT_F16, QT_Q5K, QT_Q8_0
    from prometorch_b200.ops.quant_gemv import quant_gemv
    pw, wd = _packed(rows, cols, qt, seed=rows + cols, layout=1)
    assert pw.qtype == {Q.GGMLType.Q5_K: QT_Q5K, Q.GGMLType.Q8_0: QT_Q8_0, Q.GGMLType.F16: QT_F16}[qt]
    x = torch.randn(cols, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rows * 7 + cols))
    y = quant_gemv(pw, x)
    torch.cuda.synchronize()
    ref_q8 = wd.float() @ Q.quantize_activation_q8(x)
    assert _rel(y, ref_q8) < 8e-4, _rel(y, ref_q8)
    # the gated pair and the prompt path's dequantisation read the same layout
    pw2, wd2 = _packed(rows, cols, qt, seed=rows + cols + 1, layout=1)
    y = quant_gemv(pw, x, w2=pw2)
    xq = Q.quantize_activation_q8(x)
    assert _rel(y, torch.nn.functional.silu(wd.float() @ xq) * (wd2.float() @ xq)) < 2e-3
    from prometorch_b200 import _native as N
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
    N.check(N.lib().ptb_dequant_weight(pw.data.data_ptr(), pw.qtype, pw.layout, rows, cols, out.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream), "dequant")
    torch.cuda.synchronize()
    assert torch.equal(out, wd.to(torch.bfloat16))


def test_gemv_norm_resid_gated_argmax():
    from prometorch_b200.ops.quant_gemv import quant_gemv
    cols, rows = 2560, 1536
    pw, wd = _packed(rows, cols, Q.GGMLType.Q4_K, 1)
    pw2, wd2 = _packed(rows, cols, Q.GGMLType.Q4_K, 2)
    x = torch.randn(cols, device="cuda") * 3
    nw = 1 + 0.1 * torch.randn(cols, device="cuda")
    xn = x * torch.rsqrt(x.pow(2).mean() + 1e-6) * nw
    xq = Q.quantize_activation_q8(xn)
    y = quant_gemv(pw, x, norm_weight=nw)
    assert _rel(y, wd @ xq) < 2e-4
    r = torch.randn(rows, device="cuda")
    y = quant_gemv(pw, x, norm_weight=nw, resid=r)
    assert _rel(y, r + wd @ xq) < 2e-4
    y = quant_gemv(pw, x, norm_weight=nw, w2=pw2)
    assert _rel(y, torch.nn.functional.silu(wd @ xq) * (wd2 @ xq)) < 5e-4
    y, idx = quant_gemv(pw, x, norm_weight=nw, argmax=True)
    torch.cuda.synchronize()
    assert int(idx) == int(y.argmax()) == int((wd @ xq).argmax())


@pytest.mark.parametrize("pos", [0, 5, 127, 128, 300, 1023])
@pytest.mark.parametrize("neox", [True, False])
@pytest.mark.parametrize("d,H,KV", [(128, 8, 2), (64, 8, 8), (64, 4, 2), (256, 8, 4), (256, 8, 1)])
def test_attn_decode(pos, neox, d, H, KV):
    from prometorch_b200.models.gguf_oracle import apply_rope, rms_norm, rope_tables
    from prometorch_b200.ops.quant_gemv import attn_decode
    cfg = tiny_qwen3_config(head_dim=d)
    S = 1024
    cos, sin = rope_tables(cfg, S, "cuda")
    torch.manual_seed(pos)
    kc = (torch.randn(KV, S, d, device="cuda") * 0.5).half()
    vc = (torch.randn(KV, S, d, device="cuda") * 0.5).half()
    q, k, v = torch.randn(H * d, device="cuda"), torch.randn(KV * d, device="cuda"), torch.randn(KV * d, device="cuda")
    qn, kn = 1 + 0.1 * torch.randn(d, device="cuda"), 1 + 0.1 * torch.randn(d, device="cuda")
    kc2, vc2 = kc.clone(), vc.clone()
    out = attn_decode(q, k, v, kc2, vc2, pos, cos, sin, q_norm=qn, k_norm=kn, neox=neox)
    torch.cuda.synchronize()
    # reference
    qh = apply_rope(rms_norm(q.view(1, H, d), qn, 1e-6), cos[pos:pos + 1], sin[pos:pos + 1], neox)[0]
    kh = apply_rope(rms_norm(k.view(1, KV, d), kn, 1e-6), cos[pos:pos + 1], sin[pos:pos + 1], neox)[0]
    K = kc.float().clone()
    V = vc.float().clone()
    K[:, pos] = kh.half().float()
    V[:, pos] = v.view(KV, d).half().float()
    K, V = K[:, :pos + 1], V[:, :pos + 1]
    g = H // KV
    sc = torch.einsum("hd,hsd->hs", qh, K.repeat_interleave(g, 0)) / math.sqrt(d)
    ref = torch.einsum("hs,hsd->hd", sc.softmax(-1), V.repeat_interleave(g, 0)).reshape(-1)
    assert torch.allclose(kc2[:, pos].float(), K[:, pos], atol=2e-3)
    assert _rel(out, ref) < 2e-3, _rel(out, ref)


@pytest.fixture(scope="module")
def tiny_model(tmp_path_factory):
    cfg = tiny_qwen3_config(layers=3, hidden=512, heads=8, kv_heads=2, inter=1024, vocab=1000)
    p = str(tmp_path_factory.mktemp("m") / "tiny.gguf")
    write_synthetic_gguf(p, cfg, seed=11, device="cuda", std=0.05)
    return p


def test_engine_matches_oracle(tiny_model):
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.models.gguf_oracle import OracleModel
    m = GGUFModel(tiny_model, max_seq=512, want_logits=True)
    o = OracleModel(tiny_model, device="cuda", max_seq=512, emulate_q8=True)
    toks = [3, 77, 500, 999, 12, 64, 5, 5, 901]
    for pos, t in enumerate(toks):
        nxt = m.forward_decode(t, pos)
        lg = m.logits_view().clone()
        ref = o.forward([t])[0]
        cos = torch.nn.functional.cosine_similarity(lg, ref, dim=0)
        assert cos > 0.9995, (pos, float(cos))
        assert nxt == int(lg.argmax())
    m.check_status()
    m.close()


@pytest.mark.parametrize("head_dim,heads,kv", [(64, 8, 4), (256, 4, 2)])
def test_engine_other_head_sizes(tmp_path, head_dim, heads, kv):
    """Head sizes 64 and 256 (small llamas, gemma) through the whole engine against the fp32 oracle."""
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.models.gguf_oracle import OracleModel
    cfg = tiny_qwen3_config(layers=2, hidden=512, heads=heads, kv_heads=kv, inter=1024, vocab=1000, head_dim=head_dim)
    p = str(tmp_path / "hd.gguf")
    write_synthetic_gguf(p, cfg, seed=5, device="cuda", std=0.05)
    m = GGUFModel(p, max_seq=512, want_logits=True)
    o = OracleModel(p, device="cuda", max_seq=512, emulate_q8=True)
    for pos, t in enumerate([3, 77, 500, 999, 12, 64]):
        nxt = m.forward_decode(t, pos)
        lg = m.logits_view().clone()
        ref = o.forward([t])[0]
        cos = torch.nn.functional.cosine_similarity(lg, ref, dim=0)
        assert cos > 0.9995, (pos, float(cos))
        assert nxt == int(lg.argmax())
    m.check_status()
    m.close()


@pytest.mark.parametrize("q_main,q_more", [(Q.GGMLType.Q5_K, Q.GGMLType.Q8_0), (Q.GGMLType.Q8_0, Q.GGMLType.F16)],
                         ids=["q5k+q8_0", "q8_0+f16"])
def test_engine_other_weight_types(tmp_path, q_main, q_more):
    """Files whose matrices are Q5_K / Q8_0 / F16 decode from those bytes and agree with the fp32 oracle."""
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.models.gguf_oracle import OracleModel
    cfg = tiny_qwen3_config(layers=2, hidden=512, heads=8, kv_heads=2, inter=1024, vocab=1000)
    p = str(tmp_path / "wt.gguf")
    write_synthetic_gguf(p, cfg, seed=6, device="cuda", std=0.05, q_main=q_main, q_more=q_more)
    m = GGUFModel(p, max_seq=512, want_logits=True)
    o = OracleModel(p, device="cuda", max_seq=512, emulate_q8=True)
    for pos, t in enumerate([3, 77, 500, 999, 12, 64]):
        nxt = m.forward_decode(t, pos)
        lg = m.logits_view().clone()
        ref = o.forward([t])[0]
        cos = torch.nn.functional.cosine_similarity(lg, ref, dim=0)
        assert cos > 0.9995, (pos, float(cos))
        assert nxt == int(lg.argmax())
    m.check_status()
    m.close()


def test_engine_merged_qkv_gate_up_longrope(tmp_path):
    """phi-3 style file: Q/K/V and gate/up merged, LongRoPE factors; the engine shards the merged tensors by rows."""
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.models.gguf_oracle import OracleModel
    cfg = tiny_qwen3_config(layers=2, hidden=512, heads=8, kv_heads=2, inter=1024, vocab=1000)
    p = str(tmp_path / "phi.gguf")
    write_synthetic_gguf(p, cfg, seed=8, device="cuda", std=0.05, merged=True,
                         rope_factors=([1.0 + 0.02 * i for i in range(64)], [3.0] * 64), rope_orig_ctx=4096)
    m = GGUFModel(p, max_seq=512, want_logits=True)
    o = OracleModel(p, device="cuda", max_seq=512, emulate_q8=True)
    for pos, t in enumerate([3, 77, 500, 999, 12, 64]):
        nxt = m.forward_decode(t, pos)
        lg = m.logits_view().clone()
        cos = torch.nn.functional.cosine_similarity(lg, o.forward([t])[0], dim=0)
        assert cos > 0.9995, (pos, float(cos))
        assert nxt == int(lg.argmax())
    m.check_status()
    m.close()


def test_engine_scripted_equals_stepped(tiny_model):
    from prometorch_b200.io.gguf_model import GGUFModel
    m = GGUFModel(tiny_model, max_seq=512)
    prompt = [9, 8, 7, 600, 5]
    a = m.run_script(prompt, 20)
    # stepped, host-fed
    seq = list(prompt)
    out = []
    for pos in range(len(prompt) + 19):
        nxt = m.forward_decode(seq[pos], pos)
        if pos >= len(prompt) - 1:
            out.append(nxt)
            seq.append(nxt)
    assert a == out
    b = m.generate(prompt, 20)
    assert a == b
    m.close()


# ----------------------------------------------------------------------------- device sampler
@pytest.mark.parametrize("V,top_k,top_p,temp,pen", [(151936, 40, 0.9, 0.7, 1.1), (32000, 64, 1.0, 1.3, 1.0), (1000, 5, 0.5, 0.2, 1.3),
                                                    (4096, 1, 0.9, 0.8, 1.0), (151936, 40, 0.9, 0.0, 1.2)])
def test_device_sampler_matches_oracle(V, top_k, top_p, temp, pen):
    from prometorch_b200.ops.sampling import DeviceSampler, sample_reference
    torch.manual_seed(V + top_k)
    dev = torch.device("cuda", 0)
    samp = DeviceSampler(V, dev, seed=1)
    hist = torch.randint(0, V, (300,)).tolist()
    samp.reset(hist)
    for trial in range(6):
        logits = (torch.randn(V) * 3).to(dev)
        logits[hist[trial]] += 12.0                       # a history token at the top: the penalty matters
        u = [0.0, 0.13, 0.5, 0.77, 0.95, 0.9999][trial]
        got = samp.sample(logits, temp, top_k, top_p, pen, u=u)
        want = sample_reference(logits, temp, top_k, top_p, pen, hist, u)
        assert got == want, (trial, got, want)
        hist.append(got)                                  # the kernel appended its choice to the device history


def test_device_sampler_distribution():
    from prometorch_b200.ops.sampling import DeviceSampler
    dev = torch.device("cuda", 0)
    V = 5000
    logits = torch.full((V,), -20.0, device=dev)
    logits[[7, 99, 4000]] = torch.tensor([2.0, 1.0, 0.0], device=dev)
    samp = DeviceSampler(V, dev, seed=3)
    counts = {}
    for _ in range(600):
        t = samp.sample(logits, 1.0, 3, 1.0)
        counts[t] = counts.get(t, 0) + 1
    p = torch.softmax(torch.tensor([2.0, 1.0, 0.0]), 0)
    assert set(counts) <= {7, 99, 4000}
    for tid, pi in zip([7, 99, 4000], p.tolist()):
        assert abs(counts.get(tid, 0) / 600 - pi) < 0.07


# ----------------------------------------------------------------------------- batched prompt pass
def test_dequant_segmajor_matches_oracle(tmp_path):
    from prometorch_b200 import _native as N
    from prometorch_b200.io.gguf import GGMLType
    from prometorch_b200.io.gguf_model import pack_weight
    from prometorch_b200.io.gguf_quant import dequantize, quantize
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    for qt, cols in ((GGMLType.Q4_K, 2560), (GGMLType.Q6_K, 9728), (GGMLType.Q4_K, 4096)):
        w = torch.randn(70, cols) * 0.05
        raw = quantize(w, qt)
        ref = dequantize(raw, qt, cols).to(dev)
        pw = pack_weight(raw.view(70, -1), qt, cols, dev)
        out = torch.empty(70, cols, dtype=torch.bfloat16, device=dev)
        N.check(N.lib().ptb_dequant_weight(pw.data.data_ptr(), pw.qtype, pw.layout, 70, cols, out.data_ptr(), torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert torch.equal(out, ref.to(torch.bfloat16))


def test_prefill_matches_token_by_token(tmp_path):
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    cfg = tiny_qwen3_config(layers=3, hidden=1024, heads=16, kv_heads=8, inter=2048, vocab=2048)
    path = str(tmp_path / "pf.gguf")
    write_synthetic_gguf(path, cfg, seed=11, device="cuda", std=0.05)
    a = GGUFModel(path, max_seq=512, want_logits=True)
    b = GGUFModel(path, max_seq=512, want_logits=True)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 2048, (150,), generator=g).tolist()
    assert a.supports_prefill
    a.prefill(prompt[:100])                      # first part in one pass
    a.prefill(prompt[100:-1], pos0=100)          # continuation on top of the cache
    ta = a.forward_decode(prompt[-1], len(prompt) - 1)
    for pos, t in enumerate(prompt):             # reference: one decode step per prompt token
        tb = b.forward_decode(t, pos)
    la, lb = a.logits_view().float(), b.logits_view().float()
    cos = float(torch.nn.functional.cosine_similarity(la, lb, dim=0))
    assert cos > 0.995, cos
    assert ta == tb or float(lb[ta]) > float(lb.max()) - 0.05 * float(lb.abs().max())
    # generation after a batched prefill continues coherently
    out = a.generate(prompt, 8)
    assert len(out) == 8
    a.close()
    b.close()


# ----------------------------------------------------------------------------- gemma3 structure (post-norms, GELU gate, tied + scaled embeddings)
@pytest.mark.parametrize("window", [0, 64])
def test_gemma3_structure_matches_oracle(tmp_path, window):
    from prometorch_b200.io.config import tiny_gemma3_config
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.models.gguf_oracle import OracleModel
    cfg = tiny_gemma3_config(layers=7, window=window)
    path = str(tmp_path / "g3.gguf")
    write_synthetic_gguf(path, cfg, seed=5, device="cuda", std=0.05)
    m = GGUFModel(path, max_seq=256, want_logits=True)
    assert m.cfg.has_post_norm and m.cfg.ffn_gelu and m.cfg.scale_embeddings
    o = OracleModel(path, device="cuda", max_seq=256, emulate_q8=True)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, 2048, (90 if window else 12,), generator=g).tolist()
    for pos, t in enumerate(toks):
        nxt = m.forward_decode(t, pos)
        ref = o.forward([t])[0]
        if pos % 8 == 0 or pos == len(toks) - 1:
            cos = torch.nn.functional.cosine_similarity(m.logits_view(), ref, dim=0)
            assert cos > 0.999, (pos, float(cos))
    hid = m.hidden_view().clone()
    assert torch.isfinite(hid).all()
    m.check_status()
    if not window:                                # batched prompt pass with post-norms
        m2 = GGUFModel(path, max_seq=256, want_logits=True)
        m2.prefill(toks[:-1])
        m2.forward_decode(toks[-1], len(toks) - 1)
        cos = torch.nn.functional.cosine_similarity(m2.logits_view(), m.logits_view(), dim=0)
        assert cos > 0.995, float(cos)
        m2.close()
    m.close()


def test_batched_sampler_matches_single_request_sampler():
    """``sample_batch`` (grid row per request) picks what each request's own ``DeviceSampler.sample`` picks."""
    from prometorch_b200.ops.sampling import DeviceSampler, sample_batch
    V, n = 5000, 6
    torch.manual_seed(3)
    logits = (torch.randn(n, V, device="cuda") * 3).contiguous()
    hists = [[int(x) for x in torch.randint(0, V, (k,))] for k in (0, 3, 40, 7, 1, 100)]
    cfgs = [(0.8, 40, 0.9, 1.1), (0.0, 1, 1.0, 1.0), (1.3, 64, 0.5, 1.3), (0.7, 5, 1.0, 1.0), (0.0, 8, 0.9, 1.2), (1.0, 50, 0.95, 1.05)]
    a = [DeviceSampler(V, "cuda", max_history=256, seed=10 + i) for i in range(n)]
    b = [DeviceSampler(V, "cuda", max_history=256, seed=10 + i) for i in range(n)]
    for s, t, h in zip(a, b, hists):
        s.reset(h)
        t.reset(h)
    for rnd in range(3):
        got = sample_batch(a, logits, cfgs)
        want = [t.sample(logits[i].contiguous(), *cfgs[i][:3], cfgs[i][3]) for i, t in enumerate(b)]
        assert got == want, (rnd, got, want)
        assert all(0 <= g < V for g in got)
    assert [s.n_hist for s in a] == [t.n_hist for t in b] and all(torch.equal(s.hist[:s.n_hist], t.hist[:t.n_hist]) for s, t in zip(a, b))


@pytest.mark.parametrize("q_main,q_more", [(Q.GGMLType.Q4_K, Q.GGMLType.Q6_K), (Q.GGMLType.Q5_K, Q.GGMLType.Q8_0),
                                           (Q.GGMLType.Q8_0, Q.GGMLType.F16)], ids=["q4_k_m", "q5k+q8_0", "q8_0+f16"])
def test_cpp_gguf_model_generates_the_same_ids(tmp_path, q_main, q_more):
    """promethorch/gguf.h (C++ reader, repack of every streamed weight type, engine driver) against the Python GGUFModel
    on the same file."""
    import os
    import shutil
    import subprocess
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    if shutil.which("g++") is None:
        pytest.skip("needs g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = os.path.join(root, "prometorch_b200", "lib")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = str(tmp_path / "gguf_generate")
    cmd = ["g++", "-std=c++17", "-O1", os.path.join(root, "tests", "cpp", "gguf_generate.cpp"), "-o", exe,
           f"-I{root}/prometorch_b200/cpp_api", f"-I{cuda}/include", f"-L{lib}", "-lptb200", f"-L{cuda}/lib64", "-lcudart",
           f"-Wl,-rpath,{lib}", f"-Wl,-rpath,{cuda}/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    path = str(tmp_path / "cpp.gguf")
    write_synthetic_gguf(path, tiny_qwen3_config(layers=2, hidden=512, heads=8, kv_heads=2, inter=1024, vocab=1024), seed=3, device="cpu",
                         q_main=q_main, q_more=q_more)
    prompt = [5, 300, 77, 1000, 12]
    m = GGUFModel(path, device="cuda", max_seq=256)
    want = m.run_script(prompt, 8)
    m.close()
    r = subprocess.run([exe, path, "8"] + [str(t) for t in prompt], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    ids = [int(x) for x in [ln for ln in r.stdout.splitlines() if ln.startswith("IDS")][0].split()[1:]]
    step = int([ln for ln in r.stdout.splitlines() if ln.startswith("STEP")][0].split()[1])
    assert ids == want and step == want[0], (ids, want, step)


def test_draft_model_speculative_generation(tmp_path):
    """A draft model proposes, the target verifies k tokens per batched pass: the result equals the target's own greedy
    continuation under the batched pass, with fewer target passes than tokens when the draft agrees (here the draft is the
    target itself, so every proposal is accepted up to rounding of the two numeric paths)."""
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.io.speculative import speculative_generate
    cfg = tiny_qwen3_config(layers=2, hidden=512, heads=8, kv_heads=2, inter=1024, vocab=1000)
    p = str(tmp_path / "t.gguf")
    write_synthetic_gguf(p, cfg, seed=21, device="cuda", std=0.05)
    small = tiny_qwen3_config(layers=1, hidden=256, heads=4, kv_heads=2, inter=512, vocab=1000)
    q = str(tmp_path / "d.gguf")
    write_synthetic_gguf(q, small, seed=22, device="cuda", std=0.05)
    target, same, other = GGUFModel(p, max_seq=256), GGUFModel(p, max_seq=256), GGUFModel(q, max_seq=256)
    prompt = [5, 77, 300, 901, 12, 64, 8, 8, 440, 3]
    # reference: the target alone, one batched pass per token
    ref, gaps, ctx = [], [], list(prompt)
    lg = target.prefill(ctx, 0, return_logits=True)
    for _ in range(12):
        top = lg[-1].topk(2).values
        gaps.append(float(top[0] - top[1]) / max(float(top[0].abs()), 1e-6))
        t = int(lg[-1].argmax())
        ref.append(t)
        lg = target.prefill([t, t], len(ctx), return_logits=True)[:1]     # two rows: the one-row GEMM is a different kernel
        ctx.append(t)

    def same_up_to_near_ties(got):
        # the batched pass sums in a different order for a different number of rows: only a near-tie may flip
        for i, (g_, r_) in enumerate(zip(got, ref)):
            if g_ != r_:
                return gaps[i] < 2e-2
        return len(got) == len(ref)
    out, st = speculative_generate(target, same, prompt, max_new_tokens=12, k=4)
    assert same_up_to_near_ties(out), (out, ref, gaps)
    assert st["target_passes"] < 12 and st["accepted"] >= 4, st           # an identical draft is accepted most of the time
    out2, st2 = speculative_generate(target, other, prompt, max_new_tokens=12, k=3)
    assert same_up_to_near_ties(out2), (out2, ref, gaps)                   # an unrelated draft costs passes, never tokens
    for m in (target, same, other):
        m.check_status()
        m.close()


def test_lowrank_head_agrees_with_the_engine(tiny_model):
    """The low-rank output projection, fed with the engine's final hidden state, names the engine's own arg-max whenever
    that token is among its candidates (a random 1000 x 512 head has a flat spectrum, so many candidates are kept)."""
    from prometorch_b200.io.gguf_model import GGUFModel
    m = GGUFModel(tiny_model, max_seq=128)
    m.lowrank_head(rank=256, candidate_k=200)
    hits = 0
    for pos, t in enumerate([3, 77, 500, 999, 12, 64, 5, 901]):
        nxt = m.forward_decode(t, pos)
        hits += m.next_token_lowrank() == nxt
    assert hits >= 6, hits
    m.check_status()
    m.close()


def test_deepseek2_on_the_gpu_matches_the_cpu_model(tmp_path):
    """The latent-attention + mixture-of-experts decoder in bf16 on the GPU against its fp32 run on the CPU."""
    from prometorch_b200.io.synthetic import write_synthetic_deepseek2
    from prometorch_b200.models.deepseek2 import DeepSeek2Model
    p = str(tmp_path / "ds2.gguf")
    write_synthetic_deepseek2(p, seed=9)
    cpu = DeepSeek2Model(p, device="cpu", max_seq=64)
    gpu = DeepSeek2Model(p, device="cuda", max_seq=64, dtype=torch.bfloat16)
    toks = [5, 100, 17, 250, 31, 8]
    a = cpu.forward(toks)
    b = torch.cat([gpu.forward(toks[:4]), gpu.forward(toks[4:])]).cpu()
    cos = torch.nn.functional.cosine_similarity(a, b, dim=-1)
    assert float(cos.min()) > 0.99, cos
    assert len(gpu.generate(toks[:3], max_new_tokens=4)) <= 4


def test_generate_cli_with_a_draft_model(tmp_path):
    """`python -m prometorch_b200.generate --draft`: greedy speculative decoding from the command line."""
    import subprocess
    import sys
    import os
    cfg = tiny_qwen3_config(layers=2, hidden=512, heads=8, kv_heads=2, inter=1024, vocab=1000)
    t, d = str(tmp_path / "t.gguf"), str(tmp_path / "d.gguf")
    write_synthetic_gguf(t, cfg, seed=31, device="cuda", std=0.05)
    write_synthetic_gguf(d, tiny_qwen3_config(layers=1, hidden=256, heads=4, kv_heads=2, inter=512, vocab=1000), seed=32, device="cuda", std=0.05)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "prometorch_b200.generate", t, "t300 t301 t302 t303 t304 t305 t306 t307 t308 t309", "--greedy",
                        "--max-tokens", "10", "--draft", d, "--spec-k", "3"], capture_output=True, text=True, timeout=300, cwd=root)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "[Speculative]" in r.stdout and "target passes" in r.stdout, r.stdout[-1500:]
