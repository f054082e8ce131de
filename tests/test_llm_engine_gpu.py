"""Paged KV kernels and the continuous-batching engine on a B200 against the fp32 tensor-op paths."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


@pytest.mark.parametrize("H,Hk,D", [(8, 2, 128), (4, 4, 64), (16, 2, 128), (8, 4, 64)])
def test_paged_rope_write_and_decode_kernels(H, Hk, D):
    from prometorch_b200.ops import paged as P
    dev = "cuda"
    torch.manual_seed(H * 7 + D)
    n_pages, B = 40, 3
    lens = [1, 200, 517]
    perm = torch.randperm(n_pages)
    table = torch.zeros(B, 16, dtype=torch.int32)
    used = 0
    for b, n in enumerate(lens):
        k = (n + P.PAGE - 1) // P.PAGE
        table[b, :k] = perm[used:used + k].int()
        used += k
    cos, sin = P.rope_tables(1024, D, 10000.0, dev)
    kp = torch.zeros(n_pages, Hk, P.PAGE, D, device=dev, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    kp_ref, vp_ref = kp.float().cpu(), vp.float().cpu()
    table_d = table.to(dev)
    for b, n in enumerate(lens):
        qkv = torch.randn(n, (H + 2 * Hk) * D, device=dev).bfloat16()
        pos = torch.arange(n, dtype=torch.int32, device=dev)
        req = torch.full((n,), b, dtype=torch.int32, device=dev)
        q_ref = qkv.float().cpu()
        k_ref = P.paged_rope_write(q_ref, H, Hk, D, pos.cpu(), req.cpu(), table, cos.cpu(), sin.cpu(), kp_ref, vp_ref, want_k=True)
        k_out = P.paged_rope_write(qkv, H, Hk, D, pos, req, table_d, cos, sin, kp, vp, want_k=True)
        torch.cuda.synchronize()
        assert _rel(k_out, k_ref) < 6e-3
        assert _rel(qkv[:, :H * D], q_ref[:, :H * D]) < 6e-3                       # q rotated in place
    P.check_status(dev)
    assert _rel(kp, kp_ref) < 6e-3 and _rel(vp, vp_ref) < 1e-6
    q = torch.randn(B, (H + 2 * Hk) * D, device=dev).bfloat16()                    # heads read from the packed row
    lens_d = torch.tensor(lens, dtype=torch.int32, device=dev)
    ref = P.paged_attention_reference(q.float().cpu(), H, Hk, D, torch.tensor(lens), table, kp.float().cpu(), vp.float().cpu())
    for nsplit in (1, 3):
        out = P.paged_attention_decode(q, H, Hk, D, lens_d, table_d, kp, vp, nsplit=nsplit)
        torch.cuda.synchronize()
        P.check_status(dev)
        assert out.shape == (B, H * D)
        assert _rel(out, ref) < 1e-2, (nsplit, _rel(out, ref))


def test_paged_kernels_skip_a_bad_page_id():
    from prometorch_b200.ops import paged as P
    dev = "cuda"
    H, Hk, D = 4, 2, 64
    kp = torch.zeros(4, Hk, P.PAGE, D, device=dev, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    table = torch.tensor([[99, 0]], dtype=torch.int32, device=dev)                 # page 99 is not in the pool
    q = torch.randn(1, H * D, device=dev).bfloat16()
    P.paged_attention_decode(q, H, Hk, D, torch.tensor([10], dtype=torch.int32, device=dev), table, kp, vp)
    torch.cuda.synchronize()
    with pytest.raises(IndexError):
        P.check_status(dev)
    P.check_status(dev)                                                            # the status word is cleared; the context lives


def test_engine_logits_and_batching_match_cpu_engine():
    from prometorch_b200.serve.llm import GenerationConfig, LlamaConfig, LlamaWeights, LLMEngine, Request
    cfg = LlamaConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=512)
    w = LlamaWeights.random(cfg, seed=1, dtype=torch.bfloat16)
    gpu, cpu = LLMEngine(device="cuda", max_pages=32, max_active=4), LLMEngine(device="cpu", max_pages=32, max_active=4, dtype=torch.float32)
    gpu.set_weights(w)
    cpu.set_weights(w)
    g = torch.Generator().manual_seed(3)
    prompts = [[1] + torch.randint(3, 1024, (n,), generator=g).tolist() for n in (70, 9, 130)]
    greedy = dict(temperature=0.0, repetition_penalty=1.0, top_k=1)
    # same prompt pass and the same three-request decode pass on both engines: logits agree
    for e in (gpu, cpu):
        for i, p in enumerate(prompts):
            e.submit_request(Request(i, p, GenerationConfig(max_new_tokens=8, **greedy)))
    lg, lc = [], []
    for e, out in ((gpu, lg), (cpu, lc)):
        for s in e.active:
            assert e._ensure_pages(s, s.prompt_len - 1)
            out.append(e._forward_prompt(s).float().cpu())
            s.kv_position, s.prefill_done = s.prompt_len, True
    for a, b in zip(lg, lc):
        assert _rel(a, b) < 3e-2, _rel(a, b)
    for e in (gpu, cpu):                                                           # feed both the CPU engine's choice
        for s, l in zip(e.active, lc):
            s.input_ids = [int(l.argmax())]
            assert e._ensure_pages(s, s.kv_position)
    eg, ec = gpu.embed(prompts[0]), cpu.embed(prompts[0])            # one page-table row is still free on both
    assert float(torch.nn.functional.cosine_similarity(eg.cpu(), ec, dim=0)) > 0.995
    dg, dc = gpu._forward_decode(gpu.active).float().cpu(), cpu._forward_decode(cpu.active)
    assert dg.shape == (3, 1024) and _rel(dg, dc) < 3e-2, _rel(dg, dc)
    # a full run: sampled and greedy requests together, pages come back
    eng = LLMEngine(device="cuda", max_pages=32, max_active=3)
    eng.set_weights(w)
    for i, p in enumerate(prompts + [prompts[1]]):
        cfg_i = GenerationConfig(max_new_tokens=10 + i, **greedy) if i % 2 == 0 else GenerationConfig(max_new_tokens=10 + i)
        eng.submit_request(Request(i, p, cfg_i))
    got = {}
    for _ in range(100):
        eng.step()
        got.update({r.request_id: r for r in eng.poll_responses()})
        if eng.num_active() == 0:
            break
    assert sorted(got) == [0, 1, 2, 3] and all(1 <= got[i].tokens_generated <= 10 + i for i in got)
    assert max(eng.launch_log) == 3 and eng.kv.pages_in_use == 0
    # graph replay and the eager pass give the same tokens
    outs = []
    for use_graphs in (True, False):
        e = LLMEngine(device="cuda", max_pages=32, max_active=4, use_graphs=use_graphs)
        e.set_weights(w)
        for i, p in enumerate(prompts):
            e.submit_request(Request(i, p, GenerationConfig(max_new_tokens=12, **greedy)))
        res = {}
        while e.num_active():
            e.step()
            res.update({r.request_id: r.token_ids for r in e.poll_responses()})
        outs.append(res)
    assert outs[0] == outs[1] and len(outs[0]) == 3


def test_qkv_projection_fused_with_rope_write():
    """Split-K partials summed inside the rotary kernel give the same q and pages as projection + bf16 round trip."""
    from prometorch_b200.ops import paged as P
    dev = "cuda"
    torch.manual_seed(5)
    H, Hk, D, K, n = 16, 4, 128, 2048, 8
    w = (torch.randn((H + 2 * Hk) * D, K, device=dev) * K ** -0.5).bfloat16()
    h = torch.randn(n, K, device=dev).bfloat16()
    cos, sin = P.rope_tables(512, D, 10000.0, dev)
    pos = torch.tensor([0, 5, 63, 64, 100, 127, 128, 300], dtype=torch.int32, device=dev)
    req = torch.arange(n, dtype=torch.int32, device=dev)
    table = torch.arange(n * 8, dtype=torch.int32, device=dev).view(n, 8)
    pools = [[torch.zeros(n * 8, Hk, P.PAGE, D, device=dev, dtype=torch.bfloat16) for _ in range(2)] for _ in range(2)]
    with torch.no_grad():
        q = P.qkv_rope_write(h, w, H, Hk, D, pos, req, table, cos, sin, pools[0][0], pools[0][1], fuse_sum=True)
        qkv = (h.float() @ w.float().t()).bfloat16()
        P.paged_rope_write(qkv, H, Hk, D, pos, req, table, cos, sin, pools[1][0], pools[1][1])
    torch.cuda.synchronize()
    P.check_status(dev)
    assert q.shape == (n, H * D) and _rel(q, qkv[:, :H * D]) < 6e-3
    assert _rel(pools[0][0], pools[1][0]) < 6e-3 and _rel(pools[0][1], pools[1][1]) < 6e-3


def test_hf_compat_models_on_gpu_match_cpu():
    """The Hugging Face shim's three architectures on CUDA bf16 (tcgen05 GEMM, FlashAttention, fused norms) vs CPU fp32."""
    from prometorch_b200.transformers_compat import BertModel, GPT2Model, LlamaModel
    torch.manual_seed(0)
    cases = [
        (LlamaModel, dict(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                          intermediate_size=512, rms_norm_eps=1e-5, rope_theta=10000.0)),
        (GPT2Model, dict(vocab_size=512, n_embd=256, n_layer=2, n_head=4, n_positions=256)),
        (BertModel, dict(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512,
                         max_position_embeddings=256)),
    ]
    ids = torch.randint(0, 512, (2, 136))
    for cls, cfg in cases:
        cpu = cls(cfg).eval()
        with torch.no_grad():
            for p in cpu.parameters():
                if p.dim() > 1:
                    p.normal_(0, 0.05)
                p.copy_(p.bfloat16().float())                       # both sides hold bf16-representable weights
            want = cpu(ids)
            gpu = cls(cfg).eval()
            gpu.load_state_dict(cpu.state_dict())
            got = gpu.to(device="cuda", dtype=torch.bfloat16)(ids.cuda())
        torch.cuda.synchronize()
        assert got.shape == want.shape and _rel(got, want) < 4e-2, (cls.__name__, _rel(got, want))


def test_speculative_decoding_on_gpu_agrees_with_plain_greedy():
    from prometorch_b200.serve.llm import GenerationConfig, LlamaConfig, LlamaWeights, LLMEngine, Request
    cfg = LlamaConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=512, eos_token_id=-1)
    w = LlamaWeights.random(cfg, seed=2, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(7)
    piece = torch.randint(3, 1024, (10,), generator=g).tolist()
    prompts = [[1] + piece * 6, [1] + torch.randint(3, 1024, (40,), generator=g).tolist(), [1] + piece[:4] * 20]
    greedy = dict(temperature=0.0, repetition_penalty=1.0, top_k=1)
    outs, engines = [], []
    for k in (0, 4):
        e = LLMEngine(device="cuda", max_pages=64, max_active=4, spec_tokens=k)
        e.set_weights(w)
        for i, p in enumerate(prompts):
            e.submit_request(Request(i, p, GenerationConfig(max_new_tokens=40, **greedy)))
        res = {}
        while e.num_active():
            e.step()
            res.update({r.request_id: r.token_ids for r in e.poll_responses()})
        outs.append(res)
        engines.append(e)
        assert e.kv.pages_in_use == 0 and all(len(res[i]) == 40 for i in range(3))
    # bf16 sums differ a little with the batch shape, so a near-tie may flip once in a while: compare position by position
    same = sum(a == b for i in range(3) for a, b in zip(outs[0][i], outs[1][i]))
    assert same >= 0.75 * 120, same
    assert engines[1].spec_drafted > 0 and engines[1].steps <= engines[0].steps
