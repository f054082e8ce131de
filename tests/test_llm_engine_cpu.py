"""Paged-KV continuous-batching engine on CPU: page pool, scheduling, loaders; tokens against a dense recompute."""
import json
import math
import os

import pytest
import torch

from prometorch_b200.serve.llm import (PAGE, GenerationConfig, LlamaConfig, LlamaWeights, LLMEngine, PagedKVCache, Request,
                                       load_safetensors, save_safetensors)


def tiny_cfg(**kw):
    c = LlamaConfig(vocab_size=97, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, max_position_embeddings=256, rope_theta=10000.0, bos_token_id=1, eos_token_id=2)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def dense_next_token(w: LlamaWeights, ids):
    """Greedy next id by recomputing the whole sequence with plain fp32 tensor ops (no cache, no pages)."""
    c = w.cfg
    H, Hk, Dh, T = c.num_attention_heads, c.num_key_value_heads, c.head_dim, len(ids)
    x = w.tok_emb[torch.tensor(ids)].float()
    inv = 1.0 / (c.rope_theta ** (torch.arange(0, Dh, 2, dtype=torch.float64) / Dh))
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None]
    cos, sin = ang.cos().float()[:, None], ang.sin().float()[:, None]

    def norm(v, g):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + c.rms_norm_eps) * g.float()

    def rot(t):
        a, b = t[..., :Dh // 2], t[..., Dh // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
    for L in w.layers:
        qkv = norm(x, L["attn_norm"]) @ L["wqkv"].float().t()
        q, k, v = qkv.split([H * Dh, Hk * Dh, Hk * Dh], -1)
        q, k, v = rot(q.view(T, H, Dh)), rot(k.view(T, Hk, Dh)), v.view(T, Hk, Dh)
        k, v = k.repeat_interleave(H // Hk, 1), v.repeat_interleave(H // Hk, 1)
        s = torch.einsum("thd,shd->hts", q, k) / math.sqrt(Dh)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        a = torch.einsum("hts,shd->thd", torch.softmax(s, -1), v).reshape(T, H * Dh)
        x = x + a @ L["wo"].float().t()
        gu = norm(x, L["ffn_norm"]) @ L["w_gate_up"].float().t()
        g, u = gu.chunk(2, -1)
        x = x + (torch.nn.functional.silu(g) * u) @ L["w_down"].float().t()
    return int((norm(x[-1], w.final_norm) @ w.lm_head.float().t()).argmax())


def dense_generate(w, prompt, n):
    ids, out = list(prompt), []
    for _ in range(n):
        t = dense_next_token(w, ids)
        out.append(t)
        ids.append(t)
        if t == w.cfg.eos_token_id:
            break
    return out


GREEDY = dict(temperature=0.0, repetition_penalty=1.0, top_k=1)


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "c": torch.arange(6, dtype=torch.int64).view(2, 3),
         "d": torch.randn(4, 4).half()}
    p = str(tmp_path / "x.safetensors")
    save_safetensors(t, p)
    back = load_safetensors(p)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])


def test_page_pool():
    kv = PagedKVCache(2, 2, 16, 5, "cpu", torch.float32)
    got = [kv.alloc_page() for _ in range(5)]
    assert sorted(got) == list(range(5)) and kv.alloc_page() == -1 and kv.pages_in_use == 5
    kv.free_page(got[2])
    assert kv.alloc_page() == got[2]
    assert kv.k[0].shape == (5, 2, PAGE, 16)


def test_greedy_matches_dense_recompute_across_pages():
    w = LlamaWeights.random(tiny_cfg(), seed=3)
    eng = LLMEngine(device="cpu", max_pages=16, max_active=2)
    eng.set_weights(w)
    g = torch.Generator().manual_seed(0)
    prompt = [1] + torch.randint(3, 97, (60,), generator=g).tolist()           # the generation crosses the 64-token page edge
    r = eng.generate(prompt, GenerationConfig(max_new_tokens=12, **GREEDY))
    assert r.token_ids == dense_generate(w, prompt, 12)
    assert r.tokens_generated == len(r.token_ids) and r.throughput_tok_per_s > 0
    assert eng.kv.pages_in_use == 0 and eng.num_active() == 0


def test_continuous_batching_equals_one_by_one():
    w = LlamaWeights.random(tiny_cfg(), seed=5)
    g = torch.Generator().manual_seed(1)
    prompts = [[1] + torch.randint(3, 97, (n,), generator=g).tolist() for n in (5, 70, 17, 130, 33)]
    want = [dense_generate(w, p, 6 + i) for i, p in enumerate(prompts)]
    eng = LLMEngine(device="cpu", max_pages=32, max_active=3)
    eng.set_weights(w)
    for i, p in enumerate(prompts):
        eng.submit_request(Request(10 + i, p, GenerationConfig(max_new_tokens=6 + i, **GREEDY)))
    assert eng.num_active() == 5 and len(eng.active) == 3                     # two wait for a free slot
    got = {}
    for _ in range(200):
        eng.step()
        for r in eng.poll_responses():
            got[r.request_id] = r.token_ids
        if eng.num_active() == 0:
            break
    assert got == {10 + i: want[i] for i in range(5)}
    assert max(eng.launch_log) == 3                                            # decode passes really were batched
    assert eng.kv.pages_in_use == 0 and sorted(eng.free_rows) == [0, 1, 2]


def test_stop_tokens_and_eos():
    w = LlamaWeights.random(tiny_cfg(), seed=7)
    prompt = [1, 5, 9, 11]
    ref = dense_generate(w, prompt, 8)
    eng = LLMEngine(device="cpu", max_pages=8, max_active=1)
    eng.set_weights(w)
    r = eng.generate(prompt, GenerationConfig(max_new_tokens=8, stop_tokens=[ref[2]], **GREEDY))
    assert r.token_ids == ref[:ref.index(ref[2]) + 1]


def test_pool_pressure_requeues_then_serves():
    w = LlamaWeights.random(tiny_cfg(), seed=9)
    g = torch.Generator().manual_seed(2)
    a = [1] + torch.randint(3, 97, (100,), generator=g).tolist()               # two pages each; the pool has three
    b = [1] + torch.randint(3, 97, (90,), generator=g).tolist()
    eng = LLMEngine(device="cpu", max_pages=3, max_active=2)
    eng.set_weights(w)
    eng.submit_request(Request(0, a, GenerationConfig(max_new_tokens=4, **GREEDY)))
    eng.submit_request(Request(1, b, GenerationConfig(max_new_tokens=4, **GREEDY)))
    got = {}
    for _ in range(50):
        eng.step()
        got.update({r.request_id: r.token_ids for r in eng.poll_responses()})
        if eng.num_active() == 0:
            break
    assert got[0] == dense_generate(w, a, 4) and got[1] == dense_generate(w, b, 4)
    assert eng.kv.pages_in_use == 0
    # a prompt that can never fit ends with an empty answer rather than a stall
    eng2 = LLMEngine(device="cpu", max_pages=1, max_active=1)
    eng2.set_weights(w)
    assert eng2.generate(a, GenerationConfig(max_new_tokens=4, **GREEDY)).token_ids == []


def test_sampled_generation_is_seeded_and_in_vocab():
    w = LlamaWeights.random(tiny_cfg(), seed=11)
    outs = []
    for _ in range(2):
        eng = LLMEngine(device="cpu", max_pages=8, max_active=1, seed=4)
        eng.set_weights(w)
        outs.append(eng.generate([1, 4, 8], GenerationConfig(max_new_tokens=10, temperature=0.9, top_k=20, top_p=0.95,
                                                              repetition_penalty=1.2)).token_ids)
    assert outs[0] == outs[1] and all(0 <= t < 97 for t in outs[0]) and len(outs[0]) >= 1


def test_load_hf_directory(tmp_path):
    cfg = tiny_cfg(vocab_size=300)
    w = LlamaWeights.random(cfg, seed=13)
    d = tmp_path / "model"
    d.mkdir()
    with open(d / "config.json", "w") as f:
        json.dump({k: getattr(cfg, k) for k in cfg.__dataclass_fields__}, f)
    sd = w.state_dict()
    names = sorted(sd)
    save_safetensors({k: sd[k] for k in names[:len(names) // 2]}, str(d / "model-00001-of-00002.safetensors"))
    save_safetensors({k: sd[k] for k in names[len(names) // 2:]}, str(d / "model-00002-of-00002.safetensors"))
    with open(d / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": {k: ("model-00001-of-00002.safetensors" if i < len(names) // 2 else "model-00002-of-00002.safetensors")
                                  for i, k in enumerate(names)}}, f)
    eng = LLMEngine(device="cpu", max_pages=8, max_active=1)
    assert eng.load(str(d)) and eng.loaded
    r = eng.generate("hi", GenerationConfig(max_new_tokens=5, **GREEDY))     # byte tokenizer: no tokenizer files here
    prompt = [1] + [b + 3 for b in b"hi"]
    assert r.token_ids == dense_generate(w, prompt, 5)
    assert isinstance(r.output, str)
    assert not LLMEngine(device="cpu").load(str(tmp_path / "nowhere"))


def test_paged_ops_reference_paths():
    from prometorch_b200.ops import paged as P
    torch.manual_seed(0)
    H, Hk, D, n_pages = 4, 2, 16, 6
    kp, vp = torch.zeros(n_pages, Hk, PAGE, D), torch.zeros(n_pages, Hk, PAGE, D)
    table = torch.tensor([[4, 1, 0], [2, 5, 3]], dtype=torch.int32)
    cos, sin = P.rope_tables(256, D, 10000.0, "cpu")
    lens = [70, 3]
    ks = {}
    for b, n in enumerate(lens):
        qkv = torch.randn(n, (H + 2 * Hk) * D)
        raw = qkv.clone()
        k = P.paged_rope_write(qkv, H, Hk, D, torch.arange(n, dtype=torch.int32), torch.full((n,), b, dtype=torch.int32), table, cos, sin,
                               kp, vp, want_k=True)
        ks[b] = (k, raw.view(n, H + 2 * Hk, D)[:, H + Hk:])
    # what was written is what a gather through the table reads back
    for b, n in enumerate(lens):
        pages = table[b, :(n + PAGE - 1) // PAGE].long()
        kk = kp[pages].permute(1, 0, 2, 3).reshape(Hk, -1, D)[:, :n].permute(1, 0, 2)
        vv = vp[pages].permute(1, 0, 2, 3).reshape(Hk, -1, D)[:, :n].permute(1, 0, 2)
        assert torch.allclose(kk, ks[b][0]) and torch.allclose(vv, ks[b][1])
    q = torch.randn(2, H * D)
    out = P.paged_attention_decode(q, H, Hk, D, torch.tensor(lens, dtype=torch.int32), table, kp, vp)
    for b, n in enumerate(lens):
        k, v = ks[b][0].repeat_interleave(H // Hk, 1), ks[b][1].repeat_interleave(H // Hk, 1)
        s = torch.einsum("hd,nhd->hn", q[b].view(H, D), k) / math.sqrt(D)
        ref = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), v).reshape(-1)
        assert torch.allclose(out[b], ref, atol=1e-5)
    assert P.pick_splits(1, 8, 8192) == 16 and P.pick_splits(64, 8, 8192) == 2 and P.pick_splits(4, 4, 64) == 1


def test_speculative_decoding_gives_the_same_greedy_tokens():
    """N-gram proposals verified inside the decode pass: identical output, fewer passes, mixed with a sampled request."""
    w = LlamaWeights.random(tiny_cfg(), seed=17)
    g = torch.Generator().manual_seed(5)
    base = torch.randint(3, 97, (12,), generator=g).tolist()
    prompts = [[1] + base * 4, [1] + torch.randint(3, 97, (20,), generator=g).tolist(), [1] + base[:5] * 9]
    want = [dense_generate(w, p, 24) for p in prompts]
    plain = LLMEngine(device="cpu", max_pages=32, max_active=4)
    spec = LLMEngine(device="cpu", max_pages=32, max_active=4, spec_tokens=4)
    outs = []
    for eng in (plain, spec):
        eng.set_weights(w)
        for i, p in enumerate(prompts):
            eng.submit_request(Request(i, p, GenerationConfig(max_new_tokens=24, **GREEDY)))
        eng.submit_request(Request(9, prompts[0], GenerationConfig(max_new_tokens=8, temperature=0.8, top_k=10, repetition_penalty=1.1)))
        got = {}
        while eng.num_active():
            eng.step()
            got.update({r.request_id: r.token_ids for r in eng.poll_responses()})
        outs.append(got)
        assert eng.kv.pages_in_use == 0
    for i in range(3):
        assert outs[0][i] == want[i] and outs[1][i] == want[i]
    assert 1 <= len(outs[1][9]) <= 8
    assert spec.spec_drafted > 0 and spec.spec_accepted > 0 and spec.steps < plain.steps
    # the proposal never runs past max_new_tokens or the position limit
    short = LLMEngine(device="cpu", max_pages=8, max_active=1, spec_tokens=8)
    short.set_weights(w)
    assert short.generate(prompts[0], GenerationConfig(max_new_tokens=3, **GREEDY)).token_ids == want[0][:3]


def test_batched_prompt_pass_groups_and_token_cap():
    """New requests share a prompt pass (equal lengths share the attention call); a token cap splits the pass."""
    w = LlamaWeights.random(tiny_cfg(), seed=19)
    g = torch.Generator().manual_seed(8)
    prompts = [[1] + torch.randint(3, 97, (n,), generator=g).tolist() for n in (20, 20, 20, 7, 66, 66)]
    want = [dense_generate(w, p, 5) for p in prompts]
    for cap in (16384, 50):
        eng = LLMEngine(device="cpu", max_pages=32, max_active=6)
        eng.set_weights(w)
        eng.max_prompt_tokens = cap
        calls = []
        real = eng._forward_prompts
        eng._forward_prompts = lambda batch, real=real: calls.append(len(batch)) or real(batch)
        for i, p in enumerate(prompts):
            eng.submit_request(Request(i, p, GenerationConfig(max_new_tokens=5, **GREEDY)))
        got = {}
        while eng.num_active():
            eng.step()
            got.update({r.request_id: r.token_ids for r in eng.poll_responses()})
        assert got == {i: want[i] for i in range(6)}
        assert calls == ([6] if cap == 16384 else [2, 2, 1, 1]), calls        # 21+21 | 21+8 | 67 | 67 tokens under a cap of 50


def test_stream_yields_tokens_as_they_come():
    w = LlamaWeights.random(tiny_cfg(), seed=23)
    eng = LLMEngine(device="cpu", max_pages=8, max_active=2)
    eng.set_weights(w)
    prompt = [1, 9, 33, 7]
    eng.submit_request(Request(50, [1, 2, 3], GenerationConfig(max_new_tokens=4, **GREEDY)))      # a neighbour in the batch
    seen = []
    for t in eng.stream(prompt, GenerationConfig(max_new_tokens=7, **GREEDY)):
        seen.append(t)
        assert eng.steps >= len(seen)                                 # ids arrive step by step, not at the end
    assert seen == dense_generate(w, prompt, 7)
    while eng.num_active():
        eng.step()
    assert [r.request_id for r in eng.poll_responses()] == [50]


def test_embed_returns_pages_and_matches_dense_hidden_mean():
    w = LlamaWeights.random(tiny_cfg(), seed=29)
    eng = LLMEngine(device="cpu", max_pages=4, max_active=1)
    eng.set_weights(w)
    ids = [1, 7, 50, 3, 3, 90]
    e = eng.embed(ids)
    assert e.shape == (64,) and abs(float(e.norm()) - 1.0) < 1e-5 and eng.kv.pages_in_use == 0 and eng.free_rows == [0]
    assert torch.allclose(e, eng.embed(ids)) and not torch.allclose(e, eng.embed(ids[:-1] + [91]))
    assert eng.generate(ids, GenerationConfig(max_new_tokens=3, **GREEDY)).token_ids == dense_generate(w, ids, 3)   # the engine still serves


def test_cancel_and_stats():
    w = LlamaWeights.random(tiny_cfg(), seed=31)
    eng = LLMEngine(device="cpu", max_pages=8, max_active=1)
    eng.set_weights(w)
    eng.submit_request(Request(1, [1, 4, 5], GenerationConfig(max_new_tokens=50, **GREEDY)))
    eng.submit_request(Request(2, [1, 6, 7], GenerationConfig(max_new_tokens=5, **GREEDY)))      # waits: one slot only
    for _ in range(3):
        eng.step()
    st = eng.stats()
    assert st["active"] == 1 and st["pending"] == 1 and st["pages_in_use"] == 1 and st["tokens_generated"] == 3 and st["steps"] == 3
    assert eng.cancel(1) and not eng.cancel(99)
    got = {r.request_id: r.token_ids for r in eng.poll_responses()}
    assert len(got[1]) == 3 and eng.kv.pages_in_use == 0
    while eng.num_active():
        eng.step()
    got.update({r.request_id: r.token_ids for r in eng.poll_responses()})
    assert got[2] == dense_generate(w, [1, 6, 7], 5)
    eng.submit_request(Request(3, [1, 2], GenerationConfig(max_new_tokens=5, **GREEDY)))
    eng.submit_request(Request(4, [1, 3], GenerationConfig(max_new_tokens=5, **GREEDY)))
    assert eng.cancel(4) and [r.request_id for r in eng.poll_responses()] == [4]               # cancelled while queued
