"""The native serving stack of the C++ API (json.h, tokenizer.h, chat.h, serve.h) against the Python implementations:
same token ids, same prompts, same wire format.  The test program serves fake backends, so no GPU is involved."""
import http.client
import json
import os
import shutil
import socket
import subprocess
import threading
import time

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TEXTS = ["Hello world", " leading space", "it's we're I'll they've I'm he'd don't 'quoted'", "tabs\tand\nnewlines\n\n  and   runs  ",
         "numbers 12345 and 3.14 and x2y", "punctuation!!! (really?) -- yes; no: [ok] {fine} <tag> a.b,c", "Привет, мир! Как дела?",
         "日本語のテキスト、それと English。", "café naïve über straße", "emoji \U0001F600 and ☃ snow — dash “quotes”",
         "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n", "mixed<|endoftext|>tail", "", " ", "  ", "a", "\n", "trailing space ",
         "مرحبا بالعالم ١٢٣", "x² + y³ = ½", "  \n x"]


@pytest.fixture(scope="module")
def exe(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("needs g++")
    out = str(tmp_path_factory.mktemp("serve_native") / "serve_native")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", os.path.join(ROOT, "tests", "cpp", "serve_native.cpp"), "-o", out,
           f"-I{ROOT}/prometorch_b200/cpp_api", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-4000:]
    return out


def _run(exe, *args):
    r = subprocess.run([exe, *args], capture_output=True, timeout=120)
    assert r.returncode == 0, r.stderr.decode()[-2000:]
    return json.loads(r.stdout.decode("utf-8"))


def _train_bpe(corpus, n_merges):
    """A small byte-level BPE vocabulary in GPT-2's spelling (bytes mapped to printable code points)."""
    from prometorch_b200.io.tokenizer import _B2U, _GPT2_PAT
    words = {}
    for piece in _GPT2_PAT.findall(corpus):
        w = tuple(_B2U[b] for b in piece.encode("utf-8"))
        words[w] = words.get(w, 0) + 1
    merges = []
    for _ in range(n_merges):
        pairs = {}
        for w, c in words.items():
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] = pairs.get((a, b), 0) + c
        if not pairs:
            break
        (a, b), _ = max(sorted(pairs.items()), key=lambda kv: kv[1])
        merges.append(f"{a} {b}")
        new = {}
        for w, c in words.items():
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            new[tuple(out)] = new.get(tuple(out), 0) + c
        words = new
    tokens = [_B2U[b] for b in range(256)] + [m.replace(" ", "") for m in merges]
    return tokens, merges


def _check_tokenizer(exe, tmp_path, spec, texts):
    from prometorch_b200.io.tokenizer import GGUFTokenizer
    py = GGUFTokenizer(spec["tokens"], spec["model"], spec["scores"] or None, spec["merges"] or None, spec["types"] or None, spec["bos"], spec["eos"],
                       spec["add_bos"], spec.get("pre", ""))
    spec = dict(spec, texts=texts)
    p = tmp_path / "spec.json"
    p.write_text(json.dumps(spec, ensure_ascii=False), encoding="utf-8")
    got = _run(exe, "tokenize", str(p))
    for i, t in enumerate(texts):
        want = py.encode(t)
        assert got["ids"][i] == want, (t, got["ids"][i], want)
        assert got["decoded"][i] == py.decode(want), t
        assert got["single"][i] == [py.decode_token(x) for x in want], t
    return got


def test_gpt2_tokenizer_matches_python(exe, tmp_path):
    from prometorch_b200.io.tokenizer import _GPT2_PAT
    corpus = " ".join(TEXTS) * 3 + " the quick brown fox jumps over the lazy dog " * 20 + " hello hello world world 123 123 "
    tokens, merges = _train_bpe(corpus, 300)
    tokens += ["<|im_start|>", "<|im_end|>", "<|endoftext|>"]
    types = [1] * (len(tokens) - 3) + [3, 3, 3]
    spec = {"tokens": tokens, "model": "gpt2", "scores": [], "merges": merges, "types": types, "bos": -1, "eos": len(tokens) - 1, "add_bos": False}
    got = _check_tokenizer(exe, tmp_path, spec, TEXTS)
    for i, t in enumerate(TEXTS):                       # the hand-written scanner against the pattern
        assert got["pieces"][i] == _GPT2_PAT.findall(t), t


@pytest.mark.parametrize("pre", ["qwen2", "llama3", "llama-bpe", "unknown-name"])
def test_newer_pretokenizer_patterns_match_python(exe, tmp_path, pre):
    """tokenizer.ggml.pre: the qwen2 and llama-3 split patterns (hand-written scanner in C++, `regex` in Python) cut every text
    into the same pieces and give the same ids; an unknown name falls back to GPT-2's pattern on both sides."""
    from prometorch_b200.io.tokenizer import pretokenizer_pattern
    extra = ["Hello!world it'S I'LL we'Re 12345 a\n\n  b\t\tc  \n x !!\r\n", "x=1+22*333/4444;\n\n\nif (a<b) {\r\n\treturn 7;}", "  \n", "\n \n  ",
             "(привет) 2024год №5", "a\tb \tc", "\'\'\'quote\'\'\' ...\n", "tab\t\n\tafter", " 7 days", "end \n"]
    texts = TEXTS + extra
    tokens, merges = _train_bpe(" ".join(texts) * 2, 200)
    tokens += ["<|im_start|>", "<|im_end|>", "<|endoftext|>"]
    spec = {"tokens": tokens, "model": "gpt2", "scores": [], "merges": merges, "types": [1] * (len(tokens) - 3) + [3, 3, 3], "bos": -1, "eos": -1,
            "add_bos": False, "pre": pre}
    got = _check_tokenizer(exe, tmp_path, spec, texts)
    pat = pretokenizer_pattern(pre)
    for i, t in enumerate(texts):
        if "<|" in t:
            continue                                                      # special tokens are cut out before the pattern runs
        assert got["styled_pieces"][i] == pat.findall(t), (pre, t, got["styled_pieces"][i], pat.findall(t))
        assert "".join(got["styled_pieces"][i]) == t


def test_spm_tokenizer_matches_python(exe, tmp_path):
    bar = "▁"
    base = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)]
    chars = sorted(set("".join(TEXTS).replace(" ", bar) + bar + "abcdefghijklmnopqrstuvwxyz"))
    chars = [c for c in chars if c not in "\n\t"]       # left to the byte fall-back
    words = [bar + "Hello", bar + "world", bar + "the", "ing", "er", bar + "a", "ll", "he", bar + "he", "llo", bar + "hello", "or", "ld", "wor", bar + "wor",
             bar + bar, "an", bar + "an", bar + "and", "nd", "num", "ber", "bers", bar + "num", bar + "numbers", "12", "123", "45", bar + "мир", "При", "вет",
             "日本", "日本語", "<|im_start|>", "<|im_end|>", "<|endoftext|>", "user", bar + "user", "ass", "ist", "ant", "assistant"]
    tokens = base + chars + [w for w in words if w not in chars]
    scores = [0.0] * len(base) + [-100.0 - i for i in range(len(chars))] + [-1.0 - 0.5 * i for i in range(len(tokens) - len(base) - len(chars))]
    types = [2, 3, 3] + [6] * 256 + [1] * (len(tokens) - 259)
    for s in ("<|im_start|>", "<|im_end|>", "<|endoftext|>"):
        types[tokens.index(s)] = 4
    spec = {"tokens": tokens, "model": "llama", "scores": scores, "merges": [], "types": types, "bos": 1, "eos": 2, "add_bos": True}
    _check_tokenizer(exe, tmp_path, spec, TEXTS + ["Hello world the hello", "numbers and numbers", "hellohello"])
    spec["add_bos"] = False
    _check_tokenizer(exe, tmp_path, spec, ["Hello", bar + "already marked", "tie breaks: aaaa llll"])


def test_tokenizer_from_a_gguf_file(exe, tmp_path):
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.gguf import GGUFReader
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.io.tokenizer import GGUFTokenizer
    path = str(tmp_path / "tok.gguf")
    write_synthetic_gguf(path, tiny_qwen3_config(layers=1, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=1, device="cpu")
    reader = GGUFReader(path)
    if reader.get("tokenizer.ggml.tokens") is None:
        pytest.skip("the synthetic writer put no tokenizer into the file")
    py = GGUFTokenizer.from_reader(reader)
    texts = ["hello world", "abc 123", "tok5 tok17", "éè", "x"]
    t = tmp_path / "texts.json"
    t.write_text(json.dumps(texts), encoding="utf-8")
    got = _run(exe, "gguf-tokenize", path, str(t))
    for i, s in enumerate(texts):
        assert got["ids"][i] == py.encode(s), s
        assert got["decoded"][i] == py.decode(py.encode(s)), s


def test_hf_tokenizer_files(exe, tmp_path):
    """vocab.json + merges.txt and tokenizer.json (both spellings of the merges) give the ids of the Python loader."""
    from prometorch_b200.serve.llm import load_hf_tokenizer
    tokens, merges = _train_bpe(" ".join(TEXTS) + " the quick brown fox jumps over the lazy dog " * 10, 150)
    vocab = {t: i for i, t in enumerate(tokens)}
    texts = [t for t in TEXTS if "<|" not in t]
    tj = tmp_path / "texts.json"
    tj.write_text(json.dumps(texts, ensure_ascii=False), encoding="utf-8")
    a, b, c, d = (tmp_path / n for n in ("a", "b", "c", "d"))
    for x in (a, b, c, d):
        x.mkdir()
    (a / "vocab.json").write_text(json.dumps(vocab, ensure_ascii=False), encoding="utf-8")
    (a / "merges.txt").write_text("#version: 0.2\n" + "\n".join(merges) + "\n\n", encoding="utf-8")
    (b / "tokenizer.json").write_text(json.dumps({"model": {"type": "BPE", "vocab": vocab, "merges": merges}}), encoding="utf-8")
    (c / "tokenizer.json").write_text(json.dumps({"model": {"type": "BPE", "vocab": vocab, "merges": [m.split(" ") for m in merges]}}), encoding="utf-8")
    for folder in (a, b, c):
        py = load_hf_tokenizer(str(folder))
        got = _run(exe, "hf-tokenize", str(folder), str(tj))
        for i, t in enumerate(texts):
            assert got["ids"][i] == py.encode(t), (folder.name, t)
            assert got["decoded"][i] == py.decode(py.encode(t)), (folder.name, t)
    assert load_hf_tokenizer(str(d)) is None and _run(exe, "hf-tokenize", str(d), str(tj)) is None


def test_json_roundtrip(exe, tmp_path):
    doc = {"a": [1, -2, 3.5, 1e-7, 12345678901234, True, False, None], "s": "quote \" slash \\ nl \n tab \t uni é 中 \U0001F600 ctl \u0001",
           "nested": {"empty_obj": {}, "empty_arr": [], "k": {"deep": [[[]]]}}, "order": 1, "z": 0, "b": 2}
    p = tmp_path / "doc.json"
    p.write_text(json.dumps(doc), encoding="utf-8")              # ensure_ascii: exercises \uXXXX and surrogate pairs
    got = _run(exe, "json", str(p))
    assert got == doc and list(got) == list(doc)
    p.write_text(json.dumps(doc, ensure_ascii=False), encoding="utf-8")
    assert _run(exe, "json", str(p)) == doc
    p.write_text('{"a": [1, 2,, 3]}')
    r = subprocess.run([exe, "json", str(p)], capture_output=True, timeout=60)
    assert r.returncode == 1 and b"JSON" in r.stderr


def test_chat_templates_match_python(exe, tmp_path, monkeypatch):
    from prometorch_b200.io.chat import apply_chat_template, render_messages, strip_think
    for k in ("PT_SYSTEM_PROMPT", "PROMETHORCH_SYSTEM_PROMPT", "PT_NO_THINK", "PROMETHORCH_NO_THINK"):
        monkeypatch.delenv(k, raising=False)
    cases, want = [], []
    for arch, name in [("qwen3", ""), ("qwen2", ""), ("phi3", ""), ("gemma3", ""), ("llama", "Meta Llama 3"), ("llama", "Mistral-7B"), ("other", "")]:
        for system in (None, "", "be brief"):
            for no_think in (None, True, False):
                c = {"prompt": "what is 2+2?", "arch": arch, "name": name}
                if system is not None:
                    c["system"] = system
                if no_think is not None:
                    c["no_think"] = no_think
                cases.append(c)
                want.append(apply_chat_template("what is 2+2?", arch, name, system, no_think))
        for msgs in ([{"role": "user", "content": "hi"}],
                     [{"role": "system", "content": "S1"}, {"role": "system", "content": "S2"}, {"role": "user", "content": "q1"},
                      {"role": "assistant", "content": "a1"}, {"role": "tool", "content": "t1"}, {"role": "user", "content": "q2"}],
                     [{"role": "system", "content": "only system"}], [{"role": "system", "content": ""}, {"role": "user", "content": "u"}], []):
            cases.append({"messages": msgs, "arch": arch, "name": name})
            want.append(render_messages(msgs, arch, name))
    for s in ("<think>plan</think>\n\nanswer", "no blocks", "<think>a</think>x<think>b</think>  y", "<think>unclosed"):
        cases.append({"strip": s})
        want.append(strip_think(s))
    p = tmp_path / "chat.json"
    p.write_text(json.dumps(cases), encoding="utf-8")
    got = _run(exe, "chat", str(p))
    for c, g, w in zip(cases, got, want):
        assert g == w, c
    monkeypatch.setenv("PT_SYSTEM_PROMPT", "from env")
    monkeypatch.setenv("PROMETHORCH_NO_THINK", "1")
    p.write_text(json.dumps([{"prompt": "q", "arch": "qwen3", "name": ""}]))
    assert _run(exe, "chat", str(p)) == [apply_chat_template("q", "qwen3")]


def test_native_model_loader_matches_python(exe, tmp_path):
    """model_loader.h against io/model_loader.py on every container: detected format, architecture, inferred shape parameters,
    tensor directory, shard discovery, and the stored bytes of every tensor."""
    import dataclasses
    from collections import OrderedDict
    from prometorch_b200 import serialization as S
    from prometorch_b200.io import model_loader as ML
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.safetensors import save_file
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    g = torch.Generator().manual_seed(8)

    def llama_like(qk_norm=False, bias=False, layers=2, hidden=128, heads=2, kv=1, inter=192, vocab=300):
        sd = OrderedDict()
        sd["model.embed_tokens.weight"] = torch.randn(vocab, hidden, generator=g)
        for i in range(layers):
            p = f"model.layers.{i}."
            sd[p + "self_attn.q_proj.weight"] = torch.randn(heads * 64, hidden, generator=g).bfloat16()
            sd[p + "self_attn.k_proj.weight"] = torch.randn(kv * 64, hidden, generator=g).bfloat16()
            sd[p + "self_attn.v_proj.weight"] = torch.randn(kv * 64, hidden, generator=g).half()
            sd[p + "self_attn.o_proj.weight"] = torch.randn(hidden, heads * 64, generator=g)
            if qk_norm:
                sd[p + "self_attn.q_norm.weight"] = torch.ones(64)
            if bias:
                sd[p + "self_attn.q_proj.bias"] = torch.zeros(heads * 64)
            sd[p + "mlp.up_proj.weight"] = torch.randn(inter, hidden, generator=g)
            sd[p + "mlp.down_proj.weight"] = torch.randn(hidden, inter, generator=g)
            sd[p + "input_layernorm.weight"] = torch.ones(hidden)
        sd["model.norm.weight"] = torch.ones(hidden)
        return sd
    paths = {}
    paths["gguf"] = str(tmp_path / "m.gguf")
    write_synthetic_gguf(paths["gguf"], tiny_qwen3_config(layers=2, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=3, device="cpu")
    paths["st"] = str(tmp_path / "single.safetensors")
    save_file(llama_like(qk_norm=True), paths["st"])
    paths["st_noext"] = str(tmp_path / "weights.bin")                              # content decides, not the extension
    save_file(llama_like(bias=True), paths["st_noext"])
    paths["ptor"] = str(tmp_path / "m.ptor")
    S.save_state_dict(llama_like(), paths["ptor"])
    hf = tmp_path / "hf"
    hf.mkdir()
    full = llama_like(layers=3)
    names = list(full)
    shard_a, shard_b = OrderedDict((k, full[k]) for k in names[:10]), OrderedDict((k, full[k]) for k in names[10:])
    save_file(shard_a, str(hf / "model-00001-of-00002.safetensors"))
    save_file(shard_b, str(hf / "model-00002-of-00002.safetensors"))
    (hf / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {**{k: "model-00001-of-00002.safetensors" for k in shard_a},
                                                                                 **{k: "model-00002-of-00002.safetensors" for k in shard_b}}}))
    (hf / "config.json").write_text(json.dumps({"model_type": "llama", "hidden_size": 128, "num_hidden_layers": 3, "num_attention_heads": 2,
                                                "num_key_value_heads": 1, "intermediate_size": 192, "vocab_size": 300, "rms_norm_eps": 1e-5,
                                                "rope_theta": 500000.0, "max_position_embeddings": 2048, "tie_word_embeddings": True}))
    paths["hf_dir"] = str(hf)
    paths["shard"] = str(hf / "model-00002-of-00002.safetensors")                 # naming a shard finds its siblings
    for key, path in paths.items():
        got = _run(exe, "model", path, "bytes")
        want = ML.load_model(path)
        assert got["detected"] == got["format"] == want.format == ML.detect_format(path), key
        assert got["architecture"] == want.architecture, (key, got["architecture"], want.architecture)
        wc = dataclasses.asdict(want.config)
        wc.pop("extra")
        assert got["config"] == pytest.approx(wc), (key, got["config"], wc)
        assert set(got["tensors"]) == set(want.tensors), key
        if key in ("st", "st_noext", "ptor"):                                      # file order is kept for the containers that have one
            assert list(got["tensors"]) == list(want.tensors), key
        assert got["files"] == want.files and got["total_parameters"] == want.total_parameters(), key
        for name, info in want.tensors.items():
            e = got["tensors"][name]
            assert e["dtype"] == info.dtype and e["shape"] == info.shape and e["file"] == info.file, (key, name, e, info)
            if want.format != "gguf":
                raw = ML.read_tensor(want, name).contiguous().reshape(-1).view(torch.uint8)
                assert e["nbytes"] == raw.numel() and e["byte_sum"] == int(raw.long().sum()), (key, name)
    # a .pt zip and a pickle are recognised; junk and short files are not
    pt_path = str(tmp_path / "m.pt")
    torch.save({"w": torch.ones(2)}, pt_path)
    assert _run(exe, "model", pt_path)["format"] == "pytorch"
    (tmp_path / "junk.dat").write_bytes(b"\x00" * 64)
    (tmp_path / "short").write_bytes(b"ab")
    for bad in ("junk.dat", "short", "nothing-here"):
        r = subprocess.run([exe, "model", str(tmp_path / bad)], capture_output=True, timeout=60)
        assert r.returncode == 1 and b"unknown model format" in r.stderr, bad


def test_native_block_dequantisers_match_python(exe, tmp_path):
    """gguf_cpu.h: every block format the C++ decoder reads, on random block bytes (scale fields set to finite halves), against the
    dequantisers of the Python package; Q2_K and Q3_K have no quantiser here, so random bytes are their only source."""
    from prometorch_b200.io import gguf_quant as GQ
    g = torch.Generator().manual_seed(7)
    half_fields = {GQ.GGMLType.Q4_0: [0], GQ.GGMLType.Q8_0: [0], GQ.GGMLType.Q2_K: [80, 82], GQ.GGMLType.Q3_K: [108], GQ.GGMLType.Q4_K: [0, 2],
                   GQ.GGMLType.Q5_K: [0, 2], GQ.GGMLType.Q6_K: [208]}
    for qt, fields in half_fields.items():
        bb = GQ.row_bytes(qt, 256) // (256 // (32 if qt in (GQ.GGMLType.Q4_0, GQ.GGMLType.Q8_0) else 256))
        n_blocks = 24
        raw = torch.randint(0, 256, (n_blocks, bb), generator=g, dtype=torch.int32).to(torch.uint8)
        scales = (torch.rand(n_blocks, len(fields), generator=g) * 0.1 - 0.03).to(torch.float16)
        for j, off in enumerate(fields):
            raw[:, off:off + 2] = scales[:, j:j + 1].contiguous().view(torch.uint8)
        f = tmp_path / f"blocks_{int(qt)}.bin"
        f.write_bytes(raw.numpy().tobytes())
        got = torch.tensor(_run(exe, "dequant", str(int(qt)), str(f)))
        elems = 32 if qt in (GQ.GGMLType.Q4_0, GQ.GGMLType.Q8_0) else 256
        want = GQ.dequantize(raw.reshape(1, -1), qt, n_blocks * elems).reshape(-1)
        assert got.numel() == want.numel() and torch.allclose(got, want, atol=1e-6, rtol=1e-6), (qt, float((got - want).abs().max()))


def test_native_cpu_decoder_matches_the_python_oracle(exe, tmp_path):
    """gguf_cpu.h: the C++ CPU decoder (blocks dequantised on the fly) gives the logits and the greedy ids of the fp32 oracle of
    the Python package, for the default quantisation mix and for Q5_K + Q8_0 and Q8_0 + F16 files."""
    from prometorch_b200.io import gguf_quant as GQ
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.models.gguf_oracle import OracleModel
    prompt = [300, 301, 17, 260, 5]
    for tag, q_main, q_more in (("q4km", GQ.GGMLType.Q4_K, GQ.GGMLType.Q6_K), ("q5k_q80", GQ.GGMLType.Q5_K, GQ.GGMLType.Q8_0),
                                ("q80_f16", GQ.GGMLType.Q8_0, GQ.GGMLType.F16), ("q40_q80", GQ.GGMLType.Q4_0, GQ.GGMLType.Q8_0)):
        path = str(tmp_path / f"{tag}.gguf")
        write_synthetic_gguf(path, tiny_qwen3_config(layers=2, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=11, device="cpu",
                             q_main=q_main, q_more=q_more, std=0.05)
        got = _run(exe, "cpu-generate", path, "8", *[str(t) for t in prompt])
        oracle = OracleModel(path, max_seq=256)
        oracle.forward(prompt)
        probe = oracle.forward([prompt[-1]])[-1]
        assert torch.allclose(torch.tensor(got["probe_logits"]), probe[:24], atol=2e-3, rtol=2e-3), tag
        assert got["probe_argmax"] == int(probe.argmax()), tag
        want, gaps = [], []
        oracle.reset()
        lg = oracle.forward(prompt)
        for _ in range(8):
            top = lg[-1].topk(2).values
            gaps.append(float(top[0] - top[1]))
            want.append(int(lg[-1].argmax()))
            lg = oracle.forward([want[-1]])
        for i, (a, b) in enumerate(zip(got["ids"], want)):                         # only a near-tie may split the two
            if a != b:
                assert gaps[i] < 1e-3, (tag, i, got["ids"], want, gaps)
                break
        else:
            assert got["ids"] == want, tag


def test_native_server_serves_a_gguf_file_on_the_cpu(exe, tmp_path):
    """The whole native stack without a GPU: HTTP -> C++ tokenizer -> C++ CPU decoder -> detokenised NDJSON; greedy answers equal
    the Python oracle with the Python tokenizer, sampled answers are reproducible per seed."""
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.gguf import GGUFReader
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.io.tokenizer import GGUFTokenizer
    from prometorch_b200.models.gguf_oracle import OracleModel
    path = str(tmp_path / "served.gguf")
    write_synthetic_gguf(path, tiny_qwen3_config(layers=2, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=12, device="cpu", std=0.05)
    tok = GGUFTokenizer.from_reader(GGUFReader(path))
    prompt = "t300 t301 t400 t260"
    ids = tok.encode(prompt)
    want = OracleModel(path, max_seq=256).generate_greedy(ids, 6)
    stop = {tok.eos_id}
    for i, t in enumerate(want):
        if t in stop:
            want = want[:i + 1]
            break
    s = Server(exe, "--gguf", path)
    try:
        greedy = {"num_predict": 6, "temperature": 0.0, "repeat_penalty": 1.0}
        st, _, data = _req(s.port, "POST", "/api/generate", {"model": "cpu-model", "prompt": prompt, "raw": True, "stream": False, "options": greedy})
        out = json.loads(data)
        assert st == 200 and out["prompt_eval_count"] == len(ids) and out["eval_count"] == len(want), (out, want)
        assert out["response"] == "".join(tok.decode_token(t) for t in want)
        show = json.loads(_req(s.port, "POST", "/api/show", {"model": "cpu-model"})[2])
        assert show["details"]["family"] == "qwen3" and show["model_info"]["general.name"] == "qwen3-tiny"
        sampled = {"num_predict": 8, "temperature": 1.2, "top_k": 30, "top_p": 0.95, "repeat_penalty": 1.1}
        runs = []
        for seed in (5, 5, 6):
            st, _, data = _req(s.port, "POST", "/api/generate", {"model": "cpu-model", "prompt": prompt, "raw": True, "options": dict(sampled, seed=seed)})
            lines = [json.loads(l) for l in data.decode().splitlines() if l.strip()]
            assert st == 200 and lines[-1]["done"] and 1 <= lines[-1]["eval_count"] <= 8
            runs.append("".join(l.get("response", "") for l in lines))
        assert runs[0] == runs[1]
        st, _, data = _req(s.port, "POST", "/api/chat", {"model": "cpu-model", "stream": False, "messages": [{"role": "user", "content": "t300"}],
                                                        "options": {"num_predict": 3, "temperature": 0.0, "repeat_penalty": 1.0}})
        assert st == 200 and json.loads(data)["message"]["role"] == "assistant" and json.loads(data)["eval_count"] >= 1
    finally:
        s.close()


def test_native_request_queue(exe):
    """serve::LLMEngine (submit_request / step / poll_responses / generate) behaves like the Python queue of the same name."""
    from prometorch_b200.serve import LLMEngine
    from test_serve_cpu import EchoBackend
    got = _run(exe, "engine")
    eng = LLMEngine(EchoBackend())
    a, b = eng.submit_request("one", max_tokens=3), eng.submit_request([ord(c) for c in "two"], max_tokens=5)
    assert got["ids"] == [a, b] and got["pending"] == 2
    assert got["first_step"] == eng.step() == 3
    assert got["after_first"] == {str(k): v for k, v in eng.poll_responses().items()} == {"0": [ord(c) for c in "hel"]}
    assert got["second_step"] == eng.step() == 5
    assert got["after_second"] == {str(k): v for k, v in eng.poll_responses().items()}
    assert got["empty_step"] == eng.step() == 0
    assert got["generate"] == eng.generate(["x", "y"], max_tokens=4) == ["hell", "hell"]


# ------------------------------------------------------------------------------------------------------------- server
class Server:
    def __init__(self, exe, *flags, env=None):
        self.p = subprocess.Popen([exe, "serve", *flags], stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, env=env)
        line = self.p.stdout.readline().decode()
        assert line.startswith("PORT "), line + self.p.stderr.read().decode()
        self.port = int(line.split()[1])

    def ask(self, word):
        self.p.stdin.write((word + "\n").encode())
        self.p.stdin.flush()
        return self.p.stdout.readline().decode().strip()

    def close(self):
        try:
            self.p.stdin.close()
            self.p.wait(timeout=20)
        except Exception:
            self.p.kill()


@pytest.fixture()
def server(exe):
    s = Server(exe)
    yield s
    s.close()


def _req(port, method, path, body=None, raw=None):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
    c.request(method, path, raw if raw is not None else (None if body is None else json.dumps(body)), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, dict(r.getheaders()), data


def test_native_server_routes(server):
    port = server.port
    st, hdr, data = _req(port, "GET", "/")
    assert st == 200 and b"PromeServe is running" in data
    st, hdr, data = _req(port, "GET", "/api/version")
    assert st == 200 and json.loads(data) == {"version": "0.1.0-promeserve"}
    st, hdr, data = _req(port, "GET", "/api/tags")
    tags = json.loads(data)["models"]
    e = [m for m in tags if m["name"] == "echo:1b"][0]
    assert st == 200 and e["model"] == "echo:1b" and e["size"] == 1234 and e["details"] == {"family": "qwen3", "format": "gguf", "parameter_size": "1B"}
    assert set(e) == {"name", "model", "modified_at", "size", "digest", "details"}
    st, hdr, data = _req(port, "POST", "/api/show", {"name": "echo:1b"})
    assert st == 200 and json.loads(data)["model_info"]["general.architecture"] == "qwen3"
    assert _req(port, "POST", "/api/show", {"model": "echo"})[0] == 200                      # the tag is optional
    assert _req(port, "POST", "/api/embeddings", {"model": "echo:1b", "prompt": "x"})[0] == 501
    assert _req(port, "GET", "/nope")[0] == 404
    st, hdr, data = _req(port, "OPTIONS", "/api/generate")
    assert st == 204 and hdr.get("Access-Control-Allow-Origin") == "*" and hdr.get("Access-Control-Allow-Methods") == "POST, GET, OPTIONS"
    assert hdr.get("Access-Control-Allow-Headers") == "Content-Type, Authorization"
    assert _req(port, "HEAD", "/api/tags")[0] == 200 and _req(port, "HEAD", "/other")[0] == 404


def test_native_server_generate_and_stream(server):
    port = server.port
    st, _, data = _req(port, "POST", "/api/generate", {"model": "echo:1b", "prompt": "hi", "stream": False, "raw": True,
                                                      "options": {"num_predict": 5, "temperature": 0.0}})
    out = json.loads(data)
    assert st == 200 and out["response"] == "hello" and out["done"] is True and out["eval_count"] == 5 and out["prompt_eval_count"] == 2
    assert out["model"] == "echo:1b" and out["load_duration"] == 0 and out["total_duration"] == out["prompt_eval_duration"] + out["eval_duration"]
    # options reach the backend; a raw prompt is not templated
    st, _, data = _req(port, "POST", "/api/generate", {"model": "mirror:1b", "prompt": "abc", "stream": False, "raw": True,
                                                      "options": {"top_k": 7, "temperature": 0.25}})
    assert json.loads(data)["response"] == "abc|7|25"
    st, _, data = _req(port, "POST", "/api/generate", {"model": "mirror:1b", "prompt": "abc", "stream": False, "system": "S"})
    assert json.loads(data)["response"].startswith("<|im_start|>system\nS<|im_end|>\n<|im_start|>user\nabc<|im_end|>\n<|im_start|>assistant\n|40|")
    # streaming: chunked NDJSON, one object per token, then the statistics
    st, hdr, data = _req(port, "POST", "/api/generate", {"model": "echo:1b", "prompt": "hi"})
    assert st == 200 and hdr.get("Content-Type") == "application/x-ndjson" and hdr.get("Transfer-Encoding") == "chunked"
    lines = [json.loads(l) for l in data.decode().splitlines() if l.strip()]
    assert "".join(l.get("response", "") for l in lines) == "hello world" and len(lines) == 12
    assert lines[-1]["done"] is True and all(not l["done"] for l in lines[:-1]) and lines[-1]["eval_count"] == 11
    assert all(set(l) == {"model", "created_at", "response", "done"} for l in lines[:-1])
    ps = json.loads(_req(port, "GET", "/api/ps")[2])
    assert {m["name"] for m in ps["models"]} >= {"echo:1b", "mirror:1b"} and ps["stats"]["requests"] == 4 and ps["stats"]["timeouts"] == 0
    assert ps["stats"]["tokens_generated"] >= 5 + 8 + 11 and ps["stats"]["prompt_tokens"] >= 2 + 3 + 2


def test_native_server_chat_and_tools(server):
    port = server.port
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hey"}]
    st, _, data = _req(port, "POST", "/api/chat", {"model": "mirror:1b", "stream": False, "messages": msgs})
    out = json.loads(data)
    assert st == 200 and out["message"]["role"] == "assistant"
    assert out["message"]["content"].startswith("<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhey<|im_end|>\n<|im_start|>assistant\n")
    st, hdr, data = _req(port, "POST", "/api/chat", {"model": "echo:1b", "messages": msgs})
    lines = [json.loads(l) for l in data.decode().splitlines() if l.strip()]
    assert "".join(l["message"]["content"] for l in lines) == "hello world" and lines[-1]["done"] and lines[-1]["message"]["content"] == ""
    tools = [{"type": "function", "function": {"name": "add", "parameters": {}}}]
    st, _, data = _req(port, "POST", "/api/chat", {"model": "tool:1b", "stream": False, "messages": msgs, "tools": tools})
    out = json.loads(data)
    assert out["message"]["tool_calls"] == [{"function": {"name": "add", "arguments": {"a": 1, "b": 2}}}]


def test_native_server_errors_and_limits(exe, tmp_path):
    s = Server(exe, "--max-body", "2000")
    try:
        st, _, data = _req(s.port, "POST", "/api/generate", {"model": "missing:7b", "prompt": "x", "stream": False})
        assert st == 404 and "error" in json.loads(data)
        assert _req(s.port, "POST", "/api/generate", raw="{not json")[0] == 400
        c = socket.create_connection(("127.0.0.1", s.port), timeout=10)
        c.sendall(b"POST /api/generate HTTP/1.1\r\nHost: x\r\nTransfer-Encoding: chunked\r\n\r\n5\r\nhello\r\n0\r\n\r\n")
        assert c.recv(4096).startswith(b"HTTP/1.1 400") 
        c.close()
        assert _req(s.port, "POST", "/api/generate", {"model": "echo:1b", "prompt": "x" * 5000})[0] == 413
        for bad in ("/etc/passwd", "../x", "a/b", "..", "a\\b"):
            st, _, data = _req(s.port, "POST", "/api/generate", {"model": bad, "prompt": "x", "stream": False})
            assert st == 404, bad
    finally:
        s.close()


def test_native_server_timeout_and_backpressure(exe):
    s = Server(exe, "--timeout-ms", "300", "--workers", "1", "--queue-depth", "1")
    try:
        t0 = time.time()
        st, _, data = _req(s.port, "POST", "/api/generate", {"model": "slow:1b", "prompt": "x", "raw": True, "options": {"num_predict": 200}})
        lines = [json.loads(l) for l in data.decode().splitlines() if l.strip()]
        assert st == 200 and lines[-1] == {"error": "timeout", "done": True} and 2 <= len(lines) < 40 and time.time() - t0 < 5
        # one worker busy, one connection queued: the next one is turned away
        socks = []
        for _ in range(2):
            c = socket.create_connection(("127.0.0.1", s.port), timeout=10)
            body = json.dumps({"model": "slow:1b", "prompt": "x", "raw": True, "options": {"num_predict": 200}})
            c.sendall(f"POST /api/generate HTTP/1.1\r\nHost: x\r\nContent-Length: {len(body)}\r\n\r\n{body}".encode())
            socks.append(c)
            time.sleep(0.05)
        st, hdr, _ = _req(s.port, "GET", "/api/version")
        assert st == 503 and hdr.get("Retry-After") == "1"
        for c in socks:
            c.close()
        time.sleep(0.8)
        assert _req(s.port, "GET", "/api/version")[0] == 200                          # and recovers
    finally:
        s.close()


def test_native_server_finds_models_on_disk(exe, tmp_path):
    """Model directories and the Ollama store: listing, loading by name, eviction of the least recently used."""
    d = tmp_path / "models"
    d.mkdir()
    for n in ("alpha", "beta", "gamma"):
        (d / f"{n}.gguf").write_bytes(b"x" * (10 + len(n)))
    store = tmp_path / "ollama"
    lib = store / "manifests" / "registry.ollama.ai" / "library" / "tiny"
    lib.mkdir(parents=True)
    (store / "blobs").mkdir()
    (store / "blobs" / "sha256-abc").write_bytes(b"y" * 77)
    (lib / "latest").write_text(json.dumps({"layers": [{"mediaType": "application/vnd.ollama.image.license", "digest": "sha256:zzz"},
                                                       {"mediaType": "application/vnd.ollama.image.model", "digest": "sha256:abc"}]}))
    other = store / "manifests" / "registry.ollama.ai" / "library" / "busted"
    other.mkdir(parents=True)
    (other / "latest").write_text(json.dumps({"layers": [{"mediaType": "application/vnd.ollama.image.model", "digest": "sha256:nope"}]}))
    s = Server(exe, "--model-dir", str(d), "--max-models", "2", env=dict(os.environ, OLLAMA_MODELS=str(store)))
    try:
        names = {m["name"]: m for m in json.loads(_req(s.port, "GET", "/api/tags")[2])["models"]}
        assert {"alpha", "beta", "gamma", "tiny:latest", "echo:1b"} <= set(names) and "busted:latest" not in names
        assert names["alpha"]["size"] == 15 and names["tiny:latest"]["size"] == 77
        show = json.loads(_req(s.port, "POST", "/api/show", {"model": "tiny"})[2])
        assert show["details"]["parameter_size"] == "load#1"
        assert _req(s.port, "POST", "/api/generate", {"model": "busted", "prompt": "x", "stream": False})[0] == 404
        base = int(s.ask("loaded").split()[1])
        for n in ("alpha", "beta", "alpha", "gamma"):                                   # gamma pushes out beta (alpha was used after it); tiny went first
            out = json.loads(_req(s.port, "POST", "/api/generate", {"model": n, "prompt": "x", "stream": False, "raw": True})[2])
            assert out["response"] == "hello world"
        assert int(s.ask("loaded").split()[1]) == base - 1 + 2
        tags = {m["name"]: m for m in json.loads(_req(s.port, "GET", "/api/tags")[2])["models"]}
        assert tags["alpha"]["details"]["parameter_size"] == "load#2" and tags["gamma"]["details"]["parameter_size"] == "load#4"
        assert tags["beta"]["details"]["parameter_size"] == ""                          # listed from disk again, not loaded
        # concurrent requests for a new name load it once
        out = []
        ts = [threading.Thread(target=lambda: out.append(json.loads(_req(s.port, "POST", "/api/show", {"model": "beta"})[2]))) for _ in range(4)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        assert {o["details"]["parameter_size"] for o in out} == {"load#5"}
    finally:
        s.close()


def test_native_generate_cli_prints_metadata_and_tensors(tmp_path):
    """`gguf_generate --info / --tensors` read the file without touching a GPU."""
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("needs nvcc to link the program against the native library")
    from prometorch_b200 import _build
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.gguf import GGUFReader
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    exe = str(_build.build_generate())
    path = str(tmp_path / "cli.gguf")
    write_synthetic_gguf(path, tiny_qwen3_config(layers=1, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=2, device="cpu")
    r = subprocess.run([exe, path, "--info", "--tensors"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stderr
    assert "general.architecture = 'qwen3'" in r.stdout and "architecture qwen3, 1 layers, hidden 256, 4 heads (2 kv), ffn 512" in r.stdout
    reader = GGUFReader(path)
    listed = {ln.split()[0]: ln for ln in r.stdout.splitlines() if ln.startswith(("blk.", "token_embd", "output"))}
    assert set(listed) == set(reader.tensors)
    for name, t in reader.tensors.items():
        assert listed[name].split()[-2] == str(t.nbytes) and t.qtype.name in listed[name]
    assert subprocess.run([exe], capture_output=True).returncode == 2
    assert subprocess.run([exe, path, "--bogus"], capture_output=True).returncode == 2
    r = subprocess.run([exe, str(tmp_path / "missing.gguf"), "--info"], capture_output=True, text=True)
    assert r.returncode == 1 and "cannot open" in r.stderr


def test_native_programs_run_on_the_cpu(tmp_path):
    """`lib/gguf_generate --device cpu` and `lib/promeserve --device cpu`: the shipped programs end to end without a GPU, against
    the fp32 oracle and the tokenizer of the Python package."""
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("needs nvcc to link the programs against the native library")
    from prometorch_b200 import _build
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.gguf import GGUFReader
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.io.tokenizer import GGUFTokenizer
    from prometorch_b200.models.gguf_oracle import OracleModel
    path = str(tmp_path / "prog.gguf")
    write_synthetic_gguf(path, tiny_qwen3_config(layers=2, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=13, device="cpu", std=0.05)
    tok = GGUFTokenizer.from_reader(GGUFReader(path))
    prompt = "t300 t301 t400 t260"
    ids = tok.encode(prompt)
    want = OracleModel(path, max_seq=256).generate_greedy(ids, 6)
    for i, t in enumerate(want):
        if t == tok.eos_id:
            want = want[:i + 1]
            break
    r = subprocess.run([str(_build.build_generate()), path, prompt, "--device", "cpu", "--greedy", "--max-tokens", "6"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(x) for x in [ln for ln in r.stdout.splitlines() if ln.startswith("[Ids]")][0].split()[1:]]
    assert got == want and "on CPU" in r.stdout and f"Prompt tokens: {len(ids)}" in r.stdout
    p = subprocess.Popen([str(_build.build_promeserve()), "--device", "cpu", "--model", path, "--port", "0", "--max-seq", "256"], stdout=subprocess.PIPE,
                         stderr=subprocess.PIPE, text=True)
    try:
        port = None
        for _ in range(50):
            line = p.stdout.readline()
            if not line:
                break
            if "listening on" in line:
                port = int(line.split(":")[-1].split()[0])
                assert "(cpu)" in line
                break
        assert port, p.stderr.read()[-2000:]
        st, _, data = _req(port, "POST", "/api/generate", {"model": "prog", "prompt": prompt, "raw": True, "stream": False,
                                                         "options": {"num_predict": 6, "temperature": 0.0, "repeat_penalty": 1.0}})
        out = json.loads(data)
        assert st == 200 and out["eval_count"] == len(want) and out["response"] == "".join(tok.decode_token(t) for t in want)
        assert any(m["name"] == "prog" for m in json.loads(_req(port, "GET", "/api/ps")[2])["models"])
        # a browser gets the chat page shipped in serve/web (found relative to the program); anything else the liveness text
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
        c.request("GET", "/", None, {"Accept": "text/html,application/xhtml+xml"})
        r = c.getresponse()
        page = r.read()
        c.close()
        assert r.status == 200 and r.getheader("Content-Type").startswith("text/html") and b"/api/chat" in page and b"/api/tags" in page
        assert _req(port, "GET", "/")[2] == b"PromeServe is running"
    finally:
        p.terminate()
        try:
            p.wait(timeout=20)
        except subprocess.TimeoutExpired:
            p.kill()


def test_native_cpu_decoder_reads_hugging_face_directories(exe, tmp_path):
    """gguf_cpu.h on a Hugging Face directory (config.json + safetensors, read in place): logits and greedy ids of transformers' own
    modules on the same weights, for Llama (F32, sharded), Qwen2 (biases, BF16) and Qwen3 (query / key norms, F16, tied head); then
    `lib/gguf_generate DIR --device cpu` end to end with the directory's tokenizer files."""
    transformers = pytest.importorskip("transformers")
    from prometorch_b200.io.safetensors import save_file
    prompt = [1, 17, 93, 4, 55]
    common = dict(vocab_size=400, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=96,
                  max_position_embeddings=128, rms_norm_eps=1e-5)
    cases = (("llama", transformers.LlamaConfig(**common, tie_word_embeddings=False), transformers.LlamaForCausalLM, torch.float32),
             ("qwen2", transformers.Qwen2Config(**common, tie_word_embeddings=False), transformers.Qwen2ForCausalLM, torch.bfloat16),
             ("qwen3", transformers.Qwen3Config(**common, head_dim=32, tie_word_embeddings=True), transformers.Qwen3ForCausalLM, torch.float16))
    refs = {}
    for tag, cfg, cls, dtype in cases:
        torch.manual_seed(5)
        ref = refs[tag] = cls(cfg).eval()
        with torch.no_grad():
            for n, p in ref.named_parameters():
                if n.endswith("bias") or "norm" in n:
                    p.add_(0.1 * torch.randn_like(p))                  # biases start at zero and norms at one: make them count
                p.copy_(p.to(dtype).float())                           # the values the file will hold
        d = tmp_path / tag
        d.mkdir()
        cfg.save_pretrained(str(d))
        sd = {k: v.to(dtype).contiguous() for k, v in ref.state_dict().items() if not (cfg.tie_word_embeddings and k == "lm_head.weight")}
        if tag == "llama":                                             # two shards with an index
            names = sorted(sd)
            parts = {"model-00001-of-00002.safetensors": names[:len(names) // 2], "model-00002-of-00002.safetensors": names[len(names) // 2:]}
            for fn, ks in parts.items():
                save_file({k: sd[k] for k in ks}, str(d / fn))
            (d / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": {k: fn for fn, ks in parts.items() for k in ks}}))
        else:
            save_file(sd, str(d / "model.safetensors"))
        got = _run(exe, "cpu-generate", str(d), "8", *[str(t) for t in prompt])
        with torch.no_grad():
            lg = ref(torch.tensor([prompt + [prompt[-1]]])).logits[0, -1]
            want = ref.generate(torch.tensor([prompt]), max_new_tokens=8, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(prompt):].tolist()
        assert torch.allclose(torch.tensor(got["probe_logits"]), lg[:24], atol=3e-3, rtol=3e-3), (tag, got["probe_logits"][:4], lg[:4])
        assert got["probe_argmax"] == int(lg.argmax()) and got["ids"] == want, (tag, got["ids"], want)
    # the shipped program on the Llama directory: tokenizer files of the directory, greedy ids of transformers
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        return
    from prometorch_b200 import _build
    from prometorch_b200.serve.llm import load_hf_tokenizer
    d = tmp_path / "llama"
    tokens, merges = _train_bpe(" ".join(TEXTS) + " the quick brown fox jumps over the lazy dog " * 10, 100)
    assert len(tokens) <= 400
    (d / "vocab.json").write_text(json.dumps({t: i for i, t in enumerate(tokens)}))
    (d / "merges.txt").write_text("#version: 0.2\n" + "\n".join(merges) + "\n")
    text = "the quick brown fox"
    ids = load_hf_tokenizer(str(d)).encode(text)
    r = subprocess.run([str(_build.build_generate()), str(d), text, "--device", "cpu", "--greedy", "--max-tokens", "6"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    got_ids = [int(x) for x in [ln for ln in r.stdout.splitlines() if ln.startswith("[Ids]")][0].split()[1:]]
    ref = refs["llama"]
    with torch.no_grad():
        want = ref.generate(torch.tensor([ids]), max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(ids):].tolist()
    eos = ref.config.eos_token_id
    want = want[:want.index(eos) + 1] if eos in want else want
    assert got_ids == want and f"Prompt tokens: {len(ids)}" in r.stdout, (got_ids, want, r.stdout[-500:])
    r = subprocess.run([str(_build.build_generate()), str(d), "--info", "--tensors"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "architecture llama (hf_dir), 2 layers, hidden 64, 4 heads (2 kv), ffn 96" in r.stdout, r.stdout[:400] + r.stderr[-400:]
    assert any(ln.startswith("model.layers.1.mlp.down_proj.weight") and "(64, 96)" in ln and "f32" in ln for ln in r.stdout.splitlines())
    # and the server program with the directory as its model
    tok = load_hf_tokenizer(str(d))
    p = subprocess.Popen([str(_build.build_promeserve()), "--device", "cpu", "--model", str(d) + "/", "--port", "0", "--max-seq", "128"], stdout=subprocess.PIPE,
                         stderr=subprocess.PIPE, text=True)
    try:
        port = None
        for _ in range(50):
            line = p.stdout.readline()
            if not line:
                break
            if "listening on" in line:
                port = int(line.split(":")[-1].split()[0])
                break
        assert port, p.stderr.read()[-2000:]
        st, _, data = _req(port, "POST", "/api/generate", {"model": "llama", "prompt": text, "raw": True, "stream": False,
                                                         "options": {"num_predict": 6, "temperature": 0.0, "repeat_penalty": 1.0}})
        out = json.loads(data)
        assert st == 200 and out["prompt_eval_count"] == len(ids) and out["response"] == "".join(tok.decode_token(t) for t in want), out
        tags = json.loads(_req(port, "GET", "/api/tags")[2])["models"]
        assert any(m["name"] == "llama" and m["details"]["family"] == "llama" for m in tags), tags
    finally:
        p.terminate()
        try:
            p.wait(timeout=20)
        except subprocess.TimeoutExpired:
            p.kill()
