"""The host-side C++ of the serving stack (JSON, tokenizer, chat templates, HTTP server with its worker pool) under
AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer: the same inputs as the functional tests, and any
report fails the run (the sanitizers exit non-zero and print to stderr)."""
import json
import os
import shutil
import subprocess
import threading

import pytest

import test_cpp_serve_cpu as S

ROOT = S.ROOT


def _build(tmp, name, flags):
    if shutil.which("g++") is None:
        pytest.skip("needs g++")
    out = str(tmp / name)
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags, os.path.join(ROOT, "tests", "cpp", "serve_native.cpp"), "-o", out,
           f"-I{ROOT}/prometorch_b200/cpp_api", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    if r.returncode != 0 and ("cannot find" in r.stderr or "unrecognized" in r.stderr):
        pytest.skip("this toolchain has no runtime for " + " ".join(flags))
    assert r.returncode == 0, r.stderr[-3000:]
    return out


def _clean(r):
    err = r.stderr.decode() if isinstance(r.stderr, bytes) else r.stderr
    assert r.returncode == 0 and "Sanitizer" not in err and "runtime error" not in err, err[-3000:]


@pytest.fixture(scope="module")
def asan_exe(tmp_path_factory):
    return _build(tmp_path_factory.mktemp("asan"), "serve_native_asan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"])


@pytest.fixture(scope="module")
def tsan_exe(tmp_path_factory):
    return _build(tmp_path_factory.mktemp("tsan"), "serve_native_tsan", ["-fsanitize=thread"])


ENV = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1", TSAN_OPTIONS="halt_on_error=0")


def test_tokenizer_json_and_chat_under_asan(asan_exe, tmp_path):
    from prometorch_b200.io.tokenizer import GGUFTokenizer
    tokens, merges = S._train_bpe(" ".join(S.TEXTS) * 2 + " the quick brown fox " * 10, 120)
    tokens += ["<|im_start|>", "<|im_end|>"]
    texts = S.TEXTS + ["\xff\xfe broken".encode("latin1").decode("latin1"), "a" * 3000, "<|im_start|>" * 50]
    spec = {"tokens": tokens, "model": "gpt2", "scores": [], "merges": merges, "types": [1] * (len(tokens) - 2) + [3, 3], "bos": -1, "eos": -1,
            "add_bos": False, "texts": texts}
    p = tmp_path / "gpt2.json"
    p.write_text(json.dumps(spec, ensure_ascii=False), encoding="utf-8")
    r = subprocess.run([asan_exe, "tokenize", str(p)], capture_output=True, timeout=300, env=ENV)
    _clean(r)
    py = GGUFTokenizer(tokens, "gpt2", None, merges, spec["types"], -1, -1, False)
    assert json.loads(r.stdout)["ids"] == [py.encode(t) for t in texts]
    bar = "▁"
    vocab = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + sorted(set("".join(S.TEXTS).replace(" ", bar) + bar) - set("\n\t")) + \
        [bar + "Hello", bar + "world", "ll", "he", bar + "he", "llo", bar + bar]
    spec = {"tokens": vocab, "model": "llama", "scores": [-float(i) for i in range(len(vocab))], "merges": [], "types": [], "bos": 1, "eos": 2,
            "add_bos": True, "texts": texts}
    p = tmp_path / "spm.json"
    p.write_text(json.dumps(spec, ensure_ascii=False), encoding="utf-8")
    r = subprocess.run([asan_exe, "tokenize", str(p)], capture_output=True, timeout=300, env=ENV)
    _clean(r)
    py = GGUFTokenizer(vocab, "llama", spec["scores"], None, None, 1, 2, True)
    assert json.loads(r.stdout)["ids"] == [py.encode(t) for t in texts]
    # malformed documents: the parser reports, it does not read out of bounds
    for i, bad in enumerate(['{"a": "\\u12', '{"a": [1, 2', '"\\ud800\\u0041"', '[' * 600, '{"k": tru', '"unterminated', '{"a": 1e999, "b": -}', '\\']):
        q = tmp_path / f"bad{i}.json"
        q.write_text(bad)
        r = subprocess.run([asan_exe, "json", str(q)], capture_output=True, timeout=60, env=ENV)
        err = r.stderr.decode()
        assert r.returncode in (0, 1) and "Sanitizer" not in err and "runtime error" not in err, (bad, err[-1500:])
    cases = [{"prompt": "q", "arch": a, "name": n, "system": s} for a in ("qwen3", "phi3", "gemma", "llama", "x") for n in ("", "Mistral") for s in ("", "S")]
    cases += [{"messages": [{"role": "user", "content": "u"}, {"role": "assistant", "content": "a"}, {"role": "user", "content": "v"}], "arch": "llama", "name": ""},
              {"strip": "<think>a</think>  b<think>"}]
    q = tmp_path / "chat.json"
    q.write_text(json.dumps(cases))
    _clean(subprocess.run([asan_exe, "chat", str(q)], capture_output=True, timeout=60, env=ENV))


def test_model_loader_on_damaged_files_under_asan(asan_exe, tmp_path):
    """Truncated and corrupted containers are reported as errors; the loader never reads out of bounds."""
    import struct
    import torch
    from prometorch_b200 import serialization as Ser
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.safetensors import save_file
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    good = {}
    good["st"] = tmp_path / "a.safetensors"
    save_file({"model.embed_tokens.weight": torch.randn(10, 8), "model.layers.0.self_attn.q_proj.weight": torch.randn(64, 8)}, str(good["st"]))
    good["ptor"] = tmp_path / "a.ptor"
    Ser.save_state_dict({"w": torch.randn(4, 4), "b": torch.zeros(4)}, str(good["ptor"]))
    good["gguf"] = tmp_path / "a.gguf"
    write_synthetic_gguf(str(good["gguf"]), tiny_qwen3_config(layers=1, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=3, device="cpu")
    cases = []
    for kind, path in good.items():
        raw = path.read_bytes()
        _clean(subprocess.run([asan_exe, "model", str(path), "bytes"], capture_output=True, timeout=120, env=ENV))
        for cut in (5, 9, 17, 40, len(raw) // 2, len(raw) - 1):
            q = tmp_path / f"{kind}_cut{cut}"
            q.write_bytes(raw[:cut])
            cases.append(q)
        flipped = bytearray(raw)
        for i in range(8, min(len(flipped), 200), 7):
            flipped[i] ^= 0xFF
        q = tmp_path / f"{kind}_flipped"
        q.write_bytes(bytes(flipped))
        cases.append(q)
    huge = tmp_path / "huge_header.safetensors"
    huge.write_bytes(struct.pack("<Q", 50 * 1024 * 1024) + b'{"a": 1}')
    bad_off = tmp_path / "bad_offsets.safetensors"
    hdr = b'{"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 800]}}'
    bad_off.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 8)
    cases += [huge, bad_off]
    for q in cases:
        r = subprocess.run([asan_exe, "model", str(q), "bytes"], capture_output=True, timeout=120, env=ENV)
        err = r.stderr.decode(errors="replace")
        assert r.returncode in (0, 1) and "Sanitizer" not in err and "runtime error" not in err, (q.name, err[-1500:])


def test_cpu_decoder_under_asan(asan_exe, tmp_path):
    """The C++ CPU decoder (block dequantisers, threads over rows, key / value cache) on a small file under ASan + UBSan."""
    from prometorch_b200.io import gguf_quant as GQ
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    for tag, q_main, q_more in (("a", GQ.GGMLType.Q4_K, GQ.GGMLType.Q6_K), ("b", GQ.GGMLType.Q5_K, GQ.GGMLType.Q8_0)):
        path = str(tmp_path / f"{tag}.gguf")
        write_synthetic_gguf(path, tiny_qwen3_config(layers=1, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=3, device="cpu",
                             q_main=q_main, q_more=q_more)
        r = subprocess.run([asan_exe, "cpu-generate", path, "4", "300", "301", "17"], capture_output=True, timeout=300, env=ENV)
        _clean(r)
        assert len(json.loads(r.stdout)["ids"]) == 4


def test_cpu_decoder_thread_pool_under_tsan(tsan_exe, tmp_path):
    """The worker pool that spreads the rows of every projection (job hand-over, part counter, completion wait) under TSan, with the
    same ids as the ASan build's single baseline path."""
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    path = str(tmp_path / "pool.gguf")
    write_synthetic_gguf(path, tiny_qwen3_config(layers=2, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=3, device="cpu")
    r = subprocess.run([tsan_exe, "cpu-generate", path, "6", "300", "301", "17"], capture_output=True, timeout=300, env=ENV)
    _clean(r)
    assert len(json.loads(r.stdout)["ids"]) == 6


def _hammer(exe, env, flags=()):
    s = S.Server(exe, *flags, env=env)
    try:
        errors = []

        def client(i):
            try:
                for _ in range(3):
                    st, _, data = S._req(s.port, "POST", "/api/generate", {"model": "echo:1b", "prompt": f"p{i}", "raw": True})
                    lines = [json.loads(l) for l in data.decode().splitlines() if l.strip()]
                    assert st == 200 and "".join(l.get("response", "") for l in lines) == "hello world"
                    st, _, data = S._req(s.port, "POST", "/api/chat", {"model": "mirror:1b", "stream": False, "messages": [{"role": "user", "content": f"m{i}"}]})
                    assert st == 200 and f"m{i}" in json.loads(data)["message"]["content"]
                    assert S._req(s.port, "GET", "/api/tags")[0] == 200
                    assert S._req(s.port, "POST", "/api/generate", raw="{broken")[0] == 400
                    assert S._req(s.port, "POST", "/api/show", {"model": "nobody"})[0] == 404
            except Exception as e:                       # noqa: BLE001
                errors.append(repr(e))
        ts = [threading.Thread(target=client, args=(i,)) for i in range(6)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        assert not errors, errors
    finally:
        s.close()
    err = s.p.stderr.read().decode()
    assert s.p.returncode == 0 and "Sanitizer" not in err and "runtime error" not in err, err[-4000:]


def test_server_under_asan(asan_exe):
    _hammer(asan_exe, ENV, ("--workers", "4"))


def test_server_under_tsan(tsan_exe):
    _hammer(tsan_exe, ENV, ("--workers", "4"))
