"""The native server (cpp_api/apps/promeserve.cpp) on a GPU: a synthetic GGUF file served by the C++ HTTP front end, the C++
tokenizer and the CUDA decode engine, compared with the Python model and tokenizer on the same file."""
import http.client
import json
import os
import subprocess
import time

import pytest

pytestmark = pytest.mark.gpu


def _post(port, path, body):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
    c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, data


def test_native_promeserve_serves_a_gguf_file(tmp_path):
    from prometorch_b200 import _build
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.io.tokenizer import GGUFTokenizer
    exe = _build.build_promeserve()
    path = str(tmp_path / "tiny.gguf")
    write_synthetic_gguf(path, tiny_qwen3_config(layers=2, hidden=512, heads=8, kv_heads=2, inter=1024, vocab=1024), seed=5, device="cpu")
    m = GGUFModel(path, device="cuda", max_seq=256)
    tok = GGUFTokenizer.from_reader(m.reader)
    prompt = "t300 t301 t17 t5"
    ids = tok.encode(prompt)
    assert len(ids) >= 2
    want = m.run_script(ids, 12)
    m.close()
    stop = {tok.eos_id} | {tok.vocab[t] for t in ("<|im_end|>", "<|eot_id|>", "<end_of_turn>", "<|end|>", "<|endoftext|>") if t in tok.vocab}
    for i, t in enumerate(want):                          # the server stops after a stop token, the scripted run does not
        if t in stop:
            want = want[:i + 1]
            break
    p = subprocess.Popen([str(exe), "--model", path, "--port", "0", "--max-seq", "256"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        port = None
        t0 = time.time()
        while time.time() - t0 < 120:
            line = p.stdout.readline()
            if not line:
                break
            if "listening on" in line:
                port = int(line.rsplit(":", 1)[1].split()[0])
                break
        assert port, p.stderr.read()[-2000:]
        greedy = {"num_predict": 12, "temperature": 0.0, "repeat_penalty": 1.0}
        st, data = _post(port, "/api/generate", {"model": "tiny", "prompt": prompt, "raw": True, "stream": False, "options": greedy})
        out = json.loads(data)
        assert st == 200 and out["done"] and out["prompt_eval_count"] == len(ids), out
        assert out["eval_count"] == len(want) and out["response"] == "".join(tok.decode_token(t) for t in want), (out, want)
        # streamed, sampled on the device: valid pieces, the statistics at the end, a different seed may differ
        st, data = _post(port, "/api/generate", {"model": "tiny", "prompt": prompt, "raw": True,
                                                "options": {"num_predict": 8, "temperature": 0.8, "top_k": 20, "top_p": 0.9, "seed": 7}})
        lines = [json.loads(l) for l in data.decode().splitlines() if l.strip()]
        assert st == 200 and lines[-1]["done"] and 1 <= lines[-1]["eval_count"] <= 8 and len(lines) == lines[-1]["eval_count"] + 1
        st, data = _post(port, "/api/chat", {"model": "tiny", "stream": False, "messages": [{"role": "user", "content": "t9"}],
                                            "options": {"num_predict": 4, "temperature": 0.0, "repeat_penalty": 1.0}})
        assert st == 200 and json.loads(data)["message"]["role"] == "assistant"
    finally:
        p.terminate()
        try:
            p.wait(timeout=30)
        except subprocess.TimeoutExpired:
            p.kill()


def test_native_generate_cli_matches_the_python_model(tmp_path):
    """`lib/gguf_generate` (C++ from the file to the printed text) against the Python model and tokenizer."""
    from prometorch_b200 import _build
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.io.tokenizer import GGUFTokenizer
    exe = str(_build.build_generate())
    path = str(tmp_path / "tiny.gguf")
    write_synthetic_gguf(path, tiny_qwen3_config(layers=2, hidden=512, heads=8, kv_heads=2, inter=1024, vocab=1024), seed=6, device="cpu")
    m = GGUFModel(path, device="cuda", max_seq=256)
    tok = GGUFTokenizer.from_reader(m.reader)
    prompt = "t400 t401 t27 t900 t5"
    ids = tok.encode(prompt)
    want = m.run_script(ids, 10)
    m.close()
    stop = {tok.eos_id} | {tok.vocab[t] for t in ("<|im_end|>", "<|eot_id|>", "<end_of_turn>", "<|end|>", "<|endoftext|>") if t in tok.vocab}
    for i, t in enumerate(want):
        if t in stop:
            want = want[:i + 1]
            break
    r = subprocess.run([exe, path, prompt, "--greedy", "--max-tokens", "10", "--profile"], capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    got = [int(x) for x in [ln for ln in r.stdout.splitlines() if ln.startswith("[Ids]")][0].split()[1:]]
    assert got == want, (got, want)
    assert f"[Generate] Prompt tokens: {len(ids)}" in r.stdout and "tok/s" in r.stdout
    assert "[Profile] qkv" in r.stdout and "[Profile] lm_head" in r.stdout
    # sampled on the device: the seed decides the draw
    runs = []
    for seed in ("3", "3", "4"):
        r = subprocess.run([exe, path, prompt, "--max-tokens", "12", "--temp", "1.5", "--top-k", "50", "--top-p", "0.95", "--seed", seed, "--chat"],
                           capture_output=True, text=True, timeout=240)
        assert r.returncode == 0, r.stderr[-2000:]
        runs.append([int(x) for x in [ln for ln in r.stdout.splitlines() if ln.startswith("[Ids]")][0].split()[1:]])
        assert 1 <= len(runs[-1]) <= 12 and all(0 <= t < 1024 for t in runs[-1])
    assert runs[0] == runs[1]
