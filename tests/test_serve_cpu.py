"""PromeServe over real sockets with a fake model backend: routes, NDJSON streaming, chat, errors, LLMEngine."""
import http.client
import json

import pytest

from prometorch_b200.serve import LLMEngine, ModelBackend, PromeServe, ServerConfig


class EchoBackend(ModelBackend):
    """Token = one character; generation spells a fixed answer."""
    name, architecture, model_name, size, parameter_size = "echo:1b", "qwen3", "echo", 1234, "1B"
    answer = "hello world"

    def encode(self, text):
        return [ord(c) for c in text]

    def decode_token(self, tid):
        return chr(tid)

    def generate(self, prompt_ids, options, on_token):
        self.last_prompt = "".join(chr(t) for t in prompt_ids)
        self.last_options = dict(options)
        for c in self.answer[:int(options.get("num_predict", 128))]:
            if not on_token(ord(c)):
                break
        return 0.001, 0.002


@pytest.fixture()
def server():
    be = EchoBackend()
    srv = PromeServe(ServerConfig(host="127.0.0.1", port=0, worker_threads=2), {"echo:1b": be}).start()
    yield srv, be
    srv.stop()


def _req(port, method, path, body=None):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
    c.request(method, path, None if body is None else json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, dict(r.getheaders()), data


def test_basic_routes(server):
    srv, _ = server
    st, hdr, data = _req(srv.port, "GET", "/")
    assert st == 200 and b"PromeServe is running" in data
    st, hdr, data = _req(srv.port, "GET", "/api/version")
    assert st == 200 and "version" in json.loads(data)
    st, hdr, data = _req(srv.port, "GET", "/api/tags")
    assert st == 200 and any(m["name"] == "echo:1b" for m in json.loads(data)["models"])
    st, hdr, data = _req(srv.port, "POST", "/api/show", {"name": "echo:1b"})
    assert st == 200
    st, hdr, data = _req(srv.port, "POST", "/api/embeddings", {"model": "echo:1b", "prompt": "x"})
    assert st == 501
    st, hdr, data = _req(srv.port, "GET", "/nope")
    assert st == 404
    st, hdr, data = _req(srv.port, "OPTIONS", "/api/generate")
    assert st == 204 and hdr.get("Access-Control-Allow-Origin") == "*"


def test_chat_page_for_browsers(tmp_path):
    """GET / with ``Accept: text/html`` answers the chat page (the shipped one, or ``web_root``'s); other clients keep the liveness text."""
    def get(port, path, accept=None):
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
        c.request("GET", path, None, {"Accept": accept} if accept else {})
        r = c.getresponse()
        data = r.read()
        c.close()
        return r.status, r.getheader("Content-Type"), data
    srv = PromeServe(ServerConfig(host="127.0.0.1", port=0, worker_threads=2), {"echo:1b": EchoBackend()}).start()
    try:
        st, ct, page = get(srv.port, "/", "text/html,application/xhtml+xml")
        assert st == 200 and ct.startswith("text/html") and b"/api/chat" in page and b"/api/tags" in page and b"<script src" not in page
        assert get(srv.port, "/index.html")[1].startswith("text/html")
        assert get(srv.port, "/")[2] == b"PromeServe is running" and get(srv.port, "/", "application/json")[2] == b"PromeServe is running"
    finally:
        srv.stop()
    (tmp_path / "index.html").write_text("<html>mine</html>")
    srv = PromeServe(ServerConfig(host="127.0.0.1", port=0, worker_threads=2, web_root=str(tmp_path)), {"echo:1b": EchoBackend()}).start()
    try:
        assert get(srv.port, "/", "text/html")[2] == b"<html>mine</html>"
    finally:
        srv.stop()
    srv = PromeServe(ServerConfig(host="127.0.0.1", port=0, worker_threads=2, web_root=str(tmp_path / "absent")), {"echo:1b": EchoBackend()}).start()
    try:
        assert get(srv.port, "/", "text/html")[2] == b"PromeServe is running" and get(srv.port, "/index.html")[0] == 404
    finally:
        srv.stop()


def test_generate_non_streaming_and_options(server):
    srv, be = server
    st, _, data = _req(srv.port, "POST", "/api/generate", {"model": "echo:1b", "prompt": "hi", "stream": False, "raw": True,
                                                          "options": {"num_predict": 5, "temperature": 0.0}})
    out = json.loads(data)
    assert st == 200 and out["response"] == "hello" and out["done"] is True and out["eval_count"] == 5
    assert be.last_prompt == "hi" and int(be.last_options["num_predict"]) == 5
    assert out["model"] == "echo:1b" and "total_duration" in out
    st, _, data = _req(srv.port, "GET", "/api/ps")
    ps = json.loads(data)
    assert st == 200 and ps["models"][0]["name"] == "echo:1b" and ps["stats"] == {"requests": 1, "tokens_generated": 5, "prompt_tokens": 2, "timeouts": 0}


def test_generate_streams_ndjson(server):
    srv, _ = server
    st, hdr, data = _req(srv.port, "POST", "/api/generate", {"model": "echo:1b", "prompt": "hi"})
    assert st == 200 and "ndjson" in hdr.get("Content-Type", "")
    lines = [json.loads(l) for l in data.decode().splitlines() if l.strip()]
    assert "".join(l.get("response", "") for l in lines) == "hello world"
    assert lines[-1]["done"] is True and all(not l["done"] for l in lines[:-1])


def test_chat_applies_template(server):
    srv, be = server
    st, _, data = _req(srv.port, "POST", "/api/chat", {"model": "echo:1b", "stream": False,
                                                      "messages": [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hey"}]})
    out = json.loads(data)
    assert st == 200 and out["message"]["role"] == "assistant" and out["message"]["content"] == "hello world"
    assert "<|im_start|>system\nbe brief<|im_end|>" in be.last_prompt and be.last_prompt.endswith("<|im_start|>assistant\n")


def test_errors(server):
    srv, _ = server
    st, _, data = _req(srv.port, "POST", "/api/generate", {"model": "missing:7b", "prompt": "x", "stream": False})
    assert st == 404 and "error" in json.loads(data)
    c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=20)
    c.request("POST", "/api/generate", "{not json", {"Content-Type": "application/json"})
    r = c.getresponse()
    assert r.status == 400
    c.close()
    import socket
    k = socket.create_connection(("127.0.0.1", srv.port), timeout=10)
    k.sendall(b"POST /api/generate HTTP/1.1\r\nHost: x\r\nTransfer-Encoding: chunked\r\n\r\n5\r\nhello\r\n0\r\n\r\n")
    assert k.recv(4096).startswith(b"HTTP/1.1 400")
    k.close()


def test_llm_engine_queue():
    eng = LLMEngine(EchoBackend())
    a = eng.submit_request("one", max_tokens=3)
    b = eng.submit_request("two", max_tokens=5)
    assert eng.step() == 3
    assert eng.poll_responses() == {a: [ord(c) for c in "hel"]}
    assert eng.step() == 5 and list(eng.poll_responses()) == [b]
    assert eng.generate(["x", "y"], max_tokens=4) == ["hell", "hell"]


def _tiny_hf_dir(tmp_path):
    import json
    import torch
    from prometorch_b200.serve.llm import LlamaConfig, LlamaWeights, save_safetensors
    cfg = LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=256, eos_token_id=2)
    w = LlamaWeights.random(cfg, seed=21)
    d = tmp_path / "hf"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({k: getattr(cfg, k) for k in cfg.__dataclass_fields__}))
    save_safetensors(w.state_dict(), str(d / "model.safetensors"))
    return str(d), w


def test_engine_server_batches_concurrent_callers(tmp_path):
    """Requests submitted from several threads share decode batches and each gets its own tokens."""
    import threading
    from prometorch_b200.serve.llm import EngineServer, GenerationConfig, LLMEngine
    d, w = _tiny_hf_dir(tmp_path)
    eng = LLMEngine(device="cpu", max_pages=32, max_active=4)
    assert eng.load(d)
    srv = EngineServer(eng)
    greedy = dict(temperature=0.0, repetition_penalty=1.0, top_k=1)
    prompts = [[1, 5 + i, 9, 40 + i] for i in range(4)]
    seen = {i: [] for i in range(4)}
    handles = {}
    gate = threading.Barrier(4)

    def client(i):
        gate.wait()
        handles[i] = srv.submit(prompts[i], GenerationConfig(max_new_tokens=12, **greedy), lambda t, i=i: seen[i].append(t) or True)
    ts = [threading.Thread(target=client, args=(i,)) for i in range(4)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for i in range(4):
        r = handles[i].wait(60)
        assert r is not None and r.token_ids == seen[i] and 1 <= len(seen[i]) <= 12
    # one by one on a fresh engine: the same tokens
    solo = LLMEngine(device="cpu", max_pages=32, max_active=1)
    solo.load(d)
    for i in range(4):
        assert solo.generate(prompts[i], GenerationConfig(max_new_tokens=12, **greedy)).token_ids == seen[i]
    assert srv.max_batch_seen >= 2
    # a hook that says stop ends its request early
    h = srv.submit(prompts[0], GenerationConfig(max_new_tokens=12, **greedy), lambda t: False)
    assert len(h.wait(60).token_ids) == 1
    srv.close()


def test_rest_server_serves_hf_directory_concurrently(tmp_path):
    import json
    import threading
    import urllib.request
    from prometorch_b200.serve import PromeServe, ServerConfig
    full, _ = _tiny_hf_dir(tmp_path)
    import os
    d = os.path.basename(os.path.normpath(full))            # requests name the model; the server looks in model_dirs
    srv = PromeServe(ServerConfig(port=0, device="cpu", worker_threads=4, model_dirs=[os.path.dirname(os.path.normpath(full))])).start()
    try:
        out = {}

        def call(i):
            body = json.dumps({"model": d, "prompt": f"hello {i}", "stream": False, "raw": True,
                               "options": {"num_predict": 6, "temperature": 0.0, "repeat_penalty": 1.0, "top_k": 1}}).encode()
            req = urllib.request.Request(f"http://127.0.0.1:{srv.port}/api/generate", data=body, headers={"Content-Type": "application/json"})
            out[i] = json.loads(urllib.request.urlopen(req, timeout=60).read())
        ts = [threading.Thread(target=call, args=(i,)) for i in range(3)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        assert all(out[i]["done"] and 1 <= out[i]["eval_count"] <= 6 and isinstance(out[i]["response"], str) for i in range(3))
        show = json.loads(urllib.request.urlopen(urllib.request.Request(
            f"http://127.0.0.1:{srv.port}/api/show", data=json.dumps({"model": d}).encode(), headers={"Content-Type": "application/json"}),
            timeout=30).read())
        assert show["details"]["family"] == "llama" and show["details"]["format"] == "safetensors"
        def post(path, body):
            req = urllib.request.Request(f"http://127.0.0.1:{srv.port}{path}", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
            return json.loads(urllib.request.urlopen(req, timeout=60).read())
        e1 = post("/api/embeddings", {"model": d, "prompt": "hello world"})["embedding"]
        e2 = post("/api/embed", {"model": d, "input": ["hello world", "something else"]})["embeddings"]
        assert len(e1) == 64 and abs(sum(x * x for x in e1) - 1.0) < 1e-3 and len(e2) == 2
        assert max(abs(a - b) for a, b in zip(e1, e2[0])) < 1e-5 and max(abs(a - b) for a, b in zip(e1, e2[1])) > 1e-3
        tags = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{srv.port}/api/tags", timeout=30).read())
        assert any(m["name"] == d and m["details"]["format"] == "safetensors" for m in tags["models"])
    finally:
        srv.stop()


def test_engine_server_survives_a_failing_step(tmp_path):
    """An exception inside a step ends the requests in flight with what they have and the thread keeps serving."""
    from prometorch_b200.serve.llm import EngineServer, GenerationConfig, LLMEngine
    d, _ = _tiny_hf_dir(tmp_path)
    eng = LLMEngine(device="cpu", max_pages=16, max_active=2)
    assert eng.load(d)
    srv = EngineServer(eng)
    greedy = dict(temperature=0.0, repetition_penalty=1.0, top_k=1)
    real = eng._forward_decode
    state = {"fail": True}

    def flaky(batch):
        if state["fail"]:
            state["fail"] = False
            raise RuntimeError("injected on the host")
        return real(batch)
    eng._forward_decode = flaky
    r1 = srv.submit([1, 7, 8], GenerationConfig(max_new_tokens=6, **greedy)).wait(60)
    assert r1 is not None and len(r1.token_ids) <= 6                 # ended early, not hung
    r2 = srv.submit([1, 7, 8], GenerationConfig(max_new_tokens=6, **greedy)).wait(60)
    assert r2 is not None and 1 <= len(r2.token_ids) <= 6 and eng.kv.pages_in_use == 0
    srv.close()


def test_paged_backend_stops_when_the_client_hook_says_so(tmp_path):
    from prometorch_b200.serve.server import PagedBackend
    d, _ = _tiny_hf_dir(tmp_path)
    b = PagedBackend(d, "tiny", device="cpu", max_active=2, max_pages=16)
    seen = []
    pe, ev = b.generate([1, 5, 9], {"num_predict": 40, "temperature": 0.0, "repeat_penalty": 1.0, "top_k": 1},
                        lambda t: seen.append(t) or len(seen) < 3)
    assert len(seen) == 3 and pe >= 0 and ev >= 0
    assert b.server.call(lambda eng: (eng.num_active(), eng.kv.pages_in_use)) == (0, 0)
    b.server.close()


def test_server_rejects_paths_big_bodies_and_caps_loaded_models(tmp_path):
    """A request cannot make the server open arbitrary files, post unbounded bodies or pile up models."""
    import json
    import urllib.error
    import urllib.request
    from prometorch_b200.serve.server import ApiHandlers, ModelBackend, PromeServe, ServerConfig
    srv = PromeServe(ServerConfig(port=0, device="cpu", max_body_bytes=1024)).start()
    try:
        def post(body: bytes):
            req = urllib.request.Request(f"http://127.0.0.1:{srv.port}/api/generate", data=body, headers={"Content-Type": "application/json"})
            try:
                return urllib.request.urlopen(req, timeout=30).status
            except urllib.error.HTTPError as e:
                return e.code
        assert srv.config.host == "127.0.0.1"
        for name in ("/etc/passwd", "../../secret", "a/b"):
            assert post(json.dumps({"model": name, "prompt": "x", "stream": False}).encode()) == 404
        assert post(b"{" + b" " * 4096 + b"}") == 413
    finally:
        srv.stop()

    closed, loads = [], []

    class Fake(ModelBackend):
        def __init__(self, n):
            self.name = n

        def close(self):
            closed.append(self.name)

    def loader(n):
        loads.append(n)
        return Fake(n)
    h = ApiHandlers(ServerConfig(max_loaded_models=2), {"pinned": Fake("pinned")}, loader)
    for n in ("a", "b", "a", "c"):
        h.ensure_model(n)
    assert loads == ["a", "b", "c"] and closed == ["b"]          # "a" was used more recently than "b"
    assert set(h.backends) == {"pinned", "a", "c"}


def test_python_server_serves_a_gguf_file_on_the_cpu(tmp_path):
    """`--device cpu`: a GGUF file behind the fp32 oracle; greedy answers equal the oracle's own continuation."""
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.models.gguf_oracle import OracleModel
    from prometorch_b200.serve.server import OracleBackend
    d = tmp_path / "models"
    d.mkdir()
    path = str(d / "tiny.gguf")
    write_synthetic_gguf(path, tiny_qwen3_config(layers=2, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=14, device="cpu", std=0.05)
    srv = PromeServe(ServerConfig(port=0, device="cpu", model_dirs=[str(d)], max_seq=256)).start()
    try:
        prompt = "t300 t301 t400"
        st, _, data = _req(srv.port, "POST", "/api/generate", {"model": "tiny", "prompt": prompt, "raw": True, "stream": False,
                                                              "options": {"num_predict": 5, "temperature": 0.0, "repeat_penalty": 1.0}})
        out = json.loads(data)
        backend = srv.handlers.backends["tiny"]
        assert st == 200 and isinstance(backend, OracleBackend)
        ids = backend.encode(prompt)
        want = OracleModel(path, max_seq=256).generate_greedy(ids, 5)
        for i, t in enumerate(want):
            if t in backend.stop_ids:
                want = want[:i + 1]
                break
        assert out["eval_count"] == len(want) and out["response"] == "".join(backend.decode_token(t) for t in want)
        st, _, data = _req(srv.port, "POST", "/api/generate", {"model": "tiny", "prompt": prompt, "raw": True, "options": {"num_predict": 4, "seed": 3}})
        lines = [json.loads(l) for l in data.decode().splitlines() if l.strip()]
        assert st == 200 and lines[-1]["done"] and 1 <= lines[-1]["eval_count"] <= 4
    finally:
        srv.stop()
