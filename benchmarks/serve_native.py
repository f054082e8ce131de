"""Served decode throughput of the native server: `lib/promeserve` (C++ HTTP front end, C++ tokenizer, CUDA decode engine)
answers one greedy streaming /api/generate request on the benchmark's synthetic Qwen3-4B-shape Q4_K_M file.

tok/s = eval_count / eval_duration of the final chunk (the server's own clock around the decode loop: engine steps, the
id crossing to the host, detokenisation and the chunked NDJSON write of every token), plus the wall clock of the whole
request seen by the client.  The Python server's figure for the same request is `served` in bench.py's line.

Run:  python benchmarks/serve_native.py [--model qwen3-4b] [--tokens 256] [--prompt-len 128]
"""
from __future__ import annotations

import argparse
import http.client
import json
import os
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-4b", choices=["qwen3-4b", "tiny"])
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--requests", type=int, default=3, help="the first one captures the graph; the best of the rest is reported")
    args = ap.parse_args()
    import bench as B
    from prometorch_b200 import _build
    exe = _build.build_promeserve()
    t0 = time.time()
    path, cfg = B.ensure_gguf(args.model, "cuda:0")
    t_file = time.time() - t0
    prompt = B.bench_prompt(cfg.vocab_size, args.prompt_len)
    text = " ".join(f"t{i}" for i in prompt)
    t0 = time.time()
    p = subprocess.Popen([str(exe), "--model", path, "--port", "0", "--max-seq", "4096"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    out = {"bench": "serve_native", "model": args.model, "file_s": round(t_file, 1)}
    try:
        port = None
        while time.time() - t0 < 240:
            line = p.stdout.readline()
            if not line:
                break
            if "listening on" in line:
                port = int(line.rsplit(":", 1)[1].split()[0])
                break
        if port is None:
            raise RuntimeError("the server did not come up: " + p.stderr.read()[-500:])
        out["load_s"] = round(time.time() - t0, 1)
        body = json.dumps({"model": os.path.basename(path)[:-5], "prompt": text, "raw": True, "stream": True,
                           "options": {"num_predict": args.tokens, "temperature": 0.0, "repeat_penalty": 1.0}})
        runs = []
        for _ in range(args.requests):
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=300)
            t1 = time.perf_counter()
            c.request("POST", "/api/generate", body, {"Content-Type": "application/json"})
            lines = [json.loads(l) for l in c.getresponse().read().decode().splitlines() if l.strip().startswith("{")]
            wall = time.perf_counter() - t1
            c.close()
            last = lines[-1]
            if "eval_count" not in last:
                raise RuntimeError(str(last)[:300])
            runs.append({"tok_s": round(last["eval_count"] / (last["eval_duration"] / 1e9), 2), "eval_count": last["eval_count"],
                         "prompt_eval_count": last["prompt_eval_count"], "prompt_eval_ms": round(last["prompt_eval_duration"] / 1e6, 2),
                         "chunks": len(lines), "request_wall_s": round(wall, 3)})
        best = max(runs[1:] or runs, key=lambda r: r["tok_s"])
        out.update(best, unit="tok/s", route="POST /api/generate (stream), native server", runs=[r["tok_s"] for r in runs])
    except Exception as e:                                   # noqa: BLE001
        out["error"] = repr(e)[:400]
    finally:
        p.terminate()
        try:
            p.wait(timeout=30)
        except subprocess.TimeoutExpired:
            p.kill()
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
