import argparse
import time

from .server import PromeServe, ServerConfig


def main():
    ap = argparse.ArgumentParser("promeserve")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=11434)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--model", default=None)
    ap.add_argument("--workers", type=int, default=4)
    ap.add_argument("--queue-depth", type=int, default=128)
    ap.add_argument("--timeout-ms", type=int, default=60000)
    ap.add_argument("--model-dir", action="append", default=[])
    ap.add_argument("--max-seq", type=int, default=4096)
    a = ap.parse_args()
    srv = PromeServe(ServerConfig(a.host, a.port, a.workers, a.queue_depth, a.timeout_ms, a.device, a.model, a.model_dir, a.max_seq)).start()
    print(f"[PromeServe] listening on {a.host}:{srv.port}")
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.stop()


if __name__ == "__main__":
    main()
