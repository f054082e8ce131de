import argparse
import time

from .server import PromeServe, ServerConfig


def main():
    ap = argparse.ArgumentParser("promeserve")
    ap.add_argument("--host", default="127.0.0.1", help="bind address; 0.0.0.0 serves other machines")
    ap.add_argument("--port", type=int, default=11434)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--model", default=None)
    ap.add_argument("--workers", type=int, default=4)
    ap.add_argument("--queue-depth", type=int, default=128)
    ap.add_argument("--timeout-ms", type=int, default=60000)
    ap.add_argument("--model-dir", action="append", default=[])
    ap.add_argument("--max-seq", type=int, default=4096)
    ap.add_argument("--max-models", type=int, default=2, help="models kept loaded at once")
    ap.add_argument("--allow-model-paths", action="store_true", help="let requests name models by filesystem path")
    ap.add_argument("--fp16-weights", "--fp16_weights", action="store_true",
                    help="accepted for compatibility with the reference's CLI: weights stay in their file format here")
    ap.add_argument("--web-root", default=None, help="folder whose index.html a browser gets at /; default: the page shipped with the package")
    a = ap.parse_args()
    # --model comes from the operator, so it may be a path even when requests may not name paths
    cfg = ServerConfig(a.host, a.port, a.workers, a.queue_depth, a.timeout_ms, a.device, None, a.model_dir, a.max_seq,
                       a.max_models, allow_model_paths=True, web_root=a.web_root)
    srv = PromeServe(cfg)
    if a.model:
        srv.handlers.ensure_model(a.model)
        srv.handlers.pinned.add(a.model)
    cfg.allow_model_paths = a.allow_model_paths
    srv.start()
    print(f"[PromeServe] listening on {a.host}:{srv.port}")
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.stop()


if __name__ == "__main__":
    main()
