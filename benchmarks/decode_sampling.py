#!/usr/bin/env python
"""Sampled decoding against greedy decoding through the public ``GGUFModel.generate`` call, one GPU.

    python benchmarks/decode_sampling.py [--tokens 128] [--model qwen3-4b|tiny]

The reference samples on the host and is 1.84x slower with T=0.7 / top-k 40 / top-p 0.9 than greedy
(BENCH_A100_HEAVY.md:86-91: 45.8 vs 84.4 tok/s).  Here the sampler is one kernel on the device; both modes
step token by token through the serving loop (token id in, token id out) so the ratio isolates sampling."""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--model", default="qwen3-4b", choices=["qwen3-4b", "tiny"])
    a = ap.parse_args()
    from prometorch_b200.io.config import qwen3_4b_config, tiny_qwen3_config
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    dev = "cuda:0"
    cfg = qwen3_4b_config() if a.model == "qwen3-4b" else tiny_qwen3_config(layers=4, hidden=1024, heads=16, kv_heads=8, inter=2048, vocab=4096)
    path = f"/tmp/ptb200_{a.model}_q4km_seed0.gguf"
    if not os.path.exists(path):
        write_synthetic_gguf(path + ".tmp", cfg, seed=0, device=dev)
        os.replace(path + ".tmp", path)
    model = GGUFModel(path, device=dev, max_seq=1024, want_logits=True)
    prompt = torch.randint(0, cfg.vocab_size, (64,), generator=torch.Generator().manual_seed(1)).tolist()
    res = {}
    for name, kw in (("greedy", dict(temperature=0.0)), ("sampled", dict(temperature=0.7, top_k=40, top_p=0.9, repeat_penalty=1.1))):
        model.generate(prompt, 8, on_token=lambda t: True, **kw)                  # warm-up (graph capture, sampler buffers)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = model.generate(prompt, a.tokens, on_token=lambda t: True, **kw)
        torch.cuda.synchronize()
        res[name] = len(out) / (time.perf_counter() - t0)
    # the sampling kernel alone, on the model's logits buffer
    from prometorch_b200.ops.sampling import DeviceSampler
    samp = DeviceSampler(model.logits_view().numel(), dev)
    samp.reset(prompt)
    lg = model.logits_view()
    for _ in range(3):
        samp.sample(lg, 0.7, 40, 0.9, 1.1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    import ctypes as C
    from prometorch_b200 import _native as N
    st = torch.cuda.current_stream().cuda_stream
    e0.record()
    for i in range(50):
        N.lib().ptb_sample_logits(lg.data_ptr(), lg.numel(), samp.hist.data_ptr(), samp.n_hist, samp.hist.numel(), 1.1, 0.7, 40, 0.9,
                                  0.37, samp.scratch.data_ptr(), samp.out.data_ptr(), None, st)
    e1.record()
    torch.cuda.synchronize()
    res["kernel_us"] = e0.elapsed_time(e1) / 50 * 1e3
    print(json.dumps({"metric": "sampled vs greedy decode (serving loop)", "sampler_kernel_us": round(res["kernel_us"], 1), "greedy_tok_s": round(res["greedy"], 1),
                      "sampled_tok_s": round(res["sampled"], 1), "slowdown": round(res["greedy"] / res["sampled"], 3),
                      "reference_slowdown": 1.84, "tokens": a.tokens, "model": a.model}))
    model.close()


if __name__ == "__main__":
    main()
