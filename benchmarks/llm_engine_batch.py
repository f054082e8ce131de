"""Continuous-batching throughput of the paged-KV engine: tokens/s over all requests at several batch sizes.

    python benchmarks/llm_engine_batch.py [--batches 1,8,32] [--prompt 512] [--new 64] [--layers 16 --hidden 2048 ...]

Random bf16 weights of a Llama shape (no checkpoint needed); every request gets a random prompt.  Timed with CUDA
events around the decode steps only (the prompt passes are reported separately), after a warm-up request."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from prometorch_b200.serve.llm import GenerationConfig, LlamaConfig, LlamaWeights, LLMEngine, Request  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batches", default="1,8,32")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=64)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--inter", type=int, default=5632)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--sampled", action="store_true", help="temperature 0.8, top-k 50, top-p 0.9, repetition penalty 1.1 instead of greedy")
    ap.add_argument("--spec", type=int, default=0, help="n-gram speculative decoding: ids proposed per greedy request and pass")
    ap.add_argument("--repeat-prompt", type=int, default=0, help="build each prompt from a random piece of this length, repeated")
    a = ap.parse_args()
    cfg = LlamaConfig(vocab_size=a.vocab, hidden_size=a.hidden, intermediate_size=a.inter, num_hidden_layers=a.layers,
                      num_attention_heads=a.heads, num_key_value_heads=a.kv_heads, max_position_embeddings=a.prompt + a.new + 64,
                      eos_token_id=-1)
    w = LlamaWeights.random(cfg, seed=0, dtype=torch.bfloat16, device="cuda")
    greedy = GenerationConfig(max_new_tokens=a.new, temperature=0.0, repetition_penalty=1.0, top_k=1)
    if a.sampled:
        greedy = GenerationConfig(max_new_tokens=a.new, temperature=0.8, top_k=50, top_p=0.9, repetition_penalty=1.1)
    g = torch.Generator().manual_seed(0)
    for B in [int(x) for x in a.batches.split(",")]:
        pages = B * ((a.prompt + a.new) // 64 + 2)
        eng = LLMEngine(device="cuda", max_pages=pages, max_active=B, spec_tokens=a.spec)
        eng.set_weights(w)
        eng.generate(torch.randint(3, a.vocab, (16,), generator=g).tolist(), GenerationConfig(max_new_tokens=4, temperature=0.0,
                                                                                               repetition_penalty=1.0, top_k=1))
        for rep in range(2):                             # the first round captures the graphs; the second is timed
            for i in range(B):
                if a.repeat_prompt:
                    piece = torch.randint(3, a.vocab, (a.repeat_prompt,), generator=g).tolist()
                    prompt = (piece * (a.prompt // a.repeat_prompt + 1))[:a.prompt]
                else:
                    prompt = torch.randint(3, a.vocab, (a.prompt,), generator=g).tolist()
                eng.submit_request(Request(rep * B + i, prompt, greedy))
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            torch.cuda.synchronize()
            e0.record()
            eng.step()                               # prompt passes (+ the first token of each request)
            e1.record()
            steps = 0
            while eng.num_active():
                eng.step()
                steps += 1
            e2.record()
            torch.cuda.synchronize()
            done = eng.poll_responses()
        toks = sum(r.tokens_generated for r in done) - B
        # the device side of one decode pass alone: replay the captured graph back to back
        replay_ms = None
        if eng._graphs:
            graph = max(eng._graphs.items(), key=lambda kv: kv[0])[1][0]
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(3):
                graph.replay()
            r0.record()
            for _ in range(20):
                graph.replay()
            r1.record()
            torch.cuda.synchronize()
            replay_ms = round(r0.elapsed_time(r1) / 20, 3)
        print(json.dumps({"batch": B, "prompt_len": a.prompt, "decode_steps": steps, "prompt_pass_ms": round(e0.elapsed_time(e1), 2),
                          "prompt_tok_per_s": round(B * a.prompt / e0.elapsed_time(e1) * 1e3, 1),
                          "decode_ms_per_step": round(e1.elapsed_time(e2) / max(steps, 1), 3),
                          "decode_tok_per_s": round(toks / e1.elapsed_time(e2) * 1e3, 1), "graph_replay_ms": replay_ms,
                          "sampled": a.sampled, "spec_tokens": a.spec, "spec_accept_rate": round(eng.spec_accepted / max(eng.spec_drafted, 1), 3),
                          "model": f"llama {a.layers}L/{a.hidden}/{a.heads}h/{a.kv_heads}kv ffn{a.inter} bf16"}), flush=True)
        del eng
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
