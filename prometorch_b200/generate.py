"""Command-line text generation from a GGUF file (or an Ollama model name).

    python -m prometorch_b200.generate MODEL [PROMPT] [--device cuda|cpu] [--greedy] [--max-tokens N] [--temp T]
        [--top-k K] [--top-p P] [--chat | --raw] [--info] [--tensors] [--profile] [--nprocs N]

The flags are those of the reference's ``test_gguf_inference`` (examples/gguf/test_gguf_inference.cpp:76-120):
``--info`` prints the metadata and the parsed configuration, ``--tensors`` the tensor directory, ``--chat`` wraps the
prompt in the model's chat template, ``--profile`` prints per-kernel phase times of the last token, ``--nprocs N``
runs tensor-parallel over N processes.  Where the reference's tensor parallelism is CPU-only, here ``--nprocs`` drives
N GPUs (one process per GPU, re-launched under ``torch.distributed.run``) with the fused GEMV + all-reduce kernels.
``--fp16-weights`` and ``--llama-gemv`` select kernels that have no counterpart here and are accepted and ignored.
``--device cpu`` runs the fp32 oracle (slow; for checking); with ``--nprocs N`` it runs tensor-parallel over N CPU processes (gloo).
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("prometorch_b200.generate", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model")
    ap.add_argument("prompt", nargs="?", default=None)
    ap.add_argument("--info", action="store_true")
    ap.add_argument("--tensors", action="store_true")
    ap.add_argument("--device", default="cuda", choices=["cuda", "gpu", "cpu"])
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--greedy", action="store_true")
    ap.add_argument("--chat", action="store_true")
    ap.add_argument("--raw", action="store_true")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--fp16-weights", "--fp16_weights", action="store_true")
    ap.add_argument("--llama-gemv", "--llama_gemv", action="store_true")
    ap.add_argument("--max-tokens", "--max_tokens", type=int, default=128)
    ap.add_argument("--temp", "--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--repeat-penalty", type=float, default=1.05)
    from .utils.env import env_int, env_str
    ap.add_argument("--draft", default=env_str("SPEC_DRAFT_PATH"), help="a smaller GGUF model over the same vocabulary: greedy speculative decoding")
    ap.add_argument("--spec-k", type=int, default=env_int("SPEC_K", 4), help="tokens the draft proposes per verification pass")
    ap.add_argument("--nprocs", type=int, default=1)
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--master-addr", "--master_addr", default="127.0.0.1")
    ap.add_argument("--master-port", "--master_port", type=int, default=29500)
    a = ap.parse_args(argv)
    from .io.config import TransformerConfig
    from .io.gguf import GGUFReader
    from .io.ollama import resolve_model
    path = a.model if (os.sep in a.model or a.model.endswith(".gguf")) else resolve_model(a.model)
    if a.info or a.tensors:
        r = GGUFReader(path)
        if a.info:
            for k, v in r.metadata.items():
                s = repr(v)
                print(f"{k} = {s if len(s) < 120 else s[:117] + '...'}")
            print(TransformerConfig.from_gguf(r))
        if a.tensors:
            for name, t in r.tensors.items():
                print(f"{name:48s} {str(tuple(t.shape)):24s} {t.qtype.name:6s} {t.nbytes} B")
        return 0
    if a.greedy:
        a.temp = 0.0
        a.repeat_penalty = 1.0
    prompt = a.prompt if a.prompt is not None else "Hello, how are you?"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if a.nprocs > 1 and world == 1:
        # one process per GPU under torchrun, which then runs this module again with the ranks in the environment
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.nprocs}", "--master-addr",
               a.master_addr, "--master-port", str(a.master_port), "-m", "prometorch_b200.generate"] + (argv if argv is not None else sys.argv[1:])
        return subprocess.call(cmd)
    import torch
    from .io.chat import apply_chat_template
    from .io.tokenizer import GGUFTokenizer
    rank = int(os.environ.get("RANK", "0"))
    say = print if rank == 0 else (lambda *x, **k: None)
    use_cuda = (a.device in ("cuda", "gpu") or a.cuda) and torch.cuda.is_available()
    if a.profile:
        os.environ["PTB_TRACE"] = "1"
    t0 = time.time()
    from .io.gguf import GGUFReader
    if GGUFReader(path).arch() == "deepseek2":
        # latent attention + mixture of experts: the tensor-program model (greedy), on the GPU in bf16 or on the CPU in fp32
        from .models.deepseek2 import DeepSeek2Model
        model = DeepSeek2Model(path, device="cuda" if use_cuda else "cpu", max_seq=min(4096, a.max_tokens + 2048),
                               dtype=torch.bfloat16 if use_cuda else torch.float32)
        tok = GGUFTokenizer.from_reader(model.reader)
        c = model.cfg
        say(f"[Model] deepseek2 {c.num_layers} layers, hidden {c.hidden_size}, {c.expert_count} experts ({c.expert_used_count} used), "
            f"latent cache {model.cache_bytes_per_token} B/token, loaded in {time.time() - t0:.1f} s")
        text = apply_chat_template(prompt, "deepseek2", "") if (a.chat and not a.raw) else prompt
        ids = tok.encode(text)
        say(f"[Generate] Prompt tokens: {len(ids)}")
        t1 = time.time()
        out = model.generate(ids, max_new_tokens=a.max_tokens)
        say(tok.decode(out, strip_leading_space=False))
        dt = time.time() - t1
        say(f"\n[Generate] {len(out)} tokens in {dt:.2f}s ({len(out) / max(dt, 1e-9):.1f} tok/s, prompt included)")
        return 0
    if use_cuda:
        from .io.gguf_model import GGUFModel
        symm = None
        if world > 1:
            import torch.distributed as dist
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
            from .parallel.symm import SymmGroup
            symm = SymmGroup(dist.group.WORLD, torch.device("cuda", torch.cuda.current_device()))
        model = GGUFModel(path, device=f"cuda:{torch.cuda.current_device()}", max_seq=min(4096, a.max_tokens + 2048), tp_rank=rank,
                          tp_world=world, symm=symm, want_logits=a.temp > 0 or a.repeat_penalty != 1.0)
        reader, cfg = model.reader, model.cfg
    elif world > 1:
        # tensor parallel on CPU ranks (gloo): the sharded fp32 oracle, the shape of the reference's own --nprocs path
        import torch.distributed as dist
        from .models.gguf_oracle import TPOracleModel
        dist.init_process_group("gloo")
        model = TPOracleModel(path, rank, world, max_seq=min(4096, a.max_tokens + 2048))
        reader, cfg = model.reader, model.cfg
    else:
        from .models.gguf_oracle import OracleModel
        model = OracleModel(path, device="cpu", max_seq=min(4096, a.max_tokens + 2048))
        reader, cfg = model.reader, model.cfg
    tok = GGUFTokenizer.from_reader(reader)
    say(f"[Model] {cfg.architecture} {cfg.num_layers} layers, hidden {cfg.hidden_size}, loaded in {time.time() - t0:.1f} s "
        f"on {'CUDA' if use_cuda else 'CPU'}" + (f" x{world} (tensor parallel)" if world > 1 else ""))
    text = apply_chat_template(prompt, cfg.architecture, cfg.model_name) if (a.chat and not a.raw) else prompt
    ids = tok.encode(text)
    say(f"[Generate] Prompt tokens: {len(ids)}")
    debug_tokens = env_int("DEBUG_TOKENS", 0) == 1
    if debug_tokens:
        say(f"[Tokens] prompt {ids}")
    t1 = time.time()
    out = []

    def on_token(t: int) -> bool:
        out.append(t)
        if rank == 0:
            sys.stdout.write(tok.decode([t], strip_leading_space=False))
            sys.stdout.flush()
        return True
    if use_cuda:
        stops = {cfg.eos_token_id} - {-1}
        for s in ("<|im_end|>", "<|eot_id|>", "<end_of_turn>", "<|end|>", "<|endoftext|>", "</s>"):
            if s in tok.vocab:
                stops.add(tok.vocab[s])
        if a.draft and world == 1 and a.temp <= 0.0 and a.repeat_penalty == 1.0:
            from .io.gguf_model import GGUFModel as _G
            from .io.speculative import speculative_generate
            draft = _G(a.draft, device=f"cuda:{torch.cuda.current_device()}", max_seq=model.max_seq)
            toks, st = speculative_generate(model, draft, ids, max_new_tokens=a.max_tokens, k=a.spec_k, stop_ids=stops)
            for t in toks:
                on_token(t)
            say(f"\n[Speculative] {st['accepted']} of {st['proposed']} proposals accepted, {st['target_passes']} target passes")
            draft.close()
        else:
            model.generate(ids, max_new_tokens=a.max_tokens, temperature=a.temp, top_k=a.top_k, top_p=a.top_p,
                           repeat_penalty=a.repeat_penalty, stop_ids=stops, on_token=on_token)
    else:
        for t in model.generate_greedy(ids, a.max_tokens):
            on_token(t)
    dt = time.time() - t1
    say(f"\n\n[Generate] {len(out)} tokens in {dt:.2f}s ({len(out) / max(dt, 1e-9):.1f} tok/s, prompt included)")
    if debug_tokens:
        say(f"[Tokens] generated {out}")
    if a.profile and use_cuda and world == 1:
        import ctypes as C
        n_k = 5 * cfg.num_layers + 2
        buf = (C.c_ulonglong * (8 * n_k))()
        model._lib.ptb_engine_read_trace.argtypes = [C.c_void_p, C.POINTER(C.c_ulonglong), C.c_int]
        n = model._lib.ptb_engine_read_trace(model._engine, buf, n_k)
        names = ["embed"] + ["qkv", "attention", "o", "gate/up", "down"] * cfg.num_layers + ["lm_head"]
        tot = {}
        for k in range(n):
            s = buf[8 * k:8 * k + 8]
            if s[0] and s[5]:
                tot.setdefault(names[k], []).append((s[5] - s[0]) / 1e3)
        for nm, v in tot.items():
            say(f"[Profile] {nm:10s} {len(v):4d} launches, {sum(v) / len(v):7.2f} us each (CTA 0, start to end)")
    if use_cuda:
        model.close()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
