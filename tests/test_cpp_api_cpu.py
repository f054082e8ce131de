"""The C++ torch-style API (prometorch_b200/cpp_api): a C++ program is compiled against the installed libtorch and run.
It trains the benchmark MLP for a few steps, runs all sixteen optimizers and schedulers, round-trips PTOR / .pt
checkpoints and runs DistributedDataParallel with no_sync plus tensor-parallel layers over two forked TCP ranks."""
import os
import shutil
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torch_flags():
    ti = os.path.dirname(torch.__file__)
    return [f"-I{ti}/include", f"-I{ti}/include/torch/csrc/api/include", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
            f"-L{ti}/lib", "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{ti}/lib"]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_cpp_api_trains_and_synchronises(tmp_path):
    exe = str(tmp_path / "train_mlp")
    cmd = ["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "train_mlp.cpp"), "-o", exe,
           f"-I{ROOT}/prometorch_b200/cpp_api"] + _torch_flags()
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe, str(29750 + os.getpid() % 200)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "CPP_API_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_cpp_api_amp_data_fsdp_pipeline(tmp_path):
    """GradScaler / autocast guards, datasets + DataLoader with worker threads, GPipe, and over forked ranks: sharded data
    parallelism with a ZeRO optimizer against a replica, the offload optimizer, the split all-gather, a 1F1B pipeline whose
    stage gradients equal the single-process model's."""
    exe = str(tmp_path / "parallel_api")
    cmd = ["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "parallel_api.cpp"), "-o", exe,
           f"-I{ROOT}/prometorch_b200/cpp_api"] + _torch_flags() + ["-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe, str(30050 + os.getpid() % 200), str(tmp_path / "ckpt")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "CPP_PARALLEL_API_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def _check_checkpoints(exe, tmp_path):
    """PTOR containers and PyTorch zips written by Python are read by the C++ API and written back unchanged."""
    from collections import OrderedDict
    from prometorch_b200 import serialization as S
    g = torch.Generator().manual_seed(4)
    sd = OrderedDict([("layer.weight", torch.randn(5, 7, generator=g)), ("layer.bias", torch.randn(7, generator=g)),
                      ("half", torch.randn(3, 2, generator=g).half()), ("bf16", torch.randn(4, generator=g).bfloat16()),
                      ("ids", torch.arange(6).reshape(2, 3)), ("scalar", torch.tensor(3.5)), ("bytes", torch.arange(10, dtype=torch.uint8)),
                      ("double", torch.randn(2, 2, generator=g, dtype=torch.float64)), ("empty", torch.zeros(0, 4))])
    d = tmp_path / "ckpt_io"
    d.mkdir()
    S.save_state_dict(sd, str(d / "py.ptor"))
    S.save_pytorch(dict(sd), str(d / "py.pt"))
    r = subprocess.run([exe, "io", str(d)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    seen = {"ptor": {}, "pt": {}}
    for ln in r.stdout.splitlines():
        head, sums = ln.split(" | ")
        kind, name, dtype, *shape = head.split()
        seen[kind[2:]][name] = (dtype, [int(x) for x in shape], float(sums.split()[0]), float(sums.split()[1]))
    names = {torch.float32: "Float", torch.float16: "Half", torch.bfloat16: "BFloat16", torch.int64: "Long", torch.uint8: "Byte", torch.float64: "Double"}
    for kind in ("ptor", "pt"):
        assert list(seen[kind]) == list(sd) if kind == "ptor" else set(seen[kind]) == set(sd)
        for k, t in sd.items():
            dtype, shape, total, amax = seen[kind][k]
            assert dtype == names[t.dtype] and shape == list(t.shape), (kind, k, dtype, shape)
            assert abs(total - float(t.double().sum())) < 1e-6 and abs(amax - float(t.double().abs().max() if t.numel() else 0.0)) < 1e-6, (kind, k)
    back = S.load_state_dict(str(d / "cpp.ptor"))
    back_pt = S.load_pytorch(str(d / "cpp.pt"))
    assert list(back) == list(sd)
    for k, t in sd.items():
        assert back[k].dtype == t.dtype and torch.equal(back[k], t), k
        assert back_pt[k].dtype == t.dtype and torch.equal(back_pt[k], t), k


def _check_llama(exe, tmp_path):
    """models::Llama (libtorch tensor code) on a Hugging Face directory against the Python engine's weights: logits of a
    prompt, greedy continuation with the key / value cache, and safetensors written by C++ read back by Python."""
    import json
    from prometorch_b200.io.safetensors import load_file
    from prometorch_b200.serve.llm import GenerationConfig, LlamaConfig, LlamaWeights, LLMEngine, save_safetensors
    cfg = LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      max_position_embeddings=128, eos_token_id=2)
    w = LlamaWeights.random(cfg, seed=31)
    d = tmp_path / "hf_llama"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({k: getattr(cfg, k) for k in cfg.__dataclass_fields__}))
    sd = w.state_dict()
    save_safetensors(sd, str(d / "model.safetensors"))
    out_file = str(tmp_path / "from_cpp.safetensors")
    r = subprocess.run([exe, "llama", str(d), out_file], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    got = {ln.split()[0]: ln.split()[1:] for ln in r.stdout.splitlines() if ln.startswith("L:")}
    prompt = [1, 17, 250, 3, 99, 42]
    eng = LLMEngine(device="cpu", max_pages=16, max_active=2)
    assert eng.load(str(d))
    greedy = eng.generate(prompt, GenerationConfig(max_new_tokens=10, temperature=0.0, repetition_penalty=1.0, top_k=1, stop_at_eos=False)
                          if "stop_at_eos" in GenerationConfig.__dataclass_fields__ else
                          GenerationConfig(max_new_tokens=10, temperature=0.0, repetition_penalty=1.0, top_k=1)).token_ids
    cpp = [int(t) for t in got["L:greedy"]]
    assert cpp[:len(greedy)] == greedy, (cpp, greedy)                      # the engine may stop at its end-of-sequence id
    assert [int(x) for x in got["L:shape"]] == [1, 6, 300] and len(got["L:sampled"]) == 6 and all(0 <= int(t) < 300 for t in got["L:sampled"])
    # the same logits from plain tensor code over the Python weights
    import torch.nn.functional as F
    H, Hk, Dh = 4, 2, 16
    ids = torch.tensor(prompt)
    h = sd["model.embed_tokens.weight"][ids]
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, Dh, 2, dtype=torch.float64) / Dh))
    ang = torch.arange(len(prompt), dtype=torch.float64)[:, None] * inv[None]
    cos, sin = ang.cos().float()[:, None], ang.sin().float()[:, None]

    def rms(x, wt):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * wt

    def rope(x):
        a, b = x[..., :Dh // 2], x[..., Dh // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
    for l in range(2):
        p = f"model.layers.{l}."
        x = rms(h, sd[p + "input_layernorm.weight"])
        q = rope((x @ sd[p + "self_attn.q_proj.weight"].t()).view(-1, H, Dh))
        k = rope((x @ sd[p + "self_attn.k_proj.weight"].t()).view(-1, Hk, Dh)).repeat_interleave(H // Hk, 1)
        v = (x @ sd[p + "self_attn.v_proj.weight"].t()).view(-1, Hk, Dh).repeat_interleave(H // Hk, 1)
        a = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], is_causal=True)[0].transpose(0, 1).reshape(len(prompt), -1)
        h = h + a @ sd[p + "self_attn.o_proj.weight"].t()
        x = rms(h, sd[p + "post_attention_layernorm.weight"])
        h = h + (F.silu(x @ sd[p + "mlp.gate_proj.weight"].t()) * (x @ sd[p + "mlp.up_proj.weight"].t())) @ sd[p + "mlp.down_proj.weight"].t()
    logits = rms(h, sd["model.norm.weight"]) @ sd.get("lm_head.weight", sd["model.embed_tokens.weight"]).t()
    assert [int(t) for t in got["L:argmax"]] == logits.argmax(-1).tolist()
    assert torch.allclose(torch.tensor([float(v) for v in got["L:last"]]), logits[-1, :16], atol=2e-4, rtol=1e-4)
    back = load_file(out_file)
    assert set(back) == set(sd) and all(torch.equal(back[k], sd[k]) for k in sd)


def _check_ecosystem(exe, tmp_path):
    """ecosystem.h (vision / text / audio over libtorch) against the Python modules of the same names on the same inputs."""
    import math
    from prometorch_b200 import audio, text, vision
    from prometorch_b200.vision import transforms as VT
    d = tmp_path / "eco"
    (d / "set" / "cats").mkdir(parents=True)
    (d / "set" / "dogs").mkdir()
    g = torch.Generator().manual_seed(2)
    img = torch.rand(3, 5, 7, generator=g)
    vision.save_pnm(str(d / "py.ppm"), img)
    (d / "ascii.pgm").write_bytes(b"P2\n# note\n3 2\n15\n0 5 10\n15 1 2\n")
    for cls in ("cats", "dogs"):
        for i in range(2):
            vision.save_pnm(str(d / "set" / cls / f"{i}.pgm"), torch.rand(1, 4, 4, generator=g))
    t = torch.linspace(0, 1, 16000)
    x = torch.sin(2 * math.pi * 440 * t)
    audio.save_wav(str(d / "py.wav"), x[:1600], 16000)
    r = subprocess.run([exe, "ecosystem", str(d)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    raw = {ln.split()[0][2:]: ln.split()[1:] for ln in r.stdout.splitlines() if ln.startswith("E:")}
    num = lambda k: torch.tensor([float(v) for v in raw[k]], dtype=torch.float64)           # noqa: E731

    def same(key, want, tol=1e-5):
        w = torch.as_tensor(want).double().reshape(-1)
        assert num(key).shape == w.shape and torch.allclose(num(key), w, atol=tol, rtol=tol), (key, num(key)[:6], w[:6])
    loaded = vision.load_pnm(str(d / "py.ppm"))
    same("ppm_shape", [3, 5, 7])
    same("ppm_sum", loaded.sum())
    same("pgm_ascii", vision.load_pnm(str(d / "ascii.pgm")))
    assert torch.equal(vision.load_pnm(str(d / "cpp.ppm")), loaded)
    same("transformed", VT.Compose([VT.Resize((6, 8)), VT.CenterCrop(4), VT.Normalize([0.5, 0.4, 0.3], [0.2, 0.3, 0.4])])(loaded))
    same("random_crop_shape", [3, 2])
    same("flip", loaded.flip(-1)[:1, :1])
    same("folder", [4, 2, 1, 8])
    assert raw["classes"] == ["cats", "dogs"]
    vocab = text.Vocab.build(["the cat sat", "the dog sat down", "a cat"], 1)
    same("vocab_encode", vocab.encode("the cat flew down"))
    assert " ".join(raw["vocab_decode"]) == vocab.decode([2, 4, 3]) and raw["basic"] == text.BasicTokenizer().tokenize("Hello, World! it's")
    same("char", text.CharTokenizer("hello world").encode("held z"))
    same("wordpiece", text.WordPieceTokenizer(["[UNK]", "un", "##aff", "##able", "play", "##ing", "##ed"]).encode("unaffable playing xyz played"))
    batch = [[1, 2, 3], [4], [5, 6]]
    same("pad", text.pad_sequence(batch, 9, True, 2))
    same("pad_tb", text.pad_sequence(batch, 0, False))
    same("lengths", text.sequence_lengths(batch))
    same("mask", text.padding_mask(batch).long())
    spec = audio.spectrogram(x, 400, 160)
    same("spec_shape", list(spec.shape))
    same("spec_peak", spec.mean(1).argmax())
    same("spec_probe", spec[9:13, 10:12], 1e-3)
    same("fbanks_sum", audio.melscale_fbanks(201, 40, 16000).sum(0), 1e-4)
    same("mfcc_probe", audio.mfcc(x)[:4, 5:7], 2e-3)
    q = audio.mu_law_encoding(x[:64])
    same("mulaw", q)
    same("mulaw_back", audio.mu_law_decoding(q))
    same("db", audio.amplitude_to_db(spec[9:13, 10:12], 10.0, 1e-10, 0.0, 20.0), 1e-3)
    same("resample", audio.resample(x[:100], 16000, 8000))
    wav, sr = audio.load_wav(str(d / "py.wav"))
    same("wav", [sr, wav.numel(), wav.abs().max()])
    back, sr2 = audio.load_wav(str(d / "cpp.wav"))
    assert sr2 == 8000 and back.numel() == 800 and float((back - x[:800]).abs().max()) < 1e-3


def _check_exporters(exe, tmp_path):
    """export.h: ONNX, MLIR and PTMB files written by C++ are byte-identical to the Python exporters' for the same model, and
    the C++ executor runs the file Python wrote."""
    import torch.nn as nn
    from prometorch_b200 import mlir, mobile, onnx
    from prometorch_b200 import serialization as S
    torch.manual_seed(12)
    net = nn.Sequential(nn.Linear(6, 5), nn.ReLU(), nn.Sequential(nn.Linear(5, 4), nn.Tanh()), nn.Linear(4, 3, bias=False), nn.Softmax(-1))
    d = tmp_path / "export"
    d.mkdir()
    S.save_state_dict(dict(net.state_dict()), str(d / "mlp.ptor"))
    onnx.export_mlp(net, [2, 6], str(d / "py.onnx"))
    mlir.export(net, [2, 6], str(d / "py.mlir"))
    mobile.save(net, str(d / "py.ptmb"))
    r = subprocess.run([exe, "export", str(d)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    for kind in ("onnx", "mlir", "ptmb"):
        assert (d / f"cpp.{kind}").read_bytes() == (d / f"py.{kind}").read_bytes(), kind
    raw = {ln.split()[0][2:]: torch.tensor([float(v) for v in ln.split()[1:]]) for ln in r.stdout.splitlines() if ln.startswith("E:")}
    x = torch.arange(12.0).reshape(2, 6) / 10.0
    want = net(x).detach().reshape(-1)
    assert torch.allclose(raw["mobile"], want, atol=1e-6) and torch.allclose(raw["direct"], want, atol=1e-6)
    assert torch.allclose(mobile.Executor(str(d / "cpp.ptmb")).run(x).reshape(-1), want, atol=1e-6)


def _check_schedulers(sched):
    """The learning-rate sequences of the C++ schedulers against the Python ones (same constructor arguments)."""
    from prometorch_b200 import optim as O
    L = O

    def seq(make, steps=24, metric=None):
        w = torch.nn.Parameter(torch.zeros(2))
        opt = O.SGD([w], lr=0.5)
        s = make(opt)
        out = [opt.param_groups[0]["lr"]]
        for i in range(steps):
            s.step(metric(i)) if metric else s.step()
            out.append(opt.param_groups[0]["lr"])
        return out
    want = {
        "StepLR": seq(lambda o: L.StepLR(o, 5, 0.5)), "MultiStepLR": seq(lambda o: L.MultiStepLR(o, [3, 7, 15], 0.3)),
        "ExponentialLR": seq(lambda o: L.ExponentialLR(o, 0.9)), "CosineAnnealingLR": seq(lambda o: L.CosineAnnealingLR(o, 10, 0.01)),
        "LinearLR": seq(lambda o: L.LinearLR(o, 0.25, 1.0, 8)), "ConstantLR": seq(lambda o: L.ConstantLR(o, 0.2, 6)),
        "WarmupCosineAnnealingLR": seq(lambda o: L.WarmupCosineAnnealingLR(o, 4, 20, 0.05)), "OneCycleLR": seq(lambda o: L.OneCycleLR(o, 1.0, 24, 0.25)),
        "CosineAnnealingWarmRestarts": seq(lambda o: L.CosineAnnealingWarmRestarts(o, 4, 2, 0.02)), "CyclicLR": seq(lambda o: L.CyclicLR(o, 0.1, 0.9, 3, 5)),
        "CyclicLR_triangular2": seq(lambda o: L.CyclicLR(o, 0.1, 0.9, 2, -1, "triangular2")), "PolynomialLR": seq(lambda o: L.PolynomialLR(o, 12, 2.0)),
        "LambdaLR": seq(lambda o: L.LambdaLR(o, lambda e: 1.0 / (1.0 + 0.5 * e))),
        "MultiplicativeLR": seq(lambda o: L.MultiplicativeLR(o, lambda e: 0.8 if e % 3 == 0 else 1.0)),
        "ReduceLROnPlateau": seq(lambda o: L.ReduceLROnPlateau(o, "min", 0.5, 2, 1e-3, 0.01), metric=lambda i: 1.0 - 0.1 * i if i < 5 else 0.7),
        "SequentialLR": seq(lambda o: L.SequentialLR(o, [L.LinearLR(o, 0.1, 1.0, 5), L.ExponentialLR(o, 0.8)], [5])),
        "ChainedScheduler": seq(lambda o: L.ChainedScheduler(o, [L.StepLR(o, 4, 0.5), L.ExponentialLR(o, 0.95)])),
    }
    assert set(sched) == set(want), set(sched) ^ set(want)
    bad = {}
    for name, w in want.items():
        diff = max(abs(a - b) for a, b in zip(w, sched[name]))
        if len(w) != len(sched[name]) or diff > 1e-9:
            bad[name] = (diff, [round(v, 6) for v in w[:8]], [round(v, 6) for v in sched[name][:8]])
    assert not bad, bad


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_cpp_and_python_implementations_agree(tmp_path):
    """The C++ and the Python optimizers are separate implementations of the reference's update rules: on the same start
    point and the same sequence of gradients they must end at the same parameters; the sixteen schedulers must produce the
    same learning-rate sequences; checkpoints written by one side load on the other; the C++ Llama gives the logits and the
    greedy continuation of the Python engine on the same Hugging Face directory."""
    import math
    from prometorch_b200 import optim as O
    exe = str(tmp_path / "cross_language")
    cmd = ["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "cross_language.cpp"), "-o", exe,
           f"-I{ROOT}/prometorch_b200/cpp_api"] + _torch_flags()
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    _check_checkpoints(exe, tmp_path)
    _check_llama(exe, tmp_path)
    _check_ecosystem(exe, tmp_path)
    _check_exporters(exe, tmp_path)
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    got = {ln.split()[0]: [float(v) for v in ln.split()[1:]] for ln in lines if not ln.startswith("S:")}
    sched = {ln.split()[0][2:]: [float(v) for v in ln.split()[1:]] for ln in lines if ln.startswith("S:")}
    _check_schedulers(sched)

    def start(shape, phase):
        n = math.prod(shape)
        i = torch.arange(n, dtype=torch.float64)
        return (torch.sin(i * 0.37 + phase) + 0.1 * i / n).float().reshape(shape)

    def gradient(shape, step, phase):
        n = math.prod(shape)
        i = torch.arange(n, dtype=torch.float64)
        return (torch.cos(i * 0.21 + 0.9 * step + phase) * (1.0 + 0.1 * step)).float().reshape(shape)
    cases = {"SGD": (O.SGD, dict(lr=0.05, momentum=0.9, nesterov=True, weight_decay=0.01)), "SGD_plain": (O.SGD, dict(lr=0.05)),
             "Adam": (O.Adam, dict(lr=1e-2)), "Adam_amsgrad": (O.Adam, dict(lr=1e-2, amsgrad=True, weight_decay=0.1)), "AdamW": (O.AdamW, dict(lr=1e-2)),
             "RMSprop": (O.RMSprop, dict(lr=1e-2)), "RMSprop_centered": (O.RMSprop, dict(lr=1e-2, centered=True, momentum=0.5)),
             "Lion": (O.Lion, dict(lr=3e-3, weight_decay=0.1)), "SophiaG": (O.SophiaG, dict(lr=1e-2)), "LAMB": (O.LAMB, dict(lr=1e-2)),
             "Adafactor": (O.Adafactor, dict()), "Adafactor_fixed": (O.Adafactor, dict(lr=1e-2, relative_step=False, scale_parameter=False, beta1=0.9)),
             "NAdam": (O.NAdam, dict(lr=1e-2)), "RAdam": (O.RAdam, dict(lr=2e-2)), "Adagrad": (O.Adagrad, dict(lr=0.1)), "Adadelta": (O.Adadelta, dict()),
             "Adamax": (O.Adamax, dict(lr=2e-2)), "AdamKiller": (O.AdamKiller, dict(lr=1e-2)), "ASGD": (O.ASGD, dict(lr=0.05))}
    assert set(got) == set(cases)
    worst = {}
    for name, (cls, kw) in cases.items():
        w, b = torch.nn.Parameter(start((6, 5), 0.0)), torch.nn.Parameter(start((5,), 1.0))
        opt = cls([w, b], fused=False, **kw)
        for s in range(9 if name == "RAdam" else 6):
            w.grad, b.grad = gradient((6, 5), s, 0.0), gradient((5,), s, 2.0)
            opt.step()
        want = torch.cat([w.detach().reshape(-1), b.detach().reshape(-1)]).double()
        have = torch.tensor(got[name], dtype=torch.float64)
        worst[name] = float((want - have).abs().max())
        moved = float((want - torch.cat([start((6, 5), 0.0).reshape(-1), start((5,), 1.0).reshape(-1)]).double()).abs().max())
        assert moved > 1e-4, name
    bad = {k: v for k, v in worst.items() if v > 2e-5}
    assert not bad, bad


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_cpp_headers_are_self_contained(tmp_path):
    """Every header of the C++ API compiles when it is the only include of a translation unit (no header leans on what
    another one happened to include before it)."""
    import concurrent.futures as cf
    import glob
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    headers = sorted(glob.glob(os.path.join(ROOT, "prometorch_b200", "cpp_api", "promethorch", "*.h")))
    assert len(headers) >= 26
    flags = [f for f in _torch_flags() if f.startswith(("-I", "-D"))] + [f"-I{ROOT}/prometorch_b200/cpp_api", f"-I{cuda}/include"]

    def check(h):
        name = os.path.basename(h)
        if name in ("gguf.h", "gguf_backend.h") and not os.path.exists(os.path.join(cuda, "include", "cuda_runtime.h")):
            return name, 0, ""                                   # these two need the CUDA runtime's header
        src = tmp_path / (name + ".cpp")
        src.write_text(f'#include "promethorch/{name}"\nint main() {{ return 0; }}\n')
        r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", str(src)] + flags, capture_output=True, text=True, timeout=900)
        return name, r.returncode, r.stderr[-1500:]
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        results = list(ex.map(check, headers))
    bad = {n: err for n, rc, err in results if rc != 0}
    assert not bad, bad


@pytest.mark.skipif(shutil.which("g++") is None or shutil.which("make") is None, reason="needs g++ and make")
def test_cpp_example_programs_build_and_run(tmp_path):
    """examples/cpp: the Makefile builds both programs; the MLP trains, the serving-side example reads a GGUF file, tokenises
    and continues a prompt on the CPU decoder."""
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    work = tmp_path / "cpp"
    shutil.copytree(os.path.join(ROOT, "examples", "cpp"), work)
    api = os.path.join(ROOT, "prometorch_b200", "cpp_api")
    r = subprocess.run(["make", "-C", str(work), "all", f"API={api}"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    r = subprocess.run([str(work / "mlp"), "1"], capture_output=True, text=True, timeout=600, cwd=str(work))
    assert r.returncode == 0 and "saved mlp.ptor (535818 parameters)" in r.stdout, r.stdout + r.stderr[-1500:]
    acc = float(r.stdout.split("test accuracy")[1].split("%")[0])
    assert acc > 90.0
    path = str(tmp_path / "ex.gguf")
    write_synthetic_gguf(path, tiny_qwen3_config(layers=1, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=2, device="cpu")
    r = subprocess.run([str(work / "tokenize"), path, "t300 t301", "--generate", "3"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    assert "format gguf, architecture qwen3" in r.stdout and "round trip: t300 t301" in r.stdout and "greedy continuation on the CPU decoder:" in r.stdout
