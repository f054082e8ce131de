"""CPU tests of the framework surface around the kernels: serialization, AMP, trainer, quantization, export,
JIT wrapper, domain shims, metrics/profiler, tokenizer/chat/model resolution."""
import json
import math
import os

import pytest
import torch
import torch.nn as nn

import prometorch_b200 as pt
from prometorch_b200 import amp, audio, autograd, data, jit, mlir, mobile, onnx, quantization as Q, serialization as S, text, trainer
from prometorch_b200.io import chat, ollama
from prometorch_b200.io.tokenizer import GGUFTokenizer
from prometorch_b200.utils import metrics, profiler


# ----------------------------------------------------------------------------- serialization
def test_ptor_roundtrip(tmp_path):
    sd = {"w": torch.randn(3, 5), "b": torch.arange(4, dtype=torch.int64), "h": torch.randn(2, 2).to(torch.bfloat16)}
    p = str(tmp_path / "m.ptor")
    S.save_state_dict(sd, p)
    with open(p, "rb") as f:
        assert f.read(4) == b"PTOR"
    back = S.load_state_dict(p)
    assert list(back) == list(sd)
    for k in sd:
        assert back[k].dtype == sd[k].dtype and torch.equal(back[k], sd[k])
    S.save(sd["w"], str(tmp_path / "t.ptor"))
    assert torch.equal(S.load(str(tmp_path / "t.ptor")), sd["w"])


def test_pytorch_checkpoint_interop(tmp_path):
    m = nn.Linear(4, 3)
    p = str(tmp_path / "m.pt")
    S.save_pytorch(m.state_dict(), p)
    theirs = torch.load(p, weights_only=True)              # a file we wrote is a regular PyTorch checkpoint
    assert torch.equal(theirs["weight"], m.weight)
    torch.save({"x": torch.ones(2)}, str(tmp_path / "t.pt"))
    assert torch.equal(S.load_pytorch(str(tmp_path / "t.pt"))["x"], torch.ones(2))


# ----------------------------------------------------------------------------- AMP
def test_grad_scaler_skips_on_inf_and_backs_off():
    w = nn.Parameter(torch.ones(4))
    opt = pt.optim.SGD([w], lr=0.1)
    sc = amp.GradScaler(init_scale=1024.0, growth_interval=2)
    loss = (w * 2).sum()
    sc.scale(loss).backward()
    assert torch.allclose(w.grad, torch.full((4,), 2048.0))
    sc.step(opt)
    sc.update()
    assert torch.allclose(w.detach(), torch.full((4,), 0.8))             # unscaled gradient 2 was applied
    w.grad = torch.tensor([float("inf"), 0.0, 0.0, 0.0])
    before = w.detach().clone()
    sc.step(opt)
    sc.update()
    assert torch.equal(w.detach(), before) and sc.get_scale() == 512.0   # step skipped, scale halved
    st = sc.state_dict()
    sc2 = amp.GradScaler()
    sc2.load_state_dict(st)
    assert sc2.get_scale() == 512.0


def test_autocast_policy_table_matches_what_autocast_does():
    import torch.nn.functional as F
    from prometorch_b200 import amp
    a, b = torch.randn(4, 4), torch.randn(4, 4)
    calls = {"matmul": lambda: torch.matmul(a, b), "linear": lambda: F.linear(a, b), "mm": lambda: torch.mm(a, b),
             "bmm": lambda: torch.bmm(a[None], b[None]), "conv1d": lambda: F.conv1d(a[None], b[None, :, :2]),
             "mse_loss": lambda: F.mse_loss(torch.matmul(a, b), torch.matmul(a, b)),
             "relu": lambda: torch.relu(torch.matmul(a, b)), "cat": lambda: torch.cat([torch.matmul(a, b), a])}
    with amp.AutocastCPUGuard(torch.bfloat16):
        assert amp.is_autocast_enabled("cpu") and amp.get_autocast_dtype("cpu") == torch.bfloat16
        for name, call in calls.items():
            policy, dtype = amp.get_autocast_policy(name), call().dtype
            if policy == amp.CastPolicy.LOWER_PRECISION:
                assert dtype == torch.bfloat16, name
            elif policy in (amp.CastPolicy.FP32, amp.CastPolicy.PROMOTE):
                assert dtype == torch.float32, name
            else:
                assert dtype == torch.bfloat16, name            # takes the dtype of its (bf16) input
    assert not amp.is_autocast_enabled("cpu")
    assert amp.get_autocast_policy("softmax") == amp.CastPolicy.FP32 and amp.get_autocast_policy("view") == amp.CastPolicy.UNCHANGED


def test_autocast_guard_cpu():
    a, b = torch.randn(8, 8), torch.randn(8, 8)
    with amp.AutocastGuard("cpu", torch.bfloat16):
        c = a @ b
    assert c.dtype == torch.bfloat16


# ----------------------------------------------------------------------------- autograd helpers
def test_checkpoint_and_hooks_and_anomaly():
    lin = nn.Linear(4, 4)
    x = torch.randn(2, 4, requires_grad=True)
    y = autograd.checkpoint(lambda t: torch.relu(lin(t)), x)
    seen = []
    autograd.register_hook(y, lambda g: seen.append(g.shape))
    y.sum().backward()
    assert seen == [y.shape] and x.grad is not None and lin.weight.grad is not None
    autograd.AnomalyMode.set_enabled(True)
    assert autograd.AnomalyMode.is_enabled()
    autograd.AnomalyMode.set_enabled(False)


# ----------------------------------------------------------------------------- trainer + data
class _Lit(trainer.LightningModule):
    def __init__(self):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 4))

    def forward(self, x):
        return self.net(x)

    def training_step(self, batch, idx):
        x, y = batch
        return nn.functional.cross_entropy(self(x), y)

    def validation_step(self, batch, idx):
        x, y = batch
        return {"val_loss": nn.functional.cross_entropy(self(x), y)}

    def configure_optimizers(self):
        return pt.optim.Adam(self.parameters(), lr=1e-2)


def test_trainer_fits_and_resumes(tmp_path):
    torch.manual_seed(0)
    ds = data.SyntheticImages(n=256, dim=16, classes=4)
    dl = torch.utils.data.DataLoader(ds, batch_size=32, shuffle=False)
    m = _Lit()
    with torch.no_grad():
        l0 = sum(float(m.training_step(b, 0)) for b in dl) / len(dl)
    tr = trainer.Trainer(trainer.TrainerConfig(max_epochs=3, checkpoint_dir=str(tmp_path), gradient_clip_val=1.0, accumulate_grad_batches=2))
    tr.fit(m, dl, dl)
    with torch.no_grad():
        l1 = sum(float(m.training_step(b, 0)) for b in dl) / len(dl)
    assert l1 < l0
    ck = str(tmp_path / "last.ckpt")
    tr.save_checkpoint(m, ck)
    m2 = _Lit()
    tr2 = trainer.Trainer(trainer.TrainerConfig(max_epochs=1, checkpoint_dir=str(tmp_path)))
    tr2.load_checkpoint(m2, ck)
    for a, b in zip(m.parameters(), m2.parameters()):
        assert torch.equal(a, b)


def test_synthetic_tokens_dataset():
    ds = data.SyntheticTokens(n=10, seq_len=8, vocab=50, seed=1)
    x, y = ds[3]
    assert x.shape == (8,) and y.shape == (8,) and int(x.max()) < 50 and torch.equal(x[1:], y[:-1])
    md = data.MapDataset(ds, lambda s: (s[0] + 1, s[1]))
    assert torch.equal(md[3][0], x + 1)


# ----------------------------------------------------------------------------- quantization
def test_4bit_and_int8_quantization():
    torch.manual_seed(0)
    w = torch.randn(64, 128)
    for kind in ("nf4", "fp4"):
        packed, absmax = Q.quantize_4bit(w, 64, kind)
        assert packed.dtype == torch.uint8 and packed.numel() == w.numel() // 2
        back = Q.dequantize_4bit(packed, absmax, w.shape, 64, kind)
        assert (back - w).abs().mean() < 0.15
    lin = nn.Linear(128, 64)
    q = Q.Linear4bit(lin)
    x = torch.randn(4, 128)
    assert (q(x) - lin(x)).abs().mean() < 0.2
    aq, asc = Q.quantize_per_tensor(x)
    bq, bsc = Q.quantize_per_tensor(w)
    assert (Q.int8_matmul(aq, asc, bq.t().contiguous(), bsc) - x @ w.t()).abs().max() < 0.5


def test_qat_prepare_convert():
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    x = torch.randn(32, 8)
    ref = m(x)
    qm = Q.prepare_qat(m)
    qm.train()
    qm(x).sum().backward()                                   # observers see data, gradients flow through fake-quant
    Q.freeze_observers(qm)
    cm = Q.convert(qm)
    cm.eval()
    assert (cm(x) - ref).abs().max() < 0.2


# ----------------------------------------------------------------------------- export / jit
def test_exporters_write_files(tmp_path):
    m = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    p = str(tmp_path / "m.onnx")
    onnx.export_mlp(m, (1, 8), p)
    assert os.path.getsize(p) > 8 * 16 * 4
    txt = mlir.export(m, (1, 8), str(tmp_path / "m.mlir"))
    assert "func.func" in txt and "linalg" in txt or "tosa" in txt or "arith" in txt
    mp = str(tmp_path / "m.ptmb")
    mobile.save(m, mp)
    ex = mobile.Executor(mp)
    x = torch.randn(3, 8)
    assert torch.allclose(ex.run(x), m(x), atol=1e-5)


def _affine(t: torch.Tensor) -> torch.Tensor:
    return t * 2 + 1


def test_jit_wrappers_keep_semantics():
    m = nn.Sequential(nn.Linear(8, 8), nn.Tanh())
    x = torch.randn(2, 8)
    cm = jit.compile(m)
    assert torch.allclose(cm(x), m(x))
    f = jit.script(_affine)
    assert torch.equal(f(x), x * 2 + 1)
    g = jit.trace(lambda t: t.relu(), (x,))
    assert torch.equal(g(x), x.relu())


# ----------------------------------------------------------------------------- domain shims
def test_text_tokenizers():
    v = text.Vocab(["hello", "world"])
    ids = v.encode("hello there world")
    assert v.decode(ids) == "hello <unk> world"
    bpe = text.BPETokenizer()
    bpe.train(["low lower lowest", "new newer newest"] * 5, 60)
    s = "lower newest"
    assert bpe.decode(bpe.encode(s)) == s
    wp = text.WordPieceTokenizer(["un", "##aff", "##able", "[UNK]"])
    assert wp.tokenize("unaffable") == ["un", "##aff", "##able"]


def test_audio_stft_roundtrip_and_wav(tmp_path):
    t = torch.arange(16000) / 16000.0
    x = torch.sin(2 * math.pi * 440 * t)
    spec = audio.stft(x)
    y = audio.istft(spec, length=x.numel())
    assert (x - y)[400:-400].abs().max() < 1e-3
    assert audio.mfcc(x).shape[0] == 13
    assert audio.mel_filterbank(40, 400, 16000).shape == (40, 201)
    assert abs(audio.resample(x, 16000, 8000).numel() - 8000) <= 1
    p = str(tmp_path / "a.wav")
    audio.save_wav(p, x, 16000)
    z, sr = audio.load_wav(p)
    assert sr == 16000 and (z - x).abs().max() < 1e-3


def test_vision_models_forward():
    from prometorch_b200 import vision
    x = torch.randn(2, 3, 32, 32)
    assert vision.ResNet20(num_classes=10)(x).shape == (2, 10)


# ----------------------------------------------------------------------------- metrics / profiler
def test_metrics_writer_and_profiler(tmp_path):
    p = str(tmp_path / "m.jsonl")
    w = metrics.MetricsWriter(p)
    w.log(step=1, loss=2.5)
    w.roofline("copy", seconds=1e-3, bytes_moved=1e9)
    w.close()
    rows = [json.loads(l) for l in open(p)]
    assert rows[0]["loss"] == 2.5 and 0.1 < rows[1]["fraction"] < 0.2
    prof = profiler.InferenceProfiler()
    prof.enable(True)
    prof.begin("qkv")
    prof.end("qkv")
    prof.count_tokens(3)
    assert "qkv" in prof.totals()
    t = profiler.Timer()
    assert t.elapsed_ms() >= 0.0


# ----------------------------------------------------------------------------- tokenizer / chat / model resolution
def test_gguf_tokenizer_spm_and_gpt2():
    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "h", "e", "l", "o", "▁h", "el", "lo", "▁hel", "▁hello", "w", "▁w"]
    scores = [0.0] * 259 + [-1.0, -2, -2, -2, -2, -1.5, -1.4, -1.3, -1.2, -1.0, -2, -1.6]
    types = [2, 3, 3] + [6] * 256 + [1] * 12
    tk = GGUFTokenizer(toks, "llama", scores, None, types, bos_id=1, eos_id=2, add_bos=True)
    ids = tk.encode("hello w")
    assert ids[0] == 1 and tk.decode(ids) == "hello w"
    assert tk.decode(tk.encode("héllo", add_bos=False)) == "héllo"         # byte fallback
    from prometorch_b200.io.tokenizer import _B2U
    base = [_B2U[b] for b in range(256)]
    merges = ["h e", "l l", "he ll", "hell o", "Ġ w"]
    vocab = base + ["he", "ll", "hell", "hello", "Ġw", "<|im_start|>"]
    g2 = GGUFTokenizer(vocab, "gpt2", None, merges, [1] * (len(vocab) - 1) + [3])
    ids = g2.encode("<|im_start|>hello w")
    assert ids[0] == len(vocab) - 1 and vocab[ids[1]] == "hello"
    assert g2.decode(ids, skip_special=False) == "<|im_start|>hello w"


def test_chat_templates():
    q = chat.apply_chat_template("hi", "qwen3", no_think=True)
    assert "/no_think<|im_end|>" in q and "<|im_start|>user\nhi<|im_end|>" in q and q.endswith("<|im_start|>assistant\n")
    g = chat.apply_chat_template("hi", "gemma3")
    assert "<start_of_turn>user" in g and g.rstrip().endswith("<start_of_turn>model")
    l3 = chat.apply_chat_template("hi", "llama", model_name="llama3.1", system="be brief")
    assert "<|start_header_id|>system<|end_header_id|>" in l3
    r = chat.render_messages([{"role": "system", "content": "s"}, {"role": "user", "content": "u"}], "qwen3")
    assert r.index("system") < r.index("user")
    assert chat.strip_think("<think>plan</think>answer") == "answer"


def test_ollama_resolution(tmp_path):
    root = tmp_path / "models"
    man = root / "manifests" / "registry.ollama.ai" / "library" / "qwen3"
    man.mkdir(parents=True)
    digest = "sha256:" + "ab" * 32
    (man / "4b").write_text(json.dumps({"layers": [{"mediaType": "application/vnd.ollama.image.model", "digest": digest, "size": 4}]}))
    (root / "blobs").mkdir()
    blob = root / "blobs" / digest.replace(":", "-")
    blob.write_bytes(b"GGUF")
    assert ollama.resolve_model("qwen3:4b", str(root)) == str(blob)
    direct = tmp_path / "x.gguf"
    direct.write_bytes(b"GGUF")
    assert ollama.resolve_model(str(direct)) == str(direct)
    names = [m["name"] for m in ollama.list_models(str(root))]
    assert "qwen3:4b" in names
    with pytest.raises(FileNotFoundError):
        ollama.resolve_model("nope:1b", str(root))


def test_linear_scan_reference_and_gradients():
    """h[t] = g[t] h[t-1] + x[t]: the op's CPU path against a closed form, and its autograd gradients against finite sums."""
    import torch
    from prometorch_b200.ops.scan import linear_scan, parallel_scan
    torch.manual_seed(0)
    g = torch.rand(2, 5, 3, dtype=torch.float64).requires_grad_()
    x = torch.randn(2, 5, 3, dtype=torch.float64).requires_grad_()
    h = linear_scan(g.float(), x.float())
    want = torch.zeros(2, 5, 3)
    for t in range(5):
        for s in range(t + 1):
            want[:, t] += x[:, s].float() * torch.prod(g[:, s + 1:t + 1].float(), dim=1)
    assert torch.allclose(h, want, atol=1e-5) and parallel_scan is linear_scan
    gf, xf = g.detach().float().requires_grad_(), x.detach().float().requires_grad_()
    linear_scan(gf, xf).square().sum().backward()
    # dx[t] = dh[t] + g[t+1] dx[t+1], dg[t] = dx[t] h[t-1]
    dh = 2 * h.detach()
    dx = torch.zeros_like(dh)
    for t in reversed(range(5)):
        dx[:, t] = dh[:, t] + (gf.detach()[:, t + 1] * dx[:, t + 1] if t + 1 < 5 else 0)
    hprev = torch.cat([torch.zeros(2, 1, 3), h.detach()[:, :-1]], 1)
    assert torch.allclose(xf.grad, dx, atol=1e-4) and torch.allclose(gf.grad, dx * hprev, atol=1e-4)
    with pytest.raises(ValueError):
        linear_scan(gf, xf[:, :4])


def test_every_native_switch_is_registered():
    """Every PTB_* environment variable read anywhere in the sources has an entry in utils/env.py."""
    import os
    import re
    from prometorch_b200.utils.env import NATIVE_ENV
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    read = set()
    pat = re.compile(r'(?:getenv|env_int|environ\.get|environ\[)\(?\s*"(PTB_[A-Z0-9_]+)"')
    for base in ("prometorch_b200", "benchmarks"):
        for dp, _, fs in os.walk(os.path.join(root, base)):
            for f in fs:
                if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                    read |= set(pat.findall(open(os.path.join(dp, f), errors="ignore").read()))
    read |= set(pat.findall(open(os.path.join(root, "bench.py")).read()))
    assert read, "the pattern found nothing: the test is broken"
    assert read <= set(NATIVE_ENV), sorted(read - set(NATIVE_ENV))


def test_reference_name_lists_resolve():
    """The reference's public names (nn modules, functional, top-level ops, optimizers, schedulers, distributed) exist."""
    import prometorch_b200 as pt
    nn_names = """ReLU ReLU6 LeakyReLU PReLU ELU SELU GELU Sigmoid Tanh Softmax LogSoftmax Softplus Softsign Hardtanh Hardsigmoid
        Hardswish SiLU Mish Threshold MultiheadAttention Sequential ModuleList ModuleDict ParameterList ParameterDict Conv1d Conv2d
        Conv3d ConvTranspose2d Dropout Dropout1d Dropout2d Dropout3d AlphaDropout FeatureAlphaDropout Identity Linear Bilinear
        LazyLinear Flatten Unflatten LowRankLinear L1Loss MSELoss SmoothL1Loss HuberLoss BCELoss BCEWithLogitsLoss NLLLoss
        CrossEntropyLoss KLDivLoss CosineEmbeddingLoss MarginRankingLoss TripletMarginLoss MultiMarginLoss PoissonNLLLoss
        GaussianNLLLoss CTCLoss FocalLoss DiceLoss BatchNorm1d BatchNorm2d LayerNorm GroupNorm InstanceNorm2d RMSNorm MaxPool1d
        MaxPool2d AvgPool1d AvgPool2d AdaptiveAvgPool1d AdaptiveAvgPool2d AdaptiveMaxPool2d GlobalAvgPool2d RNNCell LSTMCell
        GRUCell RNN LSTM GRU Embedding EmbeddingBag PositionalEncoding TransformerEncoderLayer TransformerEncoder
        TransformerDecoderLayer TransformerDecoder Transformer Upsample SyncBatchNorm""".split()
    missing = [n for n in nn_names if not hasattr(pt.nn, n)]
    assert not missing, missing
    top = """tensor empty zeros ones full rand randn randint arange linspace eye zeros_like ones_like from_numpy cat stack split
        chunk mm bmm matmul dot sum mean max min sqrt exp log sin cos tanh sigmoid relu softmax clamp where cumsum rsqrt norm topk
        sort nan_to_num isinf isnan isfinite multinomial einsum gather scatter masked_fill pad_sequence pack_sequence
        pack_padded_sequence pad_packed_sequence backward grad is_grad_enabled set_grad_enabled no_grad enable_grad save load
        save_state_dict load_state_dict save_pytorch load_pytorch cuda_is_available cuda_device_count compile manual_seed""".split()
    missing = [n for n in top if not hasattr(pt, n)]
    assert not missing, missing
    opt = "SGD Adam AdamW RMSprop Lion SophiaG LAMB Adafactor NAdam RAdam Adagrad Adadelta Adamax AdamKiller ASGD LBFGS EMA ParamGroup".split()
    sch = """StepLR MultiStepLR ExponentialLR CosineAnnealingLR LinearLR ConstantLR ReduceLROnPlateau WarmupCosineAnnealingLR OneCycleLR
        CosineAnnealingWarmRestarts CyclicLR PolynomialLR LambdaLR MultiplicativeLR SequentialLR ChainedScheduler""".split()
    missing = [n for n in opt + sch if not hasattr(pt.optim, n)]
    assert not missing, missing
    dist = """init_process_group destroy_process_group is_initialized get_rank get_world_size all_reduce broadcast barrier
        DistributedDataParallel DDPNoSyncGuard DDPConfig ProcessGroup ReduceOp BackendType FSDPConfig FullyShardedDataParallel
        ZeROOptimizer ZeROStage3 OffloadOptimizer Pipeline1F1BStage PipelineScheduleConfig launch parse_dist_args DistArgs
        SyncBatchNorm""".split()
    missing = [n for n in dist if not hasattr(pt.distributed, n)]
    assert not missing, missing
    par = "TPConfig ColumnParallelLinear RowParallelLinear Pipeline tp_all_gather tp_all_reduce_sum tp_barrier".split()
    missing = [n for n in par if not hasattr(pt.nn.parallel, n)]
    assert not missing, missing


def test_collective_metrics_bytes_and_roofline(tmp_path):
    """Bytes on the wire per collective, bus bandwidth and the roofline fraction of a fused compute+collective step."""
    import json
    from prometorch_b200.utils.metrics import MetricsWriter, measured_peaks, wire_bytes
    assert wire_bytes("all_reduce", 1 << 30, 8) == 2 * (1 << 30) * 7 / 8
    assert wire_bytes("reduce_scatter", 800, 4) == 600 and wire_bytes("all_gather", 800, 4) == 600
    assert wire_bytes("all_reduce", 100, 1) == 0
    w = MetricsWriter(str(tmp_path / "m.jsonl"))
    rec = w.collective("grad all-reduce", seconds=2e-3, payload_bytes=770e6, world=2)          # 770 MB over 770 GB/s = 1 ms
    assert rec["fraction"] == pytest.approx(0.5) and rec["gbps_per_direction"] == pytest.approx(385.0)
    rec = w.collective("gemm + reduce-scatter", seconds=1e-3, payload_bytes=1e6, world=8, kind="reduce_scatter", flops=1.391e12 / 2)
    assert rec["roofline_seconds"] == pytest.approx(0.5e-3) and rec["fraction"] == pytest.approx(0.5)
    w.close()
    lines = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert [l["name"] for l in lines] == ["grad all-reduce", "gemm + reduce-scatter"]
    p = tmp_path / "peaks.json"
    p.write_text(json.dumps({"hbm_gbs": 6000, "bf16_tflops": 1500, "bf16_tflops_sustained": 1300}))
    assert measured_peaks(str(p)) == {"hbm_bw": 6e12, "flops_burst": 1.5e15, "flops_sustained": 1.3e15}


def test_kernels_are_dispatcher_ops():
    """torch.ops.ptb200.* resolve by schema; gradients flow through an op call (CPU tensors take the plain-math path)."""
    import torch
    from prometorch_b200.ops import library
    library.register()
    library.register()                                    # idempotent
    x = torch.randn(4, 32, requires_grad=True)
    w = torch.randn(32, requires_grad=True)
    y = torch.ops.ptb200.rms_norm(x, w, 1e-6)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert torch.allclose(y, ref, atol=1e-5)
    y.sum().backward()
    assert x.grad is not None and w.grad is not None
    lin = torch.ops.ptb200.linear(torch.randn(3, 32), torch.randn(8, 32), None)
    assert lin.shape == (3, 8)
    gu = torch.randn(5, 16)
    assert torch.allclose(torch.ops.ptb200.swiglu(gu, False), torch.nn.functional.silu(gu[:, :8]) * gu[:, 8:], atol=1e-6)
    for name in library.SCHEMAS:
        assert hasattr(torch.ops.ptb200, name)


def test_idx_reader_mnist_and_char_dataset(tmp_path):
    import gzip
    import struct
    import numpy as np
    import torch
    from prometorch_b200.data import MNIST, CharTextDataset, DataLoader, read_idx
    rng = np.random.default_rng(0)
    imgs = rng.integers(0, 256, (12, 28, 28), dtype=np.uint8)
    labs = rng.integers(0, 10, (12,), dtype=np.uint8)
    with open(tmp_path / "train-images-idx3-ubyte", "wb") as f:
        f.write(struct.pack(">HBB", 0, 0x08, 3) + struct.pack(">III", 12, 28, 28) + imgs.tobytes())
    with gzip.open(tmp_path / "train-labels-idx1-ubyte.gz", "wb") as f:
        f.write(struct.pack(">HBB", 0, 0x08, 1) + struct.pack(">I", 12) + labs.tobytes())
    assert torch.equal(read_idx(str(tmp_path / "train-images-idx3-ubyte")), torch.from_numpy(imgs))
    ds = MNIST(str(tmp_path), train=True, flatten=True)
    x, y = ds[5]
    assert len(ds) == 12 and x.shape == (784,) and int(y) == int(labs[5]) and float(x.max()) <= 1.0
    xb, yb = next(iter(DataLoader(ds, batch_size=4)))
    assert xb.shape == (4, 784) and yb.dtype == torch.int64
    f32 = np.arange(6, dtype=">f4").reshape(2, 3)
    with open(tmp_path / "f.idx", "wb") as f:
        f.write(struct.pack(">HBB", 0, 0x0D, 2) + struct.pack(">II", 2, 3) + f32.tobytes())
    assert read_idx(str(tmp_path / "f.idx")).tolist() == [[0.0, 1.0, 2.0], [3.0, 4.0, 5.0]]
    c = CharTextDataset("hello world, hello there", block_size=5, is_text=True)
    a, b = c[3]
    assert c.decode(a) == "lo wo" and c.decode(b) == "o wor" and len(c) == len("hello world, hello there") - 5


def test_ten_model_zoo_trains():
    """examples/train_10_models.py: regression, classification, recurrent cells and the save / load round trip all reach their
    thresholds in the quick setting."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "train_10_models.py")
    spec = importlib.util.spec_from_file_location("train_10_models", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert len(mod.TASKS) == 10 and mod.main(["--quick"]) == 0


def test_generative_and_vision_examples_train():
    """examples/generative_and_vision.py: VAE, GAN, ResNet-20, ViT and the sequence-to-sequence transformer all move."""
    import importlib.util
    import os
    import warnings
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "generative_and_vision.py")
    spec = importlib.util.spec_from_file_location("generative_and_vision", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out = mod.main(["all"])
    assert out["vae"][1] < 0.95 * out["vae"][0]
    assert out["gan"][1] < out["gan"][0] - 1.0
    for name in ("resnet", "vit", "transformer"):
        assert out[name][1] < 0.7 * out[name][0], (name, out[name])


def test_top_level_falls_back_to_torch():
    import promethorch as pt
    import prometorch_b200 as ptb
    assert pt.randn_like(pt.zeros(3)).shape == (3,) and ptb.full_like(ptb.ones(2), 7.0).tolist() == [7.0, 7.0] and pt.Generator is torch.Generator
    with pytest.raises(AttributeError):
        ptb.no_such_function


def test_ecosystem_shims_cover_the_reference_surface(tmp_path):
    """audio (functional + transform modules), text (tokenizers, datasets, batching) and vision (image files) additions."""
    from prometorch_b200 import vision
    # ---- audio
    t = torch.linspace(0, 1, 16000)
    x = torch.sin(2 * math.pi * 440 * t)
    spec = audio.spectrogram(x, 400, 160)
    assert spec.shape[0] == 201 and int(spec.mean(1).argmax()) == round(440 * 400 / 16000)
    assert torch.allclose(audio.Spectrogram(400, 160)(x), spec) and audio.melscale_fbanks(201, 40, 16000).shape == (201, 40)
    mel = audio.MelSpectrogram(16000, 400, 160, 64)(x)
    assert mel.shape[0] == 64 and audio.MFCC(16000, 13, 64, 400, 160)(x).shape[0] == 13
    db = audio.AmplitudeToDB("power", top_db=80.0)(mel)
    assert float(db.max() - db.min()) <= 80.0 + 1e-4
    q = audio.mu_law_encoding(x)
    assert q.dtype == torch.int64 and int(q.min()) >= 0 and int(q.max()) <= 255
    assert float((audio.mu_law_decoding(q) - x).abs().max()) < 0.05
    assert audio.Resample(16000, 8000)(x).shape[-1] == 8000 and audio.hann_window(8).shape == (8,)
    # ---- text
    assert text.BasicTokenizer().tokenize("Hello, World! it's") == ["hello", ",", "world", "!", "it", "'", "s"]
    ct = text.CharTokenizer("hello world")
    assert ct.decode(ct.encode("hello")) == "hello" and ct.encode("z") == [0] and len(ct) == 9
    (tmp_path / "a.txt").write_text("first line\n\nsecond line\n")
    ds = text.TextFileDataset(str(tmp_path / "a.txt"), labels=[0, 1])
    assert len(ds) == 2 and ds[1] == ("second line", 1)
    (tmp_path / "a.csv").write_text("text,label\ngood film,pos\nbad film,neg\n")
    cs = text.CSVDataset(str(tmp_path / "a.csv"), label_column="label")
    assert len(cs) == 2 and cs[0] == (["good film"], "pos") and cs.header == ["text", "label"]
    (tmp_path / "a.jsonl").write_text('{"t": "one", "y": 1}\n{"t": "two", "y": 0}\n')
    js = text.JSONLDataset(str(tmp_path / "a.jsonl"), "t", "y")
    assert js[1] == ("two", 0) and text.JSONLDataset(str(tmp_path / "a.jsonl"))[0] == {"t": "one", "y": 1}
    batch = [[1, 2, 3], [4], [5, 6]]
    assert text.pad_sequence(batch).tolist() == [[1, 2, 3], [4, 0, 0], [5, 6, 0]] and text.pad_sequence(batch, batch_first=False).shape == (3, 3)
    assert text.pad_sequence(batch, padding_value=9, max_len=2).tolist() == [[1, 2], [4, 9], [5, 6]]
    assert text.sequence_lengths(batch).tolist() == [3, 1, 2] and text.padding_mask(batch).tolist() == [[False] * 3, [False, True, True], [False, False, True]]
    packed = text.pack_padded_sequence(text.pad_sequence(batch).unsqueeze(-1).float(), [3, 1, 2])
    assert packed.batch_sizes.tolist() == [3, 2, 1]
    # ---- vision
    img = torch.rand(3, 5, 7)
    vision.save_pnm(str(tmp_path / "c.ppm"), img)
    back = vision.load_image(str(tmp_path / "c.ppm"))
    assert back.shape == (3, 5, 7) and float((back - img).abs().max()) <= 0.5 / 255 + 1e-6
    (tmp_path / "g.pgm").write_bytes(b"P2\n# a comment\n3 2\n15\n0 5 10\n15 1 2\n")
    g = vision.load_pnm(str(tmp_path / "g.pgm"))
    assert g.shape == (1, 2, 3) and torch.allclose(g[0, 1], torch.tensor([15, 1, 2]) / 15)
    for cls in ("cats", "dogs"):
        (tmp_path / "set" / cls).mkdir(parents=True)
        for i in range(2):
            vision.save_pnm(str(tmp_path / "set" / cls / f"{i}.pgm"), torch.rand(1, 4, 4))
    torch.save(torch.rand(1, 4, 4), str(tmp_path / "set" / "cats" / "t.pt"))
    folder = vision.ImageFolder(str(tmp_path / "set"), transform=vision.transforms.Resize(8))
    assert len(folder) == 5 and folder.classes == ["cats", "dogs"] and folder.class_to_idx == {"cats": 0, "dogs": 1}
    xi, yi = folder[4]
    assert xi.shape == (1, 8, 8) and yi == 1
    assert vision.ConvBNReLU(3, 8, stride=2)(torch.rand(2, 3, 8, 8)).shape == (2, 8, 4, 4)
    with pytest.raises(ValueError):
        vision.load_image(str(tmp_path / "a.txt"))


def test_reference_helper_names_of_quantization_data_amp_and_exporters(tmp_path):
    # ---- post-training static quantisation
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Sequential(nn.Linear(32, 8)))
    x = torch.randn(64, 16)
    want = net(x)
    res = Q.quantize_model(net, [x[:32], x[32:]], Q.default_per_channel_qconfig())
    assert res.num_quantized == 2 and res.compression > 2.5 and isinstance(res.model[0], nn.Module)
    assert float((res.model(x) - want).abs().max()) < 0.1 and float(res.model[0].input_scale) > 0
    prepared = Q.prepare(nn.Sequential(nn.Linear(4, 4)), Q.QConfig(bits=8, symmetric=False))
    assert Q.calibrate(prepared, [torch.rand(5, 4)]) == 1 and float(prepared[0].observer.min_val) >= 0
    w = torch.randn(6, 10)
    qt = Q.quantize_per_channel(w, axis=0)
    assert qt.q.dtype == torch.int8 and qt.scale.shape == (6,) and float((qt.dequantize() - w).abs().max()) <= float(qt.scale.max()) / 2 + 1e-6
    assert Q.QuantizedTensor(torch.tensor([2, 4]), torch.tensor(0.5), torch.tensor(0.0)).dequantize().tolist() == [1.0, 2.0]
    t = torch.linspace(-2, 2, 9, requires_grad=True)
    y = Q.fake_quantize_ste(t, 0.01, 0.0, -128, 127)
    assert torch.allclose(y, Q.fake_quantize_qdq(t.detach(), 0.01, 0.0, -128, 127))
    y.sum().backward()
    assert t.grad.tolist() == [0, 0, 1, 1, 1, 1, 1, 0, 0]                      # +-1.27 is the representable range
    packed, absmax = Q.quantize_4bit(torch.randn(2, 64), 64, "int4")
    assert torch.equal(Q.dequantize_int4(packed, absmax, (2, 64)), Q.dequantize_4bit(packed, absmax, (2, 64), 64, "int4"))
    assert Q.pack_nibble(torch.tensor([3]), torch.tensor([10])).tolist() == [0xA3] and Q.Observer is Q.MinMaxObserver
    assert Q.NF4Block(packed, absmax).absmax is absmax and Q.dequantize_nf4(*Q.quantize_4bit(torch.randn(64), 64, "nf4"), (64,)).shape == (64,)
    # ---- data helpers
    ds = data.TensorDataset(torch.arange(10.0).view(10, 1), torch.arange(10))
    loader = data.make_loader(ds, data.DataLoaderOptions(batch_size=4, shuffle=True, drop_last=True, seed=3), collate_fn=data.DefaultCollate())
    batches = list(loader)
    assert len(batches) == 2 and isinstance(batches[0], data.Batch) and batches[0].data.shape == (4, 1) and batches[0].target.shape == (4,)
    again = [b.target.tolist() for b in data.make_loader(ds, data.DataLoaderOptions(batch_size=4, shuffle=True, drop_last=True, seed=3), collate_fn=data.DefaultCollate())]
    assert again == [b.target.tolist() for b in batches]
    d0, t0 = batches[0].to("cpu")
    assert d0.shape == (4, 1) and data.DefaultCollate()([data.Example(torch.ones(2), torch.tensor(1))]).target.tolist() == [1]
    tf = data.Compose([data.Lambda(lambda v: v * 2), data.Normalize([1.0, 2.0], [2.0, 4.0]), data.Flatten()])
    assert tf(torch.ones(2, 3)).tolist() == [0.5, 0.5, 0.5, 0.0, 0.0, 0.0]
    assert list(data.make_batch_sampler(data.make_sequential_sampler(ds), 4)) == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]]
    assert sorted(data.make_random_sampler(ds, seed=1)) == list(range(10))
    # ---- amp state
    assert amp.get_autocast_category("matmul") == amp.CastPolicy.LOWER_PRECISION and amp.policy_for("softmax") == amp.CastPolicy.FP32
    amp.set_autocast_cpu_dtype(torch.bfloat16)
    amp.set_autocast_cpu_enabled(True)
    try:
        assert amp.is_autocast_cpu_enabled() and torch.mm(torch.ones(2, 2), torch.ones(2, 2)).dtype == torch.bfloat16
    finally:
        amp.set_autocast_cpu_enabled(False)
    assert not amp.is_autocast_cpu_enabled() and amp.has_tensor_cores() in (True, False)
    assert amp.autocast_matmul(torch.ones(2, 2), torch.ones(2, 2)).dtype == torch.bfloat16 and amp.autocast_softmax(torch.ones(3).half()).dtype == torch.float32
    s1 = amp.make_grad_scaler(amp.GradScalerOptions(init_scale=8.0, growth_interval=1))
    assert s1.get_scale() == 8.0 and not amp.make_disabled_scaler().enabled
    # ---- exporter and jit names
    mlp = nn.Sequential(nn.Linear(4, 3), nn.ReLU(), nn.Linear(3, 2))
    assert os.path.getsize(onnx.export_model(mlp, (1, 4), str(tmp_path / "m.onnx"))) > 50
    assert "func.func" in mlir.export_mlir(mlp, (1, 4)) and mobile.MobileExecutor is mobile.Executor
    mobile.export_model(mlp, str(tmp_path / "m.ptmb"))
    assert torch.allclose(mobile.MobileExecutor(str(tmp_path / "m.ptmb")).run(torch.ones(1, 4)), mlp(torch.ones(1, 4)), atol=1e-6)
    assert jit.CompiledFn is jit.CompiledModule and jit.tracing_active() is False


def test_draft_statistics_sliding_window_and_remaining_reference_names(tmp_path):
    from prometorch_b200 import distributed as D, io
    from prometorch_b200.serve import llm
    # n-gram draft: proposes what followed the latest earlier occurrence of the current suffix
    d = io.NgramDraft(max_n=3)
    d.reset([1, 2, 3, 4, 5, 1, 2, 3])
    assert d.propose(3) == [4, 5, 1]
    d.append(4)
    assert d.propose(2) == [5, 1]
    d.reset([7, 8, 9])
    assert d.propose(4) == []
    st = io.SpecStats(proposed=8, accepted=6, target_passes=4)
    assert st.acceptance_rate == 0.75 and st.tokens_per_pass(10) == 2.5 and io.SpecStats().acceptance_rate == 0.0
    # sliding window: exact while everything fits, exact again when the window covers what matters, summary otherwise
    torch.manual_seed(0)
    H, Hk, Dh, T = 4, 2, 8, 12
    qs, ks, vs = torch.randn(T, H, Dh), torch.randn(T, Hk, Dh), torch.randn(T, Hk, Dh)

    def full(t):
        K, V = ks[:t + 1].transpose(0, 1), vs[:t + 1].transpose(0, 1)
        s = torch.einsum("kgd,ktd->kgt", qs[t].view(Hk, H // Hk, Dh), K) / Dh ** 0.5
        return torch.einsum("kgt,ktd->kgd", torch.softmax(s, -1), V).reshape(H, Dh)
    exact, windowed = io.SlidingWindowAttention(H, Hk, Dh, window=0), io.SlidingWindowAttention(H, Hk, Dh, window=5)
    for t in range(T):
        a, b = exact.step(qs[t], ks[t], vs[t]), windowed.step(qs[t], ks[t], vs[t])
        assert torch.allclose(a, full(t), atol=1e-5)
        if t < 5:
            assert torch.allclose(b, a, atol=1e-5)
    assert windowed.n_summarized == T - 5 and len(windowed.k) == 5 and torch.allclose(windowed.k_summary, ks[:T - 5].mean(0), atol=1e-5)
    assert float((b - a).abs().max()) < 2.0                       # an approximation, but of the same scale
    # names
    assert io.GGUFTPConfig(1, 4).kwargs() == {"tp_rank": 1, "tp_world": 4} and io.InferenceProfiler is not None and io.LowRankOutputProj is not None
    assert io.GGUFTensorInfo is not None and io.QuantizedWeight is io.PackedWeight
    ctx = D.DistributedContext.current()
    assert ctx.rank == 0 and ctx.world_size == 1 and ctx.is_main and D.NCCLBackend is not None
    p = nn.Parameter(torch.ones(3))
    off = D.OffloadOptimizer([p], torch.optim.SGD, lr=0.1, momentum=0.9)
    p.grad = torch.ones(3)
    off.step()
    bag = off.state_bags()[0]
    assert isinstance(bag, D.OffloadStateBag) and torch.allclose(bag["master"], torch.full((3,), 0.9)) and "momentum_buffer" in bag
    assert llm.KVCache is llm.PagedKVCache and llm.ByteBPETokenizer().decode(llm.ByteBPETokenizer().encode("hé")) .endswith("hé")


def test_promepile_names_train_and_decode_steps():
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 1))
    x = torch.randn(64, 8)
    y = torch.sin(x[:, :1]) + 0.5 * x[:, 1:2]                       # a target the network can learn
    step = jit.promepile_train(net, pt.optim.Adam(net.parameters(), lr=1e-2), nn.functional.mse_loss, max_grad_norm=1.0)
    losses = [float(step(x, target=y)) for _ in range(80)]
    assert step.steps == 80 and losses[-1] < 0.5 * losses[0] and isinstance(step, jit.CompiledTrainingStep)
    scaled = jit.promepile_train(net, pt.optim.SGD(net.parameters(), lr=1e-2), nn.functional.mse_loss, scaler=amp.GradScaler(init_scale=4.0))
    before = float(nn.functional.mse_loss(net(x), y))
    scaled(x, target=y)
    assert float(nn.functional.mse_loss(net(x), y)) < before
    fwd = jit.promepile(net)
    assert isinstance(fwd, jit.CompiledForward) and torch.allclose(fwd(x), net(x))

    class FakeModel:
        captured = 0

        def capture(self):
            self.captured += 1

        def forward_decode(self, token, pos):
            return token + pos
    m = FakeModel()
    dec = jit.CompiledDecodeStep(m)
    assert m.captured == 1 and dec(5, 7) == 12
