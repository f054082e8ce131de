"""CPU tests of the GGUF stack: block formats, container I/O, config parsing, the fp32 oracle."""
import os

import pytest
import torch

from prometorch_b200.io import gguf_quant as Q
from prometorch_b200.io.config import TransformerConfig, tiny_qwen3_config
from prometorch_b200.io.gguf import GGUFReader, GGUFWriter
from prometorch_b200.io.synthetic import write_synthetic_gguf


@pytest.mark.parametrize("qt,tol", [(Q.GGMLType.Q4_K, 0.08), (Q.GGMLType.Q5_K, 0.04), (Q.GGMLType.Q6_K, 0.02),
                                    (Q.GGMLType.Q8_0, 0.006), (Q.GGMLType.Q4_0, 0.12), (Q.GGMLType.F16, 1e-3)])
def test_quant_roundtrip(qt, tol):
    torch.manual_seed(0)
    x = torch.randn(7, 512) * 0.02
    b = Q.quantize(x, qt)
    assert b.dtype == torch.uint8 and b.shape == (7, Q.row_bytes(qt, 512))
    y = Q.dequantize(b, qt, 512)
    rel = (y - x).norm() / x.norm()
    assert rel < tol, rel


def test_q4k_scalar_reference():
    """Vectorised Q4_K dequant equals a scalar walk of the documented bit layout."""
    torch.manual_seed(1)
    x = torch.randn(1, 256)
    b = Q.quantize_q4_k(x)[0].tolist()
    import struct
    d = struct.unpack("<e", bytes(b[0:2]))[0]
    dmin = struct.unpack("<e", bytes(b[2:4]))[0]
    sc = b[4:16]
    qs = b[16:144]

    def scale_min(j):
        if j < 4:
            return sc[j] & 63, sc[j + 4] & 63
        return (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)
    ref = []
    for j in range(4):
        s1, m1 = scale_min(2 * j)
        s2, m2 = scale_min(2 * j + 1)
        chunk = qs[32 * j:32 * j + 32]
        ref += [d * s1 * (q & 0xF) - dmin * m1 for q in chunk]
        ref += [d * s2 * (q >> 4) - dmin * m2 for q in chunk]
    y = Q.dequantize_q4_k(torch.tensor(b, dtype=torch.uint8)[None], 256)[0]
    assert torch.allclose(y, torch.tensor(ref), atol=1e-6)


def test_q6k_scalar_reference():
    torch.manual_seed(2)
    x = torch.randn(1, 256)
    b = Q.quantize_q6_k(x)[0].tolist()
    import struct
    ql, qh, sc = b[0:128], b[128:192], b[192:208]
    sc = [s - 256 if s > 127 else s for s in sc]
    d = struct.unpack("<e", bytes(b[208:210]))[0]
    ref = [0.0] * 256
    for n in range(2):
        for l in range(32):
            isx = l // 16
            q1 = ((ql[n * 64 + l] & 0xF) | (((qh[n * 32 + l] >> 0) & 3) << 4)) - 32
            q2 = ((ql[n * 64 + l + 32] & 0xF) | (((qh[n * 32 + l] >> 2) & 3) << 4)) - 32
            q3 = ((ql[n * 64 + l] >> 4) | (((qh[n * 32 + l] >> 4) & 3) << 4)) - 32
            q4 = ((ql[n * 64 + l + 32] >> 4) | (((qh[n * 32 + l] >> 6) & 3) << 4)) - 32
            ref[n * 128 + l] = d * sc[n * 8 + isx] * q1
            ref[n * 128 + l + 32] = d * sc[n * 8 + isx + 2] * q2
            ref[n * 128 + l + 64] = d * sc[n * 8 + isx + 4] * q3
            ref[n * 128 + l + 96] = d * sc[n * 8 + isx + 6] * q4
    y = Q.dequantize_q6_k(torch.tensor(b, dtype=torch.uint8)[None], 256)[0]
    assert torch.allclose(y, torch.tensor(ref), atol=1e-6)


def test_gguf_roundtrip(tmp_path):
    p = str(tmp_path / "t.gguf")
    w = GGUFWriter(p)
    w.add("general.architecture", "llama")
    w.add("llama.block_count", 3)
    w.add("llama.rope.freq_base", 10000.0)
    w.add("tokenizer.ggml.tokens", ["a", "b", "c"])
    x = torch.randn(4, 256)
    w.add_tensor("m.weight", (4, 256), Q.GGMLType.Q6_K, Q.quantize(x, Q.GGMLType.Q6_K))
    w.add_tensor("n.weight", (5,), Q.GGMLType.F32, Q.quantize(torch.arange(5.0), Q.GGMLType.F32))
    w.write()
    r = GGUFReader(p)
    assert r.get("llama.block_count") == 3 and r.get("tokenizer.ggml.tokens") == ["a", "b", "c"]
    assert r.tensors["m.weight"].shape == (4, 256) and r.tensors["m.weight"].offset % 32 == 0
    assert torch.equal(r.load("n.weight"), torch.arange(5.0))
    assert (r.load("m.weight") - x).norm() / x.norm() < 0.02
    r.close()


def test_synthetic_model_and_oracle(tmp_path):
    from prometorch_b200.models.gguf_oracle import OracleModel
    cfg = tiny_qwen3_config(layers=2, hidden=256, heads=4, kv_heads=2, inter=512, vocab=300)
    p = write_synthetic_gguf(str(tmp_path / "tiny.gguf"), cfg, seed=3, device="cpu")
    r = GGUFReader(p)
    c2 = TransformerConfig.from_gguf(r)
    assert (c2.hidden_size, c2.num_layers, c2.num_heads, c2.num_kv_heads, c2.head_dim) == (256, 2, 4, 2, 128)
    assert c2.has_qk_norm and c2.rope_neox and c2.vocab_size == 300
    assert r.tensors["blk.0.attn_v.weight"].qtype == Q.GGMLType.Q6_K
    assert r.tensors["blk.0.attn_q.weight"].qtype == Q.GGMLType.Q4_K
    m = OracleModel(r)
    toks = [5, 17, 42, 250]
    full = m.forward(toks)
    m.reset()
    inc = torch.cat([m.forward([t]) for t in toks])
    assert full.shape == (4, 300)
    assert torch.allclose(full, inc, atol=1e-4), (full - inc).abs().max()


def test_tile16_layout_round_trip():
    """The tensor-pipe GEMV's weight layout, rebuilt from its description, gives back the file's blocks."""
    import torch
    from prometorch_b200.io.gguf import GGMLType
    from prometorch_b200.io.gguf_model import tile16_major
    g = torch.Generator().manual_seed(3)
    for qt, bb in ((GGMLType.Q4_K, 144), (GGMLType.Q6_K, 210)):
        n, nblk, b0, b1 = 37, 5, 1, 4
        raw = torch.randint(0, 256, (n, nblk * bb), generator=g, dtype=torch.uint8)
        packed = tile16_major(raw, qt, b0, b1)
        nb, ntile = b1 - b0, (n + 15) // 16
        assert packed.numel() == ntile * nb * 16 * bb
        want = raw.reshape(n, nblk, bb)[:, b0:b1]
        units = packed.reshape(ntile, nb, 16 * bb)
        for r in (0, 5, 15, 16, 36):
            tile, rr = divmod(r, 16)
            for b in range(nb):
                u = units[tile, b]
                if qt == GGMLType.Q4_K:
                    got = u[rr * 144:(rr + 1) * 144]
                else:
                    ql = u[rr * 128:(rr + 1) * 128].reshape(8, 16)
                    qh = u[2048 + rr * 64:2048 + (rr + 1) * 64].reshape(4, 16)
                    ql = torch.stack([ql[c ^ (rr & 7)] for c in range(8)]).reshape(-1)       # logical chunk c sits at c ^ key
                    qh = torch.stack([qh[c ^ ((rr >> 1) & 3)] for c in range(4)]).reshape(-1)
                    got = torch.cat([ql, qh, u[3072 + rr * 16:3072 + (rr + 1) * 16], u[3328 + rr * 2:3328 + (rr + 1) * 2]])
                assert torch.equal(got, want[r, b]), (qt, r, b)
        assert int(units[ntile - 1].reshape(nb, 16, -1)[:, 0].sum()) >= 0       # padded rows exist (zeros)


def test_tile16_layout_of_q5k_q8_0_f16():
    """Q5_K keeps the file's blocks; Q8_0 and F16 are rebuilt from the swizzle rule in the layout's description."""
    import torch
    from prometorch_b200.io.gguf import GGMLType
    from prometorch_b200.io.gguf_model import tile16_major
    g = torch.Generator().manual_seed(4)
    n, nblk, b0, b1 = 21, 4, 1, 3
    nb, ntile = b1 - b0, 2
    raw = torch.randint(0, 256, (n, nblk * 176), generator=g, dtype=torch.uint8)
    units = tile16_major(raw, GGMLType.Q5_K, b0, b1).reshape(ntile, nb, 16, 176)
    assert torch.equal(units[1, 1, 4], raw.reshape(n, nblk, 176)[20, b0 + 1])
    assert int(units[1, :, 5:].sum()) == 0                                   # rows 21..31 are padding
    raw = torch.randint(0, 256, (n, nblk * 8 * 34), generator=g, dtype=torch.uint8)
    units = tile16_major(raw, GGMLType.Q8_0, b0, b1).reshape(ntile, nb, 4352)
    want = raw.reshape(n, nblk, 8, 34)
    for r in (0, 7, 13, 20):
        tile, rr = divmod(r, 16)
        for b in range(nb):
            u = units[tile, b]
            q = u[rr * 256:(rr + 1) * 256].reshape(8, 32)
            for s in range(8):
                assert torch.equal(q[s ^ (rr & 7)], want[r, b0 + b, s, 2:]), (r, b, s)
                assert torch.equal(u[4096 + rr * 16 + 2 * s:4096 + rr * 16 + 2 * s + 2], want[r, b0 + b, s, :2])
    raw = torch.randint(0, 256, (n, nblk * 512), generator=g, dtype=torch.uint8)
    units = tile16_major(raw, GGMLType.F16, b0, b1).reshape(ntile, nb * 4, 16, 4, 32)      # [tile][64-value block][row][unit][32 B]
    want = raw.reshape(n, nblk, 4, 4, 32)                                                   # [row][256 block][quarter][unit][32 B]
    for r in (0, 6, 15, 17):
        tile, rr = divmod(r, 16)
        for b in range(nb):
            for qtr in range(4):
                for u in range(4):
                    assert torch.equal(units[tile, b * 4 + qtr, rr, u ^ (rr & 3)], want[r, b0 + b, qtr, u]), (r, b, qtr, u)


def _ggml_q2_k_scalar(block: bytes):
    """ggml's dequantize_row_q2_K, one block, written out as scalar loops (the golden order of values)."""
    import numpy as np
    scales, qs = block[0:16], block[16:80]
    d = float(np.frombuffer(block[80:82], dtype=np.float16)[0])
    dmin = float(np.frombuffer(block[82:84], dtype=np.float16)[0])
    y, is_, q = [], 0, 0
    for _n in range(0, 256, 128):
        shift = 0
        for _j in range(4):
            for off in (0, 16):
                sc = scales[is_]
                is_ += 1
                dl, ml = d * (sc & 0xF), dmin * (sc >> 4)
                y += [dl * ((qs[q + off + l] >> shift) & 3) - ml for l in range(16)]
            shift += 2
        q += 32
    return y


def _ggml_q3_k_scalar(block: bytes):
    import numpy as np
    hm, qs, sr = block[0:32], block[32:96], block[96:108]
    d = float(np.frombuffer(block[108:110], dtype=np.float16)[0])
    aux = list(np.frombuffer(bytes(sr), dtype=np.uint32).astype(np.uint64))
    k1, k2 = 0x03030303, 0x0f0f0f0f
    tmp = int(aux[2])
    a0, a1 = int(aux[0]), int(aux[1])
    w = [(a0 & k2) | (((tmp >> 0) & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4),
         ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)]
    scales = np.frombuffer(np.array(w, dtype=np.uint32).tobytes(), dtype=np.int8).astype(int)
    y, is_, q, m = [], 0, 0, 1
    for _n in range(0, 256, 128):
        shift = 0
        for _j in range(4):
            for off in (0, 16):
                dl = d * (scales[is_] - 32)
                is_ += 1
                y += [dl * (((qs[q + off + l] >> shift) & 3) - (0 if hm[off + l] & m else 4)) for l in range(16)]
            shift += 2
            m <<= 1
        q += 32
    return y


def test_q2k_q3k_dequant_follow_ggml_order():
    import numpy as np
    import torch
    from prometorch_b200.io.gguf import GGMLType
    from prometorch_b200.io.gguf_quant import dequantize
    rng = np.random.default_rng(0)
    for qt, nbytes, scalar, dpos in ((GGMLType.Q2_K, 84, _ggml_q2_k_scalar, (80, 82)), (GGMLType.Q3_K, 110, _ggml_q3_k_scalar, (108,))):
        raw = rng.integers(0, 256, size=(3, 2 * nbytes), dtype=np.uint8)
        for r in range(3):
            for blk in range(2):
                for p in dpos:      # sane fp16 scales
                    raw[r, blk * nbytes + p:blk * nbytes + p + 2] = np.frombuffer(np.float16(rng.uniform(0.01, 0.1)).tobytes(), dtype=np.uint8)
        got = dequantize(torch.from_numpy(raw), qt, 512)
        for r in range(3):
            want = scalar(raw[r, :nbytes].tobytes()) + scalar(raw[r, nbytes:].tobytes())
            assert torch.allclose(got[r], torch.tensor(want, dtype=torch.float32), atol=1e-6), (qt, r)


def test_merged_qkv_and_gate_up_and_longrope(tmp_path):
    """A phi-3 style file (attn_qkv, ffn_up of twice the FFN width, LongRoPE factor tensors) decodes like the same
    weights stored as separate tensors, and the factor set follows the sequence length."""
    import torch
    from prometorch_b200.io.config import TransformerConfig, tiny_qwen3_config
    from prometorch_b200.io.gguf import GGMLType, GGUFReader, GGUFWriter
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.models.gguf_oracle import OracleModel, rope_tables
    cfg = tiny_qwen3_config(layers=2, hidden=256, heads=4, kv_heads=2, inter=512, vocab=300, head_dim=64)
    merged = str(tmp_path / "merged.gguf")
    short = [1.0 + 0.01 * i for i in range(32)]
    long = [2.0 + 0.1 * i for i in range(32)]
    write_synthetic_gguf(merged, cfg, seed=2, device="cpu", merged=True, rope_factors=(short, long), rope_orig_ctx=64)
    r = GGUFReader(merged)
    c = TransformerConfig.from_gguf(r)
    assert c.rope_orig_ctx == 64 and c.rope_factors_for(64) == pytest.approx(short) and c.rope_factors_for(65) == pytest.approx(long)
    cos_s, _ = rope_tables(c, 64)
    cos_l, _ = rope_tables(c, 128)
    assert not torch.allclose(cos_s[:64], cos_l[:64])
    # the same bytes, split into separate tensors
    split = str(tmp_path / "split.gguf")
    w = GGUFWriter(split)
    for k, v in r.metadata.items():
        if not k.startswith("general.alignment"):
            w.add(k, v)
    Q, KV, I = c.q_dim, c.kv_dim, c.intermediate_size
    for name, ti in r.tensors.items():
        raw = r.raw(name).clone()
        if name.endswith("attn_qkv.weight"):
            p = name[:-len("attn_qkv.weight")]
            for part, (a, b) in (("attn_q", (0, Q)), ("attn_k", (Q, Q + KV)), ("attn_v", (Q + KV, Q + 2 * KV))):
                w.add_tensor(p + part + ".weight", (b - a, ti.shape[-1]), ti.qtype, (lambda x=raw[a:b].contiguous(): x))
        elif name.endswith("ffn_up.weight"):
            p = name[:-len("ffn_up.weight")]
            w.add_tensor(p + "ffn_gate.weight", (I, ti.shape[-1]), ti.qtype, (lambda x=raw[:I].contiguous(): x))
            w.add_tensor(p + "ffn_up.weight", (I, ti.shape[-1]), ti.qtype, (lambda x=raw[I:].contiguous(): x))
        else:
            w.add_tensor(name, ti.shape, ti.qtype, (lambda x=raw: x))
    w.write()
    toks = [5, 17, 200, 31, 8]
    a = OracleModel(merged, max_seq=64).forward(toks)
    b = OracleModel(split, max_seq=64).forward(toks)
    assert torch.equal(a, b)


def test_lowrank_output_projection_finds_the_exact_argmax():
    """A matrix with a decaying spectrum: the exact winner is among the low-rank candidates, so the speculative head
    returns the full arg-max; sampling stays inside the exact top-k."""
    import torch
    from prometorch_b200.io.gguf_quant import GGMLType, dequantize, quantize
    from prometorch_b200.io.speculative import LowRankOutputProj
    g = torch.Generator().manual_seed(0)
    vocab, hidden = 3000, 256
    A, B = torch.randn(vocab, 48, generator=g), torch.randn(48, hidden, generator=g)
    W = A @ B / 7 + 0.02 * torch.randn(vocab, hidden, generator=g)
    raw = quantize(W, GGMLType.Q6_K)
    Wq = dequantize(raw, GGMLType.Q6_K, hidden)
    lr = LowRankOutputProj(rank=64, candidate_k=32).init_from_quantized(raw, GGMLType.Q6_K, hidden)
    assert lr.valid and lr.U.shape == (vocab, 64) and lr.V.shape == (64, hidden)
    hits = 0
    for i in range(40):
        x = torch.randn(hidden, generator=g)
        want = int((Wq @ x).argmax())
        got = lr.decode_greedy(x)
        hits += got == want
        assert float(lr.last_exact.max()) == pytest.approx(float((Wq @ x)[got]), rel=1e-5)
        t = lr.decode_sample(x, temperature=0.8, top_k=5, generator=g)
        assert t in set((Wq @ x)[lr.last_candidates].topk(5).indices.tolist() and lr.last_candidates[lr.last_exact.topk(5).indices].tolist())
    assert hits >= 38, hits
    f = LowRankOutputProj(rank=32, candidate_k=16).init_from_float(W)
    x = torch.randn(hidden, generator=g)
    assert 0 <= f.decode_greedy(x) < vocab


def test_weight_layout_follows_the_number_of_ranks(monkeypatch):
    from prometorch_b200.io.gguf_model import LAYOUT_SEGMENT, LAYOUT_T16, default_layout
    monkeypatch.delenv("PTB_GEMV_LAYOUT", raising=False)
    assert default_layout(1) == LAYOUT_T16
    assert [default_layout(w) for w in (2, 4, 8)] == [LAYOUT_SEGMENT] * 3
    monkeypatch.setenv("PTB_GEMV_LAYOUT", "t16")
    assert default_layout(8) == LAYOUT_T16
    monkeypatch.setenv("PTB_GEMV_LAYOUT", "segment")
    assert default_layout(1) == LAYOUT_SEGMENT


def test_generate_cli_on_the_cpu_oracle(tmp_path, monkeypatch, capsys):
    """`python -m prometorch_b200.generate --device cpu`: the fp32 oracle behind the reference CLI's flags, the token-id dump
    switch under the reference's spelling, and `--info` / `--tensors` without a model load."""
    from prometorch_b200 import generate as G
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    p = str(tmp_path / "cli.gguf")
    write_synthetic_gguf(p, tiny_qwen3_config(layers=1, hidden=256, heads=4, kv_heads=2, inter=512, vocab=512), seed=4, device="cpu")
    monkeypatch.setenv("PT_DEBUG_TOKENS", "1")
    assert G.main([p, "t300 t301 t400", "--device", "cpu", "--greedy", "--max-tokens", "3"]) == 0
    out = capsys.readouterr().out
    assert "[Generate] Prompt tokens: 3" in out and "[Tokens] prompt [300, 301, 400]" in out and "[Tokens] generated [" in out and "tok/s" in out
    monkeypatch.delenv("PT_DEBUG_TOKENS")
    assert G.main([p, "--info", "--tensors"]) == 0
    out = capsys.readouterr().out
    assert "general.architecture = 'qwen3'" in out and "blk.0.attn_q.weight" in out and "[Tokens]" not in out


def test_generate_cli_tensor_parallel_on_cpu_ranks(tmp_path):
    """`generate --device cpu --nprocs 2`: the CLI re-launches itself under torch.distributed.run and decodes with the sharded
    oracle over gloo; the ids equal the single-process run's."""
    import os
    import subprocess
    import sys
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    p = str(tmp_path / "tp.gguf")
    write_synthetic_gguf(p, tiny_qwen3_config(layers=2, hidden=256, heads=4, kv_heads=2, inter=768, vocab=512), seed=8, device="cpu", std=0.05)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PT_DEBUG_TOKENS="1", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    outs = []
    for extra in ([], ["--nprocs", "2", "--master-port", str(29900 + os.getpid() % 90)]):
        r = subprocess.run([sys.executable, "-m", "prometorch_b200.generate", p, "t300 t301 t400", "--device", "cpu", "--greedy", "--max-tokens", "4"] + extra,
                           capture_output=True, text=True, timeout=300, env=env, cwd=root)
        assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
        line = [ln for ln in r.stdout.splitlines() if ln.startswith("[Tokens] generated")]
        assert len(line) == 1, r.stdout                                         # only rank 0 prints
        outs.append(line[0])
    assert outs[0] == outs[1]
