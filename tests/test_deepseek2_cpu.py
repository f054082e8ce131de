"""deepseek2 (latent attention + mixture of experts): the batched latent-cache model against a per-token, per-head
restatement with materialised K and V, the formulation of the reference's CPU decode
(torch/io/deepseek2_forward.h:117-520)."""
import math

import pytest
import torch

from prometorch_b200.io.gguf import GGUFReader
from prometorch_b200.io.synthetic import write_synthetic_deepseek2
from prometorch_b200.models.deepseek2 import DeepSeek2Config, DeepSeek2Model, yarn_rope_tables


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean() + eps) * w


class LoopDecoder:
    """One token at a time, one head at a time, K and V expanded and cached per head."""

    def __init__(self, path):
        self.r = GGUFReader(path)
        self.c = DeepSeek2Config.from_gguf(self.r)
        self.cos, self.sin = yarn_rope_tables(self.c, 256)
        self.K = [[] for _ in range(self.c.num_layers)]
        self.V = [[] for _ in range(self.c.num_layers)]
        self.pos = 0

    def w(self, n):
        return self.r.load(n)

    def rope(self, v, pos):
        h = v.shape[-1] // 2
        c, s = self.cos[pos], self.sin[pos]
        return torch.cat([v[:h] * c - v[h:] * s, v[:h] * s + v[h:] * c])

    def step(self, tok):
        c, pos = self.c, self.pos
        x = self.w("token_embd.weight")[tok]
        nope, rope, kvl, vd, nh = c.qk_nope, c.rope_dim, c.kv_lora_rank, c.value_length, c.num_heads
        kq = 1.0
        if c.rope_yarn and c.yarn_factor > 1:
            lf = math.log(c.yarn_factor)
            kq = (1 + 0.1 * lf) * (1 + 0.1 * c.yarn_log_multiplier * lf)
        scale = kq * kq / math.sqrt(c.key_length)
        for i in range(c.num_layers):
            p = f"blk.{i}."
            h = _rms(x, self.w(p + "attn_norm.weight"), c.rms_norm_eps)
            if self.r.has_tensor(p + "attn_q.weight"):
                q = self.w(p + "attn_q.weight") @ h
            else:
                q = self.w(p + "attn_q_b.weight") @ _rms(self.w(p + "attn_q_a.weight") @ h, self.w(p + "attn_q_a_norm.weight"), c.rms_norm_eps)
            kv = self.w(p + "attn_kv_a_mqa.weight") @ h
            lat = _rms(kv[:kvl], self.w(p + "attn_kv_a_norm.weight"), c.rms_norm_eps)
            k_pe = self.rope(kv[kvl:], pos)
            kb, vb = self.w(p + "attn_k_b.weight"), self.w(p + "attn_v_b.weight")
            k_heads, v_heads = [], []
            for hd in range(nh):
                k_nope = kb[hd].t() @ lat                     # [qk_nope] = sum_r M[r, c] lat[r]
                k_heads.append(torch.cat([k_nope, k_pe]))
                v_heads.append(vb[hd] @ lat)
            self.K[i].append(torch.stack(k_heads))
            self.V[i].append(torch.stack(v_heads))
            out = []
            for hd in range(nh):
                qh = q[hd * c.key_length:(hd + 1) * c.key_length].clone()
                qh[nope:] = self.rope(qh[nope:], pos)
                sc = torch.stack([(qh * self.K[i][t][hd]).sum() * scale for t in range(pos + 1)]).softmax(0)
                out.append(sum(sc[t] * self.V[i][t][hd] for t in range(pos + 1)))
            x = x + self.w(p + "attn_output.weight") @ torch.cat(out)
            h = _rms(x, self.w(p + "ffn_norm.weight"), c.rms_norm_eps)

            def glu(g, u, d, v):
                return d @ (torch.nn.functional.silu(g @ v) * (u @ v))
            if i < c.leading_dense:
                x = x + glu(self.w(p + "ffn_gate.weight"), self.w(p + "ffn_up.weight"), self.w(p + "ffn_down.weight"), h)
            else:
                s = torch.sigmoid(self.w(p + "ffn_gate_inp.weight") @ h)
                top = sorted(range(c.expert_count), key=lambda e: -float(s[e]))[:c.expert_used_count]
                tot = sum(float(s[e]) for e in top)
                ge, ue, de = self.w(p + "ffn_gate_exps.weight"), self.w(p + "ffn_up_exps.weight"), self.w(p + "ffn_down_exps.weight")
                y = sum((float(s[e]) / tot) * glu(ge[e], ue[e], de[e], h) for e in top)
                if self.r.has_tensor(p + "ffn_gate_shexp.weight"):
                    y = y + glu(self.w(p + "ffn_gate_shexp.weight"), self.w(p + "ffn_up_shexp.weight"), self.w(p + "ffn_down_shexp.weight"), h)
                x = x + y
        self.pos += 1
        return self.w("output.weight") @ _rms(x, self.w("output_norm.weight"), c.rms_norm_eps)


@pytest.mark.parametrize("q_lora", [0, 64])
def test_latent_cache_model_matches_the_per_head_loop(tmp_path, q_lora):
    path = str(tmp_path / "ds2.gguf")
    write_synthetic_deepseek2(path, q_lora=q_lora, seed=3 + q_lora)
    m = DeepSeek2Model(path, max_seq=64)
    ref = LoopDecoder(path)
    toks = [5, 100, 17, 250, 31, 8, 77]
    want = torch.stack([ref.step(t) for t in toks])
    got = m.forward(toks[:4])                       # a batched pass over the first tokens ...
    got = torch.cat([got] + [m.forward([t]) for t in toks[4:]])       # ... then token by token on the same cache
    assert torch.allclose(got, want, rtol=2e-4, atol=2e-4), float((got - want).abs().max())
    assert m.cache_bytes_per_token == 4 * m.cfg.num_layers * (m.cfg.kv_lora_rank + m.cfg.rope_dim)
    out = m.generate(toks[:3], max_new_tokens=4)
    assert len(out) <= 4 and all(0 <= t < m.cfg.vocab_size for t in out)


def test_yarn_tables_follow_the_ramp():
    c = DeepSeek2Config(rope_dim=32, rope_freq_base=10000.0, rope_yarn=True, yarn_factor=4.0, yarn_orig_ctx=64, yarn_log_multiplier=0.1)
    cos, sin = yarn_rope_tables(c, 8)
    m = 1 + 0.1 * math.log(4.0)
    assert cos[0].tolist() == pytest.approx([m] * 16)
    # the highest-frequency pair is extrapolated (unscaled), the lowest-frequency pair interpolated (divided by 4)
    assert float(cos[3, 0]) == pytest.approx(m * math.cos(3.0), abs=1e-5)
    inv_last = 10000.0 ** (-30.0 / 32)
    assert float(sin[5, 15]) == pytest.approx(m * math.sin(5 * inv_last / 4), abs=1e-6)
