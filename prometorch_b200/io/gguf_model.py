"""GGUFModel: load a GGUF decoder, repack its weights for the sm_100a GEMV
kernels, and drive the native decode engine.

Public surface follows the reference's ``GGUFModel``
(torch/io/gguf_model.h: ``load``, ``load_quantized_to_cuda``, ``forward``,
``forward_decode``, ``init_tensor_parallel``, ``generate``, ``chat``,
``sample_token``, ``apply_chat_template``) with these design differences:

* weights go host→device once and are repacked on the GPU (Q6_K rows become a
  16 B-aligned structure of arrays; Q4_K stays byte-identical to the file);
* the KV cache is fp16 only, laid out ``[layer][kv_head][seq][128]``;
* a whole run of tokens (prompt and generation) is enqueued as CUDA-graph
  replays with the sampled token fed back on the device;
* tensor parallelism shards Q/K/V/gate/up by rows and attn_output/ffn_down by
  256-element super-blocks along K with the same non-uniform remainder rule
  (torch/io/gguf_model.h:5239-5246) and runs on GPUs, with the partial-sum
  all-reduce fused into the GEMV kernel over NVLink peer memory.
"""
from __future__ import annotations

import ctypes as C
import math
import time
from typing import Callable, Iterable, List, Optional, Sequence

import torch

from .. import _native as N
from .config import TransformerConfig, layer_matrix_sources
from .gguf import GGUFReader
from .gguf_quant import GGMLType, dequantize, quantize

QT_Q4K, QT_Q6K, QT_F16, QT_F32, QT_Q5K, QT_Q8_0 = 0, 1, 2, 3, 4, 5


def split_blocks(nblk: int, world: int, rank: int):
    """Non-uniform block partition: the first ``nblk % world`` ranks take one extra."""
    base, rem = divmod(nblk, world)
    b0 = rank * base + min(rank, rem)
    return b0, b0 + base + (1 if rank < rem else 0)


SEG_BLOCKS = 10     # must match GEMV_SEG_BLOCKS in csrc/decode_kernels.cuh


def segments(nblk: int):
    """Block ranges of the K segments: ``ceil(nblk/10)`` segments, the first ``nblk % KS`` one longer."""
    ks = (nblk + SEG_BLOCKS - 1) // SEG_BLOCKS
    return [split_blocks(nblk, ks, s) for s in range(ks)]


def _q6k_soa(blk: torch.Tensor) -> torch.Tensor:
    """Q6_K blocks ``[N, nb, 210]`` -> structure of arrays ``[N, nb*208 + pad16(nb*2)]``."""
    n, nb = blk.shape[0], blk.shape[1]
    parts = [blk[:, :, 0:128].reshape(n, nb * 128), blk[:, :, 128:192].reshape(n, nb * 64),
             blk[:, :, 192:208].reshape(n, nb * 16), blk[:, :, 208:210].reshape(n, nb * 2)]
    pad = (-nb * 2) % 16
    if pad:
        parts.append(torch.zeros(n, pad, dtype=torch.uint8, device=blk.device))
    return torch.cat(parts, dim=1)


def repack_q6k(raw: torch.Tensor, b0: int = 0, b1: Optional[int] = None) -> torch.Tensor:
    """Row-major SoA rows (the embedding-table layout): ``ql | qh | scales | d(+pad)`` per row."""
    n = raw.shape[0]
    return _q6k_soa(raw.reshape(n, -1, 210)[:, b0:b1]).contiguous()


def slice_q4k(raw: torch.Tensor, b0: int = 0, b1: Optional[int] = None) -> torch.Tensor:
    n = raw.shape[0]
    return raw.reshape(n, -1, 144)[:, b0:b1].reshape(n, -1).contiguous()


def segment_major(raw: torch.Tensor, qtype: GGMLType, b0: int, b1: int) -> torch.Tensor:
    """The GEMV streaming layout ``[segment][row][segment bytes]`` over blocks ``[b0, b1)`` of every row."""
    n = raw.shape[0]
    bb = 144 if qtype == GGMLType.Q4_K else 210
    blk = raw.reshape(n, -1, bb)[:, b0:b1]
    out = []
    for s0, s1 in segments(b1 - b0):
        seg = blk[:, s0:s1]
        out.append(seg.reshape(n, -1).reshape(-1) if qtype == GGMLType.Q4_K else _q6k_soa(seg).reshape(-1))
    return torch.cat(out).contiguous()


LAYOUT_SEGMENT, LAYOUT_T16 = 0, 1


# bytes of one row's block as stored in the file, and values per block, for the types the tile layout takes natively
_FILE_BLOCK = {GGMLType.Q4_K: (144, 256), GGMLType.Q6_K: (210, 256), GGMLType.Q5_K: (176, 256), GGMLType.Q8_0: (34, 32),
               GGMLType.F16: (2, 1)}
_KERNEL_TYPE = {GGMLType.Q4_K: QT_Q4K, GGMLType.Q6_K: QT_Q6K, GGMLType.Q5_K: QT_Q5K, GGMLType.Q8_0: QT_Q8_0,
                GGMLType.F16: QT_F16}


def _swizzle_units(x: torch.Tensor, mask: int) -> torch.Tensor:
    """``x[..., row(16), unit, bytes]``: destination unit ``u`` takes source unit ``u ^ (row & mask)``."""
    dev = x.device
    nu = x.shape[-2]
    idx = torch.arange(nu, device=dev)[None, :] ^ (torch.arange(16, device=dev) & mask)[:, None]        # [16, nu]
    shape = [1] * (x.dim() - 3) + [16, nu, 1]
    return torch.gather(x, x.dim() - 2, idx.reshape(shape).expand_as(x))


def tile16_major(raw: torch.Tensor, qtype: GGMLType, b0: int, b1: int) -> torch.Tensor:
    """The tensor-pipe GEMV's layout over the 256-value blocks ``[b0, b1)`` of every row: rows padded with zeros to a
    multiple of 16, then ``[tile of 16 rows][block][row in tile][block bytes]`` (csrc/decode_gemv_mma.cuh):

    * Q4_K / Q5_K: the file's 144 / 176-byte blocks unchanged;
    * Q6_K: split into arrays (``ql[16][128] | qh[16][64] | scales[16][16] | d[16]``), the 16-byte chunks of a ``ql``
      row stored at ``chunk ^ (row & 7)``, those of a ``qh`` row at ``chunk ^ ((row >> 1) & 3)``;
    * Q8_0: eight file blocks per row and unit: ``q[16][256]`` with the 32-byte unit ``u`` of a row at ``u ^ (row & 7)``,
      then ``d[16][8]``;
    * F16: blocks of 64 values, ``[16][64]`` halves with the 32-byte unit ``u`` of a row at ``u ^ (row & 3)``.

    The swizzles put the eight rows one shared-memory load touches on distinct banks."""
    qtype = GGMLType(qtype)
    n = raw.shape[0]
    bb, per = _FILE_BLOCK[qtype]
    raw = raw.reshape(n, -1)
    blk = raw.reshape(n, -1, bb * (256 // per))[:, b0:b1]                  # [n, 256-value blocks, bytes]
    nb = blk.shape[1]
    n16 = (n + 15) // 16 * 16
    if n16 != n:
        blk = torch.cat([blk, torch.zeros(n16 - n, nb, blk.shape[2], dtype=torch.uint8, device=blk.device)])
    t = blk.reshape(n16 // 16, 16, nb, -1).permute(0, 2, 1, 3)             # [tile, block, row, bytes]
    if qtype in (GGMLType.Q4_K, GGMLType.Q5_K):
        return t.contiguous().reshape(-1)
    if qtype == GGMLType.Q8_0:
        f = t.reshape(-1, nb, 16, 8, 34)
        q = _swizzle_units(f[..., 2:34].contiguous(), 7)                  # [tile, block, 16, 8, 32]
        d = f[..., 0:2]
        return torch.cat([q.reshape(-1, nb, 16 * 256), d.reshape(-1, nb, 16 * 16)], dim=2).contiguous().reshape(-1)
    if qtype == GGMLType.F16:
        f = t.reshape(-1, nb, 16, 4, 4, 32).permute(0, 1, 3, 2, 4, 5)     # [tile, block, quarter(64 values), row, unit, 32 B]
        return _swizzle_units(f.contiguous(), 3).reshape(-1)
    ql = _swizzle_units(t[..., 0:128].reshape(-1, nb, 16, 8, 16), 7)
    # qh chunk key is (row >> 1) & 3
    dev = blk.device
    row = torch.arange(16, device=dev)
    qh = t[..., 128:192].reshape(-1, nb, 16, 4, 16)
    idx_h = (torch.arange(4, device=dev)[None, :] ^ ((row >> 1) & 3)[:, None])          # [16, 4]
    qh = torch.gather(qh, 3, idx_h[None, None, :, :, None].expand(qh.shape[0], nb, 16, 4, 16))
    parts = [ql.reshape(-1, nb, 16 * 128), qh.reshape(-1, nb, 16 * 64), t[..., 192:208].reshape(-1, nb, 16 * 16),
             t[..., 208:210].reshape(-1, nb, 16 * 2)]
    return torch.cat(parts, dim=2).contiguous().reshape(-1)


class PackedWeight:
    """A quantised matrix in the layout its kernel streams (``rowbytes`` > 0 only for row-major tables)."""

    def __init__(self, data: torch.Tensor, qtype: int, rows: int, cols: int, bias: Optional[torch.Tensor] = None,
                 rowbytes: int = 0, layout: int = LAYOUT_SEGMENT):
        self.data, self.qtype, self.rows, self.cols, self.bias, self.rowbytes = data, qtype, rows, cols, bias, rowbytes
        self.layout = layout
        assert data.data_ptr() % 16 == 0

    def desc(self) -> N.WeightDesc:
        return N.WeightDesc(self.data.data_ptr(), N.ptr(self.bias), self.qtype, self.rows, self.cols, self.rowbytes,
                            self.layout, 0)

    @property
    def nbytes(self) -> int:
        return self.data.numel()


def _to_kernel_type(raw: torch.Tensor, qtype: GGMLType, cols: int, layout: int = 0):
    """Bytes and type the kernels take.  The tile layout streams Q4_K, Q5_K, Q6_K, Q8_0 and F16 as they are (BF16 and
    F32 matrices become F16); anything else, and every type but Q4_K/Q6_K in the segment layout, is transcoded to Q6_K
    blocks (the only lossy step, and only for such files)."""
    qtype = GGMLType(qtype)
    if qtype in (GGMLType.Q4_K, GGMLType.Q6_K):
        return raw, qtype
    if layout == LAYOUT_T16:
        if qtype in (GGMLType.Q5_K, GGMLType.Q8_0, GGMLType.F16):
            return raw, qtype
        if qtype in (GGMLType.BF16, GGMLType.F32):
            w = dequantize(raw, qtype, cols).to(torch.float16).contiguous()
            return w.view(torch.uint8).reshape(w.shape[0], -1), GGMLType.F16
    raw = quantize(dequantize(raw, qtype, cols), GGMLType.Q6_K)
    return raw, GGMLType.Q6_K


def default_layout(tp_world: int = 1) -> int:
    """PTB_GEMV_LAYOUT (t16 / segment) if set.  Otherwise by measurement on the Qwen3-4B shape: one GPU streams tiles of
    16 rows through the tensor-pipe kernel (660 vs 629 tok/s); tensor-parallel ranks, whose matrices are a fraction of the
    size and whose steps are latency-bound, run the dp4a kernel's segment layout with two 8-warp CTAs per SM (758 vs 752
    tok/s at 2 GPUs, 840 vs 798 at 4)."""
    import os
    v = os.environ.get("PTB_GEMV_LAYOUT")
    if v is not None:
        return LAYOUT_SEGMENT if v == "segment" else LAYOUT_T16
    return LAYOUT_T16 if tp_world <= 1 else LAYOUT_SEGMENT


def pack_weight(raw: torch.Tensor, qtype: GGMLType, cols: int, device, rows=None, kblocks=None,
                bias: Optional[torch.Tensor] = None, layout: Optional[int] = None, tp_world: int = 1) -> PackedWeight:
    """``raw``: uint8 ``[N, row_bytes]`` as stored in the file -> GEMV streaming layout on ``device``.
    ``rows=(r0,r1)`` row-slices, ``kblocks=(b0,b1)`` slices super-blocks along K."""
    layout = default_layout(tp_world) if layout is None else layout
    if rows is not None:
        raw = raw[rows[0]:rows[1]]
    raw, qtype = _to_kernel_type(raw.to(device, non_blocking=True), qtype, cols, layout)
    b0, b1 = kblocks if kblocks is not None else (0, cols // 256)
    data = tile16_major(raw, qtype, b0, b1) if layout == LAYOUT_T16 else segment_major(raw, qtype, b0, b1)
    if bias is not None:
        bias = bias.to(device).float().contiguous()
        if rows is not None:
            bias = bias[rows[0]:rows[1]].contiguous()
    return PackedWeight(data, _KERNEL_TYPE[qtype], raw.shape[0], (b1 - b0) * 256, bias, layout=layout)


def pack_table(raw: torch.Tensor, qtype: GGMLType, cols: int, device) -> PackedWeight:
    """Row-major layout for row lookups (the embedding table): Q4_K rows as in the file, Q6_K rows as a structure of
    arrays, every other type as an fp16 table."""
    qtype = GGMLType(qtype)
    raw = raw.to(device, non_blocking=True)
    if qtype == GGMLType.Q4_K:
        data, qt = raw.contiguous(), QT_Q4K
    elif qtype == GGMLType.Q6_K:
        data, qt = repack_q6k(raw), QT_Q6K
    else:
        w = (raw.view(torch.float16) if qtype == GGMLType.F16 else dequantize(raw, qtype, cols).to(torch.float16)).contiguous()
        data, qt = w.view(torch.uint8).reshape(w.shape[0], -1), QT_F16
    return PackedWeight(data, qt, data.shape[0], cols, None, rowbytes=data.shape[1])


class GGUFModel:
    """Quantised decoder bound to the native decode engine on one GPU (or one TP rank)."""

    def __init__(self, path: str, device: Optional[str] = None, max_seq: int = 4096, tp_rank: int = 0,
                 tp_world: int = 1, symm=None, want_logits: bool = False):
        self.path = path
        self.reader = GGUFReader(path)
        self.cfg = TransformerConfig.from_gguf(self.reader)
        self.device = torch.device(device if device is not None else "cuda")
        if self.device.type != "cuda":
            raise RuntimeError("GGUFModel runs on a CUDA device; use models.gguf_oracle.OracleModel on the CPU")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.max_seq = int(min(max_seq, self.cfg.context_length))
        self.tp_rank, self.tp_world = tp_rank, tp_world
        self.symm = symm
        self.want_logits = want_logits
        self._engine = None
        self._keep: List[torch.Tensor] = []
        self.load_seconds = 0.0
        self.weight_bytes = 0
        self._load()

    # ------------------------------------------------------------------ loading
    @classmethod
    def load(cls, path: str, **kw) -> "GGUFModel":
        return cls(path, **kw)

    def _load(self):
        t0 = time.time()
        cfg, r, dev = self.cfg, self.reader, self.device
        W, rk = self.tp_world, self.tp_rank
        if cfg.num_heads % W or cfg.num_kv_heads % W or cfg.intermediate_size % 256:
            raise ValueError(f"tensor parallel {W}: needs heads ({cfg.num_heads}), KV heads ({cfg.num_kv_heads}) "
                             f"divisible and FFN size ({cfg.intermediate_size}) a multiple of 256")
        if (cfg.num_heads // W * cfg.head_dim) % 256:
            raise ValueError("tensor parallel: per-rank attention width must be a multiple of 256")
        if cfg.has_post_norm and cfg.hidden_size > 4096:
            raise NotImplementedError("post-attention/post-FFN norms are supported for hidden sizes up to 4096")
        torch.cuda.set_device(dev)
        hq, hkv, d = cfg.num_heads // W, cfg.num_kv_heads // W, cfg.head_dim
        fb0, fb1 = split_blocks(cfg.intermediate_size // 256, W, rk)
        ob0, ob1 = rk * hq * d // 256, (rk + 1) * hq * d // 256
        self.local_heads, self.local_kv_heads, self.local_inter = hq, hkv, (fb1 - fb0) * 256

        # one weight layout per model (the jobs of a launch share it): the world-size default, except that a file with
        # matrices the segment layout cannot stream natively (Q5_K, Q8_0, F16) stays on the tile layout
        import os
        self.layout = default_layout(W)
        if self.layout == LAYOUT_SEGMENT and os.environ.get("PTB_GEMV_LAYOUT") is None:
            kinds = {GGMLType(t.qtype) for n, t in r.tensors.items() if len(t.shape) == 2 and n.endswith(".weight") and "token_embd" not in n}
            if not kinds <= {GGMLType.Q4_K, GGMLType.Q6_K}:
                self.layout = LAYOUT_T16

        def mat(name, rows=None, kblocks=None, bias_name=None, base=None):
            """``base=(r0, r1)``: the matrix is rows r0..r1 of a merged tensor (phi-3 attn_qkv / gate+up); ``rows`` then
            counts from r0, and a bias comes from the merged tensor's bias."""
            ti = r.tensors[name]
            bias = r.load(bias_name) if bias_name and r.has_tensor(bias_name) else None
            if base is None:
                pw = pack_weight(r.raw(name), ti.qtype, ti.shape[-1], dev, rows, kblocks, bias, layout=self.layout)
            else:
                merged_bias = name[:-len("weight")] + "bias"
                if r.has_tensor(merged_bias):
                    bias = r.load(merged_bias)[base[0]:base[1]]
                lo, hi = rows if rows is not None else (0, base[1] - base[0])
                pw = pack_weight(r.raw(name), ti.qtype, ti.shape[-1], dev, (base[0] + lo, base[0] + hi), kblocks, None, layout=self.layout)
                if bias is not None:
                    pw.bias = bias[lo:hi].to(dev).float().contiguous()
            self.weight_bytes += pw.nbytes
            return pw

        def vec(name):
            if not r.has_tensor(name):
                return None
            t = r.load(name).to(dev).float().contiguous()
            self._keep.append(t)
            return t

        from ..models.gguf_oracle import rope_tables
        cos, sin = rope_tables(cfg, self.max_seq, "cpu")
        self.cos, self.sin = cos.to(dev).contiguous(), sin.to(dev).contiguous()
        self.cos_swa = self.sin_swa = None
        if cfg.swa_window and cfg.rope_swa_freq_base != cfg.rope_freq_base:
            c2, s2 = rope_tables(cfg, self.max_seq, "cpu", freq_base=cfg.rope_swa_freq_base)
            self.cos_swa, self.sin_swa = c2.to(dev).contiguous(), s2.to(dev).contiguous()

        self.layers = []
        descs = (N.LayerDesc * cfg.num_layers)()
        for i in range(cfg.num_layers):
            p = f"blk.{i}."
            src = layer_matrix_sources(r, cfg, i)           # separate tensors, or row ranges of merged qkv / gate+up
            L = dict(
                q=mat(src["q"][0], rows=(rk * hq * d, (rk + 1) * hq * d), bias_name=p + "attn_q.bias", base=src["q"][1]),
                k=mat(src["k"][0], rows=(rk * hkv * d, (rk + 1) * hkv * d), bias_name=p + "attn_k.bias", base=src["k"][1]),
                v=mat(src["v"][0], rows=(rk * hkv * d, (rk + 1) * hkv * d), bias_name=p + "attn_v.bias", base=src["v"][1]),
                o=mat(src["o"][0], kblocks=(ob0, ob1)),
                gate=mat(src["gate"][0], rows=(fb0 * 256, fb1 * 256), base=src["gate"][1]),
                up=mat(src["up"][0], rows=(fb0 * 256, fb1 * 256), base=src["up"][1]),
                down=mat(src["down"][0], kblocks=(fb0, fb1)),
                attn_norm=vec(p + "attn_norm.weight"), ffn_norm=vec(p + "ffn_norm.weight"),
                q_norm=vec(p + "attn_q_norm.weight"), k_norm=vec(p + "attn_k_norm.weight"),
                post_attn_norm=vec(p + "post_attention_norm.weight"), post_ffn_norm=vec(p + "post_ffw_norm.weight"))
            if L["gate"].qtype != L["up"].qtype:
                raise NotImplementedError("ffn_gate and ffn_up with different quantisation types")
            swa = bool(cfg.swa_window and cfg.swa_pattern and (i + 1) % cfg.swa_pattern != 0)
            self.layers.append(L)
            dsc = descs[i]
            for k in ("q", "k", "v", "o", "gate", "up", "down"):
                setattr(dsc, k, L[k].desc())
            dsc.attn_norm, dsc.ffn_norm = N.ptr(L["attn_norm"]), N.ptr(L["ffn_norm"])
            dsc.q_norm, dsc.k_norm = N.ptr(L["q_norm"]), N.ptr(L["k_norm"])
            dsc.post_attn_norm, dsc.post_ffn_norm = N.ptr(L["post_attn_norm"]), N.ptr(L["post_ffn_norm"])
            use_swa_tab = swa and self.cos_swa is not None
            dsc.cos = (self.cos_swa if use_swa_tab else self.cos).data_ptr()
            dsc.sin = (self.sin_swa if use_swa_tab else self.sin).data_ptr()
            dsc.window = cfg.swa_window if swa else 0
        self._layer_descs = descs
        te = r.tensors["token_embd.weight"]
        self.embed = pack_table(r.raw("token_embd.weight"), te.qtype, te.shape[-1], dev)
        self.table_bytes = self.embed.nbytes
        head_name = "output.weight" if r.has_tensor("output.weight") else "token_embd.weight"
        V = cfg.vocab_size
        v0, v1 = (V * rk) // W, (V * (rk + 1)) // W
        self.lm_head = mat(head_name, rows=(v0, v1))
        self.vocab_offset = v0
        self.out_norm = vec("output_norm.weight")

        m = N.ModelDesc()
        m.n_layers, m.hidden, m.n_heads, m.n_kv_heads = cfg.num_layers, cfg.hidden_size, hq, hkv
        m.head_dim, m.inter, m.vocab, m.max_seq = d, self.local_inter, V, self.max_seq
        m.eps = cfg.rms_norm_eps
        m.emb_scale = math.sqrt(cfg.hidden_size) if cfg.scale_embeddings else 1.0
        m.neox, m.act_gelu, m.norm_add_one = int(cfg.rope_neox), int(cfg.ffn_gelu), int(cfg.gemma_norm_add_one)
        m.want_logits = int(self.want_logits)
        m.embed, m.lm_head, m.out_norm = self.embed.desc(), self.lm_head.desc(), N.ptr(self.out_norm)
        m.tp_rank, m.tp_world, m.vocab_offset = rk, W, v0
        if W > 1:
            if self.symm is None:
                raise ValueError("tensor parallel decode needs a symmetric-memory group (parallel.symm.SymmGroup)")
            slot = max(cfg.hidden_size, 64)
            # three inboxes of {payload, sequence} slots: attention output, FFN down, lm_head arg-max
            self._tp_bufs = [self.symm.alloc(W * slot * 8) for _ in range(3)]
            for b in range(3):
                for p in range(W):
                    m.peer_inbox[b][p] = self._tp_bufs[b].peer_ptr(p)
            m.slot_elems = slot
            self.symm.barrier()
        self._model_desc = m
        torch.cuda.synchronize(dev)
        lib = N.lib()
        self._engine = lib.ptb_engine_create(C.byref(m), descs, None)
        if not self._engine:
            raise N.NativeError("engine: " + lib.ptb_last_error().decode())
        self._lib = lib
        self._captured = False
        self.load_seconds = time.time() - t0

    def close(self):
        if self._engine:
            self._lib.ptb_engine_destroy(self._engine)
            self._engine = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ engine access
    def capture(self):
        """Capture the per-token CUDA graph (one warm-up token runs eagerly first)."""
        if self._captured:
            return
        N.check(self._lib.ptb_engine_set_ctrl(self._engine, 0, 0, 0, 1), "set_ctrl")
        N.check(self._lib.ptb_engine_run(self._engine, 1), "warm-up token")
        N.check(self._lib.ptb_engine_sync(self._engine), "sync")
        self.check_status()
        N.check(self._lib.ptb_engine_capture(self._engine), "graph capture")
        self._captured = True

    def check_status(self):
        s = self._lib.ptb_engine_status(self._engine)
        if s != 0:
            names = {1: "a weight copy never completed (mbarrier timeout)", 2: "a peer GPU never published its flag",
                     3: "a token id fell outside the vocabulary"}
            raise N.NativeError(f"decode kernels reported status {s}: {names.get(s, 'unknown')}")

    @property
    def stream(self) -> torch.cuda.Stream:
        return torch.cuda.ExternalStream(self._lib.ptb_engine_stream(self._engine), device=self.device)

    @property
    def launches_per_token(self) -> int:
        return int(self._lib.ptb_engine_launches_per_token(self._engine))

    def _wrap(self, addr: int, n: int, dtype=torch.float32) -> torch.Tensor:
        class _Arr:
            pass
        a = _Arr()
        typestr = {torch.float32: "<f4", torch.float16: "<f2", torch.int32: "<i4"}[dtype]
        a.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (addr, False), "version": 3}
        return torch.as_tensor(a, device=self.device)

    def logits_view(self) -> torch.Tensor:
        """Device view of this rank's logits rows (valid when ``want_logits``)."""
        return self._wrap(self._lib.ptb_engine_logits(self._engine), self.lm_head.rows)

    def hidden_view(self) -> torch.Tensor:
        return self._wrap(self._lib.ptb_engine_hidden(self._engine), self.cfg.hidden_size)

    # ------------------------------------------------------------------ decoding
    def forward_decode(self, token: int, pos: int) -> int:
        """Serving step: token and position go host→device from pinned memory, one graph replay,
        the arg-max id comes back device→host.  Returns the greedy next token."""
        self.capture()
        t = self._lib.ptb_engine_step(self._engine, int(token), int(pos))
        if t < 0:
            raise N.NativeError("decode step: " + self._lib.ptb_last_error().decode())
        return t

    # ------------------------------------------------------------------ low-rank speculative output projection
    def lowrank_head(self, rank: int = 256, candidate_k: int = 64):
        """Build the low-rank approximation of the output projection (io/speculative.py) from the file's quantised rows.
        ``next_token_lowrank()`` then picks the next token from the engine's final hidden state with ``rank`` instead of
        ``hidden`` multiply-adds per vocabulary row plus ``candidate_k`` exact rows."""
        from .speculative import LowRankOutputProj
        if self.tp_world != 1:
            raise NotImplementedError("low-rank output projection: one GPU")
        name = "output.weight" if self.reader.has_tensor("output.weight") else "token_embd.weight"
        ti = self.reader.tensors[name]
        self._lowrank = LowRankOutputProj(rank, candidate_k, dtype=torch.bfloat16).init_from_quantized(
            self.reader.raw(name), ti.qtype, ti.shape[-1], device=self.device)
        return self._lowrank

    def next_token_lowrank(self) -> int:
        """Arg-max over the vocabulary through the low-rank projection, from the hidden state of the last decode step."""
        x = self.hidden_view().float()
        w = (self.out_norm + 1.0) if self.cfg.gemma_norm_add_one else self.out_norm
        x = x * torch.rsqrt(x.pow(2).mean() + self.cfg.rms_norm_eps) * w
        return self._lowrank.decode_greedy(x)

    # ------------------------------------------------------------------ batched prompt pass
    @property
    def supports_prefill(self) -> bool:
        """The batched prompt pass covers full attention (no sliding window) with head size 64 or 128, on one GPU or,
        under tensor parallelism, on every rank over its own heads and FFN columns with two all-reduces per layer."""
        return not self.cfg.swa_window and self.cfg.head_dim in (64, 128)

    def _dequant(self, pw: "PackedWeight") -> torch.Tensor:
        """bf16 ``[rows, cols]`` copy of a packed matrix in a scratch buffer shared by all matrices of that shape."""
        key = (pw.rows, pw.cols)
        buf = self._dq_scratch.get(key)
        if buf is None:
            buf = self._dq_scratch[key] = torch.empty(pw.rows, pw.cols, dtype=torch.bfloat16, device=self.device)
        st = torch.cuda.current_stream(self.device).cuda_stream
        N.check(self._lib.ptb_dequant_weight(pw.data.data_ptr(), pw.qtype, pw.layout, pw.rows, pw.cols, buf.data_ptr(), st), "dequant")
        return buf

    def _kv_views(self, layer: int):
        k, v = C.c_void_p(), C.c_void_p()
        N.check(self._lib.ptb_engine_kv_cache(self._engine, layer, C.byref(k), C.byref(v)), "kv_cache")
        n = self.local_kv_heads * self.max_seq * self.cfg.head_dim
        shape = (self.local_kv_heads, self.max_seq, self.cfg.head_dim)
        return self._wrap(k.value, n, torch.float16).view(shape), self._wrap(v.value, n, torch.float16).view(shape)

    @torch.no_grad()
    def prefill(self, tokens: Sequence[int], pos0: int = 0, return_logits: bool = False):
        """Run ``tokens`` at positions ``pos0 ..`` through the model in ONE batched pass that fills the KV cache:
        weights are dequantised to bf16 layer by layer and every projection is a tcgen05 GEMM over all prompt
        tokens, attention is the FlashAttention kernel.  Nothing is returned; decoding continues with
        ``forward_decode(next_token, pos0 + len(tokens))``.  (Token-by-token prefill costs one decode step each.)
        Under tensor parallelism the call is collective: every rank runs it with the same tokens.
        ``return_logits=True`` also applies the output norm and the lm_head to every position and returns fp32 logits
        ``[T, vocab rows of this rank]`` (what a speculative verifier needs)."""
        if not self.supports_prefill:
            raise NotImplementedError("batched prefill: no sliding window, head size 64 or 128")
        from ..ops import fused_ops as K
        from ..ops.attention import flash_attention
        from ..ops.gemm import linear
        cfg, dev = self.cfg, self.device
        T = len(tokens)
        if T == 0:
            return None
        if pos0 + T > self.max_seq:
            raise ValueError(f"prompt of {T} tokens at {pos0} exceeds max_seq {self.max_seq}")
        self.capture()
        N.check(self._lib.ptb_engine_sync(self._engine), "sync")
        if not hasattr(self, "_dq_scratch"):
            self._dq_scratch, self._pf_status = {}, torch.zeros(1, dtype=torch.int32, device=dev)
        H, d, hq, hkv = cfg.hidden_size, cfg.head_dim, self.local_heads, self.local_kv_heads
        eps, bf = cfg.rms_norm_eps, torch.bfloat16
        st = torch.cuda.current_stream(dev).cuda_stream
        ids = torch.as_tensor(list(int(t) for t in tokens), dtype=torch.int32, device=dev)
        x = torch.empty(T, H, dtype=bf, device=dev)
        e = self.embed
        N.check(self._lib.ptb_dequant_rows(e.data.data_ptr(), e.qtype, e.rowbytes, H, ids.data_ptr(), T, float(self._model_desc.emb_scale),
                                           e.rows, self._pf_status.data_ptr(), x.data_ptr(), st), "dequant_rows")

        def nw(L, name):          # bf16 norm weight (gemma stores w - 1)
            key = name + "_bf16"
            if key not in L:
                w = L[name]
                L[key] = None if w is None else ((w + 1.0) if cfg.gemma_norm_add_one else w).to(bf)
            return L[key]

        def proj(h, pw):
            y = linear(h, self._dequant(pw), None)
            return y if pw.bias is None else y + pw.bias.to(bf)

        def ksplit(h, pw):
            """A projection split along K over the ranks (attention output, FFN down): every rank multiplies its own
            columns and the partial results are summed in fp32 across the ranks (collective: all ranks prefill together)."""
            y = proj(h, pw)
            if self.tp_world > 1:
                y32 = y.float()
                self.symm.dist.all_reduce(y32, group=self.symm.pg)
                y = y32.to(bf)
            return y

        for i, L in enumerate(self.layers):
            h = K.rms_norm(x, nw(L, "attn_norm"), eps)
            q = proj(h, L["q"]).view(T, hq, d)
            k = proj(h, L["k"]).view(T, hkv, d)
            v = proj(h, L["v"]).view(T, hkv, d)
            if L["q_norm"] is not None:
                q = K.rms_norm(q.reshape(-1, d), nw(L, "q_norm"), eps).view(T, hq, d)
                k = K.rms_norm(k.reshape(-1, d), nw(L, "k_norm"), eps).view(T, hkv, d)
            q = K.rope(q.unsqueeze(0), self.cos, self.sin, bool(cfg.rope_neox), pos0)
            k = K.rope(k.unsqueeze(0), self.cos, self.sin, bool(cfg.rope_neox), pos0)
            kc, vc = self._kv_views(i)
            kc[:, pos0:pos0 + T] = k[0].permute(1, 0, 2).to(torch.float16)
            vc[:, pos0:pos0 + T] = v.permute(1, 0, 2).to(torch.float16)
            if pos0 > 0:          # earlier positions come from the cache
                k_all = kc[:, :pos0 + T].permute(1, 0, 2).to(bf).unsqueeze(0).contiguous()
                v_all = vc[:, :pos0 + T].permute(1, 0, 2).to(bf).unsqueeze(0).contiguous()
            else:
                k_all, v_all = k, v.unsqueeze(0)
            att = flash_attention(q, k_all, v_all, causal=True, q_offset=pos0).reshape(T, hq * d)
            o = ksplit(att, L["o"])
            if L["post_attn_norm"] is not None:
                o = K.rms_norm(o, nw(L, "post_attn_norm"), eps)
            x = x + o
            h = K.rms_norm(x, nw(L, "ffn_norm"), eps)
            g, u = proj(h, L["gate"]), proj(h, L["up"]).clone()       # gate and up share a scratch shape: keep one
            act = torch.nn.functional.gelu(g.float(), approximate="tanh") if cfg.ffn_gelu else torch.nn.functional.silu(g.float())
            dn = ksplit((act * u.float()).to(bf), L["down"])
            if L["post_ffn_norm"] is not None:
                dn = K.rms_norm(dn, nw(L, "post_ffn_norm"), eps)
            x = x + dn
        logits = None
        if return_logits:
            if not hasattr(self, "_out_norm_bf16"):
                w = self.out_norm
                self._out_norm_bf16 = ((w + 1.0) if cfg.gemma_norm_add_one else w).to(bf)
            logits = linear(K.rms_norm(x, self._out_norm_bf16, eps), self._dequant(self.lm_head), None).float()
        torch.cuda.current_stream(dev).synchronize()
        if int(self._pf_status):
            self._pf_status.zero_()
            raise N.NativeError("prefill: a token id fell outside the vocabulary")
        return logits

    def run_script(self, prompt: Sequence[int], n_new: int, pos0: int = 0, sync: bool = True) -> Optional[List[int]]:
        """Enqueue prompt + ``n_new`` greedy tokens as back-to-back graph replays with the
        sampled token fed back on the device; no host round trip until the end."""
        self.capture()
        n = len(prompt)
        if pos0 + n + n_new > self.max_seq:
            raise ValueError(f"{pos0 + n + n_new} positions exceed max_seq {self.max_seq}")
        arr = (C.c_int * n)(*[int(t) for t in prompt])
        N.check(self._lib.ptb_engine_begin_script(self._engine, arr, n, pos0), "begin_script")
        N.check(self._lib.ptb_engine_run(self._engine, n + n_new - 1), "run")
        if not sync:
            return None
        return self.read_generated(n, n_new)

    def read_generated(self, n_prompt: int, n_new: int) -> List[int]:
        total = n_prompt + n_new - 1
        buf = (C.c_int * total)()
        steps = self._lib.ptb_engine_read_log(self._engine, buf, total)
        self.check_status()
        if steps < total:
            raise N.NativeError(f"only {steps} of {total} decode steps ran")
        return list(buf[n_prompt - 1:total])

    def generate(self, prompt: Sequence[int], max_new_tokens: int = 128, temperature: float = 0.0, top_k: int = 40,
                 top_p: float = 0.9, repeat_penalty: float = 1.0, stop_ids: Iterable[int] = (),
                 on_token: Optional[Callable[[int], bool]] = None, seed: int = 42, _pos0: Optional[int] = None,
                 _history: Optional[Sequence[int]] = None) -> List[int]:
        """Token-level generation.  Greedy without a callback runs entirely on the device; with a
        callback (streaming) or sampling it steps token by token."""
        stop = set(int(s) for s in stop_ids)
        if self.cfg.eos_token_id >= 0:
            stop.add(self.cfg.eos_token_id)
        greedy = temperature <= 0.0 and repeat_penalty == 1.0
        if greedy and on_token is None and not stop and _pos0 is None:
            if self.supports_prefill and len(prompt) - 1 >= 8:
                self.prefill(prompt[:-1])
                return self.run_script(prompt[-1:], max_new_tokens, pos0=len(prompt) - 1)
            return self.run_script(prompt, max_new_tokens)
        if not greedy and not self.want_logits:
            raise RuntimeError("sampling needs the model opened with want_logits=True")
        # prompt (all but the last token) in one scripted run, then step
        out: List[int] = []
        n = len(prompt)
        if _pos0 is not None:                   # the caller already ran the prompt up to position _pos0
            tok, pos = int(prompt[-1]), int(_pos0)
        else:
            if n > 1:
                if self.supports_prefill and n - 1 >= 8:
                    self.prefill(prompt[:-1])                  # one batched pass over the prompt
                else:
                    self.run_script(prompt[:-1], 1)
            tok, pos = int(prompt[-1]), n - 1
        from ..ops.sampling import MAX_DEVICE_TOP_K, DeviceSampler, sample_logits
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        history = list(int(t) for t in (_history if _history is not None else prompt))
        # top-k up to 64: the whole sampler is one kernel on the device (only the chosen id comes back);
        # wider or unbounded top-k goes through tensor ops
        sampler = None
        if not greedy and 1 <= top_k <= MAX_DEVICE_TOP_K:
            sampler = DeviceSampler(self.logits_view().numel(), self.device, seed=seed)
            sampler.reset(history)
        for _ in range(max_new_tokens):
            nxt = self.forward_decode(tok, pos)
            if sampler is not None:
                nxt = sampler.sample(self.logits_view(), temperature, top_k, top_p, repeat_penalty)
            elif not greedy:
                nxt = sample_logits(self.logits_view(), temperature, top_k, top_p, repeat_penalty, history, gen)
            out.append(nxt)
            history.append(nxt)
            if on_token is not None and on_token(nxt) is False:
                break
            if nxt in stop:
                break
            tok, pos = nxt, pos + 1
            if pos + 1 >= self.max_seq:
                break
        return out
