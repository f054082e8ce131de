"""GGML block quantisation formats as vectorised tensor programs.

Every routine here is written with plain ``torch`` ops so the same code runs on
the CPU (unit tests, small models) and on a GPU (quantising a 4 B-parameter
synthetic model in well under a second).  These are the *oracle* semantics for
the CUDA dequant-GEMV kernels: a kernel test dequantises the same bytes with
``dequantize`` and compares against an fp32 matmul.

Formats (bit layouts follow the public GGML definitions; the reference restates
them in torch/io/gguf_dequant.h:119-176, 289-341, 391-430):

* ``Q4_K``  256 values / 144 B: fp16 d, fp16 dmin, 12 B packed 6-bit
  (scale, min) pairs for 8 sub-blocks of 32, 128 B of 4-bit quants.
* ``Q5_K``  256 values / 176 B: as Q4_K plus 32 B of fifth bits.
* ``Q6_K``  256 values / 210 B: 128 B low nibbles, 64 B high 2-bit pairs,
  16 int8 scales (one per 16 values), fp16 d.
* ``Q8_0``  32 values / 34 B: fp16 d, 32 int8.
* ``Q4_0``  32 values / 18 B: fp16 d, 16 B nibbles (value - 8).
* ``F32``, ``F16``, ``BF16`` pass through.
"""
from __future__ import annotations

import enum
from typing import Tuple

import torch

QK_K = 256


class GGMLType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    Q8_K = 15
    I8 = 24
    I16 = 25
    I32 = 26
    I64 = 27
    F64 = 28
    BF16 = 30


# (values per block, bytes per block)
BLOCK_INFO = {
    GGMLType.F32: (1, 4),
    GGMLType.F16: (1, 2),
    GGMLType.BF16: (1, 2),
    GGMLType.Q4_0: (32, 18),
    GGMLType.Q4_1: (32, 20),
    GGMLType.Q5_0: (32, 22),
    GGMLType.Q5_1: (32, 24),
    GGMLType.Q8_0: (32, 34),
    GGMLType.Q8_1: (32, 36),
    GGMLType.Q2_K: (256, 84),
    GGMLType.Q3_K: (256, 110),
    GGMLType.Q4_K: (256, 144),
    GGMLType.Q5_K: (256, 176),
    GGMLType.Q6_K: (256, 210),
    GGMLType.Q8_K: (256, 292),
    GGMLType.I8: (1, 1),
    GGMLType.I16: (1, 2),
    GGMLType.I32: (1, 4),
    GGMLType.I64: (1, 8),
    GGMLType.F64: (1, 8),
}


def row_bytes(qtype: GGMLType, cols: int) -> int:
    """Bytes of one row of ``cols`` values stored as ``qtype``."""
    per, nbytes = BLOCK_INFO[GGMLType(qtype)]
    if cols % per:
        raise ValueError(f"{GGMLType(qtype).name}: row length {cols} is not a multiple of {per}")
    return cols // per * nbytes


def tensor_bytes(qtype: GGMLType, shape) -> int:
    n = 1
    for s in shape[:-1]:
        n *= int(s)
    return n * row_bytes(qtype, int(shape[-1]))


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    """fp32 [...]-> uint8 [..., 2] holding the little-endian fp16 encoding."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def _bytes_f16(b: torch.Tensor) -> torch.Tensor:
    """uint8 [..., 2] -> fp32 [...]"""
    return b.contiguous().view(torch.float16).reshape(b.shape[:-1]).float()


# --------------------------------------------------------------------------- Q4_K / Q5_K scale packing


def _pack_scales_k4(sc: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    """Pack eight 6-bit scales and eight 6-bit mins into 12 bytes.

    Bytes 0-3 carry scale j (low 6 bits) with the top two bits of scale j+4,
    bytes 4-7 the same for mins, bytes 8-11 the low nibbles of scale/min j+4.
    """
    sc = sc.to(torch.int32)
    mn = mn.to(torch.int32)
    out = torch.empty(sc.shape[0], 12, dtype=torch.int32, device=sc.device)
    out[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 4:8] = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:8] & 0xF) | ((mn[:, 4:8] & 0xF) << 4)
    return out.to(torch.uint8)


def _unpack_scales_k4(q: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    q = q.to(torch.int32)
    sc = torch.empty(q.shape[0], 8, dtype=torch.int32, device=q.device)
    mn = torch.empty_like(sc)
    sc[:, 0:4] = q[:, 0:4] & 63
    mn[:, 0:4] = q[:, 4:8] & 63
    sc[:, 4:8] = (q[:, 8:12] & 0xF) | ((q[:, 0:4] >> 6) << 4)
    mn[:, 4:8] = (q[:, 8:12] >> 4) | ((q[:, 4:8] >> 6) << 4)
    return sc, mn


def _k4_scales(x: torch.Tensor, levels: int):
    """Shared affine fit for Q4_K/Q5_K: per 32-value sub-block scale and min,
    then a 6-bit quantisation of those against a per-256 super-scale."""
    nb = x.shape[0]
    sub = x.reshape(nb, 8, 32)
    mx = sub.amax(dim=2)
    mi = sub.amin(dim=2).clamp(max=0.0)          # stored min is -min >= 0
    scale = (mx - mi) / levels
    minv = -mi
    d = scale.amax(dim=1) / 63.0
    dmin = minv.amax(dim=1) / 63.0
    d = d.to(torch.float16).float()
    dmin = dmin.to(torch.float16).float()
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    inv_dmin = torch.where(dmin > 0, 1.0 / dmin, torch.zeros_like(dmin))
    sc = torch.round(scale * inv_d[:, None]).clamp(0, 63)
    mn = torch.round(minv * inv_dmin[:, None]).clamp(0, 63)
    eff_scale = d[:, None] * sc
    eff_min = dmin[:, None] * mn
    inv = torch.where(eff_scale > 0, 1.0 / eff_scale, torch.zeros_like(eff_scale))
    q = torch.round((sub + eff_min[:, :, None]) * inv[:, :, None]).clamp(0, levels)
    return d, dmin, sc, mn, q.to(torch.int32)


def quantize_q4_k(x: torch.Tensor) -> torch.Tensor:
    """fp32 [..., K] (K % 256 == 0) -> uint8 [..., K/256*144]."""
    lead, k = x.shape[:-1], x.shape[-1]
    xb = x.float().reshape(-1, QK_K)
    d, dmin, sc, mn, q = _k4_scales(xb, 15)
    nb = xb.shape[0]
    out = torch.empty(nb, 144, dtype=torch.uint8, device=x.device)
    out[:, 0:2] = _f16_bytes(d)
    out[:, 2:4] = _f16_bytes(dmin)
    out[:, 4:16] = _pack_scales_k4(sc, mn)
    # chunk j of 32 bytes: low nibble = sub-block 2j, high nibble = sub-block 2j+1
    q = q.reshape(nb, 4, 2, 32)
    out[:, 16:144] = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).to(torch.uint8).reshape(nb, 128)
    return out.reshape(*lead, k // QK_K * 144)


def dequantize_q4_k(b: torch.Tensor, k: int) -> torch.Tensor:
    lead = b.shape[:-1]
    blk = b.reshape(-1, 144)
    nb = blk.shape[0]
    d = _bytes_f16(blk[:, 0:2])
    dmin = _bytes_f16(blk[:, 2:4])
    sc, mn = _unpack_scales_k4(blk[:, 4:16])
    qs = blk[:, 16:144].to(torch.int32).reshape(nb, 4, 32)
    q = torch.stack([qs & 0xF, qs >> 4], dim=2).reshape(nb, 8, 32).float()
    y = (d[:, None] * sc.float())[:, :, None] * q - (dmin[:, None] * mn.float())[:, :, None]
    return y.reshape(*lead, k)


def quantize_q5_k(x: torch.Tensor) -> torch.Tensor:
    lead, k = x.shape[:-1], x.shape[-1]
    xb = x.float().reshape(-1, QK_K)
    d, dmin, sc, mn, q = _k4_scales(xb, 31)
    nb = xb.shape[0]
    out = torch.empty(nb, 176, dtype=torch.uint8, device=x.device)
    out[:, 0:2] = _f16_bytes(d)
    out[:, 2:4] = _f16_bytes(dmin)
    out[:, 4:16] = _pack_scales_k4(sc, mn)
    q = q.reshape(nb, 4, 2, 32)
    lo, hi = q & 0xF, q >> 4                       # hi is the fifth bit (0/1)
    out[:, 48:176] = (lo[:, :, 0, :] | (lo[:, :, 1, :] << 4)).to(torch.uint8).reshape(nb, 128)
    # qh[l] bit (2j) = fifth bit of sub-block 2j value l, bit (2j+1) = sub-block 2j+1
    shifts = torch.arange(8, device=x.device, dtype=torch.int32).reshape(1, 4, 2, 1)
    out[:, 16:48] = (hi << shifts).sum(dim=(1, 2)).to(torch.uint8)
    return out.reshape(*lead, k // QK_K * 176)


def dequantize_q5_k(b: torch.Tensor, k: int) -> torch.Tensor:
    lead = b.shape[:-1]
    blk = b.reshape(-1, 176)
    nb = blk.shape[0]
    d = _bytes_f16(blk[:, 0:2])
    dmin = _bytes_f16(blk[:, 2:4])
    sc, mn = _unpack_scales_k4(blk[:, 4:16])
    qh = blk[:, 16:48].to(torch.int32)
    qs = blk[:, 48:176].to(torch.int32).reshape(nb, 4, 32)
    lo = torch.stack([qs & 0xF, qs >> 4], dim=2).reshape(nb, 8, 32)
    shifts = torch.arange(8, device=b.device, dtype=torch.int32).reshape(1, 8, 1)
    hi = (qh[:, None, :] >> shifts) & 1
    q = (lo | (hi << 4)).float()
    y = (d[:, None] * sc.float())[:, :, None] * q - (dmin[:, None] * mn.float())[:, :, None]
    return y.reshape(*lead, k)


# --------------------------------------------------------------------------- Q6_K


def quantize_q6_k(x: torch.Tensor) -> torch.Tensor:
    """fp32 [..., K] -> uint8 [..., K/256*210].  Symmetric: value = d*scale16*(q-32)."""
    lead, k = x.shape[:-1], x.shape[-1]
    xb = x.float().reshape(-1, QK_K)
    nb = xb.shape[0]
    sub = xb.reshape(nb, 16, 16)
    amax = sub.abs().amax(dim=2)
    # signed 6-bit range is [-32, 31]; fit |x| to 31 so both signs are representable
    scale = amax / 31.0
    d = (scale.amax(dim=1) / 127.0).to(torch.float16).float()
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    sc = torch.round(scale * inv_d[:, None]).clamp(0, 127)
    eff = d[:, None] * sc
    inv = torch.where(eff > 0, 1.0 / eff, torch.zeros_like(eff))
    q = (torch.round(sub * inv[:, :, None]).clamp(-32, 31) + 32).to(torch.int32).reshape(nb, 2, 4, 32)
    lo, hi = q & 0xF, q >> 4
    out = torch.empty(nb, 210, dtype=torch.uint8, device=x.device)
    # per 128-value half n: ql[n*64 + l] = lo(l) | lo(l+64) << 4 ; ql[n*64+32+l] = lo(l+32) | lo(l+96) << 4
    ql = torch.stack([lo[:, :, 0] | (lo[:, :, 2] << 4), lo[:, :, 1] | (lo[:, :, 3] << 4)], dim=2)
    out[:, 0:128] = ql.reshape(nb, 128).to(torch.uint8)
    qh = hi[:, :, 0] | (hi[:, :, 1] << 2) | (hi[:, :, 2] << 4) | (hi[:, :, 3] << 6)
    out[:, 128:192] = qh.reshape(nb, 64).to(torch.uint8)
    out[:, 192:208] = sc.to(torch.int8).view(torch.uint8)
    out[:, 208:210] = _f16_bytes(d)
    return out.reshape(*lead, k // QK_K * 210)


def dequantize_q6_k(b: torch.Tensor, k: int) -> torch.Tensor:
    lead = b.shape[:-1]
    blk = b.reshape(-1, 210)
    nb = blk.shape[0]
    ql = blk[:, 0:128].to(torch.int32).reshape(nb, 2, 2, 32)
    qh = blk[:, 128:192].to(torch.int32).reshape(nb, 2, 32)
    sc = blk[:, 192:208].contiguous().view(torch.int8).float()
    d = _bytes_f16(blk[:, 208:210])
    lo = torch.stack([ql[:, :, 0] & 0xF, ql[:, :, 1] & 0xF, ql[:, :, 0] >> 4, ql[:, :, 1] >> 4], dim=2)
    hi = torch.stack([(qh >> 0) & 3, (qh >> 2) & 3, (qh >> 4) & 3, (qh >> 6) & 3], dim=2)
    q = ((lo | (hi << 4)) - 32).float().reshape(nb, 16, 16)
    y = (d[:, None] * sc)[:, :, None] * q
    return y.reshape(*lead, k)


# --------------------------------------------------------------------------- Q8_0 / Q4_0


def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    lead, k = x.shape[:-1], x.shape[-1]
    xb = x.float().reshape(-1, 32)
    d = (xb.abs().amax(dim=1) / 127.0).to(torch.float16).float()
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(xb * inv[:, None]).clamp(-127, 127).to(torch.int8)
    out = torch.empty(xb.shape[0], 34, dtype=torch.uint8, device=x.device)
    out[:, 0:2] = _f16_bytes(d)
    out[:, 2:34] = q.view(torch.uint8)
    return out.reshape(*lead, k // 32 * 34)


def dequantize_q8_0(b: torch.Tensor, k: int) -> torch.Tensor:
    lead = b.shape[:-1]
    blk = b.reshape(-1, 34)
    d = _bytes_f16(blk[:, 0:2])
    q = blk[:, 2:34].contiguous().view(torch.int8).float()
    return (d[:, None] * q).reshape(*lead, k)


def quantize_q4_0(x: torch.Tensor) -> torch.Tensor:
    lead, k = x.shape[:-1], x.shape[-1]
    xb = x.float().reshape(-1, 32)
    idx = xb.abs().argmax(dim=1, keepdim=True)
    mx = xb.gather(1, idx).squeeze(1)
    d = (mx / -8.0).to(torch.float16).float()
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = (torch.round(xb * inv[:, None]) + 8).clamp(0, 15).to(torch.int32)
    out = torch.empty(xb.shape[0], 18, dtype=torch.uint8, device=x.device)
    out[:, 0:2] = _f16_bytes(d)
    out[:, 2:18] = (q[:, 0:16] | (q[:, 16:32] << 4)).to(torch.uint8)
    return out.reshape(*lead, k // 32 * 18)


def dequantize_q4_0(b: torch.Tensor, k: int) -> torch.Tensor:
    lead = b.shape[:-1]
    blk = b.reshape(-1, 18)
    d = _bytes_f16(blk[:, 0:2])
    qs = blk[:, 2:18].to(torch.int32)
    q = torch.cat([qs & 0xF, qs >> 4], dim=1).float() - 8.0
    return (d[:, None] * q).reshape(*lead, k)


def dequantize_q2_k(b: torch.Tensor, k: int) -> torch.Tensor:
    """Q2_K: 84 bytes per 256 values = scales[16] (low nibble: scale, high nibble: min, per 16 values) | qs[64]
    (2-bit values) | fp16 d | fp16 dmin.  Value order as ggml stores it: each 128-value half uses 32 bytes of ``qs``;
    within a half, the four 2-bit planes (shift 0, 2, 4, 6) give 32 values each.  The reference's own routine
    (torch/io/gguf_dequant.h:437-468) walks the bits byte by byte instead, which does not match files written by
    ggml; this one does."""
    lead = b.shape[:-1]
    blk = b.reshape(-1, 84)
    sc = blk[:, 0:16].to(torch.int32)
    qs = blk[:, 16:80].to(torch.int32).reshape(-1, 2, 32)                      # [blocks, half, byte]
    d, dmin = _bytes_f16(blk[:, 80:82]), _bytes_f16(blk[:, 82:84])
    shifts = torch.tensor([0, 2, 4, 6], device=b.device, dtype=torch.int32)
    q = (qs[:, :, None, :] >> shifts[None, None, :, None]) & 3                   # [blocks, half, plane, 32]
    q = q.reshape(-1, 16, 16).float()                                            # 16 groups of 16, in value order
    dl = d[:, None] * (sc & 0xF).float()
    ml = dmin[:, None] * (sc >> 4).float()
    return (dl[:, :, None] * q - ml[:, :, None]).reshape(*lead, k)


def dequantize_q3_k(b: torch.Tensor, k: int) -> torch.Tensor:
    """Q3_K: 110 bytes per 256 values = hmask[32] (the third bit, one plane per bit position) | qs[64] (low two bits,
    laid out as in Q2_K) | scales[12] (sixteen 6-bit scales, stored minus 32) | fp16 d.
    value = d * (scale - 32) * (low2 - (0 if the high bit is set else 4))."""
    lead = b.shape[:-1]
    blk = b.reshape(-1, 110)
    hm = blk[:, 0:32].to(torch.int32)
    qs = blk[:, 32:96].to(torch.int32).reshape(-1, 2, 32)
    sr = blk[:, 96:108].to(torch.int32)
    d = _bytes_f16(blk[:, 108:110])
    # scales: low 4 bits in bytes 0-7 (two per byte: low nibbles -> scales 0-7, high nibbles -> 8-15), high 2 bits in bytes 8-11
    lo = torch.cat([sr[:, 0:8] & 0xF, sr[:, 0:8] >> 4], dim=1)                   # [blocks, 16]
    hi_bytes = sr[:, 8:12]
    hi = torch.cat([(hi_bytes >> s) & 3 for s in (0, 2, 4, 6)], dim=1)           # scales j, j+4, j+8, j+12 from byte j
    scales = (lo | (hi << 4)).float() - 32.0
    shifts = torch.tensor([0, 2, 4, 6], device=b.device, dtype=torch.int32)
    low2 = (qs[:, :, None, :] >> shifts[None, None, :, None]) & 3               # [blocks, half, plane, 32]
    bit = torch.arange(8, device=b.device, dtype=torch.int32).reshape(2, 4)      # mask bit of (half, plane)
    high = (hm[:, None, None, :] >> bit[None, :, :, None]) & 1
    q = (low2 - 4 * (1 - high)).reshape(-1, 16, 16).float()
    return (d[:, None, None] * scales[:, :, None] * q).reshape(*lead, k)


# --------------------------------------------------------------------------- dispatch


def quantize(x: torch.Tensor, qtype: GGMLType) -> torch.Tensor:
    """Quantise the last dimension of ``x``; returns a uint8 tensor of raw block bytes."""
    qtype = GGMLType(qtype)
    if qtype == GGMLType.F32:
        return x.float().contiguous().view(torch.uint8).reshape(*x.shape[:-1], x.shape[-1] * 4)
    if qtype == GGMLType.F16:
        return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape[:-1], x.shape[-1] * 2)
    if qtype == GGMLType.BF16:
        return x.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(*x.shape[:-1], x.shape[-1] * 2)
    fn = {
        GGMLType.Q4_K: quantize_q4_k,
        GGMLType.Q5_K: quantize_q5_k,
        GGMLType.Q6_K: quantize_q6_k,
        GGMLType.Q8_0: quantize_q8_0,
        GGMLType.Q4_0: quantize_q4_0,
    }.get(qtype)
    if fn is None:
        raise NotImplementedError(f"quantize: {qtype.name}")
    return fn(x)


def dequantize(b: torch.Tensor, qtype: GGMLType, cols: int) -> torch.Tensor:
    """Raw block bytes ``[..., row_bytes]`` -> fp32 ``[..., cols]``."""
    qtype = GGMLType(qtype)
    if qtype == GGMLType.F32:
        return b.contiguous().view(torch.float32).reshape(*b.shape[:-1], cols)
    if qtype == GGMLType.F16:
        return b.contiguous().view(torch.float16).reshape(*b.shape[:-1], cols).float()
    if qtype == GGMLType.BF16:
        return b.contiguous().view(torch.bfloat16).reshape(*b.shape[:-1], cols).float()
    fn = {
        GGMLType.Q4_K: dequantize_q4_k,
        GGMLType.Q5_K: dequantize_q5_k,
        GGMLType.Q6_K: dequantize_q6_k,
        GGMLType.Q8_0: dequantize_q8_0,
        GGMLType.Q4_0: dequantize_q4_0,
        GGMLType.Q2_K: dequantize_q2_k,
        GGMLType.Q3_K: dequantize_q3_k,
    }.get(qtype)
    if fn is None:
        raise NotImplementedError(f"dequantize: {qtype.name}")
    return fn(b, cols)


def quantize_activation_q8(x: torch.Tensor):
    """The activation quantisation the GEMV kernels apply to their input vector:
    per 32 values, scale = amax/127 and int8 = round(x/scale).  Returns the
    dequantised vector, so an oracle can reproduce the kernel's rounding."""
    xb = x.float().reshape(-1, 32)
    d = xb.abs().amax(dim=1) / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(xb * inv[:, None]).clamp(-127, 127)
    return (q * d[:, None]).reshape(x.shape)
