// Dequant-GEMV on the tensor pipe for the "tile of 16 rows" weight layout.
//
// The dp4a kernel in decode_kernels.cuh lets four lanes share one 256-value super-block, so every group of four
// lanes re-reads the activations from shared memory (about 3.5 bytes of shared-memory traffic per weight byte) and
// that traffic, not HBM, bounds its tile phase.  Here a warp works on 16 rows at once with integer MMA
// (mma.sync m16n8k32, u8 x s8 -> s32): the weights are the A operand straight out of the TMA tile (one 8-byte load
// per lane per 64 nibbles, no conflicts), the activations are the B operand, and shared memory is read about 1.1
// times per weight byte.  The tensor pipe has room to spare at batch 1 (one of eight output columns is used), what is
// saved is the load/store pipe.  tcgen05 has no 4-bit integer operand kind and needs its operands in shared memory,
// which would cost an unpack pass through shared memory per tile; the register-operand MMA avoids that.
//
// The eight MMA output columns are put to work as eight accumulators: a 32-value sub-block (Q4_K) or a pair of
// 16-value scale groups (Q6_K) is multiplied with a B operand that is zero except in ITS column, so after the
// eight MMAs of a super-block lane (g, t) holds the integer dot products of sub-blocks 2t and 2t+1 for rows g and g+8:
// exactly the distribution in which the four lanes of a row then apply the 6-bit scales in parallel.
//
// Weight layout "T16" (written once at load time by io/gguf_model.py):
//   rows are padded to a multiple of 16 with zero blocks; tile = 16 consecutive rows;
//   Q4_K: [tile][super-block][row in tile][144 bytes as in the GGUF file]              -> 2304 bytes per (tile, block)
//   Q6_K: [tile][super-block]{ ql[16][128] | qh[16][64] | int8 scales[16][16] | fp16 d[16] }  -> 3360 bytes;
//         the 16-byte chunks of a ql row are stored at chunk ^ (row & 7), those of a qh row at chunk ^ ((row >> 1) & 3),
//         which spreads the eight rows a load instruction touches over all banks.
//   Q5_K: as Q4_K with the file's 176-byte blocks                                      -> 2816 bytes per (tile, block)
//   Q8_0: [tile][256 values]{ q[16][256] int8, the 32-byte unit u of a row stored at u ^ (row & 7) | fp16 d[16][8] }
//         -> 4352 bytes (eight 32-value GGUF blocks per row)
//   F16:  [tile][64 values][16][64] halves, the 32-byte unit u of a row stored at u ^ (row & 3)   -> 2048 bytes;
//         here a "block" is 64 values, so such a job counts K / 64 blocks
// One (tile, block) unit is one untiled TMA bulk copy; a warp streams the blocks of its items through a private ring.
//
// Reference counterparts: q4km_persistent_gemv_kernel / q6k_gemv_kernel (aten/src/ATen/cuda/CUDAQuantGemv.cu:168-313,
// 881-976), one warp per row with __dp4a.
#pragma once
#include "decode_kernels.cuh"

#include <type_traits>

namespace ptb {

constexpr int T16_ROWS = 16;
__host__ __device__ __forceinline__ int t16_block_bytes(int qtype) {
    switch (qtype) {
        case QT_Q4K: return 16 * 144;
        case QT_Q5K: return 16 * 176;
        case QT_Q8_0: return 16 * 272;
        case QT_F16: return 16 * 128;
        default: return 16 * 210;
    }
}
// values of one row that a block holds
__host__ __device__ __forceinline__ int t16_block_vals(int qtype) { return qtype == QT_F16 ? 64 : 256; }

// D += A (16x32, u8, row-major fragments) * B (32x8, s8, column fragments), s32 accumulate.
__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_s8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D += A (16x16 f16) * B (16x8 f16), f32 accumulate.
__device__ __forceinline__ void mma_f16_k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Row of the tile that MMA row g (0..7) stands for in the Q4_K path (and g + 8 -> that row + 8).  With a row pitch of
// 144 bytes, taking rows 0,2,4,6 for lanes 0-15 and 1,3,5,7 for lanes 16-31 keeps each half-warp's 8-byte loads on
// distinct banks.
__device__ __forceinline__ int q4k_row_of(int g) { return 2 * (g & 3) + (g >> 2); }

// Bit BIT of every byte of h moved to bit 4 of that byte.
template <int BIT>
__device__ __forceinline__ uint32_t bit_to_4(uint32_t h) {
    return (BIT <= 4 ? (h << (4 - (BIT <= 4 ? BIT : 4))) : (h >> ((BIT > 4 ? BIT : 4) - 4))) & 0x10101010u;
}

// One Q4_K (Q5 = false, 144-byte blocks) or Q5_K (Q5 = true, 176-byte blocks: 32 bytes of fifth bits between the
// scales and the nibbles) super-block of 16 rows.  xq_b: the block's 256 int8 activations, xs_b[8] their scales,
// xsf32_b[8] = scale * (sum of the 32 int8 values).  Lane (g, t) adds to acc0 / acc8 its share (sub-blocks 2t, 2t+1)
// of the dot products of rows q4k_row_of(g) and q4k_row_of(g) + 8.
template <bool Q5>
__device__ __forceinline__ void q45k_block_mma(const uint8_t* blk, const int8_t* xq_b, const float* xs_b, const float* xsf32_b, int g,
                                               int t, float& acc0, float& acc8) {
    constexpr int PITCH = Q5 ? 176 : 144, QS = Q5 ? 48 : 16;
    const uint8_t* r0 = blk + q4k_row_of(g) * PITCH;
    const uint8_t* r8 = r0 + 8 * PITCH;
    // my column's activations: sub-block g, bytes 8t .. 8t+7 (k slots 4t.. and 16+4t.. of the MMA)
    const uint2 xb = *reinterpret_cast<const uint2*>(xq_b + g * 32 + 8 * t);
    uint2 ha = make_uint2(0, 0), hb = make_uint2(0, 0);
    if (Q5) {
        // byte l of the 32 holds the fifth bit of value l of sub-block s in bit s
        ha = *reinterpret_cast<const uint2*>(r0 + 16 + 8 * t);
        hb = *reinterpret_cast<const uint2*>(r8 + 16 + 8 * t);
    }
    int c[4] = {0, 0, 0, 0};
    constexpr uint32_t LO = 0x0F0F0F0Fu;
    auto chunk = [&](auto chc) {
        constexpr int ch = decltype(chc)::value;
        const uint2 wa = *reinterpret_cast<const uint2*>(r0 + QS + ch * 32 + 8 * t);
        const uint2 wb = *reinterpret_cast<const uint2*>(r8 + QS + ch * 32 + 8 * t);
        const bool lo = g == 2 * ch, hi = g == 2 * ch + 1;
        if (!Q5) {
            // low nibbles: sub-block 2ch -> column 2ch; high nibbles (kept in place, i.e. 16 x value): sub-block 2ch+1
            mma_u8s8_k32(c, wa.x & LO, wb.x & LO, wa.y & LO, wb.y & LO, lo ? xb.x : 0u, lo ? xb.y : 0u);
            mma_u8s8_k32(c, wa.x & ~LO, wb.x & ~LO, wa.y & ~LO, wb.y & ~LO, hi ? xb.x : 0u, hi ? xb.y : 0u);
        } else {
            mma_u8s8_k32(c, (wa.x & LO) | bit_to_4<2 * ch>(ha.x), (wb.x & LO) | bit_to_4<2 * ch>(hb.x),
                         (wa.y & LO) | bit_to_4<2 * ch>(ha.y), (wb.y & LO) | bit_to_4<2 * ch>(hb.y), lo ? xb.x : 0u, lo ? xb.y : 0u);
            mma_u8s8_k32(c, ((wa.x >> 4) & LO) | bit_to_4<2 * ch + 1>(ha.x), ((wb.x >> 4) & LO) | bit_to_4<2 * ch + 1>(hb.x),
                         ((wa.y >> 4) & LO) | bit_to_4<2 * ch + 1>(ha.y), ((wb.y >> 4) & LO) | bit_to_4<2 * ch + 1>(hb.y),
                         hi ? xb.x : 0u, hi ? xb.y : 0u);
        }
    };
    chunk(std::integral_constant<int, 0>{});
    chunk(std::integral_constant<int, 1>{});
    chunk(std::integral_constant<int, 2>{});
    chunk(std::integral_constant<int, 3>{});
    // c[0], c[2]: sub-block 2t of rows g, g+8;  c[1], c[3]: sub-block 2t+1 (Q4_K: 16 x it, exact multiples of 16)
    if (!Q5) {
        c[1] >>= 4;
        c[3] >>= 4;
    }
    const float2 xs2 = *reinterpret_cast<const float2*>(xs_b + 2 * t);
    const float2 sm2 = *reinterpret_cast<const float2*>(xsf32_b + 2 * t);
    const int sh = 16 * (t & 1);
    auto row_value = [&](const uint8_t* rp, int d_lo, int d_hi) -> float {
        const uint4 hdr = *reinterpret_cast<const uint4*>(rp);
        const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
        // 6-bit scales / mins of sub-blocks 2t and 2t+1
        const uint32_t a = (hdr.y >> sh) & 0xffffu, b = (hdr.z >> sh) & 0xffffu, cc = (hdr.w >> sh) & 0xffffu;
        uint32_t sc2, mn2;
        if (t < 2) { sc2 = a & 0x3f3fu; mn2 = b & 0x3f3fu; }
        else { sc2 = (cc & 0x0f0fu) | ((a & 0xc0c0u) >> 2); mn2 = ((cc >> 4) & 0x0f0fu) | ((b & 0xc0c0u) >> 2); }
        const float va = (float)((int)(sc2 & 0xffu) * d_lo) * xs2.x + (float)((int)(sc2 >> 8) * d_hi) * xs2.y;
        const float vb = (float)(mn2 & 0xffu) * sm2.x + (float)(mn2 >> 8) * sm2.y;
        return dm.x * va - dm.y * vb;
    };
    acc0 += row_value(r0, c[0], c[1]);
    acc8 += row_value(r8, c[2], c[3]);
}

// 256 values of 16 Q8_0 rows (eight 32-value blocks per row).  Sub-block s goes to output column s, so lane (g, t)
// ends up with sub-blocks 2t and 2t+1 of rows g and g + 8 and applies d[row][sub-block] * activation scale.
__device__ __forceinline__ void q80_block_mma(const uint8_t* blk, const int8_t* xq_b, const float* xs_b, int g, int t, float& acc0,
                                              float& acc8) {
    const uint8_t* r0 = blk + g * 256;
    const uint8_t* r8 = r0 + 8 * 256;
    const uint2 xb = *reinterpret_cast<const uint2*>(xq_b + g * 32 + 8 * t);
    int c[4] = {0, 0, 0, 0};
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const int u = ((s ^ (g & 7)) << 5) + 8 * t;
        const uint2 wa = *reinterpret_cast<const uint2*>(r0 + u);
        const uint2 wb = *reinterpret_cast<const uint2*>(r8 + u);
        const bool mine = g == s;
        mma_s8s8_k32(c, wa.x, wb.x, wa.y, wb.y, mine ? xb.x : 0u, mine ? xb.y : 0u);
    }
    const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(blk + 4096 + g * 16 + 4 * t));
    const float2 d8 = __half22float2(*reinterpret_cast<const __half2*>(blk + 4096 + (g + 8) * 16 + 4 * t));
    const float2 xs2 = *reinterpret_cast<const float2*>(xs_b + 2 * t);
    acc0 += d0.x * xs2.x * (float)c[0] + d0.y * xs2.y * (float)c[1];
    acc8 += d8.x * xs2.x * (float)c[2] + d8.y * xs2.y * (float)c[3];
}

// 64 values of 16 fp16 rows.  The B operand carries the int8 activations as halves (exact) in column 0 only; the
// activation scale of each 32-value group is applied to the fp32 result, so nothing can overflow fp16.  Lanes with
// t == 0 receive rows g and g + 8, the other lanes add zeros.
__device__ __forceinline__ void f16_block_mma(const uint8_t* blk, const int8_t* xq_b, const float* xs_b, int g, int t, float& acc0,
                                              float& acc8) {
    const uint8_t* r0 = blk + g * 128;
    const uint8_t* r8 = r0 + 8 * 128;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int mm = 0; mm < 2; ++mm) {
            const int m = 2 * h + mm;                     // 16 values = one 32-byte unit of each row
            const int u = ((m ^ (g & 3)) << 5) + 8 * t;
            const uint2 wa = *reinterpret_cast<const uint2*>(r0 + u);       // values 16m + 4t .. 16m + 4t + 3
            const uint2 wb = *reinterpret_cast<const uint2*>(r8 + u);
            uint32_t b0 = 0u, b1 = 0u;
            if (g == 0) {
                const char4 x4 = *reinterpret_cast<const char4*>(xq_b + 16 * m + 4 * t);
                const __half2 p0 = __halves2half2(__int2half_rn(x4.x), __int2half_rn(x4.y));
                const __half2 p1 = __halves2half2(__int2half_rn(x4.z), __int2half_rn(x4.w));
                b0 = *reinterpret_cast<const uint32_t*>(&p0);
                b1 = *reinterpret_cast<const uint32_t*>(&p1);
            }
            mma_f16_k16(c, wa.x, wb.x, wa.y, wb.y, b0, b1);
        }
        acc0 += xs_b[h] * c[0];
        acc8 += xs_b[h] * c[2];
    }
}

// One Q6_K super-block of 16 rows (layout in the header comment).  xsf16_b[16] = scale * (sum of 16 int8 values).
// Lane (g, t) adds to acc0 / acc8 its share (scale groups with q = t) of the dot products of rows g and g + 8.
__device__ __forceinline__ void q6k_block_mma(const uint8_t* blk, const int8_t* xq_b, const float* xs_b, const float* xsf16_b, int g,
                                              int t, float& acc0, float& acc8) {
    const uint8_t* ql0 = blk + g * 128;
    const uint8_t* ql8 = ql0 + 8 * 128;
    const uint8_t* qh0 = blk + 2048 + g * 64;
    const uint8_t* qh8 = qh0 + 8 * 64;
    const int8_t* sc0 = reinterpret_cast<const int8_t*>(blk + 3072 + g * 16);
    const int8_t* sc8 = sc0 + 8 * 16;
    const float d0 = __half2float(*reinterpret_cast<const __half*>(blk + 3328 + g * 2));
    const float d8 = __half2float(*reinterpret_cast<const __half*>(blk + 3328 + (g + 8) * 2));
    const int sw = g & 7, swh = (g >> 1) & 3;          // the same for row g + 8
    float r0 = 0.f, r8 = 0.f;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        // my column's activations in this half: scale group q = g >> 1, h = g & 1 -> values n*128 + q*32 + 16h + 4t ..
        const uint32_t xb = *reinterpret_cast<const uint32_t*>(xq_b + n * 128 + (g >> 1) * 32 + 16 * (g & 1) + 4 * t);
        int c[4] = {0, 0, 0, 0};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int ca = ((n * 4 + h) ^ sw) << 4, cb = ((n * 4 + 2 + h) ^ sw) << 4, chh = ((n * 2 + h) ^ swh) << 4;
            const uint32_t la0 = *reinterpret_cast<const uint32_t*>(ql0 + ca + 4 * t), lb0 = *reinterpret_cast<const uint32_t*>(ql0 + cb + 4 * t);
            const uint32_t la8 = *reinterpret_cast<const uint32_t*>(ql8 + ca + 4 * t), lb8 = *reinterpret_cast<const uint32_t*>(ql8 + cb + 4 * t);
            const uint32_t h0 = *reinterpret_cast<const uint32_t*>(qh0 + chh + 4 * t), h8 = *reinterpret_cast<const uint32_t*>(qh8 + chh + 4 * t);
            // the four scale groups q = 0..3 of (n, h): 4 low bits from ql, 2 high bits from qh (values 0..63)
            constexpr uint32_t LO = 0x0F0F0F0Fu, HI = 0x30303030u;
            const uint32_t v00 = (la0 & LO) | ((h0 << 4) & HI), v10 = (lb0 & LO) | ((h0 << 2) & HI);
            const uint32_t v20 = ((la0 >> 4) & LO) | (h0 & HI), v30 = ((lb0 >> 4) & LO) | ((h0 >> 2) & HI);
            const uint32_t v08 = (la8 & LO) | ((h8 << 4) & HI), v18 = (lb8 & LO) | ((h8 << 2) & HI);
            const uint32_t v28 = ((la8 >> 4) & LO) | (h8 & HI), v38 = ((lb8 >> 4) & LO) | ((h8 >> 2) & HI);
            // groups (q=0, h) and (q=1, h) -> columns h and 2 + h; (q=2, h), (q=3, h) -> columns 4 + h and 6 + h
            mma_u8s8_k32(c, v00, v08, v10, v18, g == h ? xb : 0u, g == 2 + h ? xb : 0u);
            mma_u8s8_k32(c, v20, v28, v30, v38, g == 4 + h ? xb : 0u, g == 6 + h ? xb : 0u);
        }
        // c[0], c[1]: row g, groups (q = t, h = 0 / 1); c[2], c[3]: row g + 8.  Stored values are q + 32.
        const float xsq = xs_b[n * 4 + t];
        const float2 sf = *reinterpret_cast<const float2*>(xsf16_b + n * 8 + 2 * t);
        const int si = n * 8 + 2 * t;
        r0 += (float)sc0[si] * (xsq * (float)c[0] - 32.0f * sf.x) + (float)sc0[si + 1] * (xsq * (float)c[1] - 32.0f * sf.y);
        r8 += (float)sc8[si] * (xsq * (float)c[2] - 32.0f * sf.x) + (float)sc8[si + 1] * (xsq * (float)c[3] - 32.0f * sf.y);
    }
    acc0 += d0 * r0;
    acc8 += d8 * r8;
}

// Job geometry for this kernel (GemvJob fields reused): KS = K-groups per row tile, seg_base / seg_rem = blocks per
// K-group (the first seg_rem groups one block longer); a CTA owns whole row tiles and its warps take (tile, K-group)
// items in turn, each warp streaming the blocks of its items through its private ring, one block per ring slot.
template <int GEMV_WARPS, int MODE = 0>
__global__ void __launch_bounds__(GEMV_WARPS * 32, GEMV_WARPS >= 16 ? 1 : 2) gemv16_kernel(const __grid_constant__ GemvParams P) {
    constexpr int GEMV_THREADS = GEMV_WARPS * 32;
    constexpr bool LEAN = MODE == 1;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = P.K, S = P.stages;
    const GemvSmem L = gemv_smem_layout(K, GEMV_WARPS, S, P.tile_bytes, P.acc_floats);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars) + warp * S;
    float* misc = reinterpret_cast<float*>(smem + L.misc);
    int8_t* xq = reinterpret_cast<int8_t*>(smem + L.xq);
    float* xs = reinterpret_cast<float*>(smem + L.xs);
    float* xsf = reinterpret_cast<float*>(smem + L.xsf);
    float* xsf32 = reinterpret_cast<float*>(smem + L.xsf32);
    float* acc = reinterpret_cast<float*>(smem + L.acc);
    uint8_t* ring = smem + L.tiles + (size_t)warp * S * P.tile_bytes;

    auto stamp = [&](int k) {
        if (P.trace && tid == 0 && blockIdx.x == 0) P.trace[k] = global_ns();
    };
    stamp(0);
    int ji = 0;
#pragma unroll
    for (int i = 1; i < GEMV_MAX_JOBS; ++i)
        if (i < P.njobs && (int)blockIdx.x >= P.job[i].cta_begin) ji = i;
    const GemvJob& J = P.job[ji];
    const int ci = blockIdx.x - J.cta_begin;
    const int ntile = (J.N + T16_ROWS - 1) / T16_ROWS;
    const int t0 = (int)(((long long)ntile * ci) / J.cta_count), t1 = (int)(((long long)ntile * (ci + 1)) / J.cta_count);
    const int KG = J.KS, qtype = J.qtype;
    const int nitems = (t1 - t0) * KG;
    const bool paired = J.w2 != nullptr;
    const int bb = t16_block_bytes(qtype);

    auto item_geom = [&](int it, int& tile, int& kb0, int& nb, int& kg) {
        const int tl = it / KG;
        kg = it - tl * KG;
        tile = t0 + tl;
        nb = J.seg_base + (kg < J.seg_rem ? 1 : 0);
        kb0 = kg * J.seg_base + min(kg, J.seg_rem);
    };
    // producer cursor (lane 0): the next (item, block) to request
    int p_it = warp, p_b = 0, p_tile = 0, p_kb0 = 0, p_nb = 0, p_kg = 0;
    if (p_it < nitems) item_geom(p_it, p_tile, p_kb0, p_nb, p_kg);
    auto issue_next = [&](int slot) {       // lane 0 only
        if (p_it >= nitems) return;
        const size_t off = ((size_t)p_tile * J.nblk + (size_t)(p_kb0 + p_b)) * bb;
        uint8_t* dst = ring + (size_t)slot * P.tile_bytes;
        mbar_expect_tx(&full[slot], paired ? 2u * bb : (uint32_t)bb);
        bulk_g2s(dst, J.w + off, (uint32_t)bb, &full[slot]);
        if (paired) bulk_g2s(dst + bb, J.w2 + off, (uint32_t)bb, &full[slot]);
        if (++p_b == p_nb) {
            p_it += GEMV_WARPS;
            p_b = 0;
            if (p_it < nitems) item_geom(p_it, p_tile, p_kb0, p_nb, p_kg);
        }
    };
    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
        fence_proxy_async();
        for (int s = 0; s < S; ++s) issue_next(s);      // the weights do not depend on the previous kernel
    }
    if (P.norm_w) {
        for (int i = tid * 32; i < K; i += GEMV_THREADS * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(P.norm_w + i));
    }
    pdl_launch_dependents();
    const bool dataflow = MODE == 2 || (!LEAN && P.x_ll != nullptr);
    if (!dataflow || P.hard_wait) pdl_wait();
    __syncthreads();
    stamp(1);
    const uint32_t gen = P.gen ? *reinterpret_cast<const volatile uint32_t*>(P.gen) : 0u;
    const uint32_t seq = gen * LL_SEQ_MUL + P.out_seq_add;
    const float in_scale = gemv_input<GEMV_WARPS, MODE>(P, gen, seq, K, xq, xs, xsf, xsf32, misc, warp, lane);
    stamp(2);

    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    auto epilogue = [&](int n, float v0, float v1) {
        v0 *= in_scale;
        v1 *= in_scale;
        if (J.bias) v0 += J.bias[n];
        float r = v0;
        switch (P.epilogue) {
            case EPI_STORE: break;
            case EPI_RESID: r = P.resid[n] + v0; break;
            case EPI_GATED: r = (P.act_gelu ? gelu_tanh(v0) : silu(v0)) * v1; break;
            case EPI_ARGMAX:
                if (P.logits) P.logits[n] = v0;
                if (v0 > best_v || (v0 == best_v && n < best_i)) { best_v = v0; best_i = n; }
                return;
            case EPI_ALLREDUCE:
            case EPI_PARTIAL: {
                const PeerInfo& pi = P.peers;
                for (int p = 0; p < pi.world; ++p) st_ll(pi.inbox[p] + (size_t)pi.rank * pi.slot_elems + n, __float_as_uint(v0), seq);
                return;
            }
        }
        if (!LEAN && J.out_ll) st_ll(J.out_ll + n, __float_as_uint(r), seq);
        else J.out[n] = r;
    };

    const int g = lane >> 2, t = lane & 3;
    const int row_a = (qtype == QT_Q4K || qtype == QT_Q5K) ? q4k_row_of(g) : g;       // the tile row MMA row g stands for
    const int npair = paired ? 2 : 1;
    // The item loop is instantiated once per weight type, so that the block loop of a launch holds one type's code only.
    auto run_items = [&](auto qt_c) {
        constexpr int QT = decltype(qt_c)::value;
        auto block = [&](const uint8_t* tp, int blk, float& r0, float& r8) {
            if constexpr (QT == QT_Q4K) q45k_block_mma<false>(tp, xq + blk * 256, xs + blk * 8, xsf32 + blk * 8, g, t, r0, r8);
            else if constexpr (QT == QT_Q5K) q45k_block_mma<true>(tp, xq + blk * 256, xs + blk * 8, xsf32 + blk * 8, g, t, r0, r8);
            else if constexpr (QT == QT_Q8_0) q80_block_mma(tp, xq + blk * 256, xs + blk * 8, g, t, r0, r8);
            else if constexpr (QT == QT_F16) f16_block_mma(tp, xq + blk * 64, xs + blk * 2, g, t, r0, r8);
            else q6k_block_mma(tp, xq + blk * 256, xs + blk * 8, xsf + blk * 16, g, t, r0, r8);
        };
        bool ok = true;
        int k = 0;
        for (int it = warp; it < nitems; it += GEMV_WARPS) {
            int tile, kb0, nb, kg;
            item_geom(it, tile, kb0, nb, kg);
            float a0 = 0.f, a8 = 0.f, b0 = 0.f, b8 = 0.f;
            for (int b = 0; b < nb; ++b, ++k) {
                const int slot = k % S;
                if (ok) ok = mbar_wait(&full[slot], (uint32_t)((k / S) & 1), P.status);
                if (k == 0) stamp(3);
                if (ok) {
                    const uint8_t* tp = ring + (size_t)slot * P.tile_bytes;
                    block(tp, kb0 + b, a0, a8);
                    if (paired) block(tp + bb, kb0 + b, b0, b8);
                }
                __syncwarp();
                if (lane == 0) issue_next(slot);
            }
            // the four lanes of a row hold its sub-block shares
            a0 += __shfl_xor_sync(0xffffffffu, a0, 1); a0 += __shfl_xor_sync(0xffffffffu, a0, 2);
            a8 += __shfl_xor_sync(0xffffffffu, a8, 1); a8 += __shfl_xor_sync(0xffffffffu, a8, 2);
            if (paired) {
                b0 += __shfl_xor_sync(0xffffffffu, b0, 1); b0 += __shfl_xor_sync(0xffffffffu, b0, 2);
                b8 += __shfl_xor_sync(0xffffffffu, b8, 1); b8 += __shfl_xor_sync(0xffffffffu, b8, 2);
            }
            if (t == 0) {
                if (KG == 1) {
                    const int n0 = tile * T16_ROWS + row_a;
                    if (n0 < J.N) epilogue(n0, a0, b0);
                    if (n0 + 8 < J.N) epilogue(n0 + 8, a8, b8);
                } else {
                    float* ap = acc + ((size_t)((tile - t0) * KG + kg) * npair) * T16_ROWS;
                    ap[row_a] = a0;
                    ap[row_a + 8] = a8;
                    if (paired) { ap[T16_ROWS + row_a] = b0; ap[T16_ROWS + row_a + 8] = b8; }
                }
            }
        }
    };
    switch (qtype) {
        case QT_Q4K: run_items(std::integral_constant<int, QT_Q4K>{}); break;
        case QT_Q5K: run_items(std::integral_constant<int, QT_Q5K>{}); break;
        case QT_Q8_0: run_items(std::integral_constant<int, QT_Q8_0>{}); break;
        case QT_F16: run_items(std::integral_constant<int, QT_F16>{}); break;
        default: run_items(std::integral_constant<int, QT_Q6K>{}); break;
    }
    stamp(4);
    if (KG > 1) {
        __syncthreads();
        for (int r = tid; r < (t1 - t0) * T16_ROWS; r += GEMV_THREADS) {
            const int tl = r / T16_ROWS, rr = r - tl * T16_ROWS;
            const int n = (t0 + tl) * T16_ROWS + rr;
            if (n >= J.N) continue;
            float v0 = 0.f, v1 = 0.f;
            for (int q = 0; q < KG; ++q) {
                const float* ap = acc + ((size_t)(tl * KG + q) * npair) * T16_ROWS;
                v0 += ap[rr];
                if (paired) v1 += ap[T16_ROWS + rr];
            }
            epilogue(n, v0, v1);
        }
    }
    stamp(5);
    if (P.epilogue == EPI_ARGMAX) gemv_argmax_tail<GEMV_WARPS>(P, best_v, best_i, misc, gen, seq);
    if (P.epilogue == EPI_ALLREDUCE) {
        // Producer-side all-reduce (plain flow under tensor parallelism): every CTA reduces its own slice of the output.
        // It polls the `world` slots of each element (filled by CTAs of this kernel on every rank), sums them in rank
        // order so that all ranks get bitwise the same vector, adds the residual and stores the plain result.
        const PeerInfo& pi = P.peers;
        const int N = J.N;
        const int n0 = (int)(((long long)N * blockIdx.x) / gridDim.x), n1 = (int)(((long long)N * (blockIdx.x + 1)) / gridDim.x);
        for (int n = n0 + tid; n < n1; n += GEMV_THREADS) {
            float v = P.resid ? P.resid[n] : 0.f;
            for (int p = 0; p < pi.world; ++p)
                v += __uint_as_float(wait_ll(pi.inbox[pi.rank] + (size_t)p * pi.slot_elems + n, seq, P.status, P.wait_ns));
            J.out[n] = v;
        }
    }
}

}  // namespace ptb
