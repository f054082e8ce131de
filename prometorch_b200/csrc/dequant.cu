// Dequantisation to bf16 for the batched prompt pass: whole matrices from the GEMV streaming layout
// ([segment][row][segment bytes], see decode_kernels.cuh) and rows of the embedding table chosen by token id.
// The prompt is then processed with the tcgen05 GEMM instead of one matrix-vector product per token
// (the reference dequantises per tile inside its prefill GEMM, aten/src/ATen/cuda/CUDAQuantGemv.cu:1115-1190).
#include "decode_kernels.cuh"

namespace ptb {

// value e (0..255) of a Q4_K super-block at `bp` (GGUF byte layout)
__device__ __forceinline__ float q4k_value(const uint8_t* bp, int e) {
    const float d = __half2float(*reinterpret_cast<const __half*>(bp));
    const float dmin = __half2float(*reinterpret_cast<const __half*>(bp + 2));
    const uint8_t* s = bp + 4;
    const int is = e >> 5;
    int scv, mv;
    if (is < 4) { scv = s[is] & 63; mv = s[is + 4] & 63; }
    else { scv = (s[is + 4] & 0xF) | ((s[is - 4] >> 6) << 4); mv = (s[is + 4] >> 4) | ((s[is] >> 6) << 4); }
    const uint8_t qb = bp[16 + (e >> 6) * 32 + (e & 31)];
    const int q = (is & 1) ? (qb >> 4) : (qb & 0xF);
    return d * scv * q - dmin * mv;
}
// value e of block b of a Q6_K structure-of-arrays segment/row of nb blocks: ql[nb*128] | qh[nb*64] | scales[nb*16] | d[nb]
__device__ __forceinline__ float q6k_value(const uint8_t* seg, int nb, int b, int e) {
    const int n = e >> 7, r = e & 127, quad = r >> 5, l = r & 31;
    const uint8_t qlb = seg[b * 128 + n * 64 + (quad & 1) * 32 + l];
    const uint8_t qhb = seg[nb * 128 + b * 64 + n * 32 + l];
    const int lo4 = (quad >> 1) ? (qlb >> 4) : (qlb & 0xF);
    const int hi2 = (qhb >> (2 * quad)) & 3;
    const int q = (lo4 | (hi2 << 4)) - 32;
    const int8_t scv = reinterpret_cast<const int8_t*>(seg + nb * 192 + b * 16)[e >> 4];
    const float d = __half2float(*reinterpret_cast<const __half*>(seg + nb * 208 + b * 2));
    return d * scv * q;
}

// grid (nblk, ceil(N / 4)), 256 threads: thread e of the block handles element e of 4 consecutive rows
__global__ void __launch_bounds__(256) dequant_segmajor_kernel(const uint8_t* __restrict__ w, int qtype, int N, int nblk, int KS,
                                                               int seg_base, int seg_rem, __nv_bfloat16* __restrict__ out) {
    const int b = blockIdx.x, e = threadIdx.x;
    // segment of block b: the first seg_rem segments hold seg_base + 1 blocks
    const int big = seg_rem * (seg_base + 1);
    int s, bi;
    if (b < big) { s = b / (seg_base + 1); bi = b - s * (seg_base + 1); }
    else { s = seg_rem + (b - big) / seg_base; bi = (b - big) - (s - seg_rem) * seg_base; }
    const int nb = seg_base + (s < seg_rem ? 1 : 0);
    const int sz0 = seg_bytes(qtype, seg_base), sz1 = seg_bytes(qtype, seg_base + 1);
    const int extra = min(s, seg_rem);
    const size_t seg_off = (size_t)N * ((size_t)s * sz0 + (size_t)extra * (sz1 - sz0));
    const int sb = s < seg_rem ? sz1 : sz0;
    for (int r = blockIdx.y * 4; r < min(N, (int)blockIdx.y * 4 + 4); ++r) {
        const uint8_t* rowseg = w + seg_off + (size_t)r * sb;
        const float v = qtype == QT_Q4K ? q4k_value(rowseg + bi * 144, e) : q6k_value(rowseg, nb, bi, e);
        out[(size_t)r * nblk * 256 + (size_t)b * 256 + e] = __float2bfloat16_rn(v);
    }
}

// The tiles-of-16-rows layout of the tensor-pipe GEMV (decode_gemv_mma.cuh).  grid (nblk, ceil(N / 4)), 256 threads.
__global__ void __launch_bounds__(256) dequant_t16_kernel(const uint8_t* __restrict__ w, int qtype, int N, int nblk,
                                                          __nv_bfloat16* __restrict__ out) {
    const int b = blockIdx.x, e = threadIdx.x;
    for (int r = blockIdx.y * 4; r < min(N, (int)blockIdx.y * 4 + 4); ++r) {
        const int tile = r >> 4, rr = r & 15;
        float v;
        if (qtype == QT_Q4K) {
            v = q4k_value(w + (((size_t)tile * nblk + b) * 16 + rr) * 144, e);
        } else if (qtype == QT_Q5K) {
            // Q4_K with a fifth bit per value: bit (sub-block) of byte (value in sub-block) of the 32 bytes at offset 16
            const uint8_t* bp = w + (((size_t)tile * nblk + b) * 16 + rr) * 176;
            const float d = __half2float(*reinterpret_cast<const __half*>(bp));
            const float dmin = __half2float(*reinterpret_cast<const __half*>(bp + 2));
            const uint8_t* s = bp + 4;
            const int is = e >> 5;
            int scv, mv;
            if (is < 4) { scv = s[is] & 63; mv = s[is + 4] & 63; }
            else { scv = (s[is + 4] & 0xF) | ((s[is - 4] >> 6) << 4); mv = (s[is + 4] >> 4) | ((s[is] >> 6) << 4); }
            const uint8_t qb = bp[48 + (e >> 6) * 32 + (e & 31)];
            const int q = ((is & 1) ? (qb >> 4) : (qb & 0xF)) | (((bp[16 + (e & 31)] >> is) & 1) << 4);
            v = d * scv * q - dmin * mv;
        } else if (qtype == QT_Q8_0) {
            const uint8_t* blk = w + ((size_t)tile * nblk + b) * 4352;
            const int u = e >> 5;
            const int8_t q = reinterpret_cast<const int8_t*>(blk + rr * 256)[((u ^ (rr & 7)) << 5) | (e & 31)];
            v = __half2float(*reinterpret_cast<const __half*>(blk + 4096 + rr * 16 + u * 2)) * (float)q;
        } else if (qtype == QT_F16) {
            // four 64-value blocks of 2048 bytes make up these 256 values
            const uint8_t* blk = w + ((size_t)tile * (nblk * 4) + (size_t)b * 4 + (e >> 6)) * 2048;
            const int i = e & 63, u = i >> 4;
            v = __half2float(reinterpret_cast<const __half*>(blk + rr * 128)[((u ^ (rr & 3)) << 4) | (i & 15)]);
        } else {
            const uint8_t* blk = w + ((size_t)tile * nblk + b) * 3360;
            const int n = e >> 7, r7 = e & 127, quad = r7 >> 5, l = r7 & 31;
            const int qi = n * 64 + (quad & 1) * 32 + l, hi = n * 32 + l;
            const uint8_t qlb = blk[rr * 128 + ((((qi >> 4) ^ (rr & 7)) << 4) | (qi & 15))];
            const uint8_t qhb = blk[2048 + rr * 64 + ((((hi >> 4) ^ ((rr >> 1) & 3)) << 4) | (hi & 15))];
            const int lo4 = (quad >> 1) ? (qlb >> 4) : (qlb & 0xF);
            const int q = (lo4 | (((qhb >> (2 * quad)) & 3) << 4)) - 32;
            const int8_t scv = reinterpret_cast<const int8_t*>(blk + 3072 + rr * 16)[e >> 4];
            const float d = __half2float(*reinterpret_cast<const __half*>(blk + 3328 + rr * 2));
            v = d * scv * q;
        }
        out[(size_t)r * nblk * 256 + (size_t)b * 256 + e] = __float2bfloat16_rn(v);
    }
}

// grid (nblk, T), 256 threads: row ids[t] of a row-major table (Q4_K bytes / Q6_K SoA rows / fp16 / fp32)
__global__ void __launch_bounds__(256) dequant_rows_kernel(const uint8_t* __restrict__ table, int qtype, int rowbytes, int nblk,
                                                           const int* __restrict__ ids, float scale, int vocab, int* status,
                                                           __nv_bfloat16* __restrict__ out) {
    const int b = blockIdx.x, t = blockIdx.y, e = threadIdx.x;
    int tok = ids[t];
    if (tok < 0 || tok >= vocab) {
        if (e == 0 && b == 0) atomicExch(status, PTB_ERR_BOUNDS);
        tok = 0;
    }
    const uint8_t* row = table + (size_t)tok * rowbytes;
    const int i = b * 256 + e;
    float v;
    if (qtype == QT_Q4K) v = q4k_value(row + b * 144, e);
    else if (qtype == QT_Q6K) v = q6k_value(row, nblk, b, e);
    else if (qtype == 2) v = __half2float(reinterpret_cast<const __half*>(row)[i]);
    else v = reinterpret_cast<const float*>(row)[i];
    out[(size_t)t * nblk * 256 + i] = __float2bfloat16_rn(v * scale);
}

}  // namespace ptb

using namespace ptb;

// w: a matrix of N rows x cols in a GEMV streaming layout -> out bf16 [N, cols] row-major.
// layout: 0 = [segment][row][segment bytes], 1 = tiles of 16 rows.
PTB_API int ptb_dequant_weight(const void* w, int qtype, int layout, int N, int cols, void* out, cudaStream_t st) {
    if (cols % 256 || N <= 0) { ptb_set_error("dequant: %d x %d not supported", N, cols); return -1; }
    const bool tile_only = qtype == QT_Q5K || qtype == QT_Q8_0 || qtype == QT_F16;
    if (!(qtype == QT_Q4K || qtype == QT_Q6K || (tile_only && layout == 1))) {
        ptb_set_error("dequant: quantisation type %d is not available in layout %d", qtype, layout);
        return -1;
    }
    const int nblk = cols / 256;
    if (layout == 1) {
        dequant_t16_kernel<<<dim3(nblk, (N + 3) / 4), 256, 0, st>>>((const uint8_t*)w, qtype, N, nblk, (__nv_bfloat16*)out);
        PTB_CUDA_OK(cudaGetLastError());
        return 0;
    }
    const int KS = (nblk + GEMV_SEG_BLOCKS - 1) / GEMV_SEG_BLOCKS;
    dequant_segmajor_kernel<<<dim3(nblk, (N + 3) / 4), 256, 0, st>>>((const uint8_t*)w, qtype, N, nblk, KS, nblk / KS, nblk % KS,
                                                                    (__nv_bfloat16*)out);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// out[t] = scale * table[ids[t]] for T ids (device int32).  status: device word, set if an id is out of range.
PTB_API int ptb_dequant_rows(const void* table, int qtype, int rowbytes, int cols, const int* ids, int T, float scale, int vocab,
                             int* status, void* out, cudaStream_t st) {
    if (cols % 256 || T <= 0) { ptb_set_error("dequant rows: %d ids x %d columns not supported", T, cols); return -1; }
    dequant_rows_kernel<<<dim3(cols / 256, T), 256, 0, st>>>((const uint8_t*)table, qtype, rowbytes, cols / 256, ids, scale, vocab, status,
                                                             (__nv_bfloat16*)out);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}
