// FlashAttention building blocks shared by the forward and backward kernels:
// swizzled shared-memory tiles filled by cp.async, ldmatrix fragment loads and
// the bf16 m16n8k16 tensor-core MMA.  (These kernels use the warp-level MMA
// path; the GEMMs of this library use tcgen05.)
#pragma once
#include "common.cuh"

namespace ptb {
namespace fa {

constexpr int BR = 64;       // query rows per CTA (4 warps x 16)
constexpr int BC = 64;       // key/value rows per tile
constexpr int THREADS = 128;

// Byte offset of 16-byte chunk `c` of row `r` in a [rows][D] bf16 tile; XOR swizzle keeps ldmatrix conflict-free.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
    return (uint32_t)(r * (D * 2) + ((c ^ (r & 7)) << 4));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;      // size 0 => the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }

// Load a [ROWS][D] tile whose global rows are `stride` elements apart; rows >= rows_valid are zero-filled.
template <int D, int ROWS>
__device__ __forceinline__ void load_tile(uint32_t smem_base, const __nv_bfloat16* g, long long stride, int rows_valid) {
    constexpr int CH = D / 8;
    for (int i = threadIdx.x; i < ROWS * CH; i += THREADS) {
        const int r = i / CH, c = i % CH;
        const bool ok = r < rows_valid;
        cp_async16(smem_base + tile_off<D>(r, c), g + (ok ? (long long)r * stride + c * 8 : 0), ok);
    }
}

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A fragment (16 rows x 16 k) of a row-major tile: rows row0.., k-chunks 2*ks, 2*ks+1.
template <int D>
__device__ __forceinline__ void load_a(uint32_t base, int row0, int ks, uint32_t* a) {
    const int l = threadIdx.x & 31;
    ldsm4(base + tile_off<D>(row0 + (l & 7) + ((l >> 3) & 1) * 8, ks * 2 + (l >> 4)), a[0], a[1], a[2], a[3]);
}
// A fragment of the TRANSPOSE of a row-major tile T[k][m]: A(m, k) = T[k][m]; m-chunk = mrow0/8.., k rows k0..k0+15.
template <int D>
__device__ __forceinline__ void load_a_t(uint32_t base, int k0, int mchunk, uint32_t* a) {
    const int l = threadIdx.x & 31;
    // matrices: (k 0-7, m lo) -> a0, (k 0-7, m hi) -> a1 ... after .trans each holds (m rows, k cols)
    ldsm4_t(base + tile_off<D>(k0 + (l & 7) + (l >> 4) * 8, mchunk + ((l >> 3) & 1)), a[0], a[1], a[2], a[3]);
}
// B fragments for two n-blocks from a tile stored [n][k] (B is "col"): n rows n0..n0+15, k-chunks 2*ks, 2*ks+1.
template <int D>
__device__ __forceinline__ void load_b(uint32_t base, int n0, int ks, uint32_t* b) {
    const int l = threadIdx.x & 31;
    ldsm4(base + tile_off<D>(n0 + (l & 7) + (l >> 4) * 8, ks * 2 + ((l >> 3) & 1)), b[0], b[1], b[2], b[3]);
}
// B fragments for two n-blocks from a tile stored [k][n]: k rows k0..k0+15, n-chunks nc, nc+1.
template <int D>
__device__ __forceinline__ void load_b_t(uint32_t base, int k0, int nc, uint32_t* b) {
    const int l = threadIdx.x & 31;
    ldsm4_t(base + tile_off<D>(k0 + (l & 7) + ((l >> 3) & 1) * 8, nc + (l >> 4)), b[0], b[1], b[2], b[3]);
}

}  // namespace fa
}  // namespace ptb
