// FlashAttention forward and backward for training: causal or full, grouped-query
// heads, head_dim 64 or 128, bf16 in/out, fp32 softmax statistics.
//
// Layout [B, T, heads, D] (the reference's kernel uses the same,
// aten/src/ATen/cuda/FlashAttention.cu:83-258, but is fp32 SIMT with one thread
// per K/V row in the backward and atomics on dQ, :356-483).
//
// Forward: one CTA per 64 query rows of one head; K/V tiles of 64 rows stream
// through a double-buffered cp.async ring; S = QK^T and O += PV on tensor cores
// with the online softmax in registers; writes O and the log-sum-exp.
// Backward: one CTA per 64 K/V rows of one KV head; it loops over the query
// heads of the group and their query tiles, recomputes P from the saved
// log-sum-exp, accumulates dK/dV in registers (so the GQA reduction needs no
// atomics) and adds its dQ contribution with fp32 atomics.
#include "flash_attn.cuh"

namespace ptb {
namespace fa {

struct FwdParams {
    const __nv_bfloat16 *q, *k, *v;
    __nv_bfloat16* o;
    float* lse;                 // [B, H, Tq]
    int B, Tq, Tk, H, Hk, causal, q_offset;
    float scale_log2;           // softmax scale * log2(e)
};

template <int D>
__global__ void __launch_bounds__(THREADS) fwd_kernel(const __grid_constant__ FwdParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TILE = BC * D * 2;
    const uint32_t sQ = smem_u32(smem), sK = sQ + BR * D * 2, sV = sK + 2 * TILE;
    const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (P.H / P.Hk);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int q0 = qt * BR;
    const long long qs = (long long)P.H * D, ks = (long long)P.Hk * D;
    const __nv_bfloat16* qp = P.q + ((long long)b * P.Tq + q0) * qs + (long long)h * D;
    const __nv_bfloat16* kp = P.k + (long long)b * P.Tk * ks + (long long)hk * D;
    const __nv_bfloat16* vp = P.v + (long long)b * P.Tk * ks + (long long)hk * D;

    int ntiles = (P.Tk + BC - 1) / BC;
    if (P.causal) ntiles = min(ntiles, (P.q_offset + q0 + BR - 1) / BC + 1);

    load_tile<D, BR>(sQ, qp, qs, P.Tq - q0);
    load_tile<D, BC>(sK, kp, ks, P.Tk);
    load_tile<D, BC>(sV, vp, ks, P.Tk);
    cp_async_commit();

    uint32_t qa[D / 16][4];
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int qrow0 = P.q_offset + q0 + warp * 16 + g, qrow1 = qrow0 + 8;

    for (int j = 0; j < ntiles; ++j) {
        const int buf = j & 1;
        if (j + 1 < ntiles) {
            const int kv1 = (j + 1) * BC;
            load_tile<D, BC>(sK + (buf ^ 1) * TILE, kp + (long long)kv1 * ks, ks, P.Tk - kv1);
            load_tile<D, BC>(sV + (buf ^ 1) * TILE, vp + (long long)kv1 * ks, ks, P.Tk - kv1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (j == 0) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) load_a<D>(sQ, warp * 16, kk, qa[kk]);
        }
        // ---- S = Q K^T for this warp's 16 rows x 64 kv columns
        float s[BC / 8][4];
#pragma unroll
        for (int nb = 0; nb < BC / 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
        const uint32_t kb = sK + buf * TILE, vb = sV + buf * TILE;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int nb = 0; nb < BC / 8; nb += 2) {
                uint32_t bfr[4];
                load_b<D>(kb, nb * 8, kk, bfr);
                mma16816(s[nb], qa[kk], bfr[0], bfr[1]);
                mma16816(s[nb + 1], qa[kk], bfr[2], bfr[3]);
            }
        }
        // ---- scale, mask, online softmax
        const int kv0 = j * BC;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < BC / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int col = kv0 + nb * 8 + 2 * t + (e & 1);
                const int row = (e < 2) ? qrow0 : qrow1;
                float v = s[nb][e] * P.scale_log2;
                if (col >= P.Tk || (P.causal && col > row)) v = -INFINITY;
                s[nb][e] = v;
                if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        const float c0 = exp2f(m0 - mu0), c1 = exp2f(m1 - mu1);
        m0 = mn0; m1 = mn1;
        l0 *= c0; l1 *= c1;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
#pragma unroll
        for (int nb = 0; nb < BC / 8; ++nb) {
            s[nb][0] = exp2f(s[nb][0] - mu0); s[nb][1] = exp2f(s[nb][1] - mu0);
            s[nb][2] = exp2f(s[nb][2] - mu1); s[nb][3] = exp2f(s[nb][3] - mu1);
            l0 += s[nb][0] + s[nb][1];
            l1 += s[nb][2] + s[nb][3];
        }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < BC / 16; ++kk) {
            uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                              pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
            for (int db = 0; db < D / 8; db += 2) {
                uint32_t bfr[4];
                load_b_t<D>(vb, kk * 16, db, bfr);
                mma16816(o[db], pa, bfr[0], bfr[1]);
                mma16816(o[db + 1], pa, bfr[2], bfr[3]);
            }
        }
        __syncthreads();
    }
    // ---- finalize
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
    __nv_bfloat16* op = P.o + ((long long)b * P.Tq) * qs + (long long)h * D;
#pragma unroll
    for (int db = 0; db < D / 8; ++db) {
        const int col = db * 8 + 2 * t;
        if (r0 < P.Tq) *reinterpret_cast<uint32_t*>(op + (long long)r0 * qs + col) = pack_bf16(o[db][0] * i0, o[db][1] * i0);
        if (r1 < P.Tq) *reinterpret_cast<uint32_t*>(op + (long long)r1 * qs + col) = pack_bf16(o[db][2] * i1, o[db][3] * i1);
    }
    if (t == 0) {
        float* lp = P.lse + ((long long)b * P.H + h) * P.Tq;
        const float ln2 = 0.6931471805599453f;
        if (r0 < P.Tq) lp[r0] = l0 > 0.f ? m0 * ln2 + logf(l0) : -INFINITY;
        if (r1 < P.Tq) lp[r1] = l1 > 0.f ? m1 * ln2 + logf(l1) : -INFINITY;
    }
}

// delta[b,h,t] = sum_d dO * O
template <int D>
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                             long long rows, int H, int Tq, float* __restrict__ dq_zero = nullptr) {
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;     // one warp per (b, t, h) row
    const int lane = threadIdx.x & 31;
    if (w >= rows) return;
    const __nv_bfloat16* op = o + w * D;
    const __nv_bfloat16* dp = dout + w * D;
    if (dq_zero) {          // the fp32 dQ accumulator has the same [B, Tq, H, D] rows: clear this one on the way
        for (int i = lane * 4; i < D; i += 128) *reinterpret_cast<float4*>(dq_zero + w * D + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float s = 0.f;
    for (int i = lane * 2; i < D; i += 64) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(op + i));
        const float2 b2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dp + i));
        s += a.x * b2.x + a.y * b2.y;
    }
    s = warp_sum(s);
    if (lane == 0) {
        const long long bt = w / H;
        const int h = (int)(w % H);
        const long long b = bt / Tq;
        const int tq = (int)(bt % Tq);
        delta[(b * H + h) * Tq + tq] = s;
    }
}

struct BwdParams {
    const __nv_bfloat16 *q, *k, *v, *dout;
    const float *lse, *delta;
    float* dq;                  // fp32 [B, Tq, H, D], zero-initialised, accumulated with atomics
    __nv_bfloat16 *dk, *dv;
    int B, Tq, Tk, H, Hk, causal, q_offset;
    float scale, scale_log2;
};

// One CTA per (kv tile, kv head, batch); each warp owns 16 of the 64 K/V rows.
template <int D>
__global__ void __launch_bounds__(THREADS) bwd_kernel(const __grid_constant__ BwdParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TILE = BC * D * 2;
    const uint32_t sK = smem_u32(smem), sV = sK + TILE, sQ = sV + TILE, sdO = sQ + TILE, sdS = sdO + TILE;   // sdS: [64 kv][64 q] bf16
    float* sL = reinterpret_cast<float*>(smem + 4 * TILE + BC * BR * 2);      // lse[64], delta[64]
    float* sDl = sL + BR;
    const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int G = P.H / P.Hk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kv0 = kt * BC;
    const long long qs = (long long)P.H * D, ks = (long long)P.Hk * D;
    const __nv_bfloat16* kp = P.k + ((long long)b * P.Tk + kv0) * ks + (long long)hk * D;
    const __nv_bfloat16* vp = P.v + ((long long)b * P.Tk + kv0) * ks + (long long)hk * D;
    load_tile<D, BC>(sK, kp, ks, P.Tk - kv0);
    load_tile<D, BC>(sV, vp, ks, P.Tk - kv0);
    cp_async_commit();

    float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f; dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f; }
    const int krow0 = kv0 + warp * 16 + g, krow1 = krow0 + 8;

    const int nq_tiles = (P.Tq + BR - 1) / BR;
    int first_q = 0;
    if (P.causal) first_q = max(0, (kv0 - P.q_offset) / BR);       // query tiles entirely before this kv tile see none of it
    for (int hh = 0; hh < G; ++hh) {
        const int h = hk * G + hh;
        for (int qt = first_q; qt < nq_tiles; ++qt) {
            const int q0 = qt * BR;
            __syncthreads();                                        // previous iteration is done with sQ/sdO/sdS/sL
            load_tile<D, BR>(sQ, P.q + ((long long)b * P.Tq + q0) * qs + (long long)h * D, qs, P.Tq - q0);
            load_tile<D, BR>(sdO, P.dout + ((long long)b * P.Tq + q0) * qs + (long long)h * D, qs, P.Tq - q0);
            cp_async_commit();
            if (threadIdx.x < BR) {
                const int r = q0 + threadIdx.x;
                const long long ix = ((long long)b * P.H + h) * P.Tq + r;
                sL[threadIdx.x] = r < P.Tq ? P.lse[ix] * 1.4426950408889634f : INFINITY;   // +inf => P = 0 for padded rows
                sDl[threadIdx.x] = r < P.Tq ? P.delta[ix] : 0.f;
            }
            cp_async_wait<0>();
            __syncthreads();
            // ---- S^T[kv 16 x q 64] = K Q^T ; dP^T = V dO^T
            float st[BR / 8][4], dp[BR / 8][4];
#pragma unroll
            for (int nb = 0; nb < BR / 8; ++nb) { st[nb][0] = st[nb][1] = st[nb][2] = st[nb][3] = 0.f; dp[nb][0] = dp[nb][1] = dp[nb][2] = dp[nb][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t ka[4], va[4];
                load_a<D>(sK, warp * 16, kk, ka);
                load_a<D>(sV, warp * 16, kk, va);
#pragma unroll
                for (int nb = 0; nb < BR / 8; nb += 2) {
                    uint32_t bq[4], bo[4];
                    load_b<D>(sQ, nb * 8, kk, bq);
                    load_b<D>(sdO, nb * 8, kk, bo);
                    mma16816(st[nb], ka, bq[0], bq[1]);
                    mma16816(st[nb + 1], ka, bq[2], bq[3]);
                    mma16816(dp[nb], va, bo[0], bo[1]);
                    mma16816(dp[nb + 1], va, bo[2], bo[3]);
                }
            }
            // ---- P^T = exp2(S^T*c - lse), dS^T = P^T (dP^T - delta) * scale
#pragma unroll
            for (int nb = 0; nb < BR / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int qc = nb * 8 + 2 * t + (e & 1);            // query column inside the tile
                    const int krow = (e < 2) ? krow0 : krow1;
                    const int qrow = P.q_offset + q0 + qc;
                    float p = exp2f(st[nb][e] * P.scale_log2 - sL[qc]);
                    if (krow >= P.Tk || (P.causal && krow > qrow)) p = 0.f;
                    st[nb][e] = p;
                    dp[nb][e] = p * (dp[nb][e] - sDl[qc]) * P.scale;
                }
            }
            // ---- dV += P^T dO ; dK += dS^T Q   (A from registers, B = dO / Q read transposed: B(k=q, n=d))
#pragma unroll
            for (int kk = 0; kk < BR / 16; ++kk) {
                uint32_t pa[4] = {pack_bf16(st[2 * kk][0], st[2 * kk][1]), pack_bf16(st[2 * kk][2], st[2 * kk][3]),
                                  pack_bf16(st[2 * kk + 1][0], st[2 * kk + 1][1]), pack_bf16(st[2 * kk + 1][2], st[2 * kk + 1][3])};
                uint32_t da[4] = {pack_bf16(dp[2 * kk][0], dp[2 * kk][1]), pack_bf16(dp[2 * kk][2], dp[2 * kk][3]),
                                  pack_bf16(dp[2 * kk + 1][0], dp[2 * kk + 1][1]), pack_bf16(dp[2 * kk + 1][2], dp[2 * kk + 1][3])};
#pragma unroll
                for (int db = 0; db < D / 8; db += 2) {
                    uint32_t bo[4], bq[4];
                    load_b_t<D>(sdO, kk * 16, db, bo);
                    load_b_t<D>(sQ, kk * 16, db, bq);
                    mma16816(dv[db], pa, bo[0], bo[1]);
                    mma16816(dv[db + 1], pa, bo[2], bo[3]);
                    mma16816(dk[db], da, bq[0], bq[1]);
                    mma16816(dk[db + 1], da, bq[2], bq[3]);
                }
            }
            // ---- stage dS^T (bf16) [kv][q] so that every warp can read all 64 kv rows of it
#pragma unroll
            for (int nb = 0; nb < BR / 8; ++nb) {
                const int c = nb * 8 + 2 * t;
                const int r0 = warp * 16 + g, r1 = r0 + 8;
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(sdS + tile_off<BR>(r0, c >> 3) + (c & 7) * 2), "r"(pack_bf16(dp[nb][0], dp[nb][1])));
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(sdS + tile_off<BR>(r1, c >> 3) + (c & 7) * 2), "r"(pack_bf16(dp[nb][2], dp[nb][3])));
            }
            __syncthreads();
            // ---- dQ[16 q rows of this warp, D] = dS[q, kv 64] K[kv 64, D], added to global with fp32 atomics
            float* dqp = P.dq + ((long long)b * P.Tq + q0) * qs + (long long)h * D;
#pragma unroll
            for (int dh = 0; dh < D / 64; ++dh) {                  // 64 columns of D at a time keeps registers in check
                float dq[8][4];
#pragma unroll
                for (int i = 0; i < 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
#pragma unroll
                for (int kk = 0; kk < BC / 16; ++kk) {
                    uint32_t a[4];
                    load_a_t<BR>(sdS, kk * 16, warp * 2, a);       // A(m = q, k = kv) = dS^T[kv][q]
#pragma unroll
                    for (int db = 0; db < 8; db += 2) {
                        uint32_t bk[4];
                        load_b_t<D>(sK, kk * 16, dh * 8 + db, bk);  // B(k = kv, n = d) = K[kv][d]
                        mma16816(dq[db], a, bk[0], bk[1]);
                        mma16816(dq[db + 1], a, bk[2], bk[3]);
                    }
                }
                const int r0 = warp * 16 + g, r1 = r0 + 8;
#pragma unroll
                for (int db = 0; db < 8; ++db) {
                    const int col = dh * 64 + db * 8 + 2 * t;
                    if (q0 + r0 < P.Tq) { atomicAdd(dqp + (long long)r0 * qs + col, dq[db][0]); atomicAdd(dqp + (long long)r0 * qs + col + 1, dq[db][1]); }
                    if (q0 + r1 < P.Tq) { atomicAdd(dqp + (long long)r1 * qs + col, dq[db][2]); atomicAdd(dqp + (long long)r1 * qs + col + 1, dq[db][3]); }
                }
            }
        }
    }
    // ---- write dK, dV for this warp's 16 kv rows
    __nv_bfloat16* dkp = P.dk + ((long long)b * P.Tk) * ks + (long long)hk * D;
    __nv_bfloat16* dvp = P.dv + ((long long)b * P.Tk) * ks + (long long)hk * D;
#pragma unroll
    for (int db = 0; db < D / 8; ++db) {
        const int col = db * 8 + 2 * t;
        if (krow0 < P.Tk) {
            *reinterpret_cast<uint32_t*>(dkp + (long long)krow0 * ks + col) = pack_bf16(dk[db][0], dk[db][1]);
            *reinterpret_cast<uint32_t*>(dvp + (long long)krow0 * ks + col) = pack_bf16(dv[db][0], dv[db][1]);
        }
        if (krow1 < P.Tk) {
            *reinterpret_cast<uint32_t*>(dkp + (long long)krow1 * ks + col) = pack_bf16(dk[db][2], dk[db][3]);
            *reinterpret_cast<uint32_t*>(dvp + (long long)krow1 * ks + col) = pack_bf16(dv[db][2], dv[db][3]);
        }
    }
}

}  // namespace fa
}  // namespace ptb

using namespace ptb;
using namespace ptb::fa;

template <int D>
static int run_fwd(const FwdParams& p, cudaStream_t st) {
    constexpr int smem = BR * D * 2 + 4 * BC * D * 2;
    static bool attr = false;
    if (!attr) { PTB_CUDA_OK(cudaFuncSetAttribute(fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); attr = true; }
    dim3 grid((p.Tq + BR - 1) / BR, p.H, p.B);
    fwd_kernel<D><<<grid, THREADS, smem, st>>>(p);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

PTB_API int ptb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Tq, int Tk, int H, int Hk,
                               int D, int causal, float scale, int q_offset, cudaStream_t st) {
    if ((D != 64 && D != 128) || H % Hk) { ptb_set_error("flash attention: head_dim %d / heads %d over %d not supported", D, H, Hk); return -1; }
    FwdParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)o, lse, B, Tq, Tk, H, Hk,
                causal, q_offset, scale * 1.4426950408889634f};
    return D == 64 ? run_fwd<64>(p, st) : run_fwd<128>(p, st);
}

template <int D>
static int run_bwd(const BwdParams& p, const void* o, cudaStream_t st) {
    const long long rows = (long long)p.B * p.Tq * p.H;
    delta_kernel<D><<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)o, p.dout, const_cast<float*>(p.delta), rows, p.H, p.Tq);
    constexpr int smem = 4 * BC * D * 2 + BC * BR * 2 + 2 * BR * 4;
    static bool attr = false;
    if (!attr) { PTB_CUDA_OK(cudaFuncSetAttribute(bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); attr = true; }
    dim3 grid((p.Tk + BC - 1) / BC, p.Hk, p.B);
    bwd_kernel<D><<<grid, THREADS, smem, st>>>(p);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// delta[b, h, t] = sum_d dO * O (fp32 [B, H, Tq]): the row term of the softmax backward.  dq_zero (optional): an fp32
// [B, Tq, H, D] buffer cleared in the same pass (the dQ accumulator of the backward kernel).
PTB_API int ptb_flash_attn_delta(const void* o, const void* dout, float* delta, int B, int Tq, int H, int D, float* dq_zero, cudaStream_t st) {
    const long long rows = (long long)B * Tq * H;
    if (rows == 0) return 0;
    const unsigned grid = (unsigned)((rows * 32 + 255) / 256);
    if (D == 64) delta_kernel<64><<<grid, 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, rows, H, Tq, dq_zero);
    else if (D == 128) delta_kernel<128><<<grid, 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, rows, H, Tq, dq_zero);
    else { ptb_set_error("flash attention: head_dim %d not supported", D); return -1; }
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// dq: fp32 [B,Tq,H,D] zero-initialised by the caller; delta: fp32 [B,H,Tq] scratch.
PTB_API int ptb_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                               float* delta, float* dq, void* dk, void* dv, void* unused, int B, int Tq, int Tk, int H, int Hk, int D,
                               int causal, float scale, int q_offset, cudaStream_t st) {
    (void)unused;
    if ((D != 64 && D != 128) || H % Hk) { ptb_set_error("flash attention: head_dim %d / heads %d over %d not supported", D, H, Hk); return -1; }
    BwdParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)dout, lse, delta, dq,
                (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, B, Tq, Tk, H, Hk, causal, q_offset, scale, scale * 1.4426950408889634f};
    return D == 64 ? run_bwd<64>(p, o, st) : run_bwd<128>(p, o, st);
}
