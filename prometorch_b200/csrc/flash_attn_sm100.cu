// FlashAttention forward on the 5th-generation tensor cores: both products of every 128 x 128 block run as
// tcgen05.mma with accumulators in tensor memory, operands arrive by TMA.
//
// One CTA per (128 query rows, head, batch).  Ten warps:
//   warp 8   TMA producer: the Q tile once, then K and V tiles of 128 keys through two-stage rings;
//   warp 9   owns tensor memory and issues the MMAs: S(j) = Q K_j^T into one of two 128-column buffers,
//            then O_j = P_j V_j into a third buffer once the softmax warps have written P_j;
//   warps 0-7  softmax.  A thread owns one query row (its tensor-memory lane) and half of the block's
//            columns: it reads its 64 scores with tcgen05.ld, exchanges the row maximum with its partner
//            thread through shared memory, writes the bf16 probabilities into a 128-byte-swizzled
//            shared-memory tile (the A operand of the second product) and keeps its half of the output
//            row in registers, rescaled by the running maximum.  The read-back of O_{j-1} is deferred
//            until after the scores of block j have been reduced, so that it overlaps the MMA of P_{j-1} V.
// Causal masking and the sequence end are applied to the blocks that need them only.  Every wait is
// bounded.  The reference's kernel is aten/src/ATen/cuda/FlashAttention.cu:83-258 (one thread per row).
#include "gemm_sm100.cuh"

int ptb_make_tmap_bf16(CUtensorMap* map, const void* base, long long inner, long long outer, long long ld, int box_inner, int box_outer);

namespace ptb {
namespace fa100 {

using namespace ptb::gemm;

constexpr int BQ = 128, BKV = 128;
constexpr int NTHREADS = 320;

struct Params {
    __nv_bfloat16* O;        // [B, Tq, H, D]
    float* lse;              // [B, H, Tq] natural-log sum of exponentials
    int B, Tq, Tk, H, Hk;
    int causal, q_offset;
    float scale_log2;        // softmax scale x log2(e)
    int* status;
};

template <int D>
struct Sm {
    static constexpr int Q_BYTES = BQ * D * 2;
    static constexpr int KV_BYTES = BKV * D * 2;
    static constexpr int P_BYTES = BQ * BKV * 2;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + Q_BYTES;
    static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
    static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
    static constexpr int OFF_RED = OFF_P + P_BYTES;          // 2 x 128 floats
    static constexpr int OFF_BAR = OFF_RED + 2 * BQ * 4;
    static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(NTHREADS, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
           const __grid_constant__ Params P) {
    using S = Sm<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sq = smem + S::OFF_Q;
    uint8_t* sk = smem + S::OFF_K;
    uint8_t* sv = smem + S::OFF_V;
    uint8_t* sp = smem + S::OFF_P;
    float* red = reinterpret_cast<float*>(smem + S::OFF_RED);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
    uint64_t* q_full = bars;             // [1]
    uint64_t* k_full = bars + 1;         // [2]
    uint64_t* k_empty = bars + 3;        // [2]
    uint64_t* v_full = bars + 5;         // [2]
    uint64_t* v_empty = bars + 7;        // [2]
    uint64_t* s_full = bars + 9;         // [2]
    uint64_t* p_ready = bars + 11;       // [1], 8 arrivals (one per softmax warp)
    uint64_t* o_full = bars + 12;        // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;           // long (late) query blocks first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (P.H / P.Hk);
    const int q0 = qb * BQ;
    // keys this block can see: [0, kv_end)
    const int kv_end = P.causal ? min(P.Tk, q0 + BQ + P.q_offset) : P.Tk;
    const int nblk = max(0, (kv_end + BKV - 1) / BKV);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); mbar_init(&s_full[s], 1); }
        mbar_init(p_ready, 8);
        mbar_init(o_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmV);
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t TM_S = 0, TM_O = 256;                           // column offsets: S buffers at 0 and 128, O_j at 256

    if (warp == 8) {
        // ---------------------------------------------------------------------------- TMA producer
        if (lane == 0 && nblk > 0) {
            bool ok = true;
            mbar_expect_tx(q_full, S::Q_BYTES);
            for (int kb = 0; kb < D / 64; ++kb) tma_load_2d(sq + kb * (BQ * 128), &tmQ, h * D + kb * 64, b * P.Tq + q0, q_full);
            for (int j = 0; j < nblk && ok; ++j) {
                const int s = j & 1;
                if (j >= 2) ok = mbar_wait(&k_empty[s], (uint32_t)(((j >> 1) - 1) & 1), P.status);
                if (!ok) break;
                mbar_expect_tx(&k_full[s], S::KV_BYTES);
                for (int kb = 0; kb < D / 64; ++kb)
                    tma_load_2d(sk + s * S::KV_BYTES + kb * (BKV * 128), &tmK, hk * D + kb * 64, b * P.Tk + j * BKV, &k_full[s]);
                if (j >= 2) ok = mbar_wait(&v_empty[s], (uint32_t)(((j >> 1) - 1) & 1), P.status);
                if (!ok) break;
                mbar_expect_tx(&v_full[s], S::KV_BYTES);
                for (int hh = 0; hh < 2; ++hh)                       // two halves of 64 keys, each D/64 chunks of [64 keys x 64 dims]
                    for (int c = 0; c < D / 64; ++c)
                        tma_load_2d(sv + s * S::KV_BYTES + hh * (D / 64) * 8192 + c * 8192, &tmV, hk * D + c * 64, b * P.Tk + j * BKV + hh * 64,
                                    &v_full[s]);
            }
            if (!ok) *abort_flag = 1;
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------------------- MMA issuer
        if (lane == 0 && nblk > 0) {
            constexpr uint32_t idesc_s = instr_desc(BQ, BKV, 0, 0);          // S = Q K^T: both K-major
            constexpr uint32_t idesc_o = instr_desc(BQ, D, 0, 1);            // O = P V: P K-major, V MN-major
            bool ok = mbar_wait(q_full, 0, P.status);
            auto issue_s = [&](int j) {
                const int s = j & 1;
                if (!mbar_wait(&k_full[s], (uint32_t)((j >> 1) & 1), P.status)) return false;
                tc_fence_after();
                const uint32_t a0 = smem_u32(sq), b0 = smem_u32(sk + s * S::KV_BYTES);
#pragma unroll
                for (int kb = 0; kb < D / 64; ++kb)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base + TM_S + (uint32_t)(s * BKV), smem_desc(a0 + kb * (BQ * 128) + k * 32, 16, 1024),
                                  smem_desc(b0 + kb * (BKV * 128) + k * 32, 16, 1024), idesc_s, (kb > 0 || k > 0) ? 1u : 0u);
                umma_commit(&k_empty[s]);
                umma_commit(&s_full[s]);
                return true;
            };
            if (ok) ok = issue_s(0);
            if (ok && nblk > 1) ok = issue_s(1);
            for (int j = 0; j < nblk && ok; ++j) {
                const int s = j & 1;
                ok = mbar_wait(p_ready, (uint32_t)(j & 1), P.status);        // P_j is in shared memory, O_{j-1} has been read
                if (ok) ok = mbar_wait(&v_full[s], (uint32_t)((j >> 1) & 1), P.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a0 = smem_u32(sp), b0 = smem_u32(sv + s * S::KV_BYTES);
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base + TM_O, smem_desc(a0 + hh * (BQ * 128) + k * 32, 16, 1024),
                                  smem_desc(b0 + hh * (D / 64) * 8192 + k * 2048, 8192, 1024), idesc_o, (hh > 0 || k > 0) ? 1u : 0u);
                umma_commit(&v_empty[s]);
                umma_commit(o_full);
                if (j + 2 < nblk) ok = issue_s(j + 2);
            }
            if (!ok) *abort_flag = 1;
        }
    } else {
        // ---------------------------------------------------------------------------- softmax warps
        const int row = 32 * (warp & 3) + lane;          // query row inside the block = tensor-memory lane
        const int hf = warp >> 2;                        // which 64 columns of S, which D/2 columns of O
        const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16);
        const int q_pos = q0 + row + P.q_offset;         // position of this query among the keys
        float o_acc[D / 2];
#pragma unroll
        for (int i = 0; i < D / 2; ++i) o_acc[i] = 0.f;
        float m_run = -INFINITY, l_part = 0.f, alpha_prev = 1.f;
        bool ok = true;
        auto add_o = [&](float alpha) {                  // o_acc = o_acc * alpha + (my half of the row of O_j)
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
                uint32_t r[32];
                tmem_ld32(lane_addr + TM_O + (uint32_t)(hf * (D / 2) + c * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(r[i]);
            }
        };
        for (int j = 0; j < nblk; ++j) {
            const int s = j & 1;
            if (ok && !*abort_flag) ok = mbar_wait(&s_full[s], (uint32_t)((j >> 1) & 1), P.status);
            else ok = false;
            tc_fence_after();
            float sc[64];
            {
                uint32_t r[32];
                tmem_ld32(lane_addr + TM_S + (uint32_t)(s * BKV + hf * 64), r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) sc[i] = __uint_as_float(r[i]) * P.scale_log2;
                tmem_ld32(lane_addr + TM_S + (uint32_t)(s * BKV + hf * 64 + 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) sc[32 + i] = __uint_as_float(r[i]) * P.scale_log2;
            }
            const int key0 = j * BKV + hf * 64;
            const bool need_mask = (key0 + 64 > P.Tk) || (P.causal && key0 + 63 > q0 + P.q_offset);
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int key = key0 + i;
                    if (key >= P.Tk || (P.causal && key > q_pos)) sc[i] = -INFINITY;
                }
            }
            // eight independent partial maxima: a 64-long dependent chain would stall the two warps a scheduler has
            float m8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) m8[i] = sc[i];
#pragma unroll
            for (int i = 8; i < 64; ++i) m8[i & 7] = fmaxf(m8[i & 7], sc[i]);
            const float mx = fmaxf(fmaxf(fmaxf(m8[0], m8[1]), fmaxf(m8[2], m8[3])), fmaxf(fmaxf(m8[4], m8[5]), fmaxf(m8[6], m8[7])));
            red[hf * BQ + row] = mx;
            softmax_sync();
            const float m_blk = fmaxf(red[row], red[BQ + row]);
            const float m_new = fmaxf(m_run, m_blk);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = exp2f(m_run - m_use);
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float p0 = exp2f(sc[2 * i] - m_use), p1 = exp2f(sc[2 * i + 1] - m_use);
                l4[i & 3] += p0 + p1;
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                pk[i] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            l_part = l_part * alpha + ((l4[0] + l4[1]) + (l4[2] + l4[3]));
            m_run = m_new;
            // the deferred read-back of O_{j-1}; its MMA ran while the scores above were reduced
            if (j > 0) {
                if (ok) ok = mbar_wait(o_full, (uint32_t)((j - 1) & 1), P.status);
                tc_fence_after();
                add_o(alpha_prev);
            }
            alpha_prev = alpha;
            // P_j -> shared memory, K-major with the 128-byte swizzle: sub-tile hf, row `row`, 16-byte chunk c at c ^ (row & 7)
            {
                uint8_t* prow = sp + hf * (BQ * 128) + row * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) * 16)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            }
            fence_proxy_async();
            tc_fence_before();
            softmax_sync();                   // also keeps `red` from being overwritten before both partners have read it
            if (lane == 0) mbar_arrive(p_ready);
        }
        if (nblk > 0) {
            if (ok) ok = mbar_wait(o_full, (uint32_t)((nblk - 1) & 1), P.status);
            tc_fence_after();
            add_o(alpha_prev);
        }
        red[hf * BQ + row] = l_part;
        softmax_sync();
        const float l = red[row] + red[BQ + row];
        const int q_idx = q0 + row;
        if (q_idx < P.Tq && ok) {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __nv_bfloat16* op = P.O + (((size_t)b * P.Tq + q_idx) * P.H + h) * D + hf * (D / 2);
#pragma unroll
            for (int i = 0; i < D / 2; i += 8) {
                uint4 o;
                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(o_acc[i + 2 * e] * inv, o_acc[i + 2 * e + 1] * inv);
                *reinterpret_cast<uint4*>(op + i) = o;
            }
            if (hf == 0) P.lse[((size_t)b * P.H + h) * P.Tq + q_idx] = l > 0.f ? m_run * 0.6931471805599453f + logf(l) : -INFINITY;
        }
        if (!ok) *abort_flag = 1;
    }
    // ---- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem_base, 512);
}

template <int D>
static int launch(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Tq, int Tk, int H, int Hk, int causal,
                  float scale, int q_offset, int* status, cudaStream_t st) {
    CUtensorMap mq, mk, mv;
    if (ptb_make_tmap_bf16(&mq, q, (long long)H * D, (long long)B * Tq, (long long)H * D, 64, BQ)) return -1;
    if (ptb_make_tmap_bf16(&mk, k, (long long)Hk * D, (long long)B * Tk, (long long)Hk * D, 64, BKV)) return -1;
    if (ptb_make_tmap_bf16(&mv, v, (long long)Hk * D, (long long)B * Tk, (long long)Hk * D, 64, 64)) return -1;
    static bool attr = false;
    if (!attr) {
        PTB_CUDA_OK(cudaFuncSetAttribute(fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Sm<D>::TOTAL));
        attr = true;
    }
    Params p;
    p.O = (__nv_bfloat16*)o; p.lse = lse; p.B = B; p.Tq = Tq; p.Tk = Tk; p.H = H; p.Hk = Hk; p.causal = causal; p.q_offset = q_offset;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    dim3 grid((Tq + BQ - 1) / BQ, H, B);
    fwd_kernel<D><<<grid, NTHREADS, Sm<D>::TOTAL, st>>>(mq, mk, mv, p);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}


// ---------------------------------------------------------------------------------------------- backward
// One CTA per (128 keys, KV head, batch); it keeps K_j and V_j in shared memory and dK_j, dV_j in tensor memory, and
// walks the query blocks that see those keys (all query heads of the KV head's group).  Per query block i:
//   S = Q_i K_j^T and dP = dO_i V_j^T               two tcgen05.mma groups into TMEM (128 columns each)
//   P = exp2(S c - lse_i),  dS = P (dP - delta_i) scale   by the thread that owns the query row (= TMEM lane)
//   dV_j += P^T dO_i,  dK_j += dS^T Q_i,  dQ_i = dS K_j   three groups; dQ_i lands in S's columns, is read back
//                                                       and added to the fp32 dQ in global memory (vector red)
// Every tile lives in shared memory in ONE layout, [64-column chunk][row][128 B, 128-byte swizzle], which the
// descriptors read as a K-major operand (rows = M or N) or as an MN-major operand (rows = K): Q_i is the A operand
// of S and the B operand of dK, dO_i the A operand of dP and the B operand of dV, K_j the B operand of S and of dQ,
// and the P / dS tiles written by the threads are A operands in both orientations.
struct BwdParams {
    const float* lse;        // [B, H, Tq] natural log
    const float* delta;      // [B, H, Tq]
    float* dq;               // [B, Tq, H, D] fp32, zero-initialised
    __nv_bfloat16* dk;       // [B, Tk, Hk, D]
    __nv_bfloat16* dv;
    int B, Tq, Tk, H, Hk;
    int causal, q_offset;
    float scale, scale_log2;
    int* status;
    int gsplit;              // CTAs per KV head: each takes group / gsplit query heads and writes its own dk / dv slice
};

template <int D>
struct SmB {
    static constexpr int TILE = 128 * D * 2;                 // K, V, Q, dO
    static constexpr int PT = 128 * 128 * 2;                 // P, dS
    static constexpr int NST = D == 64 ? 2 : 1;              // Q_i / dO_i stages: two where shared memory allows
    static constexpr int OFF_K = 0;
    static constexpr int OFF_V = OFF_K + TILE;
    static constexpr int OFF_Q = OFF_V + TILE;
    static constexpr int OFF_DO = OFF_Q + NST * TILE;
    static constexpr int OFF_P = OFF_DO + NST * TILE;
    static constexpr int OFF_DS = OFF_P + PT;
    static constexpr int OFF_BAR = OFF_DS + PT;
    static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int D>
__global__ void __launch_bounds__(NTHREADS, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
           const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ BwdParams P) {
    using S = SmB<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sk = smem + S::OFF_K;
    uint8_t* sv = smem + S::OFF_V;
    uint8_t* sq = smem + S::OFF_Q;
    uint8_t* sdo = smem + S::OFF_DO;
    uint8_t* sp = smem + S::OFF_P;
    uint8_t* sds = smem + S::OFF_DS;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
    constexpr int NST = S::NST;
    uint64_t* kv_full = bars;            // K_j, V_j loaded (once)
    uint64_t* qdo_full = bars + 1;       // [2] Q_i, dO_i loaded
    uint64_t* qdo_empty = bars + 3;      // [2] the MMAs that read them have completed
    uint64_t* sdp_full = bars + 5;       // S and dP are in TMEM
    uint64_t* pds_ready = bars + 6;      // P and dS are in shared memory (8 arrivals)
    uint64_t* dq_full = bars + 7;        // dV, dK updated, dQ_i in TMEM
    uint64_t* dq_read = bars + 8;        // dQ_i has been read back (8 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int jb = blockIdx.x, hk = blockIdx.y / P.gsplit, part = blockIdx.y % P.gsplit, b = blockIdx.z;
    const int group = (P.H / P.Hk) / P.gsplit;          // query heads this CTA walks
    const int head0 = hk * (P.H / P.Hk) + part * group;
    const int key0 = jb * 128;
    const int nq = (P.Tq + 127) / 128;
    // first query block that sees key0: rows q with q + q_offset >= key0
    const int i_start = P.causal ? max(0, (key0 - P.q_offset) / 128) : 0;
    const int per_head = max(0, nq - i_start);
    const int n_it = per_head * group;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1); mbar_init(sdp_full, 1);
        for (int st = 0; st < 2; ++st) { mbar_init(&qdo_full[st], 1); mbar_init(&qdo_empty[st], 1); }
        mbar_init(pds_ready, 8); mbar_init(dq_full, 1); mbar_init(dq_read, 8);
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 256 + D;      // dQ_i reuses S's columns

    if (warp == 8) {
        // ---------------------------------------------------------------------------- TMA producer
        if (lane == 0 && n_it > 0) {
            bool ok = true;
            mbar_expect_tx(kv_full, 2 * S::TILE);
            for (int c = 0; c < D / 64; ++c) {
                tma_load_2d(sk + c * 16384, &tmK, hk * D + c * 64, b * P.Tk + key0, kv_full);
                tma_load_2d(sv + c * 16384, &tmV, hk * D + c * 64, b * P.Tk + key0, kv_full);
            }
            for (int it = 0; it < n_it && ok; ++it) {
                const int h = head0 + it / per_head, i = i_start + it % per_head;
                const int stg = it % NST;
                if (it >= NST) ok = mbar_wait(&qdo_empty[stg], (uint32_t)(((it / NST) - 1) & 1), P.status);
                if (!ok) break;
                mbar_expect_tx(&qdo_full[stg], 2 * S::TILE);
                for (int c = 0; c < D / 64; ++c) {
                    tma_load_2d(sq + stg * S::TILE + c * 16384, &tmQ, h * D + c * 64, b * P.Tq + i * 128, &qdo_full[stg]);
                    tma_load_2d(sdo + stg * S::TILE + c * 16384, &tmDO, h * D + c * 64, b * P.Tq + i * 128, &qdo_full[stg]);
                }
            }
            if (!ok) *abort_flag = 1;
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------------------- MMA issuer
        if (lane == 0 && n_it > 0) {
            constexpr uint32_t idesc_qk = instr_desc(128, 128, 0, 0);      // S, dP: A [q, D] and B [keys, D] both K-major
            constexpr uint32_t idesc_tt = instr_desc(128, D, 1, 1);        // dV, dK: A = P / dS read MN-major, B = dO / Q MN-major
            constexpr uint32_t idesc_dq = instr_desc(128, D, 0, 1);        // dQ: A = dS K-major, B = K MN-major
            bool ok = mbar_wait(kv_full, 0, P.status);
            const uint32_t aK = smem_u32(sk), aV = smem_u32(sv), aP = smem_u32(sp), aDS = smem_u32(sds);
            for (int it = 0; it < n_it && ok; ++it) {
                const int stg = it % NST;
                const uint32_t aQ = smem_u32(sq + stg * S::TILE), aDO = smem_u32(sdo + stg * S::TILE);
                ok = mbar_wait(&qdo_full[stg], (uint32_t)((it / NST) & 1), P.status);
                if (ok && it > 0) ok = mbar_wait(dq_read, (uint32_t)((it - 1) & 1), P.status);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < D / 64; ++c)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        umma_bf16(tmem_base + TM_S, smem_desc(aQ + c * 16384 + k * 32, 16, 1024), smem_desc(aK + c * 16384 + k * 32, 16, 1024),
                                  idesc_qk, (c > 0 || k > 0) ? 1u : 0u);
                        umma_bf16(tmem_base + TM_DP, smem_desc(aDO + c * 16384 + k * 32, 16, 1024), smem_desc(aV + c * 16384 + k * 32, 16, 1024),
                                  idesc_qk, (c > 0 || k > 0) ? 1u : 0u);
                    }
                umma_commit(sdp_full);
                ok = mbar_wait(pds_ready, (uint32_t)(it & 1), P.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
                for (int kq = 0; kq < 8; ++kq) {      // K dimension = the 128 query rows, 16 per step: 2048 B further down each chunk
                    umma_bf16(tmem_base + TM_DV, smem_desc(aP + kq * 2048, 16384, 1024), smem_desc(aDO + kq * 2048, 16384, 1024), idesc_tt,
                              (kq > 0) ? 1u : acc);
                    umma_bf16(tmem_base + TM_DK, smem_desc(aDS + kq * 2048, 16384, 1024), smem_desc(aQ + kq * 2048, 16384, 1024), idesc_tt,
                              (kq > 0) ? 1u : acc);
                }
#pragma unroll
                for (int c = 0; c < 2; ++c)           // K dimension = the 128 keys: two 64-key chunks of dS, 16 keys = 32 B per step
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base + TM_S, smem_desc(aDS + c * 16384 + k * 32, 16, 1024),
                                  smem_desc(aK + (c * 4 + k) * 2048, 16384, 1024), idesc_dq, (c > 0 || k > 0) ? 1u : 0u);
                umma_commit(&qdo_empty[stg]);
                umma_commit(dq_full);
            }
            if (!ok) *abort_flag = 1;
        }
    } else {
        // ---------------------------------------------------------------------------- compute warps
        const int row = 32 * (warp & 3) + lane;          // query row of the block = TMEM lane (key row in the final read-out)
        const int hf = warp >> 2;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16);
        bool ok = true;
        for (int it = 0; it < n_it; ++it) {
            const int h = head0 + it / per_head, i = i_start + it % per_head;
            const int q_idx = i * 128 + row;
            const bool q_valid = q_idx < P.Tq;
            const size_t stat = ((size_t)b * P.H + h) * P.Tq + q_idx;
            const float lse2 = q_valid ? P.lse[stat] * 1.4426950408889634f : INFINITY;       // +inf: P = 0 for padded rows
            const float dlt = q_valid ? P.delta[stat] : 0.f;
            if (ok && !*abort_flag) ok = mbar_wait(sdp_full, (uint32_t)(it & 1), P.status);
            else ok = false;
            tc_fence_after();
            const int kbase = key0 + hf * 64;
            const int q_pos = q_idx + P.q_offset;
            const bool need_mask = (kbase + 64 > P.Tk) || (P.causal && kbase + 63 > i * 128 + P.q_offset);
            uint32_t pp[32], dd[32];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t rs[32], rd[32];
                tmem_ld32(lane_addr + TM_S + (uint32_t)(hf * 64 + c * 32), rs);
                tmem_ld32(lane_addr + TM_DP + (uint32_t)(hf * 64 + c * 32), rd);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float p0 = exp2f(__uint_as_float(rs[e]) * P.scale_log2 - lse2), p1 = exp2f(__uint_as_float(rs[e + 1]) * P.scale_log2 - lse2);
                    if (need_mask) {
                        const int k0 = kbase + c * 32 + e;
                        if (k0 >= P.Tk || (P.causal && k0 > q_pos)) p0 = 0.f;
                        if (k0 + 1 >= P.Tk || (P.causal && k0 + 1 > q_pos)) p1 = 0.f;
                    }
                    const float d0 = p0 * (__uint_as_float(rd[e]) - dlt) * P.scale, d1 = p1 * (__uint_as_float(rd[e + 1]) - dlt) * P.scale;
                    const __nv_bfloat162 ph = __floats2bfloat162_rn(p0, p1), dh = __floats2bfloat162_rn(d0, d1);
                    pp[c * 16 + e / 2] = *reinterpret_cast<const uint32_t*>(&ph);
                    dd[c * 16 + e / 2] = *reinterpret_cast<const uint32_t*>(&dh);
                }
            }
            {
                uint8_t* prow = sp + hf * 16384 + row * 128;
                uint8_t* drow = sds + hf * 16384 + row * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int off = (c ^ (row & 7)) * 16;
                    *reinterpret_cast<uint4*>(prow + off) = make_uint4(pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]);
                    *reinterpret_cast<uint4*>(drow + off) = make_uint4(dd[4 * c], dd[4 * c + 1], dd[4 * c + 2], dd[4 * c + 3]);
                }
            }
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(pds_ready);
            // ---- dQ_i: read back my half of the row and add it to global memory
            if (ok) ok = mbar_wait(dq_full, (uint32_t)(it & 1), P.status);
            tc_fence_after();
            float* dqp = P.dq + (((size_t)b * P.Tq + q_idx) * P.H + h) * D + hf * (D / 2);
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
                uint32_t r[32];
                tmem_ld32(lane_addr + TM_S + (uint32_t)(hf * (D / 2) + c * 32), r);
                tmem_ld_wait();
                if (q_valid && ok) {
#pragma unroll
                    for (int e = 0; e < 32; e += 4)
                        red_add_v4(dqp + c * 32 + e, __uint_as_float(r[e]), __uint_as_float(r[e + 1]), __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(dq_read);
        }
        // ---- dK_j, dV_j: lanes are key rows now
        const int key = key0 + row;
        if (n_it > 0 && ok && !*abort_flag) {
            tc_fence_after();
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                __nv_bfloat16* outp = (which ? P.dk : P.dv) + (size_t)part * P.B * P.Tk * P.Hk * D + (((size_t)b * P.Tk + key) * P.Hk + hk) * D +
                                      hf * (D / 2);
#pragma unroll
                for (int c = 0; c < D / 64; ++c) {
                    uint32_t r[32];
                    tmem_ld32(lane_addr + (which ? TM_DK : TM_DV) + (uint32_t)(hf * (D / 2) + c * 32), r);
                    tmem_ld_wait();
                    if (key < P.Tk) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            uint4 o;
                            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                            for (int x = 0; x < 4; ++x) oh[x] = __floats2bfloat162_rn(__uint_as_float(r[e + 2 * x]), __uint_as_float(r[e + 2 * x + 1]));
                            *reinterpret_cast<uint4*>(outp + c * 32 + e) = o;
                        }
                    }
                }
            }
        } else if (n_it == 0 && key < P.Tk) {
            // no query block sees these keys: their gradients are zero
            const size_t base = (size_t)part * P.B * P.Tk * P.Hk * D + (((size_t)b * P.Tk + key) * P.Hk + hk) * D;
            for (int d = hf * (D / 2); d < (hf + 1) * (D / 2); ++d) {
                P.dk[base + d] = __float2bfloat16_rn(0.f);
                P.dv[base + d] = __float2bfloat16_rn(0.f);
            }
        }
        if (!ok) *abort_flag = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem_base, 512);
}

template <int D>
static int launch_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta, float* dq, void* dk,
                      void* dv, int B, int Tq, int Tk, int H, int Hk, int causal, float scale, int q_offset, int gsplit, int* status,
                      cudaStream_t st) {
    CUtensorMap mq, mk, mv, mdo;
    if (ptb_make_tmap_bf16(&mq, q, (long long)H * D, (long long)B * Tq, (long long)H * D, 64, 128)) return -1;
    if (ptb_make_tmap_bf16(&mdo, dout, (long long)H * D, (long long)B * Tq, (long long)H * D, 64, 128)) return -1;
    if (ptb_make_tmap_bf16(&mk, k, (long long)Hk * D, (long long)B * Tk, (long long)Hk * D, 64, 128)) return -1;
    if (ptb_make_tmap_bf16(&mv, v, (long long)Hk * D, (long long)B * Tk, (long long)Hk * D, 64, 128)) return -1;
    static bool attr = false;
    if (!attr) {
        PTB_CUDA_OK(cudaFuncSetAttribute(bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmB<D>::TOTAL));
        attr = true;
    }
    BwdParams p;
    p.lse = lse; p.delta = delta; p.dq = dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
    p.B = B; p.Tq = Tq; p.Tk = Tk; p.H = H; p.Hk = Hk; p.causal = causal; p.q_offset = q_offset;
    p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status; p.gsplit = gsplit;
    dim3 grid((Tk + 127) / 128, Hk * gsplit, B);
    bwd_kernel<D><<<grid, NTHREADS, SmB<D>::TOTAL, st>>>(mq, mk, mv, mdo, p);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

}  // namespace fa100
}  // namespace ptb

// q [B, Tq, H, D], k/v [B, Tk, Hk, D] bf16 contiguous, D in {64, 128}; o like q; lse [B, H, Tq] fp32 (natural log).
// status: device int, set non-zero if a wait timed out.
PTB_API int ptb_flash_attn_fwd_sm100(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Tq, int Tk, int H, int Hk,
                                     int D, int causal, float scale, int q_offset, int* status, cudaStream_t st) {
    if (H % Hk) { ptb_set_error("flash attention: %d query heads over %d KV heads", H, Hk); return -1; }
    {
        int dev = 0;
        PTB_CUDA_OK(cudaGetDevice(&dev));
        PTB_CUDA_OK(cudaSetDevice(dev));     // the tensor-map encoder is a driver call: bind the primary context to this thread
    }
    if (D == 128) return ptb::fa100::launch<128>(q, k, v, o, lse, B, Tq, Tk, H, Hk, causal, scale, q_offset, status, st);
    if (D == 64) return ptb::fa100::launch<64>(q, k, v, o, lse, B, Tq, Tk, H, Hk, causal, scale, q_offset, status, st);
    ptb_set_error("flash attention (tcgen05): head size %d not supported (64, 128)", D);
    return -1;
}

extern "C" int ptb_flash_attn_delta(const void* o, const void* dout, float* delta, int B, int Tq, int H, int D, float* dq_zero, cudaStream_t st);

// Backward on tcgen05.  dq: fp32 [B, Tq, H, D] (cleared here, together with the delta pass); delta: fp32 [B, H, Tq] scratch.
// dk, dv: bf16 [gsplit][B, Tk, Hk, D]: with grouped-query heads the query heads of one KV head can be split over
// `gsplit` CTAs (a divisor of H / Hk) so that small problems fill the GPU; the caller sums the slices.
PTB_API int ptb_flash_attn_bwd_sm100(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                                     float* delta, float* dq, void* dk, void* dv, int B, int Tq, int Tk, int H, int Hk, int D, int causal,
                                     float scale, int q_offset, int gsplit, int* status, cudaStream_t st) {
    if (H % Hk || gsplit < 1 || (H / Hk) % gsplit) { ptb_set_error("flash attention: %d query heads over %d KV heads, split %d", H, Hk, gsplit); return -1; }
    {
        int dev = 0;
        PTB_CUDA_OK(cudaGetDevice(&dev));
        PTB_CUDA_OK(cudaSetDevice(dev));
    }
    if (ptb_flash_attn_delta(o, dout, delta, B, Tq, H, D, dq, st)) return -1;      // also clears dq
    if (D == 128) return ptb::fa100::launch_bwd<128>(q, k, v, dout, lse, delta, dq, dk, dv, B, Tq, Tk, H, Hk, causal, scale, q_offset, gsplit, status, st);
    if (D == 64) return ptb::fa100::launch_bwd<64>(q, k, v, dout, lse, delta, dq, dk, dv, B, Tq, Tk, H, Hk, causal, scale, q_offset, gsplit, status, st);
    ptb_set_error("flash attention (tcgen05): head size %d not supported (64, 128)", D);
    return -1;
}
