// Persistent decode kernel: one launch per token.
//
// The chain of small matrix-vector products of batch-1 decode is latency-bound when every product is
// its own launch: each one pays a launch, a prologue, a DRAM round trip and a tail, and the memory
// pipe drains in between.  Here one CTA per SM stays resident for the whole token and splits into
//   * a producer warp that walks the token's op list and streams THIS CTA's share of every weight
//     matrix, op after op, into one shared-memory ring with untiled TMA bulk copies.  Weights do not
//     depend on activations, so the producer runs ahead of the math by the depth of the ring
//     (~180 KB per SM, ~26 MB over the GPU: about one whole op) and HBM never idles;
//   * consumer warps that, per op, wait for the previous op's output (a grid-wide arrival counter),
//     normalise + quantise the input vector into shared memory, eat the tiles from the ring with the
//     same dp4a dot products as gemv_kernel, and run the epilogue (store / residual / SiLU·mul /
//     arg-max + control-block update).
// Attention (QK-norm, RoPE, fp16 KV write, one 128-position chunk per work item, partial results
// merged by the last CTA to finish a KV head) and the embedding look-up are ops of the same list.
//
// Every wait is bounded; on expiry the status word is set, the CTA stops waiting and runs to the end.
// The reference runs ~10 kernels per layer (torch/io/gguf_model.h:2575-3113).
#pragma once
#include "decode_kernels.cuh"

namespace ptb {

enum MegaKind : int { MK_EMBED = 0, MK_GEMV = 1, MK_ATTN = 2 };

struct MegaOp {
    int kind;
    int njobs, K, epilogue, act_gelu, norm_add_one;
    float eps;
    int window;
    GemvJob job[GEMV_MAX_JOBS];
    const float* x;          // GEMV input vector
    const float* norm_w;     // RMSNorm weight or null
    const float* resid;      // EPI_RESID
    const float* q_norm;     // attention
    const float* k_norm;
    const float* cos;
    const float* sin;
    __half* k_cache;
    __half* v_cache;
};

struct MegaParams {
    const MegaOp* ops;
    int n_ops, pad0;
    unsigned* bar;           // arrival counter, zero when the kernel starts
    int* status;
    int* ctrl;
    float* x;                // residual stream [hidden]
    float* qkv;              // q | k | v rows of the current layer
    float* att;              // attention output [heads * d]
    // embedding
    const uint8_t* emb_table;
    int emb_qtype, emb_rowbytes, emb_nblk, hidden, vocab;
    float emb_scale;
    // attention
    float* part_o;           // [kv_heads][max_splits][group][d]
    float* part_ml;          // [kv_heads][max_splits][group][2]
    unsigned* head_cnt;      // [kv_heads], zero between tokens
    int n_heads, n_kv_heads, group, max_seq, max_splits, neox;
    float attn_eps, scale;
    // arg-max
    float* amax_val;
    int* amax_idx;
    unsigned* ticket;
    float* logits;
    int* result;
    int row_offset, pad1;
    int* token_log;
    const int* token_script;
    // shared memory layout (bytes from the start of dynamic shared memory)
    int nslots, slot_bytes;
    int off_misc, off_xq, off_xs, off_xsf, off_xsf32, off_acc, off_attn, off_ring;
    unsigned long long* trace;   // optional [n_ops][8] stamps of CTA 0
};

template <int NT>
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory"); }
__device__ __forceinline__ void attn_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const unsigned* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Sum over the consumer threads (NT of them); buf >= 32 floats.
template <int NT>
__device__ __forceinline__ float cons_block_sum(float v, float* buf) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    cons_sync<NT>();
    if (l == 0) buf[w] = v;
    cons_sync<NT>();
    float t = (l < NT / 32) ? buf[l] : 0.0f;
    return warp_sum(t);
}

// x[K] -> optional RMSNorm -> int8 blocks of 32 (same outputs as quantize_input), by the NT consumer threads.
template <int NT, int ITEMS>
__device__ __forceinline__ void mega_quantize_input(const float* __restrict__ x, const float* __restrict__ norm_w, float eps,
                                                    int add_one, int K, int8_t* xq, float* xs, float* xsf16, float* xsf32,
                                                    float* red) {
    const int tid = threadIdx.x;
    const int items = K / 8;
    float v[ITEMS][8];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < ITEMS; ++r) {
        const int i = r * NT + tid;
        if (i < items) {
            const float4 a = __ldcg(reinterpret_cast<const float4*>(x) + 2 * i), b = __ldcg(reinterpret_cast<const float4*>(x) + 2 * i + 1);
            v[r][0] = a.x; v[r][1] = a.y; v[r][2] = a.z; v[r][3] = a.w; v[r][4] = b.x; v[r][5] = b.y; v[r][6] = b.z; v[r][7] = b.w;
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[r][k] = 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += v[r][k] * v[r][k];
    }
    float rs = 1.0f;
    if (norm_w) {
        ss = cons_block_sum<NT>(ss, red);
        rs = rsqrtf(ss / (float)K + eps);
    }
#pragma unroll
    for (int r = 0; r < ITEMS; ++r) {
        const int i = r * NT + tid;
        if (r * NT >= items) break;
        if (norm_w && i < items) {
            const float4 wa = __ldg(reinterpret_cast<const float4*>(norm_w) + 2 * i), wb = __ldg(reinterpret_cast<const float4*>(norm_w) + 2 * i + 1);
            const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int k = 0; k < 8; ++k) v[r][k] = v[r][k] * rs * (add_one ? 1.0f + w[k] : w[k]);
        }
        float am = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) am = fmaxf(am, fabsf(v[r][k]));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
        const float sc = am / 127.0f;
        const float inv = am > 0.f ? 127.0f / am : 0.f;
        int q[8], s = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) { q[k] = __float2int_rn(v[r][k] * inv); s += q[k]; }
        const int s16 = s + __shfl_xor_sync(0xffffffffu, s, 1);
        const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
        if (i < items) {
            uint2 pk;
            pk.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((q[3] & 0xff) << 24);
            pk.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((q[7] & 0xff) << 24);
            reinterpret_cast<uint2*>(xq)[i] = pk;
            if ((i & 1) == 0) xsf16[i >> 1] = sc * (float)s16;
            if ((i & 3) == 0) { xs[i >> 2] = sc; xsf32[i >> 2] = sc * (float)s32; }
        }
    }
    cons_sync<NT>();
}

// Which job of a GEMV op this CTA serves, and its rows.
struct MegaShare {
    int ji, r0, r1, nitems;
};
__device__ __forceinline__ MegaShare mega_share(const MegaOp& op, int cta) {
    MegaShare s;
    s.ji = 0;
#pragma unroll
    for (int i = 1; i < GEMV_MAX_JOBS; ++i)
        if (i < op.njobs && cta >= op.job[i].cta_begin) s.ji = i;
    const GemvJob& J = op.job[s.ji];
    const int ci = cta - J.cta_begin;
    if (ci >= J.cta_count) { s.r0 = s.r1 = 0; s.nitems = 0; return s; }
    s.r0 = (int)(((long long)J.N * ci) / J.cta_count);
    s.r1 = (int)(((long long)J.N * (ci + 1)) / J.cta_count);
    s.nitems = ((s.r1 - s.r0 + J.RW - 1) / J.RW) * J.KS;
    return s;
}

struct MegaItem { int s, nb, boff, sb, row0, rows; size_t off; };
__device__ __forceinline__ MegaItem mega_geom(const GemvJob& J, int r0, int r1, int it, int sz0, int sz1) {
    MegaItem g;
    const int rg = it / J.KS;
    g.s = it - rg * J.KS;
    const int extra = min(g.s, J.seg_rem);
    g.nb = J.seg_base + (g.s < J.seg_rem ? 1 : 0);
    g.boff = g.s * J.seg_base + extra;
    g.sb = g.s < J.seg_rem ? sz1 : sz0;
    g.row0 = r0 + rg * J.RW;
    g.rows = min(J.RW, r1 - g.row0);
    g.off = (size_t)J.N * ((size_t)g.s * sz0 + (size_t)extra * (sz1 - sz0)) + (size_t)g.row0 * g.sb;
    return g;
}

__device__ __forceinline__ void mega_norm_rope_head(const float* src, const float* nw, float eps, const float* cs, const float* sn,
                                                    int neox, float mul, float* dst, int lane) {
    float v[4];
    if (neox) { v[0] = __ldcg(src + lane); v[1] = __ldcg(src + lane + 32); v[2] = __ldcg(src + lane + 64); v[3] = __ldcg(src + lane + 96); }
    else { const float4 t = __ldcg(reinterpret_cast<const float4*>(src) + lane); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    if (nw) {
        float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        ss = warp_sum(ss);
        const float rs = rsqrtf(ss / 128.0f + eps);
        if (neox) { v[0] *= rs * nw[lane]; v[1] *= rs * nw[lane + 32]; v[2] *= rs * nw[lane + 64]; v[3] *= rs * nw[lane + 96]; }
        else { const float4 w = reinterpret_cast<const float4*>(nw)[lane]; v[0] *= rs * w.x; v[1] *= rs * w.y; v[2] *= rs * w.z; v[3] *= rs * w.w; }
    }
    if (neox) {
        const float c0 = cs[lane], s0 = sn[lane], c1 = cs[lane + 32], s1 = sn[lane + 32];
        dst[lane] = (v[0] * c0 - v[2] * s0) * mul;
        dst[lane + 64] = (v[2] * c0 + v[0] * s0) * mul;
        dst[lane + 32] = (v[1] * c1 - v[3] * s1) * mul;
        dst[lane + 96] = (v[3] * c1 + v[1] * s1) * mul;
    } else {
        const float c0 = cs[2 * lane], s0 = sn[2 * lane], c1 = cs[2 * lane + 1], s1 = sn[2 * lane + 1];
        dst[4 * lane + 0] = (v[0] * c0 - v[1] * s0) * mul;
        dst[4 * lane + 1] = (v[1] * c0 + v[0] * s0) * mul;
        dst[4 * lane + 2] = (v[2] * c1 - v[3] * s1) * mul;
        dst[4 * lane + 3] = (v[3] * c1 + v[2] * s1) * mul;
    }
}

template <int G>
struct MegaAttnShared {
    float qs[G][ATT_D];
    float kn[ATT_D];
    float sc[G][ATT_CHUNK];
    float hm[G], hl[G];
    float red[8][G][ATT_D];
    int last;
};

// One attention op: the first 256 consumer threads work through this CTA's (kv head, chunk) items.
template <int G>
__device__ __forceinline__ void mega_attn(const MegaParams& P, const MegaOp& op, uint8_t* smem_attn, int cta, int n_ctas) {
    MegaAttnShared<G>& sh = *reinterpret_cast<MegaAttnShared<G>*>(smem_attn);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos = min(__ldcg(P.ctrl + CTRL_POS), P.max_seq - 1);
    const int T = pos + 1;
    const int lo = (op.window > 0 && T > op.window) ? T - op.window : 0;
    const int first_chunk = lo / ATT_CHUNK;
    const int nchunk = (T + ATT_CHUNK - 1) / ATT_CHUNK;
    const int nact = nchunk - first_chunk;
    const int qd = P.n_heads * ATT_D, kvd = P.n_kv_heads * ATT_D;
    const float* qv = P.qkv;
    const float* kv = P.qkv + qd;
    const float* vv = P.qkv + qd + kvd;
    const float* cs = op.cos + (size_t)pos * (ATT_D / 2);
    const float* sn = op.sin + (size_t)pos * (ATT_D / 2);
    const int rg = tid >> 4, dc = tid & 15;
    for (int item = cta; item < P.n_kv_heads * nact; item += n_ctas) {
        const int kvh = item % P.n_kv_heads;
        const int c = first_chunk + item / P.n_kv_heads;
        __half* kc = op.k_cache + (size_t)kvh * P.max_seq * ATT_D;
        __half* vc = op.v_cache + (size_t)kvh * P.max_seq * ATT_D;
        const int base = c * ATT_CHUNK;
        const int t0 = max(base, lo), t1 = min(base + ATT_CHUNK, T);
        if (warp < G)
            mega_norm_rope_head(qv + (size_t)(kvh * G + warp) * ATT_D, op.q_norm, P.attn_eps, cs, sn, P.neox,
                                P.scale * 1.4426950408889634f, sh.qs[warp], lane);
        if (pos >= base && pos < base + ATT_CHUNK && warp == 7) {      // this chunk holds the new position: write K, V
            mega_norm_rope_head(kv + (size_t)kvh * ATT_D, op.k_norm, P.attn_eps, cs, sn, P.neox, 1.0f, sh.kn, lane);
            __syncwarp();
            for (int i = lane; i < ATT_D; i += 32) {
                kc[(size_t)pos * ATT_D + i] = __float2half_rn(sh.kn[i]);
                vc[(size_t)pos * ATT_D + i] = __float2half_rn(__ldcg(vv + (size_t)kvh * ATT_D + i));
            }
        }
        attn_sync();
        {   // scores: two threads per cache position, 64 dims each
            const int tl = tid >> 1, hf = tid & 1;
            const int t = base + tl;
            const bool valid = t >= t0 && t < t1;
            uint4 raw[8];
            if (valid) {
                const uint4* kp = reinterpret_cast<const uint4*>(kc + (size_t)t * ATT_D + hf * 64);
#pragma unroll
                for (int i = 0; i < 8; ++i) raw[i] = kp[i];
            }
            float s[G];
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] = 0.f;
            if (valid) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const __half2* h2 = reinterpret_cast<const __half2*>(&raw[i]);
                    float kf[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h2[k]); kf[2 * k] = f.x; kf[2 * k + 1] = f.y; }
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float4 qa = *reinterpret_cast<const float4*>(&sh.qs[g][hf * 64 + i * 8]);
                        const float4 qb = *reinterpret_cast<const float4*>(&sh.qs[g][hf * 64 + i * 8 + 4]);
                        s[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x + kf[5] * qb.y +
                                kf[6] * qb.z + kf[7] * qb.w;
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float tot = s[g] + __shfl_xor_sync(0xffffffffu, s[g], 1);
                if (hf == 0) sh.sc[g][tl] = valid ? tot : -INFINITY;
            }
        }
        uint4 vraw[ATT_CHUNK / 16];
#pragma unroll
        for (int i = 0; i < ATT_CHUNK / 16; ++i) {
            const int t = base + rg + 16 * i;
            vraw[i] = (t >= t0 && t < t1) ? *reinterpret_cast<const uint4*>(vc + (size_t)t * ATT_D + dc * 8) : make_uint4(0, 0, 0, 0);
        }
        attn_sync();
        if (warp < G) {     // softmax statistics (base 2) of head `warp`
            float m = -INFINITY;
            for (int i = lane; i < ATT_CHUNK; i += 32) m = fmaxf(m, sh.sc[warp][i]);
            m = warp_max(m);
            float l = 0.f;
            for (int i = lane; i < ATT_CHUNK; i += 32) {
                const float p = exp2f(sh.sc[warp][i] - m);
                sh.sc[warp][i] = p;
                l += p;
            }
            l = warp_sum(l);
            if (lane == 0) { sh.hm[warp] = m; sh.hl[warp] = l; }
        }
        attn_sync();
        float acc[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[g][k] = 0.f;
#pragma unroll
            for (int i = 0; i < ATT_CHUNK / 16; ++i) {
                const float p = sh.sc[g][rg + 16 * i];
                const __half2* h2 = reinterpret_cast<const __half2*>(&vraw[i]);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = __half22float2(h2[k]);
                    acc[g][2 * k] += p * f.x;
                    acc[g][2 * k + 1] += p * f.y;
                }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[g][k] += __shfl_xor_sync(0xffffffffu, acc[g][k], 16);
        }
        if (lane < 16) {
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int k = 0; k < 8; ++k) sh.red[warp][g][dc * 8 + k] = acc[g][k];
        }
        attn_sync();
        float* po = P.part_o + ((size_t)kvh * P.max_splits + c) * G * ATT_D;
        float* pml = P.part_ml + ((size_t)kvh * P.max_splits + c) * G * 2;
        for (int i = tid; i < G * ATT_D; i += 256) {
            const int g = i / ATT_D, d = i - g * ATT_D;
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) o += sh.red[w][g][d];
            if (nact == 1) P.att[(size_t)(kvh * G + g) * ATT_D + d] = o / sh.hl[g];      // a single chunk needs no merge
            else __stcg(po + i, o);
        }
        if (nact > 1) {
            if (tid < G) { __stcg(pml + 2 * tid, sh.hm[tid]); __stcg(pml + 2 * tid + 1, sh.hl[tid]); }
            __threadfence();
            attn_sync();
            if (tid == 0) {
                const unsigned t = atomicAdd(P.head_cnt + kvh, 1u);
                sh.last = (t == (unsigned)(nact - 1));
            }
            attn_sync();
            if (sh.last) {      // every chunk of this KV head is in: merge them
                __threadfence();
                for (int i = tid; i < G * ATT_D; i += 256) {
                    const int g = i / ATT_D;
                    float Mx = -INFINITY;
                    for (int cc = first_chunk; cc < nchunk; ++cc)
                        Mx = fmaxf(Mx, __ldcg(P.part_ml + (((size_t)kvh * P.max_splits + cc) * G + g) * 2));
                    float Lt = 0.f, Ot = 0.f;
                    for (int cc = first_chunk; cc < nchunk; ++cc) {
                        const float* ml = P.part_ml + (((size_t)kvh * P.max_splits + cc) * G + g) * 2;
                        const float w = exp2f(__ldcg(ml) - Mx);
                        Lt += w * __ldcg(ml + 1);
                        Ot += w * __ldcg(P.part_o + ((size_t)kvh * P.max_splits + cc) * G * ATT_D + i);
                    }
                    P.att[(size_t)kvh * G * ATT_D + i] = Ot / Lt;
                }
                if (tid == 0) P.head_cnt[kvh] = 0u;
            }
        }
        attn_sync();      // shared memory is reused by the next item
    }
}

template <int NCONS>
__global__ void __launch_bounds__((NCONS + 1) * 32, 1) decode_mega_kernel(const __grid_constant__ MegaParams P) {
    constexpr int NT = NCONS * 32;
    constexpr int QITEMS = (10240 + 8 * NT - 1) / (8 * NT);
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, n_ctas = gridDim.x;
    const int NS = P.nslots;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + NS;
    float* misc = reinterpret_cast<float*>(smem + P.off_misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 96);
    volatile int* uniform_abort = reinterpret_cast<volatile int*>(misc + 97);
    int8_t* xq = reinterpret_cast<int8_t*>(smem + P.off_xq);
    float* xs = reinterpret_cast<float*>(smem + P.off_xs);
    float* xsf = reinterpret_cast<float*>(smem + P.off_xsf);
    float* xsf32 = reinterpret_cast<float*>(smem + P.off_xsf32);
    float* acc = reinterpret_cast<float*>(smem + P.off_acc);
    uint8_t* ring = smem + P.off_ring;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        *abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async();
    }
    __syncthreads();

    if (warp == NCONS) {
        // ================================================================== producer: stream weights, op after op
        // PL lanes issue in parallel: lane k owns tiles k, k+PL, ... of every op, so that the waits on the ring
        // and the address arithmetic of up to PL tiles overlap.
        constexpr int PL = 16;
        if (lane < PL) {
            uint32_t gbase = 0;
            bool ok = true;
            uint32_t last_g = 0xffffffffu;
            for (int oi = 0; oi < P.n_ops && ok; ++oi) {
                if (P.ops[oi].kind != MK_GEMV) continue;
                const MegaShare sh = mega_share(P.ops[oi], cta);
                const GemvJob J = P.ops[oi].job[sh.ji];
                const int sz0 = seg_bytes(J.qtype, J.seg_base), sz1 = seg_bytes(J.qtype, J.seg_base + 1);
                const bool paired = J.w2 != nullptr;
                for (int it = lane; it < sh.nitems; it += PL) {
                    const uint32_t g = gbase + (uint32_t)it;
                    const uint32_t slot = g % NS, n = g / NS;
                    if (n > 0) {
                        if (*abort_flag) { ok = false; break; }
                        if (!mbar_wait(&empty[slot], (n - 1) & 1u, P.status)) { *abort_flag = 1; ok = false; break; }
                    }
                    const MegaItem t = mega_geom(J, sh.r0, sh.r1, it, sz0, sz1);
                    const uint32_t bytes = (uint32_t)t.rows * t.sb;
                    uint8_t* dst = ring + (size_t)slot * P.slot_bytes;
                    mbar_expect_tx(&full[slot], paired ? 2 * bytes : bytes);
                    bulk_g2s(dst, J.w + t.off, bytes, &full[slot]);
                    if (paired) bulk_g2s(dst + J.RW * t.sb, J.w2 + t.off, bytes, &full[slot]);
                    last_g = g;
                }
                gbase += (uint32_t)sh.nitems;
            }
            if (!ok && last_g != 0xffffffffu) {
                // give this lane's last copy a bounded time to land before the CTA leaves
                mbar_wait(&full[last_g % NS], (last_g / NS) & 1u, nullptr, 200000u);
            }
        }
    } else {
        // ================================================================== consumers
        uint32_t gbase = 0;              // ring position of this CTA's first tile of the current op
        unsigned bar_target = 0;         // arrivals that complete the previous op
        bool ok = true;
        auto stamp = [&](int oi, int k) {
            if (P.trace && tid == 0 && cta == 0) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                P.trace[(size_t)oi * 8 + k] = t;
            }
        };
        for (int oi = 0; oi < P.n_ops; ++oi) {
            const MegaOp& op = P.ops[oi];
            stamp(oi, 0);
            // parameters do not depend on the previous op: pull the RMSNorm weight towards this SM before waiting
            if (op.kind == MK_GEMV && op.norm_w) {
                for (int i = tid * 32; i < op.K; i += NT * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(op.norm_w + i));
            }
            // ---- wait until every CTA has finished the previous op
            if (oi > 0) {
                if (tid == 0 && !*abort_flag) {
                    unsigned long long t0;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
                    uint32_t spins = 0;
                    while ((int)(ld_acquire_gpu_u32(P.bar) - bar_target) < 0) {
                        if ((++spins & 1023u) == 0) {
                            unsigned long long t1;
                            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                            if (t1 - t0 > 2000000000ull) { atomicExch(P.status, PTB_ERR_FLAG_TIMEOUT); *abort_flag = 1; break; }
                        }
                    }
                }
                if (tid == 0) *uniform_abort = *abort_flag;      // one reader, so that every consumer thread sees the same value
                cons_sync<NT>();
                if (*uniform_abort) ok = false;
            }
            stamp(oi, 1);
            if (op.kind == MK_EMBED) {
                int tok = __ldcg(P.ctrl + CTRL_TOKEN);
                if (tok < 0 || tok >= P.vocab) {
                    if (tid == 0 && cta == 0) atomicExch(P.status, PTB_ERR_BOUNDS);
                    tok = 0;
                }
                const uint8_t* row = P.emb_table + (size_t)tok * P.emb_rowbytes;
                for (int i = cta * NT + tid; i < P.hidden; i += n_ctas * NT) {
                    float v;
                    const int b = i >> 8, e = i & 255;
                    if (P.emb_qtype == QT_Q4K) {
                        const uint8_t* bp = row + b * 144;
                        const float d = __half2float(*reinterpret_cast<const __half*>(bp));
                        const float dmin = __half2float(*reinterpret_cast<const __half*>(bp + 2));
                        const uint8_t* s = bp + 4;
                        const int is = e >> 5;
                        int scv, mv;
                        if (is < 4) { scv = s[is] & 63; mv = s[is + 4] & 63; }
                        else { scv = (s[is + 4] & 0xF) | ((s[is - 4] >> 6) << 4); mv = (s[is + 4] >> 4) | ((s[is] >> 6) << 4); }
                        const uint8_t qb = bp[16 + (e >> 6) * 32 + (e & 31)];
                        const int q = (is & 1) ? (qb >> 4) : (qb & 0xF);
                        v = d * scv * q - dmin * mv;
                    } else if (P.emb_qtype == QT_Q6K) {
                        const int n = e >> 7, r = e & 127, quad = r >> 5, l = r & 31;
                        const uint8_t qlb = row[b * 128 + n * 64 + (quad & 1) * 32 + l];
                        const uint8_t qhb = row[P.emb_nblk * 128 + b * 64 + n * 32 + l];
                        const int lo4 = (quad >> 1) ? (qlb >> 4) : (qlb & 0xF);
                        const int hi2 = (qhb >> (2 * quad)) & 3;
                        const int q = (lo4 | (hi2 << 4)) - 32;
                        const int8_t scv = reinterpret_cast<const int8_t*>(row + P.emb_nblk * 192 + b * 16)[e >> 4];
                        const float d = __half2float(*reinterpret_cast<const __half*>(row + P.emb_nblk * 208 + b * 2));
                        v = d * scv * q;
                    } else if (P.emb_qtype == 2) {
                        v = __half2float(reinterpret_cast<const __half*>(row)[i]);
                    } else {
                        v = reinterpret_cast<const float*>(row)[i];
                    }
                    P.x[i] = v * P.emb_scale;
                }
            } else if (op.kind == MK_ATTN) {
                if (ok && tid < 256) {
                    switch (P.group) {
                        case 1: mega_attn<1>(P, op, smem + P.off_attn, cta, n_ctas); break;
                        case 2: mega_attn<2>(P, op, smem + P.off_attn, cta, n_ctas); break;
                        case 4: mega_attn<4>(P, op, smem + P.off_attn, cta, n_ctas); break;
                        default: mega_attn<8>(P, op, smem + P.off_attn, cta, n_ctas); break;
                    }
                }
            } else {
                // ---------------------------------------------------------------- GEMV
                const MegaShare sh = mega_share(op, cta);
                const GemvJob J = op.job[sh.ji];
                const int r0 = sh.r0, r1 = sh.r1, RW = J.RW, KS = J.KS, qtype = J.qtype;
                const int op_epi = op.epilogue, op_gelu = op.act_gelu;
                const float* op_resid = op.resid;
                const bool paired = J.w2 != nullptr;
                const int sz0 = seg_bytes(qtype, J.seg_base), sz1 = seg_bytes(qtype, J.seg_base + 1);
                mega_quantize_input<NT, QITEMS>(op.x, op.norm_w, op.eps, op.norm_add_one, op.K, xq, xs, xsf, xsf32, misc);
                stamp(oi, 2);
                const int grp = lane >> 2, lane4 = lane & 3;
                const int gprw = 8 / RW;
                const int my_row = grp % RW, my_j = grp / RW;
                float best_v = -INFINITY;
                int best_i = 0x7fffffff;
                auto epilogue = [&](int n, float v0, float v1) {
                    if (J.bias) v0 += J.bias[n];
                    switch (op_epi) {
                        case EPI_STORE: J.out[n] = v0; break;
                        case EPI_RESID: J.out[n] = __ldcg(op_resid + n) + v0; break;
                        case EPI_GATED: J.out[n] = (op_gelu ? gelu_tanh(v0) : silu(v0)) * v1; break;
                        case EPI_ARGMAX:
                            if (P.logits) P.logits[n] = v0;
                            if (v0 > best_v || (v0 == best_v && n < best_i)) { best_v = v0; best_i = n; }
                            break;
                    }
                };
                for (int it = warp; it < sh.nitems; it += NCONS) {
                    const uint32_t gidx = gbase + (uint32_t)it;
                    const uint32_t slot = gidx % NS;
                    const MegaItem g = mega_geom(J, r0, r1, it, sz0, sz1);
                    if (ok) {
                        if (*abort_flag) ok = false;
                        else if (!mbar_wait(&full[slot], (gidx / NS) & 1u, P.status)) { *abort_flag = 1; ok = false; }
                    }
                    const uint8_t* tile = ring + (size_t)slot * P.slot_bytes;
                    float a0 = 0.f, a1 = 0.f;
                    if (ok && my_row < g.rows) {
                        const uint8_t* rowp = tile + (size_t)my_row * g.sb;
                        const int8_t* xq_s = xq + g.boff * 256;
                        const float* xs_s = xs + g.boff * 8;
                        const float* xsf_s = xsf + g.boff * 16;
                        const float* xsf32_s = xsf32 + g.boff * 8;
                        const bool swap = (grp & 1) && (((g.sb >> 4) & 1) == 0);
                        if (qtype == QT_Q4K) {
#pragma unroll 1
                            for (int b = my_j; b < g.nb; b += gprw) {
                                a0 += q4k_dot(rowp + b * 144, lane4, swap, xq_s + b * 256, xs_s + b * 8, xsf32_s + b * 8);
                                if (paired) a1 += q4k_dot(rowp + RW * g.sb + b * 144, lane4, swap, xq_s + b * 256, xs_s + b * 8, xsf32_s + b * 8);
                            }
                        } else {
#pragma unroll 1
                            for (int b = my_j; b < g.nb; b += gprw) {
                                a0 += q6k_dot(rowp, g.nb, b, lane4, swap, xq_s + b * 256, xs_s + b * 8, xsf_s + b * 16);
                                if (paired) a1 += q6k_dot(rowp + RW * g.sb, g.nb, b, lane4, swap, xq_s + b * 256, xs_s + b * 8, xsf_s + b * 16);
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0 && ok) mbar_arrive(&empty[slot]);      // the slot may be refilled
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        if (o < 4 || o >= 4 * RW) {
                            a0 += __shfl_xor_sync(0xffffffffu, a0, o);
                            a1 += __shfl_xor_sync(0xffffffffu, a1, o);
                        }
                    }
                    if (lane4 == 0 && my_j == 0 && my_row < g.rows) {
                        const int n = g.row0 + my_row;
                        if (KS == 1) epilogue(n, a0, a1);
                        else {
                            acc[(size_t)(n - r0) * KS + g.s] = a0;
                            if (paired) acc[(size_t)(r1 - r0) * KS + (size_t)(n - r0) * KS + g.s] = a1;
                        }
                    }
                }
                gbase += (uint32_t)sh.nitems;
                stamp(oi, 3);
                if (KS > 1) {
                    cons_sync<NT>();
                    for (int r = tid; r < r1 - r0; r += NT) {
                        float v0 = 0.f, v1 = 0.f;
                        for (int s = 0; s < KS; ++s) {
                            v0 += acc[(size_t)r * KS + s];
                            if (paired) v1 += acc[(size_t)(r1 - r0) * KS + (size_t)r * KS + s];
                        }
                        epilogue(r0 + r, v0, v1);
                    }
                }
                if (op_epi == EPI_ARGMAX) {
                    // CTA arg-max (ties -> lowest index); the last CTA to arrive finishes and advances the control block
                    cons_sync<NT>();
                    float* sv = misc;
                    int* si = reinterpret_cast<int*>(misc + 32);
                    int* is_last = reinterpret_cast<int*>(misc + 64);
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
                        const int oi2 = __shfl_xor_sync(0xffffffffu, best_i, o);
                        if (ov > best_v || (ov == best_v && oi2 < best_i)) { best_v = ov; best_i = oi2; }
                    }
                    if (lane == 0) { sv[warp] = best_v; si[warp] = best_i; }
                    cons_sync<NT>();
                    if (tid == 0) {
                        for (int w = 1; w < NCONS; ++w)
                            if (sv[w] > best_v || (sv[w] == best_v && si[w] < best_i)) { best_v = sv[w]; best_i = si[w]; }
                        __stcg(P.amax_val + cta, best_v);
                        __stcg(P.amax_idx + cta, best_i);
                        __threadfence();
                        const unsigned t = atomicAdd(P.ticket, 1u);
                        *is_last = (t == (unsigned)n_ctas - 1);
                    }
                    cons_sync<NT>();
                    if (*is_last) {
                        __threadfence();
                        float bv = -INFINITY;
                        int bi = 0x7fffffff;
                        for (int i = tid; i < n_ctas; i += NT) {
                            const float v = __ldcg(P.amax_val + i);
                            const int ix = __ldcg(P.amax_idx + i);
                            if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
                        }
                        for (int o = 16; o > 0; o >>= 1) {
                            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                            const int oi2 = __shfl_xor_sync(0xffffffffu, bi, o);
                            if (ov > bv || (ov == bv && oi2 < bi)) { bv = ov; bi = oi2; }
                        }
                        cons_sync<NT>();
                        if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
                        cons_sync<NT>();
                        if (tid == 0) {
                            for (int w = 1; w < NCONS; ++w)
                                if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
                            *P.ticket = 0u;
                            bi += P.row_offset;
                            P.result[0] = bi;
                            reinterpret_cast<float*>(P.result)[1] = bv;
                            int* ctrl = P.ctrl;
                            const int step = ctrl[CTRL_STEP];
                            if (P.token_log && step < ctrl[CTRL_LOG_CAP]) P.token_log[step] = bi;
                            ctrl[CTRL_STEP] = step + 1;
                            const int mode = ctrl[CTRL_SELF_FEED];
                            if (mode) {
                                const bool scripted = mode == 2 && P.token_script && step + 1 < ctrl[CTRL_SCRIPT_LEN];
                                ctrl[CTRL_TOKEN] = scripted ? P.token_script[step + 1] : bi;
                                ctrl[CTRL_POS] += 1;
                            }
                        }
                    }
                }
            }
            stamp(oi, 4);
            // ---- this CTA is done with the op: publish
            if (oi + 1 < P.n_ops) {
                cons_sync<NT>();                     // every consumer thread's stores are ordered before thread 0's release
                if (tid == 0) { __threadfence(); red_release_gpu_add(P.bar, 1u); }
                bar_target += (unsigned)n_ctas;
            }
        }
    }
    __syncthreads();
}

}  // namespace ptb
