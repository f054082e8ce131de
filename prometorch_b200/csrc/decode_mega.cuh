// Persistent decode kernel: one launch per token.
//
// The chain of small matrix-vector products of batch-1 decode is latency-bound when every product is
// its own launch: each one pays a launch, a prologue, a DRAM round trip and a tail, and the memory
// pipe drains in between.  Here one CTA per SM stays resident for the whole token and splits into
//   * a producer warp that walks the token's op list and streams THIS CTA's share of every weight
//     matrix, op after op, into one shared-memory ring with untiled TMA bulk copies.  Weights do not
//     depend on activations, so the producer runs ahead of the math by the depth of the ring
//     (~180 KB per SM, ~26 MB over the GPU: about one whole op) and HBM never idles;
//   * consumer warps that, per op, read the previous op's output vector, normalise + quantise it
//     into shared memory, eat the tiles from the ring with the same dp4a dot products as gemv_kernel,
//     and run the epilogue (store / residual / SiLU·mul / arg-max + control-block update).
// Attention (QK-norm, RoPE, fp16 KV write, one 128-position chunk per work item, partial results
// merged by the CTA that owns the KV head) and the embedding look-up are ops of the same list.
//
// There is no grid-wide barrier.  Every activation element travels as an 8-byte {value, sequence
// number} slot written and read as one access: a reader that sees the sequence number of the
// producing op (token generation x ops per token + op index + 1, never repeated) has the value too,
// so CTAs synchronise on exactly the data they need, with neither fences nor counters.  A value is
// overwritten only by an op that (transitively) needed every reader of the old value to finish.
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
    const uint2* x_ll;       // GEMV input vector as {value, sequence} slots, written by op `src_op`
    const uint2* resid_ll;   // EPI_RESID: slots whose value is added (already observed by this CTA)
    uint2* out_ll[GEMV_MAX_JOBS];   // output slots of each job (null: plain output only)
    int src_op, pad;
    const float* norm_w;     // RMSNorm weight or null
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
    int* status;
    int* ctrl;
    float* x;                // residual stream [hidden] (plain copy, for readers outside the kernel)
    uint2* x_ll;             // the same as slots
    const uint2* qkv_ll;     // q | k | v rows of the current layer
    uint2* att_ll;           // attention output [heads * d]
    unsigned* gen;           // token generation: read at start, advanced by the CTA that finishes the token
    // embedding
    const uint8_t* emb_table;
    int emb_qtype, emb_rowbytes, emb_nblk, hidden, vocab;
    float emb_scale;
    // attention
    uint2* part_o;           // [kv_heads][max_splits][group][d] slots
    uint2* part_ml;          // [kv_heads][max_splits][group][2] slots
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

__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Wait budget shared by the polling loops of one CTA: the first loop to run out of time records the
// timeout and raises the CTA's abort flag; after that no loop waits any more.
struct MegaWait {
    volatile int* abort_flag;
    int* status;
    __device__ __forceinline__ bool expired(uint32_t& spins, unsigned long long& t0) const {
        if ((++spins & 255u) != 0) return false;
        if (*abort_flag) return true;
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t0 == 0) { t0 = t1; return false; }
        if (t1 - t0 > 2000000000ull) { atomicExch(status, PTB_ERR_FLAG_TIMEOUT); *abort_flag = 1; return true; }
        return false;
    }
};

// One slot: spin until its sequence number is `seq`.
__device__ __forceinline__ float ll_wait(const uint2* p, uint32_t seq, const MegaWait& W) {
    uint32_t spins = 0;
    unsigned long long t0 = 0;
    uint2 v = ld_ll(p);
    while (v.y != seq) {
        if (W.expired(spins, t0)) break;
        v = ld_ll(p);
    }
    return __uint_as_float(v.x);
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

// x (slots written by the producing op) -> optional RMSNorm -> int8 blocks of 32, by the NT consumer threads.
// All of a thread's loads are in flight together; the loop repeats until every sequence number matches.
template <int NT, int ITEMS>
__device__ __forceinline__ void mega_quantize_input(const uint2* __restrict__ x_ll, uint32_t seq, const float* __restrict__ norm_w,
                                                    float eps, int add_one, int K, int8_t* xq, float* xs, float* xsf16,
                                                    float* xsf32, float* red, const MegaWait& W) {
    const int tid = threadIdx.x;
    const int items = K / 8;
    float v[ITEMS][8];
    {
        uint4 a[ITEMS][4];
        uint32_t spins = 0;
        unsigned long long t0 = 0;
        while (true) {
            bool good = true;
#pragma unroll
            for (int r = 0; r < ITEMS; ++r) {
                const int i = r * NT + tid;
                if (i < items) {
                    const uint4* p = reinterpret_cast<const uint4*>(x_ll + (size_t)i * 8);
#pragma unroll
                    for (int j = 0; j < 4; ++j) a[r][j] = ld_volatile_v4(p + j);
                }
            }
#pragma unroll
            for (int r = 0; r < ITEMS; ++r) {
                const int i = r * NT + tid;
                if (i < items) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) good = good && a[r][j].y == seq && a[r][j].w == seq;
                }
            }
            if (good || W.expired(spins, t0)) break;
        }
#pragma unroll
        for (int r = 0; r < ITEMS; ++r) {
            const int i = r * NT + tid;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[r][2 * j] = i < items ? __uint_as_float(a[r][j].x) : 0.f;
                v[r][2 * j + 1] = i < items ? __uint_as_float(a[r][j].z) : 0.f;
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < ITEMS; ++r)
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += v[r][k] * v[r][k];
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
    if (J.KS == 1) {        // the common case (K <= 2560): one segment, no divisions
        g.s = 0; g.nb = J.seg_base; g.boff = 0; g.sb = sz0;
        g.row0 = r0 + it * J.RW;
        g.rows = min(J.RW, r1 - g.row0);
        g.off = (size_t)g.row0 * sz0;
        return g;
    }
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

// One head of 128 values from slots: optional RMSNorm, rotation, scale; one warp, four values per lane.
__device__ __forceinline__ void mega_norm_rope_head(const uint2* src, uint32_t seq, const MegaWait& W, const float* nw, float eps,
                                                    const float* cs, const float* sn, int neox, float mul, float* dst, int lane) {
    float v[4];
    if (neox) {
        v[0] = ll_wait(src + lane, seq, W); v[1] = ll_wait(src + lane + 32, seq, W);
        v[2] = ll_wait(src + lane + 64, seq, W); v[3] = ll_wait(src + lane + 96, seq, W);
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = ll_wait(src + 4 * lane + k, seq, W);
    }
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
};

// One attention op: the first 256 consumer threads work through this CTA's (kv head, chunk) items; with more
// than one chunk the partial {max, sum, output} of every chunk travel as slots to CTA `kv head`, which merges.
template <int G>
__device__ __forceinline__ void mega_attn(const MegaParams& P, const MegaOp& op, uint8_t* smem_attn, int cta, int n_ctas,
                                          uint32_t seq_in, uint32_t seq_out, const MegaWait& W) {
    MegaAttnShared<G>& sh = *reinterpret_cast<MegaAttnShared<G>*>(smem_attn);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos = min(__ldcg(P.ctrl + CTRL_POS), P.max_seq - 1);
    const int T = pos + 1;
    const int lo = (op.window > 0 && T > op.window) ? T - op.window : 0;
    const int first_chunk = lo / ATT_CHUNK;
    const int nchunk = (T + ATT_CHUNK - 1) / ATT_CHUNK;
    const int nact = nchunk - first_chunk;
    const int qd = P.n_heads * ATT_D, kvd = P.n_kv_heads * ATT_D;
    const uint2* qv = P.qkv_ll;
    const uint2* kv = P.qkv_ll + qd;
    const uint2* vv = P.qkv_ll + qd + kvd;
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
            mega_norm_rope_head(qv + (size_t)(kvh * G + warp) * ATT_D, seq_in, W, op.q_norm, P.attn_eps, cs, sn, P.neox,
                                P.scale * 1.4426950408889634f, sh.qs[warp], lane);
        if (pos >= base && pos < base + ATT_CHUNK && warp == 7) {      // this chunk holds the new position: write K, V
            mega_norm_rope_head(kv + (size_t)kvh * ATT_D, seq_in, W, op.k_norm, P.attn_eps, cs, sn, P.neox, 1.0f, sh.kn, lane);
            __syncwarp();
            for (int i = lane; i < ATT_D; i += 32) {
                kc[(size_t)pos * ATT_D + i] = __float2half_rn(sh.kn[i]);
                vc[(size_t)pos * ATT_D + i] = __float2half_rn(ll_wait(vv + (size_t)kvh * ATT_D + i, seq_in, W));
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
        uint2* po = P.part_o + ((size_t)kvh * P.max_splits + c) * G * ATT_D;
        uint2* pml = P.part_ml + ((size_t)kvh * P.max_splits + c) * G * 2;
        for (int i = tid; i < G * ATT_D; i += 256) {
            const int g = i / ATT_D, d = i - g * ATT_D;
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) o += sh.red[w][g][d];
            if (nact == 1) st_ll(P.att_ll + (size_t)(kvh * G + g) * ATT_D + d, __float_as_uint(o / sh.hl[g]), seq_out);   // no merge needed
            else st_ll(po + i, __float_as_uint(o), seq_out);
        }
        if (nact > 1 && tid < G) {
            st_ll(pml + 2 * tid, __float_as_uint(sh.hm[tid]), seq_out);
            st_ll(pml + 2 * tid + 1, __float_as_uint(sh.hl[tid]), seq_out);
        }
        attn_sync();      // shared memory is reused by the next item
    }
    // ---- merge (after ALL of this CTA's items, so that no CTA waits for a partial it has yet to produce)
    if (nact > 1 && cta < P.n_kv_heads) {
        const int kvh = cta;
        for (int i = tid; i < G * ATT_D; i += 256) {
            const int g = i / ATT_D;
            uint32_t spins = 0;
            unsigned long long t0 = 0;
            float Mx, Lt, Ot;
            while (true) {
                bool good = true;
                Mx = -INFINITY;
                for (int cc = first_chunk; cc < nchunk; ++cc) {
                    const uint2 m = ld_ll(P.part_ml + (((size_t)kvh * P.max_splits + cc) * G + g) * 2);
                    good = good && m.y == seq_out;
                    Mx = fmaxf(Mx, __uint_as_float(m.x));
                }
                Lt = 0.f;
                Ot = 0.f;
                for (int cc = first_chunk; cc < nchunk; ++cc) {
                    const uint2* ml = P.part_ml + (((size_t)kvh * P.max_splits + cc) * G + g) * 2;
                    const uint2 m = ld_ll(ml), l = ld_ll(ml + 1);
                    const uint2 o = ld_ll(P.part_o + ((size_t)kvh * P.max_splits + cc) * G * ATT_D + i);
                    good = good && l.y == seq_out && o.y == seq_out;
                    const float w = exp2f(__uint_as_float(m.x) - Mx);
                    Lt += w * __uint_as_float(l.x);
                    Ot += w * __uint_as_float(o.x);
                }
                if (good || W.expired(spins, t0)) break;
            }
            st_ll(P.att_ll + (size_t)kvh * G * ATT_D + i, __float_as_uint(Ot / Lt), seq_out);
        }
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
        const MegaWait W{abort_flag, P.status};
        const uint32_t gen = __ldcg(P.gen);
        const uint32_t seq0 = gen * (uint32_t)P.n_ops + 1u;          // sequence number of op 0 of this token
        uint32_t gbase = 0;              // ring position of this CTA's first tile of the current op
        auto stamp = [&](int oi, int k) {
            if (P.trace && tid == 0 && cta == 0) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                P.trace[(size_t)oi * 8 + k] = t;
            }
        };
        for (int oi = 0; oi < P.n_ops; ++oi) {
            const MegaOp& op = P.ops[oi];
            const uint32_t seq = seq0 + (uint32_t)oi;
            stamp(oi, 0);
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
                    v *= P.emb_scale;
                    P.x[i] = v;
                    st_ll(P.x_ll + i, __float_as_uint(v), seq);
                }
            } else if (op.kind == MK_ATTN) {
                if (tid < 256) {
                    switch (P.group) {
                        case 1: mega_attn<1>(P, op, smem + P.off_attn, cta, n_ctas, seq - 1, seq, W); break;
                        case 2: mega_attn<2>(P, op, smem + P.off_attn, cta, n_ctas, seq - 1, seq, W); break;
                        case 4: mega_attn<4>(P, op, smem + P.off_attn, cta, n_ctas, seq - 1, seq, W); break;
                        default: mega_attn<8>(P, op, smem + P.off_attn, cta, n_ctas, seq - 1, seq, W); break;
                    }
                }
            } else {
                // ---------------------------------------------------------------- GEMV
                const MegaShare sh = mega_share(op, cta);
                const GemvJob J = op.job[sh.ji];
                const int r0 = sh.r0, r1 = sh.r1, RW = J.RW, KS = J.KS, qtype = J.qtype;
                const int op_epi = op.epilogue, op_gelu = op.act_gelu;
                const uint2* op_resid = op.resid_ll;
                uint2* out_ll = op.out_ll[sh.ji];
                const bool paired = J.w2 != nullptr;
                const int sz0 = seg_bytes(qtype, J.seg_base), sz1 = seg_bytes(qtype, J.seg_base + 1);
                if (sh.nitems > 0)
                    mega_quantize_input<NT, QITEMS>(op.x_ll, seq0 + (uint32_t)op.src_op, op.norm_w, op.eps, op.norm_add_one, op.K, xq, xs,
                                                    xsf, xsf32, misc, W);
                stamp(oi, 2);
                const int grp = lane >> 2, lane4 = lane & 3;
                const int gprw = 8 / RW;
                const int my_row = grp % RW, my_j = grp / RW;
                float best_v = -INFINITY;
                int best_i = 0x7fffffff;
                bool ok = true;
                auto epilogue = [&](int n, float v0, float v1) {
                    if (J.bias) v0 += J.bias[n];
                    float r = v0;
                    switch (op_epi) {
                        case EPI_STORE: break;
                        case EPI_RESID: r = __uint_as_float(ld_ll(op_resid + n).x) + v0; break;
                        case EPI_GATED: r = (op_gelu ? gelu_tanh(v0) : silu(v0)) * v1; break;
                        case EPI_ARGMAX:
                            if (P.logits) P.logits[n] = v0;
                            if (v0 > best_v || (v0 == best_v && n < best_i)) { best_v = v0; best_i = n; }
                            return;
                    }
                    if (J.out) J.out[n] = r;
                    if (out_ll) st_ll(out_ll + n, __float_as_uint(r), seq);
                };
                long long c_wait = 0, c_dot = 0, c_epi = 0;
                const bool prof = P.trace && cta == 0 && warp == 0;
                uint32_t slot = (gbase + (uint32_t)warp) % NS, phase = ((gbase + (uint32_t)warp) / NS) & 1u;
                for (int it = warp; it < sh.nitems; it += NCONS) {
                    const long long c0 = prof ? clock64() : 0;
                    const MegaItem g = mega_geom(J, r0, r1, it, sz0, sz1);
                    if (ok) {
                        if (*abort_flag) ok = false;
                        else if (!mbar_wait(&full[slot], phase, P.status)) { *abort_flag = 1; ok = false; }
                    }
                    const uint8_t* tile = ring + (size_t)slot * P.slot_bytes;
                    float a0 = 0.f, a1 = 0.f;
                    const long long c1 = prof ? clock64() : 0;
                    if (ok && my_row < g.rows) {
                        const uint8_t* rowp = tile + (size_t)my_row * g.sb;
                        const int8_t* xq_s = xq + g.boff * 256;
                        const float* xs_s = xs + g.boff * 8;
                        const float* xsf_s = xsf + g.boff * 16;
                        const float* xsf32_s = xsf32 + g.boff * 8;
                        const bool swap = (grp & 1) && (((g.sb >> 4) & 1) == 0);
                        const size_t poff = (size_t)RW * g.sb;
                        if (qtype == QT_Q4K) {
                            if (paired) tile_dots<QT_Q4K, true>(rowp, poff, g.nb, my_j, gprw, lane4, swap, xq_s, xs_s, xsf_s, xsf32_s, a0, a1);
                            else tile_dots<QT_Q4K, false>(rowp, poff, g.nb, my_j, gprw, lane4, swap, xq_s, xs_s, xsf_s, xsf32_s, a0, a1);
                        } else {
                            if (paired) tile_dots<QT_Q6K, true>(rowp, poff, g.nb, my_j, gprw, lane4, swap, xq_s, xs_s, xsf_s, xsf32_s, a0, a1);
                            else tile_dots<QT_Q6K, false>(rowp, poff, g.nb, my_j, gprw, lane4, swap, xq_s, xs_s, xsf_s, xsf32_s, a0, a1);
                        }
                    }
                    __syncwarp();
                    const long long c2 = prof ? clock64() : 0;
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
                    if (prof) { __syncwarp(); const long long c3 = clock64(); c_wait += c1 - c0; c_dot += c2 - c1; c_epi += c3 - c2; }
                    slot += NCONS;                         // NCONS < NS: at most one wrap per step
                    if (slot >= (uint32_t)NS) { slot -= NS; phase ^= 1u; }
                }
                if (prof && lane == 0) { P.trace[(size_t)oi * 8 + 5] = c_wait; P.trace[(size_t)oi * 8 + 6] = c_dot; P.trace[(size_t)oi * 8 + 7] = c_epi; }
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
                            *P.gen = gen + 1u;
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
            cons_sync<NT>();       // shared memory (quantised input, accumulators) is rewritten by the next op
        }
    }
    __syncthreads();
}

}  // namespace ptb
