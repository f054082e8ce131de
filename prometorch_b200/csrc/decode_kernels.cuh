// Device code of the batch-1 decode path.
//
//  * gemv_kernel: weight-streaming dequant-GEMV for Q4_K / Q6_K.  Weights are
//    pulled into a shared-memory ring by untiled bulk async copies (TMA) issued
//    before the kernel waits on its predecessor (the weights never depend on
//    it), the input vector is RMS-normalised and quantised to int8 blocks of 32
//    in the prologue, and the dot products run on dp4a.  Epilogues: plain store,
//    residual add, SiLU/GELU-gated product of a gate/up pair, arg-max over the
//    whole output (two-stage, last CTA finishes), and the tensor-parallel
//    variant that pushes partial sums to every peer GPU and reduces them.
//  * attn_decode_kernel: per-KV-head split-KV attention for one new token with
//    the per-head QK RMSNorm, RoPE and the fp16 KV-cache write fused in.
//  * embed_kernel: dequantise one embedding row chosen by a device-side token id.
//
// The reference's counterparts are the 17 kernels of
// aten/src/ATen/cuda/CUDAQuantGemv.cu and the 9 of FlashDecoding.cu.
#pragma once
#include "common.cuh"

namespace ptb {

constexpr int GEMV_THREADS = 512;
constexpr int GEMV_GROUPS = GEMV_THREADS / 8;   // one 8-lane group works on one (row, super-block)
constexpr int GEMV_MAX_JOBS = 3;
constexpr int MAX_PEERS = 8;

enum QType : int { QT_Q4K = 0, QT_Q6K = 1 };
enum Epilogue : int { EPI_STORE = 0, EPI_RESID = 1, EPI_GATED = 2, EPI_ARGMAX = 3, EPI_ALLREDUCE = 4 };

// Row layouts in device memory (produced once at load time):
//   Q4_K: the GGUF bytes as they are: nblk x {fp16 d, fp16 dmin, 12 B scales, 128 B quants}.
//   Q6_K: structure-of-arrays per row so every section is 16 B aligned:
//         ql[nblk*128] | qh[nblk*64] | int8 scales[nblk*16] | fp16 d[nblk] padded to 16 B.
struct GemvJob {
    const uint8_t* w;
    const uint8_t* w2;      // second matrix of a gated pair (same shape and type) or null
    const float* bias;      // optional [N]
    float* out;
    int qtype, N, rowbytes, nblk;
    int R;                  // rows per pipeline stage
    int gpr;                // 8-lane groups cooperating on one row
    int cta_begin, cta_count;
};

struct PeerInfo {           // tensor-parallel all-reduce wiring (EPI_ALLREDUCE)
    float* inbox[MAX_PEERS];        // inbox[p]: peer p's receive buffer [world][slot_floats]; inbox[rank] is local
    uint32_t* flag[MAX_PEERS];      // flag[p]: peer p's arrival counters [world]
    int rank, world;
    int slot_floats;
    uint32_t seq_mul, seq_add;      // arrival number of this call = generation * seq_mul + seq_add
};

struct GemvParams {
    GemvJob job[GEMV_MAX_JOBS];
    int njobs;
    const float* x;         // input vector [K] fp32
    const float* norm_w;    // RMSNorm weight [K] or null (no normalisation)
    float eps;
    int norm_add_one;
    int K;
    int epilogue;
    int act_gelu;
    const float* resid;     // EPI_RESID / EPI_ALLREDUCE: added to the result
    // EPI_ARGMAX scratch
    float* amax_val;        // [grid]
    int* amax_idx;          // [grid]
    unsigned* ticket;
    float* logits;          // optional full output [N] (sampling path)
    int* result;            // result[0] = arg-max id
    int row_offset;         // global id of row 0 (row-split lm_head under tensor parallelism)
    // decode control block (device): {token, pos, step, self_feed, max_log} + log
    int* ctrl;
    int* token_log;
    const int* token_script;   // self_feed == 2: tokens to feed (a prompt) before switching to the arg-max
    // EPI_ALLREDUCE
    PeerInfo peers;
    const uint32_t* gen;    // device generation counter (monotonic, one per token)
    int* status;
    int stages, stage_bytes;
};

// control block indices
enum { CTRL_TOKEN = 0, CTRL_POS = 1, CTRL_STEP = 2, CTRL_SELF_FEED = 3, CTRL_LOG_CAP = 4, CTRL_GEN = 5, CTRL_SCRIPT_LEN = 6, CTRL_WORDS = 8 };

__device__ __forceinline__ int dp4a_s(int a, int b, int c) { return __dp4a(a, b, c); }

// One 8-lane group x one Q4_K super-block.  bp -> 144 B block in shared memory.
__device__ __forceinline__ float q4k_dot(const uint8_t* bp, int lane8, const int8_t* xq, const float* xs, const float* xsf) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(bp);
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    const int j = lane8 >> 1, hf = lane8 & 1;
    const uint4 qv = *reinterpret_cast<const uint4*>(bp + 16 + lane8 * 16);
    const uint4 xl = *reinterpret_cast<const uint4*>(xq + j * 64 + hf * 16);
    const uint4 xh = *reinterpret_cast<const uint4*>(xq + j * 64 + 32 + hf * 16);
    int dlo = dp4a_s(qv.x & 0x0F0F0F0F, xl.x, 0);
    dlo = dp4a_s(qv.y & 0x0F0F0F0F, xl.y, dlo);
    dlo = dp4a_s(qv.z & 0x0F0F0F0F, xl.z, dlo);
    dlo = dp4a_s(qv.w & 0x0F0F0F0F, xl.w, dlo);
    int dhi = dp4a_s((qv.x >> 4) & 0x0F0F0F0F, xh.x, 0);
    dhi = dp4a_s((qv.y >> 4) & 0x0F0F0F0F, xh.y, dhi);
    dhi = dp4a_s((qv.z >> 4) & 0x0F0F0F0F, xh.z, dhi);
    dhi = dp4a_s((qv.w >> 4) & 0x0F0F0F0F, xh.w, dhi);
    const uint32_t s0 = hdr.y, s1 = hdr.z, s2 = hdr.w;
    int sc_lo, m_lo, sc_hi, m_hi;
    if (j < 2) {
        const int sh = 16 * j;
        sc_lo = (s0 >> sh) & 63;        m_lo = (s1 >> sh) & 63;
        sc_hi = (s0 >> (sh + 8)) & 63;  m_hi = (s1 >> (sh + 8)) & 63;
    } else {
        const int sh = 16 * (j - 2);
        sc_lo = ((s2 >> sh) & 0xF) | (((s0 >> (sh + 6)) & 3) << 4);
        m_lo = ((s2 >> (sh + 4)) & 0xF) | (((s1 >> (sh + 6)) & 3) << 4);
        sc_hi = ((s2 >> (sh + 8)) & 0xF) | (((s0 >> (sh + 14)) & 3) << 4);
        m_hi = ((s2 >> (sh + 12)) & 0xF) | (((s1 >> (sh + 14)) & 3) << 4);
    }
    const float a = (float)sc_lo * xs[2 * j] * (float)dlo + (float)sc_hi * xs[2 * j + 1] * (float)dhi;
    const float b = (float)m_lo * xsf[4 * j + hf] + (float)m_hi * xsf[4 * j + 2 + hf];
    return d * a - dmin * b;
}

// One 8-lane group x one Q6_K super-block of a structure-of-arrays row.
__device__ __forceinline__ float q6k_dot(const uint8_t* row, int nblk, int blk, int lane8, const int8_t* xq, const float* xs,
                                         const float* xsf) {
    const uint8_t* ql = row + blk * 128;
    const uint8_t* qh = row + nblk * 128 + blk * 64;
    const int8_t* sc = reinterpret_cast<const int8_t*>(row + nblk * 192 + blk * 16);
    const float d = __half2float(*reinterpret_cast<const __half*>(row + nblk * 208 + blk * 2));
    const int n = lane8 >> 2, q = lane8 & 3, which = q >> 1, l0 = (q & 1) * 16;
    const uint4 qlv = *reinterpret_cast<const uint4*>(ql + n * 64 + q * 16);
    const uint4 qhv = *reinterpret_cast<const uint4*>(qh + n * 32 + l0);
    const int e_lo = n * 128 + which * 32 + l0, e_hi = e_lo + 64;
    const int sh_lo = which * 2, sh_hi = 4 + which * 2;
    const uint4 xl = *reinterpret_cast<const uint4*>(xq + e_lo);
    const uint4 xh = *reinterpret_cast<const uint4*>(xq + e_hi);
#define PTB_Q6_LO(c) ((qlv.c & 0x0F0F0F0F) | (((qhv.c >> sh_lo) & 0x03030303) << 4))
#define PTB_Q6_HI(c) (((qlv.c >> 4) & 0x0F0F0F0F) | (((qhv.c >> sh_hi) & 0x03030303) << 4))
    int dlo = dp4a_s(PTB_Q6_LO(x), xl.x, 0);
    dlo = dp4a_s(PTB_Q6_LO(y), xl.y, dlo);
    dlo = dp4a_s(PTB_Q6_LO(z), xl.z, dlo);
    dlo = dp4a_s(PTB_Q6_LO(w), xl.w, dlo);
    int dhi = dp4a_s(PTB_Q6_HI(x), xh.x, 0);
    dhi = dp4a_s(PTB_Q6_HI(y), xh.y, dhi);
    dhi = dp4a_s(PTB_Q6_HI(z), xh.z, dhi);
    dhi = dp4a_s(PTB_Q6_HI(w), xh.w, dhi);
#undef PTB_Q6_LO
#undef PTB_Q6_HI
    const float a = (float)sc[e_lo >> 4] * (xs[e_lo >> 5] * (float)dlo - 32.0f * xsf[e_lo >> 4]);
    const float b = (float)sc[e_hi >> 4] * (xs[e_hi >> 5] * (float)dhi - 32.0f * xsf[e_hi >> 4]);
    return d * (a + b);
}

// Block-wide sum through shared memory; `buf` needs >= 32 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* buf) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) buf[w] = v;
    __syncthreads();
    float t = (l < (int)(blockDim.x >> 5)) ? buf[l] : 0.0f;
    t = warp_sum(t);
    return t;
}

// Load x[K], optionally RMS-normalise, quantise to int8 blocks of 32.
//   xq[K] int8, xs[K/32] block scales, xsf[K/16] = scale * (sum of the 16 int8 values).
__device__ __forceinline__ void quantize_input(const float* __restrict__ x, const float* __restrict__ norm_w, float eps,
                                               int add_one, int K, int8_t* xq, float* xs, float* xsf, float* red) {
    const int tid = threadIdx.x, nt = blockDim.x;
    float rs = 1.0f;
    if (norm_w) {
        float ss = 0.f;
        for (int i = tid; i < K / 4; i += nt) {
            const float4 v = reinterpret_cast<const float4*>(x)[i];
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum(ss, red);
        rs = rsqrtf(ss / (float)K + eps);
    }
    const int items = K / 8;
    const int rounds = (items + nt - 1) / nt;
    for (int r = 0; r < rounds; ++r) {
        const int i = r * nt + tid;
        float v[8];
        if (i < items) {
            const float4 a = reinterpret_cast<const float4*>(x)[2 * i], b = reinterpret_cast<const float4*>(x)[2 * i + 1];
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            if (norm_w) {
                const float4 wa = reinterpret_cast<const float4*>(norm_w)[2 * i], wb = reinterpret_cast<const float4*>(norm_w)[2 * i + 1];
                const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = v[k] * rs * (add_one ? 1.0f + w[k] : w[k]);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = 0.f;
        }
        float am = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) am = fmaxf(am, fabsf(v[k]));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
        const float sc = am / 127.0f;
        const float inv = am > 0.f ? 127.0f / am : 0.f;
        int q[8], s = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) { q[k] = __float2int_rn(v[k] * inv); s += q[k]; }
        const int s16 = s + __shfl_xor_sync(0xffffffffu, s, 1);
        if (i < items) {
            uint2 pk;
            pk.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((q[3] & 0xff) << 24);
            pk.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((q[7] & 0xff) << 24);
            reinterpret_cast<uint2*>(xq)[i] = pk;
            if ((i & 1) == 0) xsf[i >> 1] = sc * (float)s16;
            if ((i & 3) == 0) xs[i >> 2] = sc;
        }
    }
    __syncthreads();
}

__device__ __forceinline__ size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const __grid_constant__ GemvParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const int K = P.K;
    // ---- shared memory carve-up
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);                       // [stages]
    float* red = reinterpret_cast<float*>(smem + 128);                        // [2][2*GROUPS] + 32 scratch
    float* misc = red + 4 * GEMV_GROUPS;                                      // 64 floats
    int8_t* xq = reinterpret_cast<int8_t*>(misc + 64);
    float* xs = reinterpret_cast<float*>(xq + K);
    float* xsf = xs + K / 32;
    uint8_t* stage0 = smem + align_up(128 + (4 * GEMV_GROUPS + 64) * 4 + K + (K / 32) * 4 + (K / 16) * 4, 128);

    // ---- which job and which rows are mine
    int ji = 0;
#pragma unroll
    for (int i = 1; i < GEMV_MAX_JOBS; ++i)
        if (i < P.njobs && (int)blockIdx.x >= P.job[i].cta_begin) ji = i;
    const GemvJob& J = P.job[ji];
    const int ci = blockIdx.x - J.cta_begin;
    const int r0 = (int)(((long long)J.N * ci) / J.cta_count);
    const int r1 = (int)(((long long)J.N * (ci + 1)) / J.cta_count);
    const int R = J.R;
    const int nchunks = (r1 - r0 + R - 1) / R;
    const bool paired = J.w2 != nullptr;
    const int S = P.stages;
    const uint32_t mat_bytes = (uint32_t)R * J.rowbytes;   // one matrix's share of a full stage

    auto issue = [&](int c) {   // thread 0 only
        const int s = c % S;
        const int rows = min(R, r1 - (r0 + c * R));
        const uint32_t bytes = (uint32_t)rows * J.rowbytes;
        uint8_t* dst = stage0 + (size_t)s * P.stage_bytes;
        mbar_expect_tx(&full[s], paired ? 2 * bytes : bytes);
        bulk_g2s(dst, J.w + (size_t)(r0 + c * R) * J.rowbytes, bytes, &full[s]);
        if (paired) bulk_g2s(dst + mat_bytes, J.w2 + (size_t)(r0 + c * R) * J.rowbytes, bytes, &full[s]);
    };

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
        fence_proxy_async();
        // weights do not depend on the previous kernel: start streaming them now
        for (int c = 0; c < S && c < nchunks; ++c) issue(c);
    }
    pdl_launch_dependents();
    pdl_wait();
    __syncthreads();

    quantize_input(P.x, P.norm_w, P.eps, P.norm_add_one, K, xq, xs, xsf, misc);

    const int grp = tid >> 3, lane8 = tid & 7;
    const int gpr = J.gpr;
    const int my_row = grp / gpr, my_j = grp - my_row * gpr;
    const bool grp_active = my_row < R;
    const int nblk = J.nblk;
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    bool ok = true;

    for (int c = 0; c < nchunks; ++c) {
        const int s = c % S;
        const int rows = min(R, r1 - (r0 + c * R));
        if (ok) ok = mbar_wait(&full[s], (uint32_t)((c / S) & 1), P.status);
        const uint8_t* st = stage0 + (size_t)s * P.stage_bytes;
        float a0 = 0.f, a1 = 0.f;
        if (ok && grp_active && my_row < rows) {
            const uint8_t* rowp = st + (size_t)my_row * J.rowbytes;
            if (J.qtype == QT_Q4K) {
                for (int b = my_j; b < nblk; b += gpr) {
                    a0 += q4k_dot(rowp + b * 144, lane8, xq + b * 256, xs + b * 8, xsf + b * 16);
                    if (paired) a1 += q4k_dot(rowp + mat_bytes + b * 144, lane8, xq + b * 256, xs + b * 8, xsf + b * 16);
                }
            } else {
                for (int b = my_j; b < nblk; b += gpr) {
                    a0 += q6k_dot(rowp, nblk, b, lane8, xq + b * 256, xs + b * 8, xsf + b * 16);
                    if (paired) a1 += q6k_dot(rowp + mat_bytes, nblk, b, lane8, xq + b * 256, xs + b * 8, xsf + b * 16);
                }
            }
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            a0 += __shfl_xor_sync(0xffffffffu, a0, o);
            a1 += __shfl_xor_sync(0xffffffffu, a1, o);
        }
        float* rb = red + (c & 1) * 2 * GEMV_GROUPS;
        if (lane8 == 0) { rb[grp] = a0; rb[GEMV_GROUPS + grp] = a1; }
        __syncthreads();
        if (tid == 0 && c + S < nchunks) issue(c + S);
        if (tid < rows) {
            float v0 = 0.f, v1 = 0.f;
            for (int j = 0; j < gpr; ++j) { v0 += rb[tid * gpr + j]; v1 += rb[GEMV_GROUPS + tid * gpr + j]; }
            const int n = r0 + c * R + tid;
            if (J.bias) v0 += J.bias[n];
            switch (P.epilogue) {
                case EPI_STORE: J.out[n] = v0; break;
                case EPI_RESID: J.out[n] = P.resid[n] + v0; break;
                case EPI_GATED: J.out[n] = (P.act_gelu ? gelu_tanh(v0) : silu(v0)) * v1; break;
                case EPI_ARGMAX:
                    if (P.logits) P.logits[n] = v0;
                    if (v0 > best_v) { best_v = v0; best_i = n; }
                    break;
                case EPI_ALLREDUCE: {
                    // push my partial sum for element n to every rank's inbox slot [rank]
                    const PeerInfo& pi = P.peers;
                    for (int p = 0; p < pi.world; ++p) pi.inbox[p][(size_t)pi.rank * pi.slot_floats + n] = v0;
                } break;
            }
        }
    }

    if (P.epilogue == EPI_ARGMAX) {
        // CTA arg-max (ties -> lowest index), then the last CTA to arrive finishes across CTAs.
        __syncthreads();
        float* sv = red;
        int* si = reinterpret_cast<int*>(red + GEMV_GROUPS);
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
        }
        if ((tid & 31) == 0) { sv[tid >> 5] = best_v; si[tid >> 5] = best_i; }
        __syncthreads();
        __shared__ bool is_last;
        if (tid == 0) {
            for (int w = 1; w < GEMV_THREADS / 32; ++w)
                if (sv[w] > best_v || (sv[w] == best_v && si[w] < best_i)) { best_v = sv[w]; best_i = si[w]; }
            P.amax_val[blockIdx.x] = best_v;
            P.amax_idx[blockIdx.x] = best_i;
            __threadfence();
            const unsigned t = atomicAdd(P.ticket, 1u);
            is_last = (t == gridDim.x - 1);
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int i = tid; i < (int)gridDim.x; i += GEMV_THREADS) {
                const float v = __ldcg(P.amax_val + i);
                const int ix = __ldcg(P.amax_idx + i);
                if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            __syncthreads();
            if ((tid & 31) == 0) { sv[tid >> 5] = bv; si[tid >> 5] = bi; }
            __syncthreads();
            if (tid == 0) {
                for (int w = 1; w < GEMV_THREADS / 32; ++w)
                    if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
                *P.ticket = 0u;
                bi += P.row_offset;
                const PeerInfo& pi = P.peers;
                if (pi.world > 1) {
                    // every rank holds a slice of the vocabulary: exchange {value, id} pairs and
                    // let each rank pick the same winner
                    const uint32_t g = *P.gen * pi.seq_mul + pi.seq_add;
                    for (int p = 0; p < pi.world; ++p) {
                        float* slot = pi.inbox[p] + (size_t)pi.rank * pi.slot_floats;
                        slot[0] = bv;
                        slot[1] = __int_as_float(bi);
                    }
                    __threadfence_system();
                    for (int p = 0; p < pi.world; ++p) st_release_sys(pi.flag[p] + pi.rank, g);
                    for (int p = 0; p < pi.world; ++p) wait_flag_ge(pi.flag[pi.rank] + p, g, P.status);
                    bv = -INFINITY;
                    bi = 0x7fffffff;
                    for (int p = 0; p < pi.world; ++p) {
                        const float* slot = pi.inbox[pi.rank] + (size_t)p * pi.slot_floats;
                        const float v = __ldcg(slot);
                        const int ix = __float_as_int(__ldcg(slot + 1));
                        if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
                    }
                }
                P.result[0] = bi;
                reinterpret_cast<float*>(P.result)[1] = bv;
                if (P.ctrl) {
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

    if (P.epilogue == EPI_ALLREDUCE) {
        // All CTAs have pushed their slices; the last CTA of this rank publishes the
        // arrival flag to every peer, waits for all peers, reduces the `world` partial
        // vectors of its inbox in rank order (bitwise identical on every rank) and adds
        // the residual.
        const PeerInfo& pi = P.peers;
        __shared__ bool last;
        __syncthreads();
        if (tid == 0) {
            __threadfence_system();
            const unsigned t = atomicAdd(P.ticket, 1u);
            last = (t == gridDim.x - 1);
            __threadfence();
        }
        __syncthreads();
        if (last) {
            const uint32_t g = *P.gen * pi.seq_mul + pi.seq_add;
            if (tid < pi.world) {
                __threadfence_system();
                st_release_sys(pi.flag[tid] + pi.rank, g);
            }
            __syncthreads();
            if (tid < pi.world) wait_flag_ge(pi.flag[pi.rank] + tid, g, P.status);
            __syncthreads();
            const float* in = pi.inbox[pi.rank];
            const int N = J.N;
            for (int n = tid; n < N; n += GEMV_THREADS) {
                float v = P.resid ? P.resid[n] : 0.f;
                for (int p = 0; p < pi.world; ++p) v += __ldcg(in + (size_t)p * pi.slot_floats + n);
                J.out[n] = v;
            }
            if (tid == 0) *P.ticket = 0u;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Attention for one new token.
// grid (kv_heads, max_splits), 256 threads.  Split s covers cache positions [s*128, s*128+128).
// q/k/v for the new token arrive as fp32 rows of `qkv` (q: heads*d, then k: kv_heads*d, then v);
// the CTA owning the split that contains `pos` normalises/rotates K and writes K,V to the fp16 cache.
constexpr int ATT_THREADS = 256;
constexpr int ATT_CHUNK = 128;
constexpr int ATT_D = 128;
constexpr int ATT_MAX_GROUP = 8;

struct AttnParams {
    const float* q;          // [heads*d]
    const float* k;          // [kv_heads*d]
    const float* v;          // [kv_heads*d]
    const float* q_norm;     // [d] or null
    const float* k_norm;     // [d] or null
    const float* cos;        // [max_seq][d/2]
    const float* sin;
    __half* k_cache;         // [kv_heads][max_seq][d]
    __half* v_cache;
    float* out;              // [heads*d]
    float* part_o;           // [kv_heads][max_splits][group][d]
    float* part_ml;          // [kv_heads][max_splits][group][2]
    unsigned* ticket;        // [kv_heads]
    const int* ctrl;
    int group;               // q heads per kv head
    int max_seq;
    int max_splits;
    int neox;
    float eps;
    float scale;
    int window;              // sliding window (0 = full)
};

__device__ __forceinline__ void norm_rope_head(const float* src, const float* nw, float eps, const float* cs, const float* sn,
                                               int neox, float mul, float* dst /*smem [128]*/, int lane) {
    // one warp processes one head of 128 values: lane holds 4 values
    float v[4];
    if (neox) { v[0] = src[lane]; v[1] = src[lane + 32]; v[2] = src[lane + 64]; v[3] = src[lane + 96]; }
    else { const float4 t = reinterpret_cast<const float4*>(src)[lane]; v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    if (nw) {
        float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        ss = warp_sum(ss);
        const float rs = rsqrtf(ss / 128.0f + eps);
        if (neox) { v[0] *= rs * nw[lane]; v[1] *= rs * nw[lane + 32]; v[2] *= rs * nw[lane + 64]; v[3] *= rs * nw[lane + 96]; }
        else { const float4 w = reinterpret_cast<const float4*>(nw)[lane]; v[0] *= rs * w.x; v[1] *= rs * w.y; v[2] *= rs * w.z; v[3] *= rs * w.w; }
    }
    if (neox) {
        // pairs (i, i+64): lane owns i = lane and lane+32
        const float c0 = cs[lane], s0 = sn[lane], c1 = cs[lane + 32], s1 = sn[lane + 32];
        dst[lane] = (v[0] * c0 - v[2] * s0) * mul;
        dst[lane + 64] = (v[2] * c0 + v[0] * s0) * mul;
        dst[lane + 32] = (v[1] * c1 - v[3] * s1) * mul;
        dst[lane + 96] = (v[3] * c1 + v[1] * s1) * mul;
    } else {
        // pairs (2i, 2i+1): lane owns i = 2*lane, 2*lane+1
        const float c0 = cs[2 * lane], s0 = sn[2 * lane], c1 = cs[2 * lane + 1], s1 = sn[2 * lane + 1];
        dst[4 * lane + 0] = (v[0] * c0 - v[1] * s0) * mul;
        dst[4 * lane + 1] = (v[1] * c0 + v[0] * s0) * mul;
        dst[4 * lane + 2] = (v[2] * c1 - v[3] * s1) * mul;
        dst[4 * lane + 3] = (v[3] * c1 + v[2] * s1) * mul;
    }
}

__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(const __grid_constant__ AttnParams P) {
    __shared__ __align__(16) float qs[ATT_MAX_GROUP][ATT_D];
    __shared__ __align__(16) float kn[ATT_D];
    __shared__ float sc[ATT_MAX_GROUP][ATT_CHUNK];
    __shared__ float hm[ATT_MAX_GROUP], hl[ATT_MAX_GROUP];
    __shared__ __align__(16) float red[ATT_THREADS / 32][ATT_MAX_GROUP][ATT_D];   // 32 KB
    __shared__ bool last;

    pdl_launch_dependents();
    pdl_wait();

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x, split = blockIdx.y;
    const int pos = P.ctrl[CTRL_POS];
    const int T = pos + 1;
    const int lo = (P.window > 0 && T > P.window) ? T - P.window : 0;     // first visible position
    const int first_split = lo / ATT_CHUNK;
    const int nsplit = (T + ATT_CHUNK - 1) / ATT_CHUNK;
    if (split >= nsplit || split < first_split || pos >= P.max_seq) return;
    const int nactive = nsplit - first_split;
    const int G = P.group;
    const int t0 = max(split * ATT_CHUNK, lo), t1 = min(split * ATT_CHUNK + ATT_CHUNK, T);
    const int base = split * ATT_CHUNK;
    const float* cs = P.cos + (size_t)pos * (ATT_D / 2);
    const float* sn = P.sin + (size_t)pos * (ATT_D / 2);
    __half* kc = P.k_cache + (size_t)kvh * P.max_seq * ATT_D;
    __half* vc = P.v_cache + (size_t)kvh * P.max_seq * ATT_D;

    // ---- prologue: q heads of this group (normalised, rotated, pre-scaled); new K/V into the cache
    if (warp < G) norm_rope_head(P.q + (size_t)(kvh * G + warp) * ATT_D, P.q_norm, P.eps, cs, sn, P.neox, P.scale, qs[warp], lane);
    const bool owns_new = (pos >= base && pos < base + ATT_CHUNK);
    if (owns_new && warp == ATT_THREADS / 32 - 1) {
        norm_rope_head(P.k + (size_t)kvh * ATT_D, P.k_norm, P.eps, cs, sn, P.neox, 1.0f, kn, lane);
        __syncwarp();
        for (int i = lane; i < ATT_D; i += 32) {
            kc[(size_t)pos * ATT_D + i] = __float2half_rn(kn[i]);
            vc[(size_t)pos * ATT_D + i] = __float2half_rn(P.v[(size_t)kvh * ATT_D + i]);
        }
    }
    __syncthreads();

    // ---- scores: two threads per cache position, 64 dims each
    {
        const int tl = tid >> 1, hf = tid & 1;
        const int t = base + tl;
        float s[ATT_MAX_GROUP];
#pragma unroll
        for (int g = 0; g < ATT_MAX_GROUP; ++g) s[g] = 0.f;
        if (t >= t0 && t < t1) {
            const uint4* kp = reinterpret_cast<const uint4*>(kc + (size_t)t * ATT_D + hf * 64);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 raw = kp[i];
                const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
                float kf[8];
#pragma unroll
                for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h2[k]); kf[2 * k] = f.x; kf[2 * k + 1] = f.y; }
#pragma unroll
                for (int g = 0; g < ATT_MAX_GROUP; ++g) {
                    if (g < G) {
                        const float* qp = &qs[g][hf * 64 + i * 8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) s[g] += kf[k] * qp[k];
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < ATT_MAX_GROUP; ++g) {
            if (g < G) {
                const float tot = s[g] + __shfl_xor_sync(0xffffffffu, s[g], 1);
                if (hf == 0) sc[g][tl] = (t >= t0 && t < t1) ? tot : -INFINITY;
            }
        }
    }
    __syncthreads();
    // ---- softmax statistics of this split: warp g handles head g
    if (warp < G) {
        float m = -INFINITY;
        for (int i = lane; i < ATT_CHUNK; i += 32) m = fmaxf(m, sc[warp][i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = lane; i < ATT_CHUNK; i += 32) {
            const float p = __expf(sc[warp][i] - m);
            sc[warp][i] = p;
            l += p;
        }
        l = warp_sum(l);
        if (lane == 0) { hm[warp] = m; hl[warp] = l; }
    }
    __syncthreads();
    // ---- P @ V: 16 row-groups x 16 column-threads (8 dims each)
    {
        const int rg = tid >> 4, dc = tid & 15;
        float acc[ATT_MAX_GROUP][8];
#pragma unroll
        for (int g = 0; g < ATT_MAX_GROUP; ++g)
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[g][k] = 0.f;
        for (int tl = rg; tl < ATT_CHUNK; tl += 16) {
            const int t = base + tl;
            if (t < t0 || t >= t1) continue;
            const uint4 raw = *reinterpret_cast<const uint4*>(vc + (size_t)t * ATT_D + dc * 8);
            const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
            float vf[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h2[k]); vf[2 * k] = f.x; vf[2 * k + 1] = f.y; }
#pragma unroll
            for (int g = 0; g < ATT_MAX_GROUP; ++g) {
                if (g < G) {
                    const float p = sc[g][tl];
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[g][k] += p * vf[k];
                }
            }
        }
        // lanes l and l+16 hold different row-groups of the same columns
#pragma unroll
        for (int g = 0; g < ATT_MAX_GROUP; ++g)
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[g][k] += __shfl_xor_sync(0xffffffffu, acc[g][k], 16);
        if (lane < 16) {
#pragma unroll
            for (int g = 0; g < ATT_MAX_GROUP; ++g)
                if (g < G) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) red[warp][g][dc * 8 + k] = acc[g][k];
                }
        }
    }
    __syncthreads();
    // ---- combine the 8 warps; write either the final output (single split) or a partial
    for (int i = tid; i < G * ATT_D; i += ATT_THREADS) {
        const int g = i / ATT_D, d = i - g * ATT_D;
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_THREADS / 32; ++w) o += red[w][g][d];
        if (nactive == 1) {
            P.out[(size_t)(kvh * G + g) * ATT_D + d] = o / hl[g];
        } else {
            P.part_o[(((size_t)kvh * P.max_splits + split) * G + g) * ATT_D + d] = o;
        }
    }
    if (nactive == 1) return;
    if (tid < G) {
        float* ml = P.part_ml + (((size_t)kvh * P.max_splits + split) * G + tid) * 2;
        ml[0] = hm[tid];
        ml[1] = hl[tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned t = atomicAdd(P.ticket + kvh, 1u);
        last = (t == (unsigned)nactive - 1);
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    for (int i = tid; i < G * ATT_D; i += ATT_THREADS) {
        const int g = i / ATT_D, d = i - g * ATT_D;
        float M = -INFINITY;
        for (int s = first_split; s < nsplit; ++s)
            M = fmaxf(M, __ldcg(P.part_ml + (((size_t)kvh * P.max_splits + s) * G + g) * 2));
        float L = 0.f, O = 0.f;
        for (int s = first_split; s < nsplit; ++s) {
            const size_t ix = ((size_t)kvh * P.max_splits + s) * G + g;
            const float w = __expf(__ldcg(P.part_ml + ix * 2) - M);
            L += w * __ldcg(P.part_ml + ix * 2 + 1);
            O += w * __ldcg(P.part_o + ix * ATT_D + d);
        }
        P.out[(size_t)(kvh * G + g) * ATT_D + d] = O / L;
    }
    if (tid == 0) P.ticket[kvh] = 0u;
}

// ---------------------------------------------------------------------------------------------
// Embedding row -> fp32 residual stream.  Row layouts as for the GEMV (Q4_K blocks / Q6_K SoA),
// plus fp16 (qtype 2) and fp32 (qtype 3).
struct EmbedParams {
    const uint8_t* table;
    int qtype, rowbytes, nblk, H;
    float scale;
    float* out;
    const int* ctrl;
    int vocab;
    int* status;
    uint32_t* gen;       // bumped once per token (tensor-parallel generation counter) or null
};

__global__ void __launch_bounds__(256) embed_kernel(const __grid_constant__ EmbedParams P) {
    pdl_launch_dependents();
    pdl_wait();
    int tok = P.ctrl[CTRL_TOKEN];
    if (tok < 0 || tok >= P.vocab) {
        if (threadIdx.x == 0) atomicExch(P.status, PTB_ERR_BOUNDS);
        tok = 0;
    }
    if (P.gen && blockIdx.x == 0 && threadIdx.x == 0) *P.gen = *P.gen + 1;
    const uint8_t* row = P.table + (size_t)tok * P.rowbytes;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < P.H; i += gridDim.x * blockDim.x) {
        float v;
        const int b = i >> 8, e = i & 255;
        if (P.qtype == QT_Q4K) {
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
        } else if (P.qtype == QT_Q6K) {
            const int n = e >> 7, r = e & 127, quad = r >> 5, l = r & 31;
            const uint8_t qlb = row[b * 128 + n * 64 + (quad & 1) * 32 + l];
            const uint8_t qhb = row[P.nblk * 128 + b * 64 + n * 32 + l];
            const int lo4 = (quad >> 1) ? (qlb >> 4) : (qlb & 0xF);
            const int hi2 = (qhb >> (2 * quad)) & 3;
            const int q = (lo4 | (hi2 << 4)) - 32;
            const int8_t scv = reinterpret_cast<const int8_t*>(row + P.nblk * 192 + b * 16)[e >> 4];
            const float d = __half2float(*reinterpret_cast<const __half*>(row + P.nblk * 208 + b * 2));
            v = d * scv * q;
        } else if (P.qtype == 2) {
            v = __half2float(reinterpret_cast<const __half*>(row)[i]);
        } else {
            v = reinterpret_cast<const float*>(row)[i];
        }
        P.out[i] = v * P.scale;
    }
}

}  // namespace ptb
