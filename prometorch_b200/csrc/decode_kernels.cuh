// Device code of the batch-1 decode path.
//
//  * gemv_kernel: weight-streaming dequant-GEMV for Q4_K / Q6_K.  Weights are
//    pulled into a shared-memory ring by untiled bulk async copies (TMA) issued
//    before the kernel waits on its predecessor (the weights never depend on
//    it), the input vector is RMS-normalised and quantised to int8 blocks of 32
//    in the prologue, and the dot products run on dp4a.  Epilogues: plain store,
//    residual add, SiLU/GELU-gated product of a gate/up pair, arg-max over the
//    whole output (two-stage, last CTA finishes), and the partial-sum push:
//    the result goes to slot [rank] of every GPU's inbox and the CONSUMING
//    kernel adds the partial sums (and the residual) while it loads its input.
//  * Inside the engine the kernels of a token do not wait for each other at
//    launch boundaries: every vector that passes from one kernel to the next is
//    a buffer of {value, sequence} slots, the consumer is already resident
//    (launched early, its weights on their way into shared memory) and polls
//    the slots, so a hand-over costs one store-to-load latency through L2.
//  * attn_decode_kernel: per-KV-head split-KV attention for one new token with
//    the per-head QK RMSNorm, RoPE and the fp16 KV-cache write fused in.
//  * embed_kernel: dequantise one embedding row chosen by a device-side token id.
//
// The reference's counterparts are the 17 kernels of
// aten/src/ATen/cuda/CUDAQuantGemv.cu and the 9 of FlashDecoding.cu.
#pragma once
#include "common.cuh"
#include <cooperative_groups.h>

namespace ptb {

constexpr int GEMV_MAX_WARPS = 16;
constexpr int GEMV_MAX_JOBS = 3;
constexpr int GEMV_SEG_BLOCKS = 10;             // K is cut into segments of at most this many 256-value super-blocks
constexpr int MAX_PEERS = 8;

// 2 / 3: fp16 / fp32 (row tables; fp16 also as a GEMV weight in the tile layout); Q5_K and Q8_0 exist in the tile layout only
enum QType : int { QT_Q4K = 0, QT_Q6K = 1, QT_F16 = 2, QT_F32 = 3, QT_Q5K = 4, QT_Q8_0 = 5 };
enum Epilogue : int { EPI_STORE = 0, EPI_RESID = 1, EPI_GATED = 2, EPI_ARGMAX = 3, EPI_PARTIAL = 4, EPI_ALLREDUCE = 5 };
constexpr uint32_t LL_SEQ_MUL = 256;            // sequence number = token generation * LL_SEQ_MUL + index of the write within the token

// Weight layout in device memory (produced once at load time), "segment-major":
//   K is cut into KS = ceil(nblk / 10) segments (the first nblk % KS of them one block longer);
//   the matrix is stored as [segment][row][segment bytes], so the same K-segment of consecutive
//   rows is contiguous and a warp's tile (1, 2 or 4 rows x one segment) is one bulk copy.
//   Q4_K segment of nb blocks: nb x {fp16 d, fp16 dmin, 12 B scales, 128 B quants} (the GGUF bytes).
//   Q6_K segment of nb blocks: ql[nb*128] | qh[nb*64] | int8 scales[nb*16] | fp16 d[nb] padded to 16 B.
__host__ __device__ __forceinline__ int seg_bytes(int qtype, int nb) {
    return qtype == QT_Q4K ? nb * 144 : nb * 208 + ((nb * 2 + 15) & ~15);
}

struct GemvJob {
    const uint8_t* w;
    const uint8_t* w2;      // second matrix of a gated pair (same shape and type) or null
    const float* bias;      // optional [N]
    float* out;             // plain fp32 output, or
    uint2* out_ll;          // {value, sequence} slots (engine dataflow)
    int qtype, N, nblk;
    int KS, seg_base, seg_rem;
    int RW;                 // rows per warp tile: 1, 2, 4 or 8 (8/RW four-lane groups share a row)
    int cta_begin, cta_count;
};

struct PeerInfo {           // where partial sums go (EPI_PARTIAL) and the row-split arg-max pair exchange
    uint2* inbox[MAX_PEERS];        // inbox[p]: rank p's receive buffer [world][slot_elems] of {payload, sequence}
    int rank, world;                //           slots; inbox[rank] is this GPU's own buffer
    int slot_elems;
    uint32_t seq_add;               // sequence number of this call = generation * LL_SEQ_MUL + seq_add (never 0)
};

struct GemvParams {
    GemvJob job[GEMV_MAX_JOBS];
    int njobs;
    const float* x;         // input vector [K] fp32 (plain mode: the kernel waits for its predecessor), or
    const uint2* x_ll;      // input vector [K] as {value, sequence} slots with sequence gen * LL_SEQ_MUL + x_seq_add
    uint32_t x_seq_add;
    // partial sums to fold into the input: x' = x + sum_p part_ll[p][0..K) (rank order), nparts slots of part_stride
    const uint2* part_ll;
    int nparts, part_stride;
    uint32_t part_seq_add;
    uint2* x_out_ll;        // CTA 0 publishes x' here (sequence gen * LL_SEQ_MUL + x_out_seq_add) for the next consumer
    uint32_t x_out_seq_add;
    uint32_t out_seq_add;   // sequence of this kernel's own outputs (out_ll, EPI_PARTIAL, arg-max pair, records)
    // Quantised-input records, one 64-byte record per 32 input values (see reduce_block).  When set, a few warps of
    // the lowest CTAs form the input once (gather, residual update, int8 quantisation) and every CTA copies the
    // records, instead of every CTA gathering and quantising the whole vector on its own.
    uint4* rec;
    unsigned long long wait_ns;   // budget of every poll loop
    int hard_wait;                // also wait for the predecessor to finish (PTB_DATAFLOW=0: for comparisons)
    // weights of the kernel that runs next: pulled towards L2 while this kernel works (its own came the same way)
    const uint8_t* pf_ptr[4];
    unsigned pf_bytes[4];
    const float* norm_w;    // RMSNorm weight [K] or null (no normalisation)
    float eps;
    int norm_add_one;
    int K;
    int epilogue;
    int act_gelu;
    const float* resid;     // EPI_RESID: added to the result (plain mode)
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
    // EPI_PARTIAL / arg-max pair
    PeerInfo peers;
    const uint32_t* gen;    // device generation counter (monotonic, bumped by the token's last kernel)
    int* status;
    int warps;              // warps per CTA (8 or 16): selects the kernel instantiation
    int stages, tile_bytes; // per-warp ring: `stages` slots of `tile_bytes`
    int acc_floats;         // shared-memory accumulators for K-split jobs (0 if every job has KS == 1)
    unsigned long long* trace;  // optional [8] %globaltimer stamps of CTA 0's phases (profiling aid)
    // post-norm architectures (gemma3): the previous projection's raw output t (plain `post_src`, or the sum of the
    // partial slots) is normalised first: x' = x + RMSNorm(t; post_w); CTA 0 writes x' to `x_out` / `x_out_ll`
    const float* post_src;
    const float* post_w;
    float* x_out;
};

// control block indices
enum { CTRL_TOKEN = 0, CTRL_POS = 1, CTRL_STEP = 2, CTRL_SELF_FEED = 3, CTRL_LOG_CAP = 4, CTRL_GEN = 5, CTRL_SCRIPT_LEN = 6, CTRL_WORDS = 8 };

__device__ __forceinline__ int dp4a_s(int a, int b, int c) { return __dp4a(a, b, c); }
// unsigned bytes x signed bytes: used with (q & 0xF0F0F0F0), i.e. 16 x the high nibbles, the factor is divided out afterwards
__device__ __forceinline__ int dp4a_us(unsigned a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// ---- dot products: FOUR lanes cooperate on one 256-value super-block (64 weights per lane), so the
// scale decoding and the int->float work are amortised over 16 dp4a.  `swap` flips the order of a
// lane's two 16-byte loads so that the two groups sharing a shared-memory wavefront hit different banks.

__device__ __forceinline__ float q4k_dot(const uint8_t* bp, int j, bool swap, const int8_t* xq, const float* xs,
                                         const float* xsf32) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(bp);
    const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
    const uint8_t* qp = bp + 16 + j * 32;
    const uint4 qa = *reinterpret_cast<const uint4*>(qp + (swap ? 16 : 0));
    const uint4 qb = *reinterpret_cast<const uint4*>(qp + (swap ? 0 : 16));
    const int8_t* xp = xq + j * 64 + (swap ? 16 : 0);
    const int8_t* xr = xq + j * 64 + (swap ? 0 : 16);
    const uint4 xla = *reinterpret_cast<const uint4*>(xp), xha = *reinterpret_cast<const uint4*>(xp + 32);
    const uint4 xlb = *reinterpret_cast<const uint4*>(xr), xhb = *reinterpret_cast<const uint4*>(xr + 32);
    int l0 = dp4a_s(qa.x & 0x0F0F0F0F, xla.x, 0), l1 = dp4a_s(qb.x & 0x0F0F0F0F, xlb.x, 0);
    int h0 = dp4a_us(qa.x & 0xF0F0F0F0u, xha.x, 0), h1 = dp4a_us(qb.x & 0xF0F0F0F0u, xhb.x, 0);
    l0 = dp4a_s(qa.y & 0x0F0F0F0F, xla.y, l0); l1 = dp4a_s(qb.y & 0x0F0F0F0F, xlb.y, l1);
    h0 = dp4a_us(qa.y & 0xF0F0F0F0u, xha.y, h0); h1 = dp4a_us(qb.y & 0xF0F0F0F0u, xhb.y, h1);
    l0 = dp4a_s(qa.z & 0x0F0F0F0F, xla.z, l0); l1 = dp4a_s(qb.z & 0x0F0F0F0F, xlb.z, l1);
    h0 = dp4a_us(qa.z & 0xF0F0F0F0u, xha.z, h0); h1 = dp4a_us(qb.z & 0xF0F0F0F0u, xhb.z, h1);
    l0 = dp4a_s(qa.w & 0x0F0F0F0F, xla.w, l0); l1 = dp4a_s(qb.w & 0x0F0F0F0F, xlb.w, l1);
    h0 = dp4a_us(qa.w & 0xF0F0F0F0u, xha.w, h0); h1 = dp4a_us(qb.w & 0xF0F0F0F0u, xhb.w, h1);
    h0 = (h0 + h1) >> 4;            // exact: every term is a multiple of 16
    h1 = 0;
    // 6-bit scales/mins of sub-blocks 2j and 2j+1, two per 16-bit lane of the packed header
    const int sh = 16 * (j & 1);
    const uint32_t a = (hdr.y >> sh) & 0xffffu, b = (hdr.z >> sh) & 0xffffu, c = (hdr.w >> sh) & 0xffffu;
    uint32_t sc2, mn2;
    if (j < 2) { sc2 = a & 0x3f3fu; mn2 = b & 0x3f3fu; }
    else { sc2 = (c & 0x0f0fu) | ((a & 0xc0c0u) >> 2); mn2 = ((c >> 4) & 0x0f0fu) | ((b & 0xc0c0u) >> 2); }
    const float2 xs2 = *reinterpret_cast<const float2*>(xs + 2 * j);
    const float2 sm2 = *reinterpret_cast<const float2*>(xsf32 + 2 * j);
    const float va = (float)(int)((sc2 & 0xffu) * (uint32_t)(l0 + l1)) * xs2.x + (float)(int)((sc2 >> 8) * (uint32_t)(h0 + h1)) * xs2.y;
    const float vb = (float)(mn2 & 0xffu) * sm2.x + (float)(mn2 >> 8) * sm2.y;
    return dm.x * va - dm.y * vb;
}

// Q6_K structure-of-arrays segment of `nblk` blocks; lane j4 of the group: half n = j4>>1, 32-byte slab which = j4&1.
__device__ __forceinline__ float q6k_dot(const uint8_t* seg, int nblk, int blk, int j4, bool swap, const int8_t* xq,
                                         const float* xs, const float* xsf16) {
    const int n = j4 >> 1, which = j4 & 1;
    const int o0 = swap ? 16 : 0, o1 = swap ? 0 : 16;
    const uint8_t* ql = seg + blk * 128 + n * 64 + which * 32;
    const uint8_t* qh = seg + nblk * 128 + blk * 64 + n * 32;
    const int8_t* sc = reinterpret_cast<const int8_t*>(seg + nblk * 192 + blk * 16);
    const float d = __half2float(*reinterpret_cast<const __half*>(seg + nblk * 208 + blk * 2));
    const uint4 la = *reinterpret_cast<const uint4*>(ql + o0), lb = *reinterpret_cast<const uint4*>(ql + o1);
    const uint4 ha = *reinterpret_cast<const uint4*>(qh + o0), hb = *reinterpret_cast<const uint4*>(qh + o1);
    const int e_lo = n * 128 + which * 32, e_hi = e_lo + 64;
    const uint4 xla = *reinterpret_cast<const uint4*>(xq + e_lo + o0), xlb = *reinterpret_cast<const uint4*>(xq + e_lo + o1);
    const uint4 xha = *reinterpret_cast<const uint4*>(xq + e_hi + o0), xhb = *reinterpret_cast<const uint4*>(xq + e_hi + o1);
    // bring the two high bits of each value to bit positions 4-5
    const int shl = which ? 2 : 4;       // low nibbles use qh bits 0-1 (which=0) or 2-3 (which=1)
    const int shr = which ? 2 : 0;       // high nibbles use qh bits 4-5 (which=0) or 6-7 (which=1)
#define PTB_Q6_LO(L, H) (((L) & 0x0F0F0F0Fu) | (((H) << shl) & 0x30303030u))
#define PTB_Q6_HI(L, H) ((((L) >> 4) & 0x0F0F0F0Fu) | (((H) >> shr) & 0x30303030u))
    int dla = dp4a_s(PTB_Q6_LO(la.x, ha.x), xla.x, 0), dlb = dp4a_s(PTB_Q6_LO(lb.x, hb.x), xlb.x, 0);
    int dha = dp4a_s(PTB_Q6_HI(la.x, ha.x), xha.x, 0), dhb = dp4a_s(PTB_Q6_HI(lb.x, hb.x), xhb.x, 0);
    dla = dp4a_s(PTB_Q6_LO(la.y, ha.y), xla.y, dla); dlb = dp4a_s(PTB_Q6_LO(lb.y, hb.y), xlb.y, dlb);
    dha = dp4a_s(PTB_Q6_HI(la.y, ha.y), xha.y, dha); dhb = dp4a_s(PTB_Q6_HI(lb.y, hb.y), xhb.y, dhb);
    dla = dp4a_s(PTB_Q6_LO(la.z, ha.z), xla.z, dla); dlb = dp4a_s(PTB_Q6_LO(lb.z, hb.z), xlb.z, dlb);
    dha = dp4a_s(PTB_Q6_HI(la.z, ha.z), xha.z, dha); dhb = dp4a_s(PTB_Q6_HI(lb.z, hb.z), xhb.z, dhb);
    dla = dp4a_s(PTB_Q6_LO(la.w, ha.w), xla.w, dla); dlb = dp4a_s(PTB_Q6_LO(lb.w, hb.w), xlb.w, dlb);
    dha = dp4a_s(PTB_Q6_HI(la.w, ha.w), xha.w, dha); dhb = dp4a_s(PTB_Q6_HI(lb.w, hb.w), xhb.w, dhb);
#undef PTB_Q6_LO
#undef PTB_Q6_HI
    // 16-value scale groups: (e + o)/16
    const int ia = (e_lo + o0) >> 4, ib = (e_lo + o1) >> 4;
    const float xsl = xs[e_lo >> 5], xsh = xs[e_hi >> 5];
    float r = (float)sc[ia] * (xsl * (float)dla - 32.0f * xsf16[ia]);
    r += (float)sc[ib] * (xsl * (float)dlb - 32.0f * xsf16[ib]);
    r += (float)sc[ia + 4] * (xsh * (float)dha - 32.0f * xsf16[ia + 4]);
    r += (float)sc[ib + 4] * (xsh * (float)dhb - 32.0f * xsf16[ib + 4]);
    return d * r;
}

// All the dot products one 4-lane group owes to a tile: blocks my_j, my_j + gprw, ... of its row, two blocks per
// trip (and both matrices of a gated pair) so that independent dependency chains overlap in the pipeline.
template <int QT, bool PAIRED>
__device__ __forceinline__ void tile_dots(const uint8_t* rowp, size_t pair_off, int nb, int my_j, int gprw, int lane4, bool swap,
                                          const int8_t* xq_s, const float* xs_s, const float* xsf_s, const float* xsf32_s,
                                          float& a0, float& a1) {
    auto dot = [&](const uint8_t* rp, int b) -> float {
        if (QT == QT_Q4K) return q4k_dot(rp + b * 144, lane4, swap, xq_s + b * 256, xs_s + b * 8, xsf32_s + b * 8);
        return q6k_dot(rp, nb, b, lane4, swap, xq_s + b * 256, xs_s + b * 8, xsf_s + b * 16);
    };
    int b = my_j;
#pragma unroll 1
    for (; b + gprw < nb; b += 2 * gprw) {
        const float p0 = dot(rowp, b), p1 = dot(rowp, b + gprw);
        if (PAIRED) {
            const float q0 = dot(rowp + pair_off, b), q1 = dot(rowp + pair_off, b + gprw);
            a1 += q0 + q1;
        }
        a0 += p0 + p1;
    }
    if (b < nb) {
        const float p0 = dot(rowp, b);
        if (PAIRED) a1 += dot(rowp + pair_off, b);
        a0 += p0;
    }
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

// Where a kernel's input vector comes from.  Plain mode: `x` (and `post_src`) are fp32 arrays that the predecessor
// finished writing before this kernel passed its dependency wait.  Dataflow mode: `x_ll` and the `nparts` partial-sum
// slots of `part_ll` are {value, sequence} buffers that the producers may still be filling; the loads below poll them.
struct InputSrc {
    const float* x;
    const uint2* x_ll;
    uint32_t x_seq;
    const uint2* part_ll;
    int nparts, part_stride;
    uint32_t part_seq;
    const float* post_src;
    const float* post_w;
    float* x_out;
    uint2* x_out_ll;
    uint32_t x_out_seq;
    int* status;
    unsigned long long wait_ns;
};

// Load x[K] once into registers (adding the partial sums of the previous projection and, for post-norm
// architectures, normalising them first), optionally RMS-normalise, quantise to int8 blocks of 32.
//   xq[K] int8, xs[K/32] block scales, xsf16[K/16] = scale * (sum of 16 int8), xsf32[K/32] = scale * (sum of 32).
// Each thread keeps up to QIN_ITEMS 8-value items in registers: K <= QIN_ITEMS * 8 * blockDim.
template <int QIN_ITEMS, bool POST = false, bool LL = true>
__device__ __forceinline__ void quantize_input(const InputSrc& I, const float* __restrict__ norm_w, float eps,
                                               int add_one, int K, int8_t* xq, float* xs, float* xsf16, float* xsf32,
                                               float* red) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int items = K / 8;
    float v[QIN_ITEMS][8];
    float t[POST ? QIN_ITEMS : 1][8];
    float ss = 0.f;
    if (LL && (I.x_ll || I.part_ll)) {
        // ---- dataflow mode.  A status word that is already set means an earlier kernel gave up: do not wait again.
        const unsigned long long budget = (*reinterpret_cast<volatile int*>(I.status) != 0) ? 0ull : I.wait_ns;
        unsigned done = 0;
        uint64_t t0 = 0;
        for (int round = 0;; ++round) {
            bool all = true;
#pragma unroll
            for (int r = 0; r < QIN_ITEMS; ++r) {
                const int i = r * nt + tid;
                if (i < items && !((done >> r) & 1u)) {
                    float a[8], ps[8];
                    bool ok = true;
                    if (I.x_ll) ok = ll_try8(I.x_ll + 8 * (size_t)i, I.x_seq, a);
                    else {
                        const float4 lo = __ldcg(reinterpret_cast<const float4*>(I.x) + 2 * i), hi = __ldcg(reinterpret_cast<const float4*>(I.x) + 2 * i + 1);
                        a[0] = lo.x; a[1] = lo.y; a[2] = lo.z; a[3] = lo.w; a[4] = hi.x; a[5] = hi.y; a[6] = hi.z; a[7] = hi.w;
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k) ps[k] = 0.f;
                    for (int p = 0; p < I.nparts; ++p) {        // rank order: every GPU forms bitwise the same sum
                        float b[8];
                        ok = ll_try8(I.part_ll + (size_t)p * I.part_stride + 8 * (size_t)i, I.part_seq, b) && ok;
#pragma unroll
                        for (int k = 0; k < 8; ++k) ps[k] += b[k];
                    }
                    if (ok) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            v[r][k] = POST ? a[k] : a[k] + ps[k];
                            if (POST) t[r][k] = ps[k];
                        }
                        done |= 1u << r;
                    } else all = false;
                }
            }
            if (!__syncthreads_or(!all)) break;
            // Not there yet.  Back off to a cheap probe by one warp (32 slots spread over the vector) so that the CTAs
            // do not hammer L2 with full-vector reads while the producers are at work; thread 0 keeps the clock.
            bool expired = false;
            if (tid < 32) {
                const int si = tid * (K / 32);
                if (round == 0 && tid == 0) t0 = global_ns();
                t0 = __shfl_sync(0xffffffffu, t0, 0);
                for (;;) {
                    bool ok = true;
                    if (I.x_ll) ok = ld_ll(I.x_ll + si).y == I.x_seq;
                    for (int p = 0; p < I.nparts; ++p) ok = ok && ld_ll(I.part_ll + (size_t)p * I.part_stride + si).y == I.part_seq;
                    if (__all_sync(0xffffffffu, ok)) break;
                    expired = global_ns() - t0 > budget;
                    if (__any_sync(0xffffffffu, expired)) { expired = true; break; }
                    __nanosleep(40);
                }
                // the probe can pass while other slots are still missing: the clock also bounds the outer rounds
                if (!expired && round > 0) expired = __any_sync(0xffffffffu, global_ns() - t0 > budget);
            }
            if (__syncthreads_or(expired)) {
                if (tid == 0) atomicExch(I.status, PTB_ERR_FLAG_TIMEOUT);
                break;
            }
        }
#pragma unroll
        for (int r = 0; r < QIN_ITEMS; ++r)
            if (!((done >> r) & 1u)) {
#pragma unroll
                for (int k = 0; k < 8; ++k) { v[r][k] = 0.f; if (POST) t[r][k] = 0.f; }
            }
    } else {
#pragma unroll
        for (int r = 0; r < QIN_ITEMS; ++r) {
            const int i = r * nt + tid;
            if (i < items) {
                const float4 a = __ldcg(reinterpret_cast<const float4*>(I.x) + 2 * i), b = __ldcg(reinterpret_cast<const float4*>(I.x) + 2 * i + 1);
                v[r][0] = a.x; v[r][1] = a.y; v[r][2] = a.z; v[r][3] = a.w; v[r][4] = b.x; v[r][5] = b.y; v[r][6] = b.z; v[r][7] = b.w;
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) v[r][k] = 0.f;
            }
            if (POST) {
                if (i < items) {
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(I.post_src) + 2 * i), b = __ldcg(reinterpret_cast<const float4*>(I.post_src) + 2 * i + 1);
                    t[r][0] = a.x; t[r][1] = a.y; t[r][2] = a.z; t[r][3] = a.w; t[r][4] = b.x; t[r][5] = b.y; t[r][6] = b.z; t[r][7] = b.w;
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) t[r][k] = 0.f;
                }
            }
        }
    }
    if (POST) {
        // x' = x + RMSNorm(t; post_w): t is the raw output of the previous projection
        float st = 0.f;
#pragma unroll
        for (int r = 0; r < QIN_ITEMS; ++r)
#pragma unroll
            for (int k = 0; k < 8; ++k) st += t[r][k] * t[r][k];
        st = block_sum(st, red);
        const float rt = rsqrtf(st / (float)K + eps);
#pragma unroll
        for (int r = 0; r < QIN_ITEMS; ++r) {
            const int i = r * nt + tid;
            if (i < items) {
                const float4 wa = __ldg(reinterpret_cast<const float4*>(I.post_w) + 2 * i), wb = __ldg(reinterpret_cast<const float4*>(I.post_w) + 2 * i + 1);
                const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int k = 0; k < 8; ++k) v[r][k] += t[r][k] * rt * (add_one ? 1.0f + w[k] : w[k]);
            }
        }
        __syncthreads();        // `red` is reused by the next reduction
    }
    if (blockIdx.x == 0 && (I.x_out || (LL && I.x_out_ll))) {
        // the updated residual stream, published once for the consumer after next
#pragma unroll
        for (int r = 0; r < QIN_ITEMS; ++r) {
            const int i = r * nt + tid;
            if (i < items) {
                if (I.x_out) {
                    reinterpret_cast<float4*>(I.x_out)[2 * i] = make_float4(v[r][0], v[r][1], v[r][2], v[r][3]);
                    reinterpret_cast<float4*>(I.x_out)[2 * i + 1] = make_float4(v[r][4], v[r][5], v[r][6], v[r][7]);
                }
                if (LL && I.x_out_ll) {
                    uint2* o = I.x_out_ll + 8 * (size_t)i;
#pragma unroll
                    for (int k = 0; k < 8; k += 2) st_ll2(o + k, __float_as_uint(v[r][k]), __float_as_uint(v[r][k + 1]), I.x_out_seq);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < QIN_ITEMS; ++r)
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += v[r][k] * v[r][k];
    float rs = 1.0f;
    if (norm_w) {
        ss = block_sum(ss, red);
        rs = rsqrtf(ss / (float)K + eps);
    }
#pragma unroll
    for (int r = 0; r < QIN_ITEMS; ++r) {
        const int i = r * nt + tid;
        if (r * nt >= items) break;
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
    __syncthreads();
}

// ---- quantised-input records --------------------------------------------------------------------------------
// Record of block b (values 32b .. 32b+31), four 16-byte quarters, each {12 bytes payload, sequence number} written
// and read as one 16-byte access, so a quarter that shows the expected sequence number is complete:
//   quarter 0: int8 values 0-11      quarter 1: int8 values 12-23
//   quarter 2: int8 values 24-31, block scale
//   quarter 3: scale * (sum of int8 values 0-15), scale * (sum of values 16-31), sum of squares of the fp32 values
// The int8 values quantise x * norm_w (no 1/rms factor): the consumer derives 1/rms from the sums of squares and
// applies it to its dot products, so forming a block needs nothing from the other blocks.
__device__ __forceinline__ void st_rec(uint4* p, uint32_t a, uint32_t b, uint32_t c, uint32_t seq) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(seq) : "memory");
}
__device__ __forceinline__ uint4 ld_rec(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

struct GemvParams;
// One warp forms block b: polls its sources (the input slots plus the partial-sum slots of every rank, summed in rank
// order), publishes the updated residual stream, quantises and publishes the record.
__device__ __forceinline__ void reduce_block(const GemvParams& P, int b, uint32_t gen, int lane, unsigned long long budget);

// Every thread copies its share of the records into the shared-memory arrays the dot products read, polling until
// each quarter carries `seq`.  Returns the block-wide sum of the per-block sums of squares.
template <int MAXQ>
__device__ __forceinline__ float copy_records(const uint4* rec, int nblk, uint32_t seq, int8_t* xq, float* xs, float* xsf16,
                                              float* xsf32, int* status, unsigned long long budget, float* red) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int nq = 4 * nblk;
    const int rot = (int)((blockIdx.x * 97u) % (unsigned)nq);     // CTAs sweep the records in different orders
    unsigned done = 0;
    float ssq = 0.f;
    uint64_t t0 = 0;
    for (int round = 0;; ++round) {
        bool all = true;
#pragma unroll
        for (int r = 0; r < MAXQ; ++r) {
            const int it = r * nt + tid;
            if (it < nq && !((done >> r) & 1u)) {
                int qi = it + rot;
                if (qi >= nq) qi -= nq;
                const uint4 v = ld_rec(rec + qi);
                if (v.w == seq) {
                    const int blk = qi >> 2, part = qi & 3;
                    uint32_t* q32 = reinterpret_cast<uint32_t*>(xq + 32 * blk);
                    if (part == 0) { q32[0] = v.x; q32[1] = v.y; q32[2] = v.z; }
                    else if (part == 1) { q32[3] = v.x; q32[4] = v.y; q32[5] = v.z; }
                    else if (part == 2) { q32[6] = v.x; q32[7] = v.y; xs[blk] = __uint_as_float(v.z); }
                    else {
                        const float a = __uint_as_float(v.x), bsum = __uint_as_float(v.y);
                        xsf16[2 * blk] = a; xsf16[2 * blk + 1] = bsum; xsf32[blk] = a + bsum;
                        ssq += __uint_as_float(v.z);
                    }
                    done |= 1u << r;
                } else all = false;
            }
        }
        if (!__syncthreads_or(!all)) break;
        bool expired = false;          // not there yet: one warp probes a few records, thread 0 keeps the clock
        if (tid < 32) {
            if (round == 0 && tid == 0) t0 = global_ns();
            t0 = __shfl_sync(0xffffffffu, t0, 0);
            const int si = (int)(((long long)tid * nq) / 32);
            for (;;) {
                const bool ok = ld_rec(rec + si).w == seq;
                if (__all_sync(0xffffffffu, ok)) break;
                if (__any_sync(0xffffffffu, global_ns() - t0 > budget)) { expired = true; break; }
                __nanosleep(20);
            }
            if (!expired && round > 0) expired = __any_sync(0xffffffffu, global_ns() - t0 > budget);
        }
        if (__syncthreads_or(expired)) {
            if (tid == 0) atomicExch(status, PTB_ERR_FLAG_TIMEOUT);
            // fill what never came with zeros so that the kernel can finish
            for (int r = 0; r < MAXQ; ++r) {
                const int it = r * nt + tid;
                if (it < nq && !((done >> r) & 1u)) {
                    int qi = it + rot;
                    if (qi >= nq) qi -= nq;
                    const int blk = qi >> 2, part = qi & 3;
                    uint32_t* q32 = reinterpret_cast<uint32_t*>(xq + 32 * blk);
                    if (part == 0) { q32[0] = q32[1] = q32[2] = 0; }
                    else if (part == 1) { q32[3] = q32[4] = q32[5] = 0; }
                    else if (part == 2) { q32[6] = q32[7] = 0; xs[blk] = 0.f; }
                    else { xsf16[2 * blk] = xsf16[2 * blk + 1] = xsf32[blk] = 0.f; }
                }
            }
            break;
        }
    }
    return block_sum(ssq, red);
}

__host__ __device__ __forceinline__ size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Shared memory carve-up, used by the kernel and by the host-side planner.
struct GemvSmem {
    size_t bars, misc, xq, xs, xsf, xsf32, acc, tiles, total;
};
__host__ __device__ __forceinline__ GemvSmem gemv_smem_layout(int K, int warps, int stages, int tile_bytes, int acc_floats) {
    GemvSmem L;
    L.bars = 0;
    L.misc = align_up((size_t)warps * stages * 8, 128);
    L.xq = L.misc + 64 * 4;
    L.xs = L.xq + (size_t)K;
    L.xsf = L.xs + (size_t)(K / 32) * 4;
    L.xsf32 = L.xsf + (size_t)(K / 16) * 4;
    L.acc = L.xsf32 + (size_t)(K / 32) * 4;
    L.tiles = align_up(L.acc + (size_t)acc_floats * 4, 128);
    L.total = L.tiles + (size_t)warps * stages * tile_bytes;
    return L;
}

__device__ __forceinline__ void reduce_block(const GemvParams& P, int b, uint32_t gen, int lane, unsigned long long budget) {
    const int e = 32 * b + lane;
    const uint32_t xseq = gen * LL_SEQ_MUL + P.x_seq_add, pseq = gen * LL_SEQ_MUL + P.part_seq_add;
    const int nparts = P.part_ll ? P.nparts : 0;
    float v = 0.f;
    uint64_t t0 = 0;
    for (int round = 0;; ++round) {
        const uint2 a = ld_ll(P.x_ll + e);
        bool ok = a.y == xseq;
        float ps = 0.f;
        for (int p = 0; p < nparts; ++p) {              // rank order: every GPU forms bitwise the same sum
            const uint2 sl = ld_ll(P.part_ll + (size_t)p * P.part_stride + e);
            ok = ok && sl.y == pseq;
            ps += __uint_as_float(sl.x);
        }
        if (__all_sync(0xffffffffu, ok)) { v = __uint_as_float(a.x) + ps; break; }
        if (round == 0) t0 = global_ns();
        if (__any_sync(0xffffffffu, global_ns() - t0 > budget)) {
            if (lane == 0) atomicExch(P.status, PTB_ERR_FLAG_TIMEOUT);
            break;
        }
        __nanosleep(20);
    }
    if (nparts > 0 && P.x_out_ll) st_ll(P.x_out_ll + e, __float_as_uint(v), gen * LL_SEQ_MUL + P.x_out_seq_add);
    if (P.x_out) P.x_out[e] = v;
    const float ssq = warp_sum(v * v);
    float y = v;
    if (P.norm_w) {
        const float w = __ldg(P.norm_w + e);
        y = v * (P.norm_add_one ? 1.0f + w : w);
    }
    const float am = warp_max(fabsf(y));
    const float sc = am / 127.0f, inv = am > 0.f ? 127.0f / am : 0.f;
    const int q = __float2int_rn(y * inv);
    int s16 = q;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) s16 += __shfl_xor_sync(0xffffffffu, s16, o);      // lanes 0-15 / 16-31: the two halves
    const float sf = sc * (float)s16;
    const float sfa = __shfl_sync(0xffffffffu, sf, 0), sfb = __shfl_sync(0xffffffffu, sf, 16);
    // four consecutive values per word: lane j < 8 assembles word j
    const uint32_t byte = (uint32_t)q & 0xffu;
    const int j4 = 4 * (lane & 7);
    const uint32_t pk = __shfl_sync(0xffffffffu, byte, j4) | (__shfl_sync(0xffffffffu, byte, j4 + 1) << 8) |
                        (__shfl_sync(0xffffffffu, byte, j4 + 2) << 16) | (__shfl_sync(0xffffffffu, byte, j4 + 3) << 24);
    uint32_t w0 = __shfl_sync(0xffffffffu, pk, min(3 * lane, 7));
    uint32_t w1 = __shfl_sync(0xffffffffu, pk, min(3 * lane + 1, 7));
    uint32_t w2 = __shfl_sync(0xffffffffu, pk, min(3 * lane + 2, 7));
    if (lane == 2) w2 = __float_as_uint(sc);
    if (lane == 3) { w0 = __float_as_uint(sfa); w1 = __float_as_uint(sfb); w2 = __float_as_uint(ssq); }
    if (lane < 4) st_rec(P.rec + 4 * (size_t)b + lane, w0, w1, w2, gen * LL_SEQ_MUL + P.out_seq_add);
}

// The input side of a GEMV kernel: fills the shared-memory arrays the dot products read (int8 values, block scales,
// scaled block sums) from whichever source the launch names, and returns the factor the dot products still have to be
// multiplied with (1/rms of the input when the records carry the un-normalised vector, else 1).
template <int GEMV_WARPS, int MODE = 0>
__device__ __forceinline__ float gemv_input(const GemvParams& P, uint32_t gen, uint32_t seq, int K, int8_t* xq, float* xs, float* xsf,
                                            float* xsf32, float* misc, int warp, int lane) {
    constexpr int GEMV_THREADS = GEMV_WARPS * 32;
    constexpr bool LEAN = MODE == 1;
    float in_scale = 1.0f;            // 1/rms of the input when the records carry the un-normalised vector
    if (MODE == 2 || (!LEAN && P.rec && !P.post_w)) {
        const unsigned long long budget = (*reinterpret_cast<volatile int*>(P.status) != 0) ? 0ull : P.wait_ns;
        const int nblk32 = K / 32;
        // the lowest CTAs start first: two of their warps each form blocks
        if (warp < 2)
            for (int b = blockIdx.x * 2 + warp; b < nblk32; b += gridDim.x * 2) reduce_block(P, b, gen, lane, budget);
        const float ssq = copy_records<(GEMV_WARPS >= 16 ? 3 : 5)>(P.rec, nblk32, seq, xq, xs, xsf, xsf32, P.status, budget, misc);
        if (P.norm_w) in_scale = rsqrtf(ssq / (float)K + P.eps);
        __syncthreads();
    } else if (MODE != 2) {
        InputSrc I;
        I.x = P.x; I.x_ll = P.x_ll; I.x_seq = gen * LL_SEQ_MUL + P.x_seq_add;
        I.part_ll = P.part_ll; I.nparts = P.part_ll ? P.nparts : 0; I.part_stride = P.part_stride;
        I.part_seq = gen * LL_SEQ_MUL + P.part_seq_add;
        I.post_src = P.post_src; I.post_w = P.post_w; I.x_out = P.x_out; I.x_out_ll = P.x_out_ll;
        I.x_out_seq = gen * LL_SEQ_MUL + P.x_out_seq_add;
        I.status = P.status; I.wait_ns = P.wait_ns;
        if (P.post_w) quantize_input<(GEMV_WARPS >= 16 ? 1 : 2), true, !LEAN>(I, P.norm_w, P.eps, P.norm_add_one, K, xq, xs, xsf, xsf32, misc);
        else if (K <= 2 * 8 * GEMV_THREADS) quantize_input<2, false, !LEAN>(I, P.norm_w, P.eps, P.norm_add_one, K, xq, xs, xsf, xsf32, misc);
        else quantize_input<(GEMV_WARPS >= 16 ? 3 : 5), false, !LEAN>(I, P.norm_w, P.eps, P.norm_add_one, K, xq, xs, xsf, xsf32, misc);
    }
    return in_scale;
}

// Arg-max over the whole output: CTA-level reduction, then the last CTA to arrive reduces across CTAs (and, under
// tensor parallelism, exchanges {value, id} pairs with the other ranks), records the id and advances the decode
// control block for the next token.
// End of a token: log the chosen id, bump the step and generation counters and, in the self-feeding modes, make the
// id (or the next scripted prompt token) the input of the next token.  One thread.
__device__ __forceinline__ void advance_token(int* ctrl, int* token_log, const int* token_script, int id, uint32_t gen) {
    const int step = ctrl[CTRL_STEP];
    if (token_log && step < ctrl[CTRL_LOG_CAP]) token_log[step] = id;
    ctrl[CTRL_STEP] = step + 1;
    ctrl[CTRL_GEN] = (int)(gen + 1u);      // the token is over: every slot of the next one carries a new sequence
    const int mode = ctrl[CTRL_SELF_FEED];
    if (mode) {
        const bool scripted = mode == 2 && token_script && step + 1 < ctrl[CTRL_SCRIPT_LEN];
        ctrl[CTRL_TOKEN] = scripted ? token_script[step + 1] : id;
        ctrl[CTRL_POS] += 1;
    }
}

template <int GEMV_WARPS>
__device__ __forceinline__ void gemv_argmax_tail(const GemvParams& P, float best_v, int best_i, float* misc, uint32_t gen, uint32_t seq) {
    constexpr int GEMV_THREADS = GEMV_WARPS * 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (P.epilogue == EPI_ARGMAX) {
        // CTA arg-max (ties -> lowest index), then the last CTA to arrive finishes across CTAs.
        __syncthreads();
        float* sv = misc;
        int* si = reinterpret_cast<int*>(misc + 32);
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
        }
        if (lane == 0) { sv[warp] = best_v; si[warp] = best_i; }
        __syncthreads();
        __shared__ bool is_last;
        if (tid == 0) {
            for (int w = 1; w < GEMV_WARPS; ++w)
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
            if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
            __syncthreads();
            if (tid == 0) {
                for (int w = 1; w < GEMV_WARPS; ++w)
                    if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
                *P.ticket = 0u;
                bi += P.row_offset;
                const PeerInfo& pi = P.peers;
                if (pi.world > 1) {
                    // every rank holds a slice of the vocabulary: exchange {value, id} and let each rank
                    // pick the same winner
                    for (int p = 0; p < pi.world; ++p) {
                        uint2* slot = pi.inbox[p] + (size_t)pi.rank * pi.slot_elems;
                        st_ll(slot, __float_as_uint(bv), seq);
                        st_ll(slot + 1, (uint32_t)bi, seq);
                    }
                    bv = -INFINITY;
                    bi = 0x7fffffff;
                    for (int p = 0; p < pi.world; ++p) {
                        const uint2* slot = pi.inbox[pi.rank] + (size_t)p * pi.slot_elems;
                        const float v = __uint_as_float(wait_ll(slot, seq, P.status, P.wait_ns));
                        const int ix = (int)wait_ll(slot + 1, seq, P.status, P.wait_ns);
                        if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
                    }
                }
                P.result[0] = bi;
                reinterpret_cast<float*>(P.result)[1] = bv;
                if (P.ctrl) advance_token(P.ctrl, P.token_log, P.token_script, bi, gen);
            }
        }
    }

}

// MODE 0: everything.  MODE 1 ("lean"): the plain flow only (fp32 vectors in and out, launch-boundary wait); the slot
// hand-over, the input records and the L2 prefetch of the next weights are compiled out, which frees the block loop of
// their registers (no spills).  MODE 2: the dataflow with input records only (no plain or slot-polled input path).
template <int GEMV_WARPS, int MODE = 0>
__global__ void __launch_bounds__(GEMV_WARPS * 32, GEMV_WARPS >= 16 ? 1 : 2) gemv_kernel(const __grid_constant__ GemvParams P) {
    constexpr int GEMV_THREADS = GEMV_WARPS * 32;
    constexpr bool LEAN = MODE == 1;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = P.K, S = P.stages;
    const GemvSmem L = gemv_smem_layout(K, GEMV_WARPS, S, P.tile_bytes, P.acc_floats);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars) + warp * S;    // this warp's ring
    float* misc = reinterpret_cast<float*>(smem + L.misc);
    int8_t* xq = reinterpret_cast<int8_t*>(smem + L.xq);
    float* xs = reinterpret_cast<float*>(smem + L.xs);
    float* xsf = reinterpret_cast<float*>(smem + L.xsf);
    float* xsf32 = reinterpret_cast<float*>(smem + L.xsf32);
    float* acc = reinterpret_cast<float*>(smem + L.acc);
    uint8_t* ring = smem + L.tiles + (size_t)warp * S * P.tile_bytes;

    auto stamp = [&](int k) {
        if (P.trace && tid == 0 && blockIdx.x == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            P.trace[k] = t;
        }
    };
    stamp(0);
    // ---- which job and which rows are mine
    int ji = 0;
#pragma unroll
    for (int i = 1; i < GEMV_MAX_JOBS; ++i)
        if (i < P.njobs && (int)blockIdx.x >= P.job[i].cta_begin) ji = i;
    const GemvJob& J = P.job[ji];
    const int ci = blockIdx.x - J.cta_begin;
    const int r0 = (int)(((long long)J.N * ci) / J.cta_count);
    const int r1 = (int)(((long long)J.N * (ci + 1)) / J.cta_count);
    const int RW = J.RW, KS = J.KS, qtype = J.qtype;
    const int nrg = (r1 - r0 + RW - 1) / RW;
    const int nitems = nrg * KS;
    const bool paired = J.w2 != nullptr;
    const int sz0 = seg_bytes(qtype, J.seg_base), sz1 = seg_bytes(qtype, J.seg_base + 1);

    // item -> geometry
    struct Item { int s, nb, boff, sb, row0, rows; size_t off; };
    auto geom = [&](int it) {
        Item g;
        const int rg = it / KS;
        g.s = it - rg * KS;
        const int extra = min(g.s, J.seg_rem);
        g.nb = J.seg_base + (g.s < J.seg_rem ? 1 : 0);
        g.boff = g.s * J.seg_base + extra;
        g.sb = g.s < J.seg_rem ? sz1 : sz0;
        g.row0 = r0 + rg * RW;
        g.rows = min(RW, r1 - g.row0);
        g.off = (size_t)J.N * ((size_t)g.s * sz0 + (size_t)extra * (sz1 - sz0)) + (size_t)g.row0 * g.sb;
        return g;
    };
    auto issue = [&](int it, int slot) {   // lane 0 of the warp
        const Item g = geom(it);
        const uint32_t bytes = (uint32_t)g.rows * g.sb;
        uint8_t* dst = ring + (size_t)slot * P.tile_bytes;
        mbar_expect_tx(&full[slot], paired ? 2 * bytes : bytes);
        bulk_g2s(dst, J.w + g.off, bytes, &full[slot]);
        if (paired) bulk_g2s(dst + RW * g.sb, J.w2 + g.off, bytes, &full[slot]);
    };

    if (lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
        fence_proxy_async();
        // the weights do not depend on the previous kernel: start streaming them now
        for (int k = 0; k < S; ++k) {
            const int it = warp + k * GEMV_WARPS;
            if (it < nitems) issue(it, k);
        }
    }
    if (P.norm_w) {
        for (int i = tid * 32; i < K; i += GEMV_THREADS * 32)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(P.norm_w + i));
    }
    if (MODE == 0 && lane == 1) {
        // this CTA's share of the next kernel's weights, 16 KB bulk prefetches spread over the warps
        constexpr unsigned CH = 16384;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const unsigned nch = (P.pf_bytes[r] + CH - 1) / CH;
            for (unsigned c = blockIdx.x * GEMV_WARPS + warp; c < nch; c += gridDim.x * GEMV_WARPS) {
                const unsigned off = c * CH, len = min(CH, P.pf_bytes[r] - off);
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(P.pf_ptr[r] + off), "r"(len) : "memory");
            }
        }
    }
    pdl_launch_dependents();
    const bool dataflow = MODE == 2 || (!LEAN && P.x_ll != nullptr);
    // plain mode: the input is complete once the predecessor has finished.  Dataflow mode: never wait for the
    // launch boundary, the input slots validate themselves.
    if (!dataflow || P.hard_wait) pdl_wait();
    __syncthreads();
    stamp(1);
    const uint32_t gen = P.gen ? *reinterpret_cast<const volatile uint32_t*>(P.gen) : 0u;
    const uint32_t seq = gen * LL_SEQ_MUL + P.out_seq_add;

    const float in_scale = gemv_input<GEMV_WARPS, MODE>(P, gen, seq, K, xq, xs, xsf, xsf32, misc, warp, lane);
    stamp(2);

    // eight 4-lane groups per warp; neighbouring groups take neighbouring rows (same x addresses -> broadcast)
    const int grp = lane >> 2, lane4 = lane & 3;
    const int gprw = 8 / RW;
    const int my_row = grp % RW, my_j = grp / RW;
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    bool ok = true;

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
                // {partial sum, sequence number} for element n into slot [rank][n] of every rank's inbox; whoever
                // consumes the vector adds the slots up in rank order
                const PeerInfo& pi = P.peers;
                for (int p = 0; p < pi.world; ++p) st_ll(pi.inbox[p] + (size_t)pi.rank * pi.slot_elems + n, __float_as_uint(v0), seq);
                return;
            }
        }
        if (!LEAN && J.out_ll) st_ll(J.out_ll + n, __float_as_uint(r), seq);
        else J.out[n] = r;
    };

    int k = 0;
    for (int it = warp; it < nitems; it += GEMV_WARPS, ++k) {
        const int slot = k % S;
        const Item g = geom(it);
        if (ok) ok = mbar_wait(&full[slot], (uint32_t)((k / S) & 1), P.status);
        if (k == 0) stamp(3);
        const uint8_t* tile = ring + (size_t)slot * P.tile_bytes;
        float a0 = 0.f, a1 = 0.f;
        if (ok && my_row < g.rows) {
            const uint8_t* rowp = tile + (size_t)my_row * g.sb;
            const int8_t* xq_s = xq + g.boff * 256;
            const float* xs_s = xs + g.boff * 8;
            const float* xsf_s = xsf + g.boff * 16;
            const float* xsf32_s = xsf32 + g.boff * 8;
            // odd groups flip their two 16-byte loads when the row stride is an even multiple of 16 B
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
        if (lane == 0 && it + S * GEMV_WARPS < nitems) issue(it + S * GEMV_WARPS, slot);
        // lanes of a group (xor 1, 2), then the groups sharing a row: they sit RW groups = 4*RW lanes apart
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
    stamp(4);
    if (KS > 1) {
        __syncthreads();
        for (int r = tid; r < r1 - r0; r += GEMV_THREADS) {
            float v0 = 0.f, v1 = 0.f;
            for (int s = 0; s < KS; ++s) {
                v0 += acc[(size_t)r * KS + s];
                if (paired) v1 += acc[(size_t)(r1 - r0) * KS + (size_t)r * KS + s];
            }
            epilogue(r0 + r, v0, v1);
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

// ---------------------------------------------------------------------------------------------
// Attention for one new token.
// grid (kv_heads, max_splits), 256 threads.  Split s covers cache positions [s*128, s*128+128).
// q/k/v for the new token arrive as fp32 rows of `qkv` (q: heads*d, then k: kv_heads*d, then v);
// the CTA owning the split that contains `pos` normalises/rotates K and writes K,V to the fp16 cache.
constexpr int ATT_THREADS = 256;
constexpr int ATT_CHUNK = 128;
constexpr int ATT_MAX_GROUP = 8;

struct AttnParams {
    const float* q;          // [heads*d]      plain inputs (the kernel waits for its predecessor), or
    const float* k;          // [kv_heads*d]
    const float* v;          // [kv_heads*d]
    const uint2* q_ll;       // the same three vectors as {value, sequence} slots (engine dataflow)
    const uint2* k_ll;
    const uint2* v_ll;
    uint2* out_ll;           // [heads*d] output slots
    uint32_t in_seq_add, out_seq_add;
    const uint32_t* gen;
    int* status;
    unsigned long long wait_ns;
    int hard_wait;
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
    int head_dim;            // 64, 128 or 256
    int max_seq;
    int max_splits;
    int neox;
    float eps;
    float scale;
    int window;              // sliding window (0 = full)
    unsigned long long* trace;   // optional [8] %globaltimer stamps (profiling aid)
};

// A vector that is either a plain fp32 array or a buffer of {value, sequence} slots polled until it is filled.
struct VecSrc {
    const float* p;
    const uint2* ll;
    uint32_t seq;
    int* status;
    unsigned long long budget;
    __device__ __forceinline__ float get(int i) const {
        return ll ? __uint_as_float(wait_ll(ll + i, seq, status, budget)) : p[i];
    }
    // N elements at once: the loads are issued together, a slot that is not filled yet is then waited for alone
    template <int N>
    __device__ __forceinline__ void getn(const int* idx, float* v) const {
        if (!ll) {
#pragma unroll
            for (int k = 0; k < N; ++k) v[k] = p[idx[k]];
            return;
        }
        uint2 r[N];
#pragma unroll
        for (int k = 0; k < N; ++k) r[k] = ld_ll(ll + idx[k]);
#pragma unroll
        for (int k = 0; k < N; ++k) v[k] = r[k].y == seq ? __uint_as_float(r[k].x) : get(idx[k]);
    }
};

// One warp normalises (optional RMS norm over the head), rotates and scales one head of D values into dst[D].
// NeoX pairing is (i, i + D/2) and a lane owns i = lane + 32 k; the interleaved pairing is (2i, 2i+1) and a lane
// owns D/32 consecutive values.
template <int D>
__device__ __forceinline__ void norm_rope_head(const VecSrc& src, const float* nw, float eps, const float* cs, const float* sn,
                                               int neox, float mul, float* dst /*smem [D]*/, int lane) {
    constexpr int VPL = D / 32;
    float v[VPL];
    int idx[VPL];
#pragma unroll
    for (int k = 0; k < VPL; ++k) idx[k] = neox ? lane + 32 * k : VPL * lane + k;
    src.getn<VPL>(idx, v);
    if (nw) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < VPL; ++k) ss += v[k] * v[k];
        ss = warp_sum(ss);
        const float rs = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int k = 0; k < VPL; ++k) v[k] *= rs * nw[idx[k]];
    }
    if (neox) {
#pragma unroll
        for (int k = 0; k < VPL / 2; ++k) {
            const int i = lane + 32 * k;
            const float c = cs[i], s_ = sn[i];
            dst[i] = (v[k] * c - v[k + VPL / 2] * s_) * mul;
            dst[i + D / 2] = (v[k + VPL / 2] * c + v[k] * s_) * mul;
        }
    } else {
#pragma unroll
        for (int k = 0; k < VPL / 2; ++k) {
            const int j = VPL / 2 * lane + k;          // pair index
            const float c = cs[j], s_ = sn[j];
            dst[2 * j] = (v[2 * k] * c - v[2 * k + 1] * s_) * mul;
            dst[2 * j + 1] = (v[2 * k + 1] * c + v[2 * k] * s_) * mul;
        }
    }
}

// One thread-block cluster of ATT_CLUSTER CTAs per KV head.  CTA r of the cluster walks cache chunks
// r, r+CL, r+2CL, ... (128 positions each) with an online softmax, then the CTAs exchange their partial
// {max, sum, output} through distributed shared memory and each writes 1/CL of the head group's output.
// D (head size) is 64, 128 or 256; G is the number of query heads per KV head.
constexpr int ATT_CLUSTER = 8;

template <int D>
struct AttnShared {
    float qs[ATT_MAX_GROUP][D];                             // normalised, rotated, pre-scaled queries
    float kn[D];
    float sc[ATT_MAX_GROUP][ATT_CHUNK];                     // scores, then probabilities of the current chunk
    float hm[ATT_MAX_GROUP], hl[ATT_MAX_GROUP];             // chunk max / sum
    float M[ATT_MAX_GROUP], L[ATT_MAX_GROUP];               // running max / sum of this CTA (read by peers)
    float O[ATT_MAX_GROUP][D];                              // this CTA's unnormalised output (read by peers)
    float red[ATT_THREADS / 32][ATT_MAX_GROUP][D];          // cross-warp reduction
};

template <int G, int D>
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(const __grid_constant__ AttnParams P) {
    extern __shared__ __align__(16) uint8_t att_smem_raw[];
    using Shared = AttnShared<D>;
    Shared& sh = *reinterpret_cast<Shared*>(att_smem_raw);
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    auto stamp = [&](int k) {
        if (P.trace && threadIdx.x == 0 && blockIdx.x == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            P.trace[k] = t;
        }
    };
    stamp(0);
    pdl_launch_dependents();
    const bool dataflow = P.q_ll != nullptr;
    if (!dataflow || P.hard_wait) pdl_wait();
    stamp(1);

    constexpr int VPL = D / 32;                    // values of one head per lane
    constexpr int KU4 = D / 16;                    // 16-byte loads per thread for half a K row
    constexpr int DC = D / 8;                      // P@V: column threads (8 dims each) ...
    constexpr int RG = ATT_THREADS / DC;           // ... x row groups
    constexpr int VU4 = ATT_CHUNK / RG;            // 16-byte V loads per thread and chunk
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t gen = P.gen ? *reinterpret_cast<const volatile uint32_t*>(P.gen) : 0u;
    const uint32_t in_seq = gen * LL_SEQ_MUL + P.in_seq_add, out_seq = gen * LL_SEQ_MUL + P.out_seq_add;
    const unsigned long long budget = (dataflow && *reinterpret_cast<volatile int*>(P.status) != 0) ? 0ull : P.wait_ns;
    const int crank = (int)cluster.block_rank();
    const int kvh = blockIdx.x / ATT_CLUSTER;
    const int pos = min(P.ctrl[CTRL_POS], P.max_seq - 1);
    const int T = pos + 1;
    const int lo = (P.window > 0 && T > P.window) ? T - P.window : 0;     // first visible position
    const int first_chunk = lo / ATT_CHUNK;
    const int nchunk = (T + ATT_CHUNK - 1) / ATT_CHUNK;
    const float* cs = P.cos + (size_t)pos * (D / 2);
    const float* sn = P.sin + (size_t)pos * (D / 2);
    __half* kc = P.k_cache + (size_t)kvh * P.max_seq * D;
    __half* vc = P.v_cache + (size_t)kvh * P.max_seq * D;
    // my first chunk: the smallest c >= first_chunk with c % CL == crank
    int c0 = first_chunk + ((crank - first_chunk) % ATT_CLUSTER + ATT_CLUSTER) % ATT_CLUSTER;
    const bool active = c0 < nchunk;

    // ---- prologue: q heads of this group (normalised, rotated, pre-scaled by scale * log2(e));
    //      the CTA whose chunk holds `pos` normalises/rotates the new K and writes K,V into the cache
    const bool owns_new = active && ((pos / ATT_CHUNK) % ATT_CLUSTER == crank);
    if (active && warp < G) {
        const size_t o = (size_t)(kvh * G + warp) * D;
        const VecSrc qs{P.q ? P.q + o : nullptr, dataflow ? P.q_ll + o : nullptr, in_seq, P.status, budget};
        norm_rope_head<D>(qs, P.q_norm, P.eps, cs, sn, P.neox, P.scale * 1.4426950408889634f, sh.qs[warp], lane);
    }
    if (owns_new && warp == ATT_THREADS / 32 - 1) {
        const size_t o = (size_t)kvh * D;
        const VecSrc ks{P.k ? P.k + o : nullptr, dataflow ? P.k_ll + o : nullptr, in_seq, P.status, budget};
        const VecSrc vs{P.v ? P.v + o : nullptr, dataflow ? P.v_ll + o : nullptr, in_seq, P.status, budget};
        norm_rope_head<D>(ks, P.k_norm, P.eps, cs, sn, P.neox, 1.0f, sh.kn, lane);
        __syncwarp();
        float vv[VPL];
        int idx[VPL];
#pragma unroll
        for (int k = 0; k < VPL; ++k) idx[k] = lane + 32 * k;
        vs.getn<VPL>(idx, vv);
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
            const int i = lane + 32 * k;
            kc[(size_t)pos * D + i] = __float2half_rn(sh.kn[i]);
            vc[(size_t)pos * D + i] = __float2half_rn(vv[k]);
        }
    }
    if (tid < ATT_MAX_GROUP) { sh.M[tid] = -INFINITY; sh.L[tid] = 0.f; }
    __syncthreads();
    stamp(2);

    const int rg = tid / DC, dc = tid % DC;          // P@V mapping: RG row-groups x DC column-threads (8 dims each)
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[g][k] = 0.f;
    float run_m[G];                      // running max per head (same value in every thread)
#pragma unroll
    for (int g = 0; g < G; ++g) run_m[g] = -INFINITY;

    for (int c = c0; c < nchunk; c += ATT_CLUSTER) {
        const int base = c * ATT_CHUNK;
        const int t0 = max(base, lo), t1 = min(base + ATT_CHUNK, T);
        // ---- scores: two threads per cache position, D/2 dims each; all loads issued before any math
        {
            const int tl = tid >> 1, hf = tid & 1;
            const int t = base + tl;
            const bool valid = t >= t0 && t < t1;
            uint4 raw[KU4];
            if (valid) {
                const uint4* kp = reinterpret_cast<const uint4*>(kc + (size_t)t * D + hf * (D / 2));
#pragma unroll
                for (int i = 0; i < KU4; ++i) raw[i] = kp[i];
            }
            float s[G];
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] = 0.f;
            if (valid) {
#pragma unroll
                for (int i = 0; i < KU4; ++i) {
                    const __half2* h2 = reinterpret_cast<const __half2*>(&raw[i]);
                    float kf[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h2[k]); kf[2 * k] = f.x; kf[2 * k + 1] = f.y; }
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float4 qa = *reinterpret_cast<const float4*>(&sh.qs[g][hf * (D / 2) + i * 8]);
                        const float4 qb = *reinterpret_cast<const float4*>(&sh.qs[g][hf * (D / 2) + i * 8 + 4]);
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
        // V for this chunk: issue the loads now, they land while the softmax statistics are computed
        uint4 vraw[VU4];
#pragma unroll
        for (int i = 0; i < VU4; ++i) {
            const int t = base + rg + RG * i;
            vraw[i] = (t >= t0 && t < t1) ? *reinterpret_cast<const uint4*>(vc + (size_t)t * D + dc * 8) : make_uint4(0, 0, 0, 0);
        }
        __syncthreads();
        // ---- softmax statistics of this chunk (base 2): warp g handles head g
        if (warp < G) {
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
        __syncthreads();
        // ---- merge the chunk into the running state and accumulate P @ V
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float mc = sh.hm[g];
            const float mn = fmaxf(run_m[g], mc);
            const float so = exp2f(run_m[g] - mn), sc_ = exp2f(mc - mn);    // exp2f(-inf) = 0 on the first chunk
            run_m[g] = mn;
            if (tid == g) { sh.L[g] = sh.L[g] * so + sh.hl[g] * sc_; sh.M[g] = mn; }
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[g][k] *= so;
#pragma unroll
            for (int i = 0; i < VU4; ++i) {
                const float p = sh.sc[g][rg + RG * i] * sc_;
                const __half2* h2 = reinterpret_cast<const __half2*>(&vraw[i]);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = __half22float2(h2[k]);
                    acc[g][2 * k] += p * f.x;
                    acc[g][2 * k + 1] += p * f.y;
                }
            }
        }
        __syncthreads();       // sc/hm/hl are rewritten by the next chunk
    }
    stamp(3);
    // ---- combine the row-groups: first those that share a warp (32 / DC of them), then the 8 warps through shared memory
    if (active) {
#pragma unroll
        for (int off = 16; off >= DC; off >>= 1)
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[g][k] += __shfl_xor_sync(0xffffffffu, acc[g][k], off);
        if (lane < DC) {
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int k = 0; k < 8; ++k) sh.red[warp][g][(lane % DC) * 8 + k] = acc[g][k];
        }
        __syncthreads();
        for (int i = tid; i < G * D; i += ATT_THREADS) {
            const int g = i / D, d = i - g * D;
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < ATT_THREADS / 32; ++w) o += sh.red[w][g][d];
            sh.O[g][d] = o;
        }
    }
    cluster.sync();
    stamp(4);
    // ---- cluster merge: this CTA finishes G*D/CL outputs from every peer's {M, L, O}
    {
        constexpr int per = G * D / ATT_CLUSTER;
        static_assert(per <= ATT_THREADS, "one thread per merged output");
        if (tid < per) {
            const int i = crank * per + tid;
            const int g = i / D, d = i - g * D;
            float Mx = -INFINITY;
            float pm[ATT_CLUSTER];
#pragma unroll
            for (int p = 0; p < ATT_CLUSTER; ++p) {
                const Shared* ps = cluster.map_shared_rank(&sh, p);
                pm[p] = ps->M[g];
                Mx = fmaxf(Mx, pm[p]);
            }
            float Lt = 0.f, Ot = 0.f;
#pragma unroll
            for (int p = 0; p < ATT_CLUSTER; ++p) {
                if (pm[p] > -INFINITY) {
                    const Shared* ps = cluster.map_shared_rank(&sh, p);
                    const float w = exp2f(pm[p] - Mx);
                    Lt += w * ps->L[g];
                    Ot += w * ps->O[g][d];
                }
            }
            const size_t oi = (size_t)(kvh * G + g) * D + d;
            if (P.out_ll) st_ll(P.out_ll + oi, __float_as_uint(Ot / Lt), out_seq);
            else P.out[oi] = Ot / Lt;
        }
    }
    cluster.sync();      // peers may still be reading this CTA's shared memory
    stamp(5);
}

// ---------------------------------------------------------------------------------------------
// Embedding row -> fp32 residual stream.  Row layouts as for the GEMV (Q4_K blocks / Q6_K SoA),
// plus fp16 (qtype 2) and fp32 (qtype 3).
struct EmbedParams {
    const uint8_t* table;
    int qtype, rowbytes, nblk, H;
    float scale;
    float* out;          // plain fp32 row, or
    uint2* out_ll;       // {value, sequence} slots with sequence gen * LL_SEQ_MUL (the first write of the token)
    const int* ctrl;
    int vocab;
    int* status;
    const uint32_t* gen; // token generation counter (bumped by the token's last kernel)
};

static __global__ void __launch_bounds__(256) embed_kernel(const __grid_constant__ EmbedParams P) {
    pdl_launch_dependents();
    pdl_wait();
    int tok = P.ctrl[CTRL_TOKEN];
    if (tok < 0 || tok >= P.vocab) {
        if (threadIdx.x == 0) atomicExch(P.status, PTB_ERR_BOUNDS);
        tok = 0;
    }
    const uint32_t seq = (P.gen ? *reinterpret_cast<const volatile uint32_t*>(P.gen) : 0u) * LL_SEQ_MUL;
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
        if (P.out_ll) st_ll(P.out_ll + i, __float_as_uint(v * P.scale), seq);
        else P.out[i] = v * P.scale;
    }
}

}  // namespace ptb
