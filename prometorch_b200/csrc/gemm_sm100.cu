// Host side of the tcgen05 GEMM: tensor-map encoding (the driver entry point is
// resolved at run time, so the library loads on machines without a driver) and
// the launcher that picks the tile width and operand majors.
#include "gemm_sm100.cuh"
#include <cudaTypedefs.h>
#include <string.h>
#include <algorithm>
#include <mutex>

using namespace ptb;
using namespace ptb::gemm;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, row pitch `ld` elements.
int ptb_make_tmap_bf16(CUtensorMap* map, const void* base, long long inner, long long outer, long long ld, int box_inner, int box_outer) {
    EncodeTiledFn enc = get_encode();
    if (!enc) { ptb_set_error("cuTensorMapEncodeTiled is not available (no CUDA driver?)"); return -1; }
    if (((uintptr_t)base & 15) || ((ld * 2) & 15)) { ptb_set_error("TMA operand needs a 16-byte aligned base and row pitch (ld=%lld)", ld); return -1; }
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { ptb_set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return -1; }
    return 0;
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch(const Operand& ta, const Operand& tb, const Params& p, int n_sm, cudaStream_t st) {
    auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
    static bool attr = false;
    constexpr int smem = Smem<BN, STAGES>::TOTAL;
    if (!attr) {
        PTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr = true;
    }
    Params q = p;
    int n_st = q.stager_ctas ? std::min(16, std::max(1, n_sm / 8)) : 0;      // stager_ctas arrives as a yes/no request
    // the stagers and the tile CTAs wait on one another, so the whole grid must be resident at once: one CTA per SM
    const int gemm_ctas = std::max(1, std::min(p.tiles_m * p.tiles_n * std::max(1, p.splits), n_sm - n_st));
    q.stager_ctas = n_st;
    PTB_CUDA_OK(ptb_launch(kern, dim3(gemm_ctas + n_st), dim3(THREADS), (size_t)smem, st, q.pdl != 0, ta, tb, q));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

template <int BN, int STAGES>
static int launch_majors(int a_mn, int b_mn, const Operand& ta, const Operand& tb, const Params& p, int n_sm, cudaStream_t st) {
    if (!a_mn && !b_mn) return launch<BN, STAGES, false, false>(ta, tb, p, n_sm, st);
    if (!a_mn && b_mn) return launch<BN, STAGES, false, true>(ta, tb, p, n_sm, st);
    if (a_mn && !b_mn) return launch<BN, STAGES, true, false>(ta, tb, p, n_sm, st);
    return launch<BN, STAGES, true, true>(ta, tb, p, n_sm, st);
}

// Describe one operand.  ptrs: `nshards` base pointers (piece r in GPU r's memory, or one local pointer).
//   K-major (mn == 0): stored [rows_total, K] row-major, split by rows into pieces of shard_rows.
//   MN-major (mn == 1): stored [K, cols] row-major, split by rows (i.e. along K) into pieces of shard_rows.
static int make_operand(Operand& op, void* const* ptrs, int nshards, int shard_rows, long long ld, int mn, int rows_total,
                        int K, int box_rows) {
    memset(&op, 0, sizeof(op));
    op.nshards = nshards;
    op.shard_rows = shard_rows;
    if (nshards < 1 || nshards > MAX_SHARDS) { ptb_set_error("gemm: %d shards (1..%d supported)", nshards, MAX_SHARDS); return -1; }
    const int box_outer = mn ? 64 : box_rows;
    if (nshards > 1 && shard_rows % box_outer) {
        ptb_set_error("gemm: shard of %d rows must be a multiple of the %d-row TMA box", shard_rows, box_outer);
        return -1;
    }
    const long long stored_rows = mn ? K : rows_total;
    for (int r = 0; r < nshards; ++r) {
        long long rows_here = nshards > 1 ? std::min<long long>(shard_rows, stored_rows - (long long)r * shard_rows) : stored_rows;
        if (rows_here <= 0) rows_here = 1;   // an empty trailing shard is never addressed
        const long long inner = mn ? rows_total : K;
        if (ptb_make_tmap_bf16(&op.map[r], ptrs[r], inner, rows_here, ld, 64, box_outer)) return -1;
    }
    return 0;
}

#include "ptb200_types.h"
static void fill_staging(Staging& S, const PtbStaging* h) {
    memset(&S, 0, sizeof(S));
    if (!h || h->seq == 0) return;
    for (int i = 0; i < MAX_SHARDS; ++i) S.peer[i] = (const uint4*)h->peer[i];
    S.local = (uint4*)h->local;
    S.flags = (uint32_t*)h->flags;
    S.rank = h->rank; S.world = h->world; S.shard_rows = h->shard_rows; S.stored_rows = h->stored_rows;
    S.row_vec = h->row_bytes / 16;
    S.seq = h->seq;
}

// General entry point.  a_ptrs/b_ptrs: arrays of a_shards/b_shards device pointers.  c_peers (EPI_SCATTER_ADD):
// `c_shards` fp32 buffers [out_shard_rows, ldc], one per rank.
struct SplitK { int splits; long long stride; int bn; int pdl; };      // splits > 1: fp32 partials at C + s*stride; bn: 0 or a forced tile width

static int gemm_core(void* const* a_ptrs, int a_shards, int a_shard_rows, long long lda, int a_mn, void* const* b_ptrs,
                     int b_shards, int b_shard_rows, long long ldb, int b_mn, void* C, long long ldc, void* const* c_peers,
                     int c_shards, int out_shard_rows, int M, int N, int K, const float* bias, int flags, int* status,
                     int n_sm, cudaStream_t st, const PtbStaging* stage_a, const PtbStaging* stage_b, SplitK sk) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    {
        int dev = 0;
        PTB_CUDA_OK(cudaGetDevice(&dev));
        PTB_CUDA_OK(cudaSetDevice(dev));     // the tensor-map encoder is a driver call: bind the primary context to this thread
        if (n_sm <= 0) PTB_CUDA_OK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
    }
    Params p;
    memset(&p, 0, sizeof(p));
    // flags bits 8..15: this rank's slot for EPI_SCATTER_STORE
    const int scatter_rank = (flags >> 8) & 0xff;
    flags &= 0xff;
    if (flags & (EPI_SCATTER_ADD | EPI_SCATTER_STORE)) {
        if ((flags & EPI_SCATTER_STORE) && ((ldc * 2) & 15)) { ptb_set_error("gemm: scatter-store needs a 16-byte row pitch"); return -1; }
        p.scatter_rank = scatter_rank;
        if (c_shards < 1 || c_shards > MAX_SHARDS || out_shard_rows % BM) {
            ptb_set_error("gemm: scatter-add needs 1..8 output shards of a multiple of %d rows", BM);
            return -1;
        }
        for (int r = 0; r < c_shards; ++r) p.c_peer[r] = (float*)c_peers[r];
        p.out_shard_rows = out_shard_rows;
    } else if (flags & EPI_TRANS) {
        if (!(flags & EPI_OUT_F32) || ((uintptr_t)C & 3)) { ptb_set_error("gemm: transposed output is fp32"); return -1; }
    } else {
        const int out_elem = (flags & EPI_OUT_F32) ? 4 : 2;
        if (((uintptr_t)C & 15) || ((ldc * out_elem) & 15)) { ptb_set_error("gemm: C needs a 16-byte aligned base and row pitch"); return -1; }
    }
    int BN = N > 128 ? 256 : 128;
    if (BN == 256) {
        // tile quantisation: with few tiles the last wave of 128x256 tiles can leave most SMs idle; 128x128 tiles
        // run at ~0.85 of the wide tile's rate but fill the waves better
        const long long tm = (M + BM - 1) / BM;
        auto eff = [&](int bn) {
            const long long t = tm * ((N + bn - 1) / bn), waves = (t + n_sm - 1) / n_sm;
            return (double)t / (double)(waves * n_sm);
        };
        if (0.85 * eff(128) > eff(256)) BN = 128;
    }
    if (!b_mn && b_shards > 1 && b_shard_rows % 256) BN = 128;
    if (sk.bn) BN = sk.bn;
    const int kblocks = (K + BK - 1) / BK;
    p.splits = std::max(1, sk.splits);
    p.kb_per_split = (kblocks + p.splits - 1) / p.splits;
    p.splits = (kblocks + p.kb_per_split - 1) / p.kb_per_split;          // no empty split
    p.split_stride = sk.stride;
    p.pdl = sk.pdl;
    fill_staging(p.stA, stage_a);
    fill_staging(p.stB, stage_b);
    // stager CTAs are needed unless every staged operand is filled by an external copier
    p.stager_ctas = ((p.stA.seq && !(stage_a && stage_a->external)) || (p.stB.seq && !(stage_b && stage_b->external))) ? 1 : 0;
    if ((p.stA.seq && (p.stA.shard_rows % STAGE_ROWS)) || (p.stB.seq && (p.stB.shard_rows % STAGE_ROWS))) {
        ptb_set_error("gemm: staged shards must be a multiple of %d rows", STAGE_ROWS);
        return -1;
    }
    Operand oa, ob;
    if (make_operand(oa, a_ptrs, a_shards, a_shard_rows, lda, a_mn, M, K, BM)) return -1;
    if (make_operand(ob, b_ptrs, b_shards, b_shard_rows, ldb, b_mn, N, K, BN)) return -1;
    p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.bias = bias; p.flags = flags; p.status = status;
    p.tiles_m = (M + BM - 1) / BM;
    p.tiles_n = (N + BN - 1) / BN;
    if (BN == 32 || BN == 64) {
        if (a_mn || b_mn || p.stA.seq || p.stB.seq) { ptb_set_error("gemm: narrow tiles take K-major, unstaged operands"); return -1; }
        return BN == 32 ? launch<32, 10, false, false>(oa, ob, p, n_sm, st) : launch<64, 8, false, false>(oa, ob, p, n_sm, st);
    }
    if (BN == 256) return launch_majors<256, 4>(a_mn, b_mn, oa, ob, p, n_sm, st);
    return launch_majors<128, 6>(a_mn, b_mn, oa, ob, p, n_sm, st);
}

PTB_API int ptb_gemm_bf16_ex(void* const* a_ptrs, int a_shards, int a_shard_rows, long long lda, int a_mn, void* const* b_ptrs,
                             int b_shards, int b_shard_rows, long long ldb, int b_mn, void* C, long long ldc, void* const* c_peers,
                             int c_shards, int out_shard_rows, int M, int N, int K, const float* bias, int flags, int* status,
                             int n_sm, cudaStream_t st, const PtbStaging* stage_a, const PtbStaging* stage_b) {
    return gemm_core(a_ptrs, a_shards, a_shard_rows, lda, a_mn, b_ptrs, b_shards, b_shard_rows, ldb, b_mn, C, ldc, c_peers, c_shards,
                     out_shard_rows, M, N, K, bias, flags, status, n_sm, st, stage_a, stage_b, SplitK{1, 0, 0, 0});
}

// Sum the split-K partials, add the bias, apply GELU, round to bf16.  work: [splits][M][N] fp32; N a multiple of 4.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ work, int splits, long long mn, int N,
                                                            const float* __restrict__ bias, int gelu, __nv_bfloat16* __restrict__ C,
                                                            long long ldc) {
    pdl_wait();
    pdl_launch_dependents();
    const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i4 >= mn) return;
    float4 acc = *reinterpret_cast<const float4*>(work + i4);
    for (int s = 1; s < splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(work + (size_t)s * mn + i4);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const long long row = i4 / N;
    const int col = (int)(i4 - row * N);
    if (bias) { acc.x += bias[col]; acc.y += bias[col + 1]; acc.z += bias[col + 2]; acc.w += bias[col + 3]; }
    if (gelu) { acc.x = gelu_tanh(acc.x); acc.y = gelu_tanh(acc.y); acc.z = gelu_tanh(acc.z); acc.w = gelu_tanh(acc.w); }
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(C + row * ldc + col);
    o[0] = __floats2bfloat162_rn(acc.x, acc.y);
    o[1] = __floats2bfloat162_rn(acc.z, acc.w);
}

// Split-K sum fused with what follows a projection in a decoder layer, so the partials are read once and the layer
// saves a launch: (a) residual add + RMSNorm after the attention-output and MLP-down projections, (b) the gated
// activation after the packed gate/up projection.
constexpr int SKN_THREADS = 256, SKN_MAXC = 8;            // up to 8 float4 chunks per thread: N <= 8192

// One CTA per row.  h = sum_s work[s][row] + resid_in[row] (rounded to bf16, stored in resid_out); y = rmsnorm(h) * w.
__global__ void __launch_bounds__(SKN_THREADS) splitk_reduce_norm_kernel(const float* __restrict__ work, int splits, long long mn, int N,
                                                                         const __nv_bfloat16* __restrict__ resid_in,
                                                                         __nv_bfloat16* __restrict__ resid_out,
                                                                         const __nv_bfloat16* __restrict__ w, float eps,
                                                                         __nv_bfloat16* __restrict__ y) {
    __shared__ float red[32];
    pdl_wait();
    pdl_launch_dependents();
    const size_t row = blockIdx.x;
    const int nc = N / 4;
    float4 h[SKN_MAXC];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < SKN_MAXC; ++k) {
        const int c = k * SKN_THREADS + threadIdx.x;
        if (c < nc) {
            float4 a = *reinterpret_cast<const float4*>(work + row * N + (size_t)c * 4);
            for (int s = 1; s < splits; ++s) {
                const float4 v = *reinterpret_cast<const float4*>(work + (size_t)s * mn + row * N + (size_t)c * 4);
                a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
            }
            const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(resid_in + row * N + (size_t)c * 4);
            const float2 r0 = __bfloat1622float2(r2[0]), r1 = __bfloat1622float2(r2[1]);
            const __nv_bfloat162 o0 = __floats2bfloat162_rn(a.x + r0.x, a.y + r0.y), o1 = __floats2bfloat162_rn(a.z + r1.x, a.w + r1.y);
            __nv_bfloat162* out2 = reinterpret_cast<__nv_bfloat162*>(resid_out + row * N + (size_t)c * 4);
            out2[0] = o0; out2[1] = o1;
            const float2 f0 = __bfloat1622float2(o0), f1 = __bfloat1622float2(o1);      // normalise what was stored
            h[k] = make_float4(f0.x, f0.y, f1.x, f1.y);
            ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y;
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = (threadIdx.x & 31) < SKN_THREADS / 32 ? red[threadIdx.x & 31] : 0.f;
    t = warp_sum(t);
    const float rs = rsqrtf(t / (float)N + eps);
#pragma unroll
    for (int k = 0; k < SKN_MAXC; ++k) {
        const int c = k * SKN_THREADS + threadIdx.x;
        if (c < nc) {
            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(w + (size_t)c * 4);
            const float2 w0 = __bfloat1622float2(w2[0]), w1 = __bfloat1622float2(w2[1]);
            __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(y + row * N + (size_t)c * 4);
            y2[0] = __floats2bfloat162_rn(h[k].x * rs * w0.x, h[k].y * rs * w0.y);
            y2[1] = __floats2bfloat162_rn(h[k].z * rs * w1.x, h[k].w * rs * w1.y);
        }
    }
}

// out[row][c] = act(sum_s gate) * (sum_s up) for the packed projection [M, 2 I] (gate columns first).
__global__ void __launch_bounds__(256) splitk_reduce_gated_kernel(const float* __restrict__ work, int splits, long long mn, int I, int gelu,
                                                                  long long total4, __nv_bfloat16* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    const long long i4 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i4 >= total4) return;
    const long long row = (i4 * 4) / I;
    const int col = (int)(i4 * 4 - row * I);
    const float* base = work + row * 2 * I + col;
    float4 g = *reinterpret_cast<const float4*>(base), u = *reinterpret_cast<const float4*>(base + I);
    for (int s = 1; s < splits; ++s) {
        const float4 a = *reinterpret_cast<const float4*>(base + (size_t)s * mn), b = *reinterpret_cast<const float4*>(base + (size_t)s * mn + I);
        g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
        u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
    }
    auto act = [&](float x) { return gelu ? gelu_tanh(x) : silu(x); };
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(out + row * I + col);
    o[0] = __floats2bfloat162_rn(act(g.x) * u.x, act(g.y) * u.y);
    o[1] = __floats2bfloat162_rn(act(g.z) * u.z, act(g.w) * u.w);
}

// Shape of a skinny GEMM (M <= 128 rows of activations).  Returns 0 when the ordinary path should run, else
// splits | mode << 8 with mode 0: 128-wide tiles, 1: 256-wide tiles, 2: swapped operands.
//   swapped (M <= 64): the weight is the 128-row operand and the tokens are a 32- or 64-column tile, so a k-block moves
//   16 KB of weights and 4-8 KB of activations, ten stages keep ~160 KB of weights in flight per SM and the tensor
//   pipe does 128 x 32 x 64 instead of 128 x 128 x 64 per k-block; the result always goes through the reduce launch.
// The CTAs are persistent and their TMA producers run ahead across work items, so the makespan is about
// (items per SM) x (k-blocks per item x time per k-block + a partly hidden epilogue) + a fixed cost + the reduce pass.
static int pick_skinny(int M, int N, int K, int n_sm) {
    if (M > BM || n_sm <= 0) return 0;
    const int kblocks = (K + BK - 1) / BK;
    int best = 0;
    double best_cost = 1e30;
    for (int mode = 0; mode < 3; ++mode) {
        if (mode == 1 && N <= 128) continue;
        if (mode == 2 && M > 64) continue;
        if (mode != 2 && M <= 64) continue;
        const int bn = mode == 1 ? 256 : 128, tiles = (N + bn - 1) / bn;
        const double t_kb = mode == 2 ? 0.15 : mode == 1 ? 0.33 : 0.25;
        for (int s = 1; s <= 16 && s <= kblocks; ++s) {
            const int kbps = (kblocks + s - 1) / s, items = tiles * ((kblocks + kbps - 1) / kbps);
            const int per_sm = (items + n_sm - 1) / n_sm;
            const bool reduce = s > 1 || mode == 2;
            const double cost = per_sm * (kbps * t_kb + 0.4) + 3.0 + (reduce ? 2.5 + (double)s * M * N * 4.0 / 4.0e6 : 0.0);
            if (cost < best_cost - 1e-9) { best_cost = cost; best = s | (mode << 8); }
        }
    }
    if ((best >> 8) != 2 && (best & 0xff) == 1) return 0;          // one split, ordinary tiles: nothing to reduce
    return best;
}

// 0: use the ordinary GEMM; otherwise the split count of the skinny path (1 or more; its result needs the reduce launch).
PTB_API int ptb_gemm_pick_splits(int M, int N, int K, int n_sm) { return pick_skinny(M, N, K, n_sm) & 0xff; }

static int skinny_partials(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K, int splits, float* work,
                           int* status, int n_sm, cudaStream_t st, int* real_splits) {
    if (M > BM || (N & 3) || splits < 1 || !work) { ptb_set_error("gemm split-K: needs M <= %d, N %% 4 == 0, splits >= 1 and a workspace", BM); return -1; }
    void* ap[1] = {const_cast<void*>(A)};
    void* bp[1] = {const_cast<void*>(B)};
    {
        int dev = 0;
        PTB_CUDA_OK(cudaGetDevice(&dev));
        if (n_sm <= 0) PTB_CUDA_OK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
    }
    const int choice = pick_skinny(M, N, K, n_sm);
    const int mode = M <= 64 ? 2 : (((choice >> 8) == 1 && (choice & 0xff) == splits) ? 1 : 0);
    int rc;
    if (mode == 2) {
        // swapped: "A" = the weight [N, K] (rows = output features), "B" = the activations [M, K]; partials are stored
        // transposed, i.e. as [splits][M][N] like the other modes
        rc = gemm_core(bp, 1, 0, ldb, 0, ap, 1, 0, lda, 0, work, N, nullptr, 0, 0, N, M, K, nullptr, EPI_OUT_F32 | EPI_TRANS, status, n_sm, st,
                       nullptr, nullptr, SplitK{splits, (long long)M * N, M <= 32 ? 32 : 64, ptb_pdl_enabled() ? 1 : 0});
    } else {
        rc = gemm_core(ap, 1, 0, lda, 0, bp, 1, 0, ldb, 0, work, N, nullptr, 0, 0, M, N, K, nullptr, EPI_OUT_F32, status, n_sm, st, nullptr, nullptr,
                       SplitK{splits, (long long)M * N, mode == 1 ? 256 : 128, ptb_pdl_enabled() ? 1 : 0});
    }
    if (rc) return -1;
    const int kblocks = (K + BK - 1) / BK, kbps = (kblocks + splits - 1) / splits;
    *real_splits = (kblocks + kbps - 1) / kbps;
    return 0;
}

// Skinny GEMM (M <= 128), K-major operands: C[M,N] bf16 = A[M,K] B[N,K]^T (+ bias, GELU) with `splits` K-splits whose
// fp32 partials go through `work` ([splits][M][N] floats) and one reduce launch.  N must be a multiple of 4.
PTB_API int ptb_gemm_bf16_splitk(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M, int N, int K,
                                 const float* bias, int gelu, int splits, float* work, int* status, int n_sm, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    int real = 0;
    if (skinny_partials(A, lda, B, ldb, M, N, K, splits, work, status, n_sm, st, &real)) return -1;
    const long long mn = (long long)M * N;
    PTB_CUDA_OK(ptb_launch(splitk_reduce_kernel, dim3((unsigned)((mn / 4 + 255) / 256)), dim3(256), 0, st, ptb_pdl_enabled(), work, real, mn, N, bias,
                           gelu, (__nv_bfloat16*)C, ldc));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// Only the partials: work [splits'][M][N] fp32, where splits' (returned, >= 1) is the number of splits that really ran.
// The caller's next kernel sums them (e.g. ptb_paged_rope_write_partials).  Returns -1 on error.
PTB_API int ptb_gemm_bf16_splitk_partials(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K, int splits,
                                          float* work, int* status, int n_sm, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    int real = 0;
    if (skinny_partials(A, lda, B, ldb, M, N, K, splits, work, status, n_sm, st, &real)) return -1;
    return real;
}

// The same product followed, in the reduce launch, by `resid_out = P + resid_in` and `y = rmsnorm(resid_out) * norm_w`
// (all bf16, [M, N] contiguous; N <= 8192).
PTB_API int ptb_gemm_bf16_splitk_add_norm(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K, int splits,
                                          float* work, const void* resid_in, void* resid_out, const void* norm_w, float eps, void* y,
                                          int* status, int n_sm, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (N > 4 * SKN_THREADS * SKN_MAXC) { ptb_set_error("gemm split-K + norm: N %d above %d", N, 4 * SKN_THREADS * SKN_MAXC); return -1; }
    int real = 0;
    if (skinny_partials(A, lda, B, ldb, M, N, K, splits, work, status, n_sm, st, &real)) return -1;
    PTB_CUDA_OK(ptb_launch(splitk_reduce_norm_kernel, dim3(M), dim3(SKN_THREADS), 0, st, ptb_pdl_enabled(), work, real, (long long)M * N, N,
                           (const __nv_bfloat16*)resid_in, (__nv_bfloat16*)resid_out, (const __nv_bfloat16*)norm_w, eps, (__nv_bfloat16*)y));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// The packed gate/up projection (N = 2 I, gate columns first) followed by out[M, I] = act(gate) * up in the reduce launch.
PTB_API int ptb_gemm_bf16_splitk_gated(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K, int splits,
                                       float* work, int gelu, void* out, int* status, int n_sm, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (N & 7) { ptb_set_error("gemm split-K + gate: N must be a multiple of 8"); return -1; }
    int real = 0;
    if (skinny_partials(A, lda, B, ldb, M, N, K, splits, work, status, n_sm, st, &real)) return -1;
    const long long total4 = (long long)M * (N / 2) / 4;
    PTB_CUDA_OK(ptb_launch(splitk_reduce_gated_kernel, dim3((unsigned)((total4 + 255) / 256)), dim3(256), 0, st, ptb_pdl_enabled(), work, real,
                           (long long)M * N, N / 2, gelu, total4, (__nv_bfloat16*)out));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// C[M,N] (+)= op(A) op(B)^T with bf16 operands and fp32 accumulation, all operands local.
//   a_mn == 0: A is [M, K] row-major (pitch lda);  a_mn == 1: A is stored as [K, M] row-major.
//   b_mn == 0: B is [N, K] row-major (pitch ldb);  b_mn == 1: B is stored as [K, N] row-major.
//   flags: EPI_BIAS | EPI_ACCUM | EPI_OUT_F32 | EPI_GELU.  status: device int, set non-zero if a wait timed out.
PTB_API int ptb_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* C, long long ldc,
                          int M, int N, int K, const float* bias, int flags, int* status, int n_sm, cudaStream_t st) {
    void* ap[1] = {const_cast<void*>(A)};
    void* bp[1] = {const_cast<void*>(B)};
    return ptb_gemm_bf16_ex(ap, 1, 0, lda, a_mn, bp, 1, 0, ldb, b_mn, C, ldc, nullptr, 0, 0, M, N, K, bias, flags, status, n_sm, st, nullptr, nullptr);
}
