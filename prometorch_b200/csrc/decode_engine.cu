// Host side of the decode path: launch planning for the GEMV, and the engine
// that strings one token's kernels together, captures them into a CUDA graph
// (with programmatic dependent launch edges so each kernel's weight prefetch
// overlaps its predecessor's tail) and replays it per token.
//
// What the reference does in GGUFModel::forward_decode
// (torch/io/gguf_model.h:2575-3113): ~10 kernels per layer, eager on token 1,
// captured on token 2, replayed afterwards, arg-max in a separate launch plus an
// 8-byte device-to-host copy per token.  Here a layer is five kernels, the
// arg-max is the lm_head epilogue and a run of tokens needs no host round trip.
//
// Dataflow between the kernels of a token: every activation vector is a buffer of
// {value, sequence} slots.  A kernel is launched as soon as all CTAs of its predecessor
// have started, streams its weights into shared memory and polls its input slots; it
// never waits for the predecessor to drain.  The only hard boundary is the start of a
// token (the embedding kernel is launched without a programmatic edge), which is also
// what makes it safe to reuse the slot buffers: sequence numbers grow with the token
// generation counter.  Partial sums of the K-split projections (all ranks' under tensor
// parallelism, one at world size 1) land in inbox slots and are added, in rank order,
// by the prologue of whichever kernel consumes the residual stream next.
#include "decode_kernels.cuh"
#include "decode_gemv_mma.cuh"
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>
#include <string>
#include <vector>
#include <algorithm>

static thread_local char g_err[1024];
bool ptb_pdl_enabled() {
    static const bool on = [] { const char* e = getenv("PTB_PDL"); return !(e && e[0] == '0'); }();
    return on;
}

void ptb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
PTB_API const char* ptb_last_error() { return g_err; }

using namespace ptb;

// ------------------------------------------------------------------------------------------ C structs (mirrored in Python)
#include "ptb200_types.h"

static size_t g_gemv_max_dyn = 200 * 1024;
static int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

struct GemvLaunch {
    GemvParams p;
    int grid;
    size_t smem;
    int t16;          // weights in the tiles-of-16-rows layout: launch the tensor-pipe kernel
};

// Fill job geometry, CTA split, tile ring and shared memory size.  `jobs` already carry
// w/w2/out/bias/qtype/N/nblk/KS/seg_base/seg_rem.
static int plan_gemv_seg(GemvLaunch& L, int njobs, int K, int n_ctas) {
    const int want_stages = env_int("PTB_GEMV_STAGES", 4);
    const int tile_cap = env_int("PTB_GEMV_TILE_KB", 6) * 1024;
    const size_t budget = (size_t)env_int("PTB_GEMV_SMEM_KB", 100) * 1024;
    GemvParams& p = L.p;
    p.njobs = njobs;
    p.K = K;
    const int warps = env_int("PTB_GEMV_WARPS", 8) >= 16 ? 16 : 8;
    p.warps = warps;
    p.wait_ns = (unsigned long long)env_int("PTB_WAIT_MS", 2000) * 1000000ull;
    p.hard_wait = env_int("PTB_DATAFLOW", 1) == 0;
    if (K % 256 || K > 5 * 8 * 256) {
        ptb_set_error("gemv: input length %d must be a multiple of 256 and at most %d", K, 5 * 8 * 256);
        return -1;
    }
    // CTAs proportional to bytes, at least one each, never more CTAs than rows
    double total = 0;
    for (int i = 0; i < njobs; ++i) total += (double)p.job[i].N * p.job[i].nblk * (p.job[i].qtype == QT_Q4K ? 144 : 210) * (p.job[i].w2 ? 2 : 1);
    int left = n_ctas, begin = 0;
    double left_bytes = total;
    for (int i = 0; i < njobs; ++i) {
        GemvJob& j = p.job[i];
        const double b = (double)j.N * j.nblk * (j.qtype == QT_Q4K ? 144 : 210) * (j.w2 ? 2 : 1);
        int c = (i == njobs - 1) ? left : (int)(left * b / left_bytes + 0.5);
        c = std::max(1, std::min(c, left - (njobs - 1 - i)));
        c = std::min(c, j.N);
        j.cta_begin = begin;
        j.cta_count = c;
        begin += c;
        left -= c;
        left_bytes -= b;
    }
    L.grid = begin;
    // rows per warp tile: minimise the per-warp critical path, counted in super-block visits
    int tile_bytes = 0, acc_floats = 0;
    for (int i = 0; i < njobs; ++i) {
        GemvJob& j = p.job[i];
        const int pairs = j.w2 ? 2 : 1;
        const int nb = j.seg_base + (j.seg_rem ? 1 : 0);
        const int sz = seg_bytes(j.qtype, nb);
        const int rows_cta = (j.N + j.cta_count - 1) / j.cta_count;
        double best = 1e30;
        int bestRW = 1;
        for (int RW = 8; RW >= 1; RW >>= 1) {
            if (RW > 1 && RW * sz * pairs > tile_cap) continue;
            const int gprw = 8 / RW;
            const int items = ((rows_cta + RW - 1) / RW) * j.KS;
            const int rounds = (items + warps - 1) / warps;
            const double cost = rounds * ((double)((nb + gprw - 1) / gprw) * pairs + 1.0);
            if (cost < best - 1e-9) { best = cost; bestRW = RW; }
        }
        j.RW = bestRW;
        tile_bytes = std::max(tile_bytes, bestRW * sz * pairs);
        if (j.KS > 1) acc_floats = std::max(acc_floats, rows_cta * j.KS * pairs);
    }
    tile_bytes = (tile_bytes + 127) / 128 * 128;
    int stages = want_stages;
    while (stages > 2 && gemv_smem_layout(K, warps, stages, tile_bytes, acc_floats).total > budget) --stages;
    p.stages = stages;
    p.tile_bytes = tile_bytes;
    p.acc_floats = acc_floats;
    L.smem = gemv_smem_layout(K, warps, stages, tile_bytes, acc_floats).total;
    if (L.smem > g_gemv_max_dyn) {
        ptb_set_error("gemv: %zu B of shared memory needed (K=%d, tile %d B x %d stages x %d warps, %d accumulators)", L.smem, K,
                      tile_bytes, stages, warps, acc_floats);
        return -1;
    }
    return 0;
}

static int g_job_layout = 0;      // layout of the job set_job() filled last (a launch never mixes layouts)
// Tiles-of-16-rows layout: CTAs own whole row tiles (split over the jobs in proportion to their bytes); the K
// dimension of a tile is cut into KG groups so that a CTA has enough (tile, K-group) items for its warps.
static int plan_gemv16(GemvLaunch& L, int njobs, int K, int n_ctas, int force_warps = 0) {
    GemvParams& p = L.p;
    p.njobs = njobs;
    p.K = K;
    // one CTA of 16 warps per SM: half as many CTAs repeat the input gather as with two CTAs of 8 warps
    const int warps = force_warps ? force_warps : env_int("PTB_GEMV_WARPS", 16) >= 16 ? 16 : 8;
    p.warps = warps;
    p.wait_ns = (unsigned long long)env_int("PTB_WAIT_MS", 2000) * 1000000ull;
    p.hard_wait = env_int("PTB_DATAFLOW", 1) == 0;
    if (K % 256 || K > 5 * 8 * 256) {
        ptb_set_error("gemv: input length %d must be a multiple of 256 and at most %d", K, 5 * 8 * 256);
        return -1;
    }
    double total = 0;
    auto bytes_of = [](const GemvJob& j) { return (double)((j.N + 15) / 16) * j.nblk * t16_block_bytes(j.qtype) * (j.w2 ? 2 : 1); };
    for (int i = 0; i < njobs; ++i) total += bytes_of(p.job[i]);
    int left = n_ctas, begin = 0;
    double left_bytes = total;
    for (int i = 0; i < njobs; ++i) {
        GemvJob& j = p.job[i];
        const double b = bytes_of(j);
        int c = (i == njobs - 1) ? left : (int)(left * b / left_bytes + 0.5);
        c = std::max(1, std::min(c, left - (njobs - 1 - i)));
        c = std::min(c, (j.N + 15) / 16);
        j.cta_begin = begin;
        j.cta_count = c;
        begin += c;
        left -= c;
        left_bytes -= b;
    }
    L.grid = begin;
    int tile_bytes = 0, acc_floats = 0;
    const int force_kg = env_int("PTB_GEMV_KG", 0);
    for (int i = 0; i < njobs; ++i) {
        GemvJob& j = p.job[i];
        const int pairs = j.w2 ? 2 : 1;
        const int ntile = (j.N + 15) / 16;
        const int tiles_cta = (ntile + j.cta_count - 1) / j.cta_count;
        // K-groups: minimise the per-warp critical path, counted in block visits (+1 per item for its reduction)
        double best = 1e30;
        int bestKG = 1;
        for (int kg = 1; kg <= j.nblk; ++kg) {
            const int rounds = (tiles_cta * kg + warps - 1) / warps;
            const double cost = rounds * ((double)((j.nblk + kg - 1) / kg) * pairs + 1.0) + (kg > 1 ? 0.5 : 0.0);
            if (cost < best - 1e-9) { best = cost; bestKG = kg; }
        }
        if (force_kg > 0) bestKG = std::min(force_kg, j.nblk);
        j.KS = bestKG;
        j.seg_base = j.nblk / bestKG;
        j.seg_rem = j.nblk % bestKG;
        j.RW = 16;
        tile_bytes = std::max(tile_bytes, pairs * t16_block_bytes(j.qtype));
        if (bestKG > 1) acc_floats = std::max(acc_floats, tiles_cta * bestKG * pairs * 16);
    }
    tile_bytes = (tile_bytes + 127) / 128 * 128;
    // ring depth: measured on B200 (Qwen3-4B shape), rings of two or three slots per warp (budgets of 48 to 160 KB) decode
    // 1.4 % faster than the deepest rings that fit (184 to 200 KB per CTA), so the default budget is 128 KB
    const size_t budget = (size_t)env_int("PTB_GEMV_SMEM_KB", warps >= 16 ? 128 : 100) * 1024;
    int stages = std::min(env_int("PTB_GEMV_STAGES", 8), 16);
    while (stages > 2 && gemv_smem_layout(K, warps, stages, tile_bytes, acc_floats).total > budget) --stages;
    p.stages = stages;
    p.tile_bytes = tile_bytes;
    p.acc_floats = acc_floats;
    L.smem = gemv_smem_layout(K, warps, stages, tile_bytes, acc_floats).total;
    L.t16 = 1;
    // wide tiles (paired Q8_0) do not fit sixteen rings of two slots: plan again with eight warps
    if (L.smem > g_gemv_max_dyn && warps == 16) return plan_gemv16(L, njobs, K, n_ctas, 8);
    if (L.smem > g_gemv_max_dyn) {
        ptb_set_error("gemv: %zu B of shared memory needed (K=%d, tile %d B x %d stages x %d warps, %d accumulators)", L.smem, K,
                      tile_bytes, stages, warps, acc_floats);
        return -1;
    }
    return 0;
}

static int plan_gemv(GemvLaunch& L, int njobs, int K, int n_ctas);

static void set_job(GemvJob& j, const PtbWeightDesc& w, const PtbWeightDesc* w2, float* out) {
    memset(&j, 0, sizeof(j));
    g_job_layout = w.layout;
    j.w = (const uint8_t*)w.w;
    j.w2 = w2 ? (const uint8_t*)w2->w : nullptr;
    j.bias = (const float*)w.bias;
    j.out = out;
    j.qtype = w.qtype;
    j.N = w.rows;
    j.nblk = w.cols / (w.layout == 1 ? t16_block_vals(w.qtype) : 256);
    j.KS = (j.nblk + GEMV_SEG_BLOCKS - 1) / GEMV_SEG_BLOCKS;
    j.seg_base = j.nblk / j.KS;
    j.seg_rem = j.nblk % j.KS;
}

static int plan_gemv(GemvLaunch& L, int njobs, int K, int n_ctas) {
    for (int i = 0; i < njobs; ++i) {
        const int q = L.p.job[i].qtype;
        const bool ok = q == QT_Q4K || q == QT_Q6K || (g_job_layout == 1 && (q == QT_Q5K || q == QT_Q8_0 || q == QT_F16));
        if (!ok) {
            ptb_set_error("gemv: weight type %d is not available in layout %d (Q5_K, Q8_0 and fp16 need the 16-row tile layout)", q, g_job_layout);
            return -1;
        }
    }
    return g_job_layout == 1 ? plan_gemv16(L, njobs, K, n_ctas) : plan_gemv_seg(L, njobs, K, n_ctas);
}

// Bytes of one matrix in the streaming layout.
static size_t job_bytes(const GemvJob& j) {
    if (j.RW == 16) return (size_t)((j.N + 15) / 16) * j.nblk * t16_block_bytes(j.qtype);
    size_t b = 0;
    for (int s = 0; s < j.KS; ++s) b += (size_t)j.N * seg_bytes(j.qtype, j.seg_base + (s < j.seg_rem ? 1 : 0));
    return b;
}

// Make launch `a` prefetch (into L2) the weights launch `b` is going to stream, up to `cap` bytes.
static void set_prefetch(GemvLaunch& a, const GemvLaunch& b, size_t cap) {
    int r = 0;
    for (int i = 0; i < b.p.njobs && r < 4; ++i) {
        const GemvJob& j = b.p.job[i];
        const uint8_t* ptrs[2] = {j.w, j.w2};
        for (int k = 0; k < 2 && r < 4; ++k) {
            if (!ptrs[k] || cap < 16) continue;
            const size_t n = std::min(job_bytes(j), cap) & ~(size_t)15;
            a.p.pf_ptr[r] = ptrs[k];
            a.p.pf_bytes[r] = (unsigned)n;
            cap -= n;
            ++r;
        }
    }
}

static bool g_attr_done = false;
static int ensure_attrs() {
    if (g_attr_done) return 0;
    // 227 KB per CTA is shared between the kernel's static and dynamic shared memory
    cudaFuncAttributes fa;
    PTB_CUDA_OK(cudaFuncGetAttributes(&fa, (gemv_kernel<8, 0>)));
    int optin = 0, dev = 0;
    PTB_CUDA_OK(cudaGetDevice(&dev));
    PTB_CUDA_OK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    g_gemv_max_dyn = (size_t)optin - fa.sharedSizeBytes;
    const int dyn = (int)g_gemv_max_dyn;
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv_kernel<8, 0>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv_kernel<16, 0>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv16_kernel<8, 0>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv16_kernel<16, 0>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv_kernel<8, 1>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv_kernel<16, 1>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv16_kernel<8, 1>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv16_kernel<16, 1>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv_kernel<8, 2>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv_kernel<16, 2>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv16_kernel<8, 2>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute((gemv16_kernel<16, 2>), cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    g_attr_done = true;
    return 0;
}

template <typename Kern, typename Params>
static cudaError_t launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, const Params& p) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int G, int D>
static cudaError_t launch_attn_gd(const AttnParams& a, int n_kv_heads, cudaStream_t st, bool pdl) {
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<G, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(AttnShared<D>));
        if (e != cudaSuccess) return e;
        attr_done = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(n_kv_heads * ATT_CLUSTER);
    cfg.blockDim = dim3(ATT_THREADS);
    cfg.dynamicSmemBytes = sizeof(AttnShared<D>);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ATT_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, attn_decode_kernel<G, D>, a);
}
template <int D>
static cudaError_t launch_attn_d(const AttnParams& a, int n_kv_heads, cudaStream_t st, bool pdl) {
    switch (a.group) {
        case 1: return launch_attn_gd<1, D>(a, n_kv_heads, st, pdl);
        case 2: return launch_attn_gd<2, D>(a, n_kv_heads, st, pdl);
        case 4: return launch_attn_gd<4, D>(a, n_kv_heads, st, pdl);
        case 8: return launch_attn_gd<8, D>(a, n_kv_heads, st, pdl);
        default: return cudaErrorInvalidValue;
    }
}
static bool attn_head_dim_ok(int d) { return d == 64 || d == 128 || d == 256; }
static cudaError_t launch_attn(const AttnParams& a, int n_kv_heads, cudaStream_t st, bool pdl) {
    switch (a.head_dim) {
        case 64: return launch_attn_d<64>(a, n_kv_heads, st, pdl);
        case 128: return launch_attn_d<128>(a, n_kv_heads, st, pdl);
        case 256: return launch_attn_d<256>(a, n_kv_heads, st, pdl);
        default: return cudaErrorInvalidValue;
    }
}

// Which instantiation serves a launch: 1 (lean) if it uses none of the slot hand-over, the input records or the L2
// prefetch; 2 if its input comes as records and nothing else is needed; 0 otherwise.
static int gemv_mode(const GemvParams& p) {
    static const int on = env_int("PTB_GEMV_LEAN", 1);
    if (!on) return 0;
    for (int i = 0; i < 4; ++i)
        if (p.pf_bytes[i]) return 0;
    if (p.rec && !p.post_w && !p.post_src) return 2;
    if (p.x_ll || p.part_ll || p.rec || p.x_out_ll) return 0;
    for (int i = 0; i < p.njobs; ++i)
        if (p.job[i].out_ll) return 0;
    return 1;
}
#define PTB_GEMV_DISPATCH(KERN, W, THREADS)                                                                              \
    (mode == 1   ? launch_pdl(KERN<W, 1>, dim3(L.grid), dim3(THREADS), L.smem, st, pdl, L.p)                             \
     : mode == 2 ? launch_pdl(KERN<W, 2>, dim3(L.grid), dim3(THREADS), L.smem, st, pdl, L.p)                             \
                 : launch_pdl(KERN<W, 0>, dim3(L.grid), dim3(THREADS), L.smem, st, pdl, L.p))
static cudaError_t launch_gemv(const GemvLaunch& L, cudaStream_t st, bool pdl) {
    const int mode = gemv_mode(L.p);
    if (L.t16) return L.p.warps == 16 ? PTB_GEMV_DISPATCH(gemv16_kernel, 16, 512) : PTB_GEMV_DISPATCH(gemv16_kernel, 8, 256);
    return L.p.warps == 16 ? PTB_GEMV_DISPATCH(gemv_kernel, 16, 512) : PTB_GEMV_DISPATCH(gemv_kernel, 8, 256);
}
#undef PTB_GEMV_DISPATCH

// ------------------------------------------------------------------------------------------ standalone op entry points (tests, benches)

// y = epilogue(W x).  Device pointers; w2/norm_w/resid/bias may be null.
PTB_API int ptb_gemv(const void* w, const void* w2, int qtype, int rows, int cols, int rowbytes, int layout, const float* x,
                     const float* norm_w, float eps, const float* bias, const float* resid, float* out, int epilogue,
                     int act_gelu, int n_ctas, void* scratch /* >= 16 + 8*n_ctas bytes, zeroed */, int* status,
                     cudaStream_t stream) {
    if (ensure_attrs()) return -1;
    GemvLaunch L;
    memset(&L, 0, sizeof(L));
    PtbWeightDesc d{w, bias, qtype, rows, cols, rowbytes, layout, 0};
    PtbWeightDesc d2{w2, nullptr, qtype, rows, cols, rowbytes, layout, 0};
    set_job(L.p.job[0], d, w2 ? &d2 : nullptr, out);
    L.p.x = x;
    L.p.norm_w = norm_w;
    L.p.eps = eps;
    L.p.epilogue = epilogue;
    L.p.act_gelu = act_gelu;
    L.p.resid = resid;
    L.p.status = status;
    L.p.peers.world = 1;
    if (epilogue == EPI_ARGMAX) {
        uint8_t* s = (uint8_t*)scratch;
        L.p.ticket = (unsigned*)s;
        L.p.result = (int*)(s + 8);
        L.p.ctrl = nullptr;
        L.p.amax_val = (float*)(s + 64);
        L.p.amax_idx = (int*)(s + 64 + 4 * (size_t)n_ctas);
        L.p.logits = out;
    }
    if (plan_gemv(L, 1, cols, n_ctas)) return -1;
    if (getenv("PTB_GEMV_TRACE") && epilogue != EPI_ARGMAX) L.p.trace = (unsigned long long*)scratch;
    PTB_CUDA_OK(launch_gemv(L, stream, false));
    return 0;
}

PTB_API int ptb_attn_decode(const float* q, const float* k, const float* v, const float* q_norm, const float* k_norm,
                            const float* cos, const float* sin, void* k_cache, void* v_cache, float* out, float* part_o,
                            float* part_ml, unsigned* ticket, const int* ctrl, int n_kv_heads, int group, int head_dim,
                            int max_seq, int neox, float eps, int window, cudaStream_t stream) {
    if (!attn_head_dim_ok(head_dim)) {
        ptb_set_error("attn_decode: head size %d; supported: 64, 128, 256", head_dim);
        return -1;
    }
    if (!(group == 1 || group == 2 || group == 4 || group == 8)) {
        ptb_set_error("attn_decode: %d query heads per KV head; supported: 1, 2, 4, %d", group, ATT_MAX_GROUP);
        return -1;
    }
    AttnParams a;
    memset(&a, 0, sizeof(a));
    a.q = q; a.k = k; a.v = v; a.q_norm = q_norm; a.k_norm = k_norm; a.cos = cos; a.sin = sin;
    a.k_cache = (__half*)k_cache; a.v_cache = (__half*)v_cache; a.out = out; a.part_o = part_o; a.part_ml = part_ml;
    a.ticket = ticket; a.ctrl = ctrl; a.group = group; a.max_seq = max_seq;
    a.max_splits = (max_seq + ATT_CHUNK - 1) / ATT_CHUNK;
    a.head_dim = head_dim;
    a.neox = neox; a.eps = eps; a.scale = 1.0f / sqrtf((float)head_dim); a.window = window;
    PTB_CUDA_OK(launch_attn(a, n_kv_heads, stream, false));
    return 0;
}

// ------------------------------------------------------------------------------------------ engine

struct Engine {
    PtbModelDesc m;
    std::vector<PtbLayerDesc> layers;
    int dev = 0, n_sm = 148;
    bool external = false;      // tensor-parallel sums are done by the caller between launch ranges (the NCCL arm)
    cudaStream_t stream = nullptr;
    bool own_stream = true;
    // device buffers
    float *x = nullptr, *qkv = nullptr, *att = nullptr, *ffn = nullptr, *logits = nullptr;
    float *x2 = nullptr, *tmp = nullptr;      // post-norm architectures: second residual buffer, raw projection output
    float* x_final = nullptr;                 // where the residual stream ends up after the last layer
    __half *kc = nullptr, *vc = nullptr;
    float *part_o = nullptr, *part_ml = nullptr;
    unsigned* tickets = nullptr;      // [0] gemv, [1] spare, [8..] attention per kv head
    float* amax_val = nullptr;
    int* amax_idx = nullptr;
    int* ctrl = nullptr;              // CTRL_WORDS ints
    int* result = nullptr;            // {token, value bits}
    int* token_log = nullptr;
    int* script = nullptr;            // prompt tokens for scripted feeding [max_seq]
    int log_cap = 0;
    int* status = nullptr;
    int* h_pinned = nullptr;          // pinned host staging: ctrl words + result
    std::vector<GemvLaunch> gemvs;    // per layer: qkv, o, gateup, down ; last: lm_head
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    bool use_pdl = true;
    unsigned long long* trace = nullptr;   // PTB_TRACE=1: [kernels per token][8] phase stamps of the last token
    long launches_per_token = 0;
    // dataflow buffers of {value, sequence} slots
    uint2* x_ll[2] = {nullptr, nullptr};      // residual stream, ping-pong
    uint2 *qkv_ll = nullptr, *att_ll = nullptr, *ffn_ll = nullptr;
    uint2* own_inbox[2] = {nullptr, nullptr}; // world size 1: the partial-sum inboxes live here (else in symmetric memory)
    uint4* rec[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};   // quantised-input records of qkv, o, gate/up, down, lm_head
    unsigned long long wait_ns = 2000000000ull;
    bool dataflow = false;
};

static int engine_alloc(Engine* e) {
    const PtbModelDesc& m = e->m;
    const int qd = m.n_heads * m.head_dim, kvd = m.n_kv_heads * m.head_dim;
    const int splits = (m.max_seq + ATT_CHUNK - 1) / ATT_CHUNK;
    const int group = m.n_heads / m.n_kv_heads;
    PTB_CUDA_OK(cudaMalloc(&e->x, sizeof(float) * m.hidden));
    PTB_CUDA_OK(cudaMalloc(&e->x2, sizeof(float) * m.hidden));
    PTB_CUDA_OK(cudaMalloc(&e->tmp, sizeof(float) * m.hidden));
    PTB_CUDA_OK(cudaMalloc(&e->qkv, sizeof(float) * (qd + 2 * kvd)));
    PTB_CUDA_OK(cudaMalloc(&e->att, sizeof(float) * qd));
    PTB_CUDA_OK(cudaMalloc(&e->ffn, sizeof(float) * m.inter));
    PTB_CUDA_OK(cudaMalloc(&e->logits, sizeof(float) * m.lm_head.rows));
    const size_t kvbytes = sizeof(__half) * (size_t)m.n_layers * m.n_kv_heads * m.max_seq * m.head_dim;
    PTB_CUDA_OK(cudaMalloc(&e->kc, kvbytes));
    PTB_CUDA_OK(cudaMalloc(&e->vc, kvbytes));
    PTB_CUDA_OK(cudaMemset(e->kc, 0, kvbytes));
    PTB_CUDA_OK(cudaMemset(e->vc, 0, kvbytes));
    PTB_CUDA_OK(cudaMalloc(&e->part_o, sizeof(float) * (size_t)m.n_kv_heads * splits * group * m.head_dim));
    PTB_CUDA_OK(cudaMalloc(&e->part_ml, sizeof(float) * (size_t)m.n_kv_heads * splits * group * 2));
    PTB_CUDA_OK(cudaMalloc(&e->tickets, sizeof(unsigned) * (8 + m.n_kv_heads)));
    PTB_CUDA_OK(cudaMemset(e->tickets, 0, sizeof(unsigned) * (8 + m.n_kv_heads)));
    PTB_CUDA_OK(cudaMalloc(&e->amax_val, sizeof(float) * 4096));
    PTB_CUDA_OK(cudaMalloc(&e->amax_idx, sizeof(int) * 4096));
    PTB_CUDA_OK(cudaMalloc(&e->ctrl, sizeof(int) * CTRL_WORDS));
    {
        int c[CTRL_WORDS] = {0};
        c[CTRL_GEN] = 1;              // sequence numbers start above the zero the slot buffers are cleared to
        PTB_CUDA_OK(cudaMemcpy(e->ctrl, c, sizeof(c), cudaMemcpyHostToDevice));
    }
    auto ll_alloc = [](uint2** p, size_t n) {
        return cudaMalloc(p, n * sizeof(uint2)) != cudaSuccess || cudaMemset(*p, 0, n * sizeof(uint2)) != cudaSuccess;
    };
    if (ll_alloc(&e->x_ll[0], m.hidden) || ll_alloc(&e->x_ll[1], m.hidden) || ll_alloc(&e->qkv_ll, qd + 2 * kvd) ||
        ll_alloc(&e->att_ll, qd) || ll_alloc(&e->ffn_ll, m.inter)) {
        ptb_set_error("decode engine: slot buffer allocation failed");
        return -1;
    }
    if (m.tp_world <= 1 && (ll_alloc(&e->own_inbox[0], m.hidden) || ll_alloc(&e->own_inbox[1], m.hidden))) {
        ptb_set_error("decode engine: inbox allocation failed");
        return -1;
    }
    e->wait_ns = (unsigned long long)env_int("PTB_WAIT_MS", 2000) * 1000000ull;
    if (env_int("PTB_RECORDS", 1)) {
        const int klen[5] = {m.hidden, qd, m.hidden, m.inter, m.hidden};
        for (int i = 0; i < 5; ++i) {
            const size_t bytes = (size_t)(klen[i] / 32) * 64;
            if (cudaMalloc(&e->rec[i], bytes) != cudaSuccess || cudaMemset(e->rec[i], 0, bytes) != cudaSuccess) {
                ptb_set_error("decode engine: record buffer allocation failed");
                return -1;
            }
        }
    }
    PTB_CUDA_OK(cudaMalloc(&e->result, sizeof(int) * 4));
    PTB_CUDA_OK(cudaMemset(e->result, 0, sizeof(int) * 4));
    e->log_cap = 1 << 16;
    PTB_CUDA_OK(cudaMalloc(&e->token_log, sizeof(int) * e->log_cap));
    PTB_CUDA_OK(cudaMalloc(&e->script, sizeof(int) * m.max_seq));
    PTB_CUDA_OK(cudaMalloc(&e->status, sizeof(int)));
    PTB_CUDA_OK(cudaMemset(e->status, 0, sizeof(int)));
    if (2 * m.n_layers + 2 >= (int)LL_SEQ_MUL) {
        ptb_set_error("decode engine: %d layers exceed the %u writes per token a sequence number can index", m.n_layers, LL_SEQ_MUL);
        return -1;
    }
    if (env_int("PTB_TRACE", 0)) {
        PTB_CUDA_OK(cudaMalloc(&e->trace, 8 * sizeof(unsigned long long) * (5 * m.n_layers + 4)));
        PTB_CUDA_OK(cudaMemset(e->trace, 0, 8 * sizeof(unsigned long long) * (5 * m.n_layers + 4)));
    }
    PTB_CUDA_OK(cudaMallocHost(&e->h_pinned, sizeof(int) * 16));
    memset(e->h_pinned, 0, sizeof(int) * 16);
    return 0;
}

// Where the partial sums of projection `which` (0: attention output, 1: FFN down; 2: the arg-max pair) go.
static void fill_peers(const Engine* e, GemvParams& p, int which) {
    const PtbModelDesc& m = e->m;
    p.peers.rank = m.tp_world > 1 ? m.tp_rank : 0;
    p.peers.world = std::max(1, m.tp_world);
    if (m.tp_world > 1) {
        p.peers.slot_elems = m.slot_elems;
        for (int r = 0; r < m.tp_world; ++r) p.peers.inbox[r] = (uint2*)m.peer_inbox[which][r];
    } else {
        p.peers.slot_elems = m.hidden;
        p.peers.inbox[0] = which < 2 ? e->own_inbox[which] : nullptr;
    }
    p.gen = (const uint32_t*)(e->ctrl + CTRL_GEN);
}

// Plain flow: every kernel waits for its predecessor at the launch boundary and the vectors between them are ordinary
// fp32 arrays; the residual stream is updated in place by the projections' epilogues.  Under tensor parallelism the
// K-split projections push their partial sums to every rank and reduce them before they exit (producer-side all-reduce).
static int engine_plan_plain(Engine* e) {
    const PtbModelDesc& m = e->m;
    const int qd = m.n_heads * m.head_dim, kvd = m.n_kv_heads * m.head_dim;
    const int n_ctas = e->n_sm * env_int("PTB_GEMV_CTAS_PER_SM", e->layers[0].q.layout == 1 ? 1 : 2);
    const bool ext = e->external;                // partial sums are all-reduced by the caller, in place, in the residual buffer
    const bool tp = m.tp_world > 1 && !ext;
    // external sums: rank 0 adds the residual to its partial sums, the others store theirs, and the caller's all-reduce
    // over the residual buffer then leaves x + sum of partials on every rank
    const int ext_epi = m.tp_rank == 0 ? EPI_RESID : EPI_STORE;
    e->gemvs.clear();
    if (ext && (e->layers[0].post_attn_norm || e->layers[0].post_ffn_norm)) {
        ptb_set_error("external all-reduce flow: post-norm architectures are not supported");
        return -1;
    }
    // post-norm architectures: a projection stores its raw output in `tmp`; the next kernel's prologue adds
    // RMSNorm(tmp) to the residual stream, reading X[cur] and (CTA 0) writing X[cur ^ 1]
    float* X[2] = {e->x, e->x2};
    int cur = 0;
    const float* pending_w = nullptr;          // post-norm weight of the projection whose output waits in `tmp`
    bool bad = false;
    auto take_pending = [&](GemvParams& p) {
        p.x = X[cur];
        if (pending_w) {
            if (m.hidden > 4096) { ptb_set_error("post-norm architectures: hidden size %d above 4096 is not supported", m.hidden); bad = true; }
            p.post_src = e->tmp; p.post_w = pending_w; p.x_out = X[cur ^ 1];
            cur ^= 1;
            pending_w = nullptr;
        }
    };
    for (int l = 0; l < m.n_layers; ++l) {
        const PtbLayerDesc& L = e->layers[l];
        {   // q, k, v from RMSNorm(x)
            GemvLaunch g;
            memset(&g, 0, sizeof(g));
            set_job(g.p.job[0], L.q, nullptr, e->qkv);
            set_job(g.p.job[1], L.k, nullptr, e->qkv + qd);
            set_job(g.p.job[2], L.v, nullptr, e->qkv + qd + kvd);
            take_pending(g.p);
            g.p.norm_w = L.attn_norm; g.p.eps = m.eps; g.p.norm_add_one = m.norm_add_one;
            g.p.epilogue = EPI_STORE; g.p.status = e->status; g.p.peers.world = 1;
            if (plan_gemv(g, 3, m.hidden, n_ctas)) return -1;
            e->gemvs.push_back(g);
        }
        {   // x += Wo att   (post-norm: tmp = Wo att, added by the next prologue)
            GemvLaunch g;
            memset(&g, 0, sizeof(g));
            const bool post = L.post_attn_norm != nullptr;
            set_job(g.p.job[0], L.o, nullptr, post ? e->tmp : X[cur]);
            g.p.x = e->att; g.p.resid = post ? nullptr : X[cur]; g.p.status = e->status; g.p.ticket = e->tickets;
            g.p.epilogue = tp ? EPI_ALLREDUCE : ext ? ext_epi : (post ? EPI_STORE : EPI_RESID);
            g.p.peers.world = 1;
            if (tp) { fill_peers(e, g.p, 0); g.p.out_seq_add = (uint32_t)(l + 1); }
            if (plan_gemv(g, 1, L.o.cols, n_ctas)) return -1;
            e->gemvs.push_back(g);
            if (post) pending_w = L.post_attn_norm;
        }
        {   // ffn = act(Wg h) * (Wu h), h = RMSNorm(x)
            GemvLaunch g;
            memset(&g, 0, sizeof(g));
            set_job(g.p.job[0], L.gate, &L.up, e->ffn);
            take_pending(g.p);
            g.p.norm_w = L.ffn_norm; g.p.eps = m.eps; g.p.norm_add_one = m.norm_add_one;
            g.p.epilogue = EPI_GATED; g.p.act_gelu = m.act_gelu; g.p.status = e->status; g.p.peers.world = 1;
            if (plan_gemv(g, 1, m.hidden, n_ctas)) return -1;
            e->gemvs.push_back(g);
        }
        {   // x += Wd ffn
            GemvLaunch g;
            memset(&g, 0, sizeof(g));
            const bool post = L.post_ffn_norm != nullptr;
            set_job(g.p.job[0], L.down, nullptr, post ? e->tmp : X[cur]);
            g.p.x = e->ffn; g.p.resid = post ? nullptr : X[cur]; g.p.status = e->status; g.p.ticket = e->tickets;
            g.p.epilogue = tp ? EPI_ALLREDUCE : ext ? ext_epi : (post ? EPI_STORE : EPI_RESID);
            g.p.peers.world = 1;
            if (tp) { fill_peers(e, g.p, 1); g.p.out_seq_add = (uint32_t)(l + 1); }
            if (plan_gemv(g, 1, L.down.cols, n_ctas)) return -1;
            e->gemvs.push_back(g);
            if (post) pending_w = L.post_ffn_norm;
        }
    }
    {   // lm_head with fused arg-max
        GemvLaunch g;
        memset(&g, 0, sizeof(g));
        set_job(g.p.job[0], m.lm_head, nullptr, e->logits);
        take_pending(g.p);
        if (bad) return -1;
        e->x_final = X[cur];
        g.p.norm_w = m.out_norm; g.p.eps = m.eps; g.p.norm_add_one = m.norm_add_one;
        g.p.epilogue = EPI_ARGMAX; g.p.status = e->status;
        g.p.amax_val = e->amax_val; g.p.amax_idx = e->amax_idx; g.p.ticket = e->tickets + 1;
        g.p.logits = m.want_logits ? e->logits : nullptr;
        g.p.result = e->result; g.p.ctrl = e->ctrl; g.p.token_log = e->token_log; g.p.token_script = e->script; g.p.row_offset = m.vocab_offset;
        g.p.peers.world = 1;
        g.p.gen = (const uint32_t*)(e->ctrl + CTRL_GEN);
        if (ext) { g.p.ctrl = nullptr; g.p.token_log = nullptr; }      // this rank's {id, value} only; ptb_engine_finish_token ends the token
        if (tp) { fill_peers(e, g.p, 2); g.p.out_seq_add = 1; }
        if (plan_gemv(g, 1, m.hidden, std::min(n_ctas, 4096))) return -1;
        e->gemvs.push_back(g);
    }
    return 0;
}


// Dataflow (any number of GPUs).
static int engine_plan_dataflow(Engine* e) {
    const PtbModelDesc& m = e->m;
    const int qd = m.n_heads * m.head_dim, kvd = m.n_kv_heads * m.head_dim;
    const int n_ctas = e->n_sm * env_int("PTB_GEMV_CTAS_PER_SM", e->layers[0].q.layout == 1 ? 1 : 2);
    const bool tp = m.tp_world > 1;
    const int world = std::max(1, m.tp_world);
    const uint32_t* gen = (const uint32_t*)(e->ctrl + CTRL_GEN);
    e->gemvs.clear();
    // The residual stream lives in two slot buffers used in turn.  Update number u (1, 2, ... within a token; the
    // embedding is write 0 into buffer 0) is formed by the prologue of the kernel that consumes it, from buffer
    // (u - 1) & 1 plus the partial sums of the projection before it, and published by that kernel's CTA 0 into
    // buffer u & 1 with sequence index u.
    int upd = 0;
    auto consume_residual = [&](GemvParams& p, int inbox, int layer_seq, const float* post_w) {
        p.x_ll = e->x_ll[upd & 1];
        p.x_seq_add = (uint32_t)upd;
        if (inbox >= 0) {
            p.part_ll = tp ? (const uint2*)m.peer_inbox[inbox][m.tp_rank] : e->own_inbox[inbox];
            p.nparts = world;
            p.part_stride = tp ? m.slot_elems : m.hidden;
            p.part_seq_add = (uint32_t)layer_seq;
            p.post_w = post_w;
            ++upd;
            p.x_out_ll = e->x_ll[upd & 1];
            p.x_out_seq_add = (uint32_t)upd;
        }
    };
    int pending_inbox = -1, pending_seq = 0;       // the projection whose partial sums wait to be folded in
    const float* pending_w = nullptr;              // ... and its post-norm weight (gemma3) or null
    for (int l = 0; l < m.n_layers; ++l) {
        const PtbLayerDesc& L = e->layers[l];
        if ((L.post_attn_norm || L.post_ffn_norm) && m.hidden > 4096) {
            ptb_set_error("post-norm architectures: hidden size %d above 4096 is not supported", m.hidden);
            return -1;
        }
        {   // q, k, v from RMSNorm(x)
            GemvLaunch g;
            memset(&g, 0, sizeof(g));
            set_job(g.p.job[0], L.q, nullptr, nullptr);
            set_job(g.p.job[1], L.k, nullptr, nullptr);
            set_job(g.p.job[2], L.v, nullptr, nullptr);
            g.p.job[0].out_ll = e->qkv_ll; g.p.job[1].out_ll = e->qkv_ll + qd; g.p.job[2].out_ll = e->qkv_ll + qd + kvd;
            consume_residual(g.p, pending_inbox, pending_seq, pending_w);
            g.p.out_seq_add = (uint32_t)(l + 1);
            g.p.norm_w = L.attn_norm; g.p.eps = m.eps; g.p.norm_add_one = m.norm_add_one;
            g.p.epilogue = EPI_STORE; g.p.status = e->status; g.p.peers.world = 1; g.p.gen = gen;
            g.p.rec = e->rec[0];
            if (plan_gemv(g, 3, m.hidden, n_ctas)) return -1;
            e->gemvs.push_back(g);
        }
        {   // partial sums of Wo att -> inbox 0
            GemvLaunch g;
            memset(&g, 0, sizeof(g));
            set_job(g.p.job[0], L.o, nullptr, nullptr);
            g.p.x_ll = e->att_ll; g.p.x_seq_add = (uint32_t)(l + 1);
            g.p.status = e->status;
            g.p.epilogue = EPI_PARTIAL; g.p.out_seq_add = (uint32_t)(l + 1);
            fill_peers(e, g.p, 0);
            g.p.rec = e->rec[1];
            if (plan_gemv(g, 1, L.o.cols, n_ctas)) return -1;
            e->gemvs.push_back(g);
            pending_inbox = 0; pending_seq = l + 1; pending_w = L.post_attn_norm;
        }
        {   // ffn = act(Wg h) * (Wu h), h = RMSNorm(x)
            GemvLaunch g;
            memset(&g, 0, sizeof(g));
            set_job(g.p.job[0], L.gate, &L.up, nullptr);
            g.p.job[0].out_ll = e->ffn_ll;
            consume_residual(g.p, pending_inbox, pending_seq, pending_w);
            g.p.out_seq_add = (uint32_t)(l + 1);
            g.p.norm_w = L.ffn_norm; g.p.eps = m.eps; g.p.norm_add_one = m.norm_add_one;
            g.p.epilogue = EPI_GATED; g.p.act_gelu = m.act_gelu; g.p.status = e->status; g.p.peers.world = 1; g.p.gen = gen;
            g.p.rec = e->rec[2];
            if (plan_gemv(g, 1, m.hidden, n_ctas)) return -1;
            e->gemvs.push_back(g);
        }
        {   // partial sums of Wd ffn -> inbox 1
            GemvLaunch g;
            memset(&g, 0, sizeof(g));
            set_job(g.p.job[0], L.down, nullptr, nullptr);
            g.p.x_ll = e->ffn_ll; g.p.x_seq_add = (uint32_t)(l + 1);
            g.p.status = e->status;
            g.p.epilogue = EPI_PARTIAL; g.p.out_seq_add = (uint32_t)(l + 1);
            fill_peers(e, g.p, 1);
            g.p.rec = e->rec[3];
            if (plan_gemv(g, 1, L.down.cols, n_ctas)) return -1;
            e->gemvs.push_back(g);
            pending_inbox = 1; pending_seq = l + 1; pending_w = L.post_ffn_norm;
        }
    }
    {   // lm_head with fused arg-max
        GemvLaunch g;
        memset(&g, 0, sizeof(g));
        set_job(g.p.job[0], m.lm_head, nullptr, e->logits);
        consume_residual(g.p, pending_inbox, pending_seq, pending_w);
        g.p.x_out = e->x;                   // the final hidden state, also as a plain vector (tests, embeddings)
        e->x_final = e->x;
        g.p.norm_w = m.out_norm; g.p.eps = m.eps; g.p.norm_add_one = m.norm_add_one;
        g.p.epilogue = EPI_ARGMAX; g.p.status = e->status;
        g.p.amax_val = e->amax_val; g.p.amax_idx = e->amax_idx; g.p.ticket = e->tickets + 1;
        g.p.logits = m.want_logits ? e->logits : nullptr;
        g.p.result = e->result; g.p.ctrl = e->ctrl; g.p.token_log = e->token_log; g.p.token_script = e->script; g.p.row_offset = m.vocab_offset;
        g.p.out_seq_add = 1;
        fill_peers(e, g.p, 2);
        if (!tp) g.p.peers.world = 1;
        g.p.rec = e->rec[4];
        if (plan_gemv(g, 1, m.hidden, std::min(n_ctas, 4096))) return -1;
        e->gemvs.push_back(g);
    }
    return 0;
}

static int engine_plan(Engine* e) {
    // PTB_DECODE_FLOW: "plain" (launch-boundary waits; producer-side all-reduce under tensor parallelism) or "dataflow"
    // (slot hand-over, consumer-side all-reduce).  Measured on B200: plain is ahead on 1 and 2 GPUs (758 vs 736 tok/s at 2), level at 4 (841 vs 840) and behind at 8 (787 vs 868), where
    // the per-kernel hand-over latency is all that is left of a step.
    // "external" (tensor parallel only): the plain flow without any in-kernel exchange; the caller enqueues launch ranges
    // and all-reduces the residual buffer between them (ptb_engine_enqueue_range), which is how the NCCL baseline runs.
    const char* f = getenv("PTB_DECODE_FLOW");
    e->external = f && !strcmp(f, "external") && e->m.tp_world > 1;
    e->dataflow = f ? !strcmp(f, "dataflow") : e->m.tp_world >= 4;
    if (e->dataflow ? engine_plan_dataflow(e) : engine_plan_plain(e)) return -1;
    const size_t pf_cap = (size_t)env_int("PTB_PREFETCH_MB", 0) << 20;
    if (pf_cap)
        for (size_t i = 0; i < e->gemvs.size(); ++i) set_prefetch(e->gemvs[i], e->gemvs[(i + 1) % e->gemvs.size()], pf_cap);
    return 0;
}


// Enqueue launches [first, last) of one token's kernels on the engine stream.  Launch 0 is the embedding, launches
// 1 + 5 l .. 5 + 5 l are layer l's {qkv, attention, o, gate/up, down}, the last one is the lm_head.
static int engine_enqueue_range(Engine* e, long first, long last);
static int engine_enqueue(Engine* e) { return engine_enqueue_range(e, 0, 1L << 40); }
static int engine_enqueue_range(Engine* e, long first, long last) {
    const PtbModelDesc& m = e->m;
    const int qd = m.n_heads * m.head_dim, kvd = m.n_kv_heads * m.head_dim;
    const int splits = (m.max_seq + ATT_CHUNK - 1) / ATT_CHUNK;
    const bool pdl = e->use_pdl;
    long n = 0;
    EmbedParams ep;
    memset(&ep, 0, sizeof(ep));
    ep.table = (const uint8_t*)m.embed.w; ep.qtype = m.embed.qtype; ep.rowbytes = m.embed.rowbytes;
    ep.nblk = m.embed.cols / 256; ep.H = m.hidden; ep.scale = m.emb_scale; ep.ctrl = e->ctrl;
    if (e->dataflow) ep.out_ll = e->x_ll[0];
    else ep.out = e->x;
    ep.vocab = m.embed.rows; ep.status = e->status;
    ep.gen = (const uint32_t*)(e->ctrl + CTRL_GEN);
    // the first kernel of a token is launched without the programmatic edge: it must not
    // overlap the previous token's lm_head, whose epilogue updates the control block
    auto want = [&](long idx) { return idx >= first && idx < last; };
    if (want(0)) PTB_CUDA_OK(launch_pdl(embed_kernel, dim3((m.hidden + 255) / 256), dim3(256), 0, e->stream, false, ep));
    ++n;
    size_t gi = 0;
    for (int l = 0; l < m.n_layers; ++l) {
        const PtbLayerDesc& L = e->layers[l];
        GemvLaunch& g0 = e->gemvs[gi++];
        if (e->trace) g0.p.trace = e->trace + 8 * (1 + 5 * l);
        if (want(n)) PTB_CUDA_OK(launch_gemv(g0, e->stream, pdl));
        AttnParams a;
        memset(&a, 0, sizeof(a));
        if (e->dataflow) {
            a.q_ll = e->qkv_ll; a.k_ll = e->qkv_ll + qd; a.v_ll = e->qkv_ll + qd + kvd;
            a.out_ll = e->att_ll; a.in_seq_add = (uint32_t)(l + 1); a.out_seq_add = (uint32_t)(l + 1);
        } else {
            a.q = e->qkv; a.k = e->qkv + qd; a.v = e->qkv + qd + kvd;
            a.out = e->att;
        }
        a.gen = (const uint32_t*)(e->ctrl + CTRL_GEN); a.status = e->status; a.wait_ns = e->wait_ns;
        a.hard_wait = env_int("PTB_DATAFLOW", 1) == 0;
        a.q_norm = L.q_norm; a.k_norm = L.k_norm; a.cos = L.cos; a.sin = L.sin;
        a.k_cache = e->kc + (size_t)l * m.n_kv_heads * m.max_seq * m.head_dim;
        a.v_cache = e->vc + (size_t)l * m.n_kv_heads * m.max_seq * m.head_dim;
        a.out = e->att; a.part_o = e->part_o; a.part_ml = e->part_ml; a.ticket = e->tickets + 8; a.ctrl = e->ctrl;
        a.group = m.n_heads / m.n_kv_heads; a.max_seq = m.max_seq; a.max_splits = splits; a.neox = m.neox;
        a.head_dim = m.head_dim;
        a.eps = m.eps; a.scale = 1.0f / sqrtf((float)m.head_dim); a.window = L.window;
        if (e->trace) a.trace = e->trace + 8 * (2 + 5 * l);
        if (want(n + 1)) PTB_CUDA_OK(launch_attn(a, m.n_kv_heads, e->stream, pdl));
        for (int k = 0; k < 3; ++k) {
            GemvLaunch& g = e->gemvs[gi++];
            if (e->trace) g.p.trace = e->trace + 8 * (3 + k + 5 * l);
            if (want(n + 2 + k)) PTB_CUDA_OK(launch_gemv(g, e->stream, pdl));
        }
        n += 5;
    }
    GemvLaunch& gl = e->gemvs[gi++];
    if (e->trace) gl.p.trace = e->trace + 8 * (1 + 5 * m.n_layers);
    if (want(n)) PTB_CUDA_OK(launch_gemv(gl, e->stream, pdl));
    ++n;
    e->launches_per_token = n;
    return 0;
}

PTB_API void* ptb_engine_create(const PtbModelDesc* m, const PtbLayerDesc* layers, void* ext_stream) {
    if (!attn_head_dim_ok(m->head_dim)) {
        ptb_set_error("decode engine: head size %d not supported (the attention kernel is built for 64, 128 and 256)", m->head_dim);
        return nullptr;
    }
    const int grp_ = m->n_kv_heads ? m->n_heads / m->n_kv_heads : 0;
    if (m->n_heads % m->n_kv_heads || !(grp_ == 1 || grp_ == 2 || grp_ == 4 || grp_ == 8)) {
        ptb_set_error("decode engine: %d query heads over %d KV heads not supported", m->n_heads, m->n_kv_heads);
        return nullptr;
    }
    if (m->hidden % 256 || m->inter % 256) {
        ptb_set_error("decode engine: hidden (%d) and FFN (%d) sizes must be multiples of 256", m->hidden, m->inter);
        return nullptr;
    }
    Engine* e = new Engine();
    e->m = *m;
    e->layers.assign(layers, layers + m->n_layers);
    if (cudaGetDevice(&e->dev) != cudaSuccess) { ptb_set_error("no CUDA device"); delete e; return nullptr; }
    cudaDeviceGetAttribute(&e->n_sm, cudaDevAttrMultiProcessorCount, e->dev);
    e->use_pdl = env_int("PTB_PDL", 1) != 0;
    if (ext_stream) { e->stream = (cudaStream_t)ext_stream; e->own_stream = false; }
    else if (cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess) { ptb_set_error("stream create failed"); delete e; return nullptr; }
    if (ensure_attrs() || engine_alloc(e) || engine_plan(e)) { delete e; return nullptr; }
    return e;
}

PTB_API void ptb_engine_destroy(void* h) {
    Engine* e = (Engine*)h;
    if (!e) return;
    cudaStreamSynchronize(e->stream);
    if (e->exec) cudaGraphExecDestroy(e->exec);
    if (e->graph) cudaGraphDestroy(e->graph);
    cudaFree(e->x2); cudaFree(e->tmp);
    cudaFree(e->x); cudaFree(e->qkv); cudaFree(e->att); cudaFree(e->ffn); cudaFree(e->logits);
    cudaFree(e->kc); cudaFree(e->vc); cudaFree(e->part_o); cudaFree(e->part_ml); cudaFree(e->tickets);
    cudaFree(e->amax_val); cudaFree(e->amax_idx); cudaFree(e->ctrl); cudaFree(e->result); cudaFree(e->token_log); cudaFree(e->script);
    cudaFree(e->status);
    cudaFree(e->x_ll[0]); cudaFree(e->x_ll[1]); cudaFree(e->qkv_ll); cudaFree(e->att_ll); cudaFree(e->ffn_ll);
    cudaFree(e->own_inbox[0]); cudaFree(e->own_inbox[1]);
    for (int i = 0; i < 5; ++i) cudaFree(e->rec[i]);
    cudaFreeHost(e->h_pinned);
    if (e->own_stream) cudaStreamDestroy(e->stream);
    delete e;
}

// Capture one token into a graph (call once, before the first replay).
PTB_API int ptb_engine_capture(void* h) {
    Engine* e = (Engine*)h;
    if (e->exec) return 0;
    if (e->external) {
        ptb_set_error("external all-reduce flow: the caller captures ptb_engine_enqueue_range calls and its own collectives");
        return -1;
    }
    PTB_CUDA_OK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    if (engine_enqueue(e)) {
        cudaGraph_t g = nullptr;
        cudaStreamEndCapture(e->stream, &g);
        if (g) cudaGraphDestroy(g);
        return -1;
    }
    PTB_CUDA_OK(cudaStreamEndCapture(e->stream, &e->graph));
    PTB_CUDA_OK(cudaGraphInstantiate(&e->exec, e->graph, 0));
    return 0;
}

// External all-reduce flow (PTB_DECODE_FLOW=external under tensor parallelism).  A token is
//   enqueue_range(0, 4) | all-reduce x | (2) | all-reduce x | (3) | ... | lm_head | all-gather result | finish_token
// where the residual vector x is ptb_engine_buffer(h, 0) (hidden floats) and this rank's {id, value bits} pair is
// ptb_engine_buffer(h, 1).  Everything is enqueued on the engine stream, so the caller can capture it in a graph.
PTB_API int ptb_engine_enqueue_range(void* h, int first, int count) {
    Engine* e = (Engine*)h;
    if (e->exec) { ptb_set_error("enqueue_range: the engine already owns a captured graph"); return -1; }
    return engine_enqueue_range(e, first, (long)first + count);
}
PTB_API void* ptb_engine_buffer(void* h, int which) {
    Engine* e = (Engine*)h;
    return which == 0 ? (void*)e->x : which == 1 ? (void*)e->result : nullptr;
}
static __global__ void finish_token_kernel(const int* __restrict__ pairs, int world, int* result, int* ctrl, int* token_log,
                                           const int* script) {
    if (threadIdx.x || blockIdx.x) return;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int p = 0; p < world; ++p) {
        const int ix = pairs[2 * p];
        const float v = __int_as_float(pairs[2 * p + 1]);
        if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
    }
    result[0] = bi;
    result[1] = __float_as_int(bv);
    advance_token(ctrl, token_log, script, bi, (uint32_t)ctrl[CTRL_GEN]);
}
// pairs: device array [world][2] of every rank's {id, value bits} (the all-gathered result buffers).
PTB_API int ptb_engine_finish_token(void* h, const void* pairs, int world) {
    Engine* e = (Engine*)h;
    finish_token_kernel<<<1, 32, 0, e->stream>>>((const int*)pairs, world, e->result, e->ctrl, e->token_log, e->script);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// Write {token, pos, self_feed} (and the log cursor) through pinned memory on the engine stream.
PTB_API int ptb_engine_set_ctrl(void* h, int token, int pos, int self_feed, int reset_log) {
    Engine* e = (Engine*)h;
    int* p = e->h_pinned;
    if (reset_log) {
        int gen = 0;
        PTB_CUDA_OK(cudaStreamSynchronize(e->stream));
        PTB_CUDA_OK(cudaMemcpy(&gen, e->ctrl + CTRL_GEN, sizeof(int), cudaMemcpyDeviceToHost));
        p[CTRL_TOKEN] = token; p[CTRL_POS] = pos; p[CTRL_STEP] = 0; p[CTRL_SELF_FEED] = self_feed;
        p[CTRL_LOG_CAP] = e->log_cap; p[CTRL_GEN] = gen; p[6] = 0; p[7] = 0;
        PTB_CUDA_OK(cudaMemcpyAsync(e->ctrl, p, sizeof(int) * CTRL_WORDS, cudaMemcpyHostToDevice, e->stream));
    } else {
        p[CTRL_TOKEN] = token; p[CTRL_POS] = pos;
        PTB_CUDA_OK(cudaMemcpyAsync(e->ctrl, p, sizeof(int) * 2, cudaMemcpyHostToDevice, e->stream));
    }
    return 0;
}

// Enqueue `n` tokens (graph replays if captured, eager launches otherwise).  Asynchronous.
PTB_API int ptb_engine_run(void* h, int n) {
    Engine* e = (Engine*)h;
    for (int i = 0; i < n; ++i) {
        if (e->exec) PTB_CUDA_OK(cudaGraphLaunch(e->exec, e->stream));
        else if (engine_enqueue(e)) return -1;
    }
    return 0;
}

// Host-fed step, the serving loop: copy {token,pos} in from pinned memory, run one token, copy the
// sampled id back to pinned memory, wait.  Returns the id (or -1).
PTB_API int ptb_engine_step(void* h, int token, int pos) {
    Engine* e = (Engine*)h;
    if (ptb_engine_set_ctrl(h, token, pos, 0, 0)) return -1;
    if (ptb_engine_run(h, 1)) return -1;
    PTB_CUDA_OK(cudaMemcpyAsync(e->h_pinned + 8, e->result, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    PTB_CUDA_OK(cudaStreamSynchronize(e->stream));
    return e->h_pinned[8];
}

// Scripted run: feed `n` prompt tokens starting at position pos0, then keep generating from the
// arg-max.  Sets up the control block; follow with ptb_engine_run(h, n + n_new - 1).  log[n-1+i] is
// the i-th generated token.
PTB_API int ptb_engine_begin_script(void* h, const int* tokens, int n, int pos0) {
    Engine* e = (Engine*)h;
    if (n < 1 || pos0 + n > e->m.max_seq) { ptb_set_error("script of %d tokens at %d exceeds max_seq %d", n, pos0, e->m.max_seq); return -1; }
    int gen = 0;
    PTB_CUDA_OK(cudaStreamSynchronize(e->stream));
    PTB_CUDA_OK(cudaMemcpy(&gen, e->ctrl + CTRL_GEN, sizeof(int), cudaMemcpyDeviceToHost));
    PTB_CUDA_OK(cudaMemcpy(e->script, tokens, sizeof(int) * n, cudaMemcpyHostToDevice));
    int c[CTRL_WORDS] = {tokens[0], pos0, 0, 2, e->log_cap, gen, n, 0};
    PTB_CUDA_OK(cudaMemcpy(e->ctrl, c, sizeof(c), cudaMemcpyHostToDevice));
    return 0;
}

PTB_API int ptb_engine_sync(void* h) {
    Engine* e = (Engine*)h;
    PTB_CUDA_OK(cudaStreamSynchronize(e->stream));
    return 0;
}

// Copy the first n logged token ids to host memory; returns how many steps have run since the log reset.
PTB_API int ptb_engine_read_log(void* h, int* out, int n) {
    Engine* e = (Engine*)h;
    PTB_CUDA_OK(cudaStreamSynchronize(e->stream));
    int steps = 0;
    PTB_CUDA_OK(cudaMemcpy(&steps, e->ctrl + CTRL_STEP, sizeof(int), cudaMemcpyDeviceToHost));
    n = std::min(n, std::min(steps, e->log_cap));
    if (n > 0) PTB_CUDA_OK(cudaMemcpy(out, e->token_log, sizeof(int) * n, cudaMemcpyDeviceToHost));
    return steps;
}

PTB_API int ptb_engine_status(void* h) {
    Engine* e = (Engine*)h;
    int s = -1;
    if (cudaMemcpy(&s, e->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return s;
}
// Copy the phase stamps of the last token ([kernels][8] uint64 nanoseconds) to `out`; returns the kernel count.
PTB_API int ptb_engine_read_trace(void* h, unsigned long long* out, int max_kernels) {
    Engine* e = (Engine*)h;
    if (!e->trace) return 0;
    const int n = std::min(max_kernels, 5 * e->m.n_layers + 2);
    PTB_CUDA_OK(cudaStreamSynchronize(e->stream));
    PTB_CUDA_OK(cudaMemcpy(out, e->trace, sizeof(unsigned long long) * 8 * n, cudaMemcpyDeviceToHost));
    return n;
}
PTB_API void* ptb_engine_stream(void* h) { return (void*)((Engine*)h)->stream; }
PTB_API void* ptb_engine_logits(void* h) { return (void*)((Engine*)h)->logits; }
PTB_API void* ptb_engine_hidden(void* h) { Engine* e = (Engine*)h; return (void*)(e->x_final ? e->x_final : e->x); }
PTB_API void* ptb_engine_result(void* h) { return (void*)((Engine*)h)->result; }
// Device addresses of layer `layer`'s fp16 K and V caches, each [kv_heads][max_seq][head_dim].
PTB_API int ptb_engine_kv_cache(void* h, int layer, void** k, void** v) {
    Engine* e = (Engine*)h;
    if (layer < 0 || layer >= e->m.n_layers) { ptb_set_error("layer %d out of range", layer); return -1; }
    const size_t per = (size_t)e->m.n_kv_heads * e->m.max_seq * e->m.head_dim;
    *k = e->kc + per * layer;
    *v = e->vc + per * layer;
    return 0;
}
PTB_API long ptb_engine_launches_per_token(void* h) { return ((Engine*)h)->launches_per_token; }
PTB_API int ptb_engine_kv_bytes(void* h, long* out) {
    Engine* e = (Engine*)h;
    *out = 2L * sizeof(__half) * e->m.n_layers * e->m.n_kv_heads * e->m.max_seq * e->m.head_dim;
    return 0;
}

// Geometry report for one GEMV (tests and notes): rows per tile, stages, grid, smem, tile bytes.
PTB_API int ptb_gemv_plan(int qtype, int rows, int cols, int rowbytes, int layout, int paired, int n_ctas, int* out5) {
    GemvLaunch L;
    memset(&L, 0, sizeof(L));
    PtbWeightDesc d{(const void*)16, nullptr, qtype, rows, cols, rowbytes, layout, 0};
    set_job(L.p.job[0], d, paired ? &d : nullptr, nullptr);
    if (plan_gemv(L, 1, cols, n_ctas)) return -1;
    out5[0] = L.p.job[0].RW; out5[1] = L.p.stages; out5[2] = L.grid; out5[3] = (int)L.smem; out5[4] = L.p.tile_bytes;
    return 0;
}
