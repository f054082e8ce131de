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
#include "decode_kernels.cuh"
#include "decode_mega.cuh"
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
};

// Fill job geometry, CTA split, tile ring and shared memory size.  `jobs` already carry
// w/w2/out/bias/qtype/N/nblk/KS/seg_base/seg_rem.
static int plan_gemv(GemvLaunch& L, int njobs, int K, int n_ctas) {
    const int want_stages = env_int("PTB_GEMV_STAGES", 4);
    const int tile_cap = env_int("PTB_GEMV_TILE_KB", 6) * 1024;
    const size_t budget = (size_t)env_int("PTB_GEMV_SMEM_KB", 100) * 1024;
    GemvParams& p = L.p;
    p.njobs = njobs;
    p.K = K;
    const int warps = env_int("PTB_GEMV_WARPS", 8) >= 16 ? 16 : 8;
    p.warps = warps;
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

static void set_job(GemvJob& j, const PtbWeightDesc& w, const PtbWeightDesc* w2, float* out) {
    memset(&j, 0, sizeof(j));
    j.w = (const uint8_t*)w.w;
    j.w2 = w2 ? (const uint8_t*)w2->w : nullptr;
    j.bias = (const float*)w.bias;
    j.out = out;
    j.qtype = w.qtype;
    j.N = w.rows;
    j.nblk = w.cols / 256;
    j.KS = (j.nblk + GEMV_SEG_BLOCKS - 1) / GEMV_SEG_BLOCKS;
    j.seg_base = j.nblk / j.KS;
    j.seg_rem = j.nblk % j.KS;
}

static bool g_attr_done = false;
static int ensure_attrs() {
    if (g_attr_done) return 0;
    // 227 KB per CTA is shared between the kernel's static and dynamic shared memory
    cudaFuncAttributes fa;
    PTB_CUDA_OK(cudaFuncGetAttributes(&fa, gemv_kernel<8>));
    int optin = 0, dev = 0;
    PTB_CUDA_OK(cudaGetDevice(&dev));
    PTB_CUDA_OK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    g_gemv_max_dyn = (size_t)optin - fa.sharedSizeBytes;
    PTB_CUDA_OK(cudaFuncSetAttribute(gemv_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_gemv_max_dyn));
    PTB_CUDA_OK(cudaFuncSetAttribute(gemv_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g_gemv_max_dyn));
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

template <int G>
static cudaError_t launch_attn_g(const AttnParams& a, int n_kv_heads, cudaStream_t st, bool pdl) {
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(AttnShared));
        if (e != cudaSuccess) return e;
        attr_done = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(n_kv_heads * ATT_CLUSTER);
    cfg.blockDim = dim3(ATT_THREADS);
    cfg.dynamicSmemBytes = sizeof(AttnShared);
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
    return cudaLaunchKernelEx(&cfg, attn_decode_kernel<G>, a);
}
static cudaError_t launch_attn(const AttnParams& a, int n_kv_heads, cudaStream_t st, bool pdl) {
    switch (a.group) {
        case 1: return launch_attn_g<1>(a, n_kv_heads, st, pdl);
        case 2: return launch_attn_g<2>(a, n_kv_heads, st, pdl);
        case 4: return launch_attn_g<4>(a, n_kv_heads, st, pdl);
        case 8: return launch_attn_g<8>(a, n_kv_heads, st, pdl);
        default: return cudaErrorInvalidValue;
    }
}

static cudaError_t launch_gemv(const GemvLaunch& L, cudaStream_t st, bool pdl) {
    if (L.p.warps == 16) return launch_pdl(gemv_kernel<16>, dim3(L.grid), dim3(512), L.smem, st, pdl, L.p);
    return launch_pdl(gemv_kernel<8>, dim3(L.grid), dim3(256), L.smem, st, pdl, L.p);
}

// ------------------------------------------------------------------------------------------ standalone op entry points (tests, benches)

// y = epilogue(W x).  Device pointers; w2/norm_w/resid/bias may be null.
PTB_API int ptb_gemv(const void* w, const void* w2, int qtype, int rows, int cols, int rowbytes, const float* x,
                     const float* norm_w, float eps, const float* bias, const float* resid, float* out, int epilogue,
                     int act_gelu, int n_ctas, void* scratch /* >= 16 + 8*n_ctas bytes, zeroed */, int* status,
                     cudaStream_t stream) {
    if (ensure_attrs()) return -1;
    GemvLaunch L;
    memset(&L, 0, sizeof(L));
    PtbWeightDesc d{w, bias, qtype, rows, cols, rowbytes};
    PtbWeightDesc d2{w2, nullptr, qtype, rows, cols, rowbytes};
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
                            float* part_ml, unsigned* ticket, const int* ctrl, int n_kv_heads, int group, int max_seq,
                            int neox, float eps, int window, cudaStream_t stream) {
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
    a.neox = neox; a.eps = eps; a.scale = 1.0f / sqrtf((float)ATT_D); a.window = window;
    PTB_CUDA_OK(launch_attn(a, n_kv_heads, stream, false));
    return 0;
}

// ------------------------------------------------------------------------------------------ engine

struct Engine {
    PtbModelDesc m;
    std::vector<PtbLayerDesc> layers;
    int dev = 0, n_sm = 148;
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
    // persistent single-launch path (one GPU): op list on the device, arrival counter, launch geometry
    bool mega = false;
    MegaParams mp;
    MegaOp* d_ops = nullptr;
    unsigned* d_bar = nullptr;        // [0] spare, [1] token generation
    uint2 *x_ll = nullptr, *qkv_ll = nullptr, *att_ll = nullptr, *ffn_ll = nullptr, *part_o_ll = nullptr, *part_ml_ll = nullptr;
    size_t mega_smem = 0;
    int mega_warps = 15;
    int n_ops = 0;
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
    PTB_CUDA_OK(cudaMalloc(&e->part_o, sizeof(float) * (size_t)m.n_kv_heads * splits * group * ATT_D));
    PTB_CUDA_OK(cudaMalloc(&e->part_ml, sizeof(float) * (size_t)m.n_kv_heads * splits * group * 2));
    PTB_CUDA_OK(cudaMalloc(&e->tickets, sizeof(unsigned) * (8 + m.n_kv_heads)));
    PTB_CUDA_OK(cudaMemset(e->tickets, 0, sizeof(unsigned) * (8 + m.n_kv_heads)));
    PTB_CUDA_OK(cudaMalloc(&e->amax_val, sizeof(float) * 4096));
    PTB_CUDA_OK(cudaMalloc(&e->amax_idx, sizeof(int) * 4096));
    PTB_CUDA_OK(cudaMalloc(&e->ctrl, sizeof(int) * CTRL_WORDS));
    PTB_CUDA_OK(cudaMemset(e->ctrl, 0, sizeof(int) * CTRL_WORDS));
    PTB_CUDA_OK(cudaMalloc(&e->result, sizeof(int) * 4));
    PTB_CUDA_OK(cudaMemset(e->result, 0, sizeof(int) * 4));
    e->log_cap = 1 << 16;
    PTB_CUDA_OK(cudaMalloc(&e->token_log, sizeof(int) * e->log_cap));
    PTB_CUDA_OK(cudaMalloc(&e->script, sizeof(int) * m.max_seq));
    PTB_CUDA_OK(cudaMalloc(&e->status, sizeof(int)));
    PTB_CUDA_OK(cudaMemset(e->status, 0, sizeof(int)));
    if (env_int("PTB_TRACE", 0)) {
        PTB_CUDA_OK(cudaMalloc(&e->trace, 8 * sizeof(unsigned long long) * (5 * m.n_layers + 4)));
        PTB_CUDA_OK(cudaMemset(e->trace, 0, 8 * sizeof(unsigned long long) * (5 * m.n_layers + 4)));
    }
    PTB_CUDA_OK(cudaMallocHost(&e->h_pinned, sizeof(int) * 16));
    memset(e->h_pinned, 0, sizeof(int) * 16);
    return 0;
}

static void fill_peers(const Engine* e, GemvParams& p, int which, int call_idx, int calls_per_token) {
    const PtbModelDesc& m = e->m;
    p.peers.rank = m.tp_rank;
    p.peers.world = m.tp_world;
    p.peers.slot_elems = m.slot_elems;
    for (int r = 0; r < m.tp_world; ++r) p.peers.inbox[r] = (uint2*)m.peer_inbox[which][r];
    p.gen = (const uint32_t*)(e->ctrl + CTRL_GEN);
    p.peers.seq_mul = (uint32_t)calls_per_token;
    p.peers.seq_add = (uint32_t)call_idx;
}

static int engine_plan(Engine* e) {
    const PtbModelDesc& m = e->m;
    const int qd = m.n_heads * m.head_dim, kvd = m.n_kv_heads * m.head_dim;
    const int n_ctas = e->n_sm * env_int("PTB_GEMV_CTAS_PER_SM", 2);
    const bool tp = m.tp_world > 1;
    e->gemvs.clear();
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
            g.p.epilogue = tp ? EPI_ALLREDUCE : (post ? EPI_STORE : EPI_RESID);
            g.p.peers.world = 1;
            if (tp) fill_peers(e, g.p, 0, l, m.n_layers);
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
            g.p.epilogue = tp ? EPI_ALLREDUCE : (post ? EPI_STORE : EPI_RESID);
            g.p.peers.world = 1;
            if (tp) fill_peers(e, g.p, 1, l, m.n_layers);
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
        if (tp) fill_peers(e, g.p, 2, 0, 1);
        if (plan_gemv(g, 1, m.hidden, std::min(n_ctas, 4096))) return -1;
        e->gemvs.push_back(g);
    }
    return 0;
}


// ------------------------------------------------------------------------------------------ persistent single-launch path
// CTA split and rows-per-tile of one GEMV op of the persistent kernel (same rules as plan_gemv, one CTA per SM).
static int plan_mega_gemv(MegaOp& op, int njobs, int K, int n_ctas, int warps, int slot_bytes, int* acc_floats) {
    op.kind = MK_GEMV;
    op.njobs = njobs;
    op.K = K;
    if (K % 256 || K > 10240) { ptb_set_error("persistent decode: input length %d must be a multiple of 256 and at most 10240", K); return -1; }
    double total = 0;
    for (int i = 0; i < njobs; ++i) total += (double)op.job[i].N * op.job[i].nblk * (op.job[i].qtype == QT_Q4K ? 144 : 210) * (op.job[i].w2 ? 2 : 1);
    int left = n_ctas, begin = 0;
    double left_bytes = total;
    for (int i = 0; i < njobs; ++i) {
        GemvJob& j = op.job[i];
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
    for (int i = 0; i < njobs; ++i) {
        GemvJob& j = op.job[i];
        const int pairs = j.w2 ? 2 : 1;
        const int nb = j.seg_base + (j.seg_rem ? 1 : 0);
        const int sz = seg_bytes(j.qtype, nb);
        const int rows_cta = (j.N + j.cta_count - 1) / j.cta_count;
        double best = 1e30;
        int bestRW = 0;
        for (int RW = 8; RW >= 1; RW >>= 1) {
            if (RW * sz * pairs > slot_bytes) continue;
            const int gprw = 8 / RW;
            const int items = ((rows_cta + RW - 1) / RW) * j.KS;
            const int rounds = (items + warps - 1) / warps;
            const double cost = rounds * ((double)((nb + gprw - 1) / gprw) * pairs + 1.0);
            if (cost < best - 1e-9) { best = cost; bestRW = RW; }
        }
        if (!bestRW) { ptb_set_error("persistent decode: a %d-byte segment does not fit a %d-byte ring slot", sz * pairs, slot_bytes); return -1; }
        j.RW = bestRW;
        if (j.KS > 1) *acc_floats = std::max(*acc_floats, rows_cta * j.KS * pairs);
    }
    return 0;
}

template <int NCONS>
static cudaError_t launch_mega_n(const MegaParams& p, int grid, size_t smem, cudaStream_t st) {
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(decode_mega_kernel<NCONS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_done = true;
    }
    decode_mega_kernel<NCONS><<<grid, (NCONS + 1) * 32, smem, st>>>(p);
    return cudaGetLastError();
}
static cudaError_t launch_mega(const MegaParams& p, int warps, int grid, size_t smem, cudaStream_t st) {
    // consumer warps + the producer warp fill whole register-allocation groups of four warps: 11+1 or 15+1
    switch (warps) {
        case 11: return launch_mega_n<11>(p, grid, smem, st);
        default: return launch_mega_n<15>(p, grid, smem, st);
    }
}

static size_t mega_attn_smem(int group) {
    switch (group) {
        case 1: return sizeof(MegaAttnShared<1>);
        case 2: return sizeof(MegaAttnShared<2>);
        case 4: return sizeof(MegaAttnShared<4>);
        default: return sizeof(MegaAttnShared<8>);
    }
}

// Build the op list of one token and the shared-memory layout; upload the list.
static int engine_plan_mega(Engine* e) {
    const PtbModelDesc& m = e->m;
    const int qd = m.n_heads * m.head_dim, kvd = m.n_kv_heads * m.head_dim;
    const int n_ctas = e->n_sm;
    e->mega_warps = env_int("PTB_MEGA_WARPS", 15) <= 11 ? 11 : 15;
    const int slot_bytes = (env_int("PTB_MEGA_SLOT_KB", 6) * 1024 + 127) / 128 * 128;
    {
        const int splits = (m.max_seq + ATT_CHUNK - 1) / ATT_CHUNK, group = m.n_heads / m.n_kv_heads;
        if (m.n_kv_heads > n_ctas) { ptb_set_error("persistent decode: %d KV heads exceed the %d CTAs", m.n_kv_heads, n_ctas); return -1; }
        auto ll_alloc = [](uint2** p, size_t n) { return cudaMalloc(p, n * sizeof(uint2)) != cudaSuccess || cudaMemset(*p, 0, n * sizeof(uint2)) != cudaSuccess; };
        if (ll_alloc(&e->x_ll, m.hidden) || ll_alloc(&e->qkv_ll, qd + 2 * kvd) || ll_alloc(&e->att_ll, qd) || ll_alloc(&e->ffn_ll, m.inter) ||
            ll_alloc(&e->part_o_ll, (size_t)m.n_kv_heads * splits * group * ATT_D) || ll_alloc(&e->part_ml_ll, (size_t)m.n_kv_heads * splits * group * 2)) {
            ptb_set_error("persistent decode: slot buffer allocation failed");
            return -1;
        }
    }
    std::vector<MegaOp> ops;
    int acc_floats = 0, kmax = 256;
    int last_x_op = 0;               // index of the op that produced the current residual stream
    auto gemv_op = [&](int njobs, int K) -> MegaOp& { ops.emplace_back(); MegaOp& o = ops.back(); memset(&o, 0, sizeof(o)); o.kind = MK_GEMV; o.njobs = njobs; o.K = K; kmax = std::max(kmax, K); return o; };
    {
        MegaOp o;
        memset(&o, 0, sizeof(o));
        o.kind = MK_EMBED;
        ops.push_back(o);
    }
    for (int l = 0; l < m.n_layers; ++l) {
        const PtbLayerDesc& L = e->layers[l];
        {
            MegaOp& o = gemv_op(3, m.hidden);
            set_job(o.job[0], L.q, nullptr, e->qkv);
            set_job(o.job[1], L.k, nullptr, e->qkv + qd);
            set_job(o.job[2], L.v, nullptr, e->qkv + qd + kvd);
            o.x_ll = e->x_ll; o.src_op = last_x_op; o.norm_w = L.attn_norm; o.eps = m.eps; o.norm_add_one = m.norm_add_one; o.epilogue = EPI_STORE;
            o.out_ll[0] = e->qkv_ll; o.out_ll[1] = e->qkv_ll + qd; o.out_ll[2] = e->qkv_ll + qd + kvd;
            if (plan_mega_gemv(o, 3, m.hidden, n_ctas, e->mega_warps, slot_bytes, &acc_floats)) return -1;
        }
        {
            MegaOp o;
            memset(&o, 0, sizeof(o));
            o.kind = MK_ATTN;
            o.q_norm = L.q_norm; o.k_norm = L.k_norm; o.cos = L.cos; o.sin = L.sin; o.window = L.window;
            o.k_cache = e->kc + (size_t)l * m.n_kv_heads * m.max_seq * m.head_dim;
            o.v_cache = e->vc + (size_t)l * m.n_kv_heads * m.max_seq * m.head_dim;
            ops.push_back(o);
        }
        {
            MegaOp& o = gemv_op(1, L.o.cols);
            set_job(o.job[0], L.o, nullptr, e->x);
            o.x_ll = e->att_ll; o.src_op = (int)ops.size() - 2; o.resid_ll = e->x_ll; o.out_ll[0] = e->x_ll; o.epilogue = EPI_RESID;
            if (plan_mega_gemv(o, 1, L.o.cols, n_ctas, e->mega_warps, slot_bytes, &acc_floats)) return -1;
            last_x_op = (int)ops.size() - 1;
        }
        {
            MegaOp& o = gemv_op(1, m.hidden);
            set_job(o.job[0], L.gate, &L.up, e->ffn);
            o.x_ll = e->x_ll; o.src_op = last_x_op; o.norm_w = L.ffn_norm; o.eps = m.eps; o.norm_add_one = m.norm_add_one; o.epilogue = EPI_GATED;
            o.act_gelu = m.act_gelu; o.out_ll[0] = e->ffn_ll;
            if (plan_mega_gemv(o, 1, m.hidden, n_ctas, e->mega_warps, slot_bytes, &acc_floats)) return -1;
        }
        {
            MegaOp& o = gemv_op(1, L.down.cols);
            set_job(o.job[0], L.down, nullptr, e->x);
            o.x_ll = e->ffn_ll; o.src_op = (int)ops.size() - 2; o.resid_ll = e->x_ll; o.out_ll[0] = e->x_ll; o.epilogue = EPI_RESID;
            if (plan_mega_gemv(o, 1, L.down.cols, n_ctas, e->mega_warps, slot_bytes, &acc_floats)) return -1;
            last_x_op = (int)ops.size() - 1;
        }
    }
    {
        MegaOp& o = gemv_op(1, m.hidden);
        set_job(o.job[0], m.lm_head, nullptr, e->logits);
        o.x_ll = e->x_ll; o.src_op = last_x_op; o.norm_w = m.out_norm; o.eps = m.eps; o.norm_add_one = m.norm_add_one; o.epilogue = EPI_ARGMAX;
        if (plan_mega_gemv(o, 1, m.hidden, n_ctas, e->mega_warps, slot_bytes, &acc_floats)) return -1;
    }
    e->n_ops = (int)ops.size();
    PTB_CUDA_OK(cudaMalloc(&e->d_ops, sizeof(MegaOp) * ops.size()));
    PTB_CUDA_OK(cudaMemcpy(e->d_ops, ops.data(), sizeof(MegaOp) * ops.size(), cudaMemcpyHostToDevice));
    PTB_CUDA_OK(cudaMalloc(&e->d_bar, 64));
    PTB_CUDA_OK(cudaMemset(e->d_bar, 0, 64));

    MegaParams& p = e->mp;
    memset(&p, 0, sizeof(p));
    p.ops = e->d_ops; p.n_ops = e->n_ops; p.gen = e->d_bar + 1; p.status = e->status; p.ctrl = e->ctrl;
    p.x = e->x; p.x_ll = e->x_ll; p.qkv_ll = e->qkv_ll; p.att_ll = e->att_ll;
    p.emb_table = (const uint8_t*)m.embed.w; p.emb_qtype = m.embed.qtype; p.emb_rowbytes = m.embed.rowbytes; p.emb_nblk = m.embed.cols / 256;
    p.hidden = m.hidden; p.vocab = m.embed.rows; p.emb_scale = m.emb_scale;
    p.part_o = e->part_o_ll; p.part_ml = e->part_ml_ll;
    p.n_heads = m.n_heads; p.n_kv_heads = m.n_kv_heads; p.group = m.n_heads / m.n_kv_heads; p.max_seq = m.max_seq;
    p.max_splits = (m.max_seq + ATT_CHUNK - 1) / ATT_CHUNK; p.neox = m.neox; p.attn_eps = m.eps; p.scale = 1.0f / sqrtf((float)m.head_dim);
    p.amax_val = e->amax_val; p.amax_idx = e->amax_idx; p.ticket = e->tickets + 1; p.logits = m.want_logits ? e->logits : nullptr;
    p.result = e->result; p.row_offset = m.vocab_offset; p.token_log = e->token_log; p.token_script = e->script;
    // shared memory: barriers | misc | quantised input | K-split accumulators | attention scratch | ring
    int optin = 0;
    PTB_CUDA_OK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, e->dev));
    const size_t cap = (size_t)optin - 1024;          // room for the kernel's static shared memory
    const int max_slots = 64;
    size_t off = align_up((size_t)2 * max_slots * 8, 128);
    p.off_misc = (int)off; off += 512;
    p.off_xq = (int)off; off += (size_t)kmax;
    p.off_xs = (int)off; off += (size_t)(kmax / 32) * 4;
    p.off_xsf = (int)off; off += (size_t)(kmax / 16) * 4;
    p.off_xsf32 = (int)off; off += (size_t)(kmax / 32) * 4;
    p.off_acc = (int)off; off += (size_t)acc_floats * 4;
    off = align_up(off, 16);
    p.off_attn = (int)off; off += mega_attn_smem(p.group);
    off = align_up(off, 128);
    p.off_ring = (int)off;
    if (off + 4 * (size_t)slot_bytes > cap) { ptb_set_error("persistent decode: %zu B of fixed shared memory leave no room for the ring", off); return -1; }
    p.slot_bytes = slot_bytes;
    p.nslots = (int)std::min<size_t>(max_slots, (cap - off) / slot_bytes);
    const int want = env_int("PTB_MEGA_SLOTS", 0);
    if (want >= 16 && want < p.nslots) p.nslots = want;
    if (p.nslots < 16) { ptb_set_error("persistent decode: only %d ring slots fit; at least 16 are needed", p.nslots); return -1; }
    e->mega_smem = off + (size_t)p.nslots * slot_bytes;
    if (e->trace) p.trace = e->trace;
    return 0;
}

// Enqueue one token's kernels on the engine stream.
static int engine_enqueue(Engine* e) {
    const PtbModelDesc& m = e->m;
    const int qd = m.n_heads * m.head_dim, kvd = m.n_kv_heads * m.head_dim;
    const int splits = (m.max_seq + ATT_CHUNK - 1) / ATT_CHUNK;
    const bool pdl = e->use_pdl;
    long n = 0;
    if (e->mega) {
        PTB_CUDA_OK(launch_mega(e->mp, e->mega_warps, e->n_sm, e->mega_smem, e->stream));
        e->launches_per_token = 1;
        return 0;
    }
    EmbedParams ep;
    memset(&ep, 0, sizeof(ep));
    ep.table = (const uint8_t*)m.embed.w; ep.qtype = m.embed.qtype; ep.rowbytes = m.embed.rowbytes;
    ep.nblk = m.embed.cols / 256; ep.H = m.hidden; ep.scale = m.emb_scale; ep.out = e->x; ep.ctrl = e->ctrl;
    ep.vocab = m.embed.rows; ep.status = e->status;
    ep.gen = m.tp_world > 1 ? (uint32_t*)(e->ctrl + CTRL_GEN) : nullptr;
    // the first kernel of a token is launched without the programmatic edge: it must not
    // overlap the previous token's lm_head, whose epilogue updates the control block
    PTB_CUDA_OK(launch_pdl(embed_kernel, dim3((m.hidden + 255) / 256), dim3(256), 0, e->stream, false, ep));
    ++n;
    size_t gi = 0;
    for (int l = 0; l < m.n_layers; ++l) {
        const PtbLayerDesc& L = e->layers[l];
        GemvLaunch& g0 = e->gemvs[gi++];
        if (e->trace) g0.p.trace = e->trace + 8 * (1 + 5 * l);
        PTB_CUDA_OK(launch_gemv(g0, e->stream, pdl));
        AttnParams a;
        memset(&a, 0, sizeof(a));
        a.q = e->qkv; a.k = e->qkv + qd; a.v = e->qkv + qd + kvd;
        a.q_norm = L.q_norm; a.k_norm = L.k_norm; a.cos = L.cos; a.sin = L.sin;
        a.k_cache = e->kc + (size_t)l * m.n_kv_heads * m.max_seq * m.head_dim;
        a.v_cache = e->vc + (size_t)l * m.n_kv_heads * m.max_seq * m.head_dim;
        a.out = e->att; a.part_o = e->part_o; a.part_ml = e->part_ml; a.ticket = e->tickets + 8; a.ctrl = e->ctrl;
        a.group = m.n_heads / m.n_kv_heads; a.max_seq = m.max_seq; a.max_splits = splits; a.neox = m.neox;
        a.eps = m.eps; a.scale = 1.0f / sqrtf((float)m.head_dim); a.window = L.window;
        if (e->trace) a.trace = e->trace + 8 * (2 + 5 * l);
        PTB_CUDA_OK(launch_attn(a, m.n_kv_heads, e->stream, pdl));
        for (int k = 0; k < 3; ++k) {
            GemvLaunch& g = e->gemvs[gi++];
            if (e->trace) g.p.trace = e->trace + 8 * (3 + k + 5 * l);
            PTB_CUDA_OK(launch_gemv(g, e->stream, pdl));
        }
        n += 5;
    }
    GemvLaunch& gl = e->gemvs[gi++];
    if (e->trace) gl.p.trace = e->trace + 8 * (1 + 5 * m.n_layers);
    PTB_CUDA_OK(launch_gemv(gl, e->stream, pdl));
    ++n;
    e->launches_per_token = n;
    return 0;
}

PTB_API void* ptb_engine_create(const PtbModelDesc* m, const PtbLayerDesc* layers, void* ext_stream) {
    if (m->head_dim != ATT_D) {
        ptb_set_error("decode engine: head_dim %d not supported (kernels are built for %d)", m->head_dim, ATT_D);
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
    // one GPU: the whole token as one persistent launch (PTB_MEGA=1; the default is the kernel-per-op graph)
    bool any_post = false;
    for (int l = 0; l < m->n_layers; ++l) any_post = any_post || layers[l].post_attn_norm || layers[l].post_ffn_norm;
    e->mega = m->tp_world <= 1 && !any_post && env_int("PTB_MEGA", 0) != 0;
    if (e->mega && engine_plan_mega(e)) { delete e; return nullptr; }
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
    cudaFree(e->d_ops); cudaFree(e->d_bar);
    cudaFree(e->x_ll); cudaFree(e->qkv_ll); cudaFree(e->att_ll); cudaFree(e->ffn_ll); cudaFree(e->part_o_ll); cudaFree(e->part_ml_ll);
    cudaFreeHost(e->h_pinned);
    if (e->own_stream) cudaStreamDestroy(e->stream);
    delete e;
}

// Capture one token into a graph (call once, before the first replay).
PTB_API int ptb_engine_capture(void* h) {
    Engine* e = (Engine*)h;
    if (e->exec) return 0;
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
PTB_API int ptb_gemv_plan(int qtype, int rows, int cols, int rowbytes, int paired, int n_ctas, int* out5) {
    GemvLaunch L;
    memset(&L, 0, sizeof(L));
    PtbWeightDesc d{(const void*)16, nullptr, qtype, rows, cols, rowbytes};
    set_job(L.p.job[0], d, paired ? &d : nullptr, nullptr);
    if (plan_gemv(L, 1, cols, n_ctas)) return -1;
    out5[0] = L.p.job[0].RW; out5[1] = L.p.stages; out5[2] = L.grid; out5[3] = (int)L.smem; out5[4] = L.p.tile_bytes;
    return 0;
}
