// Paged KV cache for the continuous-batching engine: rotary + page write, and one-token attention over a page table.
//
// The reference's engine (torch/serve/llm.h:299-334, 806-818) keeps the cache in 64-token pages that a request
// picks from a shared pool, and walks them on the CPU one request after another.  Here the pool is one bf16
// tensor per layer, [page][kv_head][64][D]; a step of the engine serves every active request in one batch:
//   paged_rope_write_kernel  rotates q (in place) and k of the new tokens and stores k, v in the slot the page
//                            table gives for (request, position);
//   paged_attn_decode_kernel one CTA per (kv head, request, split): its warps walk the request's pages with an
//                            online softmax for the whole GQA group, merge through shared memory, and either
//                            finish or leave a partial (max, sum, acc) for paged_attn_merge_kernel.
// A page id outside the pool is never dereferenced: the kernel records PTB_ERR_BOUNDS and skips the page.
#include "common.cuh"
#include <algorithm>

namespace ptb {

constexpr int PAGE = 64;
constexpr int PA_WARPS = 4;
constexpr int PA_THREADS = PA_WARPS * 32;

struct PagedWriteParams {
    __nv_bfloat16* qkv;            // [n, (H + 2 Hk) D]: q heads, then k heads, then v heads
    const int* pos;                // [n] position of each token in its request
    const int* req;                // [n] row of the page table
    const int* page_table;         // [requests, pt_stride] page ids
    int pt_stride, n_pages;
    const float* cos;              // [max_pos, D/2]
    const float* sin;
    __nv_bfloat16* k_pages;        // [n_pages, Hk, PAGE, D]
    __nv_bfloat16* v_pages;
    __nv_bfloat16* k_out;          // optional [n, Hk, D]: the rotated keys, contiguous (prompt pass)
    int n, H, Hk, D, max_pos;
    int* status;
    // when `work` is set the projection arrives as split-K partials [splits][n][(H + 2 Hk) D] fp32 (qkv is unused) and
    // the rotated q goes to q_out [n, H D] bf16
    const float* work;
    int splits;
    long long split_stride;
    __nv_bfloat16* q_out;
};

// Element `e` of token `i`'s projection row: from the bf16 row, or the sum of the split-K partials.
__device__ __forceinline__ float proj_elem(const PagedWriteParams& P, const __nv_bfloat16* row, size_t i, int e, int width) {
    if (!P.work) return __bfloat162float(row[e]);
    const float* w = P.work + i * width + e;
    float a = w[0];
    for (int s = 1; s < P.splits; ++s) a += w[(size_t)s * P.split_stride];
    return a;
}

// One CTA per token.  Rotation pairs are (j, j + D/2) within a head (the Hugging Face Llama convention).
__global__ void __launch_bounds__(256) paged_rope_write_kernel(const __grid_constant__ PagedWriteParams P) {
    pdl_wait();
    pdl_launch_dependents();
    const int i = blockIdx.x;
    const int half = P.D / 2;
    const int pos = P.pos[i];
    const int width = (P.H + 2 * P.Hk) * P.D;
    __nv_bfloat16* row = P.qkv ? P.qkv + (size_t)i * width : nullptr;
    const int page_slot = pos / PAGE, in_page = pos % PAGE;
    const int page = P.page_table[(size_t)P.req[i] * P.pt_stride + min(page_slot, P.pt_stride - 1)];
    const bool ok = pos >= 0 && pos < P.max_pos && page_slot < P.pt_stride && page >= 0 && page < P.n_pages;
    if (!ok) {
        if (threadIdx.x == 0 && P.status) atomicExch(P.status, PTB_ERR_BOUNDS);
        return;
    }
    const float* cs = P.cos + (size_t)pos * half;
    const float* sn = P.sin + (size_t)pos * half;
    const int n_rot = (P.H + P.Hk) * half;
    for (int e = threadIdx.x; e < n_rot; e += blockDim.x) {
        const int h = e / half, j = e % half;
        const float a = proj_elem(P, row, i, h * P.D + j, width), b = proj_elem(P, row, i, h * P.D + j + half, width);
        const float c = cs[j], s = sn[j];
        const __nv_bfloat16 ra = __float2bfloat16_rn(a * c - b * s), rb = __float2bfloat16_rn(b * c + a * s);
        if (h < P.H) {
            __nv_bfloat16* hp = P.work ? P.q_out + ((size_t)i * P.H + h) * P.D : row + (size_t)h * P.D;
            hp[j] = ra; hp[j + half] = rb;
        } else {
            const int kh = h - P.H;
            __nv_bfloat16* dst = P.k_pages + (((size_t)page * P.Hk + kh) * PAGE + in_page) * P.D;
            dst[j] = ra; dst[j + half] = rb;
            if (P.k_out) {
                __nv_bfloat16* ko = P.k_out + ((size_t)i * P.Hk + kh) * P.D;
                ko[j] = ra; ko[j + half] = rb;
            }
        }
    }
    const int v0 = (P.H + P.Hk) * P.D;
    for (int e = threadIdx.x; e < P.Hk * P.D; e += blockDim.x) {
        const int kh = e / P.D, d = e % P.D;
        P.v_pages[(((size_t)page * P.Hk + kh) * PAGE + in_page) * P.D + d] =
            P.work ? __float2bfloat16_rn(proj_elem(P, row, i, v0 + e, width)) : row[v0 + e];
    }
}

struct PagedAttnParams {
    const __nv_bfloat16* q;        // [B, q_stride] with head h at column h * D
    long long q_stride;
    __nv_bfloat16* out;            // [B, H * D]
    const int* lens;               // [B] tokens in the cache (the new one included)
    const int* page_table;
    int pt_stride, n_pages;
    const __nv_bfloat16* k_pages;
    const __nv_bfloat16* v_pages;
    float* work;                   // [B, H, nsplit, D + 2] partial (acc, max, sum) when nsplit > 1
    int B, H, Hk, nsplit;
    float scale_log2;              // softmax scale times log2(e)
    int* status;
};

template <int D, int G>
__global__ void __launch_bounds__(PA_THREADS, (G <= 4 ? 8 : 6)) paged_attn_decode_kernel(const __grid_constant__ PagedAttnParams P) {
    constexpr int DV = D / 32;                        // output dims per lane (4 or 2)
    static_assert(DV == 4 || DV == 2, "head size 128 or 64");
    __shared__ float q_s[G][D];
    __shared__ float p_s[PA_WARPS][G][PAGE];
    __shared__ float acc_s[PA_WARPS][G][D];
    __shared__ float ml_s[PA_WARPS][G][2];
    const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    pdl_launch_dependents();
    for (int e = threadIdx.x; e < G * D; e += PA_THREADS) {
        const int g = e / D, d = e % D;
        q_s[g][d] = __bfloat162float(P.q[(size_t)b * P.q_stride + (size_t)(kvh * G + g) * D + d]) * P.scale_log2;
    }
    __syncthreads();
    const int len = P.lens[b];
    const int npages = min((len + PAGE - 1) / PAGE, P.pt_stride);
    // pages of this split, dealt to the warps round-robin
    const int per = (npages + P.nsplit - 1) / P.nsplit;
    const int p_lo = split * per, p_hi = min(p_lo + per, npages);
    float m[G], l[G], acc[G][DV];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < DV; ++i) acc[g][i] = 0.f;
    }
    for (int pg = p_lo + warp; pg < p_hi; pg += PA_WARPS) {
        const int page = P.page_table[(size_t)b * P.pt_stride + pg];
        if (page < 0 || page >= P.n_pages) {
            if (lane == 0 && P.status) atomicExch(P.status, PTB_ERR_BOUNDS);
            continue;
        }
        const int valid = min(PAGE, len - pg * PAGE);
        const __nv_bfloat16* kb = P.k_pages + ((size_t)page * P.Hk + kvh) * PAGE * D;
        const __nv_bfloat16* vb = P.v_pages + ((size_t)page * P.Hk + kvh) * PAGE * D;
        // scores: each lane owns tokens lane and lane + 32 and walks their rows in 16-byte pieces
        float s[2][G];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int t = lane + r * 32;
#pragma unroll
            for (int g = 0; g < G; ++g) s[r][g] = 0.f;
            if (t < valid) {
                const uint4* kr = reinterpret_cast<const uint4*>(kb + (size_t)t * D);
#pragma unroll 8
                for (int c = 0; c < D / 8; ++c) {
                    const uint4 raw = kr[c];
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
                    float kf[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h2[i]); kf[2 * i] = f.x; kf[2 * i + 1] = f.y; }
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][c * 8]);
                        const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][c * 8 + 4]);
                        s[r][g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] + qb.x * kf[4] + qb.y * kf[5] + qb.z * kf[6] + qb.w * kf[7];
                    }
                }
            } else {
#pragma unroll
                for (int g = 0; g < G; ++g) s[r][g] = -INFINITY;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float mx = warp_max(fmaxf(s[0][g], s[1][g]));
            const float m_new = fmaxf(m[g], mx);                       // finite: a page always has a valid token
            const float corr = exp2f(m[g] - m_new);
            const float p0 = exp2f(s[0][g] - m_new), p1 = exp2f(s[1][g] - m_new);
            p_s[warp][g][lane] = p0;
            p_s[warp][g][lane + 32] = p1;
            l[g] = l[g] * corr + warp_sum(p0 + p1);
            m[g] = m_new;
#pragma unroll
            for (int i = 0; i < DV; ++i) acc[g][i] *= corr;
        }
        __syncwarp();
        // P V: each lane owns DV consecutive output dims.  Sixteen rows are fetched (kept packed) before they are used so
        // that sixteen loads are in flight per lane; rows past `valid` belong to the page (readable) and carry p = 0.
        constexpr int PF = 16;
        for (int t0 = 0; t0 < valid; t0 += PF) {
            if constexpr (DV == 4) {
                uint2 raw[PF];
#pragma unroll
                for (int u = 0; u < PF; ++u) raw[u] = *reinterpret_cast<const uint2*>(vb + (size_t)(t0 + u) * D + lane * 4);
#pragma unroll
                for (int u = 0; u < PF; ++u) {
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
                    const float2 a = __bfloat1622float2(h2[0]), c = __bfloat1622float2(h2[1]);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float p = p_s[warp][g][t0 + u];
                        acc[g][0] += p * a.x; acc[g][1] += p * a.y; acc[g][2] += p * c.x; acc[g][3] += p * c.y;
                    }
                }
            } else {
                uint32_t raw[PF];
#pragma unroll
                for (int u = 0; u < PF; ++u) raw[u] = *reinterpret_cast<const uint32_t*>(vb + (size_t)(t0 + u) * D + lane * 2);
#pragma unroll
                for (int u = 0; u < PF; ++u) {
                    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[u]));
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float p = p_s[warp][g][t0 + u];
                        acc[g][0] += p * a.x; acc[g][1] += p * a.y;
                    }
                }
            }
        }
        __syncwarp();
    }
    // merge the warps
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int i = 0; i < DV; ++i) acc_s[warp][g][lane * DV + i] = acc[g][i];
        if (lane == 0) { ml_s[warp][g][0] = m[g]; ml_s[warp][g][1] = l[g]; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < G * D; e += PA_THREADS) {
        const int g = e / D, d = e % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < PA_WARPS; ++w) M = fmaxf(M, ml_s[w][g][0]);
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < PA_WARPS; ++w) {
            const float f = ml_s[w][g][0] == -INFINITY ? 0.f : exp2f(ml_s[w][g][0] - M);
            L += ml_s[w][g][1] * f;
            o += acc_s[w][g][d] * f;
        }
        const int h = kvh * G + g;
        if (P.nsplit == 1) {
            P.out[((size_t)b * P.H + h) * D + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
        } else {
            float* wk = P.work + (((size_t)b * P.H + h) * P.nsplit + split) * (D + 2);
            wk[d] = o;
            if (d == 0) { wk[D] = M; wk[D + 1] = L; }
        }
    }
}

// Combine the splits of one (request, head): grid (H, B), D threads.
__global__ void paged_attn_merge_kernel(const float* __restrict__ work, __nv_bfloat16* __restrict__ out, int H, int D, int nsplit) {
    pdl_wait();
    pdl_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const float* wk = work + ((size_t)b * H + h) * nsplit * (D + 2);
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, wk[s * (D + 2) + D]);
    float L = 0.f, o = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = wk[s * (D + 2) + D];
        const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
        L += wk[s * (D + 2) + D + 1] * f;
        o += wk[s * (D + 2) + d] * f;
    }
    out[((size_t)b * H + h) * D + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
}

template <int D>
static int launch_decode(const PagedAttnParams& p, int G, cudaStream_t st) {
    dim3 grid(p.Hk, p.B, p.nsplit);
    const bool pdl = ptb_pdl_enabled();
    cudaError_t e;
    switch (G) {
        case 1: e = ptb_launch(paged_attn_decode_kernel<D, 1>, grid, dim3(PA_THREADS), 0, st, pdl, p); break;
        case 2: e = ptb_launch(paged_attn_decode_kernel<D, 2>, grid, dim3(PA_THREADS), 0, st, pdl, p); break;
        case 4: e = ptb_launch(paged_attn_decode_kernel<D, 4>, grid, dim3(PA_THREADS), 0, st, pdl, p); break;
        case 8: e = ptb_launch(paged_attn_decode_kernel<D, 8>, grid, dim3(PA_THREADS), 0, st, pdl, p); break;
        default: ptb_set_error("paged attention: group size %d not in {1, 2, 4, 8}", G); return -1;
    }
    PTB_CUDA_OK(e);
    return 0;
}

}  // namespace ptb

using namespace ptb;

// Rotate q and k of `n` new tokens, store k and v in their page slots.  qkv: [n, (H + 2 Hk) D] bf16 (q rotated in
// place); pos / req: [n]; page_table: [requests, pt_stride]; cos / sin: [max_pos, D/2] fp32; k_out optional.
static int rope_write(void* qkv, const float* work, int splits, void* q_out, int n, int H, int Hk, int D, const int* pos, const int* req,
                      const int* page_table, int pt_stride, int n_pages, const float* cos, const float* sin, int max_pos, void* k_pages,
                      void* v_pages, void* k_out, int* status, cudaStream_t st) {
    if (n <= 0) return 0;
    if (D % 2) { ptb_set_error("paged_rope_write: odd head size"); return -1; }
    PagedWriteParams p;
    p.work = work; p.splits = splits; p.split_stride = (long long)n * (H + 2 * Hk) * D; p.q_out = (__nv_bfloat16*)q_out;
    p.qkv = (__nv_bfloat16*)qkv; p.pos = pos; p.req = req; p.page_table = page_table; p.pt_stride = pt_stride; p.n_pages = n_pages;
    p.cos = cos; p.sin = sin; p.k_pages = (__nv_bfloat16*)k_pages; p.v_pages = (__nv_bfloat16*)v_pages; p.k_out = (__nv_bfloat16*)k_out;
    p.n = n; p.H = H; p.Hk = Hk; p.D = D; p.max_pos = max_pos; p.status = status;
    PTB_CUDA_OK(ptb_launch(paged_rope_write_kernel, dim3(n), dim3(256), 0, st, ptb_pdl_enabled(), p));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

PTB_API int ptb_paged_rope_write(void* qkv, int n, int H, int Hk, int D, const int* pos, const int* req, const int* page_table,
                                 int pt_stride, int n_pages, const float* cos, const float* sin, int max_pos, void* k_pages,
                                 void* v_pages, void* k_out, int* status, cudaStream_t st) {
    return rope_write(qkv, nullptr, 0, nullptr, n, H, Hk, D, pos, req, page_table, pt_stride, n_pages, cos, sin, max_pos, k_pages, v_pages, k_out,
                      status, st);
}

// The same, reading the projection as split-K partials `work` [splits][n][(H + 2 Hk) D] fp32 (what ptb_gemm_bf16_splitk_partials
// leaves) and writing the rotated q to q_out [n, H D] bf16: the sum of the partials costs no launch of its own.
PTB_API int ptb_paged_rope_write_partials(const float* work, int splits, void* q_out, int n, int H, int Hk, int D, const int* pos,
                                          const int* req, const int* page_table, int pt_stride, int n_pages, const float* cos,
                                          const float* sin, int max_pos, void* k_pages, void* v_pages, int* status, cudaStream_t st) {
    if (!work || splits < 1 || !q_out) { ptb_set_error("paged_rope_write_partials: needs partials and an output for q"); return -1; }
    return rope_write(nullptr, work, splits, q_out, n, H, Hk, D, pos, req, page_table, pt_stride, n_pages, cos, sin, max_pos, k_pages, v_pages,
                      nullptr, status, st);
}

// Floats of workspace ptb_paged_attn_decode needs for `nsplit` > 1.
PTB_API long long ptb_paged_attn_work_floats(int B, int H, int D, int nsplit) { return nsplit > 1 ? (long long)B * H * nsplit * (D + 2) : 0; }

// One new token per request attends to its pages.  q: [B, q_stride] bf16; out: [B, H D] bf16; lens: [B].
PTB_API int ptb_paged_attn_decode(const void* q, long long q_stride, void* out, int B, int H, int Hk, int D, const int* lens,
                                  const int* page_table, int pt_stride, int n_pages, const void* k_pages, const void* v_pages,
                                  float scale, float* work, int nsplit, int* status, cudaStream_t st) {
    if (B <= 0) return 0;
    if (Hk <= 0 || H % Hk) { ptb_set_error("paged attention: %d heads over %d kv heads", H, Hk); return -1; }
    if (nsplit < 1 || (nsplit > 1 && !work)) { ptb_set_error("paged attention: nsplit %d needs a workspace", nsplit); return -1; }
    PagedAttnParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = (__nv_bfloat16*)out; p.lens = lens; p.page_table = page_table;
    p.pt_stride = pt_stride; p.n_pages = n_pages; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.work = work; p.B = B; p.H = H; p.Hk = Hk; p.nsplit = nsplit; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    int rc;
    if (D == 128) rc = launch_decode<128>(p, H / Hk, st);
    else if (D == 64) rc = launch_decode<64>(p, H / Hk, st);
    else { ptb_set_error("paged attention: head size %d not in {64, 128}", D); return -1; }
    if (rc) return rc;
    if (nsplit > 1)
        PTB_CUDA_OK(ptb_launch(paged_attn_merge_kernel, dim3(H, B), dim3(D), 0, st, ptb_pdl_enabled(), (const float*)work, (__nv_bfloat16*)out, H, D, nsplit));
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}
