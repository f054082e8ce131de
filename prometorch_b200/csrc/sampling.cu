// Token sampling on the device: repetition penalty, temperature, top-k, top-p and the draw, in one launch.
//
// The reference copies all logits to the host and sorts them there for every token
// (torch/io/gguf_model.h:7658-7748), which makes sampled decoding 1.84x slower than greedy.  Here the
// selection is a radix step: a histogram over the top 12 bits of an order-preserving key of the penalised
// logits tells which bins hold the k best; those few dozen to few hundred elements are collected, sorted
// by one CTA, and temperature, the top-p cut and an inverse-CDF draw (uniform number from the caller)
// finish the job.  Two passes over the logits (L2-resident), three short launches.
#include "common.cuh"
#include "ptb200_types.h"
#include <algorithm>
#include <vector>

namespace ptb {

constexpr int SAMP_THREADS = 256;
constexpr int SAMP_BINS = 4096;         // histogram over the top 12 bits of the order-preserving key
constexpr int SAMP_MAX_K = 64;
constexpr int SAMP_MAX_CAND = 4096;

struct SampleParams {
    const float* logits;
    int V;
    int* history;            // ids seen so far (prompt + generated), may be null; capacity hist_cap
    int n_hist, hist_cap;    // the chosen id is appended at history[n_hist] when it fits
    float repeat_penalty, temperature, top_p, u;
    int top_k;
    unsigned* counters;      // [0] number of candidates; zero between calls.  [1] candidates dropped so far because more
                             // than SAMP_MAX_CAND logits fell into the threshold bin (sticky; see ptb_sample_dropped)
    unsigned* hist;          // [SAMP_BINS], zero between calls
    float* cand_val;         // [SAMP_MAX_CAND]
    int* cand_idx;
    float* xp;               // [V] logits after the repetition penalty
    int* out;                // out[0] = token id, out[1] = float bits of its probability
    int* ctrl_token;         // optional: also written here (device-side feedback)
};

// Order-preserving map float -> uint (larger float, larger key); NaN sorts below everything real.
__device__ __forceinline__ uint32_t ordered_key(float x) {
    if (x != x) return 0u;
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Pass 1: penalised logits and the histogram of their keys.
__device__ __forceinline__ void sample_hist_body(const SampleParams& P) {
    __shared__ uint32_t sh[SAMP_BINS];
    const int tid = threadIdx.x;
    for (int i = tid; i < SAMP_BINS; i += SAMP_THREADS) sh[i] = 0u;
    __syncthreads();
    const int per = (P.V + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(lo + per, P.V);
    for (int i = lo + tid; i < hi; i += SAMP_THREADS) P.xp[i] = P.logits[i];
    __syncthreads();
    if (P.repeat_penalty != 1.0f && P.history) {
        // every history id in my range is penalised exactly once: the first occurrence in the history does it
        for (int i = tid; i < P.n_hist; i += SAMP_THREADS) {
            const int t = P.history[i];
            if (t < lo || t >= hi) continue;
            bool first = true;
            for (int j = 0; j < i; ++j)
                if (P.history[j] == t) { first = false; break; }
            if (first) {
                const float x = P.logits[t];
                P.xp[t] = x > 0.f ? x / P.repeat_penalty : x * P.repeat_penalty;
            }
        }
    }
    __syncthreads();
    for (int i = lo + tid; i < hi; i += SAMP_THREADS) atomicAdd(&sh[ordered_key(P.xp[i]) >> 20], 1u);
    __syncthreads();
    for (int i = tid; i < SAMP_BINS; i += SAMP_THREADS)
        if (sh[i]) atomicAdd(&P.hist[i], sh[i]);
}

// Pass 2: every CTA finds the bin that holds the k-th largest key, then collects the elements of that bin and above.
__global__ void __launch_bounds__(SAMP_THREADS) sample_hist_kernel(const __grid_constant__ SampleParams P) { sample_hist_body(P); }
// Batched form: one grid row (blockIdx.y) per request, parameters read from device memory.
__global__ void __launch_bounds__(SAMP_THREADS) sample_hist_batch_kernel(const SampleParams* __restrict__ ps) { sample_hist_body(ps[blockIdx.y]); }

__device__ __forceinline__ void sample_collect_body(const SampleParams& P) {
    __shared__ uint32_t part[SAMP_THREADS];
    __shared__ int thr_bin;
    const int tid = threadIdx.x;
    constexpr int PER = SAMP_BINS / SAMP_THREADS;            // bins per thread, thread 0 owns the highest bins
    uint32_t mine = 0;
    const int b_hi = SAMP_BINS - 1 - tid * PER;
    for (int j = 0; j < PER; ++j) mine += P.hist[b_hi - j];
    part[tid] = mine;
    __syncthreads();
    if (tid == 0) {
        uint32_t cum = 0;
        int t = 0;
        for (; t < SAMP_THREADS; ++t) {
            if (cum + part[t] >= (uint32_t)P.top_k) break;
            cum += part[t];
        }
        int bin = 0;
        if (t < SAMP_THREADS) {
            bin = SAMP_BINS - 1 - t * PER;
            for (int j = 0; j < PER; ++j, --bin) {
                cum += P.hist[bin];
                if (cum >= (uint32_t)P.top_k) break;
            }
        }
        thr_bin = max(bin, 0);
    }
    __syncthreads();
    const uint32_t tb = (uint32_t)thr_bin;
    const int per = (P.V + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(lo + per, P.V);
    for (int i = lo + tid; i < hi; i += SAMP_THREADS) {
        const float x = P.xp[i];
        if ((ordered_key(x) >> 20) >= tb) {
            const unsigned slot = atomicAdd(P.counters, 1u);
            if (slot < SAMP_MAX_CAND) { P.cand_val[slot] = x; P.cand_idx[slot] = i; }
        }
    }
}

__global__ void __launch_bounds__(SAMP_THREADS) sample_collect_kernel(const __grid_constant__ SampleParams P) { sample_collect_body(P); }
__global__ void __launch_bounds__(SAMP_THREADS) sample_collect_batch_kernel(const SampleParams* __restrict__ ps) { sample_collect_body(ps[blockIdx.y]); }

// Bitonic sort, descending by value (ties: lower index first), `n` a power of two, in shared memory.
__device__ __forceinline__ void bitonic_desc(float* v, int* ix, int n, int tid, int nthreads) {
    for (int k = 2; k <= n; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < n; i += nthreads) {
                const int p = i ^ j;
                if (p > i) {
                    const bool up = (i & k) == 0;                         // this pair sorts descending when `up`
                    const float a = v[i], b = v[p];
                    const int ia = ix[i], ib = ix[p];
                    const bool a_first = a > b || (a == b && ia < ib);    // a belongs before b in descending order
                    if (up ? !a_first : a_first) { v[i] = b; v[p] = a; ix[i] = ib; ix[p] = ia; }
                }
            }
            __syncthreads();
        }
    }
}

// Pass 3 (one CTA): sort the candidates, temperature softmax over the k best, top-p cut, inverse-CDF draw.
__device__ __forceinline__ void sample_final_body(const SampleParams& P) {
    __shared__ float sv[SAMP_MAX_CAND];
    __shared__ int si[SAMP_MAX_CAND];
    const int tid = threadIdx.x;
    const int n_cand = (int)min(*P.counters, (unsigned)SAMP_MAX_CAND);
    if (tid == 0 && *P.counters > (unsigned)SAMP_MAX_CAND) P.counters[1] += *P.counters - (unsigned)SAMP_MAX_CAND;
    int n = 64;
    while (n < n_cand) n <<= 1;
    for (int i = tid; i < n; i += 1024) {
        sv[i] = i < n_cand ? P.cand_val[i] : -INFINITY;
        si[i] = i < n_cand ? P.cand_idx[i] : 0x7fffffff;
    }
    __syncthreads();
    bitonic_desc(sv, si, n, tid, 1024);
    for (int i = tid; i < SAMP_BINS; i += 1024) P.hist[i] = 0u;       // ready for the next call
    if (tid == 0) {
        const int k = min(P.top_k, n_cand);
        int choice = 0;
        float pc = 1.0f;
        if (P.temperature > 0.f && k > 0) {
            const float inv_t = 1.0f / P.temperature, m = sv[0] * inv_t;
            float z = 0.f;
            for (int i = 0; i < k; ++i) z += expf(sv[i] * inv_t - m);
            // top-p: keep the shortest prefix whose mass reaches top_p (always the first), renormalise, draw
            float kept = 0.f;
            int n_keep = k;
            if (P.top_p > 0.f && P.top_p < 1.f) {
                n_keep = 0;
                for (int i = 0; i < k; ++i) {
                    if (kept >= P.top_p * z) break;
                    kept += expf(sv[i] * inv_t - m);
                    ++n_keep;
                }
            } else {
                kept = z;
            }
            const float target = P.u * kept;
            float cum = 0.f;
            choice = n_keep - 1;
            for (int i = 0; i < n_keep; ++i) {
                cum += expf(sv[i] * inv_t - m);
                if (target < cum) { choice = i; break; }
            }
            pc = expf(sv[choice] * inv_t - m) / kept;
        }
        P.out[0] = si[choice];
        P.out[1] = __float_as_int(pc);
        if (P.ctrl_token) *P.ctrl_token = si[choice];
        if (P.history && P.n_hist < P.hist_cap) P.history[P.n_hist] = si[choice];
        *P.counters = 0u;
    }
}

__global__ void __launch_bounds__(1024) sample_final_kernel(const __grid_constant__ SampleParams P) { sample_final_body(P); }
__global__ void __launch_bounds__(1024) sample_final_batch_kernel(const SampleParams* __restrict__ ps) { sample_final_body(ps[blockIdx.x]); }

}  // namespace ptb

using namespace ptb;

static void fill_sample_params(SampleParams& p, const float* logits, int V, int* history, int n_hist, int hist_cap, float repeat_penalty,
                               float temperature, int top_k, float top_p, float u, void* scratch, int* out, int* ctrl_token) {
    p.logits = logits; p.V = V; p.history = history; p.n_hist = n_hist; p.hist_cap = hist_cap; p.repeat_penalty = repeat_penalty;
    p.temperature = temperature; p.top_p = top_p; p.u = u; p.top_k = top_k;
    uint8_t* s = (uint8_t*)scratch;
    p.counters = (unsigned*)s;
    p.hist = (unsigned*)(s + 64);
    p.cand_val = (float*)(s + 64 + SAMP_BINS * 4);
    p.cand_idx = (int*)(s + 64 + SAMP_BINS * 4 + SAMP_MAX_CAND * 4);
    p.xp = (float*)(s + 64 + SAMP_BINS * 4 + SAMP_MAX_CAND * 8);
    p.out = out; p.ctrl_token = ctrl_token;
}

// Bytes of scratch for a vocabulary of V entries (zero it once before the first call).
// How many candidates the sampler behind `scratch` has dropped since the scratch was zeroed (0 unless thousands of
// logits are tied at the top-k boundary); a non-zero count means some draws ignored tied candidates.
PTB_API int ptb_sample_dropped(const void* scratch, unsigned* out) {
    PTB_CUDA_OK(cudaMemcpy(out, (const unsigned*)scratch + 1, sizeof(unsigned), cudaMemcpyDeviceToHost));
    return 0;
}

PTB_API long long ptb_sample_scratch_bytes(int V) { return 64 + (long long)SAMP_BINS * 4 + (long long)SAMP_MAX_CAND * 8 + (long long)V * 4; }

// history: device array of `hist_cap` ids of which the first n_hist are valid; the chosen id is appended.
// top_k in 1..64.  `u` uniform in [0, 1).  temperature <= 0 returns the arg-max after the penalty.
// Three launches: histogram of the penalised logits, collection of the bins that hold the k best, final sort + draw.
PTB_API int ptb_sample_logits(const float* logits, int V, int* history, int n_hist, int hist_cap, float repeat_penalty, float temperature,
                              int top_k, float top_p, float u, void* scratch, int* out, int* ctrl_token, cudaStream_t st) {
    if (top_k < 1 || top_k > SAMP_MAX_K) { ptb_set_error("sample: top_k %d outside 1..%d", top_k, SAMP_MAX_K); return -1; }
    if (V < 1) { ptb_set_error("sample: empty vocabulary"); return -1; }
    SampleParams p;
    fill_sample_params(p, logits, V, history, n_hist, hist_cap, repeat_penalty, temperature, top_k, top_p, u, scratch, out, ctrl_token);
    const int grid = std::max(1, std::min(148, (V + 1023) / 1024));
    sample_hist_kernel<<<grid, SAMP_THREADS, 0, st>>>(p);
    sample_collect_kernel<<<grid, SAMP_THREADS, 0, st>>>(p);
    sample_final_kernel<<<1, 1024, 0, st>>>(p);
    PTB_CUDA_OK(cudaGetLastError());
    return grid;
}

// Sample `n` requests in three launches (grid row = request).  `reqs`: host array; `d_params`: device scratch of
// ptb_sample_batch_param_bytes(n) bytes that receives the kernel parameters (one stream-ordered copy).
PTB_API long long ptb_sample_batch_param_bytes(int n) { return (long long)n * sizeof(SampleParams); }

PTB_API int ptb_sample_logits_batch(const PtbSampleRequest* reqs, int n, int V, void* d_params, cudaStream_t st) {
    if (n <= 0) return 0;
    if (V < 1 || n > 4096) { ptb_set_error("sample batch: bad vocabulary or more than 4096 requests"); return -1; }
    static thread_local std::vector<SampleParams> host;
    host.resize(n);
    for (int i = 0; i < n; ++i) {
        const PtbSampleRequest& r = reqs[i];
        if (r.top_k < 1 || r.top_k > SAMP_MAX_K) { ptb_set_error("sample batch: top_k %d outside 1..%d", r.top_k, SAMP_MAX_K); return -1; }
        fill_sample_params(host[i], r.logits, V, r.history, r.n_hist, r.hist_cap, r.repeat_penalty, r.temperature, r.top_k, r.top_p, r.u,
                           r.scratch, r.out, nullptr);
    }
    PTB_CUDA_OK(cudaMemcpyAsync(d_params, host.data(), (size_t)n * sizeof(SampleParams), cudaMemcpyHostToDevice, st));
    const int grid = std::max(1, std::min(148, (V + 1023) / 1024));
    const SampleParams* dp = (const SampleParams*)d_params;
    sample_hist_batch_kernel<<<dim3(grid, n), SAMP_THREADS, 0, st>>>(dp);
    sample_collect_batch_kernel<<<dim3(grid, n), SAMP_THREADS, 0, st>>>(dp);
    sample_final_batch_kernel<<<n, 1024, 0, st>>>(dp);
    PTB_CUDA_OK(cudaGetLastError());
    return grid;
}
