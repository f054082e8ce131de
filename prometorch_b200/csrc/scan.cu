// Gated linear recurrence  h[b,t,d] = g[b,t,d] * h[b,t-1,d] + x[b,t,d]  (h[b,-1,d] = 0) over [B, T, D] tensors.
//
// The reference walks the time axis serially, one thread per (b, d) (aten/src/ATen/cuda/CUDAKernels.cu:869-906), which
// leaves the machine idle when B*D is small.  The recurrence is an associative scan over pairs (gate, value):
// (g2, x2) o (g1, x1) = (g1 g2, g2 x1 + x2), so time is cut into chunks of 64 steps:
//   scan_chunk_kernel  every (b, chunk, d) scans its chunk from zero and leaves the chunk's (product of gates, end value);
//   scan_fix_kernel    every (b, chunk, d) folds the aggregates of the chunks before it into a carry and adds
//                      carry * (running product of gates) to its elements.
// Threads run along d, so every access is coalesced.  The backward pass is the same scan run from the last step to the
// first with the gates shifted by one step (a[t] = dh[t] + g[t+1] a[t+1]); dx = a and dg[t] = a[t] * h[t-1].
#include "common.cuh"

namespace ptb {

constexpr int SCAN_CHUNK = 64;
constexpr int SCAN_THREADS = 128;

template <typename T> __device__ __forceinline__ float ld_f(const T* p) { return (float)*p; }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st_f(T* p, float v) { *p = (T)v; }
template <> __device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

struct ScanParams {
    const void* g;
    const void* x;
    void* out;              // h (forward) or a (backward)
    float* agg;             // [B, chunks, 2, D]: product of the chunk's gates, the chunk's end value
    const void* h;          // backward only: the forward result, for dg
    void* dg;               // backward only
    int B, T, D, chunks, reverse;
};

// Step s of a chunk in walking order -> time index, and the gate that multiplies the state arriving at that step.
__device__ __forceinline__ int step_time(const ScanParams& P, int chunk, int s) {
    const int k = chunk * SCAN_CHUNK + s;
    return P.reverse ? P.T - 1 - k : k;
}
template <typename T>
__device__ __forceinline__ float step_gate(const ScanParams& P, const T* g, size_t base, int t, int d) {
    if (!P.reverse) return ld_f(g + base + (size_t)t * P.D + d);
    return t + 1 < P.T ? ld_f(g + base + (size_t)(t + 1) * P.D + d) : 0.f;
}

template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS) scan_chunk_kernel(const __grid_constant__ ScanParams P) {
    const int d = blockIdx.x * SCAN_THREADS + threadIdx.x, chunk = blockIdx.y, b = blockIdx.z;
    if (d >= P.D) return;
    const size_t base = (size_t)b * P.T * P.D;
    const T* g = (const T*)P.g;
    const T* x = (const T*)P.x;
    T* out = (T*)P.out;
    float hcur = 0.f, prod = 1.f;
    const int n = min(SCAN_CHUNK, P.T - chunk * SCAN_CHUNK);
    for (int s = 0; s < n; ++s) {
        const int t = step_time(P, chunk, s);
        const float gt = step_gate(P, g, base, t, d);
        hcur = gt * hcur + ld_f(x + base + (size_t)t * P.D + d);
        prod *= gt;
        st_f(out + base + (size_t)t * P.D + d, hcur);
    }
    float* a = P.agg + (((size_t)b * P.chunks + chunk) * 2) * P.D + d;
    a[0] = prod;
    a[P.D] = hcur;
}

template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS) scan_fix_kernel(const __grid_constant__ ScanParams P) {
    const int d = blockIdx.x * SCAN_THREADS + threadIdx.x, chunk = blockIdx.y, b = blockIdx.z;
    if (d >= P.D) return;
    const size_t base = (size_t)b * P.T * P.D;
    const T* g = (const T*)P.g;
    T* out = (T*)P.out;
    float carry = 0.f;                                   // state that enters this chunk
    for (int c = 0; c < chunk; ++c) {
        const float* a = P.agg + (((size_t)b * P.chunks + c) * 2) * P.D + d;
        carry = a[0] * carry + a[P.D];
    }
    const int n = min(SCAN_CHUNK, P.T - chunk * SCAN_CHUNK);
    float prod = 1.f;
    for (int s = 0; s < n; ++s) {
        const int t = step_time(P, chunk, s);
        prod *= step_gate(P, g, base, t, d);
        const size_t i = base + (size_t)t * P.D + d;
        float v = ld_f(out + i);
        if (chunk > 0) {
            v += prod * carry;
            st_f(out + i, v);
        }
        if (P.dg) {                                      // backward: dg[t] = a[t] * h[t-1]
            const float hp = t > 0 ? ld_f((const T*)P.h + i - P.D) : 0.f;
            st_f((T*)P.dg + i, v * hp);
        }
    }
}

template <typename T>
static void launch_scan(const ScanParams& p, cudaStream_t st) {
    dim3 grid((p.D + SCAN_THREADS - 1) / SCAN_THREADS, p.chunks, p.B);
    scan_chunk_kernel<T><<<grid, SCAN_THREADS, 0, st>>>(p);
    if (p.chunks > 1 || p.dg) scan_fix_kernel<T><<<grid, SCAN_THREADS, 0, st>>>(p);
}

}  // namespace ptb

using namespace ptb;

// Floats of scratch for ptb_linear_scan_fwd / _bwd.
PTB_API long long ptb_linear_scan_scratch_floats(int B, int T, int D) { return (long long)B * ((T + SCAN_CHUNK - 1) / SCAN_CHUNK) * 2 * D; }

// h = scan(g, x) over dim 1 of [B, T, D] tensors (bf16 or fp32, contiguous).  agg: scratch of the size above.
PTB_API int ptb_linear_scan_fwd(const void* g, const void* x, void* h, float* agg, int B, int T, int D, int bf16, cudaStream_t st) {
    if (B <= 0 || T <= 0 || D <= 0) return 0;
    ScanParams p;
    p.g = g; p.x = x; p.out = h; p.agg = agg; p.h = nullptr; p.dg = nullptr;
    p.B = B; p.T = T; p.D = D; p.chunks = (T + SCAN_CHUNK - 1) / SCAN_CHUNK; p.reverse = 0;
    if (bf16) launch_scan<__nv_bfloat16>(p, st); else launch_scan<float>(p, st);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// dx[t] = dh[t] + g[t+1] dx[t+1];  dg[t] = dx[t] * h[t-1].
PTB_API int ptb_linear_scan_bwd(const void* g, const void* h, const void* dh, void* dx, void* dg, float* agg, int B, int T, int D, int bf16,
                                cudaStream_t st) {
    if (B <= 0 || T <= 0 || D <= 0) return 0;
    ScanParams p;
    p.g = g; p.x = dh; p.out = dx; p.agg = agg; p.h = h; p.dg = dg;
    p.B = B; p.T = T; p.D = D; p.chunks = (T + SCAN_CHUNK - 1) / SCAN_CHUNK; p.reverse = 1;
    if (bf16) launch_scan<__nv_bfloat16>(p, st); else launch_scan<float>(p, st);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}
