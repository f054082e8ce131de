// Collectives fused with their neighbouring element-wise work, written
// directly against peer memory (plain loads/stores over NVLink; every rank has
// every peer's buffer mapped, see symm.cu).
//
//  * ddp_allreduce_kernel    — in-place two-shot all-reduce of a gradient bucket:
//    rank r sums slice r of all peers' buckets in fp32, applies the 1/world
//    scale, and writes the result into slice r of every peer's bucket.  This is
//    the reference's per-parameter `all_reduce` + host-side `*1/W`
//    (torch/distributed/ddp.cpp:1067-1091) as one kernel per bucket.
//  * fsdp_rs_adamw_kernel    — gradient reduce-scatter fused with the sharded
//    AdamW step: the summed slice never goes to memory as a gradient; it updates
//    the fp32 master shard and its moments and emits the bf16 shard the next
//    forward's GEMMs read (reference: torch/distributed/fsdp.h:268-322 + ZeROOptimizer).
//  * allgather_kernel        — push a local shard into every peer's full buffer.
//
// Synchronisation is two flag barriers per call (arrival counters in symmetric
// memory, release/acquire at system scope).  Every wait is bounded by a wall-clock
// budget (ptb_set_collective_timeout_ms, default 10 s or PTB_COLLECTIVE_TIMEOUT_MS):
// on expiry the kernel records PTB_ERR_FLAG_TIMEOUT, skips its work, still signals
// its peers and resets its ticket, so the channel can be used again, and returns.
#include "common.cuh"
#include <stdlib.h>
#include <algorithm>

namespace ptb {

constexpr int COLL_THREADS = 512;

struct PeerSet {
    void* buf[8];             // peer r's data buffer (same layout on every rank)
    uint32_t* flag[8];        // peer r's flag block: [2][8] arrival words (phase, source rank)
    void* buf2[8];            // optional second buffer per peer (fp32 master gradients of the bucket all-reduce)
    int rank, world;
    unsigned long long budget_ns;
};

// All CTAs call this.  `phase` 0: only signals from CTA 0; every CTA waits for all peers.
__device__ __forceinline__ bool barrier_in(const PeerSet& P, uint32_t seq, int* status) {
    if (blockIdx.x == 0 && threadIdx.x < P.world) st_release_sys(P.flag[threadIdx.x] + 0 * 8 + P.rank, seq);
    bool ok = true;
    if (threadIdx.x < P.world) ok = wait_flag_ge(P.flag[P.rank] + 0 * 8 + threadIdx.x, seq, status, P.budget_ns);
    return __syncthreads_and(ok);
}

// After all CTAs of this rank are done: the last one tells every peer and waits for every peer.  `ok` false (the
// entry barrier ran out of time): the peers are still told and the ticket is still reset, without waiting again.
__device__ __forceinline__ void barrier_out(const PeerSet& P, uint32_t seq, unsigned* ticket, int* status, bool ok = true) {
    __shared__ bool last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(ticket, 1u);
        last = (t == gridDim.x - 1);
        __threadfence();
    }
    __syncthreads();
    if (!last) return;
    if (threadIdx.x < P.world) {
        __threadfence_system();
        st_release_sys(P.flag[threadIdx.x] + 1 * 8 + P.rank, seq);
        if (ok) wait_flag_ge(P.flag[P.rank] + 1 * 8 + threadIdx.x, seq, status, P.budget_ns);
    }
    __syncthreads();
    if (threadIdx.x == 0) *ticket = 0u;
}

__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float* f) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

// Slice of `n_vec` 16-byte vectors owned by `rank`.
__device__ __forceinline__ void slice_of(long long n_vec, int rank, int world, long long& v0, long long& v1) {
    v0 = n_vec * rank / world;
    v1 = n_vec * (rank + 1) / world;
}

// MASTER (bf16 buckets only): the reduced, scaled slice is written as fp32 into every peer's second buffer (the
// master-gradient bucket an fp32 optimizer reads) instead of back into the bf16 bucket: the cast costs no extra pass.
template <bool BF16, bool MASTER>
__global__ void __launch_bounds__(COLL_THREADS) ddp_allreduce_kernel(const __grid_constant__ PeerSet P, long long n_vec, float scale,
                                                                   uint32_t seq, unsigned* ticket, int* status) {
    const bool ok = barrier_in(P, seq, status);
    long long v0, v1;
    slice_of(n_vec, P.rank, P.world, v0, v1);
    if (!ok) v1 = v0;
    for (long long v = v0 + (long long)blockIdx.x * COLL_THREADS + threadIdx.x; v < v1; v += (long long)gridDim.x * COLL_THREADS) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        uint4 in[8];
#pragma unroll
        for (int p = 0; p < 8; ++p)
            if (p < P.world) in[p] = __ldcg(reinterpret_cast<const uint4*>(P.buf[p]) + v);
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            if (p < P.world) {
                if (BF16) {
                    float f[8];
                    bf16x8_to_f32(in[p], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += f[j];
                } else {
                    const float* f = reinterpret_cast<const float*>(&in[p]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[j] += f[j];
                }
            }
        }
        uint4 out;
        if (BF16) {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] *= scale;
            if (MASTER) {
                const uint4 lo = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
                const uint4 hi = make_uint4(__float_as_uint(acc[4]), __float_as_uint(acc[5]), __float_as_uint(acc[6]), __float_as_uint(acc[7]));
#pragma unroll
                for (int p = 0; p < 8; ++p)
                    if (p < P.world) {
                        reinterpret_cast<uint4*>(P.buf2[p])[2 * v] = lo;
                        reinterpret_cast<uint4*>(P.buf2[p])[2 * v + 1] = hi;
                    }
                continue;
            }
            out = f32_to_bf16x8(acc);
        } else {
            float* o = reinterpret_cast<float*>(&out);
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = acc[j] * scale;
        }
#pragma unroll
        for (int p = 0; p < 8; ++p)
            if (p < P.world) reinterpret_cast<uint4*>(P.buf[p])[v] = out;
    }
    barrier_out(P, seq, ticket, status, ok);
}

struct AdamWArgs {
    float* master;            // fp32 [shard]
    float* m;
    float* v;
    __nv_bfloat16* shard_out; // bf16 [shard] — the parameter shard the GEMMs read
    float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale;
};

// Gradient buffers are bf16 [n_vec * 8] on every rank; rank r owns vectors slice_of(r).
__global__ void __launch_bounds__(COLL_THREADS) fsdp_rs_adamw_kernel(const __grid_constant__ PeerSet P, const __grid_constant__ AdamWArgs A,
                                                                   long long n_vec, uint32_t seq, unsigned* ticket, int* status) {
    const bool ok = barrier_in(P, seq, status);
    long long v0, v1;
    slice_of(n_vec, P.rank, P.world, v0, v1);
    if (!ok) v1 = v0;          // no update from gradients that are not known to be complete
    for (long long v = v0 + (long long)blockIdx.x * COLL_THREADS + threadIdx.x; v < v1; v += (long long)gridDim.x * COLL_THREADS) {
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 0.f;
        uint4 in[8];
#pragma unroll
        for (int p = 0; p < 8; ++p)
            if (p < P.world) in[p] = __ldcg(reinterpret_cast<const uint4*>(P.buf[p]) + v);
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            if (p < P.world) {
                float f[8];
                bf16x8_to_f32(in[p], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) g[j] += f[j];
            }
        }
        const long long e = (v - v0) * 8;      // element offset inside the local shard
        float pw[8], mm[8], vv[8];
        *reinterpret_cast<float4*>(pw) = *reinterpret_cast<const float4*>(A.master + e);
        *reinterpret_cast<float4*>(pw + 4) = *reinterpret_cast<const float4*>(A.master + e + 4);
        *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(A.m + e);
        *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(A.m + e + 4);
        *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(A.v + e);
        *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(A.v + e + 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float gj = g[j] * A.grad_scale;
            pw[j] *= 1.f - A.lr * A.wd;
            mm[j] = A.beta1 * mm[j] + (1.f - A.beta1) * gj;
            vv[j] = A.beta2 * vv[j] + (1.f - A.beta2) * gj * gj;
            pw[j] -= (A.lr / A.bc1) * mm[j] / (sqrtf(vv[j]) / sqrtf(A.bc2) + A.eps);
        }
        *reinterpret_cast<float4*>(A.master + e) = *reinterpret_cast<float4*>(pw);
        *reinterpret_cast<float4*>(A.master + e + 4) = *reinterpret_cast<float4*>(pw + 4);
        *reinterpret_cast<float4*>(A.m + e) = *reinterpret_cast<float4*>(mm);
        *reinterpret_cast<float4*>(A.m + e + 4) = *reinterpret_cast<float4*>(mm + 4);
        *reinterpret_cast<float4*>(A.v + e) = *reinterpret_cast<float4*>(vv);
        *reinterpret_cast<float4*>(A.v + e + 4) = *reinterpret_cast<float4*>(vv + 4);
        reinterpret_cast<uint4*>(A.shard_out)[v - v0] = f32_to_bf16x8(pw);
    }
    barrier_out(P, seq, ticket, status, ok);
}

// Copy my shard (shard_vec vectors) into slot [rank] of every peer's full buffer.
__global__ void __launch_bounds__(COLL_THREADS) allgather_kernel(const __grid_constant__ PeerSet P, const uint4* __restrict__ shard,
                                                               long long shard_vec, uint32_t seq, unsigned* ticket, int* status) {
    const bool ok = barrier_in(P, seq, status);
    if (!ok) shard_vec = 0;
    for (long long v = (long long)blockIdx.x * COLL_THREADS + threadIdx.x; v < shard_vec; v += (long long)gridDim.x * COLL_THREADS) {
        const uint4 x = shard[v];
#pragma unroll
        for (int p = 0; p < 8; ++p)
            if (p < P.world) reinterpret_cast<uint4*>(P.buf[p])[(long long)P.rank * shard_vec + v] = x;
    }
    barrier_out(P, seq, ticket, status);
}

// A flag barrier on its own (tests of the timeout path, and `tp_barrier`).
__global__ void peer_barrier_kernel(const __grid_constant__ PeerSet P, uint32_t seq, unsigned* ticket, int* status) {
    const bool ok = barrier_in(P, seq, status);
    barrier_out(P, seq, ticket, status, ok);
}

}  // namespace ptb

using namespace ptb;

// Wall-clock budget of every wait in these kernels.
static unsigned long long g_budget_ns = [] {
    const char* e = getenv("PTB_COLLECTIVE_TIMEOUT_MS");
    const long ms = e && *e ? atol(e) : 10000;
    return (unsigned long long)(ms > 0 ? ms : 1) * 1000000ull;
}();
PTB_API void ptb_set_collective_timeout_ms(int ms) { g_budget_ns = (unsigned long long)(ms > 0 ? ms : 1) * 1000000ull; }
PTB_API int ptb_get_collective_timeout_ms() { return (int)(g_budget_ns / 1000000ull); }

static void fill(PeerSet& P, void* const* bufs, void* const* flags, int rank, int world, void* const* bufs2 = nullptr) {
    for (int i = 0; i < 8; ++i) {
        P.buf[i] = i < world ? bufs[i] : nullptr;
        P.flag[i] = i < world ? (uint32_t*)flags[i] : nullptr;
        P.buf2[i] = (bufs2 && i < world) ? bufs2[i] : nullptr;
    }
    P.rank = rank;
    P.world = world;
    P.budget_ns = g_budget_ns;
}

// bufs/flags: host arrays of `world` device pointers (this rank's view of every peer's buffer / flag block).
// numel must be a multiple of 8 (bf16) or 4 (fp32).  ticket: device word, zero.  seq: strictly increasing per flag block.
PTB_API int ptb_ddp_allreduce(void* const* bufs, void* const* flags, int rank, int world, long long numel, int bf16, float scale,
                              unsigned seq, unsigned* ticket, int* status, int n_ctas, cudaStream_t st) {
    if (world > 8) { ptb_set_error("at most 8 peers"); return -1; }
    const int per = bf16 ? 8 : 4;
    if (numel % per) { ptb_set_error("bucket length %lld must be a multiple of %d", numel, per); return -1; }
    PeerSet P;
    fill(P, bufs, flags, rank, world);
    if (bf16) ddp_allreduce_kernel<true, false><<<n_ctas, COLL_THREADS, 0, st>>>(P, numel / per, scale, seq, ticket, status);
    else ddp_allreduce_kernel<false, false><<<n_ctas, COLL_THREADS, 0, st>>>(P, numel / per, scale, seq, ticket, status);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// The same reduction of a bf16 bucket with the result cast to fp32: every rank's `master_bufs` buffer (fp32, `numel`
// elements, symmetric like the bucket) receives the reduced, scaled gradients; the bf16 bucket keeps its local values.
PTB_API int ptb_ddp_allreduce_master(void* const* bufs, void* const* master_bufs, void* const* flags, int rank, int world,
                                     long long numel, float scale, unsigned seq, unsigned* ticket, int* status, int n_ctas,
                                     cudaStream_t st) {
    if (world > 8) { ptb_set_error("at most 8 peers"); return -1; }
    if (numel % 8) { ptb_set_error("bucket length %lld must be a multiple of 8", numel); return -1; }
    PeerSet P;
    fill(P, bufs, flags, rank, world, master_bufs);
    ddp_allreduce_kernel<true, true><<<n_ctas, COLL_THREADS, 0, st>>>(P, numel / 8, scale, seq, ticket, status);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// Reduce-scatter into an fp32 accumulator: slice `rank` of every peer's bf16 gradient buffer is summed in fp32, scaled and
// ADDED to `acc` (this rank's 1/world of the gradient).  The buffers can be reused as soon as the kernel is over (its
// closing barrier says every rank has read), which is what a gradient window shared by all layers needs; the optimizer
// then steps from `acc` once per iteration.
__global__ void __launch_bounds__(COLL_THREADS) fsdp_rs_accum_kernel(const __grid_constant__ PeerSet P, float* __restrict__ acc, float scale,
                                                                   long long n_vec, uint32_t seq, unsigned* ticket, int* status) {
    const bool ok = barrier_in(P, seq, status);
    long long v0, v1;
    slice_of(n_vec, P.rank, P.world, v0, v1);
    if (!ok) v1 = v0;
    for (long long v = v0 + (long long)blockIdx.x * COLL_THREADS + threadIdx.x; v < v1; v += (long long)gridDim.x * COLL_THREADS) {
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 0.f;
        uint4 in[8];
#pragma unroll
        for (int p = 0; p < 8; ++p)
            if (p < P.world) in[p] = __ldcg(reinterpret_cast<const uint4*>(P.buf[p]) + v);
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            if (p < P.world) {
                float f[8];
                bf16x8_to_f32(in[p], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) g[j] += f[j];
            }
        }
        float* a = acc + (v - v0) * 8;
        float4 a0 = *reinterpret_cast<float4*>(a), a1 = *reinterpret_cast<float4*>(a + 4);
        a0.x += g[0] * scale; a0.y += g[1] * scale; a0.z += g[2] * scale; a0.w += g[3] * scale;
        a1.x += g[4] * scale; a1.y += g[5] * scale; a1.z += g[6] * scale; a1.w += g[7] * scale;
        *reinterpret_cast<float4*>(a) = a0;
        *reinterpret_cast<float4*>(a + 4) = a1;
    }
    barrier_out(P, seq, ticket, status, ok);
}

// Owner side of the row-parallel GEMM's scatter-store epilogue: the `world` bf16 partial tiles that the ranks stored into this
// rank's slots are summed in fp32 in one pass (optionally on top of a residual) and written once as bf16.
__global__ void __launch_bounds__(256) slot_sum_kernel(const uint4* __restrict__ parts, int world, long long slot_vec,
                                                       const uint4* __restrict__ resid, uint4* __restrict__ out) {
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < slot_vec; v += (long long)gridDim.x * blockDim.x) {
        float acc[8];
        if (resid) bf16x8_to_f32(resid[v], acc);
        else {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        }
        for (int p = 0; p < world; ++p) {
            float f[8];
            bf16x8_to_f32(parts[(long long)p * slot_vec + v], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += f[j];
        }
        out[v] = f32_to_bf16x8(acc);
    }
}
// parts: [world][slot_elems] bf16 (local memory); resid (optional) and out: [slot_elems] bf16.
PTB_API int ptb_slot_sum(const void* parts, int world, long long slot_elems, const void* resid, void* out, cudaStream_t st) {
    if (world < 1 || slot_elems % 8) { ptb_set_error("slot sum: %lld elements per slot must be a multiple of 8", slot_elems); return -1; }
    const long long nv = slot_elems / 8;
    if (nv == 0) return 0;
    const int blocks = (int)std::min<long long>((nv + 255) / 256, 148 * 8);
    slot_sum_kernel<<<blocks, 256, 0, st>>>((const uint4*)parts, world, nv, (const uint4*)resid, (uint4*)out);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

// numel: elements of the full gradient (a multiple of 8 * world); acc: numel / world floats.
PTB_API int ptb_fsdp_rs_accum(void* const* bufs, void* const* flags, int rank, int world, long long numel, float* acc, float scale,
                              unsigned seq, unsigned* ticket, int* status, int n_ctas, cudaStream_t st) {
    if (world < 1 || world > 8 || numel % (8LL * world)) { ptb_set_error("fsdp accumulate: length %lld must be a multiple of 8*world", numel); return -1; }
    PeerSet P;
    fill(P, bufs, flags, rank, world);
    fsdp_rs_accum_kernel<<<n_ctas, COLL_THREADS, 0, st>>>(P, acc, scale, numel / 8, seq, ticket, status);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

PTB_API int ptb_fsdp_rs_adamw(void* const* bufs, void* const* flags, int rank, int world, long long numel, float* master, float* m,
                              float* v, void* shard_out, float lr, float beta1, float beta2, float eps, float wd, int step,
                              float grad_scale, unsigned seq, unsigned* ticket, int* status, int n_ctas, cudaStream_t st) {
    if (world > 8 || numel % (8LL * world)) { ptb_set_error("fsdp: length %lld must be a multiple of 8*world", numel); return -1; }
    PeerSet P;
    fill(P, bufs, flags, rank, world);
    AdamWArgs A;
    A.master = master; A.m = m; A.v = v; A.shard_out = (__nv_bfloat16*)shard_out;
    A.lr = lr; A.beta1 = beta1; A.beta2 = beta2; A.eps = eps; A.wd = wd;
    A.bc1 = 1.f - powf(beta1, (float)step);
    A.bc2 = 1.f - powf(beta2, (float)step);
    A.grad_scale = grad_scale;
    fsdp_rs_adamw_kernel<<<n_ctas, COLL_THREADS, 0, st>>>(P, A, numel / 8, seq, ticket, status);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

PTB_API int ptb_allgather(void* const* bufs, void* const* flags, int rank, int world, const void* shard, long long shard_bytes,
                          unsigned seq, unsigned* ticket, int* status, int n_ctas, cudaStream_t st) {
    if (world > 8 || shard_bytes % 16) { ptb_set_error("allgather: shard of %lld bytes must be a multiple of 16", shard_bytes); return -1; }
    PeerSet P;
    fill(P, bufs, flags, rank, world);
    allgather_kernel<<<n_ctas, COLL_THREADS, 0, st>>>(P, (const uint4*)shard, shard_bytes / 16, seq, ticket, status);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

PTB_API int ptb_peer_barrier(void* const* flags, int rank, int world, unsigned seq, unsigned* ticket, int* status, cudaStream_t st) {
    if (world < 1 || world > 8) { ptb_set_error("peer barrier: %d ranks; 1 to 8 are supported", world); return -1; }
    PeerSet P;
    void* none[8] = {0};
    fill(P, none, flags, rank, world);
    peer_barrier_kernel<<<1, 32, 0, st>>>(P, seq, ticket, status);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}
