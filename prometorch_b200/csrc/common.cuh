// Shared device/host helpers for the sm_100a kernels: error handling, warp
// reductions, and thin wrappers over the PTX this library relies on
// (mbarrier, bulk async copies, programmatic dependent launch, system-scope
// acquire/release).  Every wait in here is bounded: on expiry the helper
// records a code in a status word and returns, it never traps or spins forever.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#define PTB_API extern "C" __attribute__((visibility("default")))

// Last error text, readable from Python through ptb_last_error().
void ptb_set_error(const char* fmt, ...);
// Whether chained kernels are launched with programmatic stream serialization (PTB_PDL=0 turns it off).
bool ptb_pdl_enabled();

#define PTB_CUDA_OK(expr)                                                                      \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess) {                                                               \
            ptb_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return -1;                                                                         \
        }                                                                                      \
    } while (0)

// Status codes written by kernels into their status word.
enum PtbStatus : int {
    PTB_OK = 0,
    PTB_ERR_MBARRIER_TIMEOUT = 1,   // a bulk copy never completed
    PTB_ERR_FLAG_TIMEOUT = 2,       // a peer never published its flag
    PTB_ERR_BOUNDS = 3,             // an index fell outside its extent
};

namespace ptb {

constexpr int kWarp = 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and records PTB_ERR_MBARRIER_TIMEOUT) if the phase did not complete within
// `budget_ns` of wall-clock time (%globaltimer, read every 256 polls, so the budget does not depend on the SM clock).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, uint64_t budget_ns = 2000000000ull) {
    for (uint32_t i = 0; i < 256u; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        for (uint32_t i = 0; i < 256u; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        uint64_t t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > budget_ns) break;
    }
    if (status) atomicExch(status, PTB_ERR_MBARRIER_TIMEOUT);
    return false;
}

// ---- bulk async copy global -> shared (TMA, untiled).  dst, src 16 B aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- programmatic dependent launch ---------------------------------------
// wait: block until the preceding kernel in the stream has completed and its
// writes are visible.  launch_dependents: allow the next kernel to begin its
// prologue.  Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Host side: chained kernels are launched with programmatic stream serialization unless PTB_PDL=0.  A kernel that is
// launched this way calls pdl_wait() before it touches global memory (every thread, before any early return).
template <typename... KArgs, typename... Args>
inline cudaError_t ptb_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args&&... args) {
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
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- system-scope flags (peer GPUs over NVLink) ---------------------------
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Spin until *p >= want (generation counters only grow).  Bounded by a wall
// clock budget in nanoseconds; returns false and records the timeout on expiry.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t want, int* status, uint64_t budget_ns = 1000000000ull) {
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint32_t i = 0;; ++i) {
        if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
        if ((i & 63u) == 63u) {
            uint64_t t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > budget_ns) break;
        }
    }
    if (status) atomicExch(status, PTB_ERR_FLAG_TIMEOUT);
    return false;
}

// ---- "data + sequence number" slots (8 bytes, written and read as one access): a reader that sees
// the expected sequence number also sees the payload, so no fence and no separate flag is needed.
__device__ __forceinline__ void st_ll(uint2* p, uint32_t data, uint32_t seq) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(seq) : "memory");
}
__device__ __forceinline__ uint2 ld_ll(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// Poll a slot until it carries `seq`; bounded by a nanosecond budget.  Returns the payload (0 on timeout).
__device__ __forceinline__ uint32_t wait_ll(const uint2* p, uint32_t seq, int* status, uint64_t budget_ns = 1000000000ull) {
    uint2 v = ld_ll(p);
    if (v.y == seq) return v.x;
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint32_t i = 0;; ++i) {
        v = ld_ll(p);
        if (v.y == seq) return v.x;
        if ((i & 63u) == 63u) {
            uint64_t t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > budget_ns) break;
        }
    }
    if (status) atomicExch(status, PTB_ERR_FLAG_TIMEOUT);
    return 0u;
}

// Two neighbouring slots in one 16-byte access (each 8-byte half stays whole, so each carries its own check).
__device__ __forceinline__ void st_ll2(uint2* p, uint32_t d0, uint32_t d1, uint32_t seq) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(seq), "r"(d1), "r"(seq) : "memory");
}
__device__ __forceinline__ uint4 ld_ll2(const uint2* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// Eight consecutive slots (64 bytes, 16-byte aligned) -> eight floats; true when all eight carry `seq`.
__device__ __forceinline__ bool ll_try8(const uint2* p, uint32_t seq, float* v) {
    const uint4 a = ld_ll2(p), b = ld_ll2(p + 2), c = ld_ll2(p + 4), d = ld_ll2(p + 6);
    v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.z); v[2] = __uint_as_float(b.x); v[3] = __uint_as_float(b.z);
    v[4] = __uint_as_float(c.x); v[5] = __uint_as_float(c.z); v[6] = __uint_as_float(d.x); v[7] = __uint_as_float(d.z);
    return a.y == seq && a.w == seq && b.y == seq && b.w == seq && c.y == seq && c.w == seq && d.y == seq && d.w == seq;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float gelu_tanh(float x) {
    const float k = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}

}  // namespace ptb
