// bf16 GEMM on the 5th-generation tensor cores: tcgen05.mma issued by one
// thread, operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte
// swizzle), fp32 accumulators in tensor memory (TMEM), epilogue through
// tcgen05.ld.  Persistent CTAs, one per SM, walk the output tiles; the two
// 256-column accumulators alternate so the epilogue of one tile overlaps the
// main loop of the next.
//
//   C[M,N] (+)= op(A) * op(B)      A: M x K,  B: N x K  ("K-major": K contiguous)
//                                  or stored transposed ("MN-major": M resp. N contiguous)
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocator + MMA
// issuer, warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w%4) .. +32).
// The reference's GEMM is cublasSgemm in fp32 (aten/src/ATen/cuda/CUDABlas.cu:455-479).
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace ptb {
namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;              // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;

constexpr int MAX_SHARDS = 8;

enum EpiFlags : int { EPI_BIAS = 1, EPI_ACCUM = 2, EPI_OUT_F32 = 4, EPI_GELU = 8, EPI_SCATTER_ADD = 16, EPI_SCATTER_STORE = 32,
                      EPI_TRANS = 64 };   // EPI_TRANS: element (row, col) is stored at C[col * ldc + row] (fp32 only)

// An operand whose stored matrix is split by rows over up to eight GPUs (each piece in that GPU's
// memory, mapped here): piece r holds stored rows [r*shard_rows, (r+1)*shard_rows).  The producer warp
// picks the tensor map from the row coordinate of the box it fetches, so the "all-gather" of a sharded
// weight or activation happens tile by tile inside the GEMM's TMA pipeline (plain, non-multicast TMA
// loads from peer memory).  nshards == 1 is the ordinary local operand.
struct Operand {
    CUtensorMap map[MAX_SHARDS];
    int nshards, shard_rows;
};

// Staging of a row-sharded operand (the fused all-gather): the stored matrix lives row-sharded over the
// ranks, rank r owning stored rows [r*shard_rows, (r+1)*shard_rows) INSIDE its own full-size symmetric
// buffer.  A few extra CTAs of the GEMM grid ("stagers") copy the peers' rows into this GPU's buffer in
// 128-row blocks, each block crossing NVLink exactly once, and publish a per-block flag; the TMA producer
// of the GEMM CTAs waits for the flags of the rows it is about to fetch and then reads local memory.
// Copy and math overlap block by block inside one launch.  seq == 0 disables staging.
constexpr int STAGE_ROWS = 128;
struct Staging {
    const uint4* peer[MAX_SHARDS];   // peer r's full-size buffer (this GPU's mapping); peer[rank] is `local`
    uint4* local;
    uint32_t* flags;                 // [ceil(stored_rows / 128)] last sequence number staged
    int rank, world, shard_rows, stored_rows;
    long long row_vec;               // 16-byte vectors per stored row (= pitch)
    uint32_t seq;
};

struct Params {
    int M, N, K;
    void* C;                // bf16 or fp32 [M, ldc]
    long long ldc;
    const float* bias;      // [N] fp32 (EPI_BIAS)
    int flags;
    int* status;
    int tiles_m, tiles_n;
    // EPI_SCATTER_ADD (GEMM -> reduce-scatter): output rows [r*out_shard_rows, ...) belong to rank r and are
    // added (fp32 atomics over NVLink) into that rank's buffer c_peer[r] of shape [out_shard_rows, ldc]
    // EPI_SCATTER_STORE: the same ownership, but each rank writes its bf16 partial tile into slot [scatter_rank] of
    // the owner's buffer ([world][out_shard_rows][ldc] bf16) with 16-byte stores; the owner sums the slots afterwards
    float* c_peer[MAX_SHARDS];
    int out_shard_rows;
    int scatter_rank;
    int stager_ctas;        // CTAs [0, stager_ctas) are stagers (lowest indices: dispatched first); the rest compute tiles
    // split-K (skinny M: too few output tiles to fill the machine): work item = (tile, split); split s runs k-blocks
    // [s*kb_per_split, (s+1)*kb_per_split) and stores its fp32 partial at C + s*split_stride; the caller sums them
    int splits, kb_per_split;
    long long split_stride;
    int pdl;                // launched with programmatic stream serialization: the producer waits for the previous kernel
    Staging stA, stB;
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Producer side: make sure stored rows [r0, r0 + nrows) have been staged for this sequence number.
__device__ __forceinline__ bool wait_staged(const Staging& S, int r0, int nrows, int* status) {
    if (S.seq == 0) return true;
    const int last = min(r0 + nrows, S.stored_rows) - 1;
    for (int blk = r0 / STAGE_ROWS; blk <= last / STAGE_ROWS; ++blk) {
        if ((blk * STAGE_ROWS) / S.shard_rows == S.rank && ((blk + 1) * STAGE_ROWS - 1) / S.shard_rows == S.rank) continue;   // my own rows
        uint64_t t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        uint32_t i = 0;
        while ((int32_t)(ld_acquire_gpu(S.flags + blk) - S.seq) < 0) {
            if ((++i & 255u) == 0) {
                uint64_t t1;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                if (t1 - t0 > 2000000000ull) { if (status) atomicExch(status, PTB_ERR_FLAG_TIMEOUT); return false; }
            }
        }
    }
    fence_proxy_async_all();        // the rows were written with ordinary stores; the TMA engine reads them next
    return true;
}

// Stager CTA: copy 128-row blocks that belong to other ranks from their memory into the local buffer.
// One thread drives the TMA engine: bulk loads from the peer into a ring of shared-memory slots, bulk stores
// from there to local memory, `NSLOT` pieces of up to `SLOT_BYTES` in flight, so that a handful of CTAs keeps
// NVLink busy.  `bar`: NSLOT mbarriers initialised with count 1; `ring`: NSLOT slots of SLOT_STRIDE bytes.
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src_smem)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

template <int NSLOT, int SLOT_STRIDE>
__device__ __forceinline__ void run_stager(const Staging& S, int stager, int n_stagers, uint8_t* ring, uint64_t* bar, uint32_t& uses,
                                           int* status) {
    if (S.seq == 0 || threadIdx.x != 0) return;
    constexpr uint32_t SLOT_BYTES = 32768;
    static_assert(SLOT_STRIDE >= (int)SLOT_BYTES, "a pipeline stage must hold one staging piece");
    const int nblk = (S.stored_rows + STAGE_ROWS - 1) / STAGE_ROWS;
    for (int blk = stager; blk < nblk; blk += n_stagers) {
        const int r0 = blk * STAGE_ROWS, r1 = min(r0 + STAGE_ROWS, S.stored_rows);
        const int owner = r0 / S.shard_rows;
        if (owner == S.rank || (int32_t)(ld_acquire_gpu(S.flags + blk) - S.seq) >= 0) continue;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(S.peer[owner] + (long long)r0 * S.row_vec);
        uint8_t* dst = reinterpret_cast<uint8_t*>(S.local + (long long)r0 * S.row_vec);
        const long long total = (long long)(r1 - r0) * S.row_vec * 16;
        const int npieces = (int)((total + SLOT_BYTES - 1) / SLOT_BYTES);
        auto piece_bytes = [&](int q) { return (uint32_t)min((long long)SLOT_BYTES, total - (long long)q * SLOT_BYTES); };
        auto load = [&](int q) {       // piece q of this block into slot (uses + q) % NSLOT
            const uint32_t slot = (uses + (uint32_t)q) % NSLOT;
            mbar_expect_tx(&bar[slot], piece_bytes(q));
            bulk_g2s(ring + (size_t)slot * SLOT_STRIDE, src + (long long)q * SLOT_BYTES, piece_bytes(q), &bar[slot]);
        };
        for (int q = 0; q < min(NSLOT - 1, npieces); ++q) load(q);
        bool ok = true;
        for (int q = 0; q < npieces && ok; ++q) {
            const uint32_t u = uses + (uint32_t)q, slot = u % NSLOT;
            ok = mbar_wait(&bar[slot], (u / NSLOT) & 1u, status);
            if (!ok) break;
            fence_proxy_async_all();
            bulk_s2g(dst + (long long)q * SLOT_BYTES, ring + (size_t)slot * SLOT_STRIDE, piece_bytes(q));
            bulk_commit();
            if (q + NSLOT - 1 < npieces) {
                bulk_wait_read<1>();          // the store of piece q-1 has read its slot: that slot takes piece q+NSLOT-1
                load(q + NSLOT - 1);
            }
        }
        uses += (uint32_t)npieces;
        bulk_wait<0>();                       // every store of this block has completed
        if (!ok) return;
        fence_proxy_async_all();
        __threadfence();
        st_release_gpu(S.flags + blk, S.seq);
    }
}

// ---- PTX wrappers -----------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle.  K-major: rows of 128 B, 8-row groups 1024 B apart
// (SBO).  MN-major: 64-element chunks `lbo_bytes` apart, 8 k-rows 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;          // descriptor version of this architecture
    d |= (uint64_t)2 << 61;          // SWIZZLE_128B
    return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, M x N tile, operand majors (0 = K-major, 1 = MN-major).
__host__ __device__ constexpr uint32_t instr_desc(int M_, int N_, int a_mn, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(N_ >> 3) << 17) |
           ((uint32_t)(M_ >> 4) << 24);
}

template <int BN, int STAGES>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BAR_OFF + 256 + 1024;      // + barriers + slack for 1024 B alignment
};

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ Operand opA, const __grid_constant__ Operand opB, const __grid_constant__ Params P) {
    using S = Smem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;      // [2]
    uint64_t* acc_empty = acc_full + 2;       // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_mn = P.tiles_m * P.tiles_n;
    const int num_tiles = tiles_mn * P.splits;
    const int kblocks = (P.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&opA.map[0]);
        prefetch_tmap(&opB.map[0]);
    }
    if (P.pdl) pdl_launch_dependents();           // the next kernel may set itself up; it waits for this grid to finish
    const int n_gemm = (int)gridDim.x - P.stager_ctas;
    const int cta = (int)blockIdx.x - P.stager_ctas;
    if (cta < 0) {
        // ---------------------------------------------------------------------- stager CTA (no TMEM, no tiles)
        __syncthreads();                      // the pipeline barriers are initialised
        if constexpr (S::STAGE_BYTES >= 32768) {          // narrow-tile instantiations are never launched with stagers
            uint32_t uses = 0;
            run_stager<STAGES, S::STAGE_BYTES>(P.stA, blockIdx.x, P.stager_ctas, smem, full, uses, P.status);
            run_stager<STAGES, S::STAGE_BYTES>(P.stB, blockIdx.x, P.stager_ctas, smem, full, uses, P.status);
        }
        return;
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            // an MN-major staged operand is walked along K in full by every tile: once the first tile has
            // seen all of its blocks staged, later tiles need not look at the flags again
            bool first_tile = true;
            if (P.pdl) pdl_wait();                // nothing of this kernel touched global memory before this point
            for (int t = cta; t < num_tiles && ok; t += n_gemm, first_tile = false) {
                const int tt = t % tiles_mn, sp = t / tiles_mn;
                const int m0 = (tt % P.tiles_m) * BM, n0 = (tt / P.tiles_m) * BN;
                const int kb_lo = sp * P.kb_per_split, kb_hi = min(kblocks, kb_lo + P.kb_per_split);
                for (int kb = kb_lo; kb < kb_hi && ok; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES) ok = mbar_wait(&empty[s], (uint32_t)(((it / STAGES) - 1) & 1), P.status);
                    if (!ok) break;
                    uint8_t* sa = smem + s * S::STAGE_BYTES;
                    uint8_t* sb = sa + S::A_BYTES;
                    mbar_expect_tx(&full[s], S::STAGE_BYTES);
                    // rows being staged from peers must have landed before the TMA engine reads them
                    if (A_MN ? first_tile : kb == kb_lo) ok = wait_staged(P.stA, A_MN ? kb * BK : m0, A_MN ? BK : BM, P.status);
                    if (ok && (B_MN ? first_tile : kb == kb_lo)) ok = wait_staged(P.stB, B_MN ? kb * BK : n0, B_MN ? BK : BN, P.status);
                    if (!ok) break;
                    // the box's row coordinate selects the shard (and so the GPU) it is fetched from
                    if (A_MN) {
                        const int r = kb * BK, sh = opA.nshards > 1 ? r / opA.shard_rows : 0;
                        for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * 8192, &opA.map[sh], m0 + c * 64, r - sh * opA.shard_rows, &full[s]);
                    } else {
                        const int sh = opA.nshards > 1 ? m0 / opA.shard_rows : 0;
                        tma_load_2d(sa, &opA.map[sh], kb * BK, m0 - sh * opA.shard_rows, &full[s]);
                    }
                    if (B_MN) {
                        const int r = kb * BK, sh = opB.nshards > 1 ? r / opB.shard_rows : 0;
                        for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * 8192, &opB.map[sh], n0 + c * 64, r - sh * opB.shard_rows, &full[s]);
                    } else {
                        const int sh = opB.nshards > 1 ? n0 / opB.shard_rows : 0;
                        tma_load_2d(sb, &opB.map[sh], kb * BK, n0 - sh * opB.shard_rows, &full[s]);
                    }
                }
            }
            if (!ok) *abort_flag = 1;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
            int it = 0, tl = 0;
            bool ok = true;
            for (int t = cta; t < num_tiles && ok; t += n_gemm, ++tl) {
                const int b = tl & 1;
                if (tl >= 2) ok = mbar_wait(&acc_empty[b], (uint32_t)(((tl >> 1) - 1) & 1), P.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * BN);
                const int kb_lo = (t / tiles_mn) * P.kb_per_split, kb_hi = min(kblocks, kb_lo + P.kb_per_split);
                for (int kb = kb_lo; kb < kb_hi && ok; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (uint32_t)((it / STAGES) & 1), P.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * S::STAGE_BYTES), sb = sa + S::A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // K-major: 16 bf16 = 32 B further along the swizzled row; MN-major: 16 k-rows = 2048 B further
                        const uint64_t da = A_MN ? smem_desc(sa + k * 2048, 8192, 1024) : smem_desc(sa + k * 32, 16, 1024);
                        const uint64_t db = B_MN ? smem_desc(sb + k * 2048, 8192, 1024) : smem_desc(sb + k * 32, 16, 1024);
                        umma_bf16(d_tmem, da, db, idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);          // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(&acc_full[b]);   // accumulator complete
            }
            if (!ok) *abort_flag = 1;
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;                     // TMEM lane quarter this warp may read
        int tl = 0;
        bool ok = true;
        for (int t = cta; t < num_tiles && ok; t += n_gemm, ++tl) {
            const int b = tl & 1;
            const int tt = t % tiles_mn, sp = t / tiles_mn;
            const int m0 = (tt % P.tiles_m) * BM, n0 = (tt / P.tiles_m) * BN;
            ok = mbar_wait(&acc_full[b], (uint32_t)((tl >> 1) & 1), P.status);
            if (!ok) break;
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BN);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + c, r);
                tmem_ld_wait();
                const int col = n0 + c;
                if (row < P.M && col < P.N) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (P.flags & EPI_BIAS) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (col + j < P.N) v[j] += P.bias[col + j];
                    }
                    if (P.flags & EPI_GELU) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
                    }
                    if (P.flags & EPI_TRANS) {
                        // swapped operands (rows = output features, columns = tokens): a warp's 32 lanes hold 32
                        // consecutive features of one token, so each store instruction writes 128 contiguous bytes
                        float* cp = reinterpret_cast<float*>(P.C) + (size_t)sp * P.split_stride + (size_t)col * P.ldc + row;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col + j < P.N) cp[(size_t)j * P.ldc] = v[j];
                    } else if (P.flags & EPI_SCATTER_ADD) {
                        const int owner = row / P.out_shard_rows;
                        float* cp = P.c_peer[owner] + (size_t)(row - owner * P.out_shard_rows) * P.ldc + col;
                        for (int j = 0; j < 32 && col + j < P.N; ++j) atomicAdd(cp + j, v[j]);
                    } else if (P.flags & EPI_SCATTER_STORE) {
                        const int owner = row / P.out_shard_rows;
                        __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(P.c_peer[owner]) +
                                            ((size_t)P.scatter_rank * P.out_shard_rows + (row - owner * P.out_shard_rows)) * P.ldc + col;
                        if (col + 32 <= P.N) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 o;
                                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                                for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
                                *reinterpret_cast<uint4*>(cp + j) = o;
                            }
                        } else {
                            for (int j = 0; j < 32 && col + j < P.N; ++j) cp[j] = __float2bfloat16_rn(v[j]);
                        }
                    } else if (P.flags & EPI_OUT_F32) {
                        float* cp = reinterpret_cast<float*>(P.C) + (size_t)sp * P.split_stride + (size_t)row * P.ldc + col;
                        if (col + 32 <= P.N) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                if (P.flags & EPI_ACCUM) { const float4 p = *reinterpret_cast<float4*>(cp + j); o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w; }
                                *reinterpret_cast<float4*>(cp + j) = o;
                            }
                        } else {
                            for (int j = 0; j < 32 && col + j < P.N; ++j) cp[j] = (P.flags & EPI_ACCUM) ? cp[j] + v[j] : v[j];
                        }
                    } else {
                        __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(P.C) + (size_t)row * P.ldc + col;
                        if (col + 32 <= P.N) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                if (P.flags & EPI_ACCUM) {
                                    const uint4 pv = *reinterpret_cast<uint4*>(cp + j);
                                    const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&pv);
#pragma unroll
                                    for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(ph[e]); v[j + 2 * e] += f.x; v[j + 2 * e + 1] += f.y; }
                                }
                                uint4 o;
                                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                                for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
                                *reinterpret_cast<uint4*>(cp + j) = o;
                            }
                        } else {
                            for (int j = 0; j < 32 && col + j < P.N; ++j)
                                cp[j] = __float2bfloat16_rn((P.flags & EPI_ACCUM) ? __bfloat162float(cp[j]) + v[j] : v[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);
        }
        if (!ok) *abort_flag = 1;
    }
    // ---- teardown: every role has left its loop (waits are bounded), TMEM goes back
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace gemm
}  // namespace ptb
