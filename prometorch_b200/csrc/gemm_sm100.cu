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
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int n_sm, cudaStream_t st) {
    auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
    static bool attr = false;
    constexpr int smem = Smem<BN, STAGES>::TOTAL;
    if (!attr) {
        PTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr = true;
    }
    const int grid = std::min(p.tiles_m * p.tiles_n, n_sm);
    kern<<<grid, THREADS, smem, st>>>(ta, tb, p);
    PTB_CUDA_OK(cudaGetLastError());
    return 0;
}

template <int BN, int STAGES>
static int launch_majors(int a_mn, int b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int n_sm, cudaStream_t st) {
    if (!a_mn && !b_mn) return launch<BN, STAGES, false, false>(ta, tb, p, n_sm, st);
    if (!a_mn && b_mn) return launch<BN, STAGES, false, true>(ta, tb, p, n_sm, st);
    if (a_mn && !b_mn) return launch<BN, STAGES, true, false>(ta, tb, p, n_sm, st);
    return launch<BN, STAGES, true, true>(ta, tb, p, n_sm, st);
}

// C[M,N] (+)= op(A) op(B)^T with bf16 operands and fp32 accumulation.
//   a_mn == 0: A is [M, K] row-major (pitch lda);  a_mn == 1: A is stored as [K, M] row-major.
//   b_mn == 0: B is [N, K] row-major (pitch ldb);  b_mn == 1: B is stored as [K, N] row-major.
//   flags: EPI_BIAS | EPI_ACCUM | EPI_OUT_F32 | EPI_GELU.  status: device int, set non-zero if a wait timed out.
PTB_API int ptb_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* C, long long ldc,
                          int M, int N, int K, const float* bias, int flags, int* status, int n_sm, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int out_elem = (flags & EPI_OUT_F32) ? 4 : 2;
    if (((uintptr_t)C & 15) || ((ldc * out_elem) & 15)) { ptb_set_error("gemm: C needs a 16-byte aligned base and row pitch"); return -1; }
    {
        // the tensor-map encoder is a driver call: make sure this thread (e.g. an autograd worker) has the
        // device's primary context current
        int dev = 0;
        PTB_CUDA_OK(cudaGetDevice(&dev));
        PTB_CUDA_OK(cudaSetDevice(dev));
        if (n_sm <= 0) PTB_CUDA_OK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
    }
    const int BN = N > 128 ? 256 : 128;
    CUtensorMap ta, tb;
    if (a_mn) { if (ptb_make_tmap_bf16(&ta, A, M, K, lda, 64, 64)) return -1; }
    else { if (ptb_make_tmap_bf16(&ta, A, K, M, lda, BK, BM)) return -1; }
    if (b_mn) { if (ptb_make_tmap_bf16(&tb, B, N, K, ldb, 64, 64)) return -1; }
    else { if (ptb_make_tmap_bf16(&tb, B, K, N, ldb, BK, BN)) return -1; }
    Params p;
    memset(&p, 0, sizeof(p));
    p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.bias = bias; p.flags = flags; p.status = status;
    p.tiles_m = (M + BM - 1) / BM;
    p.tiles_n = (N + BN - 1) / BN;
    if (BN == 256) return launch_majors<256, 4>(a_mn, b_mn, ta, tb, p, n_sm, st);
    return launch_majors<128, 6>(a_mn, b_mn, ta, tb, p, n_sm, st);
}
