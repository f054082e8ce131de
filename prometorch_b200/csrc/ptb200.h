// Public C interface of libptb200.so: every entry point of the native library, grouped by source file.
//
// All functions are `extern "C"`; tensors cross the boundary as device pointers, launches go to the stream given
// (0 = the legacy default stream).  Functions returning int return 0 on success and -1 on failure, in which case
// ptb_last_error() holds a message for the calling thread.  Kernels that wait (on a copy, a flag of a peer GPU)
// bound their waits and report through a device status word: 0 ok, 1 a bulk copy never completed, 2 a peer never
// published its flag, 3 an index fell outside its extent.
//
// The reference exposes its native layer as C++ headers (c10/, aten/, torch/csrc/); here the native layer is this
// C ABI, which the Python package binds with ctypes and which C or C++ programs can link directly.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct PtbModelDesc PtbModelDesc;      // decode engine descriptors: layouts in decode_engine.cu, mirrored by prometorch_b200/_native.py
typedef struct PtbLayerDesc PtbLayerDesc;
typedef struct PtbStaging PtbStaging;          // staging request of the sharded-operand GEMM: layout in gemm_sm100.cu

// ---------------------------------------------------------------------------- collectives.cu
// bufs/flags: host arrays of `world` device pointers (this rank's view of every peer's buffer / flag block).
// numel must be a multiple of 8 (bf16) or 4 (fp32).  ticket: device word, zero.  seq: strictly increasing per flag block.
int ptb_ddp_allreduce(void* const* bufs, void* const* flags, int rank, int world, long long numel, int bf16, float scale, unsigned seq, unsigned* ticket, int* status, int n_ctas, cudaStream_t st);

int ptb_fsdp_rs_adamw(void* const* bufs, void* const* flags, int rank, int world, long long numel, float* master, float* m, float* v, void* shard_out, float lr, float beta1, float beta2, float eps, float wd, int step, float grad_scale, unsigned seq, unsigned* ticket, int* status, int n_ctas, cudaStream_t st);

int ptb_allgather(void* const* bufs, void* const* flags, int rank, int world, const void* shard, long long shard_bytes, unsigned seq, unsigned* ticket, int* status, int n_ctas, cudaStream_t st);

int ptb_peer_barrier(void* const* flags, int rank, int world, unsigned seq, unsigned* ticket, int* status, cudaStream_t st);

// ---------------------------------------------------------------------------- decode_engine.cu
const char* ptb_last_error();

// y = epilogue(W x).  Device pointers; w2/norm_w/resid/bias may be null.
int ptb_gemv(const void* w, const void* w2, int qtype, int rows, int cols, int rowbytes, const float* x, const float* norm_w, float eps, const float* bias, const float* resid, float* out, int epilogue, int act_gelu, int n_ctas, void* scratch /* >= 16 + 8*n_ctas bytes, zeroed */, int* status, cudaStream_t stream);

int ptb_attn_decode(const float* q, const float* k, const float* v, const float* q_norm, const float* k_norm, const float* cos, const float* sin, void* k_cache, void* v_cache, float* out, float* part_o, float* part_ml, unsigned* ticket, const int* ctrl, int n_kv_heads, int group, int max_seq, int neox, float eps, int window, cudaStream_t stream);

void* ptb_engine_create(const PtbModelDesc* m, const PtbLayerDesc* layers, void* ext_stream);

void ptb_engine_destroy(void* h);

// Capture one token into a graph (call once, before the first replay).
int ptb_engine_capture(void* h);

// Write {token, pos, self_feed} (and the log cursor) through pinned memory on the engine stream.
int ptb_engine_set_ctrl(void* h, int token, int pos, int self_feed, int reset_log);

// Enqueue `n` tokens (graph replays if captured, eager launches otherwise).  Asynchronous.
int ptb_engine_run(void* h, int n);

// Host-fed step, the serving loop: copy {token,pos} in from pinned memory, run one token, copy the
// sampled id back to pinned memory, wait.  Returns the id (or -1).
int ptb_engine_step(void* h, int token, int pos);

// Scripted run: feed `n` prompt tokens starting at position pos0, then keep generating from the
// arg-max.  Sets up the control block; follow with ptb_engine_run(h, n + n_new - 1).  log[n-1+i] is
// the i-th generated token.
int ptb_engine_begin_script(void* h, const int* tokens, int n, int pos0);

int ptb_engine_sync(void* h);

// Copy the first n logged token ids to host memory; returns how many steps have run since the log reset.
int ptb_engine_read_log(void* h, int* out, int n);

int ptb_engine_status(void* h);

// Copy the phase stamps of the last token ([kernels][8] uint64 nanoseconds) to `out`; returns the kernel count.
int ptb_engine_read_trace(void* h, unsigned long long* out, int max_kernels);

void* ptb_engine_stream(void* h);

void* ptb_engine_logits(void* h);

void* ptb_engine_hidden(void* h);

void* ptb_engine_result(void* h);

// Device addresses of layer `layer`'s fp16 K and V caches, each [kv_heads][max_seq][head_dim].
int ptb_engine_kv_cache(void* h, int layer, void** k, void** v);

long ptb_engine_launches_per_token(void* h);

int ptb_engine_kv_bytes(void* h, long* out);

// Geometry report for one GEMV (tests and notes): rows per tile, stages, grid, smem, tile bytes.
int ptb_gemv_plan(int qtype, int rows, int cols, int rowbytes, int paired, int n_ctas, int* out5);

// ---------------------------------------------------------------------------- dequant.cu
// w: a matrix of N rows x cols in the GEMV streaming layout -> out bf16 [N, cols] row-major.
int ptb_dequant_segmajor(const void* w, int qtype, int N, int cols, void* out, cudaStream_t st);

// out[t] = scale * table[ids[t]] for T ids (device int32).  status: device word, set if an id is out of range.
int ptb_dequant_rows(const void* table, int qtype, int rowbytes, int cols, const int* ids, int T, float scale, int vocab, int* status, void* out, cudaStream_t st);

// ---------------------------------------------------------------------------- flash_attn.cu
int ptb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Tq, int Tk, int H, int Hk, int D, int causal, float scale, int q_offset, cudaStream_t st);

// dq: fp32 [B,Tq,H,D] zero-initialised by the caller; delta: fp32 [B,H,Tq] scratch.
int ptb_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse, float* delta, float* dq, void* dk, void* dv, void* unused, int B, int Tq, int Tk, int H, int Hk, int D, int causal, float scale, int q_offset, cudaStream_t st);

// ---------------------------------------------------------------------------- flash_attn_sm100.cu
// q [B, Tq, H, D], k/v [B, Tk, Hk, D] bf16 contiguous, D in {64, 128}; o like q; lse [B, H, Tq] fp32 (natural log).
// status: device int, set non-zero if a wait timed out.
int ptb_flash_attn_fwd_sm100(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Tq, int Tk, int H, int Hk, int D, int causal, float scale, int q_offset, int* status, cudaStream_t st);

// ---------------------------------------------------------------------------- gemm_sm100.cu
// General entry point.  a_ptrs/b_ptrs: arrays of a_shards/b_shards device pointers.  c_peers (EPI_SCATTER_ADD):
// `c_shards` fp32 buffers [out_shard_rows, ldc], one per rank.
int ptb_gemm_bf16_ex(void* const* a_ptrs, int a_shards, int a_shard_rows, long long lda, int a_mn, void* const* b_ptrs, int b_shards, int b_shard_rows, long long ldb, int b_mn, void* C, long long ldc, void* const* c_peers, int c_shards, int out_shard_rows, int M, int N, int K, const float* bias, int flags, int* status, int n_sm, cudaStream_t st, const PtbStaging* stage_a, const PtbStaging* stage_b);

// C[M,N] (+)= op(A) op(B)^T with bf16 operands and fp32 accumulation, all operands local.
//   a_mn == 0: A is [M, K] row-major (pitch lda);  a_mn == 1: A is stored as [K, M] row-major.
//   b_mn == 0: B is [N, K] row-major (pitch ldb);  b_mn == 1: B is stored as [K, N] row-major.
//   flags: EPI_BIAS | EPI_ACCUM | EPI_OUT_F32 | EPI_GELU.  status: device int, set non-zero if a wait timed out.
int ptb_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* C, long long ldc, int M, int N, int K, const float* bias, int flags, int* status, int n_sm, cudaStream_t st);

// ---------------------------------------------------------------------------- optim_kernels.cu
int ptb_opt_chunk();

int ptb_opt_tensor_bytes();

// tensors: device array of OptTensor rows; chunks: device int2 array of n_chunks entries; h: 16 host floats.
int ptb_multi_tensor_opt(const void* tensors, const void* chunks, int n_chunks, int kind, int grad_bf16, const float* h, const float* grad_scale, const int* skip, cudaStream_t stream);

// Total gradient norm into out[0], clip coefficient into out[1]; found_inf (optional) is set to 1 if any
// gradient is inf/nan.  `partial` holds n_chunks floats of scratch.
int ptb_multi_tensor_grad_norm(const void* tensors, const void* chunks, int n_chunks, int grad_bf16, float* partial, float max_norm, float extra_scale, float* out, int* found_inf, cudaStream_t stream);

int ptb_multi_tensor_scale(const void* tensors, const void* chunks, int n_chunks, int grad_bf16, const float* scale, cudaStream_t stream);

// ---------------------------------------------------------------------------- sampling.cu
// Bytes of scratch for a vocabulary of V entries (zero it once before the first call).
long long ptb_sample_scratch_bytes(int V);

// history: device array of `hist_cap` ids of which the first n_hist are valid; the chosen id is appended.
// top_k in 1..64.  `u` uniform in [0, 1).  temperature <= 0 returns the arg-max after the penalty.
// Three launches: histogram of the penalised logits, collection of the bins that hold the k best, final sort + draw.
int ptb_sample_logits(const float* logits, int V, int* history, int n_hist, int hist_cap, float repeat_penalty, float temperature, int top_k, float top_p, float u, void* scratch, int* out, int* ctrl_token, cudaStream_t st);

// ---------------------------------------------------------------------------- symm.cu
int ptb_symm_alloc(size_t bytes, void** ptr, void* handle64);

int ptb_symm_open(const void* handle64, void** ptr);

int ptb_symm_close(void* ptr);

int ptb_symm_free(void* ptr);

// Same-process variant (one process driving several GPUs, used by tests): enable peer access.
int ptb_enable_peer_access(int dev, int peer);

// ---------------------------------------------------------------------------- train_kernels.cu
int ptb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int H, float eps, const void* resid_in, void* resid_out, int bf16, cudaStream_t st);

// dw_partial: [n_ctas, H] fp32 scratch.
int ptb_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw, float* dw_partial, int n_ctas, long long rows, int H, const void* dresid, int bf16, cudaStream_t st);

int ptb_rope(const void* x, void* y, const float* cos, const float* sin, long long B, int T_, int heads, int D, int neox, int backward, int pos_offset, int bf16, cudaStream_t st);

int ptb_gated_act_fwd(const void* gu, void* out, long long rows, int I, int gelu, int bf16, cudaStream_t st);

int ptb_gated_act_bwd(const void* gu, const void* dout, void* dgu, long long rows, int I, int gelu, int bf16, cudaStream_t st);

// logits [rows, ld] (V valid columns), target int64 [rows]; loss fp32 [rows]; dlogits may alias logits or be null.
int ptb_xent(const void* logits, const long long* target, float* loss, float* lse, void* dlogits, long long rows, int V, long long ld, float grad_scale, long long ignore_index, int bf16, cudaStream_t st);

int ptb_rmsnorm_bwd_static(const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw, int n_ctas, long long rows, int H, const void* dresid, int bf16, cudaStream_t st);

#ifdef __cplusplus
}
#endif
