// C++ convenience layer over the C interface (ptb200.h): exceptions instead of return codes and RAII for the
// decode engine.  Header-only; link against libptb200.so.
#pragma once
#include <stdexcept>
#include <string>
#include <vector>

#include "ptb200.h"

namespace ptb200 {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// Throw if a library call failed; the message is the library's per-thread error string.
inline void check(int rc, const char* what) {
    if (rc != 0) {
        const char* m = ptb_last_error();
        throw Error(std::string(what) + ": " + (m && *m ? m : "failed"));
    }
}

// C = op(A) op(B)^T on the tcgen05 path (bf16 in, bf16 or fp32 out).  See ptb_gemm_bf16 for the operand conventions.
inline void gemm_bf16(const void* A, long long lda, bool a_mn, const void* B, long long ldb, bool b_mn, void* C, long long ldc, int M, int N,
                      int K, const float* bias, int flags, int* status, cudaStream_t st) {
    check(ptb_gemm_bf16(A, lda, a_mn ? 1 : 0, B, ldb, b_mn ? 1 : 0, C, ldc, M, N, K, bias, flags, status, 0, st), "gemm_bf16");
}

// One quantised decoder bound to the current device: owns the KV cache, the per-token CUDA graph and the control block.
class DecodeEngine {
public:
    DecodeEngine(const PtbModelDesc& model, const PtbLayerDesc* layers, cudaStream_t stream = nullptr)
        : h_(ptb_engine_create(&model, layers, (void*)stream)) {
        if (!h_) throw Error(std::string("engine: ") + ptb_last_error());
    }
    DecodeEngine(const DecodeEngine&) = delete;
    DecodeEngine& operator=(const DecodeEngine&) = delete;
    DecodeEngine(DecodeEngine&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    ~DecodeEngine() {
        if (h_) ptb_engine_destroy(h_);
    }

    void capture() { check(ptb_engine_capture(h_), "capture"); }
    // Serving step: {token, position} in from pinned memory, one token's kernels, the arg-max id back.
    int step(int token, int pos) {
        const int t = ptb_engine_step(h_, token, pos);
        if (t < 0) throw Error(std::string("step: ") + ptb_last_error());
        return t;
    }
    // Feed `prompt` from position pos0, then generate n_new tokens with the sampled id fed back on the device.
    std::vector<int> generate(const std::vector<int>& prompt, int n_new, int pos0 = 0) {
        check(ptb_engine_begin_script(h_, prompt.data(), (int)prompt.size(), pos0), "begin_script");
        check(ptb_engine_run(h_, (int)prompt.size() + n_new - 1), "run");
        std::vector<int> log(prompt.size() + n_new);
        const int steps = ptb_engine_read_log(h_, log.data(), (int)log.size());
        if (steps < 0) throw Error(std::string("read_log: ") + ptb_last_error());
        return std::vector<int>(log.begin() + (prompt.size() - 1), log.begin() + steps);
    }
    int status() const { return ptb_engine_status(h_); }
    float* logits() const { return (float*)ptb_engine_logits(h_); }
    float* hidden() const { return (float*)ptb_engine_hidden(h_); }
    cudaStream_t stream() const { return (cudaStream_t)ptb_engine_stream(h_); }
    void* handle() const { return h_; }

private:
    void* h_;
};

}  // namespace ptb200
