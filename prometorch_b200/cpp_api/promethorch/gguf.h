// promethorch C++ API: GGUF models on the native decode engine.
//
//   promethorch::io::gguf::GGUFReader   memory-mapped GGUF v2/v3 reader (metadata, tensor directory, raw blocks)
//   promethorch::io::GGUFModel          load(path) / forward_decode(token, pos) / generate(prompt ids, n) / run_prompt / sample
//
// GGUFModel is the C++ face of what the Python class of the same name does: parse the file, repack the quantised
// matrices into the decode kernels' streaming layout (tiles of 16 rows, csrc/decode_gemv_mma.cuh), upload them, and
// drive the engine of libptb200 (CUDA graph per token, arg-max fed back on the device).  The reference's counterpart is
// torch::io::GGUFModel (torch/io/gguf_model.h: load / forward_decode / generate).  This header covers dense decoder
// architectures with Q4_K / Q5_K / Q6_K / Q8_0 / F16 matrices (llama, mistral, qwen2, qwen3); other
// files go through the Python loader, which also transcodes the remaining block types.
//
// Link with libptb200.so and the CUDA runtime.  Needs no libtorch.
#pragma once
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../csrc/ptb200.h"
#include "gguf_reader.h"

namespace promethorch {
namespace io {

class GGUFModel {
 public:
    GGUFModel() = default;
    ~GGUFModel() { close(); }
    GGUFModel(const GGUFModel&) = delete;
    GGUFModel& operator=(const GGUFModel&) = delete;

    TransformerConfig config;

    // Parse, repack, upload and create the engine on the current CUDA device.
    // want_logits: keep the fp32 logits of every step on the device (needed by sample()).
    void load(const std::string& path, int max_seq = 4096, bool want_logits = false) {
        close();
        want_logits_ = want_logits;
        reader_.open(path);
        config.parse(reader_);
        max_seq_ = std::min(max_seq, config.context_length);
        const auto& c = config;
        std::vector<PtbLayerDesc> layers((size_t)c.num_layers);
        std::memset(layers.data(), 0, sizeof(PtbLayerDesc) * layers.size());
        rope_tables();
        for (int l = 0; l < c.num_layers; ++l) {
            const std::string p = "blk." + std::to_string(l) + ".";
            PtbLayerDesc& L = layers[(size_t)l];
            L.q = matrix(p + "attn_q.weight");
            L.k = matrix(p + "attn_k.weight");
            L.v = matrix(p + "attn_v.weight");
            L.o = matrix(p + "attn_output.weight");
            L.gate = matrix(p + "ffn_gate.weight");
            L.up = matrix(p + "ffn_up.weight");
            L.down = matrix(p + "ffn_down.weight");
            if (L.gate.qtype != L.up.qtype) throw std::runtime_error("GGUFModel: ffn_gate and ffn_up with different quantisation types");
            L.attn_norm = vector_f32(p + "attn_norm.weight");
            L.ffn_norm = vector_f32(p + "ffn_norm.weight");
            L.q_norm = reader_.has_tensor(p + "attn_q_norm.weight") ? vector_f32(p + "attn_q_norm.weight") : nullptr;
            L.k_norm = reader_.has_tensor(p + "attn_k_norm.weight") ? vector_f32(p + "attn_k_norm.weight") : nullptr;
            L.cos = cos_;
            L.sin = sin_;
        }
        PtbModelDesc m;
        std::memset(&m, 0, sizeof(m));
        m.n_layers = c.num_layers; m.hidden = c.hidden_size; m.n_heads = c.num_heads; m.n_kv_heads = c.num_kv_heads;
        m.head_dim = c.head_dim; m.inter = c.intermediate_size; m.vocab = c.vocab_size; m.max_seq = max_seq_;
        m.eps = (float)c.rms_norm_eps; m.emb_scale = 1.0f; m.neox = c.rope_neox ? 1 : 0;
        m.embed = table("token_embd.weight");
        m.lm_head = matrix(c.tie_word_embeddings ? "token_embd.weight" : "output.weight");
        m.out_norm = vector_f32("output_norm.weight");
        m.tp_rank = 0; m.tp_world = 1;
        m.want_logits = want_logits ? 1 : 0;
        check_cuda(cudaDeviceSynchronize(), "upload");
        engine_ = ptb_engine_create(&m, layers.data(), nullptr);
        if (!engine_) throw std::runtime_error(std::string("GGUFModel: ") + ptb_last_error());
    }
    void close() {
        if (engine_) ptb_engine_destroy(engine_);
        engine_ = nullptr;
        for (void* p : device_) cudaFree(p);
        device_.clear();
        captured_ = false;
        cos_ = sin_ = nullptr;
        samp_hist_ = samp_scratch_ = samp_out_ = nullptr;
        samp_n_hist_ = 0;
    }
    // One decode step fed from the host: returns the arg-max id of the next token.
    int forward_decode(int token, int pos) {
        ensure_captured();
        const int t = ptb_engine_step(engine_, token, pos);
        if (t < 0) throw std::runtime_error(std::string("forward_decode: ") + ptb_last_error());
        check_status();
        return t;
    }
    // Greedy generation: the prompt and n_new tokens as back-to-back graph replays, no host round trip in between.
    std::vector<int> generate(const std::vector<int>& prompt, int n_new) {
        if (prompt.empty()) throw std::runtime_error("generate: empty prompt");
        ensure_captured();
        if (ptb_engine_begin_script(engine_, prompt.data(), (int)prompt.size(), 0)) fail("begin_script");
        if (ptb_engine_run(engine_, (int)prompt.size() + n_new - 1)) fail("run");
        std::vector<int> log(prompt.size() + (size_t)n_new);
        const int steps = ptb_engine_read_log(engine_, log.data(), (int)log.size());
        if (steps < 0) fail("read_log");
        check_status();
        return std::vector<int>(log.begin() + (long)(prompt.size() - 1), log.begin() + std::min<long>(steps, (long)log.size()));
    }
    // The prompt as one scripted run (no host round trip between its tokens); returns the arg-max after its last token.
    int run_prompt(const std::vector<int>& prompt, int pos0 = 0) {
        if (prompt.empty()) throw std::runtime_error("run_prompt: empty prompt");
        if (pos0 + (int)prompt.size() + 1 > max_seq_) throw std::runtime_error("run_prompt: the prompt does not fit max_seq");
        ensure_captured();
        if (ptb_engine_begin_script(engine_, prompt.data(), (int)prompt.size(), pos0)) fail("begin_script");
        if (ptb_engine_run(engine_, (int)prompt.size())) fail("run");
        std::vector<int> log(prompt.size());
        if (ptb_engine_read_log(engine_, log.data(), (int)log.size()) < (int)log.size()) fail("read_log");
        check_status();
        return log.back();
    }
    // Device pointer to the fp32 logits of the last step ([vocab]); valid when loaded with want_logits.
    const float* logits() const { return want_logits_ ? (const float*)ptb_engine_logits(engine_) : nullptr; }
    // Start a sampled continuation: the ids that count for the repetition penalty, and the seed of the draws.
    void sampler_reset(const std::vector<int>& history, uint64_t seed = 42) {
        if (!want_logits_) throw std::runtime_error("sampling needs the model loaded with want_logits = true");
        if (!samp_hist_) {
            check_cuda(cudaMalloc(&samp_hist_, sizeof(int) * kHistCap), "cudaMalloc");
            const size_t sb = (size_t)ptb_sample_scratch_bytes(config.vocab_size);
            check_cuda(cudaMalloc(&samp_scratch_, sb), "cudaMalloc");
            check_cuda(cudaMemset(samp_scratch_, 0, sb), "cudaMemset");
            check_cuda(cudaMalloc(&samp_out_, 2 * sizeof(int)), "cudaMalloc");
            device_.push_back(samp_hist_);
            device_.push_back(samp_scratch_);
            device_.push_back(samp_out_);
        }
        const size_t n = std::min(history.size(), (size_t)kHistCap);
        if (n) check_cuda(cudaMemcpy(samp_hist_, history.data() + (history.size() - n), n * sizeof(int), cudaMemcpyHostToDevice), "cudaMemcpy");
        samp_n_hist_ = (int)n;
        rng_state_ = seed * 0x9E3779B97F4A7C15ull + 0xD1B54A32D192ED03ull;
    }
    // One draw from the logits of the last step on the device (penalty, temperature, top-k <= 64, top-p, inverse-CDF draw);
    // only the chosen id crosses to the host.  The id is appended to the penalty history.
    int sample(double temperature, int top_k, double top_p, double repeat_penalty) {
        if (!samp_hist_) sampler_reset({});
        top_k = top_k < 1 || top_k > 64 ? 64 : top_k;
        rng_state_ ^= rng_state_ << 13; rng_state_ ^= rng_state_ >> 7; rng_state_ ^= rng_state_ << 17;      // xorshift64
        const float u = (float)((rng_state_ >> 40) * (1.0 / 16777216.0));
        cudaStream_t st = (cudaStream_t)ptb_engine_stream(engine_);
        if (ptb_sample_logits(logits(), config.vocab_size, (int*)samp_hist_, samp_n_hist_, kHistCap, (float)repeat_penalty, (float)temperature, top_k,
                              (float)top_p, u, samp_scratch_, (int*)samp_out_, nullptr, st) < 0)
            fail("sample_logits");
        int host[2] = {0, 0};
        check_cuda(cudaMemcpyAsync(host, samp_out_, sizeof host, cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync");
        check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize");
        if (samp_n_hist_ < kHistCap) ++samp_n_hist_;
        return host[0];
    }
    // Phase stamps of the last token (PTB_TRACE=1 at load): [kernels][8] nanoseconds; returns the kernel count.
    int read_trace(unsigned long long* out, int max_kernels) { return ptb_engine_read_trace(engine_, out, max_kernels); }
    int max_seq() const { return max_seq_; }
    size_t weight_bytes() const { return weight_bytes_; }
    const gguf::GGUFReader& reader() const { return reader_; }

 private:
    static void check_cuda(cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string("GGUFModel: ") + what + ": " + cudaGetErrorString(e));
    }
    [[noreturn]] void fail(const char* what) { throw std::runtime_error(std::string(what) + ": " + ptb_last_error()); }
    void check_status() {
        const int s = ptb_engine_status(engine_);
        if (s != 0) throw std::runtime_error("GGUFModel: the decode engine reported status " + std::to_string(s));
    }
    void ensure_captured() {
        if (captured_) return;
        if (ptb_engine_set_ctrl(engine_, 0, 0, 0, 1) || ptb_engine_run(engine_, 1) || ptb_engine_sync(engine_)) fail("warm-up token");
        check_status();
        if (ptb_engine_capture(engine_)) fail("graph capture");
        captured_ = true;
    }
    void* upload(const void* host, size_t n) {
        void* d = nullptr;
        check_cuda(cudaMalloc(&d, n), "cudaMalloc");
        check_cuda(cudaMemcpy(d, host, n, cudaMemcpyHostToDevice), "cudaMemcpy");
        device_.push_back(d);
        return d;
    }
    const float* vector_f32(const std::string& name) {
        const auto& t = reader_.tensor(name);
        if (t.type != gguf::F32) throw std::runtime_error("GGUFModel: " + name + " is expected to be F32");
        return (const float*)upload(reader_.data(t), t.nbytes);
    }
    // A matrix in the tiles-of-16-rows streaming layout (csrc/decode_gemv_mma.cuh): Q4_K / Q5_K blocks as in the file,
    // Q6_K split into swizzled arrays, Q8_0 as q[16][256] (32-byte units at unit ^ (row & 7)) + d[16][8], F16 in blocks of
    // 64 values (32-byte units at unit ^ (row & 3)).
    PtbWeightDesc matrix(const std::string& name) {
        const auto& t = reader_.tensor(name);
        int qt, bb;              // engine type code, bytes of one (tile, 256-value block) unit / 16
        switch (t.type) {
            case gguf::Q4_K: qt = 0; bb = 144; break;
            case gguf::Q6_K: qt = 1; bb = 210; break;
            case gguf::Q5_K: qt = 4; bb = 176; break;
            case gguf::Q8_0: qt = 5; bb = 272; break;
            case gguf::F16: qt = 2; bb = 512; break;
            default:
                throw std::runtime_error("GGUFModel (C++): " + name + " has block type " + std::to_string(t.type) +
                                         "; Q4_K, Q5_K, Q6_K, Q8_0 and F16 are handled here");
        }
        const int rows = (int)t.shape[0], cols = (int)t.shape[1], nblk = cols / 256;
        if (cols % 256) throw std::runtime_error("GGUFModel: " + name + ": row length must be a multiple of 256");
        const int ntile = (rows + 15) / 16;
        std::vector<uint8_t> out((size_t)ntile * nblk * 16 * bb, 0);
        const uint8_t* src = reader_.data(t);
        for (int r = 0; r < rows; ++r) {
            const int tile = r >> 4, rr = r & 15;
            for (int b = 0; b < nblk; ++b) {
                const uint8_t* blk = src + ((size_t)r * nblk + b) * bb;          // the row's bytes for these 256 values
                uint8_t* unit = out.data() + ((size_t)tile * nblk + b) * 16 * bb;
                switch (t.type) {
                    case gguf::Q4_K: std::memcpy(unit + rr * 144, blk, 144); break;
                    case gguf::Q5_K: std::memcpy(unit + rr * 176, blk, 176); break;
                    case gguf::Q8_0:
                        for (int u = 0; u < 8; ++u) {                             // eight {fp16 d, 32 x int8} file blocks
                            std::memcpy(unit + rr * 256 + ((u ^ (rr & 7)) << 5), blk + u * 34 + 2, 32);
                            std::memcpy(unit + 4096 + rr * 16 + u * 2, blk + u * 34, 2);
                        }
                        break;
                    case gguf::F16:
                        for (int q = 0; q < 4; ++q)                               // four 64-value blocks of 2048 bytes
                            for (int u = 0; u < 4; ++u)
                                std::memcpy(unit + q * 2048 + rr * 128 + ((u ^ (rr & 3)) << 5), blk + q * 128 + u * 32, 32);
                        break;
                    default:
                        // ql[16][128] | qh[16][64] | scales[16][16] | d[16]; 16-byte chunks of a row stored at chunk ^ key(row)
                        for (int ch = 0; ch < 8; ++ch) std::memcpy(unit + rr * 128 + ((ch ^ (rr & 7)) << 4), blk + ch * 16, 16);
                        for (int ch = 0; ch < 4; ++ch) std::memcpy(unit + 2048 + rr * 64 + ((ch ^ ((rr >> 1) & 3)) << 4), blk + 128 + ch * 16, 16);
                        std::memcpy(unit + 3072 + rr * 16, blk + 192, 16);
                        std::memcpy(unit + 3328 + rr * 2, blk + 208, 2);
                        break;
                }
            }
        }
        PtbWeightDesc d;
        std::memset(&d, 0, sizeof(d));
        d.w = upload(out.data(), out.size());
        d.qtype = qt;
        d.rows = rows;
        d.cols = cols;
        d.layout = 1;
        weight_bytes_ += out.size();
        return d;
    }
    // Row-major rows for look-ups (the embedding): Q4_K as in the file; Q6_K rows as ql | qh | scales | d(+pad to 16).
    PtbWeightDesc table(const std::string& name) {
        const auto& t = reader_.tensor(name);
        const int rows = (int)t.shape[0], cols = (int)t.shape[1], nblk = cols / 256;
        PtbWeightDesc d;
        std::memset(&d, 0, sizeof(d));
        d.rows = rows;
        d.cols = cols;
        const uint8_t* src = reader_.data(t);
        if (t.type == gguf::Q4_K) {
            d.qtype = 0;
            d.rowbytes = nblk * 144;
            d.w = upload(src, (size_t)rows * d.rowbytes);
        } else if (t.type == gguf::Q6_K) {
            const int pad = (16 - (nblk * 2) % 16) % 16;
            d.qtype = 1;
            d.rowbytes = nblk * 210 + pad;
            std::vector<uint8_t> out((size_t)rows * d.rowbytes, 0);
            for (int r = 0; r < rows; ++r)
                for (int b = 0; b < nblk; ++b) {
                    const uint8_t* blk = src + ((size_t)r * nblk + b) * 210;
                    uint8_t* row = out.data() + (size_t)r * d.rowbytes;
                    std::memcpy(row + b * 128, blk, 128);
                    std::memcpy(row + nblk * 128 + b * 64, blk + 128, 64);
                    std::memcpy(row + nblk * 192 + b * 16, blk + 192, 16);
                    std::memcpy(row + nblk * 208 + b * 2, blk + 208, 2);
                }
            d.w = upload(out.data(), out.size());
        } else if (t.type == gguf::F16 || t.type == gguf::F32) {
            d.qtype = t.type == gguf::F16 ? 2 : 3;
            d.rowbytes = cols * (t.type == gguf::F16 ? 2 : 4);
            d.w = upload(src, (size_t)rows * d.rowbytes);
        } else if (t.type == gguf::Q8_0 || t.type == gguf::Q5_K) {
            // other block types become an fp16 table, as in the Python loader (rows are looked up one at a time)
            std::vector<float> out((size_t)rows * cols);
            for (int r = 0; r < rows; ++r) {
                float* y = out.data() + (size_t)r * cols;
                if (t.type == gguf::Q8_0) {
                    const uint8_t* row = src + (size_t)r * (cols / 32) * 34;
                    for (int b = 0; b < cols / 32; ++b) {
                        const float dd = half_to_float(row + b * 34);
                        const int8_t* q = (const int8_t*)(row + b * 34 + 2);
                        for (int i = 0; i < 32; ++i) y[b * 32 + i] = dd * (float)q[i];
                    }
                } else {
                    const uint8_t* row = src + (size_t)r * nblk * 176;
                    for (int b = 0; b < nblk; ++b) {
                        const uint8_t* blk = row + b * 176;
                        const float dd = half_to_float(blk), dmin = half_to_float(blk + 2);
                        const uint8_t *sc = blk + 4, *qh = blk + 16, *qs = blk + 48;
                        for (int is = 0; is < 8; ++is) {          // sub-block of 32 values: 6-bit scale and minimum
                            int scv, mv;
                            if (is < 4) { scv = sc[is] & 63; mv = sc[is + 4] & 63; }
                            else { scv = (sc[is + 4] & 0xF) | ((sc[is - 4] >> 6) << 4); mv = (sc[is + 4] >> 4) | ((sc[is] >> 6) << 4); }
                            for (int l = 0; l < 32; ++l) {
                                const uint8_t qb = qs[(is >> 1) * 32 + l];
                                const int q = ((is & 1) ? (qb >> 4) : (qb & 0xF)) | (((qh[l] >> is) & 1) << 4);
                                y[b * 256 + is * 32 + l] = dd * scv * q - dmin * mv;
                            }
                        }
                    }
                }
            }
            std::vector<uint16_t> h(out.size());
            for (size_t i = 0; i < out.size(); ++i) h[i] = float_to_half(out[i]);
            d.qtype = 2;
            d.rowbytes = cols * 2;
            d.w = upload(h.data(), h.size() * 2);
        } else {
            throw std::runtime_error("GGUFModel (C++): embedding table of block type " + std::to_string(t.type) + " is not handled here");
        }
        return d;
    }
    static uint16_t float_to_half(float f) {          // round to nearest even, like torch's conversion
        uint32_t x;
        std::memcpy(&x, &f, 4);
        const uint32_t sign = (x >> 16) & 0x8000u;
        x &= 0x7FFFFFFFu;
        if (x >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (x > 0x7F800000u ? 0x200u : 0u));
        if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);                     // rounds to infinity
        if (x < 0x38800000u) {                                                       // subnormal half or zero
            if (x < 0x33000000u) return (uint16_t)sign;
            const int e = (int)(x >> 23);
            uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
            const int shift = 126 - e;                                               // 14 .. 24
            uint32_t hm = m >> shift;
            const uint32_t rem = m & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
            if (rem > halfway || (rem == halfway && (hm & 1u))) ++hm;
            return (uint16_t)(sign | hm);
        }
        uint32_t hm = ((x - 0x38000000u) >> 13);
        const uint32_t rem = x & 0x1FFFu;
        if (rem > 0x1000u || (rem == 0x1000u && (hm & 1u))) ++hm;
        return (uint16_t)(sign | hm);
    }
    static float half_to_float(const uint8_t* p) {
        uint16_t h;
        std::memcpy(&h, p, 2);
        const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FFu;
        uint32_t bits;
        if (exp == 0) {
            if (man == 0) bits = sign;
            else {                                    // subnormal: normalise
                int e = -1;
                uint32_t m = man;
                do { ++e; m <<= 1; } while (!(m & 0x400u));
                bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FFu) << 13);
            }
        } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
        else bits = sign | ((exp + 112) << 23) | (man << 13);
        float f;
        std::memcpy(&f, &bits, 4);
        return f;
    }
    void rope_tables() {
        const int half = config.head_dim / 2;
        std::vector<float> c((size_t)max_seq_ * half), s((size_t)max_seq_ * half);
        for (int i = 0; i < half; ++i) {
            const double inv = std::pow(config.rope_freq_base, -2.0 * i / config.head_dim);
            for (int p = 0; p < max_seq_; ++p) {
                c[(size_t)p * half + i] = (float)std::cos(p * inv);
                s[(size_t)p * half + i] = (float)std::sin(p * inv);
            }
        }
        cos_ = (const float*)upload(c.data(), c.size() * 4);
        sin_ = (const float*)upload(s.data(), s.size() * 4);
    }

    gguf::GGUFReader reader_;
    void* engine_ = nullptr;
    std::vector<void*> device_;
    const float *cos_ = nullptr, *sin_ = nullptr;
    int max_seq_ = 0;
    bool captured_ = false, want_logits_ = false;
    size_t weight_bytes_ = 0;
    static constexpr int kHistCap = 1 << 16;
    void *samp_hist_ = nullptr, *samp_scratch_ = nullptr, *samp_out_ = nullptr;
    int samp_n_hist_ = 0;
    uint64_t rng_state_ = 42;
};

}  // namespace io
}  // namespace promethorch
