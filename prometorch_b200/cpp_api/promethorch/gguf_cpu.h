// promethorch C++ API: a GGUF decoder on the CPU (no CUDA, no libtorch), and the server backend over it.
//
//   io::GGUFCpuModel     load(path) / forward(token, pos) -> logits / generate(prompt, n): fp32 math over the quantised
//                        blocks of the file (dequantised on the fly, row by row, from the memory map), fp16-rounded
//                        key / value cache, rows of every projection spread over the machine's threads.  `path` may also
//                        be a Hugging Face directory (config.json + *.safetensors in F32 / F16 / BF16, sharded or not):
//                        the tensors are read in place from the mapped files under their Hugging Face names
//   serve::CpuBackend    ModelBackend (serve.h) = GGUFCpuModel + the file's (or the directory's) tokenizer + sampling on the host
//
// This is the reference path of the native programs (`--device cpu`): the same computation as the fp32 oracle of the Python
// package (models/gguf_oracle.py) and as the reference's CPU decode (torch/io/gguf_model.h:7300-7340), for checking and for
// machines without a GPU; it is not fast.  Dense decoders only (llama, mistral, qwen2, qwen3) with F32 / F16 / BF16 / Q4_0 /
// Q8_0 / Q2_K / Q3_K / Q4_K / Q5_K / Q6_K tensors.
#pragma once
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <condition_variable>
#include <random>
#include <set>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

#include "gguf_reader.h"
#include "model_loader.h"
#include "serve.h"
#include "tokenizer.h"

namespace promethorch {
namespace io {

namespace cpu_detail {
inline float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FF;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            uint32_t m = man;
            do { ++e; m <<= 1; } while (!(m & 0x400));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FF) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}
// Round to the nearest half and back (what an fp16 key / value cache keeps).
inline float round_to_half(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000;
    const int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t man = x & 0x7FFFFF;
    uint16_t h;
    if (((x >> 23) & 0xFF) == 0xFF) h = (uint16_t)(sign | 0x7C00 | (man ? 0x200 : 0));
    else if (exp >= 31) h = (uint16_t)(sign | 0x7C00);
    else if (exp <= 0) {
        if (exp < -10) h = (uint16_t)sign;
        else {
            man |= 0x800000;
            const int shift = 14 - exp;
            uint32_t v = man >> shift;
            const uint32_t rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
            if (rem > halfway || (rem == halfway && (v & 1))) ++v;
            h = (uint16_t)(sign | v);
        }
    } else {
        uint32_t v = ((uint32_t)exp << 10) | (man >> 13);
        const uint32_t rem = man & 0x1FFF;
        if (rem > 0x1000 || (rem == 0x1000 && (v & 1))) ++v;
        h = (uint16_t)(sign | v);
    }
    return half_to_float(h);
}
inline uint16_t rd16(const uint8_t* p) { uint16_t v; std::memcpy(&v, p, 2); return v; }
inline void scale_min_k4(int j, const uint8_t* q, int& sc, int& m) {
    if (j < 4) { sc = q[j] & 63; m = q[j + 4] & 63; }
    else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}
// One block of `type` at `p` -> its values in `y`; returns the number of values.
inline int dequant_block(uint32_t type, const uint8_t* p, float* y) {
    switch (type) {
        case gguf::F32: std::memcpy(y, p, 4); return 1;
        case gguf::F16: y[0] = half_to_float(rd16(p)); return 1;
        case gguf::BF16: { uint32_t b = (uint32_t)rd16(p) << 16; std::memcpy(y, &b, 4); return 1; }
        case gguf::Q8_0: {
            const float d = half_to_float(rd16(p));
            const int8_t* q = (const int8_t*)(p + 2);
            for (int i = 0; i < 32; ++i) y[i] = d * q[i];
            return 32;
        }
        case gguf::Q4_0: {                                   // fp16 d | 16 bytes: low nibbles are values 0-15, high nibbles 16-31, stored plus 8
            const float d = half_to_float(rd16(p));
            for (int i = 0; i < 16; ++i) { y[i] = d * ((int)(p[2 + i] & 0xF) - 8); y[i + 16] = d * ((int)(p[2 + i] >> 4) - 8); }
            return 32;
        }
        case gguf::Q2_K: {                                   // scales[16] (low nibble scale, high nibble min, per 16 values) | qs[64] | fp16 d | fp16 dmin
            const uint8_t *sc = p, *qs = p + 16;
            const float d = half_to_float(rd16(p + 80)), dmin = half_to_float(rd16(p + 82));
            for (int half = 0; half < 2; ++half)             // 128 values use 32 bytes; the four bit planes give 32 values each
                for (int plane = 0; plane < 4; ++plane)
                    for (int l = 0; l < 32; ++l) {
                        const int idx = half * 128 + plane * 32 + l, grp = idx / 16;
                        const int q = (qs[half * 32 + l] >> (2 * plane)) & 3;
                        y[idx] = d * (float)(sc[grp] & 0xF) * (float)q - dmin * (float)(sc[grp] >> 4);
                    }
            return 256;
        }
        case gguf::Q3_K: {                                   // hmask[32] | qs[64] (low two bits, planes as in Q2_K) | scales[12] (sixteen 6-bit, minus 32) | fp16 d
            const uint8_t *hm = p, *qs = p + 32, *sr = p + 96;
            const float d = half_to_float(rd16(p + 108));
            int scales[16];
            for (int j = 0; j < 16; ++j) {
                const int lo = j < 8 ? (sr[j] & 0xF) : (sr[j - 8] >> 4);
                const int hi = (sr[8 + (j % 4)] >> (2 * (j / 4))) & 3;
                scales[j] = (lo | (hi << 4)) - 32;
            }
            for (int half = 0; half < 2; ++half)
                for (int plane = 0; plane < 4; ++plane)
                    for (int l = 0; l < 32; ++l) {
                        const int idx = half * 128 + plane * 32 + l;
                        const int low2 = (qs[half * 32 + l] >> (2 * plane)) & 3;
                        const int high = (hm[l] >> (half * 4 + plane)) & 1;
                        y[idx] = d * (float)scales[idx / 16] * (float)(low2 - (high ? 0 : 4));
                    }
            return 256;
        }
        case gguf::Q4_K: {
            const float d = half_to_float(rd16(p)), dmin = half_to_float(rd16(p + 2));
            const uint8_t *scales = p + 4, *q = p + 16;
            for (int c = 0; c < 4; ++c, q += 32, y += 64) {
                int s1, m1, s2, m2;
                scale_min_k4(2 * c, scales, s1, m1);
                scale_min_k4(2 * c + 1, scales, s2, m2);
                for (int l = 0; l < 32; ++l) {
                    y[l] = d * s1 * (q[l] & 0xF) - dmin * m1;
                    y[l + 32] = d * s2 * (q[l] >> 4) - dmin * m2;
                }
            }
            return 256;
        }
        case gguf::Q5_K: {
            const float d = half_to_float(rd16(p)), dmin = half_to_float(rd16(p + 2));
            const uint8_t *scales = p + 4, *qh = p + 16, *q = p + 48;
            for (int c = 0; c < 4; ++c, q += 32, y += 64) {
                int s1, m1, s2, m2;
                scale_min_k4(2 * c, scales, s1, m1);
                scale_min_k4(2 * c + 1, scales, s2, m2);
                const int u1 = 1 << (2 * c), u2 = 2 << (2 * c);
                for (int l = 0; l < 32; ++l) {
                    y[l] = d * s1 * ((q[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - dmin * m1;
                    y[l + 32] = d * s2 * ((q[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - dmin * m2;
                }
            }
            return 256;
        }
        case gguf::Q6_K: {
            const uint8_t *ql = p, *qh = p + 128;
            const int8_t* sc = (const int8_t*)(p + 192);
            const float d = half_to_float(rd16(p + 208));
            for (int n = 0; n < 2; ++n, y += 128, ql += 64, qh += 32, sc += 8)
                for (int l = 0; l < 32; ++l) {
                    const int is = l / 16;
                    const int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32, q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32, q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                    y[l] = d * sc[is] * q1;
                    y[l + 32] = d * sc[is + 2] * q2;
                    y[l + 64] = d * sc[is + 4] * q3;
                    y[l + 96] = d * sc[is + 6] * q4;
                }
            return 256;
        }
        default: throw std::runtime_error("GGUFCpuModel: tensor type " + std::to_string(type) + " is not supported on this path");
    }
}
// Rows [r0, r1) of y = M x for block-quantised rows: each block is dequantised into a small buffer and multiplied into sixteen
// running sums (a form the compiler turns into vector code), blocks are added up in double.  Compiled twice on x86-64 (AVX2 + FMA
// and baseline) and picked at load time by the CPU's features; sanitizer builds keep the single baseline version.
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__) && !defined(__SANITIZE_THREAD__) && !defined(__SANITIZE_ADDRESS__)
#define PROMETHORCH_CPU_CLONES __attribute__((target_clones("arch=haswell", "default")))
#else
#define PROMETHORCH_CPU_CLONES
#endif
PROMETHORCH_CPU_CLONES
static void block_rows(const uint8_t* data, uint32_t type, size_t row_bytes, int cols, int block_elems, int block_bytes, const float* x, float* y, int r0, int r1) {
    float tmp[256];
    for (int r = r0; r < r1; ++r) {
        const uint8_t* p = data + (size_t)r * row_bytes;
        double acc = 0;
        for (int c = 0; c < cols; c += block_elems, p += block_bytes) {
            const int n = dequant_block(type, p, tmp);            // 32 or 256 values
            float lane[16] = {0};
            for (int i = 0; i < n; i += 16)
                for (int j = 0; j < 16; ++j) lane[j] += tmp[i + j] * x[c + i + j];
            float part = 0;
            for (int j = 0; j < 16; ++j) part += lane[j];
            acc += part;
        }
        y[r] = (float)acc;
    }
}

// A fixed set of worker threads that run the parts of one job at a time; the caller works too and returns when every part is done.
class Pool {
 public:
    explicit Pool(int n) {
        for (int i = 1; i < n; ++i) ts_.emplace_back([this] { loop(); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> l(m_);
            stop_ = true;
            ++gen_;
        }
        cv_.notify_all();
        for (auto& t : ts_) t.join();
    }
    Pool(const Pool&) = delete;
    Pool& operator=(const Pool&) = delete;
    void run(int parts, const std::function<void(int)>& fn) {
        {
            std::lock_guard<std::mutex> l(m_);
            fn_ = &fn;
            parts_ = parts;
            next_ = 0;
            pending_ = parts;
            ++gen_;
        }
        cv_.notify_all();
        drain();
        std::unique_lock<std::mutex> l(m_);
        done_.wait(l, [&] { return pending_ == 0; });
        fn_ = nullptr;
    }

 private:
    void drain() {
        for (;;) {
            int part;
            const std::function<void(int)>* fn;
            {
                std::lock_guard<std::mutex> l(m_);
                if (!fn_ || next_ >= parts_) return;
                part = next_++;
                fn = fn_;
            }
            (*fn)(part);
            std::lock_guard<std::mutex> l(m_);
            if (--pending_ == 0) done_.notify_all();
        }
    }
    void loop() {
        unsigned long long seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> l(m_);
                cv_.wait(l, [&] { return gen_ != seen; });
                seen = gen_;
                if (stop_) return;
            }
            drain();
        }
    }
    std::vector<std::thread> ts_;
    std::mutex m_;
    std::condition_variable cv_, done_;
    const std::function<void(int)>* fn_ = nullptr;
    int parts_ = 0, next_ = 0, pending_ = 0;
    unsigned long long gen_ = 0;
    bool stop_ = false;
};
}  // namespace cpu_detail

class GGUFCpuModel {
 public:
    TransformerConfig config;

    void load(const std::string& path, int max_seq = 4096, int threads = 0) {
        threads_ = threads > 0 ? threads : (int)std::max(1u, std::thread::hardware_concurrency());
        if (loader::detail::is_dir(path) || loader::detect_format(path) == "safetensors") { load_hf(path, max_seq); return; }
        reader_.open(path);
        config.parse(reader_);
        max_seq_ = std::min(max_seq, config.context_length);
        const auto& c = config;
        layers_.assign((size_t)c.num_layers, Layer());
        for (int l = 0; l < c.num_layers; ++l) {
            const std::string p = "blk." + std::to_string(l) + ".";
            Layer& L = layers_[(size_t)l];
            L.q = mat(p + "attn_q.weight"); L.k = mat(p + "attn_k.weight"); L.v = mat(p + "attn_v.weight"); L.o = mat(p + "attn_output.weight");
            L.gate = mat(p + "ffn_gate.weight"); L.up = mat(p + "ffn_up.weight"); L.down = mat(p + "ffn_down.weight");
            L.attn_norm = vec(p + "attn_norm.weight"); L.ffn_norm = vec(p + "ffn_norm.weight");
            if (reader_.has_tensor(p + "attn_q_norm.weight")) { L.q_norm = vec(p + "attn_q_norm.weight"); L.k_norm = vec(p + "attn_k_norm.weight"); }
            for (const char* b : {"attn_q.bias", "attn_k.bias", "attn_v.bias"})
                if (reader_.has_tensor(p + b)) (std::string(b) == "attn_q.bias" ? L.qb : (std::string(b) == "attn_k.bias" ? L.kb : L.vb)) = vec(p + b);
            L.kc.assign((size_t)max_seq_ * c.num_kv_heads * c.head_dim, 0.f);
            L.vc.assign((size_t)max_seq_ * c.num_kv_heads * c.head_dim, 0.f);
        }
        embed_ = mat("token_embd.weight");
        head_ = c.tie_word_embeddings ? embed_ : mat("output.weight");
        out_norm_ = vec("output_norm.weight");
        finish_load();
    }
    int max_seq() const { return max_seq_; }
    bool from_hf() const { return !hf_.tensors.empty(); }
    const gguf::GGUFReader& reader() const { return reader_; }                 // of a GGUF file (empty for a Hugging Face directory)
    const loader::ModelWeights& hf_weights() const { return hf_; }             // of a Hugging Face directory (empty for a GGUF file)

    // One token at position `pos` (positions must be fed in order from 0): the logits of the next token.  With want_logits false the
    // output projection is skipped and the returned vector is stale: for prompt tokens before the last.
    const std::vector<float>& forward(int token, int pos, bool want_logits = true) {
        const auto& c = config;
        if (pos < 0 || pos >= max_seq_) throw std::runtime_error("GGUFCpuModel: position outside the cache");
        if (token < 0 || token >= c.vocab_size) throw std::runtime_error("GGUFCpuModel: token id outside the vocabulary");
        const int D = c.hidden_size, H = c.num_heads, Hk = c.num_kv_heads, Dh = c.head_dim, I = c.intermediate_size, half = Dh / 2, g = H / Hk;
        std::vector<float> x((size_t)D), h((size_t)D), q((size_t)H * Dh), k((size_t)Hk * Dh), v((size_t)Hk * Dh), att((size_t)H * Dh), o((size_t)D),
            gate((size_t)I), up((size_t)I), dn((size_t)D);
        row(embed_, token, x.data());
        for (auto& L : layers_) {
            rms(x.data(), L.attn_norm.data(), h.data(), D);
            matvec(L.q, h.data(), q.data());
            matvec(L.k, h.data(), k.data());
            matvec(L.v, h.data(), v.data());
            if (!L.qb.empty()) for (int i = 0; i < H * Dh; ++i) q[(size_t)i] += L.qb[(size_t)i];
            if (!L.kb.empty()) for (int i = 0; i < Hk * Dh; ++i) { k[(size_t)i] += L.kb[(size_t)i]; v[(size_t)i] += L.vb[(size_t)i]; }
            if (!L.q_norm.empty()) {
                for (int hh = 0; hh < H; ++hh) rms(&q[(size_t)hh * Dh], L.q_norm.data(), &q[(size_t)hh * Dh], Dh);
                for (int hh = 0; hh < Hk; ++hh) rms(&k[(size_t)hh * Dh], L.k_norm.data(), &k[(size_t)hh * Dh], Dh);
            }
            for (int hh = 0; hh < H; ++hh) rope(&q[(size_t)hh * Dh], pos, half);
            for (int hh = 0; hh < Hk; ++hh) rope(&k[(size_t)hh * Dh], pos, half);
            float* kc = &L.kc[(size_t)pos * Hk * Dh];
            float* vc = &L.vc[(size_t)pos * Hk * Dh];
            for (int i = 0; i < Hk * Dh; ++i) { kc[i] = cpu_detail::round_to_half(k[(size_t)i]); vc[i] = cpu_detail::round_to_half(v[(size_t)i]); }
            const float scale = 1.0f / std::sqrt((float)Dh);
            std::vector<float> s((size_t)pos + 1);
            for (int hh = 0; hh < H; ++hh) {
                const int kh = hh / g;
                float mx = -INFINITY;
                for (int t = 0; t <= pos; ++t) {
                    const float* kt = &L.kc[((size_t)t * Hk + kh) * Dh];
                    float d = 0;
                    for (int i = 0; i < Dh; ++i) d += q[(size_t)hh * Dh + i] * kt[i];
                    s[(size_t)t] = d * scale;
                    mx = std::max(mx, s[(size_t)t]);
                }
                float z = 0;
                for (int t = 0; t <= pos; ++t) { s[(size_t)t] = std::exp(s[(size_t)t] - mx); z += s[(size_t)t]; }
                float* a = &att[(size_t)hh * Dh];
                std::fill(a, a + Dh, 0.f);
                for (int t = 0; t <= pos; ++t) {
                    const float w = s[(size_t)t] / z;
                    const float* vt = &L.vc[((size_t)t * Hk + kh) * Dh];
                    for (int i = 0; i < Dh; ++i) a[i] += w * vt[i];
                }
            }
            matvec(L.o, att.data(), o.data());
            for (int i = 0; i < D; ++i) x[(size_t)i] += o[(size_t)i];
            rms(x.data(), L.ffn_norm.data(), h.data(), D);
            matvec(L.gate, h.data(), gate.data());
            matvec(L.up, h.data(), up.data());
            for (int i = 0; i < I; ++i) gate[(size_t)i] = gate[(size_t)i] / (1.0f + std::exp(-gate[(size_t)i])) * up[(size_t)i];
            matvec(L.down, gate.data(), dn.data());
            for (int i = 0; i < D; ++i) x[(size_t)i] += dn[(size_t)i];
        }
        if (!want_logits) return logits_;                       // a prompt token that is not the last: only its keys and values are needed
        rms(x.data(), out_norm_.data(), h.data(), D);
        matvec(head_, h.data(), logits_.data());
        return logits_;
    }
    int argmax() const { return (int)(std::max_element(logits_.begin(), logits_.end()) - logits_.begin()); }
    // Greedy continuation of `prompt` (the arg-max after every step).
    std::vector<int> generate(const std::vector<int>& prompt, int n_new) {
        std::vector<int> out;
        int pos = 0;
        for (size_t i = 0; i < prompt.size(); ++i, ++pos) forward(prompt[i], pos, i + 1 == prompt.size());
        for (int i = 0; i < n_new && pos < max_seq_; ++i) {
            const int t = argmax();
            out.push_back(t);
            if (i + 1 < n_new) forward(t, pos++);
        }
        return out;
    }

 private:
    struct Matrix { const uint8_t* data = nullptr; uint32_t type = 0; int rows = 0, cols = 0, block_elems = 1, block_bytes = 4; size_t row_bytes = 0; };
    struct Layer {
        Matrix q, k, v, o, gate, up, down;
        std::vector<float> attn_norm, ffn_norm, q_norm, k_norm, qb, kb, vb, kc, vc;
    };
    // A read-only mapping of one weight file of a Hugging Face directory.
    struct Mapped {
        const uint8_t* base = nullptr;
        size_t size = 0;
        Mapped() = default;
        Mapped(const Mapped&) = delete;
        Mapped& operator=(const Mapped&) = delete;
        ~Mapped() { if (base) ::munmap((void*)base, size); }
        void open(const std::string& path) {
            const int fd = ::open(path.c_str(), O_RDONLY);
            if (fd < 0) throw std::runtime_error("GGUFCpuModel: cannot open " + path);
            struct stat st;
            if (::fstat(fd, &st) != 0 || st.st_size <= 0) { ::close(fd); throw std::runtime_error("GGUFCpuModel: cannot size " + path); }
            size = (size_t)st.st_size;
            void* p = ::mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
            ::close(fd);
            if (p == MAP_FAILED) throw std::runtime_error("GGUFCpuModel: mmap failed for " + path);
            base = (const uint8_t*)p;
        }
    };
    void finish_load() {
        const auto& c = config;
        const int half = c.head_dim / 2;
        cos_.assign((size_t)max_seq_ * half, 0.f);
        sin_.assign((size_t)max_seq_ * half, 0.f);
        for (int i = 0; i < half; ++i) {
            const double inv = std::pow(c.rope_freq_base, -2.0 * i / c.head_dim);
            for (int p = 0; p < max_seq_; ++p) { cos_[(size_t)p * half + i] = (float)std::cos(p * inv); sin_[(size_t)p * half + i] = (float)std::sin(p * inv); }
        }
        logits_.assign((size_t)c.vocab_size, 0.f);
        pool_.reset(threads_ > 1 ? new cpu_detail::Pool(threads_) : nullptr);
    }
    // A Hugging Face directory (or one .safetensors file beside its config.json): Llama-family names
    // (model.layers.N.self_attn.q_proj.weight ...), rotary halves split as in the checkpoint (first half / second half).
    void load_hf(const std::string& path, int max_seq) {
        hf_ = loader::load_model(path);
        const loader::ModelConfig& m = hf_.config;
        const std::string& a = hf_.architecture;
        if (!(a == "llama" || a == "mistral" || a == "qwen2" || a == "qwen3"))
            throw std::runtime_error("GGUFCpuModel: architecture '" + a + "' of " + path + " is not a dense Llama-family decoder");
        pre_ = hf_.tensors.count("model.embed_tokens.weight") ? "model." : "";
        if (!hf_.tensors.count(pre_ + "embed_tokens.weight")) throw std::runtime_error("GGUFCpuModel: no embed_tokens.weight in " + path);
        config.architecture = a;
        config.hidden_size = (int)m.hidden_size; config.num_layers = (int)m.num_layers; config.num_heads = (int)m.num_heads;
        config.num_kv_heads = (int)(m.num_kv_heads ? m.num_kv_heads : m.num_heads); config.intermediate_size = (int)m.intermediate_size;
        config.head_dim = (int)(m.head_dim ? m.head_dim : m.hidden_size / std::max<int64_t>(m.num_heads, 1));
        config.context_length = m.context_length > 0 ? (int)m.context_length : 8192;
        config.rope_freq_base = m.rope_freq_base; config.rms_norm_eps = m.rms_norm_eps;
        config.vocab_size = (int)hf_.tensors.at(pre_ + "embed_tokens.weight").shape.at(0);
        config.tie_word_embeddings = !hf_.tensors.count("lm_head.weight");
        config.rope_neox = true;
        config.has_qk_norm = hf_.tensors.count(pre_ + "layers.0.self_attn.q_norm.weight") > 0;
        if (config.hidden_size <= 0 || config.num_layers <= 0 || config.num_heads <= 0 || config.intermediate_size <= 0)
            throw std::runtime_error("GGUFCpuModel: " + path + " has no usable config.json");
        max_seq_ = std::min(max_seq, config.context_length);
        const auto& c = config;
        layers_.assign((size_t)c.num_layers, Layer());
        for (int l = 0; l < c.num_layers; ++l) {
            const std::string p = pre_ + "layers." + std::to_string(l) + ".";
            Layer& L = layers_[(size_t)l];
            L.q = hf_mat(p + "self_attn.q_proj.weight"); L.k = hf_mat(p + "self_attn.k_proj.weight"); L.v = hf_mat(p + "self_attn.v_proj.weight");
            L.o = hf_mat(p + "self_attn.o_proj.weight");
            L.gate = hf_mat(p + "mlp.gate_proj.weight"); L.up = hf_mat(p + "mlp.up_proj.weight"); L.down = hf_mat(p + "mlp.down_proj.weight");
            L.attn_norm = hf_vec(p + "input_layernorm.weight"); L.ffn_norm = hf_vec(p + "post_attention_layernorm.weight");
            if (c.has_qk_norm) { L.q_norm = hf_vec(p + "self_attn.q_norm.weight"); L.k_norm = hf_vec(p + "self_attn.k_norm.weight"); }
            if (hf_.tensors.count(p + "self_attn.q_proj.bias")) {
                L.qb = hf_vec(p + "self_attn.q_proj.bias"); L.kb = hf_vec(p + "self_attn.k_proj.bias"); L.vb = hf_vec(p + "self_attn.v_proj.bias");
            }
            L.kc.assign((size_t)max_seq_ * c.num_kv_heads * c.head_dim, 0.f);
            L.vc.assign((size_t)max_seq_ * c.num_kv_heads * c.head_dim, 0.f);
        }
        embed_ = hf_mat(pre_ + "embed_tokens.weight");
        head_ = c.tie_word_embeddings ? embed_ : hf_mat("lm_head.weight");
        out_norm_ = hf_vec(pre_ + "norm.weight");
        finish_load();
    }
    const uint8_t* hf_bytes(const loader::TensorInfo& t, uint32_t& type) {
        if (t.dtype == "f32") type = gguf::F32;
        else if (t.dtype == "f16") type = gguf::F16;
        else if (t.dtype == "bf16") type = gguf::BF16;
        else throw std::runtime_error("GGUFCpuModel: " + t.name + " has dtype " + t.dtype + " (F32, F16 and BF16 are read)");
        auto& mp = maps_[t.file];
        if (!mp) { mp.reset(new Mapped()); mp->open(t.file); }
        const size_t width = type == gguf::F32 ? 4 : 2;
        if (t.nbytes != (uint64_t)t.numel() * width || t.offset + t.nbytes > mp->size) throw std::runtime_error("GGUFCpuModel: " + t.name + " lies outside " + t.file);
        return mp->base + t.offset;
    }
    Matrix hf_mat(const std::string& name) {
        auto it = hf_.tensors.find(name);
        if (it == hf_.tensors.end()) throw std::runtime_error("GGUFCpuModel: no tensor " + name);
        if (it->second.shape.size() != 2) throw std::runtime_error("GGUFCpuModel: " + name + " is not a matrix");
        Matrix m;
        m.data = hf_bytes(it->second, m.type);
        m.rows = (int)it->second.shape[0];
        m.cols = (int)it->second.shape[1];
        m.block_elems = 1;
        m.block_bytes = m.type == gguf::F32 ? 4 : 2;
        m.row_bytes = (size_t)m.cols * m.block_bytes;
        return m;
    }
    std::vector<float> hf_vec(const std::string& name) {
        auto it = hf_.tensors.find(name);
        if (it == hf_.tensors.end()) throw std::runtime_error("GGUFCpuModel: no tensor " + name);
        uint32_t type = 0;
        const uint8_t* p = hf_bytes(it->second, type);
        const int bb = type == gguf::F32 ? 4 : 2;
        std::vector<float> out((size_t)it->second.numel());
        for (size_t i = 0; i < out.size(); ++i) cpu_detail::dequant_block(type, p + i * bb, &out[i]);
        return out;
    }
    Matrix mat(const std::string& name) {
        const auto& t = reader_.tensor(name);
        if (t.shape.size() != 2) throw std::runtime_error("GGUFCpuModel: " + name + " is not a matrix");
        Matrix m;
        m.data = reader_.data(t);
        m.type = t.type;
        m.rows = (int)t.shape[0];
        m.cols = (int)t.shape[1];
        gguf::block_geometry(t.type, m.block_elems, m.block_bytes);
        if (m.cols % m.block_elems) throw std::runtime_error("GGUFCpuModel: " + name + " has rows that are not whole blocks");
        m.row_bytes = (size_t)(m.cols / m.block_elems) * m.block_bytes;
        float probe[256];
        cpu_detail::dequant_block(m.type, m.data, probe);              // rejects unsupported types at load
        return m;
    }
    std::vector<float> vec(const std::string& name) {
        const auto& t = reader_.tensor(name);
        int be, bb;
        gguf::block_geometry(t.type, be, bb);
        int64_t n = 1;
        for (auto d : t.shape) n *= d;
        std::vector<float> out((size_t)n);
        const uint8_t* p = reader_.data(t);
        float tmp[256];
        for (int64_t i = 0; i < n; i += be, p += bb) {
            cpu_detail::dequant_block(t.type, p, tmp);
            std::memcpy(&out[(size_t)i], tmp, sizeof(float) * (size_t)std::min<int64_t>(be, n - i));
        }
        return out;
    }
    void row(const Matrix& m, int r, float* y) const {
        const uint8_t* p = m.data + (size_t)r * m.row_bytes;
        for (int c = 0; c < m.cols; c += m.block_elems, p += m.block_bytes) cpu_detail::dequant_block(m.type, p, y + c);
    }
    // y = M x, rows spread over the pool's threads.
    void matvec(const Matrix& m, const float* x, float* y) const {
        auto work = [&](int r0, int r1) {
            if (m.block_elems != 1) { cpu_detail::block_rows(m.data, m.type, m.row_bytes, m.cols, m.block_elems, m.block_bytes, x, y, r0, r1); return; }
            for (int r = r0; r < r1; ++r) {                    // plain F32 / F16 / BF16 rows: products in float, sums in double
                const uint8_t* p = m.data + (size_t)r * m.row_bytes;
                double acc = 0;
                if (m.type == gguf::F32) for (int c = 0; c < m.cols; ++c) { float w; std::memcpy(&w, p + 4 * (size_t)c, 4); acc += w * x[c]; }
                else if (m.type == gguf::F16) for (int c = 0; c < m.cols; ++c) acc += cpu_detail::half_to_float(cpu_detail::rd16(p + 2 * (size_t)c)) * x[c];
                else for (int c = 0; c < m.cols; ++c) { const uint32_t b = (uint32_t)cpu_detail::rd16(p + 2 * (size_t)c) << 16; float w; std::memcpy(&w, &b, 4); acc += w * x[c]; }
                y[r] = (float)acc;
            }
        };
        const int nt = (int)std::min<int64_t>(threads_, std::max<int64_t>(1, (int64_t)m.rows * m.cols / (1 << 16)));
        if (nt <= 1 || !pool_) { work(0, m.rows); return; }
        pool_->run(nt, [&](int t) { work((int)((int64_t)m.rows * t / nt), (int)((int64_t)m.rows * (t + 1) / nt)); });
    }
    void rms(const float* x, const float* w, float* y, int n) const {
        double ss = 0;
        for (int i = 0; i < n; ++i) ss += (double)x[i] * x[i];
        const float r = 1.0f / std::sqrt((float)(ss / n) + (float)config.rms_norm_eps);
        for (int i = 0; i < n; ++i) y[i] = x[i] * r * w[i];
    }
    void rope(float* x, int pos, int half) const {
        const float *c = &cos_[(size_t)pos * half], *s = &sin_[(size_t)pos * half];
        if (config.rope_neox) {
            for (int i = 0; i < half; ++i) { const float a = x[i], b = x[i + half]; x[i] = a * c[i] - b * s[i]; x[i + half] = b * c[i] + a * s[i]; }
        } else {
            for (int i = 0; i < half; ++i) { const float a = x[2 * i], b = x[2 * i + 1]; x[2 * i] = a * c[i] - b * s[i]; x[2 * i + 1] = b * c[i] + a * s[i]; }
        }
    }

    gguf::GGUFReader reader_;
    std::vector<Layer> layers_;
    Matrix embed_, head_;
    loader::ModelWeights hf_;
    std::string pre_;
    std::map<std::string, std::unique_ptr<Mapped>> maps_;
    std::unique_ptr<cpu_detail::Pool> pool_;
    std::vector<float> out_norm_, cos_, sin_, logits_;
    int max_seq_ = 0, threads_ = 1;
};

}  // namespace io

namespace serve {

// The server backend over the CPU decoder: tokenizer of the file, sampling on the host (repetition penalty, temperature,
// top-k, top-p, inverse-CDF draw from a seeded generator).
class CpuBackend : public ModelBackend {
 public:
    CpuBackend(const std::string& path, const std::string& name_, int max_seq = 4096) {
        model_.load(path, max_seq);
        name = name_;
        architecture = model_.config.architecture;
        char buf[32];
        if (model_.from_hf()) {
            // a Hugging Face directory: its byte-level BPE files, the end-of-sequence ids of config.json / generation_config.json
            namespace L = io::loader::detail;
            const std::string dir = L::is_dir(path) ? path : L::dirname(path);
            if (!io::load_hf_tokenizer(dir, tok_)) throw std::runtime_error("CpuBackend: " + dir + " has neither vocab.json + merges.txt nor tokenizer.json");
            model_name = L::basename(dir);
            size = 0;
            for (const auto& f : model_.hf_weights().files) size += store::file_size(f);
            std::snprintf(buf, sizeof buf, "%.1fB", (double)model_.hf_weights().total_parameters() / 1e9);
            for (const char* f : {"/generation_config.json", "/config.json"}) {
                if (!L::is_file(dir + f)) continue;
                const json::Value e = json::parse(L::slurp(dir + f))["eos_token_id"];
                if (e.is_number()) stop_.insert((int)e.as_int());
                if (e.is_array()) for (const auto& v : e.items()) if (v.is_number()) stop_.insert((int)v.as_int());
                if (!stop_.empty()) break;
            }
        } else {
            tok_ = io::GGUFTokenizer::from_reader(model_.reader());
            model_name = model_.reader().has("general.name") ? model_.reader().get("general.name").s : "";
            size = store::file_size(path);
            unsigned long long bytes = 0;
            for (const auto& kv : model_.reader().tensors()) bytes += kv.second.nbytes;
            std::snprintf(buf, sizeof buf, "%.1fB", (double)bytes / 0.5625 / 1e9);
        }
        parameter_size = buf;
        if (tok_.eos_id() >= 0) stop_.insert(tok_.eos_id());
        for (const char* t : {"<|im_end|>", "<|eot_id|>", "<end_of_turn>", "<|end|>", "<|endoftext|>"})
            if (tok_.token_id(t) >= 0) stop_.insert(tok_.token_id(t));
    }
    std::vector<int> encode(const std::string& text) override { return tok_.encode(text); }
    std::string decode_token(int id) override { return tok_.decode_token(id); }
    std::pair<double, double> generate(const std::vector<int>& prompt, const GenerateOptions& opt, const std::function<bool(int)>& on_token) override {
        using clock = std::chrono::steady_clock;
        const int n = (int)prompt.size();
        if (n + 2 > model_.max_seq()) throw std::runtime_error("the prompt does not fit the context of " + std::to_string(model_.max_seq()) + " tokens");
        const int n_new = std::max(0, std::min(opt.num_predict, model_.max_seq() - n - 1));
        const auto t0 = clock::now();
        for (int i = 0; i + 1 < n; ++i) model_.forward(prompt[(size_t)i], i, false);
        const auto t1 = clock::now();
        std::vector<int> history = prompt;
        std::mt19937_64 rng((uint64_t)opt.seed);
        int tok = prompt.back(), pos = n - 1;
        for (int i = 0; i < n_new; ++i) {
            const std::vector<float>& logits = model_.forward(tok, pos);
            const int next = sample(logits, history, opt, rng);
            history.push_back(next);
            if (!on_token(next) || stop_.count(next)) break;
            tok = next;
            if (++pos + 1 >= model_.max_seq()) break;
        }
        const auto t2 = clock::now();
        return {std::chrono::duration<double>(t1 - t0).count(), std::chrono::duration<double>(t2 - t1).count()};
    }
    io::GGUFCpuModel& model() { return model_; }
    const io::GGUFTokenizer& tokenizer() const { return tok_; }

    // Penalty on the ids seen so far, then the k best by (value, smaller id first), softmax at the temperature, the shortest
    // prefix reaching top_p, and a draw.  temperature <= 0: the arg-max after the penalty.
    static int sample(const std::vector<float>& logits, const std::vector<int>& history, const GenerateOptions& opt, std::mt19937_64& rng) {
        std::vector<float> x = logits;
        if (opt.repeat_penalty != 1.0) {
            std::set<int> seen(history.begin(), history.end());
            for (int t : seen)
                if (t >= 0 && t < (int)x.size()) x[(size_t)t] = x[(size_t)t] > 0 ? x[(size_t)t] / (float)opt.repeat_penalty : x[(size_t)t] * (float)opt.repeat_penalty;
        }
        const int V = (int)x.size();
        const int k = opt.top_k > 0 ? std::min(opt.top_k, V) : V;
        std::vector<int> order((size_t)V);
        for (int i = 0; i < V; ++i) order[(size_t)i] = i;
        std::partial_sort(order.begin(), order.begin() + k, order.end(), [&](int a, int b) { return x[(size_t)a] != x[(size_t)b] ? x[(size_t)a] > x[(size_t)b] : a < b; });
        if (opt.temperature <= 0.0) return order[0];
        std::vector<double> p((size_t)k);
        double z = 0;
        for (int i = 0; i < k; ++i) { p[(size_t)i] = std::exp((x[(size_t)order[(size_t)i]] - x[(size_t)order[0]]) / opt.temperature); z += p[(size_t)i]; }
        int keep = k;
        double kept = z;
        if (opt.top_p > 0.0 && opt.top_p < 1.0) {
            keep = 0;
            kept = 0;
            while (keep < k && kept < opt.top_p * z) kept += p[(size_t)keep++];
        }
        double u = std::uniform_real_distribution<double>(0.0, 1.0)(rng) * kept;
        for (int i = 0; i < keep; ++i) {
            u -= p[(size_t)i];
            if (u <= 0) return order[(size_t)i];
        }
        return order[(size_t)keep - 1];
    }

 private:
    io::GGUFCpuModel model_;
    io::GGUFTokenizer tok_;
    std::set<int> stop_;
};

}  // namespace serve
}  // namespace promethorch
