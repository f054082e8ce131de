// promethorch C++ API: the GGUF file reader (no CUDA, no libtorch).
//
//   promethorch::io::gguf::GGUFReader   memory-mapped GGUF v2/v3 reader: metadata of every value type, the tensor
//                                       directory (shapes in torch order), raw block bytes
// Used by GGUFModel (gguf.h), by the tokenizer (tokenizer.h) and by the server (serve.h).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace promethorch {
namespace io {
namespace gguf {

enum GGMLType : uint32_t { F32 = 0, F16 = 1, Q4_0 = 2, Q8_0 = 8, Q2_K = 10, Q3_K = 11, Q4_K = 12, Q5_K = 13, Q6_K = 14, BF16 = 30 };

struct Value {                       // one metadata value: a scalar, a string or an array of them
    uint32_t type = 0;
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0;
    bool b = false;
    std::string s;
    std::vector<Value> arr;
    double as_float() const { return type == 6 || type == 12 ? f : (type == 5 || type == 3 || type == 1 || type == 11 ? (double)i : (double)u); }
    int64_t as_int() const { return type == 6 || type == 12 ? (int64_t)f : (type == 5 || type == 3 || type == 1 || type == 11 ? i : (int64_t)u); }
};

struct TensorInfo {
    std::string name;
    std::vector<int64_t> shape;      // torch order (GGML stores the dimensions reversed)
    uint32_t type = 0;
    uint64_t offset = 0;             // from the start of the data section
    uint64_t nbytes = 0;
};

inline void block_geometry(uint32_t type, int& elems, int& bytes) {
    switch (type) {
        case F32: elems = 1; bytes = 4; break;
        case F16: case BF16: elems = 1; bytes = 2; break;
        case Q4_0: elems = 32; bytes = 18; break;
        case Q8_0: elems = 32; bytes = 34; break;
        case Q2_K: elems = 256; bytes = 84; break;
        case Q3_K: elems = 256; bytes = 110; break;
        case Q4_K: elems = 256; bytes = 144; break;
        case Q5_K: elems = 256; bytes = 176; break;
        case Q6_K: elems = 256; bytes = 210; break;
        default: throw std::runtime_error("GGUF: unsupported tensor type " + std::to_string(type));
    }
}

class GGUFReader {
 public:
    GGUFReader() = default;
    explicit GGUFReader(const std::string& path) { open(path); }
    ~GGUFReader() { close(); }
    GGUFReader(const GGUFReader&) = delete;
    GGUFReader& operator=(const GGUFReader&) = delete;

    void open(const std::string& path) {
        close();
        fd_ = ::open(path.c_str(), O_RDONLY);
        if (fd_ < 0) throw std::runtime_error("GGUF: cannot open " + path);
        struct stat st;
        ::fstat(fd_, &st);
        size_ = (size_t)st.st_size;
        base_ = (const uint8_t*)::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (base_ == MAP_FAILED) { base_ = nullptr; throw std::runtime_error("GGUF: mmap failed for " + path); }
        size_t p = 0;
        if (rd<uint32_t>(p) != 0x46554747u) throw std::runtime_error("GGUF: bad magic in " + path);
        const uint32_t version = rd<uint32_t>(p);
        if (version < 2 || version > 3) throw std::runtime_error("GGUF: unsupported version " + std::to_string(version));
        const uint64_t n_tensors = rd<uint64_t>(p), n_kv = rd<uint64_t>(p);
        for (uint64_t k = 0; k < n_kv; ++k) {
            const std::string key = rd_str(p);
            const uint32_t type = rd<uint32_t>(p);
            metadata_[key] = rd_value(p, type);
        }
        for (uint64_t t = 0; t < n_tensors; ++t) {
            TensorInfo ti;
            ti.name = rd_str(p);
            const uint32_t nd = rd<uint32_t>(p);
            std::vector<int64_t> dims(nd);
            for (auto& d : dims) d = (int64_t)rd<uint64_t>(p);
            ti.shape.assign(dims.rbegin(), dims.rend());
            ti.type = rd<uint32_t>(p);
            ti.offset = rd<uint64_t>(p);
            int be, bb;
            block_geometry(ti.type, be, bb);
            int64_t n = 1;
            for (auto d : dims) n *= d;
            ti.nbytes = (uint64_t)(n / be) * bb;
            tensors_[ti.name] = ti;
        }
        const uint64_t align = has("general.alignment") ? (uint64_t)get("general.alignment").as_int() : 32;
        data_ = (p + align - 1) / align * align;
    }
    void close() {
        if (base_) ::munmap((void*)base_, size_);
        if (fd_ >= 0) ::close(fd_);
        base_ = nullptr;
        fd_ = -1;
        metadata_.clear();
        tensors_.clear();
    }
    bool has(const std::string& key) const { return metadata_.count(key) != 0; }
    const Value& get(const std::string& key) const {
        auto it = metadata_.find(key);
        if (it == metadata_.end()) throw std::runtime_error("GGUF: no metadata key " + key);
        return it->second;
    }
    std::string arch() const { return has("general.architecture") ? get("general.architecture").s : "llama"; }
    double arch_float(const std::string& k, double dflt) const { return has(arch() + "." + k) ? get(arch() + "." + k).as_float() : dflt; }
    int64_t arch_int(const std::string& k, int64_t dflt) const { return has(arch() + "." + k) ? get(arch() + "." + k).as_int() : dflt; }
    bool has_tensor(const std::string& n) const { return tensors_.count(n) != 0; }
    const TensorInfo& tensor(const std::string& n) const {
        auto it = tensors_.find(n);
        if (it == tensors_.end()) throw std::runtime_error("GGUF: no tensor " + n);
        return it->second;
    }
    const uint8_t* data(const TensorInfo& t) const {
        if (data_ + t.offset + t.nbytes > size_) throw std::runtime_error("GGUF: tensor " + t.name + " runs past the end of the file");
        return base_ + data_ + t.offset;
    }
    const std::map<std::string, TensorInfo>& tensors() const { return tensors_; }
    const std::map<std::string, Value>& metadata() const { return metadata_; }

 private:
    template <typename T>
    T rd(size_t& p) const {
        if (p + sizeof(T) > size_) throw std::runtime_error("GGUF: truncated file");
        T v;
        std::memcpy(&v, base_ + p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string rd_str(size_t& p) const {
        const uint64_t n = rd<uint64_t>(p);
        if (p + n > size_) throw std::runtime_error("GGUF: truncated string");
        std::string s((const char*)base_ + p, n);
        p += n;
        return s;
    }
    Value rd_value(size_t& p, uint32_t type) const {
        Value v;
        v.type = type;
        switch (type) {
            case 0: v.u = rd<uint8_t>(p); break;
            case 1: v.i = rd<int8_t>(p); break;
            case 2: v.u = rd<uint16_t>(p); break;
            case 3: v.i = rd<int16_t>(p); break;
            case 4: v.u = rd<uint32_t>(p); break;
            case 5: v.i = rd<int32_t>(p); break;
            case 6: v.f = rd<float>(p); break;
            case 7: v.b = rd<uint8_t>(p) != 0; v.u = v.b; break;
            case 8: v.s = rd_str(p); break;
            case 9: {
                const uint32_t et = rd<uint32_t>(p);
                const uint64_t n = rd<uint64_t>(p);
                v.arr.reserve(n);
                for (uint64_t k = 0; k < n; ++k) v.arr.push_back(rd_value(p, et));
                break;
            }
            case 10: v.u = rd<uint64_t>(p); break;
            case 11: v.i = rd<int64_t>(p); break;
            case 12: v.f = rd<double>(p); break;
            default: throw std::runtime_error("GGUF: unknown metadata type " + std::to_string(type));
        }
        return v;
    }
    int fd_ = -1;
    const uint8_t* base_ = nullptr;
    size_t size_ = 0, data_ = 0;
    std::map<std::string, Value> metadata_;
    std::map<std::string, TensorInfo> tensors_;
};

}  // namespace gguf

// The shape parameters of a dense decoder, from the metadata of its file (llama, mistral, qwen2, qwen3).
struct TransformerConfig {
    std::string architecture = "llama";
    int vocab_size = 0, hidden_size = 0, num_layers = 0, num_heads = 0, num_kv_heads = 0, intermediate_size = 0, head_dim = 0;
    int context_length = 8192;
    double rope_freq_base = 10000.0, rms_norm_eps = 1e-6;
    bool has_qk_norm = false, rope_neox = false, tie_word_embeddings = false;
    void parse(const gguf::GGUFReader& r) {
        architecture = r.arch();
        hidden_size = (int)r.arch_int("embedding_length", 0);
        num_layers = (int)r.arch_int("block_count", 0);
        num_heads = (int)r.arch_int("attention.head_count", 0);
        num_kv_heads = (int)r.arch_int("attention.head_count_kv", num_heads);
        intermediate_size = (int)r.arch_int("feed_forward_length", 0);
        context_length = (int)r.arch_int("context_length", 8192);
        rope_freq_base = r.arch_float("rope.freq_base", 10000.0);
        rms_norm_eps = r.arch_float("attention.layer_norm_rms_epsilon", 1e-6);
        const int key_len = (int)r.arch_int("attention.key_length", 0);
        head_dim = key_len > 0 ? key_len : hidden_size / std::max(num_heads, 1);
        vocab_size = (int)r.tensor("token_embd.weight").shape[0];
        tie_word_embeddings = !r.has_tensor("output.weight");
        has_qk_norm = architecture == "qwen3";
        rope_neox = architecture == "qwen2" || architecture == "qwen3" || architecture == "phi3" || architecture == "gemma";
        if (!(architecture == "llama" || architecture == "mistral" || architecture == "qwen2" || architecture == "qwen3"))
            throw std::runtime_error("GGUF models in C++: architecture '" + architecture + "' is served by the Python loader");
    }
};


}  // namespace io
}  // namespace promethorch
