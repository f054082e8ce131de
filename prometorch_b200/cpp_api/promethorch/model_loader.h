// promethorch C++ API: one loader for every weight container a server may be pointed at (no libtorch, no CUDA).
//
//   detect_format(path)      "gguf" / "safetensors" / "pytorch" / "ptor" / "hf_dir" / "unknown": magic bytes first (GGUF, PTOR,
//                            the safetensors length + '{' header, ZIP or pickle for .pt), extension second
//   load_model(path)         ModelWeights: per-tensor name / dtype / shape / file, the architecture and the shape parameters
//                            inferred from tensor names and shapes (and from config.json next to Hugging Face weights)
//   read_tensor_bytes(...)   the raw little-endian bytes of one tensor (safetensors, PTOR and GGUF blocks), read lazily
//   SafeTensorsFile          header parser of the safetensors container
//
// Counterpart of the reference's promeserve/model_loader.h (detect_format :170-227, infer_architecture :998-1058,
// infer_config_from_tensors :1060-1141, load_model :1197-1249) and of io/model_loader.py of this package, which it matches
// field by field.  PyTorch .pt files are recognised but their tensors are listed only through the libtorch side
// (serialization.h); ONNX initialisers are out of scope.
#pragma once
#include <dirent.h>
#include <sys/stat.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <regex>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "gguf_reader.h"
#include "json.h"

namespace promethorch {
namespace io {
namespace loader {

struct TensorInfo {
    std::string name, dtype = "unknown", file;
    std::vector<int64_t> shape;
    uint64_t offset = 0, nbytes = 0;         // where the bytes sit in `file` (safetensors, PTOR); GGUF blocks go through the reader
    int64_t numel() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
};

struct ModelConfig {
    int64_t hidden_size = 0, num_layers = 0, num_heads = 0, num_kv_heads = 0, intermediate_size = 0, vocab_size = 0, head_dim = 0, context_length = 0;
    double rms_norm_eps = 1e-6, rope_freq_base = 10000.0;
    bool tie_word_embeddings = false;
};

struct ModelWeights {
    std::string architecture, format = "unknown", source_path;
    std::map<std::string, TensorInfo> tensors;
    std::vector<std::string> order;          // tensor names in file order
    ModelConfig config;
    std::vector<std::string> files;
    int64_t total_parameters() const {
        int64_t n = 0;
        for (const auto& kv : tensors) n += kv.second.numel();
        return n;
    }
};

namespace detail {
inline bool is_file(const std::string& p) { struct stat st; return ::stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode); }
inline bool is_dir(const std::string& p) { struct stat st; return ::stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode); }
inline int64_t file_size(const std::string& p) { struct stat st; return ::stat(p.c_str(), &st) == 0 ? (int64_t)st.st_size : -1; }
inline std::string dirname(const std::string& p) {
    const size_t s = p.find_last_of('/');
    return s == std::string::npos ? "." : (s == 0 ? "/" : p.substr(0, s));
}
inline std::string basename(const std::string& p) {
    const size_t s = p.find_last_of('/');
    return s == std::string::npos ? p : p.substr(s + 1);
}
inline std::string lower(std::string s) { for (auto& c : s) c = (char)std::tolower((unsigned char)c); return s; }
inline std::string slurp(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("model_loader: cannot open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}
template <typename T>
inline T rd(std::ifstream& f) {
    T v;
    f.read((char*)&v, sizeof(T));
    if (!f) throw std::runtime_error("model_loader: unexpected end of file");
    return v;
}
}  // namespace detail

inline std::string detect_format(const std::string& path) {
    using namespace detail;
    if (is_dir(path)) return is_file(path + "/config.json") ? "hf_dir" : "unknown";
    std::ifstream f(path, std::ios::binary);
    if (!f) return "unknown";
    unsigned char head[9] = {0};
    f.read((char*)head, 9);
    const std::streamsize got = f.gcount();
    if (got < 4) return "unknown";
    if (std::memcmp(head, "GGUF", 4) == 0) return "gguf";
    if (std::memcmp(head, "PTOR", 4) == 0) return "ptor";
    if (got >= 9) {                                        // before the pickle test: a header length may start with byte 0x80
        uint64_t n;
        std::memcpy(&n, head, 8);
        if (n >= 2 && n < 100ull * 1024 * 1024 && (int64_t)n <= file_size(path) - 8 && head[8] == '{') return "safetensors";
    }
    if (std::memcmp(head, "PK\x03\x04", 4) == 0 || (head[0] == 0x80 && head[1] >= 2 && head[1] <= 5)) return "pytorch";
    const std::string b = lower(basename(path));
    const size_t dot = b.find_last_of('.');
    const std::string ext = dot == std::string::npos ? "" : b.substr(dot);
    if (ext == ".safetensors") return "safetensors";
    if (ext == ".gguf") return "gguf";
    if (ext == ".bin" || ext == ".pt" || ext == ".pth") return "pytorch";
    if (ext == ".ptor") return "ptor";
    return "unknown";
}

// The safetensors container: u64 header length, JSON header {name: {dtype, shape, data_offsets}, "__metadata__": {...}}, data.
class SafeTensorsFile {
 public:
    explicit SafeTensorsFile(const std::string& path) : path_(path) {
        std::ifstream f(path, std::ios::binary);
        if (!f) throw std::runtime_error("safetensors: cannot open " + path);
        const uint64_t n = detail::rd<uint64_t>(f);
        if (n < 2 || n > 100ull * 1024 * 1024) throw std::runtime_error("safetensors: implausible header length in " + path);
        std::string hdr((size_t)n, '\0');
        f.read(&hdr[0], (std::streamsize)n);
        if (!f) throw std::runtime_error("safetensors: truncated header in " + path);
        data_start_ = 8 + n;
        const json::Value h = json::parse(hdr);
        const int64_t size = detail::file_size(path);
        for (const auto& kv : h.members()) {
            if (kv.first == "__metadata__") {
                for (const auto& m : kv.second.members()) metadata_[m.first] = m.second.as_string();
                continue;
            }
            TensorInfo t;
            t.name = kv.first;
            t.dtype = detail::lower(kv.second["dtype"].as_string());
            for (const auto& d : kv.second["shape"].items()) t.shape.push_back(d.as_int());
            const auto& off = kv.second["data_offsets"];
            if (off.size() != 2) throw std::runtime_error("safetensors: bad data_offsets of " + t.name);
            t.offset = data_start_ + (uint64_t)off.at(0).as_int();
            t.nbytes = (uint64_t)(off.at(1).as_int() - off.at(0).as_int());
            if ((int64_t)(t.offset + t.nbytes) > size) throw std::runtime_error("safetensors: tensor " + t.name + " runs past the end of " + path);
            t.file = path;
            order_.push_back(t.name);
            tensors_[t.name] = std::move(t);
        }
    }
    const std::vector<std::string>& keys() const { return order_; }
    const TensorInfo& info(const std::string& name) const {
        auto it = tensors_.find(name);
        if (it == tensors_.end()) throw std::runtime_error("safetensors: no tensor " + name + " in " + path_);
        return it->second;
    }
    const std::map<std::string, std::string>& metadata() const { return metadata_; }

 private:
    std::string path_;
    uint64_t data_start_ = 0;
    std::vector<std::string> order_;
    std::map<std::string, TensorInfo> tensors_;
    std::map<std::string, std::string> metadata_;
};

// From tensor names: Hugging Face and GGUF naming of the families the runtime knows.
inline std::string infer_architecture(const std::vector<std::string>& names) {
    auto any = [&](const char* pattern) {
        const std::regex re(pattern);
        for (const auto& n : names)
            if (std::regex_search(n, re)) return true;
        return false;
    };
    if (any("(^|[^A-Za-z0-9_])blk\\.[0-9]+\\.attn_q\\.weight")) return "llama";        // GGUF layout; the file's metadata names the exact family
    if (any("encoder\\.layer\\.0\\.attention\\.self\\.query\\.weight")) return "bert";
    if (any("(^|\\.)h\\.0\\.attn\\.c_attn\\.weight")) return "gpt2";
    if (any("layers\\.0\\.self_attn\\.q_proj\\.weight")) {
        if (any("layers\\.0\\.self_attn\\.q_norm\\.weight")) return "qwen3";
        if (any("layers\\.0\\.self_attn\\.q_proj\\.bias")) return "qwen2";
        if (any("layers\\.0\\.pre_feedforward_layernorm\\.weight")) return "gemma2";
        return "llama";
    }
    if (any("layers\\.0\\.self_attn\\.qkv_proj\\.weight")) return "phi3";
    return "unknown";
}

// Fill the shape parameters that the tensor shapes determine (embedding, projections, layer count).
inline void infer_config_from_tensors(ModelWeights& mw) {
    ModelConfig& c = mw.config;
    const auto& t = mw.tensors;
    auto shape = [&](std::initializer_list<const char*> cands) -> const std::vector<int64_t>* {
        for (const char* k : cands)
            for (const char* pre : {"", "model.", "transformer.", "bert."}) {
                auto it = t.find(std::string(pre) + k);
                if (it != t.end()) return &it->second.shape;
            }
        return nullptr;
    };
    if (auto emb = shape({"embed_tokens.weight", "wte.weight", "embeddings.word_embeddings.weight", "token_embd.weight"}))
        if (emb->size() >= 2) { c.vocab_size = (*emb)[0]; c.hidden_size = (*emb)[1]; }
    int64_t max_layer = -1;
    const std::regex layer_re("(?:layers|h|layer|blk)\\.([0-9]+)\\.");
    bool has_c_fc = false;
    for (const auto& kv : t) {
        std::smatch m;
        if (std::regex_search(kv.first, m, layer_re)) max_layer = std::max<int64_t>(max_layer, std::stoll(m[1].str()));
        has_c_fc |= kv.first.find("h.0.mlp.c_fc.weight") != std::string::npos;
    }
    c.num_layers = max_layer + 1;
    auto q = shape({"layers.0.self_attn.q_proj.weight", "blk.0.attn_q.weight"});
    auto k = shape({"layers.0.self_attn.k_proj.weight", "blk.0.attn_k.weight"});
    auto up = shape({"layers.0.mlp.up_proj.weight", "blk.0.ffn_up.weight", "h.0.mlp.c_fc.weight", "encoder.layer.0.intermediate.dense.weight"});
    if (up && up->size() >= 2) c.intermediate_size = (has_c_fc && (*up)[0] == c.hidden_size) ? (*up)[1] : (*up)[0];
    if (auto qn = shape({"layers.0.self_attn.q_norm.weight", "blk.0.attn_q_norm.weight"})) c.head_dim = (*qn)[0];
    if (q && c.hidden_size) {
        const int64_t q0 = (*q)[0];
        if (!c.head_dim) c.head_dim = (q0 % 128 == 0 && c.hidden_size >= 2048) ? 128 : (q0 % 64 == 0 ? 64 : q0);
        c.num_heads = q0 / c.head_dim;
        if (k) c.num_kv_heads = (*k)[0] / c.head_dim;
    }
    bool has_head = false;
    for (const auto& kv : t) {
        const std::string& n = kv.first;
        has_head |= n == "output.weight" || (n.size() >= 14 && n.compare(n.size() - 14, 14, "lm_head.weight") == 0);
    }
    c.tie_word_embeddings = !has_head;
}

inline void apply_hf_config(ModelWeights& mw, const json::Value& cfg) {
    ModelConfig& c = mw.config;
    auto geti = [&](const char* a, const char* b, int64_t d) {
        if (cfg[a].is_number()) return (int64_t)cfg[a].as_int();
        if (b && cfg[b].is_number()) return (int64_t)cfg[b].as_int();
        return d;
    };
    c.hidden_size = geti("hidden_size", "n_embd", c.hidden_size);
    c.num_layers = geti("num_hidden_layers", "n_layer", c.num_layers);
    c.num_heads = geti("num_attention_heads", "n_head", c.num_heads);
    c.num_kv_heads = geti("num_key_value_heads", nullptr, c.num_heads);
    c.intermediate_size = geti("intermediate_size", "n_inner", c.intermediate_size);
    c.vocab_size = geti("vocab_size", nullptr, c.vocab_size);
    c.head_dim = geti("head_dim", nullptr, c.num_heads ? c.hidden_size / c.num_heads : 0);
    c.context_length = geti("max_position_embeddings", "n_positions", c.context_length);
    if (cfg["rms_norm_eps"].is_number()) c.rms_norm_eps = cfg["rms_norm_eps"].as_double();
    if (cfg["rope_theta"].is_number()) c.rope_freq_base = cfg["rope_theta"].as_double();
    if (cfg["tie_word_embeddings"].is_bool()) c.tie_word_embeddings = cfg["tie_word_embeddings"].as_bool();
    if (cfg["model_type"].is_string() && !cfg["model_type"].as_string().empty()) mw.architecture = cfg["model_type"].as_string();
}

// The files of a sharded checkpoint: what model.safetensors.index.json lists, else *-00001-of-0000N.* siblings.
inline std::vector<std::string> find_shard_files(const std::string& path) {
    using namespace detail;
    const std::string d = is_dir(path) ? path : dirname(path);
    const std::string idx = d + "/model.safetensors.index.json";
    if (is_file(idx)) {
        std::set<std::string> names;
        const json::Value index = json::parse(slurp(idx));          // named: a range-for over a member of a temporary would dangle
        for (const auto& kv : index["weight_map"].members()) names.insert(kv.second.as_string());
        std::vector<std::string> out;
        for (const auto& n : names) out.push_back(d + "/" + n);
        return out;
    }
    if (is_dir(path) && is_file(d + "/model.safetensors")) return {d + "/model.safetensors"};
    std::smatch m;
    const std::string base = basename(path);
    if (std::regex_match(base, m, std::regex("(.*)-([0-9]{5})-of-([0-9]{5})(\\..*)"))) {
        std::vector<std::string> out;
        const int n = std::min(std::stoi(m[3].str()), 99999);
        for (int i = 1; i <= n; ++i) {
            char num[16];
            std::snprintf(num, sizeof num, "%05d", i);
            out.push_back(d + "/" + m[1].str() + "-" + num + "-of-" + m[3].str() + m[4].str());
        }
        return out;
    }
    return {path};
}

namespace detail {
inline const char* ptor_dtype(int code) {
    switch (code) {
        case 0: return "uint8";
        case 1: return "int8";
        case 2: return "int16";
        case 3: return "int32";
        case 4: return "int64";
        case 5: return "float16";
        case 6: return "float32";
        case 7: return "float64";
        case 9: return "complex64";
        case 10: return "complex128";
        case 11: return "bool";
        case 12: return "bfloat16";
        case 17: return "float8_e4m3fn";
        case 18: return "float8_e5m2";
        default: return nullptr;
    }
}
inline const char* gguf_dtype(uint32_t t) {
    switch (t) {
        case gguf::F32: return "f32";
        case gguf::F16: return "f16";
        case gguf::BF16: return "bf16";
        case gguf::Q4_0: return "q4_0";
        case gguf::Q8_0: return "q8_0";
        case gguf::Q2_K: return "q2_k";
        case gguf::Q3_K: return "q3_k";
        case gguf::Q4_K: return "q4_k";
        case gguf::Q5_K: return "q5_k";
        case gguf::Q6_K: return "q6_k";
        default: return "unknown";
    }
}
inline void finish_dir(ModelWeights& mw, const std::string& dir) {
    if (is_file(dir + "/config.json")) apply_hf_config(mw, json::parse(slurp(dir + "/config.json")));
}
}  // namespace detail

// Metadata of every tensor of `path` (a file of a known format, or a Hugging Face directory).
inline ModelWeights load_model(const std::string& path) {
    using namespace detail;
    ModelWeights mw;
    mw.format = detect_format(path);
    mw.source_path = path;
    if (mw.format == "unknown") throw std::runtime_error(path + ": unknown model format");
    if (mw.format == "gguf") {
        gguf::GGUFReader r(path);
        mw.files = {path};
        for (const auto& kv : r.tensors()) {
            TensorInfo t;
            t.name = kv.first;
            t.dtype = gguf_dtype(kv.second.type);
            t.shape = kv.second.shape;
            t.file = path;
            t.nbytes = kv.second.nbytes;
            mw.order.push_back(t.name);
            mw.tensors[t.name] = std::move(t);
        }
        mw.architecture = r.arch();
        infer_config_from_tensors(mw);
        ModelConfig& c = mw.config;
        auto nz = [](int64_t v, int64_t d) { return v ? v : d; };
        c.num_heads = nz(r.arch_int("attention.head_count", c.num_heads), c.num_heads);
        c.num_kv_heads = nz(r.arch_int("attention.head_count_kv", c.num_kv_heads ? c.num_kv_heads : c.num_heads), c.num_heads);
        c.context_length = r.arch_int("context_length", 0);
        const double fb = r.arch_float("rope.freq_base", c.rope_freq_base), eps = r.arch_float("attention.layer_norm_rms_epsilon", c.rms_norm_eps);
        c.rope_freq_base = fb != 0 ? fb : c.rope_freq_base;
        c.rms_norm_eps = eps != 0 ? eps : c.rms_norm_eps;
        if (c.num_heads && !c.head_dim) c.head_dim = nz(r.arch_int("attention.key_length", 0), c.hidden_size / c.num_heads);
        return mw;
    }
    if (mw.format == "safetensors" || mw.format == "hf_dir") {
        const bool sharded_name = std::regex_search(basename(path), std::regex("-[0-9]{5}-of-[0-9]{5}\\."));
        std::vector<std::string> files = (mw.format == "hf_dir" || sharded_name) ? find_shard_files(path) : std::vector<std::string>{path};
        std::vector<std::string> kept;
        for (const auto& f : files)
            if (is_file(f) && detect_format(f) == "safetensors") kept.push_back(f);
        mw.files = kept;
        for (const auto& fpath : kept) {
            SafeTensorsFile f(fpath);
            for (const auto& name : f.keys()) {
                if (!mw.tensors.count(name)) mw.order.push_back(name);
                mw.tensors[name] = f.info(name);
            }
        }
        mw.architecture = infer_architecture(mw.order);
        infer_config_from_tensors(mw);
        finish_dir(mw, mw.format == "hf_dir" ? path : dirname(path));
        return mw;
    }
    if (mw.format == "ptor") {
        std::ifstream f(path, std::ios::binary);
        char magic[4];
        f.read(magic, 4);
        if (rd<uint32_t>(f) != 1) throw std::runtime_error(path + ": unsupported PTOR version");
        const uint64_t count = rd<uint64_t>(f);
        mw.files = {path};
        for (uint64_t i = 0; i < count; ++i) {
            TensorInfo t;
            const uint32_t nl = rd<uint32_t>(f);
            if (nl > (1u << 20)) throw std::runtime_error(path + ": implausible tensor name length");
            t.name.resize(nl);
            f.read(&t.name[0], nl);
            const int code = rd<uint8_t>(f);
            const char* dt = ptor_dtype(code);
            if (!dt) throw std::runtime_error(path + ": unknown dtype code " + std::to_string(code));
            t.dtype = dt;
            const uint32_t nd = rd<uint32_t>(f);
            if (nd > 64) throw std::runtime_error(path + ": implausible rank");
            for (uint32_t d = 0; d < nd; ++d) t.shape.push_back(rd<int64_t>(f));
            t.nbytes = rd<uint64_t>(f);
            t.offset = (uint64_t)f.tellg();
            t.file = path;
            f.seekg((std::streamoff)t.nbytes, std::ios::cur);
            if (!f) throw std::runtime_error(path + ": tensor " + t.name + " runs past the end of the file");
            mw.order.push_back(t.name);
            mw.tensors[t.name] = std::move(t);
        }
        mw.architecture = infer_architecture(mw.order);
        infer_config_from_tensors(mw);
        return mw;
    }
    // "pytorch": the container is recognised; listing its tensors needs the unpickler of the libtorch side
    mw.files = {path};
    return mw;
}

// The stored bytes of one tensor (little-endian values for safetensors / PTOR, quantised blocks for GGUF).
inline std::vector<uint8_t> read_tensor_bytes(const ModelWeights& mw, const std::string& name) {
    auto it = mw.tensors.find(name);
    if (it == mw.tensors.end()) throw std::runtime_error("model_loader: no tensor " + name);
    const TensorInfo& t = it->second;
    if (mw.format == "gguf") {
        gguf::GGUFReader r(t.file);
        const auto& gi = r.tensor(name);
        const uint8_t* p = r.data(gi);
        return std::vector<uint8_t>(p, p + gi.nbytes);
    }
    if (mw.format == "pytorch") throw std::runtime_error("model_loader: tensors of .pt files are read through serialization.h");
    std::ifstream f(t.file, std::ios::binary);
    if (!f) throw std::runtime_error("model_loader: cannot open " + t.file);
    f.seekg((std::streamoff)t.offset);
    std::vector<uint8_t> out((size_t)t.nbytes);
    f.read((char*)out.data(), (std::streamsize)t.nbytes);
    if (!f) throw std::runtime_error("model_loader: short read of " + name);
    return out;
}

}  // namespace loader
}  // namespace io
}  // namespace promethorch
