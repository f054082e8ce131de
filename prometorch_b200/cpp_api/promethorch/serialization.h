// promethorch C++ API: checkpoint I/O.
//
//  * save / load / save_state_dict / load_state_dict: the PTOR container ("PTOR", u32 version 1, u64 count, then per
//    tensor: u32 name length, name, u8 dtype code, u32 ndim, i64 sizes, u64 nbytes, raw little-endian data;
//    torch/serialization.h:17-197 of the reference), byte-compatible with files the reference and the Python package
//    write.
//  * save_pytorch / load_pytorch: PyTorch zip checkpoints through libtorch's restricted unpickler (tensors and plain
//    containers only; it executes no code from the file), the policy of torch/serialization_pytorch.h:734-878.
#pragma once
#include "model_loader.h"
#include <torch/torch.h>

#include <cstdint>
#include <fstream>
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace promethorch {
using Tensor = at::Tensor;
using OrderedStateDict = std::vector<std::pair<std::string, Tensor>>;

namespace detail {
inline int ptor_code(c10::ScalarType t) {
    switch (t) {
        case c10::kByte: return 0;
        case c10::kChar: return 1;
        case c10::kShort: return 2;
        case c10::kInt: return 3;
        case c10::kLong: return 4;
        case c10::kHalf: return 5;
        case c10::kFloat: return 6;
        case c10::kDouble: return 7;
        case c10::kComplexFloat: return 9;
        case c10::kComplexDouble: return 10;
        case c10::kBool: return 11;
        case c10::kBFloat16: return 12;
        default: throw std::runtime_error("serialization: dtype has no PTOR code");
    }
}
inline c10::ScalarType ptor_dtype(int code) {
    static const c10::ScalarType tab[13] = {c10::kByte, c10::kChar, c10::kShort, c10::kInt, c10::kLong, c10::kHalf, c10::kFloat,
                                            c10::kDouble, c10::kFloat /*8: unused*/, c10::kComplexFloat, c10::kComplexDouble, c10::kBool,
                                            c10::kBFloat16};
    if (code < 0 || code > 12 || code == 8) throw std::runtime_error("serialization: unknown dtype code " + std::to_string(code));
    return tab[code];
}
template <typename T>
inline void put(std::ostream& f, T v) { f.write(reinterpret_cast<const char*>(&v), sizeof(T)); }
template <typename T>
inline T get(std::istream& f) {
    T v;
    f.read(reinterpret_cast<char*>(&v), sizeof(T));
    if (!f) throw std::runtime_error("serialization: read failed (unexpected end of file)");
    return v;
}
inline void write_tensor(std::ostream& f, const std::string& name, const Tensor& t0) {
    const Tensor t = t0.detach().cpu().contiguous();
    put<uint32_t>(f, (uint32_t)name.size());
    f.write(name.data(), (std::streamsize)name.size());
    put<uint8_t>(f, (uint8_t)ptor_code(t.scalar_type()));
    put<uint32_t>(f, (uint32_t)t.dim());
    for (int64_t s : t.sizes()) put<int64_t>(f, s);
    const uint64_t nbytes = (uint64_t)t.numel() * t.element_size();
    put<uint64_t>(f, nbytes);
    if (nbytes) f.write(reinterpret_cast<const char*>(t.data_ptr()), (std::streamsize)nbytes);
}
inline std::pair<std::string, Tensor> read_tensor(std::istream& f) {
    const uint32_t nl = get<uint32_t>(f);
    if (nl > (1u << 20)) throw std::runtime_error("serialization: implausible name length");
    std::string name(nl, '\0');
    f.read(&name[0], nl);
    const int code = get<uint8_t>(f);
    const uint32_t nd = get<uint32_t>(f);
    if (nd > 64) throw std::runtime_error("serialization: implausible rank");
    std::vector<int64_t> sizes(nd);
    for (auto& s : sizes) {
        s = get<int64_t>(f);
        if (s < 0) throw std::runtime_error("serialization: negative size");
    }
    const uint64_t nbytes = get<uint64_t>(f);
    Tensor t = torch::empty(sizes, torch::TensorOptions().dtype(ptor_dtype(code)));
    if (nbytes != (uint64_t)t.numel() * t.element_size()) throw std::runtime_error("serialization: nbytes mismatch");
    if (nbytes) {
        f.read(reinterpret_cast<char*>(t.data_ptr()), (std::streamsize)nbytes);
        if (!f) throw std::runtime_error("serialization: read failed (unexpected end of file)");
    }
    return {name, t};
}
inline uint64_t check_header(std::istream& f) {
    char magic[4];
    f.read(magic, 4);
    if (!f || std::string(magic, 4) != "PTOR") throw std::runtime_error("serialization: invalid file format (bad magic)");
    if (get<uint32_t>(f) != 1) throw std::runtime_error("serialization: unsupported format version");
    return get<uint64_t>(f);
}
}  // namespace detail

inline void save_state_dict(const OrderedStateDict& sd, const std::string& path) {
    std::ofstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("serialization: cannot open " + path);
    f.write("PTOR", 4);
    detail::put<uint32_t>(f, 1);
    detail::put<uint64_t>(f, sd.size());
    for (auto& kv : sd) detail::write_tensor(f, kv.first, kv.second);
}
inline OrderedStateDict load_state_dict(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("serialization: cannot open " + path);
    const uint64_t n = detail::check_header(f);
    OrderedStateDict out;
    for (uint64_t i = 0; i < n; ++i) out.push_back(detail::read_tensor(f));
    return out;
}
// A single tensor is stored under the name "tensor".
inline void save(const Tensor& t, const std::string& path) { save_state_dict({{"tensor", t}}, path); }
inline Tensor load(const std::string& path) {
    auto sd = load_state_dict(path);
    if (sd.size() != 1) throw std::runtime_error("serialization: " + path + " holds a state dict, not a single tensor");
    return sd[0].second;
}
// Module state: parameters and buffers by their dotted names.
inline OrderedStateDict state_dict(const torch::nn::Module& m) {
    OrderedStateDict out;
    for (auto& kv : m.named_parameters()) out.emplace_back(kv.key(), kv.value());
    for (auto& kv : m.named_buffers()) out.emplace_back(kv.key(), kv.value());
    return out;
}
inline void load_state_dict(torch::nn::Module& m, const OrderedStateDict& sd, bool strict = true) {
    torch::NoGradGuard ng;
    std::map<std::string, Tensor> have;
    for (auto& kv : m.named_parameters()) have[kv.key()] = kv.value();
    for (auto& kv : m.named_buffers()) have[kv.key()] = kv.value();
    size_t used = 0;
    for (auto& kv : sd) {
        auto it = have.find(kv.first);
        if (it == have.end()) {
            if (strict) throw std::runtime_error("load_state_dict: unexpected key " + kv.first);
            continue;
        }
        if (it->second.sizes() != kv.second.sizes()) throw std::runtime_error("load_state_dict: shape mismatch for " + kv.first);
        it->second.copy_(kv.second);
        ++used;
    }
    if (strict && used != have.size()) throw std::runtime_error("load_state_dict: missing keys");
}
inline void save(const torch::nn::Module& m, const std::string& path) { save_state_dict(state_dict(m), path); }
inline void load(torch::nn::Module& m, const std::string& path, bool strict = true) { load_state_dict(m, load_state_dict(path), strict); }

// PyTorch-compatible checkpoints of a name -> tensor dictionary.
inline void save_pytorch(const OrderedStateDict& sd, const std::string& path) {
    c10::Dict<std::string, Tensor> d;
    for (auto& kv : sd) d.insert(kv.first, kv.second.detach().cpu());
    const std::vector<char> bytes = torch::pickle_save(d);
    std::ofstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("serialization: cannot open " + path);
    f.write(bytes.data(), (std::streamsize)bytes.size());
}
inline OrderedStateDict load_pytorch(const std::string& path) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) throw std::runtime_error("serialization: cannot open " + path);
    std::vector<char> bytes((size_t)f.tellg());
    f.seekg(0);
    f.read(bytes.data(), (std::streamsize)bytes.size());
    const c10::IValue v = torch::pickle_load(bytes);
    OrderedStateDict out;
    if (v.isTensor()) {
        out.emplace_back("tensor", v.toTensor());
    } else if (v.isGenericDict()) {
        for (auto& kv : v.toGenericDict()) {
            if (!kv.key().isString() || !kv.value().isTensor()) throw std::runtime_error("load_pytorch: only name -> tensor dictionaries are accepted");
            out.emplace_back(kv.key().toStringRef(), kv.value().toTensor());
        }
    } else {
        throw std::runtime_error("load_pytorch: only tensors and name -> tensor dictionaries are accepted");
    }
    return out;
}

// ---- safetensors (u64 header length, JSON header, raw little-endian data) to and from name -> tensor dictionaries
namespace detail {
inline c10::ScalarType safetensors_dtype(const std::string& d) {
    if (d == "f64") return c10::kDouble;
    if (d == "f32") return c10::kFloat;
    if (d == "f16") return c10::kHalf;
    if (d == "bf16") return c10::kBFloat16;
    if (d == "i64") return c10::kLong;
    if (d == "i32") return c10::kInt;
    if (d == "i16") return c10::kShort;
    if (d == "i8") return c10::kChar;
    if (d == "u8") return c10::kByte;
    if (d == "bool") return c10::kBool;
    throw std::runtime_error("safetensors: unsupported dtype " + d);
}
inline const char* safetensors_name(c10::ScalarType t) {
    switch (t) {
        case c10::kDouble: return "F64";
        case c10::kFloat: return "F32";
        case c10::kHalf: return "F16";
        case c10::kBFloat16: return "BF16";
        case c10::kLong: return "I64";
        case c10::kInt: return "I32";
        case c10::kShort: return "I16";
        case c10::kChar: return "I8";
        case c10::kByte: return "U8";
        case c10::kBool: return "BOOL";
        default: throw std::runtime_error("safetensors: unsupported tensor dtype");
    }
}
}  // namespace detail

inline OrderedStateDict load_safetensors(const std::string& path) {
    io::loader::SafeTensorsFile f(path);
    std::ifstream in(path, std::ios::binary);
    OrderedStateDict out;
    for (const auto& name : f.keys()) {
        const auto& info = f.info(name);
        Tensor t = torch::empty(info.shape, torch::TensorOptions().dtype(detail::safetensors_dtype(info.dtype)));
        if ((uint64_t)t.nbytes() != info.nbytes) throw std::runtime_error("safetensors: size of " + name + " does not match its shape");
        in.seekg((std::streamoff)info.offset);
        in.read((char*)t.data_ptr(), (std::streamsize)info.nbytes);
        if (!in) throw std::runtime_error("safetensors: short read of " + name);
        out.emplace_back(name, t);
    }
    return out;
}
// Every file of a Hugging Face directory (or the siblings of a shard).
inline OrderedStateDict load_safetensors_sharded(const std::string& path) {
    OrderedStateDict out;
    for (const auto& file : io::loader::find_shard_files(path))
        for (auto& kv : load_safetensors(file)) out.push_back(std::move(kv));
    return out;
}
inline void save_safetensors(const OrderedStateDict& sd, const std::string& path, const std::map<std::string, std::string>& metadata = {}) {
    json::Value header = json::Value::object();
    if (!metadata.empty()) {
        json::Value m = json::Value::object();
        for (const auto& kv : metadata) m.set(kv.first, kv.second);
        header.set("__metadata__", m);
    }
    std::vector<Tensor> data;
    uint64_t offset = 0;
    for (const auto& kv : sd) {
        Tensor t = kv.second.detach().cpu().contiguous();
        json::Value e = json::Value::object(), shape = json::Value::array(), off = json::Value::array();
        for (auto d : t.sizes()) shape.push_back((long long)d);
        off.push_back((long long)offset);
        off.push_back((long long)(offset + t.nbytes()));
        e.set("dtype", detail::safetensors_name(t.scalar_type()));
        e.set("shape", shape);
        e.set("data_offsets", off);
        header.set(kv.first, e);
        offset += t.nbytes();
        data.push_back(t);
    }
    std::string h = header.dump();
    while (h.size() % 8) h.push_back(' ');               // the data section starts on an 8-byte boundary
    std::ofstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("serialization: cannot open " + path);
    const uint64_t n = h.size();
    f.write((const char*)&n, 8);
    f.write(h.data(), (std::streamsize)h.size());
    for (const auto& t : data) f.write((const char*)t.data_ptr(), (std::streamsize)t.nbytes());
}

}  // namespace promethorch
