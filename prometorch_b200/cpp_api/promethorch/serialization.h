// promethorch C++ API: checkpoint I/O.
//
//  * save / load / save_state_dict / load_state_dict: the PTOR container ("PTOR", u32 version 1, u64 count, then per
//    tensor: u32 name length, name, u8 dtype code, u32 ndim, i64 sizes, u64 nbytes, raw little-endian data;
//    torch/serialization.h:17-197 of the reference), byte-compatible with files the reference and the Python package
//    write.
//  * save_pytorch / load_pytorch: PyTorch zip checkpoints through libtorch's restricted unpickler (tensors and plain
//    containers only; it executes no code from the file), the policy of torch/serialization_pytorch.h:734-878.
#pragma once
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

}  // namespace promethorch
