// promethorch C++ API: the model exporters of the reference (torch/onnx/export.h, torch/mlir/export.h, torch/mobile/executor.h)
// for chains of Linear layers and activations held in a torch::nn::Sequential.
//
//   onnx::export_model(seq, input_shape, path)     ONNX protobuf written by hand (Gemm / Relu / Sigmoid / Tanh / Softmax nodes)
//   mlir::export_mlir(seq, input_shape[, path])    MLIR text (linalg / arith sketch)
//   mobile::export_model(seq, path)                the flat PTMB format; mobile::MobileExecutor(path).run(x) executes it
//
// The files are byte-identical to what the Python exporters of this package write for the same model.
#pragma once
#include <torch/torch.h>

#include <cstdint>
#include <fstream>
#include <functional>
#include <sstream>
#include <string>
#include <vector>

namespace promethorch {

namespace export_detail {
enum Kind : uint8_t { None = 0, Linear = 1, ReLU = 2, Sigmoid = 3, Tanh = 4, GELU = 5, SiLU = 6, Softmax = 7 };
struct Op {
    Kind kind = None;
    at::Tensor weight, bias;
};
// The Linear layers and activations of a Sequential, in order (nested Sequentials are walked depth first).
inline void walk(const torch::nn::Module& m, std::vector<Op>& out) {
    for (const auto& child : m.children()) {
        if (auto* l = child->as<torch::nn::LinearImpl>()) out.push_back({Linear, l->weight, l->bias});
        else if (child->as<torch::nn::ReLUImpl>()) out.push_back({ReLU, {}, {}});
        else if (child->as<torch::nn::SigmoidImpl>()) out.push_back({Sigmoid, {}, {}});
        else if (child->as<torch::nn::TanhImpl>()) out.push_back({Tanh, {}, {}});
        else if (child->as<torch::nn::GELUImpl>()) out.push_back({GELU, {}, {}});
        else if (child->as<torch::nn::SiLUImpl>()) out.push_back({SiLU, {}, {}});
        else if (child->as<torch::nn::SoftmaxImpl>()) out.push_back({Softmax, {}, {}});
        else walk(*child, out);
    }
}
inline std::string shape_str(const std::vector<int64_t>& s) {
    std::string out;
    for (size_t i = 0; i < s.size(); ++i) out += (i ? "x" : "") + std::to_string(s[i]);
    return out;
}
}  // namespace export_detail

namespace onnx {
namespace pb {
inline std::string varint(uint64_t n) {
    std::string out;
    for (;;) {
        const uint8_t b = n & 0x7F;
        n >>= 7;
        out.push_back((char)(b | (n ? 0x80 : 0)));
        if (!n) return out;
    }
}
inline std::string field(int num, int wt, const std::string& payload) { return varint(((uint64_t)num << 3) | (uint64_t)wt) + (wt == 2 ? varint(payload.size()) + payload : payload); }
inline std::string str(int num, const std::string& s) { return field(num, 2, s); }
inline std::string tensor(const std::string& name, const at::Tensor& t0) {
    at::Tensor t = t0.detach().to(torch::kFloat).contiguous().cpu();
    std::string b;
    for (auto d : t.sizes()) b += field(1, 0, varint((uint64_t)d));
    return b + field(2, 0, varint(1)) + str(8, name) + field(9, 2, std::string((const char*)t.data_ptr(), (size_t)t.nbytes()));
}
inline std::string value_info(const std::string& name, const std::vector<int64_t>& shape) {
    std::string dims;
    for (auto d : shape) dims += field(1, 2, field(1, 0, varint((uint64_t)d)));
    const std::string ttype = field(1, 0, varint(1)) + field(2, 2, dims);
    return str(1, name) + field(2, 2, field(1, 2, ttype));
}
inline std::string node(const std::string& op, const std::vector<std::string>& ins, const std::vector<std::string>& outs) {
    std::string b;
    for (const auto& i : ins) b += str(1, i);
    for (const auto& o : outs) b += str(2, o);
    return b + str(4, op);
}
}  // namespace pb

inline std::string export_model(const torch::nn::Module& model, const std::vector<int64_t>& input_shape, const std::string& path, int opset = 13) {
    std::vector<export_detail::Op> ops;
    export_detail::walk(model, ops);
    std::vector<std::string> nodes, inits;
    std::string cur = "input";
    std::vector<int64_t> shape = input_shape;
    int k = 0;
    for (const auto& op : ops) {
        const std::string ks = std::to_string(k);
        if (op.kind == export_detail::Linear) {
            inits.push_back(pb::tensor("w" + ks, op.weight.t()));
            inits.push_back(pb::tensor("b" + ks, op.bias.defined() ? op.bias : torch::zeros({op.weight.size(0)})));
            nodes.push_back(pb::node("Gemm", {cur, "w" + ks, "b" + ks}, {"h" + ks}));
            cur = "h" + ks;
            shape.back() = op.weight.size(0);
            ++k;
        } else if (op.kind == export_detail::ReLU || op.kind == export_detail::Sigmoid || op.kind == export_detail::Tanh || op.kind == export_detail::Softmax) {
            const char* name = op.kind == export_detail::ReLU ? "Relu" : (op.kind == export_detail::Sigmoid ? "Sigmoid" : (op.kind == export_detail::Tanh ? "Tanh" : "Softmax"));
            nodes.push_back(pb::node(name, {cur}, {"a" + ks}));
            cur = "a" + ks;
            ++k;
        }
    }
    std::string graph;
    for (const auto& n : nodes) graph += pb::field(1, 2, n);
    graph += pb::str(2, "prometorch_b200");
    for (const auto& t : inits) graph += pb::field(5, 2, t);
    graph += pb::field(11, 2, pb::value_info("input", input_shape)) + pb::field(12, 2, pb::value_info(cur, shape));
    const std::string model_pb = pb::field(1, 0, pb::varint(8)) + pb::str(2, "prometorch_b200") + pb::field(7, 2, graph) +
                                 pb::field(8, 2, pb::str(1, "") + pb::field(2, 0, pb::varint((uint64_t)opset)));
    std::ofstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("onnx::export_model: cannot open " + path);
    f.write(model_pb.data(), (std::streamsize)model_pb.size());
    return path;
}
}  // namespace onnx

namespace mlir {
inline std::string export_mlir(const torch::nn::Module& model, const std::vector<int64_t>& input_shape, const std::string& path = "") {
    using export_detail::shape_str;
    std::vector<export_detail::Op> ops;
    export_detail::walk(model, ops);
    std::vector<std::string> lines{"module {", "  func.func @forward(%arg0: tensor<" + shape_str(input_shape) + "xf32>) -> tensor<*xf32> {"};
    std::string cur = "%arg0";
    std::vector<int64_t> shape = input_shape;
    int k = 0;
    for (const auto& op : ops) {
        const std::string ks = std::to_string(k);
        if (op.kind == export_detail::Linear) {
            const std::string wshape = std::to_string(op.weight.size(0)) + "x" + std::to_string(op.weight.size(1));
            std::vector<int64_t> out_shape = shape;
            out_shape.back() = op.weight.size(0);
            lines.push_back("    %w" + ks + " = arith.constant dense_resource<w" + ks + "> : tensor<" + wshape + "xf32>");
            lines.push_back("    %h" + ks + " = linalg.matmul_transpose_b ins(" + cur + ", %w" + ks + " : tensor<" + shape_str(shape) + "xf32>, tensor<" + wshape +
                            "xf32>) -> tensor<" + shape_str(out_shape) + "xf32>");
            cur = "%h" + ks;
            shape = out_shape;
            ++k;
        } else if (op.kind != export_detail::Softmax && op.kind != export_detail::None) {
            static const char* names[] = {"", "", "relu", "sigmoid", "tanh", "gelu", "silu"};
            lines.push_back("    %a" + ks + " = \"prometorch." + names[op.kind] + "\"(" + cur + ") : (tensor<" + shape_str(shape) + "xf32>) -> tensor<" + shape_str(shape) + "xf32>");
            cur = "%a" + ks;
            ++k;
        }
    }
    lines.push_back("    return " + cur + " : tensor<" + shape_str(shape) + "xf32>");
    lines.push_back("  }");
    lines.push_back("}");
    std::string textv;
    for (size_t i = 0; i < lines.size(); ++i) textv += (i ? "\n" : "") + lines[i];
    if (!path.empty()) {
        std::ofstream f(path);
        if (!f) throw std::runtime_error("mlir::export_mlir: cannot open " + path);
        f << textv;
    }
    return textv;
}
}  // namespace mlir

namespace mobile {
// "PTMB", u32 version 1, u32 op count; per op: u8 kind, and for a Linear: weight, u8 has-bias, bias (tensor = u32 rank, i64 sizes, fp32 data).
inline void write_tensor(std::ofstream& f, const at::Tensor& t0) {
    at::Tensor t = t0.detach().to(torch::kFloat).contiguous().cpu();
    const uint32_t nd = (uint32_t)t.dim();
    f.write((const char*)&nd, 4);
    for (auto s : t.sizes()) { const int64_t v = s; f.write((const char*)&v, 8); }
    f.write((const char*)t.data_ptr(), (std::streamsize)t.nbytes());
}
inline void export_model(const torch::nn::Module& model, const std::string& path) {
    std::vector<export_detail::Op> ops;
    export_detail::walk(model, ops);
    std::ofstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("mobile::export_model: cannot open " + path);
    const uint32_t version = 1, n = (uint32_t)ops.size();
    f.write("PTMB", 4);
    f.write((const char*)&version, 4);
    f.write((const char*)&n, 4);
    for (const auto& op : ops) {
        const uint8_t kind = op.kind;
        f.write((const char*)&kind, 1);
        if (op.kind == export_detail::Linear) {
            write_tensor(f, op.weight);
            const uint8_t has = op.bias.defined();
            f.write((const char*)&has, 1);
            if (has) write_tensor(f, op.bias);
        }
    }
}
class MobileExecutor {
 public:
    explicit MobileExecutor(const std::string& path) {
        std::ifstream f(path, std::ios::binary);
        char magic[4];
        if (!f || !f.read(magic, 4) || std::string(magic, 4) != "PTMB") throw std::runtime_error(path + ": not a PTMB file");
        uint32_t version, n;
        f.read((char*)&version, 4);
        f.read((char*)&n, 4);
        for (uint32_t i = 0; i < n; ++i) {
            uint8_t kind;
            f.read((char*)&kind, 1);
            export_detail::Op op;
            op.kind = (export_detail::Kind)kind;
            if (kind == export_detail::Linear) {
                op.weight = read_tensor(f);
                uint8_t has;
                f.read((char*)&has, 1);
                if (has) op.bias = read_tensor(f);
            }
            if (!f) throw std::runtime_error(path + ": truncated PTMB file");
            ops_.push_back(op);
        }
    }
    at::Tensor run(at::Tensor x) const {
        torch::NoGradGuard ng;
        for (const auto& op : ops_) {
            switch (op.kind) {
                case export_detail::Linear: x = torch::nn::functional::linear(x, op.weight, op.bias); break;
                case export_detail::ReLU: x = torch::relu(x); break;
                case export_detail::Sigmoid: x = torch::sigmoid(x); break;
                case export_detail::Tanh: x = torch::tanh(x); break;
                case export_detail::GELU: x = torch::gelu(x); break;
                case export_detail::SiLU: x = torch::silu(x); break;
                case export_detail::Softmax: x = torch::softmax(x, -1); break;
                default: throw std::runtime_error("MobileExecutor: unknown op kind");
            }
        }
        return x;
    }
    size_t num_ops() const { return ops_.size(); }

 private:
    static at::Tensor read_tensor(std::ifstream& f) {
        uint32_t nd;
        f.read((char*)&nd, 4);
        if (nd > 8) throw std::runtime_error("PTMB: implausible rank");
        std::vector<int64_t> shape(nd);
        for (auto& s : shape) f.read((char*)&s, 8);
        at::Tensor t = torch::empty(shape, torch::kFloat);
        f.read((char*)t.data_ptr(), (std::streamsize)t.nbytes());
        return t;
    }
    std::vector<export_detail::Op> ops_;
};
}  // namespace mobile

}  // namespace promethorch
