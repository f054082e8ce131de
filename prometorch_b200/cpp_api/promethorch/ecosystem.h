// promethorch C++ API: the vision / text / audio helpers of the reference (torch/vision, torch/text, torch/audio) over libtorch.
//
//   vision::  load_pnm / save_pnm / load_image (PGM and PPM natively), ImageFolder (root/<class>/<file>), transforms on float
//             images [C, H, W]: Compose, Normalize, Resize (bilinear), CenterCrop, RandomCrop, RandomHorizontalFlip, Lambda
//   text::    Vocab, BasicTokenizer, CharTokenizer, WordPieceTokenizer, pad_sequence, sequence_lengths, padding_mask
//   audio::   hann_window, stft, spectrogram, mel_filterbank / melscale_fbanks, amplitude_to_db, mfcc, mu_law_encoding / decoding,
//             resample, save_wav / load_wav (16-bit PCM)
//
// The numbers equal those of the Python modules of the same names (vision/, text/, audio/ of this package) on the same inputs.
#pragma once
#include <dirent.h>
#include <sys/stat.h>
#include <torch/torch.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>
#include <functional>
#include <map>
#include <memory>
#include <random>
#include <sstream>
#include <string>
#include <vector>

namespace promethorch {

// ================================================================================================= vision
namespace vision {
using Tensor = at::Tensor;

// A binary (P5 / P6) or ASCII (P2 / P3) PGM / PPM file as float [C, H, W] in [0, 1].
inline Tensor load_pnm(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("load_pnm: cannot open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string data = ss.str();
    size_t pos = 0;
    std::vector<std::string> fields;
    while (fields.size() < 4) {                           // magic, width, height, maximum; white space and # comments between them
        while (pos < data.size() && (std::isspace((unsigned char)data[pos]) || data[pos] == '#')) {
            if (data[pos] == '#') while (pos < data.size() && data[pos] != '\n') ++pos;
            else ++pos;
        }
        const size_t start = pos;
        while (pos < data.size() && !std::isspace((unsigned char)data[pos])) ++pos;
        if (start == pos) throw std::runtime_error(path + ": truncated PNM header");
        fields.push_back(data.substr(start, pos - start));
    }
    const std::string& magic = fields[0];
    const int64_t w = std::stoll(fields[1]), h = std::stoll(fields[2]), maxval = std::stoll(fields[3]);
    if ((magic != "P2" && magic != "P3" && magic != "P5" && magic != "P6") || w <= 0 || h <= 0 || maxval <= 0 || maxval >= 65536)
        throw std::runtime_error(path + ": not a PGM / PPM file");
    const int64_t c = (magic == "P3" || magic == "P6") ? 3 : 1, n = w * h * c;
    Tensor vals = torch::empty({n}, torch::kFloat);
    float* out = vals.data_ptr<float>();
    if (magic == "P5" || magic == "P6") {
        ++pos;                                            // exactly one white-space byte ends the header
        const int64_t width = maxval > 255 ? 2 : 1;
        if ((int64_t)data.size() - (int64_t)pos < n * width) throw std::runtime_error(path + ": truncated pixel data");
        const unsigned char* p = (const unsigned char*)data.data() + pos;
        for (int64_t i = 0; i < n; ++i) out[i] = width == 2 ? (float)((p[2 * i] << 8) | p[2 * i + 1]) : (float)p[i];
    } else {
        std::istringstream rest(data.substr(pos));
        for (int64_t i = 0; i < n; ++i)
            if (!(rest >> out[i])) throw std::runtime_error(path + ": truncated pixel data");
    }
    return (vals / (double)maxval).view({h, w, c}).permute({2, 0, 1}).contiguous();
}
// [C, H, W] (C = 1 or 3) in [0, 1] as a binary PGM / PPM file.
inline void save_pnm(const std::string& path, const Tensor& x) {
    TORCH_CHECK(x.dim() == 3 && (x.size(0) == 1 || x.size(0) == 3), "save_pnm: expected [1 or 3, H, W]");
    Tensor b = (x.clamp(0, 1) * 255 + 0.5).to(torch::kByte).permute({1, 2, 0}).contiguous();
    std::ofstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("save_pnm: cannot open " + path);
    f << (x.size(0) == 3 ? "P6\n" : "P5\n") << x.size(2) << " " << x.size(1) << "\n255\n";
    f.write((const char*)b.data_ptr(), b.numel());
}
inline bool is_supported_image(const std::string& path) {
    std::string low = path;
    for (auto& ch : low) ch = (char)std::tolower((unsigned char)ch);
    for (const char* e : {".ppm", ".pgm", ".pnm"})
        if (low.size() >= 4 && low.compare(low.size() - 4, 4, e) == 0) return true;
    return false;
}
inline Tensor load_image(const std::string& path) {
    if (!is_supported_image(path)) throw std::runtime_error(path + ": unsupported image format (PGM / PPM are read natively)");
    return load_pnm(path);
}

namespace transforms {
using Transform = std::function<Tensor(const Tensor&)>;
inline Transform Compose(std::vector<Transform> ts) {
    return [ts](const Tensor& x) { Tensor y = x; for (const auto& t : ts) y = t(y); return y; };
}
inline Transform Lambda(Transform fn) { return fn; }
inline Transform Normalize(std::vector<double> mean, std::vector<double> std_) {
    Tensor m = torch::tensor(mean, torch::kFloat).view({-1, 1, 1}), s = torch::tensor(std_, torch::kFloat).view({-1, 1, 1});
    return [m, s](const Tensor& x) { return (x - m.to(x.dtype())) / s.to(x.dtype()); };
}
inline Transform Resize(int64_t h, int64_t w = -1) {
    if (w < 0) w = h;
    return [h, w](const Tensor& x) {
        namespace F = torch::nn::functional;
        return F::interpolate(x.unsqueeze(0), F::InterpolateFuncOptions().size(std::vector<int64_t>{h, w}).mode(torch::kBilinear).align_corners(false)).squeeze(0);
    };
}
inline Transform CenterCrop(int64_t th, int64_t tw = -1) {
    if (tw < 0) tw = th;
    return [th, tw](const Tensor& x) {
        const int64_t h = x.size(-2), w = x.size(-1), i = (h - th) / 2, j = (w - tw) / 2;
        return x.slice(-2, i, i + th).slice(-1, j, j + tw);
    };
}
inline Transform RandomCrop(int64_t th, int64_t tw = -1, int64_t padding = 0, uint64_t seed = 0) {
    if (tw < 0) tw = th;
    auto rng = std::make_shared<std::mt19937_64>(seed);
    return [th, tw, padding, rng](const Tensor& x) {
        Tensor y = padding ? torch::constant_pad_nd(x, {padding, padding, padding, padding}, 0) : x;
        const int64_t h = y.size(-2), w = y.size(-1);
        const int64_t i = std::uniform_int_distribution<int64_t>(0, h - th)(*rng), j = std::uniform_int_distribution<int64_t>(0, w - tw)(*rng);
        return y.slice(-2, i, i + th).slice(-1, j, j + tw);
    };
}
inline Transform RandomHorizontalFlip(double p = 0.5, uint64_t seed = 0) {
    auto rng = std::make_shared<std::mt19937_64>(seed);
    return [p, rng](const Tensor& x) { return std::uniform_real_distribution<double>(0, 1)(*rng) < p ? x.flip({-1}) : x; };
}
}  // namespace transforms

// root/<class>/<file>: classes are the sorted sub-directories, samples the supported image files inside them.
class ImageFolder {
 public:
    explicit ImageFolder(const std::string& root, transforms::Transform transform = nullptr) : transform_(std::move(transform)) {
        for (const auto& c : list(root, true)) classes.push_back(c);
        for (size_t i = 0; i < classes.size(); ++i)
            for (const auto& f : list(root + "/" + classes[i], false))
                if (is_supported_image(f)) samples.emplace_back(root + "/" + classes[i] + "/" + f, (int64_t)i);
    }
    size_t size() const { return samples.size(); }
    std::pair<Tensor, int64_t> get(size_t i) const {
        Tensor x = load_image(samples.at(i).first);
        return {transform_ ? transform_(x) : x, samples[i].second};
    }
    std::vector<std::string> classes;
    std::vector<std::pair<std::string, int64_t>> samples;

 private:
    static std::vector<std::string> list(const std::string& d, bool dirs) {
        std::vector<std::string> out;
        if (DIR* dir = ::opendir(d.c_str())) {
            while (struct dirent* e = ::readdir(dir)) {
                const std::string n = e->d_name;
                if (n == "." || n == "..") continue;
                struct stat st;
                if (::stat((d + "/" + n).c_str(), &st) == 0 && (dirs ? S_ISDIR(st.st_mode) : S_ISREG(st.st_mode))) out.push_back(n);
            }
            ::closedir(dir);
        }
        std::sort(out.begin(), out.end());
        return out;
    }
    transforms::Transform transform_;
};
}  // namespace vision

// ================================================================================================= text
namespace text {
using Tensor = at::Tensor;

inline std::vector<std::string> split_whitespace(const std::string& s) {
    std::istringstream in(s);
    std::vector<std::string> out;
    std::string w;
    while (in >> w) out.push_back(w);
    return out;
}

class Vocab {
 public:
    explicit Vocab(const std::vector<std::string>& tokens = {}, const std::vector<std::string>& specials = {"<pad>", "<unk>"}) {
        for (const auto& t : specials) add(t);
        for (const auto& t : tokens) add(t);
        auto it = stoi.find("<unk>");
        unk = it == stoi.end() ? 0 : it->second;
    }
    // Words of the texts by falling frequency (ties in order of first appearance), at least min_freq times.
    static Vocab build(const std::vector<std::string>& texts, int64_t min_freq = 1, const std::vector<std::string>& specials = {"<pad>", "<unk>"}) {
        std::map<std::string, std::pair<int64_t, int64_t>> count;       // word -> (count, first seen)
        int64_t seen = 0;
        for (const auto& t : texts)
            for (const auto& w : split_whitespace(t)) {
                auto it = count.find(w);
                if (it == count.end()) count[w] = {1, seen++};
                else ++it->second.first;
            }
        std::vector<std::pair<std::string, std::pair<int64_t, int64_t>>> v(count.begin(), count.end());
        std::stable_sort(v.begin(), v.end(), [](const auto& a, const auto& b) { return a.second.first != b.second.first ? a.second.first > b.second.first : a.second.second < b.second.second; });
        std::vector<std::string> toks;
        for (const auto& kv : v)
            if (kv.second.first >= min_freq) toks.push_back(kv.first);
        return Vocab(toks, specials);
    }
    int64_t add(const std::string& t) {
        auto it = stoi.find(t);
        if (it != stoi.end()) return it->second;
        stoi[t] = (int64_t)itos.size();
        itos.push_back(t);
        return (int64_t)itos.size() - 1;
    }
    size_t size() const { return itos.size(); }
    std::vector<int64_t> encode(const std::string& textv) const {
        std::vector<int64_t> out;
        for (const auto& w : split_whitespace(textv)) { auto it = stoi.find(w); out.push_back(it == stoi.end() ? unk : it->second); }
        return out;
    }
    std::string decode(const std::vector<int64_t>& ids) const {
        std::string out;
        for (size_t i = 0; i < ids.size(); ++i) out += (i ? " " : "") + itos.at((size_t)ids[i]);
        return out;
    }
    std::vector<std::string> itos;
    std::map<std::string, int64_t> stoi;
    int64_t unk = 0;
};

// Lower-cases (optionally) and cuts ASCII punctuation off as tokens of its own; words are runs of letters, digits, '_' and
// bytes of multi-byte characters.
class BasicTokenizer {
 public:
    explicit BasicTokenizer(bool lowercase = true) : lowercase_(lowercase) {}
    std::vector<std::string> tokenize(const std::string& textv) const {
        std::vector<std::string> out;
        std::string cur;
        for (unsigned char c : textv) {
            const bool word = std::isalnum(c) || c == '_' || c >= 0x80;
            if (word) cur.push_back(lowercase_ && c < 0x80 ? (char)std::tolower(c) : (char)c);
            else {
                if (!cur.empty()) { out.push_back(cur); cur.clear(); }
                if (!std::isspace(c)) out.emplace_back(1, (char)c);
            }
        }
        if (!cur.empty()) out.push_back(cur);
        return out;
    }

 private:
    bool lowercase_;
};

// One id per byte-string character of the corpus (UTF-8 aware); id 0 is the unknown character.
class CharTokenizer {
 public:
    explicit CharTokenizer(const std::string& corpus = "") {
        std::vector<std::string> chars = split_chars(corpus);
        std::sort(chars.begin(), chars.end());
        chars.erase(std::unique(chars.begin(), chars.end()), chars.end());
        itos.push_back("<unk>");
        for (const auto& c : chars) { stoi[c] = (int64_t)itos.size(); itos.push_back(c); }
    }
    size_t size() const { return itos.size(); }
    std::vector<int64_t> encode(const std::string& textv) const {
        std::vector<int64_t> out;
        for (const auto& c : split_chars(textv)) { auto it = stoi.find(c); out.push_back(it == stoi.end() ? 0 : it->second); }
        return out;
    }
    std::string decode(const std::vector<int64_t>& ids) const {
        std::string out;
        for (auto i : ids)
            if (i > 0 && i < (int64_t)itos.size()) out += itos[(size_t)i];
        return out;
    }
    static std::vector<std::string> split_chars(const std::string& s) {
        std::vector<std::string> out;
        for (size_t i = 0; i < s.size();) {
            const unsigned char c = (unsigned char)s[i];
            size_t n = c >= 0xF0 ? 4 : (c >= 0xE0 ? 3 : (c >= 0xC0 ? 2 : 1));
            n = std::min(n, s.size() - i);
            out.push_back(s.substr(i, n));
            i += n;
        }
        return out;
    }
    std::vector<std::string> itos;
    std::map<std::string, int64_t> stoi;
};

// Greedy longest-match-first word pieces ("##" marks a continuation); a word that cannot be covered becomes the unknown token.
class WordPieceTokenizer {
 public:
    explicit WordPieceTokenizer(const std::vector<std::string>& vocab, std::string unk = "[UNK]", size_t max_chars = 100) : unk_(std::move(unk)), max_chars_(max_chars) {
        for (size_t i = 0; i < vocab.size(); ++i) vocab_[vocab[i]] = (int64_t)i;
    }
    std::vector<std::string> tokenize(const std::string& textv) const {
        std::vector<std::string> out;
        for (const auto& w : split_whitespace(textv)) {
            const auto chars = CharTokenizer::split_chars(w);
            if (chars.size() > max_chars_) { out.push_back(unk_); continue; }
            std::vector<std::string> pieces;
            size_t i = 0;
            bool bad = false;
            while (i < chars.size()) {
                size_t j = chars.size();
                std::string cur;
                while (i < j) {
                    std::string sub = i > 0 ? "##" : "";
                    for (size_t k = i; k < j; ++k) sub += chars[k];
                    if (vocab_.count(sub)) { cur = sub; break; }
                    --j;
                }
                if (cur.empty()) { bad = true; break; }
                pieces.push_back(cur);
                i = j;
            }
            if (bad) out.push_back(unk_);
            else out.insert(out.end(), pieces.begin(), pieces.end());
        }
        return out;
    }
    std::vector<int64_t> encode(const std::string& textv) const {
        std::vector<int64_t> out;
        auto u = vocab_.find(unk_);
        for (const auto& t : tokenize(textv)) { auto it = vocab_.find(t); out.push_back(it != vocab_.end() ? it->second : (u != vocab_.end() ? u->second : 0)); }
        return out;
    }

 private:
    std::map<std::string, int64_t> vocab_;
    std::string unk_;
    size_t max_chars_;
};

// Lists of ids -> one [B, T] int64 tensor, cut or padded to max_len (default: the longest).
inline Tensor pad_sequence(const std::vector<std::vector<int64_t>>& batch, int64_t padding_value = 0, bool batch_first = true, int64_t max_len = -1) {
    int64_t T = max_len;
    if (T < 0) { T = 0; for (const auto& s : batch) T = std::max<int64_t>(T, (int64_t)s.size()); }
    Tensor out = torch::full({(int64_t)batch.size(), T}, padding_value, torch::kLong);
    for (size_t i = 0; i < batch.size(); ++i) {
        const int64_t n = std::min<int64_t>((int64_t)batch[i].size(), T);
        if (n) out[(int64_t)i].slice(0, 0, n).copy_(torch::tensor(std::vector<int64_t>(batch[i].begin(), batch[i].begin() + n), torch::kLong));
    }
    return batch_first ? out : out.t().contiguous();
}
inline Tensor sequence_lengths(const std::vector<std::vector<int64_t>>& batch) {
    std::vector<int64_t> l;
    for (const auto& s : batch) l.push_back((int64_t)s.size());
    return torch::tensor(l, torch::kLong);
}
// [B, T] bool, true where a position holds padding.
inline Tensor padding_mask(const std::vector<std::vector<int64_t>>& batch, int64_t max_len = -1) {
    Tensor lens = sequence_lengths(batch);
    const int64_t T = max_len >= 0 ? max_len : (batch.empty() ? 0 : lens.max().item<int64_t>());
    return torch::arange(T).unsqueeze(0) >= lens.clamp_max(T).unsqueeze(1);
}
}  // namespace text

// ================================================================================================= audio
namespace audio {
using Tensor = at::Tensor;

inline Tensor hann_window(int64_t n) { return torch::hann_window(n); }
inline Tensor stft(const Tensor& x, int64_t n_fft = 400, int64_t hop_length = 160, Tensor window = {}) {
    if (!window.defined()) window = torch::hann_window(n_fft, x.options().dtype(torch::kFloat));
    return torch::stft(x, n_fft, hop_length, c10::nullopt, window, /*center=*/true, /*pad_mode=*/"reflect", /*normalized=*/false, /*onesided=*/c10::nullopt, /*return_complex=*/true);
}
// |STFT|^power, [..., n_fft / 2 + 1, frames].
inline Tensor spectrogram(const Tensor& x, int64_t n_fft = 400, int64_t hop_length = 160, Tensor window = {}, double power = 2.0) {
    return stft(x, n_fft, hop_length, std::move(window)).abs().pow(power);
}
inline double hz_to_mel(double f) { return 2595.0 * std::log10(1.0 + f / 700.0); }
// Triangular mel filters [n_mels, n_fft / 2 + 1].
inline Tensor mel_filterbank(int64_t n_mels, int64_t n_fft, int64_t sample_rate) {
    Tensor mels = torch::linspace(hz_to_mel(0.0), hz_to_mel(sample_rate / 2.0), n_mels + 2);
    Tensor hz = 700.0 * (torch::pow(10.0, mels / 2595.0) - 1.0);
    Tensor bins = torch::floor((double)(n_fft + 1) * hz / (double)sample_rate).to(torch::kLong);
    Tensor fb = torch::zeros({n_mels, n_fft / 2 + 1});
    auto acc = fb.accessor<float, 2>();
    auto b = bins.accessor<int64_t, 1>();
    for (int64_t m = 1; m <= n_mels; ++m) {
        const int64_t l = b[m - 1], c = b[m], r = b[m + 1];
        for (int64_t k = l; k < c; ++k) acc[m - 1][k] = (float)(k - l) / (float)std::max<int64_t>(c - l, 1);
        for (int64_t k = c; k < r; ++k) acc[m - 1][k] = (float)(r - k) / (float)std::max<int64_t>(r - c, 1);
    }
    return fb;
}
inline Tensor melscale_fbanks(int64_t n_freqs, int64_t n_mels, int64_t sample_rate) { return mel_filterbank(n_mels, (n_freqs - 1) * 2, sample_rate).t().contiguous(); }
inline Tensor amplitude_to_db(const Tensor& x, double multiplier = 10.0, double amin = 1e-10, double db_multiplier = 0.0, double top_db = -1.0) {
    Tensor db = multiplier * torch::log10(x.clamp_min(amin)) - multiplier * db_multiplier;
    return top_db >= 0 ? torch::maximum(db, db.amax() - top_db) : db;
}
inline Tensor mfcc(const Tensor& x, int64_t sample_rate = 16000, int64_t n_mfcc = 13, int64_t n_mels = 40, int64_t n_fft = 400, int64_t hop_length = 160) {
    Tensor power = stft(x, n_fft, hop_length).abs().pow(2);
    Tensor logmel = torch::log(torch::matmul(mel_filterbank(n_mels, n_fft, sample_rate), power) + 1e-10);
    Tensor n = torch::arange(n_mels, torch::kFloat);
    Tensor dct = torch::cos(M_PI / (double)n_mels * (n.unsqueeze(0) + 0.5) * torch::arange(n_mfcc, torch::kFloat).unsqueeze(1)) * std::sqrt(2.0 / (double)n_mels);
    return torch::matmul(dct, logmel);
}
// Signal in [-1, 1] -> integers in [0, quantization_channels).
inline Tensor mu_law_encoding(const Tensor& x, int64_t quantization_channels = 256) {
    const double mu = (double)quantization_channels - 1.0;
    Tensor y = torch::sign(x) * torch::log1p(mu * x.abs().clamp_max(1.0)) / std::log1p(mu);
    return ((y + 1) / 2 * mu + 0.5).to(torch::kLong);
}
inline Tensor mu_law_decoding(const Tensor& q, int64_t quantization_channels = 256) {
    const double mu = (double)quantization_channels - 1.0;
    Tensor y = q.to(torch::kFloat) / mu * 2 - 1;
    return torch::sign(y) * (torch::exp(y.abs() * std::log1p(mu)) - 1) / mu;
}
inline Tensor resample(const Tensor& x, int64_t orig_rate, int64_t new_rate) {
    namespace F = torch::nn::functional;
    const int64_t n = (int64_t)std::llround((double)x.size(-1) * (double)new_rate / (double)orig_rate);
    return F::interpolate(x.reshape({1, 1, -1}), F::InterpolateFuncOptions().size(std::vector<int64_t>{n}).mode(torch::kLinear).align_corners(false)).reshape({n});
}
inline void save_wav(const std::string& path, const Tensor& x, int64_t sample_rate = 16000) {
    Tensor pcm = (x.clamp(-1, 1) * 32767).to(torch::kShort).cpu().contiguous();
    const uint32_t bytes = (uint32_t)(pcm.numel() * 2), riff = 36 + bytes, fmt = 16, sr = (uint32_t)sample_rate, byte_rate = sr * 2;
    const uint16_t pcm_tag = 1, channels = 1, block = 2, bits = 16;
    std::ofstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("save_wav: cannot open " + path);
    f.write("RIFF", 4); f.write((const char*)&riff, 4); f.write("WAVEfmt ", 8); f.write((const char*)&fmt, 4);
    f.write((const char*)&pcm_tag, 2); f.write((const char*)&channels, 2); f.write((const char*)&sr, 4); f.write((const char*)&byte_rate, 4);
    f.write((const char*)&block, 2); f.write((const char*)&bits, 2); f.write("data", 4); f.write((const char*)&bytes, 4);
    f.write((const char*)pcm.data_ptr(), bytes);
}
// (samples in [-1, 1], sample rate) of a 16-bit PCM file.
inline std::pair<Tensor, int64_t> load_wav(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("load_wav: cannot open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string b = ss.str();
    if (b.size() < 44 || b.compare(0, 4, "RIFF") != 0) throw std::runtime_error(path + ": not a RIFF file");
    uint32_t sr, n;
    std::memcpy(&sr, b.data() + 24, 4);
    const size_t i = b.find("data");
    if (i == std::string::npos || i + 8 > b.size()) throw std::runtime_error(path + ": no data chunk");
    std::memcpy(&n, b.data() + i + 4, 4);
    n = (uint32_t)std::min<size_t>(n, b.size() - i - 8);
    Tensor pcm = torch::empty({(int64_t)(n / 2)}, torch::kShort);
    std::memcpy(pcm.data_ptr(), b.data() + i + 8, (n / 2) * 2);
    return {pcm.to(torch::kFloat) / 32767.0, (int64_t)sr};
}
}  // namespace audio

}  // namespace promethorch
