// promethorch C++ API: the tokenizer a GGUF file describes (tokenizer.ggml.*).
//
// Two models: SentencePiece-style BPE ("llama": U+2581 as the word boundary, merges ordered by vocabulary score, <0xNN>
// byte fall-back) and GPT-2 byte-level BPE ("gpt2": pre-tokeniser pattern, merges by rank).  Special tokens (control /
// user-defined types, and every <|...|> entry) are split out before either runs.  Counterpart of the reference's
// GGUFTokenizer (torch/io/tokenizer.h:24-646); it produces the ids of the Python class of this package on the same text.
//
// The GPT-2 pattern needs the Unicode classes "letter" and "number".  Without a Unicode database they are decided by
// ranges: ASCII exactly; above ASCII, a code point is a letter unless it lies in a block of punctuation, symbols,
// combining marks, digits or emoji listed in `classify`.  Text in the Latin, Greek, Cyrillic, Hebrew, Arabic, Indic and
// CJK scripts splits as under the true classes; rare symbols outside the listed blocks may join a neighbouring word.
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <map>
#include <queue>
#include <sstream>
#include <string>
#include <tuple>
#include <unordered_map>
#include <utility>
#include <vector>

#include "gguf_reader.h"
#include "json.h"

namespace promethorch {
namespace io {

namespace utf8 {
// Decodes one code point at s[i].  A malformed sequence comes back as 0xFFFD with `len` = the bytes of its longest
// well-formed prefix (at least one), which is how a lenient decoder counts replacement characters; `ok` says which.
inline uint32_t next(const std::string& s, size_t i, int& len, bool* ok = nullptr) {
    const unsigned char c = (unsigned char)s[i];
    if (ok) *ok = true;
    if (c < 0x80) { len = 1; return c; }
    const int n = c >= 0xF0 && c <= 0xF4 ? 4 : (c >= 0xE0 && c < 0xF0 ? 3 : (c >= 0xC2 && c < 0xE0 ? 2 : 0));
    if (ok) *ok = false;
    if (n == 0) { len = 1; return 0xFFFD; }
    uint32_t cp = n == 2 ? (c & 0x1Fu) : (n == 3 ? (c & 0x0Fu) : (c & 0x07u));
    int k = 1;
    for (; k < n && i + (size_t)k < s.size(); ++k) {
        const unsigned char d = (unsigned char)s[i + (size_t)k];
        unsigned char lo = 0x80, hi = 0xBF;
        if (k == 1) {                                   // no overlong forms, no surrogates, nothing above U+10FFFF
            if (c == 0xE0) lo = 0xA0;
            if (c == 0xED) hi = 0x9F;
            if (c == 0xF0) lo = 0x90;
            if (c == 0xF4) hi = 0x8F;
        }
        if (d < lo || d > hi) break;
        cp = (cp << 6) | (d & 0x3Fu);
    }
    len = k;
    if (k < n) return 0xFFFD;
    if (ok) *ok = true;
    return cp;
}
inline void append(uint32_t c, std::string& out) {
    if (c < 0x80) out.push_back((char)c);
    else if (c < 0x800) { out.push_back((char)(0xC0 | (c >> 6))); out.push_back((char)(0x80 | (c & 0x3F))); }
    else if (c < 0x10000) { out.push_back((char)(0xE0 | (c >> 12))); out.push_back((char)(0x80 | ((c >> 6) & 0x3F))); out.push_back((char)(0x80 | (c & 0x3F))); }
    else { out.push_back((char)(0xF0 | (c >> 18))); out.push_back((char)(0x80 | ((c >> 12) & 0x3F))); out.push_back((char)(0x80 | ((c >> 6) & 0x3F))); out.push_back((char)(0x80 | (c & 0x3F))); }
}
// Malformed sequences become U+FFFD, as a lenient decoder does.
inline std::string sanitize(const std::string& s) {
    std::string out;
    for (size_t i = 0; i < s.size();) {
        int len;
        bool ok;
        next(s, i, len, &ok);
        if (ok) out.append(s, i, (size_t)len);
        else out += "\xEF\xBF\xBD";
        i += (size_t)len;
    }
    return out;
}
}  // namespace utf8

class GGUFTokenizer {
 public:
    enum CharClass { Space, Letter, Number, Other };
    // Which split pattern the vocabulary was trained with (tokenizer.ggml.pre): GPT-2's, the qwen2 one (single digits, one leading
    // symbol joins a word, newlines close a run) or the llama-3 one (digits in groups of up to three).
    enum PreStyle { GPT2, Qwen2, Llama3 };
    static PreStyle style_of(std::string pre) {
        for (auto& c : pre) c = (char)std::tolower((unsigned char)c);
        for (const char* n : {"qwen2", "qwen", "deepseek-r1-qwen", "qwen3"})
            if (pre == n) return Qwen2;
        for (const char* n : {"llama3", "llama-bpe", "llama-v3", "llama4", "smaug-bpe"})
            if (pre == n) return Llama3;
        return GPT2;
    }

    GGUFTokenizer() = default;
    GGUFTokenizer(std::vector<std::string> tokens, std::string model = "llama", std::vector<float> scores = {}, const std::vector<std::string>& merges = {},
                  std::vector<int> token_types = {}, int bos_id = -1, int eos_id = -1, bool add_bos = false, const std::string& pre = "")
        : tokens_(std::move(tokens)), model_(std::move(model)), scores_(std::move(scores)), types_(std::move(token_types)), bos_id_(bos_id),
          eos_id_(eos_id), add_bos_(add_bos), style_(style_of(pre)) {
        if (scores_.size() != tokens_.size()) scores_.assign(tokens_.size(), 0.0f);
        if (types_.size() != tokens_.size()) types_.assign(tokens_.size(), 1);
        for (size_t i = 0; i < tokens_.size(); ++i) vocab_[tokens_[i]] = (int)i;        // a repeated entry keeps its last id
        for (size_t r = 0; r < merges.size(); ++r) {
            const size_t sp = merges[r].find(' ');
            if (sp == std::string::npos) continue;
            ranks_[merges[r].substr(0, sp) + '\x01' + merges[r].substr(sp + 1)] = (int)r;
        }
        for (int b = 0; b < 256; ++b) {
            char name[8];
            std::snprintf(name, sizeof name, "<0x%02X>", b);
            auto it = vocab_.find(name);
            byte_ids_[b] = it == vocab_.end() ? -1 : it->second;
        }
        for (size_t i = 0; i < tokens_.size(); ++i) {
            const std::string& t = tokens_[i];
            const bool marked = t.size() >= 2 && t.compare(0, 2, "<|") == 0 && t.compare(t.size() - 2, 2, "|>") == 0;
            if (!t.empty() && (types_[i] == 3 || types_[i] == 4 || marked)) specials_.push_back(t);
        }
        std::stable_sort(specials_.begin(), specials_.end(), [](const std::string& a, const std::string& b) { return a.size() > b.size(); });
        build_byte_maps();
    }
    static GGUFTokenizer from_reader(const gguf::GGUFReader& r) {
        if (!r.has("tokenizer.ggml.tokens")) throw std::runtime_error("GGUF file carries no tokenizer");
        std::vector<std::string> tokens, merges;
        std::vector<float> scores;
        std::vector<int> types;
        for (const auto& v : r.get("tokenizer.ggml.tokens").arr) tokens.push_back(v.s);
        if (r.has("tokenizer.ggml.scores"))
            for (const auto& v : r.get("tokenizer.ggml.scores").arr) scores.push_back((float)v.as_float());
        if (r.has("tokenizer.ggml.merges"))
            for (const auto& v : r.get("tokenizer.ggml.merges").arr) merges.push_back(v.s);
        if (r.has("tokenizer.ggml.token_type"))
            for (const auto& v : r.get("tokenizer.ggml.token_type").arr) types.push_back((int)v.as_int());
        auto geti = [&](const char* k) { return r.has(k) ? (int)r.get(k).as_int() : -1; };
        const bool add_bos = r.has("tokenizer.ggml.add_bos_token") && r.get("tokenizer.ggml.add_bos_token").b;
        return GGUFTokenizer(std::move(tokens), r.has("tokenizer.ggml.model") ? r.get("tokenizer.ggml.model").s : "llama", std::move(scores), merges,
                             std::move(types), geti("tokenizer.ggml.bos_token_id"), geti("tokenizer.ggml.eos_token_id"), add_bos,
                             r.has("tokenizer.ggml.pre") ? r.get("tokenizer.ggml.pre").s : "");
    }

    int vocab_size() const { return (int)tokens_.size(); }
    int bos_id() const { return bos_id_; }
    int eos_id() const { return eos_id_; }
    const std::string& model() const { return model_; }
    // -1 when the text is not a vocabulary entry.
    int token_id(const std::string& text) const { auto it = vocab_.find(text); return it == vocab_.end() ? -1 : it->second; }
    const std::string& token_text(int id) const { return tokens_.at((size_t)id); }

    // add_bos: -1 = as the file says, 0 / 1 = forced.
    std::vector<int> encode(const std::string& text, int add_bos = -1, bool parse_special = true) const {
        std::vector<int> ids;
        if ((add_bos < 0 ? add_bos_ : add_bos != 0) && bos_id_ >= 0) ids.push_back(bos_id_);
        bool first = true;
        auto plain = [&](const std::string& part) {
            if (part.empty()) return;
            if (model_ == "gpt2") encode_gpt2(part, ids);
            else encode_spm(part, first, ids);
            first = false;
        };
        if (!parse_special || specials_.empty()) { plain(text); return ids; }
        size_t start = 0, i = 0;
        while (i < text.size()) {
            const std::string* hit = nullptr;
            for (const auto& s : specials_)                                  // longest first
                if (text.compare(i, s.size(), s) == 0) { hit = &s; break; }
            if (!hit) { ++i; continue; }
            plain(text.substr(start, i - start));
            ids.push_back(vocab_.at(*hit));
            first = false;
            i += hit->size();
            start = i;
        }
        plain(text.substr(start));
        return ids;
    }

    std::string decode_token(int id) const { return decode({id}, true, false); }
    std::string decode(const std::vector<int>& ids, bool skip_special = true, bool strip_leading_space = true) const {
        std::string buf;
        for (int id : ids) {
            if (id < 0 || id >= (int)tokens_.size()) continue;
            if (skip_special && (types_[(size_t)id] == 3 || id == bos_id_)) continue;
            const std::string& t = tokens_[(size_t)id];
            if (model_ == "gpt2") {
                for (size_t i = 0; i < t.size();) {
                    int len;
                    const uint32_t cp = utf8::next(t, i, len);
                    auto it = unicode_to_byte_.find(cp);
                    buf.push_back(it != unicode_to_byte_.end() ? (char)it->second : (cp > 255 ? '?' : (char)cp));
                    i += (size_t)len;
                }
            } else if (t.size() == 6 && t.compare(0, 3, "<0x") == 0 && t[5] == '>') {
                buf.push_back((char)std::stoi(t.substr(3, 2), nullptr, 16));
            } else {
                for (size_t i = 0; i < t.size();) {
                    if (t.compare(i, 3, "\xE2\x96\x81") == 0) { buf.push_back(' '); i += 3; }
                    else buf.push_back(t[i++]);
                }
            }
        }
        std::string s = utf8::sanitize(buf);
        if (model_ != "gpt2" && strip_leading_space && !s.empty() && s[0] == ' ') s.erase(0, 1);
        return s;
    }

    // Class of a code point for the GPT-2 pattern (see the note at the top of the file).
    static CharClass classify(uint32_t c) {
        if (c < 0x80) {
            if (c == ' ' || (c >= 9 && c <= 13) || (c >= 0x1C && c <= 0x1F)) return Space;
            if ((c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z')) return Letter;
            if (c >= '0' && c <= '9') return Number;
            return Other;
        }
        if (c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) || c == 0x2028 || c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000)
            return Space;
        if (c == 0xB2 || c == 0xB3 || c == 0xB9 || (c >= 0xBC && c <= 0xBE)) return Number;
        static const uint32_t digits[][2] = {{0x0660, 0x0669}, {0x06F0, 0x06F9}, {0x07C0, 0x07C9}, {0x0966, 0x096F}, {0x09E6, 0x09EF}, {0x0A66, 0x0A6F},
                                             {0x0AE6, 0x0AEF}, {0x0B66, 0x0B6F}, {0x0BE6, 0x0BF2}, {0x0C66, 0x0C6F}, {0x0CE6, 0x0CEF}, {0x0D66, 0x0D6F},
                                             {0x0E50, 0x0E59}, {0x0ED0, 0x0ED9}, {0x0F20, 0x0F33}, {0x1040, 0x1049}, {0x17E0, 0x17E9}, {0x2070, 0x2070},
                                             {0x2074, 0x2079}, {0x2080, 0x2089}, {0x2150, 0x2189}, {0x2460, 0x249B}, {0x24EA, 0x24FF}, {0x2776, 0x2793},
                                             {0x3007, 0x3007}, {0x3021, 0x3029}, {0x3038, 0x303A}, {0x3192, 0x3195}, {0x3220, 0x3229}, {0x3248, 0x324F},
                                             {0x3251, 0x325F}, {0x3280, 0x3289}, {0x32B1, 0x32BF}, {0xFF10, 0xFF19}, {0x1D7CE, 0x1D7FF}};
        for (const auto& r : digits)
            if (c >= r[0] && c <= r[1]) return Number;
        if (c <= 0xBF) return (c == 0xAA || c == 0xB5 || c == 0xBA) ? Letter : Other;
        if (c == 0xD7 || c == 0xF7) return Other;
        static const uint32_t other[][2] = {
            {0x02C2, 0x02C5}, {0x02D2, 0x02DF}, {0x02E5, 0x02EB}, {0x02ED, 0x02ED}, {0x02EF, 0x036F},       // modifier symbols, combining marks
            {0x0375, 0x0375}, {0x037E, 0x037E}, {0x0384, 0x0385}, {0x0387, 0x0387}, {0x03F6, 0x03F6},
            {0x0482, 0x0489}, {0x055A, 0x055F}, {0x0589, 0x058F}, {0x0591, 0x05CF}, {0x05F3, 0x05F4},
            {0x0600, 0x061F}, {0x064B, 0x065F}, {0x066A, 0x066D}, {0x0670, 0x0670}, {0x06D4, 0x06D4}, {0x06D6, 0x06E4}, {0x06E7, 0x06ED},
            {0x0900, 0x0903}, {0x093A, 0x093C}, {0x093E, 0x094F}, {0x0951, 0x0957}, {0x0962, 0x0965}, {0x0970, 0x0970},
            {0x0E31, 0x0E31}, {0x0E34, 0x0E3F}, {0x0E47, 0x0E4F}, {0x0E5A, 0x0E5B},
            {0x1AB0, 0x1AFF}, {0x1DC0, 0x1DFF},
            {0x200B, 0x2027}, {0x202A, 0x202E}, {0x2030, 0x205E}, {0x2060, 0x206F}, {0x207A, 0x207E}, {0x208A, 0x208E}, {0x20A0, 0x20FF},
            {0x2100, 0x2101}, {0x2103, 0x2106}, {0x2108, 0x2109}, {0x2114, 0x2114}, {0x2116, 0x2118}, {0x211E, 0x2123}, {0x2125, 0x2125},
            {0x2127, 0x2127}, {0x2129, 0x2129}, {0x212E, 0x212E}, {0x213A, 0x213B}, {0x2140, 0x2144}, {0x214A, 0x214D}, {0x214F, 0x214F},
            {0x2190, 0x245F}, {0x249C, 0x24E9}, {0x2500, 0x2775}, {0x2794, 0x2BFF}, {0x2CE5, 0x2CEA}, {0x2CEF, 0x2CF1}, {0x2CF9, 0x2CFF},
            {0x2E00, 0x2E2E}, {0x2E30, 0x2FFF}, {0x3001, 0x3004}, {0x3008, 0x3020}, {0x302A, 0x3030}, {0x3036, 0x3037}, {0x303D, 0x303F},
            {0x3099, 0x309C}, {0x30A0, 0x30A0}, {0x30FB, 0x30FB}, {0x3190, 0x3191}, {0x3196, 0x319F}, {0x31C0, 0x31EF}, {0x3200, 0x321F},
            {0x322A, 0x3247}, {0x3250, 0x3250}, {0x3260, 0x327F}, {0x328A, 0x32B0}, {0x32C0, 0x33FF}, {0x4DC0, 0x4DFF},
            {0xA490, 0xA4CF}, {0xA700, 0xA716}, {0xA720, 0xA721}, {0xA789, 0xA78A}, {0xD800, 0xF8FF},
            {0xFB29, 0xFB29}, {0xFD3E, 0xFD3F}, {0xFDFC, 0xFDFF}, {0xFE00, 0xFE6F}, {0xFEFF, 0xFEFF}, {0xFF01, 0xFF0F}, {0xFF1A, 0xFF20},
            {0xFF3B, 0xFF40}, {0xFF5B, 0xFF65}, {0xFFE0, 0xFFFF}, {0x1D000, 0x1D3FF}, {0x1F000, 0x1FAFF}, {0xE0000, 0x10FFFF}};
        for (const auto& r : other)
            if (c >= r[0] && c <= r[1]) return Other;
        return Letter;
    }

    // The pieces of the newer patterns (qwen2, llama-3):
    //   contraction (either case) | one optional char that is no CR / LF / letter / number, then letters+ | one number (qwen2) or
    //   up to three (llama-3) | optional space, others+, then CR / LF* | spaces* ending in CR / LF+ | spaces+(?!non-space) | spaces+
    static std::vector<std::string> pieces(const std::string& text, PreStyle style) {
        if (style == GPT2) return gpt2_pieces(text);
        struct Cp { size_t at; uint32_t c; CharClass k; };
        std::vector<Cp> cps;
        for (size_t i = 0; i < text.size();) {
            int len;
            const uint32_t c = utf8::next(text, i, len);
            cps.push_back({i, c, classify(c)});
            i += (size_t)len;
        }
        const size_t n = cps.size();
        std::vector<std::string> out;
        auto cut = [&](size_t a, size_t b) { out.push_back(text.substr(cps[a].at, (b < n ? cps[b].at : text.size()) - cps[a].at)); };
        auto lower = [](uint32_t c) { return c >= 'A' && c <= 'Z' ? c + 32 : c; };
        auto newline = [&](size_t i) { return cps[i].c == '\r' || cps[i].c == '\n'; };
        size_t i = 0;
        while (i < n) {
            if (cps[i].c == '\'' && i + 1 < n) {                           // contractions, either case
                const uint32_t a = lower(cps[i + 1].c), b = i + 2 < n ? lower(cps[i + 2].c) : 0;
                size_t take = 0;
                if (a == 's' || a == 't' || a == 'm' || a == 'd') take = 2;
                if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) take = 3;
                if (take) { cut(i, i + take); i += take; continue; }
            }
            {                                                              // one optional leading symbol or blank, then letters
                size_t j = i;
                if (cps[i].k != Letter && cps[i].k != Number && !newline(i) && i + 1 < n && cps[i + 1].k == Letter) j = i + 1;
                if (cps[j].k == Letter) {
                    size_t e = j;
                    while (e < n && cps[e].k == Letter) ++e;
                    cut(i, e);
                    i = e;
                    continue;
                }
            }
            if (cps[i].k == Number) {
                size_t e = i + 1;
                if (style == Llama3)
                    while (e < n && e < i + 3 && cps[e].k == Number) ++e;
                cut(i, e);
                i = e;
                continue;
            }
            {                                                              // optional space, symbols, then the newlines that follow
                size_t j = i;
                if (cps[i].c == ' ' && i + 1 < n && cps[i + 1].k == Other) j = i + 1;
                if (cps[j].k == Other) {
                    size_t e = j;
                    while (e < n && cps[e].k == Other) ++e;
                    while (e < n && newline(e)) ++e;
                    cut(i, e);
                    i = e;
                    continue;
                }
            }
            size_t e = i;                                                  // a run of white space
            while (e < n && cps[e].k == Space) ++e;
            size_t last_nl = n;
            for (size_t k = i; k < e; ++k)
                if (newline(k)) last_nl = k;
            if (last_nl != n) e = last_nl + 1;                             // up to the last newline of the run
            else if (e < n && e - i > 1) --e;                              // leave the last blank for the piece that follows
            cut(i, e);
            i = e;
        }
        return out;
    }

    // The pieces the GPT-2 pattern cuts `text` into:
    //   's|'t|'re|'ve|'m|'ll|'d| ?letters+| ?numbers+| ?others+|spaces+(?!non-space)|spaces+
    static std::vector<std::string> gpt2_pieces(const std::string& text) {
        struct Cp { size_t at; uint32_t c; CharClass k; };
        std::vector<Cp> cps;
        for (size_t i = 0; i < text.size();) {
            int len;
            const uint32_t c = utf8::next(text, i, len);
            cps.push_back({i, c, classify(c)});
            i += (size_t)len;
        }
        const size_t n = cps.size();
        std::vector<std::string> out;
        auto cut = [&](size_t a, size_t b) { out.push_back(text.substr(cps[a].at, (b < n ? cps[b].at : text.size()) - cps[a].at)); };
        size_t i = 0;
        while (i < n) {
            if (cps[i].c == '\'' && i + 1 < n) {
                const uint32_t a = cps[i + 1].c, b = i + 2 < n ? cps[i + 2].c : 0;
                size_t take = 0;
                if (a == 's' || a == 't' || a == 'm' || a == 'd') take = 2;
                if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) take = 3;
                if (take) { cut(i, i + take); i += take; continue; }
            }
            size_t j = i;
            if (cps[i].c == ' ' && i + 1 < n && cps[i + 1].k != Space) j = i + 1;         // the optional leading space
            if (cps[j].k != Space) {
                const CharClass k = cps[j].k;
                size_t e = j;
                while (e < n && cps[e].k == k) ++e;
                cut(i, e);
                i = e;
                continue;
            }
            size_t e = i;
            while (e < n && cps[e].k == Space) ++e;
            if (e < n && e - i > 1) --e;             // leave the last one for the piece that follows
            cut(i, e);
            i = e;
        }
        return out;
    }

 private:
    void build_byte_maps() {
        std::vector<int> bs;
        for (int b = '!'; b <= '~'; ++b) bs.push_back(b);
        for (int b = 0xA1; b <= 0xAC; ++b) bs.push_back(b);
        for (int b = 0xAE; b <= 0xFF; ++b) bs.push_back(b);
        std::vector<bool> direct(256, false);
        for (int b : bs) direct[(size_t)b] = true;
        int extra = 0;
        for (int b = 0; b < 256; ++b) {
            const uint32_t cp = direct[(size_t)b] ? (uint32_t)b : (uint32_t)(256 + extra++);
            std::string u;
            utf8::append(cp, u);
            byte_to_unicode_[b] = u;
            unicode_to_byte_[cp] = (unsigned char)b;
        }
    }
    int score_of_pair(const std::string& a, const std::string& b, float& score) const {
        auto it = vocab_.find(a + b);
        if (it == vocab_.end()) return -1;
        score = scores_[(size_t)it->second];
        return it->second;
    }
    void encode_spm(const std::string& part, bool prefix_space, std::vector<int>& out) const {
        static const std::string bar = "\xE2\x96\x81";
        std::string text;
        for (char c : part) {
            if (c == ' ') text += bar;
            else text.push_back(c);
        }
        if (prefix_space && text.compare(0, 3, bar) != 0) text = bar + text;
        if (text.empty()) return;
        if (text.compare(0, 3, bar) == 0) {            // every word is a vocabulary entry of its own: no merging needed
            std::vector<int> ids;
            bool all = true;
            size_t p = 3;
            while (all) {
                const size_t q = text.find(bar, p);
                auto it = vocab_.find(bar + text.substr(p, q == std::string::npos ? std::string::npos : q - p));
                if (it == vocab_.end()) all = false;
                else ids.push_back(it->second);
                if (q == std::string::npos) break;
                p = q + 3;
            }
            if (all) { out.insert(out.end(), ids.begin(), ids.end()); return; }
        }
        std::vector<std::string> syms;
        for (size_t i = 0; i < text.size();) {
            int len;
            utf8::next(text, i, len);
            syms.push_back(text.substr(i, (size_t)len));
            i += (size_t)len;
        }
        const int n = (int)syms.size();
        std::vector<int> prev((size_t)n), nxt((size_t)n);
        std::vector<bool> alive((size_t)n, true);
        for (int i = 0; i < n; ++i) { prev[(size_t)i] = i - 1; nxt[(size_t)i] = i + 1; }
        struct Cand { float score; int i; std::string a, b; };
        auto worse = [](const Cand& x, const Cand& y) {                      // best = highest score, then leftmost, then smallest text
            if (x.score != y.score) return x.score < y.score;
            if (x.i != y.i) return x.i > y.i;
            if (x.a != y.a) return x.a > y.a;
            return x.b > y.b;
        };
        std::priority_queue<Cand, std::vector<Cand>, decltype(worse)> heap(worse);
        auto push = [&](int i) {
            const int j = nxt[(size_t)i];
            if (j >= n) return;
            float sc;
            if (score_of_pair(syms[(size_t)i], syms[(size_t)j], sc) >= 0) heap.push({sc, i, syms[(size_t)i], syms[(size_t)j]});
        };
        for (int i = 0; i + 1 < n; ++i) push(i);
        while (!heap.empty()) {
            Cand c = heap.top();
            heap.pop();
            const int i = c.i, j = nxt[(size_t)i];
            if (!alive[(size_t)i] || j >= n || !alive[(size_t)j] || syms[(size_t)i] != c.a || syms[(size_t)j] != c.b) continue;
            syms[(size_t)i] = c.a + c.b;
            alive[(size_t)j] = false;
            nxt[(size_t)i] = nxt[(size_t)j];
            if (nxt[(size_t)j] < n) prev[(size_t)nxt[(size_t)j]] = i;
            if (prev[(size_t)i] >= 0) push(prev[(size_t)i]);
            push(i);
        }
        for (int i = 0; i < n;) {
            if (alive[(size_t)i]) {
                auto it = vocab_.find(syms[(size_t)i]);
                if (it != vocab_.end()) out.push_back(it->second);
                else
                    for (unsigned char b : syms[(size_t)i]) out.push_back(byte_ids_[b] >= 0 ? byte_ids_[b] : 0);
                i = nxt[(size_t)i];
            } else {
                ++i;
            }
        }
    }
    void encode_gpt2(const std::string& part, std::vector<int>& out) const {
        for (const std::string& piece : pieces(part, style_)) {
            std::vector<std::string> word;
            for (unsigned char b : piece) word.push_back(byte_to_unicode_[b]);
            while (word.size() > 1) {
                int best = -1;
                size_t at = 0;
                for (size_t i = 0; i + 1 < word.size(); ++i) {
                    auto it = ranks_.find(word[i] + '\x01' + word[i + 1]);
                    if (it != ranks_.end() && (best < 0 || it->second < best)) { best = it->second; at = i; }
                }
                if (best < 0) break;
                word[at] += word[at + 1];
                word.erase(word.begin() + (long)at + 1);
            }
            for (const std::string& tok : word) {
                auto it = vocab_.find(tok);
                if (it != vocab_.end()) { out.push_back(it->second); continue; }
                for (size_t i = 0; i < tok.size();) {                        // unknown merge result: its characters one by one
                    int len;
                    utf8::next(tok, i, len);
                    auto c = vocab_.find(tok.substr(i, (size_t)len));
                    out.push_back(c == vocab_.end() ? 0 : c->second);
                    i += (size_t)len;
                }
            }
        }
    }

    std::vector<std::string> tokens_;
    std::string model_ = "llama";
    std::vector<float> scores_;
    std::vector<int> types_;
    int bos_id_ = -1, eos_id_ = -1;
    bool add_bos_ = false;
    PreStyle style_ = GPT2;
    std::unordered_map<std::string, int> vocab_;
    std::unordered_map<std::string, int> ranks_;
    int byte_ids_[256];
    std::vector<std::string> specials_;
    std::string byte_to_unicode_[256];
    std::unordered_map<uint32_t, unsigned char> unicode_to_byte_;
};

// The byte-level BPE tokenizer of a Hugging Face checkpoint directory: vocab.json + merges.txt, or the "model" section of
// tokenizer.json (merges as "a b" strings or as pairs).  Returns false when the directory has neither (torch/serve/llm.h:94-297).
inline bool load_hf_tokenizer(const std::string& model_dir, GGUFTokenizer& out) {
    auto slurp = [](const std::string& p, std::string& text) {
        std::ifstream f(p, std::ios::binary);
        if (!f) return false;
        std::stringstream ss;
        ss << f.rdbuf();
        text = ss.str();
        return true;
    };
    std::string vj, mt, tj;
    json::Value vocab;
    std::vector<std::string> merges;
    if (slurp(model_dir + "/vocab.json", vj) && slurp(model_dir + "/merges.txt", mt)) {
        vocab = json::parse(vj);
        std::istringstream lines(mt);
        std::string ln;
        while (std::getline(lines, ln)) {
            if (!ln.empty() && ln.back() == '\r') ln.pop_back();
            const bool blank = ln.find_first_not_of(" \t") == std::string::npos;
            if (!blank && ln.compare(0, 8, "#version") != 0) merges.push_back(ln);
        }
    } else if (slurp(model_dir + "/tokenizer.json", tj)) {
        const json::Value doc = json::parse(tj);
        vocab = doc["model"]["vocab"];
        for (const auto& m : doc["model"]["merges"].items()) {
            if (m.is_string()) merges.push_back(m.as_string());
            else if (m.is_array() && m.size() == 2) merges.push_back(m.at(0).as_string() + " " + m.at(1).as_string());
        }
    }
    if (!vocab.is_object() || vocab.size() == 0) return false;
    long long top = -1;
    for (const auto& kv : vocab.members()) top = std::max(top, kv.second.as_int(-1));
    if (top < 0 || top > (1ll << 24)) return false;
    std::vector<std::string> tokens((size_t)top + 1);
    for (const auto& kv : vocab.members())
        if (kv.second.as_int(-1) >= 0) tokens[(size_t)kv.second.as_int()] = kv.first;
    out = GGUFTokenizer(std::move(tokens), "gpt2", {}, merges);
    return true;
}

}  // namespace io
}  // namespace promethorch
