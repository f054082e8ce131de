// promethorch C++ API: chat prompt templates per architecture.
//
// ChatML (qwen2 / qwen3, with the /no_think option), phi-3, gemma, llama-3 and mistral [INST]: the formats of
// torch/io/gguf_model.h:4178-4239 of the reference.  The default system prompt and the PT_SYSTEM_PROMPT / PT_NO_THINK
// switches are kept (PROMETHORCH_* spellings too).  Same output as the Python module of this package for the same input.
#pragma once
#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <string>
#include <vector>

namespace promethorch {
namespace io {
namespace chat {

inline const char* default_system() { return "You are a helpful assistant."; }

struct Message {
    std::string role, content;
};

namespace detail {
inline const char* env(const std::string& name) {
    if (const char* v = std::getenv(("PROMETHORCH_" + name).c_str())) return v;
    return std::getenv(("PT_" + name).c_str());
}
inline bool any_of(const std::string& a, std::initializer_list<const char*> names) {
    for (const char* n : names)
        if (a == n) return true;
    return false;
}
}  // namespace detail

// `system`: nullptr = the environment's or the default system prompt; "" = none.  no_think: -1 = from the environment.
inline std::string apply_chat_template(const std::string& prompt, const std::string& architecture, const std::string& model_name = "",
                                       const std::string* system = nullptr, int no_think = -1) {
    std::string sys = system ? *system : (detail::env("SYSTEM_PROMPT") ? detail::env("SYSTEM_PROMPT") : default_system());
    if (no_think < 0) {
        const char* v = detail::env("NO_THINK");
        no_think = v && v[0] == '1';
    }
    const std::string& a = architecture;
    if (detail::any_of(a, {"qwen3", "qwen2"})) {
        std::string sb;
        if (no_think && a == "qwen3") sb = "<|im_start|>system\n" + (sys.empty() ? std::string("/no_think") : sys + "\n/no_think") + "<|im_end|>\n";
        else if (!sys.empty()) sb = "<|im_start|>system\n" + sys + "<|im_end|>\n";
        return sb + "<|im_start|>user\n" + prompt + "<|im_end|>\n<|im_start|>assistant\n";
    }
    if (detail::any_of(a, {"phi3", "phi2"}))
        return (sys.empty() ? "" : "<|system|>\n" + sys + "<|end|>\n") + "<|user|>\n" + prompt + "<|end|>\n<|assistant|>\n";
    if (detail::any_of(a, {"gemma3", "gemma2", "gemma"}))
        return "<start_of_turn>user\n" + (sys.empty() ? prompt : sys + "\n\n" + prompt) + "<end_of_turn>\n<start_of_turn>model\n";
    if (a == "llama") {
        std::string lower = model_name;
        std::transform(lower.begin(), lower.end(), lower.begin(), [](unsigned char c) { return (char)std::tolower(c); });
        if (lower.find("mistral") != std::string::npos)
            return sys.empty() ? "<s>[INST] " + prompt + " [/INST]" : "<s>[INST] <<SYS>>\n" + sys + "\n<</SYS>>\n\n" + prompt + " [/INST]";
        const std::string sb = sys.empty() ? "" : "<|start_header_id|>system<|end_header_id|>\n\n" + sys + "<|eot_id|>";
        return "<|begin_of_text|>" + sb + "<|start_header_id|>user<|end_header_id|>\n\n" + prompt + "<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n";
    }
    return prompt;
}

// A list of {role, content} messages -> one prompt.  System messages become the system block; earlier turns are replayed
// in the architecture's format (ChatML) or folded into the last user prompt (the others); the result ends with the
// assistant header.
inline std::string render_messages(const std::vector<Message>& messages, const std::string& architecture, const std::string& model_name = "") {
    std::string system;
    bool has_system = false;
    std::vector<const Message*> turns;
    for (const auto& m : messages) {
        if (m.role == "system") {
            if (has_system) system += "\n";
            system += m.content;
            has_system = true;
        } else if (m.role == "user" || m.role == "assistant" || m.role == "tool") {
            turns.push_back(&m);
        }
    }
    if (system.empty()) has_system = false;            // an empty system message counts as none
    const std::string* sys = has_system ? &system : nullptr;
    if (turns.empty()) return apply_chat_template("", architecture, model_name, sys);
    if (architecture == "qwen3" || architecture == "qwen2") {
        const std::string s = has_system ? system : default_system();
        std::string out = s.empty() ? "" : "<|im_start|>system\n" + s + "<|im_end|>\n";
        for (const Message* m : turns) out += "<|im_start|>" + (m->role == "tool" ? std::string("user") : m->role) + "\n" + m->content + "<|im_end|>\n";
        return out + "<|im_start|>assistant\n";
    }
    std::string hist;
    for (size_t i = 0; i + 1 < turns.size(); ++i) hist += (i ? "\n" : "") + turns[i]->role + ": " + turns[i]->content;
    const std::string& last = turns.back()->content;
    return apply_chat_template(turns.size() > 1 ? hist + "\n" + last : last, architecture, model_name, sys);
}

// Removes <think>...</think> blocks and the white space that follows them.
inline std::string strip_think(const std::string& text) {
    std::string out;
    size_t p = 0;
    for (;;) {
        const size_t a = text.find("<think>", p);
        const size_t b = a == std::string::npos ? a : text.find("</think>", a);
        if (a == std::string::npos || b == std::string::npos) { out += text.substr(p); return out; }
        out += text.substr(p, a - p);
        p = b + 8;
        while (p < text.size() && std::isspace((unsigned char)text[p])) ++p;
    }
}

}  // namespace chat
}  // namespace io
}  // namespace promethorch
