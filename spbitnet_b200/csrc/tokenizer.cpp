// Byte-level BPE tokenizer for HuggingFace tokenizer.json files (Llama 3 / GPT-4 style), host only.
//
// Behaviour follows spbitnet::Tokenizer of the reference (include/spbitnet/tokenizer.h, src/tokenizer.cpp):
//   * pre-tokeniser: the GPT-4 split pattern approximated for ASCII -- letters are [A-Za-z], digits [0-9],
//     white space the six C-locale space characters, every other byte (all of UTF-8 beyond ASCII included)
//     counts as punctuation; alternatives tried in the pattern's order (src/tokenizer.cpp:107-233);
//   * BPE: repeatedly merge every occurrence of the adjacent pair with the lowest merge rank (:239-281);
//   * encode adds no BOS / EOS and drops pieces that are not in the vocabulary (:341-357);
//   * decode skips special tokens and ids outside the vocabulary (:359-374).
// The reference keeps tokens in GPT-2's printable stand-in alphabet (one code point per byte) and maps text into
// it; here the vocabulary and the merge table are mapped back to raw bytes once, at load, so the merge loop works
// on the text's own bytes.  The two are the same computation because the byte <-> code point table is a bijection;
// a vocabulary entry that uses a code point outside that table can never match an encoded text in the reference
// either, and keeps its raw JSON string here (special tokens such as "<|begin_of_text|>" are plain ASCII).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/spbitnet_b200.h"
#include "json_min.h"

namespace spb {
int fail(int code, const char* fmt, ...);
}

struct spb_tokenizer {
    std::unordered_map<std::string, int> id_of;          // raw-byte token -> id
    std::vector<std::string> token_of;                   // id -> the bytes the token decodes to ("" for unused ids)
    std::unordered_set<int> special;
    std::unordered_map<std::string, int> merge_rank;     // left + '\0' + right (raw bytes) -> rank
};

namespace {

// GPT-2's bytes_to_unicode: printable bytes stand for themselves, the other 68 are numbered from U+0100 on.
struct ByteAlphabet {
    uint32_t cp_of_byte[256];
    std::unordered_map<uint32_t, uint8_t> byte_of_cp;
    ByteAlphabet() {
        bool printable[256] = {};
        for (int b = '!'; b <= '~'; ++b) printable[b] = true;
        for (int b = 0xA1; b <= 0xAC; ++b) printable[b] = true;
        for (int b = 0xAE; b <= 0xFF; ++b) printable[b] = true;
        uint32_t next = 256;
        for (int b = 0; b < 256; ++b) {
            cp_of_byte[b] = printable[b] ? static_cast<uint32_t>(b) : next++;
            byte_of_cp[cp_of_byte[b]] = static_cast<uint8_t>(b);
        }
    }
};
const ByteAlphabet& alphabet() {
    static const ByteAlphabet a;
    return a;
}

// UTF-8 string in the stand-in alphabet -> raw bytes.  Code points without a byte are dropped (what the
// reference's decode does with them, src/tokenizer.cpp:93-104); the return value tells whether there were none.
bool to_raw_bytes(const std::string& s, std::string* out) {
    bool complete = true;
    out->clear();
    const auto& tab = alphabet().byte_of_cp;
    size_t i = 0;
    while (i < s.size()) {
        const unsigned char c = static_cast<unsigned char>(s[i]);
        uint32_t cp;
        int len;
        if (c < 0x80) { cp = c; len = 1; }
        else if (c < 0xE0) { cp = c & 0x1Fu; len = 2; }
        else if (c < 0xF0) { cp = c & 0x0Fu; len = 3; }
        else { cp = c & 0x07u; len = 4; }
        for (int j = 1; j < len && i + j < s.size(); ++j) cp = (cp << 6) | (static_cast<unsigned char>(s[i + j]) & 0x3Fu);
        i += static_cast<size_t>(len);
        const auto it = tab.find(cp);
        if (it == tab.end()) complete = false;
        else *out += static_cast<char>(it->second);
    }
    return complete;
}

inline bool is_letter(unsigned char c) { return (c >= 'A' && c <= 'Z') || (c >= 'a' && c <= 'z'); }
inline bool is_digit(unsigned char c) { return c >= '0' && c <= '9'; }
inline bool is_space(unsigned char c) { return c == ' ' || (c >= '\t' && c <= '\r'); }
inline bool is_newline(unsigned char c) { return c == '\r' || c == '\n'; }
inline unsigned char lower(unsigned char c) { return (c >= 'A' && c <= 'Z') ? static_cast<unsigned char>(c + 32) : c; }

// Length of the piece that starts at p (always >= 1 for p < n).
size_t next_piece(const unsigned char* t, size_t p, size_t n) {
    // 's 't 'm 'd 're 've 'll, any case
    if (t[p] == '\'' && p + 1 < n) {
        const unsigned char a = lower(t[p + 1]);
        if (p + 2 < n) {
            const unsigned char b = lower(t[p + 2]);
            if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) return 3;
        }
        if (a == 's' || a == 't' || a == 'm' || a == 'd') return 2;
    }
    // an optional single byte that is neither letter, digit, CR nor LF, then letters
    {
        size_t i = p;
        if (!is_letter(t[i]) && !is_digit(t[i]) && !is_newline(t[i])) ++i;
        const size_t first = i;
        while (i < n && is_letter(t[i])) ++i;
        if (i > first) return i - p;
    }
    // one to three digits
    {
        size_t i = p;
        while (i < n && i - p < 3 && is_digit(t[i])) ++i;
        if (i > p) return i - p;
    }
    // an optional blank, then bytes that are neither space, letter nor digit, then any CR / LF
    {
        size_t i = p;
        if (t[i] == ' ') ++i;
        const size_t first = i;
        while (i < n && !is_space(t[i]) && !is_letter(t[i]) && !is_digit(t[i])) ++i;
        if (i > first) {
            while (i < n && is_newline(t[i])) ++i;
            return i - p;
        }
    }
    // white space other than CR / LF, then at least one CR / LF
    {
        size_t i = p;
        while (i < n && is_space(t[i]) && !is_newline(t[i])) ++i;
        const size_t first = i;
        while (i < n && is_newline(t[i])) ++i;
        if (i > first) return i - p;
    }
    // a run of white space: taken whole when the text ends behind it, and also when it does not (the pattern's
    // last two alternatives, the second without the look-ahead, cover both)
    {
        size_t i = p;
        while (i < n && is_space(t[i])) ++i;
        if (i > p) return i - p;
    }
    return 1;
}

// BPE over the raw bytes of one piece; appends the ids of the resulting symbols that are in the vocabulary.
void bpe_piece(const spb_tokenizer& tk, const std::string& piece, std::vector<int>* ids) {
    std::vector<std::string> sym;
    sym.reserve(piece.size());
    for (char c : piece) sym.emplace_back(1, c);
    std::string key;
    while (sym.size() >= 2) {
        int best = -1, best_rank = 0x7FFFFFFF;
        for (size_t i = 0; i + 1 < sym.size(); ++i) {
            key.assign(sym[i]);
            key += '\0';
            key += sym[i + 1];
            const auto it = tk.merge_rank.find(key);
            if (it != tk.merge_rank.end() && it->second < best_rank) {
                best_rank = it->second;
                best = static_cast<int>(i);
            }
        }
        if (best < 0) break;
        const std::string left = sym[static_cast<size_t>(best)], right = sym[static_cast<size_t>(best) + 1];
        std::vector<std::string> merged;
        merged.reserve(sym.size());
        for (size_t i = 0; i < sym.size();) {
            if (i + 1 < sym.size() && sym[i] == left && sym[i + 1] == right) {
                merged.push_back(left + right);
                i += 2;
            } else {
                merged.push_back(std::move(sym[i]));
                ++i;
            }
        }
        sym.swap(merged);
    }
    for (const std::string& s : sym) {
        const auto it = tk.id_of.find(s);
        if (it != tk.id_of.end()) ids->push_back(it->second);
    }
}

}  // namespace

extern "C" spb_tokenizer* spb_tokenizer_load(const char* tokenizer_json_path) {
    if (!tokenizer_json_path) {
        spb::fail(SPB_E_INVALID, "spb_tokenizer_load: null path");
        return nullptr;
    }
    std::ifstream f(tokenizer_json_path, std::ios::binary);
    if (!f) {
        spb::fail(SPB_E_INVALID, "spb_tokenizer_load: cannot open %s", tokenizer_json_path);
        return nullptr;
    }
    std::stringstream buf;
    buf << f.rdbuf();
    const std::string text = buf.str();
    spb::json::Value root;
    try {
        root = spb::json::parse(text);
    } catch (const std::exception& e) {
        spb::fail(SPB_E_FORMAT, "spb_tokenizer_load: %s", e.what());
        return nullptr;
    }
    auto* tk = new spb_tokenizer();
    int max_id = -1;
    std::string raw;
    std::vector<std::pair<int, std::string>> decoded;
    auto add = [&](const std::string& token, int id) {
        if (id < 0) return;
        // a token spelled with a code point outside the alphabet can never equal a piece of encoded text; it keeps
        // its spelling as the key (unreachable) and decodes to its mappable part
        const bool mapped = to_raw_bytes(token, &raw);
        tk->id_of[mapped ? raw : token] = id;
        decoded.emplace_back(id, raw);
        if (id > max_id) max_id = id;
    };
    const spb::json::Value* model = root.find("model");
    if (model) {
        if (const spb::json::Value* vocab = model->find("vocab"))
            for (const auto& m : vocab->members) add(m.first, static_cast<int>(m.second.as_int(-1)));
    }
    if (const spb::json::Value* added = root.find("added_tokens")) {
        for (const spb::json::Value& at : added->items) {
            const spb::json::Value* id = at.find("id");
            const spb::json::Value* content = at.find("content");
            if (!id || !content || !content->is(spb::json::Value::String)) continue;
            const int i = static_cast<int>(id->as_int(-1));
            const spb::json::Value* sp = at.find("special");
            const bool special = sp && sp->as_bool();
            add(content->str, i);  // overrides a vocabulary entry of the same spelling
            if (special && i >= 0) tk->special.insert(i);
        }
    }
    tk->token_of.assign(static_cast<size_t>(max_id + 1), std::string());
    for (auto& d : decoded) tk->token_of[static_cast<size_t>(d.first)] = std::move(d.second);
    if (model) {
        if (const spb::json::Value* merges = model->find("merges")) {
            int rank = 0;
            std::string l, r, lraw, rraw;
            for (const spb::json::Value& m : merges->items) {
                // "left right" (one blank), or ["left", "right"] in newer files
                if (m.is(spb::json::Value::String)) {
                    const size_t sp = m.str.find(' ');
                    if (sp == std::string::npos) { ++rank; continue; }
                    l = m.str.substr(0, sp);
                    r = m.str.substr(sp + 1);
                } else if (m.is(spb::json::Value::Array) && m.items.size() == 2) {
                    l = m.items[0].str;
                    r = m.items[1].str;
                } else {
                    ++rank;
                    continue;
                }
                const bool lok = to_raw_bytes(l, &lraw), rok = to_raw_bytes(r, &rraw);
                if (lok && rok) {
                    std::string key = lraw;
                    key += '\0';
                    key += rraw;
                    tk->merge_rank.emplace(std::move(key), rank);  // the first (highest-priority) rank of a pair stays
                }
                ++rank;
            }
        }
    }
    return tk;
}

extern "C" void spb_tokenizer_destroy(spb_tokenizer* t) { delete t; }

extern "C" int spb_tokenizer_vocab_size(const spb_tokenizer* t) { return t ? static_cast<int>(t->token_of.size()) : 0; }

extern "C" int spb_tokenizer_encode(const spb_tokenizer* t, const char* text, size_t text_bytes, int* ids, int capacity) {
    if (!t || (!text && text_bytes) || capacity < 0 || (capacity > 0 && !ids))
        return spb::fail(SPB_E_INVALID, "spb_tokenizer_encode: bad arguments");
    std::vector<int> out;
    const unsigned char* p = reinterpret_cast<const unsigned char*>(text);
    for (size_t pos = 0; pos < text_bytes;) {
        const size_t len = next_piece(p, pos, text_bytes);
        bpe_piece(*t, std::string(text + pos, len), &out);
        pos += len;
    }
    const int n = static_cast<int>(out.size());
    for (int i = 0; i < n && i < capacity; ++i) ids[i] = out[static_cast<size_t>(i)];
    return n;
}

extern "C" int spb_tokenizer_decode(const spb_tokenizer* t, const int* ids, int n, char* out, size_t capacity) {
    if (!t || (n > 0 && !ids) || n < 0 || (capacity > 0 && !out)) return spb::fail(SPB_E_INVALID, "spb_tokenizer_decode: bad arguments");
    std::string s;
    for (int i = 0; i < n; ++i) {
        const int id = ids[i];
        if (id < 0 || id >= static_cast<int>(t->token_of.size()) || t->special.count(id)) continue;
        s += t->token_of[static_cast<size_t>(id)];
    }
    if (capacity > 0) {
        const size_t k = s.size() < capacity - 1 ? s.size() : capacity - 1;
        std::memcpy(out, s.data(), k);
        out[k] = '\0';
    }
    return static_cast<int>(s.size());
}
