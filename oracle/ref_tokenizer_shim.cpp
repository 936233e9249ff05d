// ref_tokenizer_shim.cpp -- extern "C" doorway onto the UNMODIFIED reference tokenizer (include/spbitnet/tokenizer.h,
// src/tokenizer.cpp, compiled where it lies).  TEST INFRASTRUCTURE ONLY: it pins spb_tokenizer_* against the
// reference's own encode / decode on the same tokenizer.json.
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include "spbitnet/tokenizer.h"

extern "C" {

void* reftok_load(const char* path) {
    try {
        return new spbitnet::Tokenizer(spbitnet::Tokenizer::load(path));
    } catch (const std::exception&) {
        return nullptr;
    }
}
void reftok_destroy(void* h) { delete static_cast<spbitnet::Tokenizer*>(h); }
int reftok_vocab_size(void* h) { return static_cast<spbitnet::Tokenizer*>(h)->vocab_size(); }
int reftok_encode(void* h, const char* text, size_t n, int* ids, int capacity) {
    const auto v = static_cast<spbitnet::Tokenizer*>(h)->encode(std::string(text, n));
    for (size_t i = 0; i < v.size() && static_cast<int>(i) < capacity; ++i) ids[i] = v[i];
    return static_cast<int>(v.size());
}
int reftok_decode(void* h, const int* ids, int n, char* out, size_t capacity) {
    const std::string s = static_cast<spbitnet::Tokenizer*>(h)->decode(std::vector<int>(ids, ids + n));
    if (capacity) {
        const size_t k = s.size() < capacity - 1 ? s.size() : capacity - 1;
        std::memcpy(out, s.data(), k);
        out[k] = 0;
    }
    return static_cast<int>(s.size());
}

}  // extern "C"
