// Tagged words: vectors handed from producers to consumers element by element, without a barrier or a flag.
//
// Every 64-bit word holds two halves (32 bits of data) and the tag of the step that wrote it, stored with ONE 8-byte
// store, which arrives whole; a reader that sees the tag it expects has the data.  Used between the blocks of the
// persistent decode kernel (barrier-free form) and between GPUs (a producing kernel's epilogue stores the words
// straight into every peer's staging area over NVLink; the consuming kernel polls its local copy).  Every poll is
// bounded; tags only grow, so a slot's previous contents never look current.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace spb {

__device__ __forceinline__ uint32_t ll_read1(const uint2* p, unsigned tag, long long limit, int* fail) {
    uint32_t d, t;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(d), "=r"(t) : "l"(p));
    if (t == tag) return d;
    const long long t0 = clock64();
    for (;;) {
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(d), "=r"(t) : "l"(p));
        if (t == tag) return d;
        if (clock64() - t0 > limit) *fail = 1;
        if (*reinterpret_cast<volatile int*>(fail)) return d;  // this wait or another one of the block ran out
    }
}
// four consecutive words = eight halves
__device__ __forceinline__ uint4 ll_read4(const uint2* p, unsigned tag, long long limit, int* fail) {
    uint32_t d[4], t[4];
    long long t0 = 0;
    for (int spin = 0;; ++spin) {
#pragma unroll
        for (int i = 0; i < 4; ++i) asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(d[i]), "=r"(t[i]) : "l"(p + i));
        if (t[0] == tag && t[1] == tag && t[2] == tag && t[3] == tag) break;
        if (spin == 0) t0 = clock64();
        else if (clock64() - t0 > limit) *fail = 1;
        if (*reinterpret_cast<volatile int*>(fail)) break;  // this wait or another one of the block ran out
    }
    return make_uint4(d[0], d[1], d[2], d[3]);
}
__device__ __forceinline__ void ll_write(uint2* p, uint32_t data, unsigned tag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(tag) : "memory");
}

// Where a producer's output vector goes as tagged words: the same word index in every destination (the staging
// areas of this rank in every GPU's exchange buffer, or one buffer for the blocks of one kernel).
constexpr int kLlMaxDest = 8;
struct LlFan {
    uint2* dst[kLlMaxDest];
    int ndst;             // 0: no fan-out
    const unsigned* seq;  // device word: the words carry *seq + 1 (read by the producer after its dependency wait)
};
__device__ __forceinline__ void ll_fan_write(const LlFan& f, size_t word, uint32_t data, unsigned tag) {
#pragma unroll
    for (int i = 0; i < kLlMaxDest; ++i)
        if (i < f.ndst) ll_write(f.dst[i] + word, data, tag);
}

}  // namespace spb
