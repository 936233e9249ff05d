// Split-KV decode attention for one new token (replaces attention_scores_gpu + softmax_gpu +
// attention_output_gpu of the reference, src/kernels/inference_kernels.cu:241-371, as one
// pass over the KV cache).
//
// The reference gives a head to one block and walks the positions serially; at a few
// hundred positions that is latency bound (a dependent global load per position).  Here the
// positions are cut into chunks of 16 or 32; block (kv head, chunk) serves every query head
// of the GQA group from one read of its K and V rows (all of them in flight at once, staged in
// shared memory) and writes an un-normalised partial result {max, sum, sum(e*V)} per (head, chunk)
// to a scratch buffer.  A second tiny kernel merges the chunks of a head with the usual
// log-sum-exp weights and rounds to half.  Scores, exponentials and the weighted sum are
// fp32 as in the reference; only the order of the additions differs.  (A first form with chunks
// of 64 positions whose rows went from global memory to registers in four dependent rounds took
// 20 us per chunk at the 2B-4T shape, half of a decode layer's time.)
#include <algorithm>

#include "attention_body.cuh"
#include "fused_ops.cuh"

namespace spb {

template <int G>
__global__ void __launch_bounds__(kAttnThreads) attn_split_kernel(
    const __half* __restrict__ Q, const __half* __restrict__ K, const __half* __restrict__ V,
    float* __restrict__ scratch, int num_kv_heads, int head_dim, int max_seq_len, int nsplit_max,
    float scale, int seq_len_arg, const int* __restrict__ d_pos, unsigned* counters, __half* out, const LlFan fan) {
    extern __shared__ __align__(16) uint8_t attn_sm[];
    __shared__ int s_last;
    grid_dep_launch();
    grid_dep_wait();
    const int seq_len = d_pos ? (*d_pos + 1) : seq_len_arg;
    const unsigned fan_tag = fan.ndst ? *reinterpret_cast<const volatile unsigned*>(fan.seq) + 1u : 0u;
    const int kvh = blockIdx.x, split = blockIdx.y;
    if (split * attn_chunk(seq_len) >= seq_len) return;
    attn_chunk_block<G>(Q, K, V, scratch, kvh, split, head_dim, max_seq_len, nsplit_max, scale, seq_len, attn_sm);
    if (!counters) return;  // the chunks are merged by attn_combine_kernel
    // One launch: the block that completes a KV head's chunk count merges them (and leaves the count at zero for the
    // next call).  The fence is cumulative over the block's stores, which the barrier made known to thread 0.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned old = atomicAdd(counters + kvh, 1u);
        const int last = old + 1u == static_cast<unsigned>(attn_nsplit(seq_len));
        if (last) atomicExch(counters + kvh, 0u);
        __threadfence();
        s_last = last;
    }
    __syncthreads();
    if (s_last)
        attn_merge_group<G>(scratch, out, kvh, head_dim, nsplit_max, attn_nsplit(seq_len), reinterpret_cast<float*>(attn_sm),
                            fan.ndst ? &fan : nullptr, fan_tag);
}

template <int G>
__global__ void __launch_bounds__(kAttnThreads) attn_combine_kernel(const float* __restrict__ scratch,
                                                                    __half* __restrict__ out, int head_dim,
                                                                    int nsplit_max, int seq_len_arg,
                                                                    const int* __restrict__ d_pos) {
    extern __shared__ __align__(16) float merge_sm[];
    grid_dep_launch();
    grid_dep_wait();
    const int seq_len = d_pos ? (*d_pos + 1) : seq_len_arg;
    attn_merge_group<G>(scratch, out, blockIdx.x, head_dim, nsplit_max, attn_nsplit(seq_len), merge_sm);
}

// seq_len is taken from *d_pos + 1 when d_pos is given (graph replay), else from seq_len.
int decode_attention_split(const void* Q, const void* K, const void* V, void* out, int num_heads,
                           int num_kv_heads, int head_dim, int max_seq_len, int seq_len, const int* d_pos,
                           float scale, float* scratch, void* stream, unsigned* counters, const LlFan* fan) {
    const char* name = "decode_attention_split";
    if (fan && (!counters || (num_heads * head_dim) % 2)) return fail(SPB_E_INVALID, "%s: a fan-out wants the merge in the launch", name);
    const LlFan fanv = fan ? *fan : LlFan{};
    if (num_heads % num_kv_heads) return fail(SPB_E_UNSUPPORTED, "%s: %d heads over %d KV heads", name, num_heads, num_kv_heads);
    const int G = num_heads / num_kv_heads;
    if (!decode_attention_split_supported(num_heads, num_kv_heads, head_dim) ||
        ((reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(V)) & 15u))
        return fail(SPB_E_UNSUPPORTED, "%s: group %d / head_dim %d / alignment outside the kernel's range", name, G, head_dim);
    if (reinterpret_cast<uintptr_t>(scratch) & 7u) return fail(SPB_E_INVALID, "%s: the scratch buffer must be 8-byte aligned", name);
    const int nsplit_max = attn_nsplit_max(max_seq_len);
    const int nsplit = d_pos ? nsplit_max : attn_nsplit(seq_len);
    const size_t msmem = sizeof(float) * attn_merge_smem_floats(G, max_seq_len);
    const size_t smem = counters ? std::max(attn_smem_bytes(G, head_dim), msmem) : attn_smem_bytes(G, head_dim);
    const dim3 grid(num_kv_heads, nsplit);
    const __half* q = static_cast<const __half*>(Q);
    const __half* k = static_cast<const __half*>(K);
    const __half* v = static_cast<const __half*>(V);
    int rc = SPB_OK;
#define SPB_ATTN_CASE(GG)                                                                                  \
    case GG:                                                                                               \
        if ((rc = ensure_dynamic_smem(name, attn_split_kernel<GG>, smem))) return rc;                      \
        if ((rc = ensure_dynamic_smem(name, attn_combine_kernel<GG>, msmem))) return rc;                   \
        rc = launch(name, attn_split_kernel<GG>, grid, dim3(kAttnThreads), smem, stream, q, k, v, scratch, \
                    num_kv_heads, head_dim, max_seq_len, nsplit_max, scale, seq_len, d_pos, counters,      \
                    static_cast<__half*>(out), fanv);                                                      \
        if (rc || counters) return rc;                                                                     \
        return launch("attn_combine", attn_combine_kernel<GG>, dim3(num_kv_heads), dim3(kAttnThreads), msmem, stream, \
                      static_cast<const float*>(scratch), static_cast<__half*>(out), head_dim, nsplit_max, seq_len, d_pos);
    switch (G) {
        SPB_ATTN_CASE(1) SPB_ATTN_CASE(2) SPB_ATTN_CASE(3) SPB_ATTN_CASE(4) SPB_ATTN_CASE(5) SPB_ATTN_CASE(6)
        SPB_ATTN_CASE(7) SPB_ATTN_CASE(8)
        default: return fail(SPB_E_UNSUPPORTED, "%s: group %d", name, G);
    }
#undef SPB_ATTN_CASE
    return rc;
}

bool decode_attention_split_supported(int num_heads, int num_kv_heads, int head_dim) {
    return num_kv_heads > 0 && num_heads % num_kv_heads == 0 && num_heads / num_kv_heads <= kMaxGroup && head_dim >= 8 &&
           head_dim <= 256 && head_dim % 8 == 0;
}

size_t decode_attention_scratch_bytes(int num_heads, int head_dim, int max_seq_len) {
    return sizeof(float) * attn_scratch_floats(num_heads, head_dim, max_seq_len);
}

}  // namespace spb

using namespace spb;

extern "C" size_t spb_decode_attention_scratch_bytes(int num_heads, int head_dim, int max_seq_len) {
    if (num_heads <= 0 || head_dim <= 0 || max_seq_len <= 0) return 0;
    return decode_attention_scratch_bytes(num_heads, head_dim, max_seq_len);
}

extern "C" int spb_decode_attention_split(const void* Q, const void* K_cache, const void* V_cache, void* output,
                                          int num_heads, int num_kv_heads, int head_dim, int max_seq_len,
                                          int seq_len, float scale, void* scratch, size_t scratch_bytes,
                                          void* stream) {
    const char* name = "spb_decode_attention_split";
    if (num_heads < 0 || num_kv_heads <= 0 || head_dim <= 0) return fail(SPB_E_INVALID, "%s: bad shape", name);
    if (seq_len < 1 || seq_len > max_seq_len) return fail(SPB_E_INVALID, "%s: seq_len outside the cache", name);
    if (num_heads == 0) return SPB_OK;
    if (!Q || !K_cache || !V_cache || !output || !scratch) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (scratch_bytes < decode_attention_scratch_bytes(num_heads, head_dim, max_seq_len))
        return fail(SPB_E_INVALID, "%s: scratch of %zu bytes is smaller than spb_decode_attention_scratch_bytes()", name,
                    scratch_bytes);
    return decode_attention_split(Q, K_cache, V_cache, output, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len,
                                  nullptr, scale, static_cast<float*>(scratch), stream);
}
