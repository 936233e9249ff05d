// Host launchers of the fused decode-step kernels (fused_ops.cu); engine-internal.
// `vectors` > 1 runs the op on that many consecutive vectors (the tokens of a prefill batch): vector b of every
// operand starts b * its length after the first, d_absmax is an array, and token b sits at position *d_pos + b.
// rope_scatter / decode_attention_pos with seq_stride != 0 treat the vectors as one token each of independent
// sequences instead (batched decode): all at position *d_pos, sequence b's K and V caches b * seq_stride elements
// after the first sequence's.
#pragma once
#include "ll_words.cuh"
#include "spb_common.cuh"

namespace spb {

// rope_gpu on one (even, odd) pair of a head at position pos (src/kernels/inference_kernels.cu, rope_kernel):
// angle = pos / theta^(2 pair / head_dim), fp32 rotation, rounded to half.  The fused multiply-adds are written out
// so that every kernel that rotates (rope_scatter, the persistent decode step) rounds alike.
__device__ __forceinline__ void rope_angle(int pos, int pair, int head_dim, float theta, float& c, float& s) {
    const float freq = 1.0f / powf(theta, static_cast<float>(2 * pair) / static_cast<float>(head_dim));
    const float angle = static_cast<float>(pos) * freq;
    c = cosf(angle);
    s = sinf(angle);
}
__device__ __forceinline__ void rope_apply(float x0, float x1, float c, float s, __half& y0, __half& y1) {
    y0 = __float2half_rn(__fmaf_rn(x0, c, -__fmul_rn(x1, s)));
    y1 = __float2half_rn(__fmaf_rn(x0, s, __fmul_rn(x1, c)));
}
__device__ __forceinline__ void rope_rotate(float x0, float x1, int pos, int pair, int head_dim, float theta,
                                            __half& y0, __half& y1) {
    float c, s;
    rope_angle(pos, pair, head_dim, theta, c, s);
    rope_apply(x0, x1, c, s, y0, y1);
}

int residual_norm_quant(const void* delta, const float* sub_w, void* x, const float* w, void* xn_out,
                        int8_t* xq, float* d_absmax, int n, float eps, void* stream, int vectors = 1);
int relu2_norm_quant(const void* gate, const void* up, const float* sub_w, void* h_out, int8_t* hq,
                     float* d_absmax, int n, float eps, void* stream, int vectors = 1);
int rope_scatter(void* q, const void* k, const void* v, void* kcache, void* vcache, int num_heads,
                 int num_kv_heads, int head_dim, int max_seq_len, float theta, const int* d_pos,
                 void* stream, int vectors = 1, size_t seq_stride = 0);
int decode_attention_pos(const void* Q, const void* K, const void* V, void* out, int num_heads,
                         int num_kv_heads, int head_dim, int max_seq_len, float scale, const int* d_pos,
                         void* stream, int vectors = 1, size_t seq_stride = 0);
// attention.cu: split-KV decode attention.  seq_len comes from *d_pos + 1 when d_pos is given.
// `counters` (optional): num_kv_heads zeroed words; with them the merge of a KV head's chunks runs inside the same
// launch, in the block that finishes last, instead of as a second kernel.  They are left at zero.
// `fan` (with counters): the output goes out as tagged words to every destination of the fan instead of to `out`.
int decode_attention_split(const void* Q, const void* K, const void* V, void* out, int num_heads,
                           int num_kv_heads, int head_dim, int max_seq_len, int seq_len, const int* d_pos,
                           float scale, float* scratch, void* stream, unsigned* counters = nullptr,
                           const LlFan* fan = nullptr);
size_t decode_attention_scratch_bytes(int num_heads, int head_dim, int max_seq_len);
// the split kernel takes GQA groups of up to 8 heads and head dims that are multiples of 8 up to 256 (16-byte aligned Q, K, V)
bool decode_attention_split_supported(int num_heads, int num_kv_heads, int head_dim);
int embed_token(const void* embed, void* x, int hidden, const int* d_prompt, int n_prompt,
                const int* d_next, const int* d_pos, void* stream);
int argmax_advance(const float* logits, int n, float* bval, int* bidx, int nblocks, int* d_next,
                   int* d_out, int* d_pos, void* stream);
int set_int(int* dst, int value, void* stream);
// prefill.cu: row-batched forms, one block per token of the batch
int embed_rows(const void* embed, const int* d_tokens, void* x, int hidden, int vectors, void* stream);
int absmax_quantize_rows(const void* in, int8_t* out, float* d_absmax, int n, int vectors, void* stream);
int dequantize_rows(const int32_t* acc, void* out, const float* d_absmax, float gamma, int rows, int vectors,
                    void* stream);

// gemv_prepared.cu: BitLinear on weights re-laid by spb_prepare_weights; quantised activation, scaled half output
int prepared_bitlinear_q8(const void* prep, const int8_t* xq, void* out_half, const float* d_absmax, float gamma, int rows,
                          int cols, void* stream);

// gemv.cu: up to three BitLinear layers that consume the same activation vector, one launch.
struct BitLinearGroup {
    const uint32_t* meta[3];
    const uint32_t* values[3];
    void* out[3];  // half
    float gamma[3];
    int rows[3], ms[3], vs[3];
    int nmat, cols;
    const void* prep[3];  // optional: spb_prepare_weights copies of the matrices.  With all of them given, the launches
                          // with a producer (amax, resnorm, relu2) multiply on them when the group fits their one-wave
                          // form (gemv_prepared.cu: prepared_group_fused), else on the packed format
};
bool bitlinear_group_is_fast(const BitLinearGroup& g);
// activation already quantised (absmax_quantize_gpu output)
int bitlinear_q8_group(const BitLinearGroup& g, const int8_t* xq, const float* d_absmax, void* stream);
// activation = half vector; absmax formed inside the launch
int bitlinear_amax_group(const BitLinearGroup& g, const void* x_half, void* stream);
// What a q/k/v launch does with its rows instead of storing them as they are: matrix 0 (q) is rotated in place of
// the store (rope_gpu) and goes to out[0]; matrix 1 (k) is rotated and written to row *d_pos of the K cache, matrix 2
// (v) to row *d_pos of the V cache (scatter_kv_gpu): the launch absorbs the rope_scatter kernel.
struct RopeScatter {
    const int* d_pos;
    float theta;
    int head_dim, max_seq_len;
    void* kcache;  // [kv head][max_seq_len][head_dim] half
    void* vcache;
};
// Up to three BitLinears of the same width on prepared weights and one quantised activation, one launch
// (gemv_prepared.cu).  With `rope` they are q, k, v: q and k rows are rotated for the position in *rope->d_pos, k and
// v rows go to the cache rows of that position (out_half[1], out_half[2] are then not written).
// With `fans` (one per matrix, at most two matrices, even row counts) the rows go out as tagged words to every
// destination of the matrix's fan instead of to out_half.
int prepared_bitlinear_q8_group(const void* const* prep, void* const* out_half, const float* gamma, const int* rows, int n,
                                const int8_t* xq, const float* d_absmax, int cols, const RopeScatter* rope, void* stream,
                                const LlFan* fans = nullptr);
// activation = quantised rms_norm(w_norm) of x_out = x_in + [rms_norm(w_sub)](delta); block 0 writes x_out.
// With `rope` the group must be q, k, v (see RopeScatter).
int bitlinear_resnorm_group(const BitLinearGroup& g, const void* x_in, const void* delta, const float* w_sub,
                            const float* w_norm, void* x_out, float eps, void* stream, const RopeScatter* rope = nullptr);
// activation = quantised [rms_norm(w_sub)](relu(gate)^2 * up)
int bitlinear_relu2_group(const BitLinearGroup& g, const void* gate, const void* up, const float* w_sub, float eps,
                          void* stream);

}  // namespace spb
