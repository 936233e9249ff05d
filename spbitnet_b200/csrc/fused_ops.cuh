// Host launchers of the fused decode-step kernels (fused_ops.cu); engine-internal.
// `vectors` > 1 runs the op on that many consecutive vectors (the tokens of a prefill batch): vector b of every
// operand starts b * its length after the first, d_absmax is an array, and token b sits at position *d_pos + b.
// rope_scatter / decode_attention_pos with seq_stride != 0 treat the vectors as one token each of independent
// sequences instead (batched decode): all at position *d_pos, sequence b's K and V caches b * seq_stride elements
// after the first sequence's.
#pragma once
#include "spb_common.cuh"

namespace spb {

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
int decode_attention_split(const void* Q, const void* K, const void* V, void* out, int num_heads,
                           int num_kv_heads, int head_dim, int max_seq_len, int seq_len, const int* d_pos,
                           float scale, float* scratch, void* stream);
size_t decode_attention_scratch_bytes(int num_heads, int head_dim, int max_seq_len);
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

// gemv.cu: up to three BitLinear layers that consume the same activation vector, one launch.
struct BitLinearGroup {
    const uint32_t* meta[3];
    const uint32_t* values[3];
    void* out[3];  // half
    float gamma[3];
    int rows[3], ms[3], vs[3];
    int nmat, cols;
};
bool bitlinear_group_is_fast(const BitLinearGroup& g);
// activation already quantised (absmax_quantize_gpu output)
int bitlinear_q8_group(const BitLinearGroup& g, const int8_t* xq, const float* d_absmax, void* stream);
// activation = half vector; absmax formed inside the launch
int bitlinear_amax_group(const BitLinearGroup& g, const void* x_half, void* stream);
// activation = quantised rms_norm(w_norm) of x_out = x_in + [rms_norm(w_sub)](delta); block 0 writes x_out
int bitlinear_resnorm_group(const BitLinearGroup& g, const void* x_in, const void* delta, const float* w_sub,
                            const float* w_norm, void* x_out, float eps, void* stream);
// activation = quantised [rms_norm(w_sub)](relu(gate)^2 * up)
int bitlinear_relu2_group(const BitLinearGroup& g, const void* gate, const void* up, const float* w_sub, float eps,
                          void* stream);

}  // namespace spb
