// Host launchers of the fused decode-step kernels (fused_ops.cu); engine-internal.
#pragma once
#include "spb_common.cuh"

namespace spb {

int residual_norm_quant(const void* delta, const float* sub_w, void* x, const float* w, void* xn_out,
                        int8_t* xq, float* d_absmax, int n, float eps, void* stream);
int relu2_norm_quant(const void* gate, const void* up, const float* sub_w, void* h_out, int8_t* hq,
                     float* d_absmax, int n, float eps, void* stream);
int rope_scatter(void* q, const void* k, const void* v, void* kcache, void* vcache, int num_heads,
                 int num_kv_heads, int head_dim, int max_seq_len, float theta, const int* d_pos,
                 void* stream);
int decode_attention_pos(const void* Q, const void* K, const void* V, void* out, int num_heads,
                         int num_kv_heads, int head_dim, int max_seq_len, float scale, const int* d_pos,
                         void* stream);
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
