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
int embed_token(const void* embed, void* x, int hidden, const int* d_prompt, int n_prompt,
                const int* d_next, const int* d_pos, void* stream);
int argmax_advance(const float* logits, int n, float* bval, int* bidx, int nblocks, int* d_next,
                   int* d_out, int* d_pos, void* stream);
int set_int(int* dst, int value, void* stream);

// gemv.cu: up to three BitLinear layers that consume the same quantised activation, one launch.
int bitlinear_q8_group(const uint32_t* const* meta, const uint32_t* const* values, void* const* out,
                       const float* gamma, const int* rows, const int* ms, const int* vs, int nmat,
                       const int8_t* xq, const float* d_absmax, int cols, void* stream);

}  // namespace spb
