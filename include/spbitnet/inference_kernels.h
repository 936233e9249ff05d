#pragma once
// Drop-in replacement for the reference's include/spbitnet/inference_kernels.h: the same
// fifteen functions in namespace spbitnet with the same signatures, forwarding to the
// sm_100a library through its C-ABI.
#include <cstdint>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "b200_check.h"

namespace spbitnet {

inline void rms_norm_gpu(const half* input, const float* weight, half* output, int size, float eps,
                         cudaStream_t stream = nullptr) {  // reference inference_kernels.h:14-15
    SPB200_CHECK(spb_rms_norm(input, weight, output, size, eps, stream));
}
inline void absmax_quantize_gpu(const half* input, int8_t* output, float* d_absmax, int size,
                                cudaStream_t stream = nullptr) {  // :19-20
    SPB200_CHECK(spb_absmax_quantize(input, output, d_absmax, size, stream));
}
inline void absmax_reduce_gpu(const half* input, float* d_absmax, int size, cudaStream_t stream = nullptr) {  // :24-25
    SPB200_CHECK(spb_absmax_reduce(input, d_absmax, size, stream));
}
inline void dequantize_gpu(const int32_t* input, half* output, const float* d_absmax, float gamma, int size,
                           cudaStream_t stream = nullptr) {  // :29-30
    SPB200_CHECK(spb_dequantize(input, output, d_absmax, gamma, size, stream));
}
inline void rope_gpu(half* vec, int num_heads, int head_dim, int pos, float theta,
                     cudaStream_t stream = nullptr) {  // :33-34
    SPB200_CHECK(spb_rope(vec, num_heads, head_dim, pos, theta, stream));
}
inline void scatter_kv_gpu(const half* src, half* cache, int num_kv_heads, int head_dim, int max_seq_len, int pos,
                           cudaStream_t stream = nullptr) {  // :38-39
    SPB200_CHECK(spb_scatter_kv(src, cache, num_kv_heads, head_dim, max_seq_len, pos, stream));
}
inline void attention_scores_gpu(const half* Q, const half* K_cache, float* scores, int num_heads, int num_kv_heads,
                                 int head_dim, int max_seq_len, int seq_len, float scale,
                                 cudaStream_t stream = nullptr) {  // :44-47
    SPB200_CHECK(spb_attention_scores(Q, K_cache, scores, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len,
                                      scale, stream));
}
inline void softmax_gpu(float* scores, int num_heads, int max_seq_len, int seq_len,
                        cudaStream_t stream = nullptr) {  // :51-52
    SPB200_CHECK(spb_softmax(scores, num_heads, max_seq_len, seq_len, stream));
}
inline void attention_output_gpu(const float* scores, const half* V_cache, half* output, int num_heads,
                                 int num_kv_heads, int head_dim, int max_seq_len, int seq_len,
                                 cudaStream_t stream = nullptr) {  // :56-59
    SPB200_CHECK(spb_attention_output(scores, V_cache, output, num_heads, num_kv_heads, head_dim, max_seq_len,
                                      seq_len, stream));
}
inline void relu2_mul_gpu(const half* gate, const half* up, half* output, int size,
                          cudaStream_t stream = nullptr) {  // :62-63
    SPB200_CHECK(spb_relu2_mul(gate, up, output, size, stream));
}
inline void relu2_mul_f32_gpu(const half* gate, const half* up, float* output, int size,
                              cudaStream_t stream = nullptr) {  // :67-68
    SPB200_CHECK(spb_relu2_mul_f32(gate, up, output, size, stream));
}
inline void rms_norm_f32in_gpu(const float* input, const float* weight, half* output, int size, float eps,
                               cudaStream_t stream = nullptr) {  // :72-73
    SPB200_CHECK(spb_rms_norm_f32in(input, weight, output, size, eps, stream));
}
inline void float_to_half_gpu(const float* input, half* output, int size, cudaStream_t stream = nullptr) {  // :76-77
    SPB200_CHECK(spb_float_to_half(input, output, size, stream));
}
inline void residual_add_gpu(const half* a, const half* b, half* output, int size,
                             cudaStream_t stream = nullptr) {  // :80-81
    SPB200_CHECK(spb_residual_add(a, b, output, size, stream));
}
inline void half_gemv_gpu(const half* W, const half* x, float* y, int rows, int cols,
                          cudaStream_t stream = nullptr) {  // :86-87
    SPB200_CHECK(spb_half_gemv(W, x, y, rows, cols, stream));
}

}  // namespace spbitnet
