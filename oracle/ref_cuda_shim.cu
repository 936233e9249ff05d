// ref_cuda_shim.cu -- extern "C" doorway onto the UNMODIFIED reference CUDA
// wrappers (include/spbitnet/sparse_ternary_kernels.h, inference_kernels.h),
// linked with the reference's own src/kernels/*.cu recompiled for sm_100a.
// TEST INFRASTRUCTURE ONLY: on a GPU it is the second checker beside the CPU
// oracle, and the bench times it as "the reference kernel on the same GPU".
#include "spbitnet/inference_kernels.h"
#include "spbitnet/sparse_ternary_kernels.h"

extern "C" {

void refcuda_unpack(const uint32_t* meta, const uint32_t* values, int8_t* out, int rows,
                    int cols, int ms, int vs, void* stream) {
    spbitnet::sparse_ternary_unpack_gpu(meta, values, out, rows, cols, ms, vs,
                                        static_cast<cudaStream_t>(stream));
}
void refcuda_gemv(const uint32_t* meta, const uint32_t* values, const int8_t* x, int32_t* y,
                  int rows, int cols, int ms, int vs, void* stream) {
    spbitnet::sparse_ternary_gemv_gpu(meta, values, x, y, rows, cols, ms, vs,
                                      static_cast<cudaStream_t>(stream));
}
void refcuda_fused_bitlinear(const uint32_t* meta, const uint32_t* values, const void* x,
                             void* out, const float* d_absmax, float gamma, int rows, int cols,
                             int ms, int vs, void* stream) {
    spbitnet::fused_sparse_bitlinear_gpu(meta, values, static_cast<const half*>(x),
                                         static_cast<half*>(out), d_absmax, gamma, rows, cols,
                                         ms, vs, static_cast<cudaStream_t>(stream));
}
void refcuda_absmax_reduce(const void* x, float* d_absmax, int n, void* stream) {
    spbitnet::absmax_reduce_gpu(static_cast<const half*>(x), d_absmax, n,
                                static_cast<cudaStream_t>(stream));
}
void refcuda_absmax_quantize(const void* x, int8_t* q, float* d_absmax, int n, void* stream) {
    spbitnet::absmax_quantize_gpu(static_cast<const half*>(x), q, d_absmax, n,
                                  static_cast<cudaStream_t>(stream));
}
void refcuda_rms_norm(const void* x, const float* w, void* out, int n, float eps, void* stream) {
    spbitnet::rms_norm_gpu(static_cast<const half*>(x), w, static_cast<half*>(out), n, eps,
                           static_cast<cudaStream_t>(stream));
}
void refcuda_half_gemv(const void* W, const void* x, float* y, int rows, int cols, void* stream) {
    spbitnet::half_gemv_gpu(static_cast<const half*>(W), static_cast<const half*>(x), y, rows,
                            cols, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

extern "C" {

void refcuda_dequantize(const int32_t* in, void* out, const float* d_absmax, float gamma, int n, void* stream) {
    spbitnet::dequantize_gpu(in, static_cast<half*>(out), d_absmax, gamma, n, static_cast<cudaStream_t>(stream));
}
void refcuda_rope(void* vec, int num_heads, int head_dim, int pos, float theta, void* stream) {
    spbitnet::rope_gpu(static_cast<half*>(vec), num_heads, head_dim, pos, theta, static_cast<cudaStream_t>(stream));
}
void refcuda_scatter_kv(const void* src, void* cache, int num_kv_heads, int head_dim, int max_seq_len, int pos,
                        void* stream) {
    spbitnet::scatter_kv_gpu(static_cast<const half*>(src), static_cast<half*>(cache), num_kv_heads, head_dim,
                             max_seq_len, pos, static_cast<cudaStream_t>(stream));
}
void refcuda_attention_scores(const void* Q, const void* K, float* scores, int num_heads, int num_kv_heads,
                              int head_dim, int max_seq_len, int seq_len, float scale, void* stream) {
    spbitnet::attention_scores_gpu(static_cast<const half*>(Q), static_cast<const half*>(K), scores, num_heads,
                                   num_kv_heads, head_dim, max_seq_len, seq_len, scale,
                                   static_cast<cudaStream_t>(stream));
}
void refcuda_softmax(float* scores, int num_heads, int max_seq_len, int seq_len, void* stream) {
    spbitnet::softmax_gpu(scores, num_heads, max_seq_len, seq_len, static_cast<cudaStream_t>(stream));
}
void refcuda_attention_output(const float* scores, const void* V, void* out, int num_heads, int num_kv_heads,
                              int head_dim, int max_seq_len, int seq_len, void* stream) {
    spbitnet::attention_output_gpu(scores, static_cast<const half*>(V), static_cast<half*>(out), num_heads,
                                   num_kv_heads, head_dim, max_seq_len, seq_len, static_cast<cudaStream_t>(stream));
}
void refcuda_relu2_mul_f32(const void* gate, const void* up, float* out, int n, void* stream) {
    spbitnet::relu2_mul_f32_gpu(static_cast<const half*>(gate), static_cast<const half*>(up), out, n,
                                static_cast<cudaStream_t>(stream));
}
void refcuda_rms_norm_f32in(const float* in, const float* w, void* out, int n, float eps, void* stream) {
    spbitnet::rms_norm_f32in_gpu(in, w, static_cast<half*>(out), n, eps, static_cast<cudaStream_t>(stream));
}
void refcuda_residual_add(const void* a, const void* b, void* out, int n, void* stream) {
    spbitnet::residual_add_gpu(static_cast<const half*>(a), static_cast<const half*>(b), static_cast<half*>(out), n,
                               static_cast<cudaStream_t>(stream));
}

}  // extern "C"
