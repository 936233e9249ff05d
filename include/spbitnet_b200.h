/*
 * spbitnet_b200.h -- C-ABI of the B200 (sm_100a) sparse-ternary inference hot path.
 *
 * One plain-C entry point per host wrapper of the reference engine API
 * (namespace spbitnet, include/spbitnet/sparse_ternary_kernels.h and
 * include/spbitnet/inference_kernels.h in the reference project), with the
 * same argument order and meaning.  Differences from the C++ originals, all
 * forced by the C boundary:
 *   - cudaStream_t is passed as void* (NULL = the legacy default stream);
 *   - half* is passed as void* (IEEE binary16, 2 bytes per element);
 *   - every call returns an int status instead of calling exit(): 0 on
 *     success, a negative SPB_E_* otherwise; spb_last_error_string() describes
 *     the last failure on the calling thread.
 * All pointers are DEVICE pointers owned by the caller unless a parameter is
 * documented as host memory.  Calls are asynchronous on the given stream and
 * never synchronise, allocate or free (the engine and the *_host calls are the
 * exception: they own buffers).  rows==0 or cols==0 returns 0 without a launch,
 * like the reference (src/kernels/sparse_ternary.cu:244,261,280).
 *
 * The weight format is the reference's (include/spbitnet/sparse_ternary_tensor.h:12-39):
 * per group of four consecutive columns a 4-bit position bitmap with two bits
 * set (meta, 8 groups per uint32, LSB first) and a 2-bit sign pair (values, 16
 * groups per uint32, LSB first; bit0 = lower-index non-zero, 0 => +1, 1 => -1).
 * Row strides are in uint32 words.  cols must be a multiple of 4.
 */
#ifndef SPBITNET_B200_H
#define SPBITNET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPB_OK 0
#define SPB_E_INVALID (-1)     /* bad argument (null pointer, cols % 4, negative size ...) */
#define SPB_E_CUDA (-2)        /* a CUDA runtime call or launch failed */
#define SPB_E_TIMEOUT (-3)     /* a bounded device-side wait ran out */
#define SPB_E_UNSUPPORTED (-4) /* shape outside what the kernel handles */
#define SPB_E_FORMAT (-5)      /* packed data fails validation */

const char* spb_last_error_string(void);
/* Library version string, e.g. "spbitnet_b200 0.1 sm_100a". */
const char* spb_version(void);
/* 1 (default): kernels are launched with programmatic dependent launch so that the
 * weight prefetch of one kernel overlaps the tail of the previous one on the same
 * stream.  0: plain stream-ordered launches.  Returns the previous setting. */
int spb_set_pdl(int enabled);
/* Which GEMV kernel the sparse-ternary entry points use when the layout allows the fast paths:
 * 0 (default) = automatic: the warp-level sparse MMA kernel (mma.sp m16n8k64: the format is re-encoded
 *     in registers, not decoded) for int8 activations and one matrix per launch when cols % 256 == 0,
 *     row strides are multiples of 4 words and meta / values / x are 16-byte aligned; the pair kernel
 *     otherwise and for the fused half-input forms;
 * 1 = pair kernel (SIMT: one dp4a per two groups), 4 = warp-level sparse MMA kernel wherever the layout allows
 * it, the fused half-input and multi-matrix forms included.  Other values behave like 0.
 * Results are identical on valid bitmaps.  Returns the previous setting. */
int spb_set_gemv_variant(int variant);

/* ---- sparse-ternary kernels: include/spbitnet/sparse_ternary_kernels.h ---------- */

/* sparse_ternary_unpack_gpu (sparse_ternary_kernels.h:16-19; src/kernels/sparse_ternary.cu:58-102,240-254).
 * out: rows*cols int8, row-major. */
int spb_sparse_ternary_unpack(const uint32_t* meta, const uint32_t* values, int8_t* out,
                              int rows, int cols, int meta_row_stride, int values_row_stride,
                              void* stream);

/* sparse_ternary_gemv_gpu (sparse_ternary_kernels.h:29-33; src/kernels/sparse_ternary.cu:116-168,256-272).
 * x: cols int8; y: rows int32 accumulators, bit-exact. */
int spb_sparse_ternary_gemv(const uint32_t* meta, const uint32_t* values, const int8_t* x,
                            int32_t* y, int rows, int cols, int meta_row_stride,
                            int values_row_stride, void* stream);

/* Work-list form: one launch computes n independent GEMVs (the semantics of n calls of
 * spb_sparse_ternary_gemv) with a persistent grid, so per-launch fixed costs are paid once.
 * d_items is a DEVICE array of n items that the caller uploads once (a decode step's list is
 * static); it must be 16-byte aligned and satisfy spb_gemv_batch_check, which validates the HOST
 * copy: cols a multiple of 256 (at most 32768), row strides multiples of 4 words, meta/values/x
 * 16-byte aligned.  max_rows / max_cols bound the items (max_cols sizes shared memory); an item
 * with more than max_cols columns is skipped by the kernel (its y is left untouched), never copied. */
typedef struct {
    const uint32_t* meta;
    const uint32_t* values;
    const int8_t* x;
    int32_t* y;
    int rows, cols, meta_row_stride, values_row_stride;
} spb_gemv_item;
int spb_gemv_batch_check(const spb_gemv_item* h_items, int n);
int spb_sparse_ternary_gemv_batch(const spb_gemv_item* d_items, int n, int max_rows, int max_cols,
                                  void* stream);

/* The same walk with the dequantisation of dequantize_gpu applied in fp32 and kept
 * in fp32: y[r] = float(acc[r]) * ((gamma * absmax) / 127.0f), evaluated in that
 * order (src/kernels/inference_kernels.cu:169-170).  d_absmax: 1 float on the device.
 * y_acc may be NULL; when given it also receives the int32 accumulators. */
int spb_sparse_ternary_gemv_scaled(const uint32_t* meta, const uint32_t* values, const int8_t* x,
                                   float* y, int32_t* y_acc, const float* d_absmax, float gamma,
                                   int rows, int cols, int meta_row_stride,
                                   int values_row_stride, void* stream);

/* fused_sparse_bitlinear_gpu (sparse_ternary_kernels.h:43-48; src/kernels/sparse_ternary.cu:181-234,274-291).
 * x: cols half, quantised inline with *d_absmax; output: rows half. */
int spb_fused_sparse_bitlinear(const uint32_t* meta, const uint32_t* values, const void* x,
                               void* output, const float* d_absmax, float gamma, int rows,
                               int cols, int meta_row_stride, int values_row_stride,
                               void* stream);

/* BitLinear on an activation that is already quantised (absmax_quantize_gpu output):
 * the integer walk of sparse_ternary_gemv_gpu followed by dequantize_gpu in one
 * launch.  Results equal spb_fused_sparse_bitlinear on the unquantised vector. */
int spb_sparse_bitlinear_q8(const uint32_t* meta, const uint32_t* values, const int8_t* xq,
                            void* output, const float* d_absmax, float gamma, int rows,
                            int cols, int meta_row_stride, int values_row_stride,
                            void* stream);

/* Batched form.  The reference has no sparse_ternary_gemm; its batched path is
 * CuSparseLtGemm::execute (include/spbitnet/cusparselt_backend.h:47-50), whose operand
 * layout this follows: X is [cols, n] column-major with ld = cols (n activation rows
 * of cols int8), Y is [rows, n] column-major with ld = rows (n output rows of rows
 * int32).  Y[j*rows + r] = sum_c W[r][c] * X[j*cols + c].  Any n >= 1. */
int spb_sparse_ternary_gemm(const uint32_t* meta, const uint32_t* values, const int8_t* X,
                            int32_t* Y, int rows, int cols, int n, int meta_row_stride,
                            int values_row_stride, void* stream);

/* BitLinear over a batch of quantised activation rows: the product above followed by dequantize_gpu
 * (src/kernels/inference_kernels.cu:162-171) per activation row, i.e. what n calls of spb_sparse_bitlinear_q8
 * give.  Xq: n rows of cols int8 (absmax_quantize_gpu outputs); d_absmax: their n scales (device);
 * output: n rows of `rows` half, output[j*rows + r] = half(float(acc) * (gamma * d_absmax[j] / 127)).
 * The default forms write the scaled output from their own epilogues; the other forms (set by
 * spb_set_gemm_variant, or taken for layouts the tensor-core forms do not cover) need acc_workspace, a device
 * buffer of n * rows int32 whose contents are overwritten, and answer SPB_E_UNSUPPORTED when it is NULL.
 * The reference has no batched BitLinear; its prefill calls fused_sparse_bitlinear_gpu once per token
 * (src/main.cpp:266-267, src/inference.cu:106-117). */
int spb_sparse_bitlinear_gemm(const uint32_t* meta, const uint32_t* values, const int8_t* Xq, void* output,
                              const float* d_absmax, float gamma, int32_t* acc_workspace, int rows, int cols,
                              int n, int meta_row_stride, int values_row_stride, void* stream);

/* Which form spb_sparse_ternary_gemm uses: 0 (default) = automatic: up to 32 batch rows the warp-level
 * sparse MMA form (mma.sp m16n8k64, operands re-encoded in registers; needs cols % 256 == 0, row strides
 * that are multiples of 4 words and 16-byte aligned meta / values / X), above that the tcgen05 sparse form
 * (tcgen05.mma.sp: sign bytes as the compressed operand, index pairs in tensor memory), the SIMT form where
 * the layout allows neither; 1 = SIMT form, 3 = tcgen05 sparse form for any n, 4 = warp-level sparse MMA
 * form where it applies.  Other values behave like 0.  Results are identical.  Returns the previous setting. */
int spb_set_gemm_variant(int variant);
/* Weight rows per block of the tcgen05 sparse form: 0 (default) = automatic, 1 = 128 rows, 2 = 256 rows (two
 * accumulators on one activation tile; needs more than 128 batch rows).  Results are identical; a testing and
 * measurement aid.  Returns the previous setting. */
int spb_set_gemm_row_halves(int halves);
/* Number of bounded device-side waits of the tcgen05 product that ran out since the library was loaded, over all
 * GPUs of the process; 0 in a healthy run, -1 if the counter cannot be read.  Synchronises the current device.
 * A block whose wait ran out skips its epilogue and frees its tensor memory, so the outputs of that call are
 * unspecified.  The kernel entry points are asynchronous and cannot report this themselves: callers of
 * spb_sparse_ternary_gemm / spb_sparse_bitlinear_gemm that need the guarantee compare this counter before and
 * after (once the stream is synchronised).  The engine does so at its own synchronisation points
 * (spb_engine_prefill, spb_engine_generate, spb_engine_copy_logits) and returns SPB_E_TIMEOUT when it moved. */
int spb_gemm_tc_timeouts(void);
/* Testing aid, no counterpart in the reference: launches one block that allocates tensor memory, waits with the
 * product kernel's bounded wait (limit_cycles, clamped to [1000, 40000000] SM clocks) on a barrier that nobody
 * arrives at, counts the run-out like the product kernel, frees its tensor memory and returns; then synchronises
 * the stream.  Returns SPB_E_TIMEOUT (the expected answer: the wait ran out and was reported) or SPB_E_CUDA.
 * Nothing is left in flight and the context stays usable. */
int spb_debug_bounded_wait_selftest(long long limit_cycles, void* stream);

/* ---- transformer kernels: include/spbitnet/inference_kernels.h ------------------- */

/* rms_norm_gpu (inference_kernels.h:14-15; src/kernels/inference_kernels.cu:15-56). input may alias output. */
int spb_rms_norm(const void* input, const float* weight, void* output, int size, float eps,
                 void* stream);
/* absmax_quantize_gpu (inference_kernels.h:19-20; inference_kernels.cu:69-114). */
int spb_absmax_quantize(const void* input, int8_t* output, float* d_absmax, int size,
                        void* stream);
/* absmax_reduce_gpu (inference_kernels.h:24-25; inference_kernels.cu:120-148). */
int spb_absmax_reduce(const void* input, float* d_absmax, int size, void* stream);
/* dequantize_gpu (inference_kernels.h:29-30; inference_kernels.cu:162-171). */
int spb_dequantize(const int32_t* input, void* output, const float* d_absmax, float gamma,
                   int size, void* stream);
/* rope_gpu (inference_kernels.h:33-34; inference_kernels.cu:185-206). In place. */
int spb_rope(void* vec, int num_heads, int head_dim, int pos, float theta, void* stream);
/* scatter_kv_gpu (inference_kernels.h:38-39; inference_kernels.cu:215-227). */
int spb_scatter_kv(const void* src, void* cache, int num_kv_heads, int head_dim,
                   int max_seq_len, int pos, void* stream);
/* attention_scores_gpu (inference_kernels.h:44-47; inference_kernels.cu:241-275). */
int spb_attention_scores(const void* Q, const void* K_cache, float* scores, int num_heads,
                         int num_kv_heads, int head_dim, int max_seq_len, int seq_len,
                         float scale, void* stream);
/* softmax_gpu (inference_kernels.h:51-52; inference_kernels.cu:283-339). In place. */
int spb_softmax(float* scores, int num_heads, int max_seq_len, int seq_len, void* stream);
/* attention_output_gpu (inference_kernels.h:56-59; inference_kernels.cu:350-371). */
int spb_attention_output(const float* scores, const void* V_cache, void* output, int num_heads,
                         int num_kv_heads, int head_dim, int max_seq_len, int seq_len,
                         void* stream);
/* relu2_mul_gpu (inference_kernels.h:62-63; inference_kernels.cu:379-390). */
int spb_relu2_mul(const void* gate, const void* up, void* output, int size, void* stream);
/* relu2_mul_f32_gpu (inference_kernels.h:67-68; inference_kernels.cu:399-410). */
int spb_relu2_mul_f32(const void* gate, const void* up, float* output, int size, void* stream);
/* rms_norm_f32in_gpu (inference_kernels.h:72-73; inference_kernels.cu:418-455). */
int spb_rms_norm_f32in(const float* input, const float* weight, void* output, int size,
                       float eps, void* stream);
/* float_to_half_gpu (inference_kernels.h:76-77; inference_kernels.cu:460-466). */
int spb_float_to_half(const float* input, void* output, int size, void* stream);
/* residual_add_gpu (inference_kernels.h:80-81; inference_kernels.cu:471-479). */
int spb_residual_add(const void* a, const void* b, void* output, int size, void* stream);
/* half_gemv_gpu (inference_kernels.h:86-87; inference_kernels.cu:488-531). */
int spb_half_gemv(const void* W, const void* x, float* y, int rows, int cols, void* stream);

/* One-launch decode attention for a single new token: attention_scores_gpu, softmax_gpu
 * and attention_output_gpu (src/inference.cu:188-202) without the scores round trip.
 * Q: (num_heads, head_dim) half; caches (num_kv_heads, max_seq_len, head_dim) half;
 * output (num_heads, head_dim) half. */
int spb_decode_attention(const void* Q, const void* K_cache, const void* V_cache, void* output,
                         int num_heads, int num_kv_heads, int head_dim, int max_seq_len,
                         int seq_len, float scale, void* stream);

/* The same result as spb_decode_attention from a split-KV pass: the positions are cut into
 * chunks served by separate blocks (all query heads of a GQA group share one read of their K/V
 * rows) and merged by a second small kernel.  Needs a device scratch buffer of at least
 * spb_decode_attention_scratch_bytes(num_heads, head_dim, max_seq_len) bytes, owned by the caller;
 * its contents need no initialisation and are overwritten.  num_heads must be a multiple of
 * num_kv_heads with at most 8 query heads per KV head; head_dim <= 256. */
size_t spb_decode_attention_scratch_bytes(int num_heads, int head_dim, int max_seq_len);
int spb_decode_attention_split(const void* Q, const void* K_cache, const void* V_cache, void* output,
                               int num_heads, int num_kv_heads, int head_dim, int max_seq_len, int seq_len,
                               float scale, void* scratch, size_t scratch_bytes, void* stream);

/* No counterpart in the reference.  spb_decode_attention_split for callers that cannot supply the
 * scratch buffer: an engine whose device buffers were all laid out up front (the reference's
 * InferenceEngine is one), code inside a stream capture, or a serving loop that must not stall
 * the GPU cannot call cudaMalloc between decode steps.  The partial results go to an array built
 * into the library instead (spb_decode_attention_noalloc_capacity() bytes, 2 MiB, resident on every
 * GPU that loads the library until the process exits); the call allocates and frees nothing.
 * Shapes whose partial results (spb_decode_attention_scratch_bytes) exceed the capacity are refused
 * with SPB_E_UNSUPPORTED.  The first call on a device looks up the array's device address (one
 * cudaGetSymbolAddress, with that device current); make that first call outside any stream capture.
 * All calls on a device share the one array: calls that may overlap on the GPU (different
 * streams without ordering) race on it and must be serialised by the caller. */
size_t spb_decode_attention_noalloc_capacity(void);
int spb_decode_attention_noalloc(const void* Q, const void* K_cache, const void* V_cache, void* output,
                                 int num_heads, int num_kv_heads, int head_dim, int max_seq_len, int seq_len,
                                 float scale, void* stream);

/* ---- host-side format helpers: include/spbitnet/sparse_ternary_tensor.h ----------- */

/* Row strides in uint32 words (sparse_ternary_tensor.h:254-264). */
int spb_meta_words_per_row(int cols);
int spb_values_words_per_row(int cols);
/* SparseTernaryTensor::pack_from_dense (sparse_ternary_tensor.h:58-108). HOST pointers.
 * meta/values are overwritten.  SPB_E_FORMAT if a group keeps other than two entries. */
int spb_pack_from_dense(const int8_t* weights, const uint8_t* mask, int rows, int cols,
                        uint32_t* meta, uint32_t* values);
/* SparseTernaryTensor::pack_with_pruning (sparse_ternary_tensor.h:123-191). HOST pointers. */
int spb_pack_with_pruning(const float* latent, int rows, int cols, uint32_t* meta,
                          uint32_t* values);
/* SparseTernaryTensor::unpack_to_int8 (sparse_ternary_tensor.h:197-232). HOST pointers. */
int spb_unpack_to_int8_host(const uint32_t* meta, const uint32_t* values, int rows, int cols,
                            int meta_row_stride, int values_row_stride, int8_t* out);
/* SPB_OK when every visited bitmap has exactly two bits set, else SPB_E_FORMAT. HOST pointers.
 * The reference leaves other bitmaps undefined: its GPU table maps them to positions (0,0)
 * (src/kernels/sparse_ternary.cu:34-51) while its CPU unpack yields as many non-zeros as bits.
 * Loaders should reject them with this call; the GPU entry points require valid bitmaps and
 * give an unspecified (but memory-safe) result otherwise. */
int spb_validate_packed(const uint32_t* meta, int rows, int cols, int meta_row_stride);

/* Conversion on the GPU (the pruning + quantisation + packing steps of python/convert_model.py:88-138,
 * 141-207, 270-283 in one kernel): weights is a device float32 matrix (rows x cols, weights_row_stride
 * floats between rows, cols % 4 == 0); meta / values receive the packed arrays, byte-identical to what the
 * converter writes (two largest |w| per group of four, the higher index on ties; a kept weight is -1 exactly
 * when w < 0).  abs_sum, if not NULL, is a device double that the kernel ADDS sum |w| to (zero it first):
 * gamma = abs_sum / (rows * cols).  The sum is accumulated in double precision and may differ from numpy's
 * float32 mean in the last bits.  The reference converts on the CPU only; this entry point has no GPU
 * counterpart there. */
int spb_prune_pack_gpu(const float* weights, int rows, int cols, size_t weights_row_stride, uint32_t* meta,
                       uint32_t* values, int meta_row_stride, int values_row_stride, double* abs_sum, void* stream);

/* ---- engine: include/spbitnet/inference.h:23-70, src/inference.cu ----------------- */

/* ---- prepared weights: the packed format re-laid once for the warp-level sparse MMA --------------------------------
 * An owner of weights that uploads them once (an engine) may trade the packed rows for a device-private layout of the
 * same density (1.5 bits per weight) in which the GEMV finds its tensor-core operands almost ready: per tile of 16
 * rows and 256 columns, 768 contiguous bytes = the lanes' metadata words (bitmaps already as index pairs) and the
 * lanes' sign bits in the order a byte permute expands them.  Results are the packed GEMV's, bit for bit.  It pays
 * for matrices of tens of megabytes (4.9 against 3.2 TB/s at 28672 x 8192); small ones are quicker in the packed form.
 * cols must be a multiple of 256 (<= 65536); rows beyond a multiple of 16 are padded inside the buffer. */
/* Bytes of the prepared form (0 for a shape it does not take). */
size_t spb_prepared_weights_bytes(int rows, int cols);
/* Packed rows (device, strides in uint32 words as everywhere) -> prepared buffer (device, 16-byte aligned). */
int spb_prepare_weights(const uint32_t* d_meta, const uint32_t* d_values, int rows, int cols, int meta_row_stride,
                        int values_row_stride, void* d_prepared, void* stream);
/* y[r] = sum_c W[r, c] * x[c], int32, as spb_sparse_ternary_gemv.  x 16-byte aligned. */
int spb_prepared_gemv(const void* d_prepared, const int8_t* d_x, int32_t* d_y, int rows, int cols, void* stream);
/* As spb_sparse_bitlinear_q8: out[r] = half(float(acc) * gamma * absmax / 127). */
int spb_prepared_bitlinear_q8(const void* d_prepared, const int8_t* d_xq, void* d_out_half, const float* d_absmax,
                              float gamma, int rows, int cols, void* stream);

typedef struct spb_engine spb_engine;

typedef struct {
    int hidden_size, num_hidden_layers, num_attention_heads, num_key_value_heads;
    int head_dim, intermediate_size, vocab_size, max_position_embeddings;
    float rms_norm_eps, rope_theta;
} spb_model_config; /* the fields of ModelConfig the forward pass reads (include/spbitnet/model.h:22-38) */

/* InferenceEngine::InferenceEngine (src/inference.cu:16-69): allocates KV caches and
 * scratch on the current device.  Weights are attached afterwards; the engine borrows them. */
spb_engine* spb_engine_create(const spb_model_config* cfg);
void spb_engine_destroy(spb_engine* e);
/* SparseLinear (include/spbitnet/model.h:46-60). which: 0 q, 1 k, 2 v, 3 o, 4 gate, 5 up, 6 down. */
int spb_engine_set_linear(spb_engine* e, int layer, int which, const uint32_t* d_meta,
                          const uint32_t* d_values, float gamma, int rows, int cols,
                          int meta_stride, int values_stride);
/* TransformerLayer norms (model.h:63-83). which: 0 input_layernorm, 1 post_attention_layernorm,
 * 2 attn_sub_norm, 3 ffn_sub_norm (2 and 3 optional). */
int spb_engine_set_norm(spb_engine* e, int layer, int which, const float* d_weight);
/* embed_tokens / lm_head (NULL = tied) / final_norm (model.h:118-128). */
int spb_engine_set_globals(spb_engine* e, const void* d_embed, const void* d_lm_head,
                           const float* d_final_norm);
/* InferenceEngine::forward (src/inference.cu:123-283): one token, returns the DEVICE
 * logits pointer (vocab_size floats) through *d_logits. */
int spb_engine_forward(spb_engine* e, int token_id, const float** d_logits);
/* InferenceEngine::reset (src/inference.cu:91-100). */
int spb_engine_reset(spb_engine* e);
/* InferenceEngine::seq_len (include/spbitnet/inference.h:38). */
int spb_engine_seq_len(const spb_engine* e);
/* The greedy loop of src/main.cpp:266-300 with the arg-max on the device (first
 * maximum wins, like std::max_element): feeds prompt[0..n_prompt-2], then generates
 * max_tokens tokens starting from prompt[n_prompt-1]; stops early at eos_token_id
 * (pass -1 for none).  prompt/out_tokens are HOST pointers; returns the number of
 * tokens written to out_tokens, or a negative status. */
int spb_engine_generate(spb_engine* e, const int* prompt, int n_prompt, int max_tokens,
                        int eos_token_id, int* out_tokens);
/* Copies the last forward's logits to HOST memory (vocab_size floats); synchronises. */
int spb_engine_copy_logits(spb_engine* e, float* h_logits);

/* Batched prefill: n tokens (HOST array) enter the model together from the engine's current position, as n
 * calls of spb_engine_forward would feed them one by one (the reference's prefill is that loop,
 * src/main.cpp:266-267).  The BitLinear layers run as spb_sparse_ternary_gemm over the n quantised activation
 * rows; norms, quantisation, RoPE and the KV scatter run per row with the rounding points of the
 * token-serial step, so integer accumulators and int8 activations are identical and the logits of the last
 * token (the only ones formed; *d_logits, device, vocab_size floats) agree with the token-serial ones within
 * the attention kernels' summation order.  Tokens are processed at most 1024 at a time (or the chunk set by
 * spb_engine_set_prefill_chunk); the first call that needs them allocates the batch buffers (about 150 KB per
 * token of the chunk at the 2B-4T shape, sized by the longest chunk seen).  Synchronises the engine's stream
 * before returning. */
int spb_engine_prefill(spb_engine* e, const int* tokens, int n, const float** d_logits);
/* How spb_engine_generate feeds the prompt: 0 (default) = token by token like the reference's loop;
 * c > 0 = as batches of up to min(c, 1024) tokens through the prefill path above (spb_engine_prefill uses
 * the same chunk when it is set, else 1024).  Returns the previous
 * setting, or a negative status. */
int spb_engine_set_prefill_chunk(spb_engine* e, int chunk);
/* How the layers of a decode token are run:
 *   0 (default) and 1: a chain of five PDL-linked kernels per layer (the vector ops fused into the BitLinear launches,
 *     RoPE and the KV scatter into the q/k/v launch, the merge of the attention chunks into the attention launch);
 *   2 the persistent kernel: one cooperative launch per token, a block per SM, grid barriers between the stages of
 *     a layer, weights prefetched into shared memory; SPB_E_UNSUPPORTED at the next step if the model does not fit.
 *     Measured slower than the chain so far (see the design notes), hence not the default;
 *   3 the chain with every vector op group as its own launch (the reference's op order, for testing);
 *   4 the persistent kernel without grid barriers: every stage writes its output vector as 8-byte words {two
 *     halves, tag} (tag = launch count and layer), the consumers poll the words they need until the tag is there,
 *     and every block keeps the residual stream in its shared memory.  Needs at least as many 16-row tiles as SMs
 *     in every projection (hidden size >= 16 x SMs), else SPB_E_UNSUPPORTED at the next step.
 * All modes produce the same tokens and logits bit for bit.  Every wait of the persistent kernel (grid barrier,
 * tagged word, weight copy) is bounded (about a second); when one runs out the step's results are unspecified, the
 * library's timeout counter moves (SPB_E_TIMEOUT from the engine call that synchronises next) and spb_engine_reset
 * clears the barrier state and the tagged words. */
int spb_engine_set_decode_mode(spb_engine* e, int mode);
/* Whether the chain of fused launches (decode modes 0 and 1) multiplies on prepared copies of the matrices
 * (spb_prepare_weights; the engine builds and owns them, as large as the packed tensors, when the next step is set
 * up): 1 (default) yes, for every group of matrices that fits the one-wave form of that kernel, 0 no (the
 * packed-format kernels).  With the copies a warp holds all its weights in registers before its launch's dependency
 * resolves.  Same tokens and logits bit for bit. */
int spb_engine_set_prepared_weights(spb_engine* e, int on);
/* 1 when the last step that was set up runs the persistent kernel. */
int spb_engine_decode_is_persistent(const spb_engine* e);
/* Test aid: two blocks at a grid barrier that expects three; both waits run out after limit_cycles (clamped),
 * the run-out is counted, the kernel returns.  Returns SPB_E_TIMEOUT when that happened as it must. */
int spb_debug_grid_barrier_selftest(long long limit_cycles, void* stream);
/* Diagnostic: persistent decode kernels enqueued (or captured) after this call record stage times.  d_trace is device
 * memory for 2 x 4096 64-bit words, or NULL to switch the recording off: thread 0 of the first block writes words
 * [0, 4096), thread 0 of the last block [4096, 8192); word 20 * layer + k is the global nanosecond timer at point k of
 * that layer (0-3 stage 1: weights there, activation produced, rows done, barrier passed; 4-6 stage 2: next slab
 * issued, attention chunks done, barrier passed; 7-10, 11-14, 15-18 stages 3, 4, 5 as stage 1).  Each token overwrites
 * the previous one's marks.  python -m spbitnet_b200.decode_trace prints the table. */
void spb_debug_set_decode_trace(void* d_trace);

/* ---- model directory loader: include/spbitnet/model.h:88-145, src/model.cu:179-311 ---------------------- */

typedef struct spb_model spb_model;
/* Model::load: reads <dir>/config.json, <dir>/manifest.json and the weight files into ONE device allocation on the
 * current device (sizes checked against shapes and strides, sparse bitmaps validated).  NULL on failure
 * (spb_last_error_string says why).  The reference throws std::runtime_error instead. */
spb_model* spb_model_load(const char* model_dir);
void spb_model_destroy(spb_model* m);
/* ModelConfig (model.h:22-38): the fields of spb_model_config plus bos_token_id / eos_token_id (either may be NULL). */
int spb_model_get_config(const spb_model* m, spb_model_config* cfg, int* bos_token_id, int* eos_token_id);
size_t spb_model_device_bytes(const spb_model* m);
/* Attaches every tensor of the model to an engine created with the model's config (the engine borrows them). */
int spb_model_attach(const spb_model* m, spb_engine* e);

/* ---- tokenizer: include/spbitnet/tokenizer.h, src/tokenizer.cpp (host only) --------------------------- */

typedef struct spb_tokenizer spb_tokenizer;
/* Tokenizer::load (tokenizer.h:20, src/tokenizer.cpp:287-339): a HuggingFace tokenizer.json (byte-level BPE). */
spb_tokenizer* spb_tokenizer_load(const char* tokenizer_json_path);
void spb_tokenizer_destroy(spb_tokenizer* t);
int spb_tokenizer_vocab_size(const spb_tokenizer* t);
/* Tokenizer::encode (tokenizer.h:23, src/tokenizer.cpp:341-357): no BOS / EOS added.  Writes at most `capacity`
 * ids and returns the number the text encodes to (call with capacity 0 to size the buffer), or a negative status. */
int spb_tokenizer_encode(const spb_tokenizer* t, const char* text, size_t text_bytes, int* ids, int capacity);
/* Tokenizer::decode / decode_token (tokenizer.h:26-29, src/tokenizer.cpp:359-374): special tokens and ids outside
 * the vocabulary are skipped.  Writes at most capacity - 1 bytes and a terminating zero; returns the byte length
 * of the whole text, or a negative status. */
int spb_tokenizer_decode(const spb_tokenizer* t, const int* ids, int n, char* out, size_t capacity);

/* ---- row-sharded engine: one rank of a tensor-parallel group, one process per GPU ----------------------
 * No counterpart in the reference (it is single-GPU).  The decode step of InferenceEngine::forward
 * (src/inference.cu:123-283) with every matrix split by output rows over `world` ranks and no reduction anywhere,
 * so every rank's integer accumulators, half outputs and logits are bit-identical to the same step on one rank:
 * q/k/v by whole KV heads (RoPE, KV cache and attention stay local), o / gate / up / down by rows, the LM head by
 * vocabulary rows; norms, quantisation and residual adds replicated.  The slices meet through an exchange kernel
 * that stores them into every rank's exchange buffer over NVLink (peer mappings of one CUDA IPC allocation per
 * rank) and waits, bounded by time, for the peers' sequence-numbered flags: 4 exchanges per layer + 1 per token.
 * batch > 1 decodes that many independent sequences in lock step with the batched product.
 * Set-up per rank: create (current device) -> row_range / set_linear (the rank's row slices) / set_norm /
 * set_globals -> ipc_handle, all-gather the 64-byte handles by any host channel, set_peers -> a host barrier ->
 * generate / step (every rank calls with the same arguments).  A rank whose wait for a peer runs out reports
 * SPB_E_TIMEOUT at its next synchronisation and skips all later waits; the engine must then be recreated. */
typedef struct spb_shard_engine spb_shard_engine;
/* world 1..8 (at most num_key_value_heads), batch 1..64; hidden_size, intermediate_size and head_dim multiples of 8. */
spb_shard_engine* spb_shard_engine_create(const spb_model_config* cfg, int rank, int world, int batch);
void spb_shard_engine_destroy(spb_shard_engine* e);
/* Rows [start, stop) of the full matrix that this rank owns.  which: 0 q, 1 k, 2 v, 3 o, 4 gate, 5 up, 6 down,
 * 7 LM head (vocabulary rows). */
int spb_shard_engine_row_range(const spb_shard_engine* e, int which, int* start, int* stop);
/* The rank's row slice of a matrix (SparseLinear, include/spbitnet/model.h:46-60): rows = stop - start. */
int spb_shard_engine_set_linear(spb_shard_engine* e, int layer, int which, const uint32_t* d_meta, const uint32_t* d_values,
                                float gamma, int rows, int cols, int meta_stride, int values_stride);
/* Full norm vectors (replicated).  which as spb_engine_set_norm. */
int spb_shard_engine_set_norm(spb_shard_engine* e, int layer, int which, const float* d_weight);
/* d_embed: the full embedding table; d_lm_head_rows: this rank's vocabulary rows of the LM head (of the embedding
 * table when tied); d_final_norm: full. */
int spb_shard_engine_set_globals(spb_shard_engine* e, const void* d_embed, const void* d_lm_head_rows, const float* d_final_norm);
/* 64-byte CUDA IPC handle of this rank's exchange buffer (HOST pointer). */
int spb_shard_engine_ipc_handle(spb_shard_engine* e, void* handle_out);
/* handles: world x 64 bytes in rank order (HOST); the entry of this rank is ignored. */
int spb_shard_engine_set_peers(spb_shard_engine* e, const void* handles);
/* The same for buffers this GPU can already address (ranks in one process with peer access enabled): world device
 * pointers to buffers of spb_shard_engine_exchange_bytes bytes, zero-filled; the entry of this rank is ignored. */
int spb_shard_engine_set_peer_pointers(spb_shard_engine* e, void* const* buffers);
size_t spb_shard_engine_exchange_bytes(const spb_shard_engine* e);
/* Bound of every wait for a peer (default 5000 ms). */
int spb_shard_engine_set_timeout_ms(spb_shard_engine* e, int ms);
/* Whether the engine keeps a prepared copy (spb_prepare_weights) of the slices set with spb_shard_engine_set_linear
 * and multiplies on it: 1 (default) for slices of 4 M weights and more (k and v go with q), 2 for every slice the layout takes, 0 for
 * none.  It applies to the single-sequence step of wide models (hidden size >= 4096), which multiplies matrix by
 * matrix on the quantised vector; elsewhere the setting has no effect.  The copies are the engine's (as large as
 * the slices); results are the same bit for bit.  May be called before or after the slices are set. */
int spb_shard_engine_set_prepared_weights(spb_shard_engine* e, int on);
/* How the single-sequence step of a wide model exchanges slices between the ranks:
 *   2 (default) the kernel that computes a slice (attention merge, prepared GEMV) stores it from its epilogue, as
 *     {two halves, sequence number} words, straight into every rank's staging area over NVLink, and the kernel that
 *     consumes the gathered vector polls its local staging area: no exchange launch and no gathered copy (a slice
 *     whose matrix has no prepared copy falls back to form 0);
 *   1 the consuming kernel (one block) sends this rank's slice and collects the peers' itself;
 *   0 a launch of its own does both (the form every other step uses).
 * Same results bit for bit; the waits are bounded the same way in every form. */
int spb_shard_engine_set_exchange_fold(spb_shard_engine* e, int form);
int spb_shard_engine_reset(spb_shard_engine* e);
int spb_shard_engine_seq_len(const spb_shard_engine* e);
/* One decode step: tokens[batch] (HOST) enter at the current position; synchronises.  Afterwards the rank's logits
 * rows are available through spb_shard_engine_copy_logits. */
int spb_shard_engine_step(spb_shard_engine* e, const int* tokens);
/* h_logits_rows: batch x (stop - start of which = 7) floats (HOST): this rank's vocabulary rows of the last step. */
int spb_shard_engine_copy_logits(spb_shard_engine* e, float* h_logits_rows);
/* The greedy loop of src/main.cpp:266-300 for `batch` sequences: prompt is n_prompt x batch token ids (HOST,
 * position-major), out_tokens max_tokens x batch.  Feeds prompt[0 .. n_prompt-2], then generates max_tokens tokens
 * from prompt[n_prompt-1]; no EOS stop.  Returns max_tokens or a negative status. */
int spb_shard_engine_generate(spb_shard_engine* e, const int* prompt, int n_prompt, int max_tokens, int* out_tokens);

#ifdef __cplusplus
}
#endif
#endif /* SPBITNET_B200_H */
