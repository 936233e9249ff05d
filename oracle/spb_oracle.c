/*
 * spb_oracle.c -- CPU restatement of the spbitnet sparse-ternary hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the parity tests,
 * the smoke test and the bench's cpu_baseline leg compare the CUDA kernels
 * against.  Nothing in the shipped library links, loads or calls it.
 *
 * Every function restates, in plain scalar C, the behaviour of one piece of
 * the reference (paths are relative to the reference project root) and names
 * the lines it follows.  It is pinned against the reference's own header
 * (compiled unchanged into oracle/_ref by oracle/Makefile), its Python
 * packers and its known-answer tests; see tests/test_oracle_*.py.
 *
 * Numerics: all floating point is IEEE binary32 evaluated in the order the
 * reference source writes it, built with -ffp-contract=off.  __float2int_rn
 * is nearbyintf under the default rounding mode (ties to even); __float2half
 * is the round-to-nearest-even conversion of _Float16.  Reductions follow the
 * reference kernels' 256-thread strided partials and shuffle trees so that
 * the sums are the ones the reference GPU code forms, up to its FMA
 * contraction.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 half_t;

static inline float h2f(uint16_t h) {
    half_t v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t f2h(float f) {
    half_t v = (half_t)f; /* round to nearest even, like __float2half */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

/* ------------------------------------------------------------------------
 * Format.  include/spbitnet/sparse_ternary_tensor.h:36-39 (constants),
 * :254-264 (row strides).
 * ---------------------------------------------------------------------- */
int spbo_meta_words_per_row(int cols) { return (cols / 4 + 7) / 8; }
int spbo_values_words_per_row(int cols) { return (cols / 4 + 15) / 16; }

/* include/spbitnet/sparse_ternary_tensor.h:58-108 (pack_from_dense).
 * meta/values must be zero-filled by the caller (the reference constructor
 * zero-fills, :45-46).  Returns 0, or -(1+group index) for the first group
 * whose mask does not keep exactly two entries (the reference asserts). */
long spbo_pack_from_dense(const int8_t* w, const uint8_t* mask, int rows,
                          int cols, uint32_t* meta, uint32_t* values) {
    const int gpr = cols / 4;
    const size_t ms = (size_t)spbo_meta_words_per_row(cols);
    const size_t vs = (size_t)spbo_values_words_per_row(cols);
    for (int r = 0; r < rows; ++r) {
        for (int g = 0; g < gpr; ++g) {
            const size_t base = (size_t)r * cols + (size_t)g * 4;
            int cnt = 0;
            for (int i = 0; i < 4; ++i) cnt += mask[base + i] ? 1 : 0;
            if (cnt != 2) return -(1 + (long)r * gpr + g);
            uint32_t bitmap = 0, signs = 0;
            int nz = 0;
            for (int i = 0; i < 4; ++i) {
                if (mask[base + i]) {
                    bitmap |= 1u << i;
                    /* a kept zero packs as +1 (:86-91) */
                    signs |= (uint32_t)(w[base + i] < 0 ? 1u : 0u) << nz;
                    ++nz;
                }
            }
            meta[r * ms + g / 8] |= bitmap << ((g % 8) * 4);
            values[r * vs + g / 16] |= signs << ((g % 16) * 2);
        }
    }
    return 0;
}

/* include/spbitnet/sparse_ternary_tensor.h:123-191 (pack_with_pruning):
 * keep the two largest |latent| per group, lower index wins ties (stable
 * sort, :141-145), sign bit set only when latent < -0.5 (:166-169). */
void spbo_pack_with_pruning(const float* latent, int rows, int cols,
                            uint32_t* meta, uint32_t* values) {
    const int gpr = cols / 4;
    const size_t ms = (size_t)spbo_meta_words_per_row(cols);
    const size_t vs = (size_t)spbo_values_words_per_row(cols);
    for (int r = 0; r < rows; ++r) {
        for (int g = 0; g < gpr; ++g) {
            const size_t base = (size_t)r * cols + (size_t)g * 4;
            int idx[4] = {0, 1, 2, 3};
            /* stable insertion sort, descending |latent| */
            for (int i = 1; i < 4; ++i) {
                int k = idx[i], j = i - 1;
                while (j >= 0 && fabsf(latent[base + k]) > fabsf(latent[base + idx[j]])) {
                    idx[j + 1] = idx[j];
                    --j;
                }
                idx[j + 1] = k;
            }
            uint8_t keep[4] = {0, 0, 0, 0};
            keep[idx[0]] = 1;
            keep[idx[1]] = 1;
            uint32_t bitmap = 0, signs = 0;
            int nz = 0;
            for (int i = 0; i < 4; ++i) {
                if (keep[i]) {
                    bitmap |= 1u << i;
                    signs |= (uint32_t)(latent[base + i] < -0.5f ? 1u : 0u) << nz;
                    ++nz;
                }
            }
            meta[r * ms + g / 8] |= bitmap << ((g % 8) * 4);
            values[r * vs + g / 16] |= signs << ((g % 16) * 2);
        }
    }
}

/* include/spbitnet/sparse_ternary_tensor.h:197-232 (unpack_to_int8), with the
 * row strides as parameters so padded layouts can be checked too.  A bitmap
 * with other than two bits set yields as many non-zeros as it has bits, the
 * sign pair consumed LSB first (:219-229). */
void spbo_unpack_to_int8(const uint32_t* meta, const uint32_t* values, int rows,
                         int cols, int meta_stride, int values_stride,
                         int8_t* out) {
    const int gpr = cols / 4;
    memset(out, 0, (size_t)rows * cols);
    for (int r = 0; r < rows; ++r) {
        for (int g = 0; g < gpr; ++g) {
            const size_t base = (size_t)r * cols + (size_t)g * 4;
            uint32_t bitmap = (meta[(size_t)r * meta_stride + g / 8] >> ((g % 8) * 4)) & 0xF;
            uint32_t signs = (values[(size_t)r * values_stride + g / 16] >> ((g % 16) * 2)) & 0x3;
            int nz = 0;
            for (int i = 0; i < 4; ++i) {
                if (bitmap & (1u << i)) {
                    out[base + i] = ((signs >> nz) & 1u) ? (int8_t)-1 : (int8_t)1;
                    ++nz;
                }
            }
        }
    }
}

/* 0 when every bitmap nibble of every visited group has exactly two bits
 * set, else -(1+flat group index) of the first that does not.  The reference
 * leaves other bitmaps undefined: its GPU LUT maps them to (0,0)
 * (src/kernels/sparse_ternary.cu:34-51) while its CPU unpack does what the
 * function above does. */
long spbo_validate(const uint32_t* meta, int rows, int cols, int meta_stride) {
    const int gpr = cols / 4;
    for (int r = 0; r < rows; ++r)
        for (int g = 0; g < gpr; ++g) {
            uint32_t b = (meta[(size_t)r * meta_stride + g / 8] >> ((g % 8) * 4)) & 0xF;
            if (__builtin_popcount(b) != 2) return -(1 + (long)r * gpr + g);
        }
    return 0;
}

/* ------------------------------------------------------------------------
 * Integer kernels.
 * ---------------------------------------------------------------------- */

/* tests/test_sparse_ternary.cu:17-33 (cpu_sparse_gemv): unpack to dense int8,
 * then a row-major int32 dot product.  Unpacks one row at a time; the values
 * formed are the same. */
void spbo_sparse_gemv(const uint32_t* meta, const uint32_t* values,
                      const int8_t* x, int32_t* y, int rows, int cols,
                      int meta_stride, int values_stride) {
    int8_t* dense = (int8_t*)malloc((size_t)cols);
    for (int r = 0; r < rows; ++r) {
        spbo_unpack_to_int8(meta + (size_t)r * meta_stride,
                            values + (size_t)r * values_stride, 1, cols,
                            meta_stride, values_stride, dense);
        int32_t sum = 0;
        for (int c = 0; c < cols; ++c) sum += (int32_t)dense[c] * (int32_t)x[c];
        y[r] = sum;
    }
    free(dense);
}

/* tests/test_cusparselt.cu:16-28 (cpu_int8_gemm): D[m,n] = A[m,k] * B[k,n],
 * all row-major. */
void spbo_int8_gemm(const int8_t* A, const int8_t* B, int32_t* D, int m, int k,
                    int n) {
    for (int r = 0; r < m; ++r)
        for (int c = 0; c < n; ++c) {
            int32_t sum = 0;
            for (int j = 0; j < k; ++j)
                sum += (int32_t)A[(size_t)r * k + j] * (int32_t)B[(size_t)j * n + c];
            D[(size_t)r * n + c] = sum;
        }
}

/* Batched form in the layout CuSparseLtGemm::execute takes
 * (include/spbitnet/cusparselt_backend.h:47-50): X is [k,n] column-major with
 * ld=k, i.e. n activation rows of k int8; Y is [m,n] column-major with ld=m,
 * i.e. n output rows of m int32.  Y[j][r] = sum_c W[r][c] * X[j][c]. */
void spbo_sparse_gemm(const uint32_t* meta, const uint32_t* values,
                      const int8_t* X, int32_t* Y, int rows, int cols, int n,
                      int meta_stride, int values_stride) {
    int8_t* dense = (int8_t*)malloc((size_t)cols);
    for (int r = 0; r < rows; ++r) {
        spbo_unpack_to_int8(meta + (size_t)r * meta_stride,
                            values + (size_t)r * values_stride, 1, cols,
                            meta_stride, values_stride, dense);
        for (int j = 0; j < n; ++j) {
            const int8_t* xr = X + (size_t)j * cols;
            int32_t sum = 0;
            for (int c = 0; c < cols; ++c) sum += (int32_t)dense[c] * (int32_t)xr[c];
            Y[(size_t)j * rows + r] = sum;
        }
    }
    free(dense);
}

/* ------------------------------------------------------------------------
 * Reduction helpers that follow the reference kernels' order: 256 threads
 * take strided partials, each warp folds with __shfl_down_sync (offsets
 * 16..1), then warp 0 folds the 8 warp results the same way.
 * ---------------------------------------------------------------------- */
static float tree256_sum(float* part /* 256 */) {
    float warp[32];
    for (int w = 0; w < 8; ++w) {
        float v[32];
        memcpy(v, part + 32 * w, sizeof v);
        for (int off = 16; off > 0; off >>= 1)
            for (int l = 0; l < 32; ++l)
                v[l] = v[l] + ((l + off < 32) ? v[l + off] : v[l]);
        /* lanes whose partner is out of range read their own value in
         * hardware; lane 0 never depends on them */
        warp[w] = v[0];
    }
    for (int l = 8; l < 32; ++l) warp[l] = 0.0f;
    for (int off = 16; off > 0; off >>= 1)
        for (int l = 0; l < 32; ++l)
            warp[l] = warp[l] + ((l + off < 32) ? warp[l + off] : warp[l]);
    return warp[0];
}

/* ------------------------------------------------------------------------
 * Activation quantisation.
 * ---------------------------------------------------------------------- */

/* src/kernels/inference_kernels.cu:120-148 (absmax_reduce_kernel).  A max is
 * order independent, so a plain loop gives the same value. */
float spbo_absmax_reduce(const uint16_t* x, int n) {
    float m = 0.0f;
    for (int i = 0; i < n; ++i) m = fmaxf(m, fabsf(h2f(x[i])));
    return m;
}

/* src/kernels/inference_kernels.cu:69-114 (absmax_quantize_kernel):
 * scale = 127/absmax in fp32 (0 when absmax is 0, :103), q = clamp(rn(x*scale)). */
float spbo_absmax_quantize(const uint16_t* x, int8_t* q, int n) {
    const float absmax = spbo_absmax_reduce(x, n);
    const float scale = (absmax > 0.0f) ? 127.0f / absmax : 0.0f;
    for (int i = 0; i < n; ++i) {
        float v = h2f(x[i]) * scale;
        int qi = (int)nearbyintf(v);
        if (qi > 127) qi = 127;
        if (qi < -128) qi = -128;
        q[i] = (int8_t)qi;
    }
    return absmax;
}

/* src/kernels/inference_kernels.cu:162-171 (dequantize_kernel):
 * scale = gamma * absmax / 127.0f left to right, out = half(float(acc)*scale). */
void spbo_dequantize(const int32_t* acc, uint16_t* out, float absmax,
                     float gamma, int n) {
    const float scale = gamma * absmax / 127.0f;
    for (int i = 0; i < n; ++i) out[i] = f2h((float)acc[i] * scale);
}

/* The fp32 value before the half rounding, for the 1-ulp check of the
 * scaled output. */
void spbo_dequantize_f32(const int32_t* acc, float* out, float absmax,
                         float gamma, int n) {
    const float scale = gamma * absmax / 127.0f;
    for (int i = 0; i < n; ++i) out[i] = (float)acc[i] * scale;
}

/* src/kernels/sparse_ternary.cu:181-234 (fused_sparse_bitlinear_kernel):
 * inline quantisation with the same rule as absmax_quantize (:198-217), the
 * integer walk, then half(float(acc) * (gamma*absmax/127)) (:231-232). */
void spbo_fused_bitlinear(const uint32_t* meta, const uint32_t* values,
                          const uint16_t* x, uint16_t* out, float absmax,
                          float gamma, int rows, int cols, int meta_stride,
                          int values_stride) {
    int8_t* q = (int8_t*)malloc((size_t)cols);
    int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)rows);
    const float scale = (absmax > 0.0f) ? 127.0f / absmax : 0.0f;
    for (int i = 0; i < cols; ++i) {
        int qi = (int)nearbyintf(h2f(x[i]) * scale);
        if (qi > 127) qi = 127;
        if (qi < -128) qi = -128;
        q[i] = (int8_t)qi;
    }
    spbo_sparse_gemv(meta, values, q, acc, rows, cols, meta_stride, values_stride);
    spbo_dequantize(acc, out, absmax, gamma, rows);
    free(q);
    free(acc);
}

/* ------------------------------------------------------------------------
 * The rest of a decode step.
 * ---------------------------------------------------------------------- */

/* src/kernels/inference_kernels.cu:15-56 (rms_norm_kernel): in-place safe. */
void spbo_rms_norm(const uint16_t* x, const float* w, uint16_t* out, int n,
                   float eps) {
    float part[256];
    for (int t = 0; t < 256; ++t) {
        float s = 0.0f;
        for (int i = t; i < n; i += 256) {
            float v = h2f(x[i]);
            s += v * v;
        }
        part[t] = s;
    }
    const float sum = tree256_sum(part);
    const float scale = 1.0f / sqrtf(sum / (float)n + eps);
    for (int i = 0; i < n; ++i) out[i] = f2h(h2f(x[i]) * scale * w[i]);
}

/* src/kernels/inference_kernels.cu:418-455 (rms_norm_f32in_kernel). */
void spbo_rms_norm_f32in(const float* x, const float* w, uint16_t* out, int n,
                         float eps) {
    float part[256];
    for (int t = 0; t < 256; ++t) {
        float s = 0.0f;
        for (int i = t; i < n; i += 256) s += x[i] * x[i];
        part[t] = s;
    }
    const float sum = tree256_sum(part);
    const float scale = 1.0f / sqrtf(sum / (float)n + eps);
    for (int i = 0; i < n; ++i) out[i] = f2h(x[i] * scale * w[i]);
}

/* src/kernels/inference_kernels.cu:185-206 (rope_kernel): adjacent pairs
 * (2i, 2i+1), fp32 powf/cosf/sinf, in place. */
void spbo_rope(uint16_t* vec, int num_heads, int head_dim, int pos, float theta) {
    const int hp = head_dim / 2;
    for (int h = 0; h < num_heads; ++h)
        for (int p = 0; p < hp; ++p) {
            float freq = 1.0f / powf(theta, (float)(2 * p) / (float)head_dim);
            float angle = (float)pos * freq;
            float c = cosf(angle), s = sinf(angle);
            int idx = h * head_dim + 2 * p;
            float x0 = h2f(vec[idx]), x1 = h2f(vec[idx + 1]);
            vec[idx] = f2h(x0 * c - x1 * s);
            vec[idx + 1] = f2h(x0 * s + x1 * c);
        }
}

/* src/kernels/inference_kernels.cu:215-227 (scatter_kv_kernel). */
void spbo_scatter_kv(const uint16_t* src, uint16_t* cache, int num_kv_heads,
                     int head_dim, int max_seq_len, int pos) {
    for (int h = 0; h < num_kv_heads; ++h)
        memcpy(cache + ((size_t)h * max_seq_len + pos) * head_dim,
               src + (size_t)h * head_dim, sizeof(uint16_t) * (size_t)head_dim);
}

/* src/kernels/inference_kernels.cu:241-275 (attention_scores_kernel): a warp
 * per (head, position); lane strides the head dimension, shuffle-down fold. */
void spbo_attention_scores(const uint16_t* Q, const uint16_t* K, float* scores,
                           int num_heads, int num_kv_heads, int head_dim,
                           int max_seq_len, int seq_len, float scale) {
    for (int h = 0; h < num_heads; ++h) {
        const int kv = h * num_kv_heads / num_heads;
        for (int j = 0; j < seq_len; ++j) {
            const uint16_t* q = Q + (size_t)h * head_dim;
            const uint16_t* k = K + ((size_t)kv * max_seq_len + j) * head_dim;
            float v[32];
            for (int l = 0; l < 32; ++l) {
                float a = 0.0f;
                for (int d = l; d < head_dim; d += 32) a += h2f(q[d]) * h2f(k[d]);
                v[l] = a;
            }
            for (int off = 16; off > 0; off >>= 1)
                for (int l = 0; l < 32; ++l)
                    v[l] = v[l] + ((l + off < 32) ? v[l + off] : v[l]);
            scores[(size_t)h * max_seq_len + j] = v[0] * scale;
        }
    }
}

/* src/kernels/inference_kernels.cu:283-339 (softmax_kernel): max, then
 * exp(x-max) and its sum, then multiply by 1/sum; first seq_len entries. */
void spbo_softmax(float* scores, int num_heads, int max_seq_len, int seq_len) {
    for (int h = 0; h < num_heads; ++h) {
        float* hs = scores + (size_t)h * max_seq_len;
        float mx = -1e30f;
        for (int j = 0; j < seq_len; ++j) mx = fmaxf(mx, hs[j]);
        float part[256];
        for (int t = 0; t < 256; ++t) {
            float s = 0.0f;
            for (int j = t; j < seq_len; j += 256) {
                float e = expf(hs[j] - mx);
                hs[j] = e;
                s += e;
            }
            part[t] = s;
        }
        const float inv = 1.0f / tree256_sum(part);
        for (int j = 0; j < seq_len; ++j) hs[j] *= inv;
    }
}

/* src/kernels/inference_kernels.cu:350-371 (attention_output_kernel): one
 * thread per output dim, serial over positions. */
void spbo_attention_output(const float* scores, const uint16_t* V, uint16_t* out,
                           int num_heads, int num_kv_heads, int head_dim,
                           int max_seq_len, int seq_len) {
    for (int h = 0; h < num_heads; ++h) {
        const int kv = h * num_kv_heads / num_heads;
        const float* hs = scores + (size_t)h * max_seq_len;
        const uint16_t* v = V + (size_t)kv * max_seq_len * head_dim;
        for (int d = 0; d < head_dim; ++d) {
            float acc = 0.0f;
            for (int j = 0; j < seq_len; ++j)
                acc += hs[j] * h2f(v[(size_t)j * head_dim + d]);
            out[(size_t)h * head_dim + d] = f2h(acc);
        }
    }
}

/* src/kernels/inference_kernels.cu:379-390 (relu2_mul_kernel). */
void spbo_relu2_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out, int n) {
    for (int i = 0; i < n; ++i) {
        float r = fmaxf(0.0f, h2f(gate[i]));
        out[i] = f2h(r * r * h2f(up[i]));
    }
}

/* src/kernels/inference_kernels.cu:399-410 (relu2_mul_f32_kernel). */
void spbo_relu2_mul_f32(const uint16_t* gate, const uint16_t* up, float* out, int n) {
    for (int i = 0; i < n; ++i) {
        float r = fmaxf(0.0f, h2f(gate[i]));
        out[i] = r * r * h2f(up[i]);
    }
}

/* src/kernels/inference_kernels.cu:460-466 (float_to_half_kernel). */
void spbo_float_to_half(const float* in, uint16_t* out, int n) {
    for (int i = 0; i < n; ++i) out[i] = f2h(in[i]);
}

/* src/kernels/inference_kernels.cu:471-479 (residual_add_kernel). */
void spbo_residual_add(const uint16_t* a, const uint16_t* b, uint16_t* out, int n) {
    for (int i = 0; i < n; ++i) out[i] = f2h(h2f(a[i]) + h2f(b[i]));
}

/* src/kernels/inference_kernels.cu:488-531 (half_gemv_kernel): warp per row,
 * each lane takes 8-wide chunks strided by 32 chunks, then a scalar tail,
 * then the shuffle-down fold. */
void spbo_half_gemv(const uint16_t* W, const uint16_t* x, float* y, int rows,
                    int cols) {
    const int cols_v = cols >> 3;
    for (int r = 0; r < rows; ++r) {
        const uint16_t* row = W + (size_t)r * cols;
        float v[32];
        for (int l = 0; l < 32; ++l) {
            float a = 0.0f;
            for (int j = l; j < cols_v; j += 32)
                for (int k = 0; k < 8; ++k) a += h2f(row[j * 8 + k]) * h2f(x[j * 8 + k]);
            for (int j = (cols_v << 3) + l; j < cols; j += 32) a += h2f(row[j]) * h2f(x[j]);
            v[l] = a;
        }
        for (int off = 16; off > 0; off >>= 1)
            for (int l = 0; l < 32; ++l)
                v[l] = v[l] + ((l + off < 32) ? v[l + off] : v[l]);
        y[r] = v[0];
    }
}

/* ------------------------------------------------------------------------
 * Engine: src/inference.cu:16-69 (buffers), :91-100 (reset), :106-117
 * (bitlinear = absmax_reduce then the fused kernel), :123-283 (forward).
 * Weights are borrowed pointers set by the caller.
 * ---------------------------------------------------------------------- */
typedef struct {
    const uint32_t* meta;
    const uint32_t* values;
    float gamma;
    int rows, cols, meta_stride, values_stride;
} spbo_linear;

typedef struct {
    spbo_linear q, k, v, o, gate, up, down;
    const float* input_ln;
    const float* post_attn_ln;
    const float* attn_sub_norm; /* may be NULL */
    const float* ffn_sub_norm;  /* may be NULL */
} spbo_layer;

typedef struct {
    int hidden, layers, heads, kv_heads, head_dim, inter, vocab, max_seq;
    float eps, theta;
    spbo_layer* layer;
    const uint16_t* embed;   /* (vocab, hidden) half */
    const uint16_t* lm_head; /* (vocab, hidden) half; == embed when tied */
    const float* final_norm;
    uint16_t **kc, **vc;
    uint16_t *x, *res, *q, *kv, *gate, *up;
    float *mlp, *scores, *logits;
    int seq_len;
} spbo_engine;

spbo_engine* spbo_engine_create(int hidden, int layers, int heads, int kv_heads,
                                int head_dim, int inter, int vocab, int max_seq,
                                float eps, float theta) {
    spbo_engine* e = (spbo_engine*)calloc(1, sizeof *e);
    e->hidden = hidden; e->layers = layers; e->heads = heads; e->kv_heads = kv_heads;
    e->head_dim = head_dim; e->inter = inter; e->vocab = vocab; e->max_seq = max_seq;
    e->eps = eps; e->theta = theta;
    e->layer = (spbo_layer*)calloc((size_t)layers, sizeof(spbo_layer));
    e->kc = (uint16_t**)calloc((size_t)layers, sizeof(uint16_t*));
    e->vc = (uint16_t**)calloc((size_t)layers, sizeof(uint16_t*));
    const size_t kvn = (size_t)kv_heads * max_seq * head_dim;
    for (int l = 0; l < layers; ++l) {
        e->kc[l] = (uint16_t*)calloc(kvn, 2);
        e->vc[l] = (uint16_t*)calloc(kvn, 2);
    }
    const int qdim = heads * head_dim > hidden ? heads * head_dim : hidden;
    e->x = (uint16_t*)calloc((size_t)qdim, 2);
    e->res = (uint16_t*)calloc((size_t)hidden, 2);
    e->q = (uint16_t*)calloc((size_t)qdim, 2);
    e->kv = (uint16_t*)calloc((size_t)kv_heads * head_dim, 2);
    e->gate = (uint16_t*)calloc((size_t)inter, 2);
    e->up = (uint16_t*)calloc((size_t)inter, 2);
    e->mlp = (float*)calloc((size_t)inter, 4);
    e->scores = (float*)calloc((size_t)heads * max_seq, 4);
    e->logits = (float*)calloc((size_t)vocab, 4);
    return e;
}

void spbo_engine_destroy(spbo_engine* e) {
    if (!e) return;
    for (int l = 0; l < e->layers; ++l) { free(e->kc[l]); free(e->vc[l]); }
    free(e->kc); free(e->vc); free(e->layer);
    free(e->x); free(e->res); free(e->q); free(e->kv); free(e->gate); free(e->up);
    free(e->mlp); free(e->scores); free(e->logits);
    free(e);
}

/* which: 0 q, 1 k, 2 v, 3 o, 4 gate, 5 up, 6 down */
void spbo_engine_set_linear(spbo_engine* e, int layer, int which,
                            const uint32_t* meta, const uint32_t* values,
                            float gamma, int rows, int cols, int meta_stride,
                            int values_stride) {
    spbo_linear* L = &e->layer[layer].q + which;
    L->meta = meta; L->values = values; L->gamma = gamma; L->rows = rows;
    L->cols = cols; L->meta_stride = meta_stride; L->values_stride = values_stride;
}

/* which: 0 input_ln, 1 post_attn_ln, 2 attn_sub_norm, 3 ffn_sub_norm */
void spbo_engine_set_norm(spbo_engine* e, int layer, int which, const float* w) {
    spbo_layer* L = &e->layer[layer];
    if (which == 0) L->input_ln = w;
    else if (which == 1) L->post_attn_ln = w;
    else if (which == 2) L->attn_sub_norm = w;
    else L->ffn_sub_norm = w;
}

void spbo_engine_set_globals(spbo_engine* e, const uint16_t* embed,
                             const uint16_t* lm_head, const float* final_norm) {
    e->embed = embed;
    e->lm_head = lm_head ? lm_head : embed;
    e->final_norm = final_norm;
}

void spbo_engine_reset(spbo_engine* e) {
    e->seq_len = 0;
    const size_t kvn = (size_t)e->kv_heads * e->max_seq * e->head_dim;
    for (int l = 0; l < e->layers; ++l) {
        memset(e->kc[l], 0, kvn * 2);
        memset(e->vc[l], 0, kvn * 2);
    }
}

int spbo_engine_seq_len(const spbo_engine* e) { return e->seq_len; }

static void bitlinear(const uint16_t* in, int n, const spbo_linear* L, uint16_t* out) {
    const float absmax = spbo_absmax_reduce(in, n); /* src/inference.cu:110 */
    spbo_fused_bitlinear(L->meta, L->values, in, out, absmax, L->gamma, L->rows,
                         L->cols, L->meta_stride, L->values_stride);
}

/* src/inference.cu:123-283.  Returns the engine's logits buffer. */
const float* spbo_engine_forward(spbo_engine* e, int token) {
    const int pos = e->seq_len, H = e->hidden, hd = e->head_dim;
    const int seq_len = pos + 1;
    memcpy(e->x, e->embed + (size_t)token * H, (size_t)H * 2);
    for (int l = 0; l < e->layers; ++l) {
        const spbo_layer* L = &e->layer[l];
        memcpy(e->res, e->x, (size_t)H * 2);
        spbo_rms_norm(e->res, L->input_ln, e->x, H, e->eps);
        bitlinear(e->x, H, &L->q, e->q);
        bitlinear(e->x, H, &L->k, e->kv);
        spbo_rope(e->q, e->heads, hd, pos, e->theta);
        spbo_rope(e->kv, e->kv_heads, hd, pos, e->theta);
        spbo_scatter_kv(e->kv, e->kc[l], e->kv_heads, hd, e->max_seq, pos);
        bitlinear(e->x, H, &L->v, e->kv);
        spbo_scatter_kv(e->kv, e->vc[l], e->kv_heads, hd, e->max_seq, pos);
        const float attn_scale = 1.0f / sqrtf((float)hd);
        spbo_attention_scores(e->q, e->kc[l], e->scores, e->heads, e->kv_heads, hd,
                              e->max_seq, seq_len, attn_scale);
        spbo_softmax(e->scores, e->heads, e->max_seq, seq_len);
        spbo_attention_output(e->scores, e->vc[l], e->x, e->heads, e->kv_heads, hd,
                              e->max_seq, seq_len);
        bitlinear(e->x, L->o.cols, &L->o, e->q);
        if (L->attn_sub_norm) spbo_rms_norm(e->q, L->attn_sub_norm, e->q, H, e->eps);
        spbo_residual_add(e->q, e->res, e->x, H);
        memcpy(e->res, e->x, (size_t)H * 2);
        spbo_rms_norm(e->res, L->post_attn_ln, e->x, H, e->eps);
        bitlinear(e->x, H, &L->gate, e->gate);
        bitlinear(e->x, H, &L->up, e->up);
        spbo_relu2_mul_f32(e->gate, e->up, e->mlp, e->inter);
        if (L->ffn_sub_norm)
            spbo_rms_norm_f32in(e->mlp, L->ffn_sub_norm, e->gate, e->inter, e->eps);
        else
            spbo_float_to_half(e->mlp, e->gate, e->inter);
        bitlinear(e->gate, e->inter, &L->down, e->q);
        spbo_residual_add(e->q, e->res, e->x, H);
    }
    spbo_rms_norm(e->x, e->final_norm, e->res, H, e->eps);
    spbo_half_gemv(e->lm_head, e->res, e->logits, e->vocab, H);
    e->seq_len++;
    return e->logits;
}

/* src/main.cpp:285-287: std::max_element, the first maximum wins. */
int spbo_argmax(const float* v, int n) {
    int best = 0;
    for (int i = 1; i < n; ++i)
        if (v[i] > v[best]) best = i;
    return best;
}

/* ------------------------------------------------------------------------
 * Threaded GEMV for the timed CPU baseline: the same scalar row loop, rows
 * split into contiguous slices, one per thread.  No algorithmic change.
 * ---------------------------------------------------------------------- */
#include <pthread.h>
typedef struct {
    const uint32_t *meta, *values;
    const int8_t* x;
    int32_t* y;
    int r0, r1, cols, ms, vs;
} gemv_job;

static void* gemv_worker(void* p) {
    gemv_job* j = (gemv_job*)p;
    spbo_sparse_gemv(j->meta + (size_t)j->r0 * j->ms, j->values + (size_t)j->r0 * j->vs,
                     j->x, j->y + j->r0, j->r1 - j->r0, j->cols, j->ms, j->vs);
    return NULL;
}

void spbo_sparse_gemv_mt(const uint32_t* meta, const uint32_t* values,
                         const int8_t* x, int32_t* y, int rows, int cols,
                         int meta_stride, int values_stride, int threads) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    pthread_t tid[256];
    gemv_job job[256];
    for (int t = 0; t < threads; ++t) {
        job[t] = (gemv_job){meta, values, x, y,
                            (int)((long)rows * t / threads),
                            (int)((long)rows * (t + 1) / threads),
                            cols, meta_stride, values_stride};
        pthread_create(&tid[t], NULL, gemv_worker, &job[t]);
    }
    for (int t = 0; t < threads; ++t) pthread_join(tid[t], NULL);
}
