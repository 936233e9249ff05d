// The non-GEMV kernels of a decode step, behind the reference's host-wrapper API
// (include/spbitnet/inference_kernels.h; src/kernels/inference_kernels.cu).
// All arithmetic is fp32 in the reference's operation order; storage types and
// rounding points (half after norm / rope / residual / attention output, fp32 for
// scores, relu2*up and logits) are the reference's.
#include "spb_common.cuh"

namespace spb {

constexpr int kBlock = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    return v;
}
// Block-wide reductions for blockDim.x <= 1024; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* sh /* 32 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? sh[lane] : 0.0f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* sh /* 32 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? sh[lane] : -INFINITY;
    return warp_max(t);
}

// ---- rms_norm_gpu / rms_norm_f32in_gpu (inference_kernels.cu:15-56, 418-455) ----------
template <typename TIn>
__global__ void __launch_bounds__(1024) rms_norm_kernel(const TIn* __restrict__ in,
                                                        const float* __restrict__ w,
                                                        __half* __restrict__ out, int n, float eps) {
    __shared__ float sh[32];
    grid_dep_launch();
    grid_dep_wait();
    float s = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = static_cast<float>(in[i]);
        s += v * v;
    }
    const float total = block_sum(s, sh);
    const float scale = rsqrtf(total / static_cast<float>(n) + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = static_cast<float>(in[i]);
        out[i] = __float2half_rn(__fmul_rn(__fmul_rn(v, scale), w[i]));
    }
}

// ---- absmax_reduce_gpu / absmax_quantize_gpu (inference_kernels.cu:69-148) -------------
template <bool QUANT>
__global__ void __launch_bounds__(1024) absmax_kernel(const __half* __restrict__ in,
                                                      int8_t* __restrict__ q,
                                                      float* __restrict__ d_absmax, int n) {
    __shared__ float sh[32];
    grid_dep_launch();
    grid_dep_wait();
    float m = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, fabsf(__half2float(in[i])));
    const float absmax = block_max(m, sh);
    if (threadIdx.x == 0) *d_absmax = absmax;
    if (QUANT) {
        const float scale = quant_scale(absmax);
        for (int i = threadIdx.x; i < n; i += blockDim.x)
            q[i] = static_cast<int8_t>(quantize_one(__half2float(in[i]), scale));
    }
}

// ---- dequantize_gpu (inference_kernels.cu:162-171) --------------------------------------
__global__ void dequantize_kernel(const int32_t* __restrict__ in, __half* __restrict__ out,
                                  const float* __restrict__ d_absmax, float gamma, int n) {
    grid_dep_launch();
    grid_dep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float dq = dequant_scale(gamma, *d_absmax);
    out[i] = __float2half_rn(__fmul_rn(static_cast<float>(in[i]), dq));
}

// ---- rope_gpu (inference_kernels.cu:185-206) --------------------------------------------
__device__ __forceinline__ void rope_pair(float x0, float x1, int pair, int head_dim, int pos,
                                          float theta, float& y0, float& y1) {
    const float freq = 1.0f / powf(theta, static_cast<float>(2 * pair) / static_cast<float>(head_dim));
    const float angle = static_cast<float>(pos) * freq;
    const float c = cosf(angle), s = sinf(angle);
    y0 = x0 * c - x1 * s;
    y1 = x0 * s + x1 * c;
}

__global__ void rope_kernel(__half* __restrict__ vec, int num_heads, int head_dim, int pos,
                            float theta) {
    grid_dep_launch();
    grid_dep_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const int hp = head_dim / 2;
    if (t >= num_heads * hp) return;
    const int head = t / hp, pair = t % hp;
    const int idx = head * head_dim + 2 * pair;
    float y0, y1;
    rope_pair(__half2float(vec[idx]), __half2float(vec[idx + 1]), pair, head_dim, pos, theta, y0, y1);
    vec[idx] = __float2half_rn(y0);
    vec[idx + 1] = __float2half_rn(y1);
}

// ---- scatter_kv_gpu (inference_kernels.cu:215-227) --------------------------------------
__global__ void scatter_kv_kernel(const __half* __restrict__ src, __half* __restrict__ cache,
                                  int num_kv_heads, int head_dim, int max_seq_len, int pos) {
    grid_dep_launch();
    grid_dep_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= num_kv_heads * head_dim) return;
    const int h = t / head_dim, d = t % head_dim;
    cache[(static_cast<size_t>(h) * max_seq_len + pos) * head_dim + d] = src[t];
}

// ---- attention_scores_gpu (inference_kernels.cu:241-275) --------------------------------
__global__ void __launch_bounds__(kBlock) attention_scores_kernel(
    const __half* __restrict__ Q, const __half* __restrict__ K, float* __restrict__ scores,
    int num_heads, int num_kv_heads, int head_dim, int max_seq_len, int seq_len, float scale) {
    grid_dep_launch();
    grid_dep_wait();
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y;
    const int j = blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5);
    if (j >= seq_len) return;
    const int kv = head * num_kv_heads / num_heads;
    const __half* q = Q + static_cast<size_t>(head) * head_dim;
    const __half* k = K + (static_cast<size_t>(kv) * max_seq_len + j) * head_dim;
    float acc = 0.0f;
    for (int d = lane; d < head_dim; d += 32) acc += __half2float(q[d]) * __half2float(k[d]);
    acc = warp_sum(acc);
    if (lane == 0) scores[static_cast<size_t>(head) * max_seq_len + j] = acc * scale;
}

// ---- softmax_gpu (inference_kernels.cu:283-339) ------------------------------------------
__global__ void __launch_bounds__(kBlock) softmax_kernel(float* __restrict__ scores,
                                                         int max_seq_len, int seq_len) {
    __shared__ float sh[32];
    grid_dep_launch();
    grid_dep_wait();
    float* hs = scores + static_cast<size_t>(blockIdx.x) * max_seq_len;
    float m = -1e30f;
    for (int j = threadIdx.x; j < seq_len; j += blockDim.x) m = fmaxf(m, hs[j]);
    m = block_max(m, sh);
    float s = 0.0f;
    for (int j = threadIdx.x; j < seq_len; j += blockDim.x) {
        const float e = expf(hs[j] - m);
        hs[j] = e;
        s += e;
    }
    s = block_sum(s, sh);
    const float inv = 1.0f / s;
    for (int j = threadIdx.x; j < seq_len; j += blockDim.x) hs[j] *= inv;
}

// ---- attention_output_gpu (inference_kernels.cu:350-371) --------------------------------
// Positions are split over the warps of the block (the reference walks them serially
// in one thread per output dim); partial sums are combined in shared memory.
__global__ void __launch_bounds__(kBlock) attention_output_kernel(
    const float* __restrict__ scores, const __half* __restrict__ V, __half* __restrict__ out,
    int num_heads, int num_kv_heads, int head_dim, int max_seq_len, int seq_len) {
    extern __shared__ float part[];  // (kBlock/32) x head_dim
    grid_dep_launch();
    grid_dep_wait();
    const int head = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = kBlock / 32;
    const int kv = head * num_kv_heads / num_heads;
    const float* hs = scores + static_cast<size_t>(head) * max_seq_len;
    const __half* v = V + static_cast<size_t>(kv) * max_seq_len * head_dim;
    for (int d0 = 0; d0 < head_dim; d0 += 32) {
        const int d = d0 + lane;
        float acc = 0.0f;
        if (d < head_dim)
            for (int j = warp; j < seq_len; j += nw)
                acc += hs[j] * __half2float(v[static_cast<size_t>(j) * head_dim + d]);
        if (d < head_dim) part[warp * head_dim + d] = acc;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.0f;
        for (int w = 0; w < nw; ++w) acc += part[w * head_dim + d];
        out[static_cast<size_t>(head) * head_dim + d] = __float2half_rn(acc);
    }
}

// ---- one-launch decode attention ----------------------------------------------------------
// One block per query head: scores into shared memory, softmax there, then P*V.
__global__ void __launch_bounds__(kBlock) decode_attention_kernel(
    const __half* __restrict__ Q, const __half* __restrict__ K, const __half* __restrict__ V,
    __half* __restrict__ out, int num_heads, int num_kv_heads, int head_dim, int max_seq_len,
    int seq_len, float scale) {
    extern __shared__ float dsm[];  // seq_len scores, then (kBlock/32) x head_dim partials
    __shared__ float sh[32];
    grid_dep_launch();
    grid_dep_wait();
    float* sc = dsm;
    float* part = dsm + ((seq_len + 31) & ~31);
    const int head = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = kBlock / 32;
    const int kv = head * num_kv_heads / num_heads;
    const __half* q = Q + static_cast<size_t>(head) * head_dim;
    const __half* kbase = K + static_cast<size_t>(kv) * max_seq_len * head_dim;
    const __half* vbase = V + static_cast<size_t>(kv) * max_seq_len * head_dim;

    float m = -1e30f;
    for (int j = warp; j < seq_len; j += nw) {
        const __half* k = kbase + static_cast<size_t>(j) * head_dim;
        float acc = 0.0f;
        for (int d = lane; d < head_dim; d += 32) acc += __half2float(q[d]) * __half2float(k[d]);
        acc = warp_sum(acc) * scale;
        if (lane == 0) sc[j] = acc;
        m = fmaxf(m, acc);
    }
    m = block_max(m, sh);  // contains the barrier that publishes sc[]
    float s = 0.0f;
    for (int j = threadIdx.x; j < seq_len; j += blockDim.x) {
        const float e = expf(sc[j] - m);
        sc[j] = e;
        s += e;
    }
    s = block_sum(s, sh);
    const float inv = 1.0f / s;
    for (int j = threadIdx.x; j < seq_len; j += blockDim.x) sc[j] *= inv;
    __syncthreads();
    for (int d0 = 0; d0 < head_dim; d0 += 32) {
        const int d = d0 + lane;
        float acc = 0.0f;
        if (d < head_dim)
            for (int j = warp; j < seq_len; j += nw)
                acc += sc[j] * __half2float(vbase[static_cast<size_t>(j) * head_dim + d]);
        if (d < head_dim) part[warp * head_dim + d] = acc;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.0f;
        for (int w = 0; w < nw; ++w) acc += part[w * head_dim + d];
        out[static_cast<size_t>(head) * head_dim + d] = __float2half_rn(acc);
    }
}

// ---- element-wise kernels (inference_kernels.cu:379-410, 460-479) -----------------------
__global__ void relu2_mul_kernel(const __half* __restrict__ g, const __half* __restrict__ u,
                                 __half* __restrict__ out, int n) {
    grid_dep_launch();
    grid_dep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float r = fmaxf(0.0f, __half2float(g[i]));
    out[i] = __float2half_rn(__fmul_rn(__fmul_rn(r, r), __half2float(u[i])));
}
__global__ void relu2_mul_f32_kernel(const __half* __restrict__ g, const __half* __restrict__ u,
                                     float* __restrict__ out, int n) {
    grid_dep_launch();
    grid_dep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float r = fmaxf(0.0f, __half2float(g[i]));
    out[i] = __fmul_rn(__fmul_rn(r, r), __half2float(u[i]));
}
__global__ void float_to_half_kernel(const float* __restrict__ in, __half* __restrict__ out, int n) {
    grid_dep_launch();
    grid_dep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(in[i]);
}
__global__ void residual_add_kernel(const __half* __restrict__ a, const __half* __restrict__ b,
                                    __half* __restrict__ out, int n) {
    grid_dep_launch();
    grid_dep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(__half2float(a[i]) + __half2float(b[i]));
}

// ---- half_gemv_gpu (inference_kernels.cu:488-531) ----------------------------------------
// lm_head: rows x cols half times cols half -> rows fp32.  HBM bound (656 MB at the
// 2B-4T shape).  x is converted to fp32 once per block into shared memory; each warp
// streams two rows at a time with 128-bit loads (when cols % 8 == 0 and W is 16-byte
// aligned) and accumulates in fp32.
template <bool VEC>
__global__ void __launch_bounds__(kBlock) half_gemv_kernel(const __half* __restrict__ W,
                                                           const __half* __restrict__ x,
                                                           float* __restrict__ y, int rows, int cols) {
    extern __shared__ float xs[];
    grid_dep_launch();
    grid_dep_wait();
    for (int i = threadIdx.x; i < cols; i += blockDim.x) xs[i] = __half2float(x[i]);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (kBlock / 32);
    const int warp = blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5);
    if (VEC) {
        const int cv = cols >> 3;
        for (int r = warp * 2; r < rows; r += warps_total * 2) {
            const bool two = (r + 1 < rows);
            const uint4* w0 = reinterpret_cast<const uint4*>(W + static_cast<size_t>(r) * cols);
            const uint4* w1 = reinterpret_cast<const uint4*>(W + static_cast<size_t>(r + (two ? 1 : 0)) * cols);
            float a0 = 0.0f, a1 = 0.0f;
            for (int j = lane; j < cv; j += 32) {
                uint4 p0, p1;
                asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(p0.x), "=r"(p0.y), "=r"(p0.z), "=r"(p0.w) : "l"(w0 + j));
                asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(p1.x), "=r"(p1.y), "=r"(p1.z), "=r"(p1.w) : "l"(w1 + j));
                const float4 xa = *reinterpret_cast<const float4*>(xs + 8 * j);
                const float4 xb = *reinterpret_cast<const float4*>(xs + 8 * j + 4);
                const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                const uint32_t q0[4] = {p0.x, p0.y, p0.z, p0.w};
                const uint32_t q1[4] = {p1.x, p1.y, p1.z, p1.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&q0[k]));
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&q1[k]));
                    a0 = fmaf(f0.x, xv[2 * k], a0);
                    a0 = fmaf(f0.y, xv[2 * k + 1], a0);
                    a1 = fmaf(f1.x, xv[2 * k], a1);
                    a1 = fmaf(f1.y, xv[2 * k + 1], a1);
                }
            }
            a0 = warp_sum(a0);
            a1 = warp_sum(a1);
            if (lane == 0) {
                y[r] = a0;
                if (two) y[r + 1] = a1;
            }
        }
    } else {
        for (int r = warp; r < rows; r += warps_total) {
            const __half* w = W + static_cast<size_t>(r) * cols;
            float a = 0.0f;
            for (int j = lane; j < cols; j += 32) a = fmaf(__half2float(w[j]), xs[j], a);
            a = warp_sum(a);
            if (lane == 0) y[r] = a;
        }
    }
}

static int grid_for(int n) { return (n + kBlock - 1) / kBlock; }
static int norm_threads(int n) {
    int t = ((n + 3) / 4 + 31) & ~31;  // about four elements per thread
    return max(32, min(1024, t));
}

}  // namespace spb

using namespace spb;

#define SPB_REQUIRE(cond, name, what) \
    do { if (!(cond)) return fail(SPB_E_INVALID, "%s: %s", name, what); } while (0)

extern "C" int spb_rms_norm(const void* input, const float* weight, void* output, int size, float eps,
                            void* stream) {
    SPB_REQUIRE(size >= 0, "spb_rms_norm", "negative size");
    if (size == 0) return SPB_OK;
    SPB_REQUIRE(input && weight && output, "spb_rms_norm", "null pointer");
    return launch("spb_rms_norm", rms_norm_kernel<__half>, dim3(1), dim3(norm_threads(size)), 0, stream,
                  static_cast<const __half*>(input), weight, static_cast<__half*>(output), size, eps);
}

extern "C" int spb_rms_norm_f32in(const float* input, const float* weight, void* output, int size,
                                  float eps, void* stream) {
    SPB_REQUIRE(size >= 0, "spb_rms_norm_f32in", "negative size");
    if (size == 0) return SPB_OK;
    SPB_REQUIRE(input && weight && output, "spb_rms_norm_f32in", "null pointer");
    return launch("spb_rms_norm_f32in", rms_norm_kernel<float>, dim3(1), dim3(norm_threads(size)), 0,
                  stream, input, weight, static_cast<__half*>(output), size, eps);
}

extern "C" int spb_absmax_quantize(const void* input, int8_t* output, float* d_absmax, int size,
                                   void* stream) {
    SPB_REQUIRE(size >= 0, "spb_absmax_quantize", "negative size");
    SPB_REQUIRE(d_absmax && (size == 0 || (input && output)), "spb_absmax_quantize", "null pointer");
    return launch("spb_absmax_quantize", absmax_kernel<true>, dim3(1), dim3(norm_threads(size)), 0,
                  stream, static_cast<const __half*>(input), output, d_absmax, size);
}

extern "C" int spb_absmax_reduce(const void* input, float* d_absmax, int size, void* stream) {
    SPB_REQUIRE(size >= 0, "spb_absmax_reduce", "negative size");
    SPB_REQUIRE(d_absmax && (size == 0 || input), "spb_absmax_reduce", "null pointer");
    return launch("spb_absmax_reduce", absmax_kernel<false>, dim3(1), dim3(norm_threads(size)), 0,
                  stream, static_cast<const __half*>(input), static_cast<int8_t*>(nullptr), d_absmax, size);
}

extern "C" int spb_dequantize(const int32_t* input, void* output, const float* d_absmax, float gamma,
                              int size, void* stream) {
    SPB_REQUIRE(size >= 0, "spb_dequantize", "negative size");
    if (size == 0) return SPB_OK;
    SPB_REQUIRE(input && output && d_absmax, "spb_dequantize", "null pointer");
    return launch("spb_dequantize", dequantize_kernel, dim3(grid_for(size)), dim3(kBlock), 0, stream,
                  input, static_cast<__half*>(output), d_absmax, gamma, size);
}

extern "C" int spb_rope(void* vec, int num_heads, int head_dim, int pos, float theta, void* stream) {
    SPB_REQUIRE(num_heads >= 0 && head_dim >= 0 && head_dim % 2 == 0, "spb_rope", "bad shape");
    const int pairs = num_heads * (head_dim / 2);
    if (pairs == 0) return SPB_OK;
    SPB_REQUIRE(vec, "spb_rope", "null pointer");
    return launch("spb_rope", rope_kernel, dim3(grid_for(pairs)), dim3(kBlock), 0, stream,
                  static_cast<__half*>(vec), num_heads, head_dim, pos, theta);
}

extern "C" int spb_scatter_kv(const void* src, void* cache, int num_kv_heads, int head_dim,
                              int max_seq_len, int pos, void* stream) {
    SPB_REQUIRE(num_kv_heads >= 0 && head_dim >= 0, "spb_scatter_kv", "bad shape");
    SPB_REQUIRE(pos >= 0 && pos < max_seq_len, "spb_scatter_kv", "pos outside the cache");
    const int total = num_kv_heads * head_dim;
    if (total == 0) return SPB_OK;
    SPB_REQUIRE(src && cache, "spb_scatter_kv", "null pointer");
    return launch("spb_scatter_kv", scatter_kv_kernel, dim3(grid_for(total)), dim3(kBlock), 0, stream,
                  static_cast<const __half*>(src), static_cast<__half*>(cache), num_kv_heads, head_dim,
                  max_seq_len, pos);
}

extern "C" int spb_attention_scores(const void* Q, const void* K_cache, float* scores, int num_heads,
                                    int num_kv_heads, int head_dim, int max_seq_len, int seq_len,
                                    float scale, void* stream) {
    SPB_REQUIRE(num_heads >= 0 && num_kv_heads > 0 && head_dim > 0, "spb_attention_scores", "bad shape");
    SPB_REQUIRE(seq_len >= 0 && seq_len <= max_seq_len, "spb_attention_scores", "seq_len outside the cache");
    if (num_heads == 0 || seq_len == 0) return SPB_OK;
    SPB_REQUIRE(Q && K_cache && scores, "spb_attention_scores", "null pointer");
    dim3 grid((seq_len + kBlock / 32 - 1) / (kBlock / 32), num_heads);
    return launch("spb_attention_scores", attention_scores_kernel, grid, dim3(kBlock), 0, stream,
                  static_cast<const __half*>(Q), static_cast<const __half*>(K_cache), scores, num_heads,
                  num_kv_heads, head_dim, max_seq_len, seq_len, scale);
}

extern "C" int spb_softmax(float* scores, int num_heads, int max_seq_len, int seq_len, void* stream) {
    SPB_REQUIRE(num_heads >= 0 && seq_len >= 0 && seq_len <= max_seq_len, "spb_softmax", "bad shape");
    if (num_heads == 0 || seq_len == 0) return SPB_OK;
    SPB_REQUIRE(scores, "spb_softmax", "null pointer");
    return launch("spb_softmax", softmax_kernel, dim3(num_heads), dim3(kBlock), 0, stream, scores,
                  max_seq_len, seq_len);
}

extern "C" int spb_attention_output(const float* scores, const void* V_cache, void* output,
                                    int num_heads, int num_kv_heads, int head_dim, int max_seq_len,
                                    int seq_len, void* stream) {
    SPB_REQUIRE(num_heads >= 0 && num_kv_heads > 0 && head_dim > 0, "spb_attention_output", "bad shape");
    SPB_REQUIRE(seq_len >= 0 && seq_len <= max_seq_len, "spb_attention_output", "seq_len outside the cache");
    if (num_heads == 0) return SPB_OK;
    SPB_REQUIRE(scores && V_cache && output, "spb_attention_output", "null pointer");
    const size_t smem = sizeof(float) * (kBlock / 32) * head_dim;
    SPB_REQUIRE(smem <= 48 * 1024, "spb_attention_output", "head_dim too large");
    return launch("spb_attention_output", attention_output_kernel, dim3(num_heads), dim3(kBlock), smem,
                  stream, scores, static_cast<const __half*>(V_cache), static_cast<__half*>(output),
                  num_heads, num_kv_heads, head_dim, max_seq_len, seq_len);
}

extern "C" int spb_decode_attention(const void* Q, const void* K_cache, const void* V_cache,
                                    void* output, int num_heads, int num_kv_heads, int head_dim,
                                    int max_seq_len, int seq_len, float scale, void* stream) {
    SPB_REQUIRE(num_heads >= 0 && num_kv_heads > 0 && head_dim > 0, "spb_decode_attention", "bad shape");
    SPB_REQUIRE(seq_len >= 1 && seq_len <= max_seq_len, "spb_decode_attention", "seq_len outside the cache");
    if (num_heads == 0) return SPB_OK;
    SPB_REQUIRE(Q && K_cache && V_cache && output, "spb_decode_attention", "null pointer");
    const size_t smem = sizeof(float) * (((seq_len + 31) & ~31) + (kBlock / 32) * head_dim);
    if (smem > 200 * 1024) return fail(SPB_E_UNSUPPORTED, "spb_decode_attention: seq_len %d too long", seq_len);
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(decode_attention_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (err != cudaSuccess) return fail(SPB_E_CUDA, "spb_decode_attention: %s", cudaGetErrorString(err));
    }
    return launch("spb_decode_attention", decode_attention_kernel, dim3(num_heads), dim3(kBlock), smem,
                  stream, static_cast<const __half*>(Q), static_cast<const __half*>(K_cache),
                  static_cast<const __half*>(V_cache), static_cast<__half*>(output), num_heads,
                  num_kv_heads, head_dim, max_seq_len, seq_len, scale);
}

extern "C" int spb_relu2_mul(const void* gate, const void* up, void* output, int size, void* stream) {
    SPB_REQUIRE(size >= 0, "spb_relu2_mul", "negative size");
    if (size == 0) return SPB_OK;
    SPB_REQUIRE(gate && up && output, "spb_relu2_mul", "null pointer");
    return launch("spb_relu2_mul", relu2_mul_kernel, dim3(grid_for(size)), dim3(kBlock), 0, stream,
                  static_cast<const __half*>(gate), static_cast<const __half*>(up),
                  static_cast<__half*>(output), size);
}

extern "C" int spb_relu2_mul_f32(const void* gate, const void* up, float* output, int size, void* stream) {
    SPB_REQUIRE(size >= 0, "spb_relu2_mul_f32", "negative size");
    if (size == 0) return SPB_OK;
    SPB_REQUIRE(gate && up && output, "spb_relu2_mul_f32", "null pointer");
    return launch("spb_relu2_mul_f32", relu2_mul_f32_kernel, dim3(grid_for(size)), dim3(kBlock), 0, stream,
                  static_cast<const __half*>(gate), static_cast<const __half*>(up), output, size);
}

extern "C" int spb_float_to_half(const float* input, void* output, int size, void* stream) {
    SPB_REQUIRE(size >= 0, "spb_float_to_half", "negative size");
    if (size == 0) return SPB_OK;
    SPB_REQUIRE(input && output, "spb_float_to_half", "null pointer");
    return launch("spb_float_to_half", float_to_half_kernel, dim3(grid_for(size)), dim3(kBlock), 0, stream,
                  input, static_cast<__half*>(output), size);
}

extern "C" int spb_residual_add(const void* a, const void* b, void* output, int size, void* stream) {
    SPB_REQUIRE(size >= 0, "spb_residual_add", "negative size");
    if (size == 0) return SPB_OK;
    SPB_REQUIRE(a && b && output, "spb_residual_add", "null pointer");
    return launch("spb_residual_add", residual_add_kernel, dim3(grid_for(size)), dim3(kBlock), 0, stream,
                  static_cast<const __half*>(a), static_cast<const __half*>(b),
                  static_cast<__half*>(output), size);
}

extern "C" int spb_half_gemv(const void* W, const void* x, float* y, int rows, int cols, void* stream) {
    SPB_REQUIRE(rows >= 0 && cols >= 0, "spb_half_gemv", "negative size");
    if (rows == 0) return SPB_OK;
    SPB_REQUIRE(W && x && y, "spb_half_gemv", "null pointer");
    const size_t smem = sizeof(float) * static_cast<size_t>(cols);
    if (smem > 200 * 1024) return fail(SPB_E_UNSUPPORTED, "spb_half_gemv: cols %d too large", cols);
    const bool vec = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0;
    auto kernel = vec ? half_gemv_kernel<true> : half_gemv_kernel<false>;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (err != cudaSuccess) return fail(SPB_E_CUDA, "spb_half_gemv: %s", cudaGetErrorString(err));
    }
    const int rows_per_block = (kBlock / 32) * 2;
    int grid = (rows + rows_per_block - 1) / rows_per_block;
    grid = max(1, min(grid, sm_count() * 8));
    return launch("spb_half_gemv", kernel, dim3(grid), dim3(kBlock), smem, stream,
                  static_cast<const __half*>(W), static_cast<const __half*>(x), y, rows, cols);
}
