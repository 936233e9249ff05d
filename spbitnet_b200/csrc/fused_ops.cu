// Fused single-launch forms of the small vector ops between the BitLinear GEMVs of a
// decode step (src/inference.cu:123-283).  Each kernel keeps every rounding point of
// the op sequence it replaces, so its outputs equal running the reference wrappers one
// after the other:
//   residual_norm_quant : [rms_norm(sub_norm)] -> residual_add -> rms_norm -> absmax_quantize
//   relu2_norm_quant    : relu2_mul_f32 -> rms_norm_f32in | float_to_half -> absmax_quantize
//   rope_scatter        : rope(Q), rope(K), scatter_kv(K), scatter_kv(V)
//   embed / argmax      : the D2D embedding copy and the host arg-max of src/main.cpp:285-287
// The position is read from device memory so that one captured CUDA graph serves every
// token of a sequence.
#include "fused_ops.cuh"

namespace spb {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    return v;
}
__device__ __forceinline__ float bsum(float v, float* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = wsum(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    return wsum((lane < nw) ? sh[lane] : 0.0f);
}
__device__ __forceinline__ float bmax(float v, float* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = wmax(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    return wmax((lane < nw) ? sh[lane] : 0.0f);
}

// x (residual stream, half, n) is updated in place when delta is given:
//   d  = sub_w ? half(delta * rsqrt(mean(delta^2)+eps) * sub_w) : delta      (rms_norm_gpu)
//   x  = half(float(d) + float(x))                                           (residual_add_gpu)
// then  xn = half(x * rsqrt(mean(x^2)+eps) * w)                              (rms_norm_gpu)
//       absmax = max|xn| ; xq = clamp(rn(xn * 127/absmax))                   (absmax_quantize_gpu)
// xn_out (optional) receives xn.
__global__ void __launch_bounds__(1024) residual_norm_quant_kernel(
    const __half* __restrict__ delta, const float* __restrict__ sub_w, __half* __restrict__ x,
    const float* __restrict__ w, __half* __restrict__ xn_out, int8_t* __restrict__ xq,
    float* __restrict__ d_absmax, int n, float eps) {
    extern __shared__ float buf[];  // n floats
    __shared__ float sh[32];
    grid_dep_launch();
    grid_dep_wait();
    const int tid = threadIdx.x, nt = blockDim.x;
    {   // one block per vector: block b works on the b-th vector of n elements (prefill batches; decode has one)
        const size_t off = static_cast<size_t>(blockIdx.x) * n;
        if (delta) delta += off;
        x += off;
        if (xn_out) xn_out += off;
        xq += off;
        d_absmax += blockIdx.x;
    }
    if (delta) {
        float sub_scale = 1.0f;
        if (sub_w) {
            float s = 0.0f;
            for (int i = tid; i < n; i += nt) {
                const float v = __half2float(delta[i]);
                s += v * v;
            }
            sub_scale = rsqrtf(bsum(s, sh) / static_cast<float>(n) + eps);
        }
        for (int i = tid; i < n; i += nt) {
            float d = __half2float(delta[i]);
            if (sub_w) d = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(d, sub_scale), sub_w[i])));
            const __half r = __float2half_rn(d + __half2float(x[i]));
            x[i] = r;
            buf[i] = __half2float(r);
        }
    } else {
        for (int i = tid; i < n; i += nt) buf[i] = __half2float(x[i]);
    }
    float s = 0.0f;
    for (int i = tid; i < n; i += nt) s += buf[i] * buf[i];
    const float scale = rsqrtf(bsum(s, sh) / static_cast<float>(n) + eps);
    float m = 0.0f;
    for (int i = tid; i < n; i += nt) {
        const __half h = __float2half_rn(__fmul_rn(__fmul_rn(buf[i], scale), w[i]));
        if (xn_out) xn_out[i] = h;
        const float v = __half2float(h);
        buf[i] = v;
        m = fmaxf(m, fabsf(v));
    }
    const float absmax = bmax(m, sh);
    if (tid == 0) *d_absmax = absmax;
    const float qs = quant_scale(absmax);
    for (int i = tid; i < n; i += nt) xq[i] = static_cast<int8_t>(quantize_one(buf[i], qs));
}

// m = max(0,gate)^2 * up in fp32 (relu2_mul_f32_gpu); h = sub_w ? half(m * rsqrt(mean(m^2)+eps) * sub_w)
// (rms_norm_f32in_gpu) : half(m) (float_to_half_gpu); then absmax_quantize_gpu of h.
__global__ void __launch_bounds__(1024) relu2_norm_quant_kernel(
    const __half* __restrict__ gate, const __half* __restrict__ up, const float* __restrict__ sub_w,
    __half* __restrict__ h_out, int8_t* __restrict__ hq, float* __restrict__ d_absmax, int n, float eps) {
    extern __shared__ float buf[];
    __shared__ float sh[32];
    grid_dep_launch();
    grid_dep_wait();
    const int tid = threadIdx.x, nt = blockDim.x;
    {   // one block per vector, as in residual_norm_quant_kernel
        const size_t off = static_cast<size_t>(blockIdx.x) * n;
        gate += off;
        up += off;
        if (h_out) h_out += off;
        hq += off;
        d_absmax += blockIdx.x;
    }
    float s = 0.0f;
    for (int i = tid; i < n; i += nt) {
        const float r = fmaxf(0.0f, __half2float(gate[i]));
        const float v = __fmul_rn(__fmul_rn(r, r), __half2float(up[i]));
        buf[i] = v;
        s += v * v;
    }
    float scale = 1.0f;
    if (sub_w) scale = rsqrtf(bsum(s, sh) / static_cast<float>(n) + eps);
    float m = 0.0f;
    for (int i = tid; i < n; i += nt) {
        const __half h = sub_w ? __float2half_rn(__fmul_rn(__fmul_rn(buf[i], scale), sub_w[i]))
                               : __float2half_rn(buf[i]);
        if (h_out) h_out[i] = h;
        const float v = __half2float(h);
        buf[i] = v;
        m = fmaxf(m, fabsf(v));
    }
    const float absmax = bmax(m, sh);
    if (tid == 0) *d_absmax = absmax;
    const float qs = quant_scale(absmax);
    for (int i = tid; i < n; i += nt) hq[i] = static_cast<int8_t>(quantize_one(buf[i], qs));
}

// rope_gpu on Q (in place) and on K, then scatter_kv_gpu of the roped K and of V at *d_pos.
__global__ void __launch_bounds__(256) rope_scatter_kernel(__half* __restrict__ q,
                                                           const __half* __restrict__ k,
                                                           const __half* __restrict__ v,
                                                           __half* __restrict__ kcache,
                                                           __half* __restrict__ vcache, int num_heads,
                                                           int num_kv_heads, int head_dim,
                                                           int max_seq_len, float theta,
                                                           const int* __restrict__ d_pos, size_t seq_stride) {
    grid_dep_launch();
    grid_dep_wait();
    // blockIdx.y = token of a prefill batch (0 in decode): its vectors follow one another, its position is *d_pos + y.
    // With seq_stride != 0 the vectors are one token each of independent sequences instead: all at position *d_pos,
    // sequence y's caches seq_stride elements after sequence y - 1's.
    const int pos = *d_pos + (seq_stride ? 0 : blockIdx.y);
    kcache += seq_stride * blockIdx.y;
    vcache += seq_stride * blockIdx.y;
    q += static_cast<size_t>(blockIdx.y) * num_heads * head_dim;
    k += static_cast<size_t>(blockIdx.y) * num_kv_heads * head_dim;
    v += static_cast<size_t>(blockIdx.y) * num_kv_heads * head_dim;
    const int hp = head_dim / 2;
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const int q_pairs = num_heads * hp, k_pairs = num_kv_heads * hp;
    if (t < q_pairs + k_pairs) {
        const bool is_q = t < q_pairs;
        const int tt = is_q ? t : t - q_pairs;
        const int head = tt / hp, pair = tt % hp;
        const int idx = head * head_dim + 2 * pair;
        const __half* src = is_q ? q : k;
        __half y0, y1;
        rope_rotate(__half2float(src[idx]), __half2float(src[idx + 1]), pos, pair, head_dim, theta, y0, y1);
        if (is_q) {
            q[idx] = y0;
            q[idx + 1] = y1;
        } else {
            __half* dst = kcache + (static_cast<size_t>(head) * max_seq_len + pos) * head_dim + 2 * pair;
            dst[0] = y0;
            dst[1] = y1;
        }
    } else {
        const int e = (t - q_pairs - k_pairs) * 2;  // two V elements per thread
        if (e < num_kv_heads * head_dim) {
            const int head = e / head_dim, d = e % head_dim;
            __half* dst = vcache + (static_cast<size_t>(head) * max_seq_len + pos) * head_dim + d;
            dst[0] = v[e];
            dst[1] = v[e + 1];
        }
    }
}

// Decode attention with the sequence length taken from *d_pos + 1.  Same algorithm as
// decode_attention_kernel in decode_ops.cu.
__global__ void __launch_bounds__(256) decode_attention_pos_kernel(
    const __half* __restrict__ Q, const __half* __restrict__ K, const __half* __restrict__ V,
    __half* __restrict__ out, int num_heads, int num_kv_heads, int head_dim, int max_seq_len,
    float scale, const int* __restrict__ d_pos, size_t seq_stride) {
    extern __shared__ float dsm[];
    __shared__ float sh[32];
    grid_dep_launch();
    grid_dep_wait();
    // blockIdx.y = token of a prefill batch (0 in decode): it sees the positions up to its own.  With
    // seq_stride != 0: one token each of independent sequences at position *d_pos, caches seq_stride apart.
    const int seq_len = *d_pos + (seq_stride ? 0 : blockIdx.y) + 1;
    K += seq_stride * blockIdx.y;
    V += seq_stride * blockIdx.y;
    Q += static_cast<size_t>(blockIdx.y) * num_heads * head_dim;
    out += static_cast<size_t>(blockIdx.y) * num_heads * head_dim;
    float* sc = dsm;
    float* part = dsm + ((max_seq_len + 31) & ~31);
    const int head = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int kv = head * num_kv_heads / num_heads;
    const __half* q = Q + static_cast<size_t>(head) * head_dim;
    const __half* kbase = K + static_cast<size_t>(kv) * max_seq_len * head_dim;
    const __half* vbase = V + static_cast<size_t>(kv) * max_seq_len * head_dim;
    float m = -1e30f;
    for (int j = warp; j < seq_len; j += nw) {
        const __half* k = kbase + static_cast<size_t>(j) * head_dim;
        float acc = 0.0f;
        for (int d = lane; d < head_dim; d += 32) acc += __half2float(q[d]) * __half2float(k[d]);
        acc = wsum(acc) * scale;
        if (lane == 0) sc[j] = acc;
        m = fmaxf(m, acc);
    }
    {   // block max over values that may be negative
        m = wmax(m);
        __syncthreads();
        if (lane == 0) sh[warp] = m;
        __syncthreads();
        m = wmax((lane < nw) ? sh[lane] : -1e30f);
    }
    float s = 0.0f;
    for (int j = threadIdx.x; j < seq_len; j += blockDim.x) {
        const float e = expf(sc[j] - m);
        sc[j] = e;
        s += e;
    }
    s = bsum(s, sh);
    const float inv = 1.0f / s;
    for (int j = threadIdx.x; j < seq_len; j += blockDim.x) sc[j] *= inv;
    __syncthreads();
    for (int d0 = 0; d0 < head_dim; d0 += 32) {
        const int d = d0 + lane;
        float acc = 0.0f;
        if (d < head_dim) {
            for (int j = warp; j < seq_len; j += nw)
                acc += sc[j] * __half2float(vbase[static_cast<size_t>(j) * head_dim + d]);
            part[warp * head_dim + d] = acc;
        }
    }
    __syncthreads();
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.0f;
        for (int w = 0; w < nw; ++w) acc += part[w * head_dim + d];
        out[static_cast<size_t>(head) * head_dim + d] = __float2half_rn(acc);
    }
}

// Token selection + embedding row copy.  token = forced ? forced[pos] (prompt) : *d_next.
__global__ void __launch_bounds__(256) embed_kernel(const __half* __restrict__ embed,
                                                    __half* __restrict__ x, int hidden,
                                                    const int* __restrict__ d_prompt, int n_prompt,
                                                    const int* __restrict__ d_next,
                                                    const int* __restrict__ d_pos) {
    grid_dep_launch();
    grid_dep_wait();
    const int pos = *d_pos;
    const int token = (d_prompt && pos < n_prompt) ? d_prompt[pos] : *d_next;
    const __half* row = embed + static_cast<size_t>(token) * hidden;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x) x[i] = row[i];
}

// Arg-max, first maximum wins (std::max_element).  Stage 1: one candidate per block.
__global__ void __launch_bounds__(1024) argmax_stage1_kernel(const float* __restrict__ v, int n,
                                                             float* __restrict__ bval,
                                                             int* __restrict__ bidx) {
    __shared__ float sv[32];
    __shared__ int si[32];
    grid_dep_launch();
    grid_dep_wait();
    float best = -INFINITY;
    int besti = 0x7FFFFFFF;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float x = v[i];
        if (x > best || (x == best && i < besti) || besti == 0x7FFFFFFF) {
            best = x;
            besti = i;
        }
    }
    auto better = [](float a, int ai, float b, int bi) {
        if (bi == 0x7FFFFFFF) return true;
        if (ai == 0x7FFFFFFF) return false;
        return a > b || (a == b && ai < bi);
    };
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, off);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, besti, off);
        if (!better(best, besti, ov, oi)) { best = ov; besti = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = besti; }
    __syncthreads();
    if (warp == 0) {
        best = (lane < nw) ? sv[lane] : -INFINITY;
        besti = (lane < nw) ? si[lane] : 0x7FFFFFFF;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, off);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, besti, off);
            if (!better(best, besti, ov, oi)) { best = ov; besti = oi; }
        }
        if (lane == 0) { bval[blockIdx.x] = best; bidx[blockIdx.x] = besti; }
    }
}

// Stage 2: one warp folds the block candidates, publishes the token, records it at
// d_out[pos] (when given) and advances the position.
__global__ void __launch_bounds__(32) argmax_stage2_kernel(const float* __restrict__ bval,
                                                           const int* __restrict__ bidx, int nblocks,
                                                           int* __restrict__ d_next,
                                                           int* __restrict__ d_out,
                                                           int* __restrict__ d_pos) {
    grid_dep_launch();
    grid_dep_wait();
    float best = -INFINITY;
    int besti = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < nblocks; i += 32) {
        const float x = bval[i];
        const int xi = bidx[i];
        if (xi != 0x7FFFFFFF && (besti == 0x7FFFFFFF || x > best || (x == best && xi < besti))) {
            best = x;
            besti = xi;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, off);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, besti, off);
        if (oi != 0x7FFFFFFF && (besti == 0x7FFFFFFF || ov > best || (ov == best && oi < besti))) {
            best = ov;
            besti = oi;
        }
    }
    if (threadIdx.x == 0) {
        const int pos = *d_pos;
        *d_next = besti;
        if (d_out) d_out[pos] = besti;
        *d_pos = pos + 1;
    }
}

__global__ void set_int_kernel(int* __restrict__ dst, int value) {
    grid_dep_launch();
    grid_dep_wait();
    *dst = value;
}

static int fused_threads(int n) {
    int t = ((n + 3) / 4 + 31) & ~31;
    return max(32, min(1024, t));
}

int residual_norm_quant(const void* delta, const float* sub_w, void* x, const float* w, void* xn_out,
                        int8_t* xq, float* d_absmax, int n, float eps, void* stream, int vectors) {
    const size_t smem = sizeof(float) * static_cast<size_t>(n);
    if (smem > 200 * 1024) return fail(SPB_E_UNSUPPORTED, "residual_norm_quant: n=%d too large", n);
    if (smem > 48 * 1024) cudaFuncSetAttribute(residual_norm_quant_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return launch("residual_norm_quant", residual_norm_quant_kernel, dim3(vectors), dim3(fused_threads(n)), smem,
                  stream, static_cast<const __half*>(delta), sub_w, static_cast<__half*>(x), w,
                  static_cast<__half*>(xn_out), xq, d_absmax, n, eps);
}

int relu2_norm_quant(const void* gate, const void* up, const float* sub_w, void* h_out, int8_t* hq,
                     float* d_absmax, int n, float eps, void* stream, int vectors) {
    const size_t smem = sizeof(float) * static_cast<size_t>(n);
    if (smem > 200 * 1024) return fail(SPB_E_UNSUPPORTED, "relu2_norm_quant: n=%d too large", n);
    if (smem > 48 * 1024) cudaFuncSetAttribute(relu2_norm_quant_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return launch("relu2_norm_quant", relu2_norm_quant_kernel, dim3(vectors), dim3(fused_threads(n)), smem, stream,
                  static_cast<const __half*>(gate), static_cast<const __half*>(up), sub_w,
                  static_cast<__half*>(h_out), hq, d_absmax, n, eps);
}

int rope_scatter(void* q, const void* k, const void* v, void* kcache, void* vcache, int num_heads,
                 int num_kv_heads, int head_dim, int max_seq_len, float theta, const int* d_pos,
                 void* stream, int vectors, size_t seq_stride) {
    const int threads = (num_heads + num_kv_heads) * (head_dim / 2) + num_kv_heads * head_dim / 2;
    return launch("rope_scatter", rope_scatter_kernel, dim3((threads + 255) / 256, vectors), dim3(256), 0, stream,
                  static_cast<__half*>(q), static_cast<const __half*>(k), static_cast<const __half*>(v),
                  static_cast<__half*>(kcache), static_cast<__half*>(vcache), num_heads, num_kv_heads,
                  head_dim, max_seq_len, theta, d_pos, seq_stride);
}

int decode_attention_pos(const void* Q, const void* K, const void* V, void* out, int num_heads,
                         int num_kv_heads, int head_dim, int max_seq_len, float scale, const int* d_pos,
                         void* stream, int vectors, size_t seq_stride) {
    const size_t smem = sizeof(float) * (((max_seq_len + 31) & ~31) + 8 * static_cast<size_t>(head_dim));
    if (smem > 200 * 1024) return fail(SPB_E_UNSUPPORTED, "decode_attention: max_seq_len %d too long", max_seq_len);
    if (smem > 48 * 1024) cudaFuncSetAttribute(decode_attention_pos_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return launch("decode_attention_pos", decode_attention_pos_kernel, dim3(num_heads, vectors), dim3(256), smem,
                  stream, static_cast<const __half*>(Q), static_cast<const __half*>(K),
                  static_cast<const __half*>(V), static_cast<__half*>(out), num_heads, num_kv_heads,
                  head_dim, max_seq_len, scale, d_pos, seq_stride);
}

int embed_token(const void* embed, void* x, int hidden, const int* d_prompt, int n_prompt,
                const int* d_next, const int* d_pos, void* stream) {
    return launch("embed_token", embed_kernel, dim3((hidden + 255) / 256), dim3(256), 0, stream,
                  static_cast<const __half*>(embed), static_cast<__half*>(x), hidden, d_prompt, n_prompt,
                  d_next, d_pos);
}

int argmax_advance(const float* logits, int n, float* bval, int* bidx, int nblocks, int* d_next,
                   int* d_out, int* d_pos, void* stream) {
    int rc = launch("argmax_stage1", argmax_stage1_kernel, dim3(nblocks), dim3(1024), 0, stream, logits, n,
                    bval, bidx);
    if (rc) return rc;
    return launch("argmax_stage2", argmax_stage2_kernel, dim3(1), dim3(32), 0, stream,
                  static_cast<const float*>(bval), static_cast<const int*>(bidx), nblocks, d_next, d_out,
                  d_pos);
}

int set_int(int* dst, int value, void* stream) {
    return launch("set_int", set_int_kernel, dim3(1), dim3(1), 0, stream, dst, value);
}

}  // namespace spb
