// Row-batched small ops of the batched prefill: the same arithmetic as the single-vector wrappers, one block per
// token of the batch, so that a batch of T prompt tokens gives the values T calls of
// InferenceEngine::forward (src/inference.cu:123-283) would give for the integer and element-wise parts.
//   embed_rows           : the embedding row copy of src/inference.cu:128-131 for T tokens
//   absmax_quantize_rows : absmax_quantize_gpu (src/kernels/inference_kernels.cu:69-114) per row
//   dequantize_rows      : dequantize_gpu (src/kernels/inference_kernels.cu:162-171) per row, each row with its own absmax
#include "fused_ops.cuh"

namespace spb {

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    return v;
}

__global__ void __launch_bounds__(256) embed_rows_kernel(const __half* __restrict__ embed,
                                                         const int* __restrict__ tokens,
                                                         __half* __restrict__ x, int hidden) {
    grid_dep_launch();
    grid_dep_wait();
    const int token = tokens[blockIdx.x];
    const __half* row = embed + static_cast<size_t>(token) * hidden;
    __half* dst = x + static_cast<size_t>(blockIdx.x) * hidden;
    if ((hidden & 7) == 0) {
        const uint4* r4 = reinterpret_cast<const uint4*>(row);
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) d4[i] = r4[i];
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = row[i];
    }
}

__global__ void __launch_bounds__(1024) absmax_quantize_rows_kernel(const __half* __restrict__ in,
                                                                    int8_t* __restrict__ out,
                                                                    float* __restrict__ d_absmax, int n) {
    __shared__ float sh[32];
    grid_dep_launch();
    grid_dep_wait();
    in += static_cast<size_t>(blockIdx.x) * n;
    out += static_cast<size_t>(blockIdx.x) * n;
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = (nt + 31) >> 5;
    float m = 0.0f;
    for (int i = tid; i < n; i += nt) m = fmaxf(m, fabsf(__half2float(in[i])));
    m = warp_max(m);
    if (lane == 0) sh[warp] = m;
    __syncthreads();
    const float absmax = warp_max(lane < nw ? sh[lane] : 0.0f);
    if (tid == 0) d_absmax[blockIdx.x] = absmax;
    const float qs = quant_scale(absmax);
    for (int i = tid; i < n; i += nt) out[i] = static_cast<int8_t>(quantize_one(__half2float(in[i]), qs));
}

// grid (ceil(rows / (256 * 4)), T): four accumulators per thread
__global__ void __launch_bounds__(256) dequantize_rows_kernel(const int32_t* __restrict__ acc,
                                                              __half* __restrict__ out,
                                                              const float* __restrict__ d_absmax, float gamma,
                                                              int rows) {
    grid_dep_launch();
    grid_dep_wait();
    const float scale = dequant_scale(gamma, d_absmax[blockIdx.y]);
    const size_t base = static_cast<size_t>(blockIdx.y) * rows;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < rows && (rows & 3) == 0) {
        const int4 a = *reinterpret_cast<const int4*>(acc + base + i);
        const __half2 lo = __halves2half2(__float2half_rn(__fmul_rn(static_cast<float>(a.x), scale)),
                                          __float2half_rn(__fmul_rn(static_cast<float>(a.y), scale)));
        const __half2 hi = __halves2half2(__float2half_rn(__fmul_rn(static_cast<float>(a.z), scale)),
                                          __float2half_rn(__fmul_rn(static_cast<float>(a.w), scale)));
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&lo);
        o.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(out + base + i) = o;
    } else {
        for (int j = i; j < min(i + 4, rows); ++j)
            out[base + j] = __float2half_rn(__fmul_rn(static_cast<float>(acc[base + j]), scale));
    }
}

}  // namespace

int embed_rows(const void* embed, const int* d_tokens, void* x, int hidden, int vectors, void* stream) {
    return launch("embed_rows", embed_rows_kernel, dim3(vectors), dim3(256), 0, stream,
                  static_cast<const __half*>(embed), d_tokens, static_cast<__half*>(x), hidden);
}

int absmax_quantize_rows(const void* in, int8_t* out, float* d_absmax, int n, int vectors, void* stream) {
    int t = ((n + 3) / 4 + 31) & ~31;
    t = max(32, min(1024, t));
    return launch("absmax_quantize_rows", absmax_quantize_rows_kernel, dim3(vectors), dim3(t), 0, stream,
                  static_cast<const __half*>(in), out, d_absmax, n);
}

int dequantize_rows(const int32_t* acc, void* out, const float* d_absmax, float gamma, int rows, int vectors,
                    void* stream) {
    return launch("dequantize_rows", dequantize_rows_kernel, dim3((rows + 1023) / 1024, vectors), dim3(256), 0,
                  stream, acc, static_cast<__half*>(out), d_absmax, gamma, rows);
}

}  // namespace spb
