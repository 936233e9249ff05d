// Split-KV decode attention for one new token (replaces attention_scores_gpu + softmax_gpu +
// attention_output_gpu of the reference, src/kernels/inference_kernels.cu:241-371, as one
// pass over the KV cache).
//
// The reference gives a head to one block and walks the positions serially; at a few
// hundred positions that is latency bound (a dependent global load per position).  Here the
// positions are cut into chunks of kChunk; block (kv head, chunk) serves every query head
// of the GQA group from one read of its K and V rows, keeps several rows in flight per
// warp, and writes an un-normalised partial result {max, sum, sum(e*V)} per (head, chunk)
// to a scratch buffer.  A second tiny kernel merges the chunks of a head with the usual
// log-sum-exp weights and rounds to half.  Scores, exponentials and the weighted sum are
// fp32 as in the reference; only the order of the additions differs.
#include "fused_ops.cuh"

namespace spb {

constexpr int kChunk = 64;       // positions per block
constexpr int kRowsPerWarp = kChunk / 8;  // kAttnThreads / 32 warps share a chunk
constexpr int kAttnThreads = 256;
constexpr int kMaxGroup = 8;     // query heads per KV head held in registers

// scratch layout: [head][split][2 + head_dim] floats = {m, l, o[0..head_dim)}
__host__ __device__ inline size_t attn_scratch_floats(int num_heads, int head_dim, int max_seq_len) {
    const int nsplit = (max_seq_len + kChunk - 1) / kChunk;
    return static_cast<size_t>(num_heads) * nsplit * (head_dim + 2);
}

template <int G>
__global__ void __launch_bounds__(kAttnThreads) attn_split_kernel(
    const __half* __restrict__ Q, const __half* __restrict__ K, const __half* __restrict__ V,
    float* __restrict__ scratch, int num_kv_heads, int head_dim, int max_seq_len, int nsplit_max,
    float scale, int seq_len_arg, const int* __restrict__ d_pos) {
    extern __shared__ float asm_[];  // [G][kChunk] scores, then [8 warps][G][head_dim] partial outputs
    grid_dep_launch();
    grid_dep_wait();
    const int seq_len = d_pos ? (*d_pos + 1) : seq_len_arg;
    const int kvh = blockIdx.x, split = blockIdx.y;
    const int p0 = split * kChunk;
    if (p0 >= seq_len) return;
    const int np = min(kChunk, seq_len - p0);
    float* sc = asm_;
    float* po = asm_ + G * kChunk;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = kAttnThreads / 32;
    const __half* kbase = K + (static_cast<size_t>(kvh) * max_seq_len + p0) * head_dim;
    const __half* vbase = V + (static_cast<size_t>(kvh) * max_seq_len + p0) * head_dim;
    const int ndl = (head_dim + 31) / 32;  // dims per lane, at most 8 (head_dim <= 256)

    // ---- scores: warp w takes positions w, w+8, ...: all of a warp's rows are in flight at once -------
    float qreg[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            qreg[g][i] = (i < ndl && d < head_dim)
                             ? __half2float(Q[(static_cast<size_t>(kvh) * G + g) * head_dim + d]) : 0.0f;
        }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        float kv[kRowsPerWarp / 2][8];
#pragma unroll
        for (int u = 0; u < kRowsPerWarp / 2; ++u) {
            const int j = warp + (half * (kRowsPerWarp / 2) + u) * nw;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = lane + 32 * i;
                kv[u][i] = (i < ndl && d < head_dim && j < np)
                               ? __half2float(kbase[static_cast<size_t>(j) * head_dim + d]) : 0.0f;
            }
        }
#pragma unroll
        for (int u = 0; u < kRowsPerWarp / 2; ++u) {
            const int j = warp + (half * (kRowsPerWarp / 2) + u) * nw;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float acc = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc += qreg[g][i] * kv[u][i];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
                if (lane == 0 && j < np) sc[g * kChunk + j] = acc * scale;
            }
        }
    }
    __syncthreads();

    // ---- per head: chunk max, exponentials, chunk sum (warp g handles head g, strided) -----
    for (int g = warp; g < G; g += nw) {
        float m = -1e30f;
        for (int j = lane; j < np; j += 32) m = fmaxf(m, sc[g * kChunk + j]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
        float l = 0.0f;
        for (int j = lane; j < np; j += 32) {
            const float e = expf(sc[g * kChunk + j] - m);
            sc[g * kChunk + j] = e;
            l += e;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, off);
        if (lane == 0) {
            float* dst = scratch + (static_cast<size_t>(kvh * G + g) * nsplit_max + split) * (head_dim + 2);
            dst[0] = m;
            dst[1] = l;
        }
    }
    __syncthreads();

    // ---- sum_j e[g][j] * V[j][d]: warp w takes positions w, w+8, ... (four rows in flight), lane l the dims
    //      l, l+32, ...; the eight partial sums meet in shared memory ------------------------------------
    {
        float acc[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float vv[kRowsPerWarp / 2][8];
#pragma unroll
            for (int u = 0; u < kRowsPerWarp / 2; ++u) {
                const int j = warp + (half * (kRowsPerWarp / 2) + u) * nw;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int d = lane + 32 * i;
                    vv[u][i] = (i < ndl && d < head_dim && j < np)
                                   ? __half2float(vbase[static_cast<size_t>(j) * head_dim + d]) : 0.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < kRowsPerWarp / 2; ++u) {
                const int j = warp + (half * (kRowsPerWarp / 2) + u) * nw;
                if (j < np) {
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float e = sc[g * kChunk + j];
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[g][i] += e * vv[u][i];
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = lane + 32 * i;
                if (i < ndl && d < head_dim) po[(warp * G + g) * head_dim + d] = acc[g][i];
            }
        __syncthreads();
        for (int t = tid; t < G * head_dim; t += kAttnThreads) {
            const int g = t / head_dim, dd = t - g * head_dim;
            float o = 0.0f;
#pragma unroll
            for (int w = 0; w < kAttnThreads / 32; ++w) o += po[(w * G + g) * head_dim + dd];
            scratch[(static_cast<size_t>(kvh * G + g) * nsplit_max + split) * (head_dim + 2) + 2 + dd] = o;
        }
    }
}

__global__ void __launch_bounds__(128) attn_combine_kernel(const float* __restrict__ scratch,
                                                           __half* __restrict__ out, int head_dim,
                                                           int nsplit_max, int seq_len_arg,
                                                           const int* __restrict__ d_pos) {
    grid_dep_launch();
    grid_dep_wait();
    const int seq_len = d_pos ? (*d_pos + 1) : seq_len_arg;
    const int nsplit = (seq_len + kChunk - 1) / kChunk;
    const int head = blockIdx.x;
    const float* base = scratch + static_cast<size_t>(head) * nsplit_max * (head_dim + 2);
    float M = -1e30f;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, base[s * (head_dim + 2)]);
    float L = 0.0f;
    for (int s = 0; s < nsplit; ++s) L += base[s * (head_dim + 2) + 1] * expf(base[s * (head_dim + 2)] - M);
    const float inv = 1.0f / L;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float o = 0.0f;
        for (int s = 0; s < nsplit; ++s)
            o += base[s * (head_dim + 2) + 2 + d] * expf(base[s * (head_dim + 2)] - M);
        out[static_cast<size_t>(head) * head_dim + d] = __float2half_rn(o * inv);
    }
}

// seq_len is taken from *d_pos + 1 when d_pos is given (graph replay), else from seq_len.
int decode_attention_split(const void* Q, const void* K, const void* V, void* out, int num_heads,
                           int num_kv_heads, int head_dim, int max_seq_len, int seq_len, const int* d_pos,
                           float scale, float* scratch, void* stream) {
    const char* name = "decode_attention_split";
    if (num_heads % num_kv_heads) return fail(SPB_E_UNSUPPORTED, "%s: %d heads over %d KV heads", name, num_heads, num_kv_heads);
    const int G = num_heads / num_kv_heads;
    if (G > kMaxGroup || head_dim > 256 || head_dim < 1)
        return fail(SPB_E_UNSUPPORTED, "%s: group %d / head_dim %d outside the kernel's range", name, G, head_dim);
    const int nsplit_max = (max_seq_len + kChunk - 1) / kChunk;
    const int nsplit = d_pos ? nsplit_max : (seq_len + kChunk - 1) / kChunk;
    const size_t smem = sizeof(float) * (static_cast<size_t>(G) * kChunk + (kAttnThreads / 32) * G * head_dim);
    const dim3 grid(num_kv_heads, nsplit);
    const __half* q = static_cast<const __half*>(Q);
    const __half* k = static_cast<const __half*>(K);
    const __half* v = static_cast<const __half*>(V);
    int rc = SPB_OK;
#define SPB_ATTN_CASE(GG)                                                                              \
    case GG:                                                                                           \
        if (smem > 48 * 1024)                                                                          \
            cudaFuncSetAttribute(attn_split_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                 static_cast<int>(smem));                                              \
        rc = launch(name, attn_split_kernel<GG>, grid, dim3(kAttnThreads), smem, stream, q, k, v, scratch, \
                    num_kv_heads, head_dim, max_seq_len, nsplit_max, scale, seq_len, d_pos);               \
        break;
    switch (G) {
        SPB_ATTN_CASE(1) SPB_ATTN_CASE(2) SPB_ATTN_CASE(3) SPB_ATTN_CASE(4) SPB_ATTN_CASE(5) SPB_ATTN_CASE(6)
        SPB_ATTN_CASE(7) SPB_ATTN_CASE(8)
        default: return fail(SPB_E_UNSUPPORTED, "%s: group %d", name, G);
    }
#undef SPB_ATTN_CASE
    if (rc) return rc;
    return launch("attn_combine", attn_combine_kernel, dim3(num_heads), dim3(128), 0, stream,
                  static_cast<const float*>(scratch), static_cast<__half*>(out), head_dim, nsplit_max, seq_len, d_pos);
}

size_t decode_attention_scratch_bytes(int num_heads, int head_dim, int max_seq_len) {
    return sizeof(float) * attn_scratch_floats(num_heads, head_dim, max_seq_len);
}

}  // namespace spb

using namespace spb;

extern "C" size_t spb_decode_attention_scratch_bytes(int num_heads, int head_dim, int max_seq_len) {
    if (num_heads <= 0 || head_dim <= 0 || max_seq_len <= 0) return 0;
    return decode_attention_scratch_bytes(num_heads, head_dim, max_seq_len);
}

extern "C" int spb_decode_attention_split(const void* Q, const void* K_cache, const void* V_cache, void* output,
                                          int num_heads, int num_kv_heads, int head_dim, int max_seq_len,
                                          int seq_len, float scale, void* scratch, size_t scratch_bytes,
                                          void* stream) {
    const char* name = "spb_decode_attention_split";
    if (num_heads < 0 || num_kv_heads <= 0 || head_dim <= 0) return fail(SPB_E_INVALID, "%s: bad shape", name);
    if (seq_len < 1 || seq_len > max_seq_len) return fail(SPB_E_INVALID, "%s: seq_len outside the cache", name);
    if (num_heads == 0) return SPB_OK;
    if (!Q || !K_cache || !V_cache || !output || !scratch) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (scratch_bytes < decode_attention_scratch_bytes(num_heads, head_dim, max_seq_len))
        return fail(SPB_E_INVALID, "%s: scratch of %zu bytes is smaller than spb_decode_attention_scratch_bytes()", name,
                    scratch_bytes);
    return decode_attention_split(Q, K_cache, V_cache, output, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len,
                                  nullptr, scale, static_cast<float*>(scratch), stream);
}
