// Device-side bodies of the split-KV decode attention (attention.cu), shared with the persistent decode-step
// kernel so that both form the same partial sums in the same order (every multiply-add is written as an explicit
// fmaf, so the two kernels cannot contract differently).
//
// The positions 0 .. seq_len-1 of a KV head are cut into chunks of C positions, C = attn_chunk(seq_len): 16 up to
// 512 positions, 32 beyond.  A block of kAttnThreads threads takes one (KV head, chunk): it brings the chunk's K
// and V rows and the G query vectors of the head's GQA group into shared memory with one round of 16-byte loads
// (everything in flight at once: the step is one memory round trip long), then
//   scores   warp w takes positions w, w + 8, ..: lane l the dims l, l + 32, .., shuffle reduction;
//   softmax  warp g takes head g: chunk max, exponentials, chunk sum (one position per lane);
//   output   thread t takes (head, dim) pairs t, t + 256, ..: sum over the chunk's positions in order;
// and writes the un-normalised partial result {max, sum, sum(e * V)} of every head to the scratch buffer.  The
// chunks of a head are merged with the usual log-sum-exp weights (attn_merge_group).
#pragma once
#include "ll_words.cuh"
#include "spb_common.cuh"

namespace spb {

constexpr int kAttnThreads = 256;
constexpr int kAttnMaxChunk = 32;  // positions per block, at most
constexpr int kMaxGroup = 8;       // query heads per KV head

__host__ __device__ inline int attn_chunk(int seq_len) { return seq_len <= 512 ? 16 : 32; }
__host__ __device__ inline int attn_nsplit(int seq_len) {
    const int c = attn_chunk(seq_len);
    return (seq_len + c - 1) / c;
}
// the largest number of chunks any seq_len <= max_seq_len has
__host__ __device__ inline int attn_nsplit_max(int max_seq_len) {
    const int a = attn_nsplit(max_seq_len < 512 ? max_seq_len : 512);
    const int b = max_seq_len > 512 ? attn_nsplit(max_seq_len) : 0;
    return a > b ? a : b;
}
// scratch layout: [head][split][2 + head_dim] floats = {m, l, o[0..head_dim)}
__host__ __device__ inline size_t attn_scratch_floats(int num_heads, int head_dim, int max_seq_len) {
    return static_cast<size_t>(num_heads) * attn_nsplit_max(max_seq_len) * (head_dim + 2);
}
// shared memory of a block: K and V rows of a chunk, the group's query vectors (half), the scores (float)
__host__ __device__ inline size_t attn_smem_bytes(int G, int head_dim) {
    return static_cast<size_t>(2 * kAttnMaxChunk + G) * head_dim * 2 + static_cast<size_t>(G) * kAttnMaxChunk * 4;
}

// Vectors that blocks of the same grid publish element by element (the persistent decode kernel without grid
// barriers): every 64-bit word holds two halves and the tag of the step that wrote it, stored with one 8-byte store,
// so a reader that sees the tag it expects has the data.  ll_read polls (bounded) until `n` consecutive words carry
// `tag` and returns their data words; on a run-out it sets *fail and returns what it has.
struct LlSource {
    const uint2* q;      // the query vectors: heads * head_dim / 2 words
    const uint2* k;      // the new K row of every KV head: kv heads * head_dim / 2 words
    const uint2* v;
    unsigned tag;
    int pos;             // the position the new rows belong to
    long long limit;     // cycles
    int* fail;           // shared-memory flag
};
// Work of one block on chunk `split` of KV head `kvh` (split * attn_chunk(seq_len) < seq_len).  head_dim is a
// multiple of 8 and at most 256; Q, K, V are 16-byte aligned.  They and the scratch are accessed with L2 loads
// and plain stores: in the persistent decode kernel other blocks of the same grid wrote them.
// With `ll` the query vectors and the K, V rows of position ll->pos come from tagged words instead of Q and the caches.
template <int G>
__device__ __forceinline__ void attn_chunk_block(const __half* Q, const __half* K, const __half* V, float* scratch,
                                                 int kvh, int split, int head_dim, int max_seq_len, int nsplit_max,
                                                 float scale, int seq_len, uint8_t* smem, const LlSource* ll = nullptr) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = attn_chunk(seq_len);
    const int p0 = split * C;
    const int np = min(C, seq_len - p0);
    __half* Ks = reinterpret_cast<__half*>(smem);
    __half* Vs = Ks + kAttnMaxChunk * head_dim;
    __half* Qs = Vs + kAttnMaxChunk * head_dim;
    float* sc = reinterpret_cast<float*>(Qs + G * head_dim);

    // ---- one round of loads: the chunk's rows are contiguous in the cache, the group's query vectors in Q ----
    {
        const size_t row0 = (static_cast<size_t>(kvh) * max_seq_len + p0) * head_dim;
        const uint4* kg = reinterpret_cast<const uint4*>(K + row0);
        const uint4* vg = reinterpret_cast<const uint4*>(V + row0);
        const uint4* qg = reinterpret_cast<const uint4*>(Q + static_cast<size_t>(kvh) * G * head_dim);
        const int nkv4 = np * head_dim / 8, nq4 = G * head_dim / 8;  // at most 1024 and 256
        uint4 kr[4], vr[4], qr = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * kAttnThreads;
            kr[i] = make_uint4(0, 0, 0, 0);
            vr[i] = make_uint4(0, 0, 0, 0);
            if (idx < nkv4) {
                kr[i] = __ldcg(kg + idx);
                vr[i] = __ldcg(vg + idx);
            }
        }
        if (tid < nq4 && !ll) qr = __ldcg(qg + tid);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * kAttnThreads;
            if (idx < nkv4) {
                reinterpret_cast<uint4*>(Ks)[idx] = kr[i];
                reinterpret_cast<uint4*>(Vs)[idx] = vr[i];
            }
        }
        if (tid < nq4 && !ll) reinterpret_cast<uint4*>(Qs)[tid] = qr;
    }
    __syncthreads();
    if (ll) {
        const int hw = head_dim >> 1;  // words per vector
        uint32_t* Qw = reinterpret_cast<uint32_t*>(Qs);
        for (int i = tid; i < G * hw; i += kAttnThreads) Qw[i] = ll_read1(ll->q + static_cast<size_t>(kvh) * G * hw + i, ll->tag, ll->limit, ll->fail);
        const int j = ll->pos - p0;  // the new position's row, if this chunk holds it
        if (j >= 0 && j < np) {
            if (tid < hw)
                reinterpret_cast<uint32_t*>(Ks + j * head_dim)[tid] = ll_read1(ll->k + static_cast<size_t>(kvh) * hw + tid, ll->tag, ll->limit, ll->fail);
            else if (tid < 2 * hw)
                reinterpret_cast<uint32_t*>(Vs + j * head_dim)[tid - hw] = ll_read1(ll->v + static_cast<size_t>(kvh) * hw + tid - hw, ll->tag, ll->limit, ll->fail);
        }
        __syncthreads();
    }

    // ---- scores ------------------------------------------------------------------------------------------
    {
        float qreg[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = lane + 32 * i;
                qreg[g][i] = d < head_dim ? __half2float(Qs[g * head_dim + d]) : 0.0f;
            }
        for (int j = warp; j < np; j += kAttnThreads / 32) {
            float kv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = lane + 32 * i;
                kv[i] = d < head_dim ? __half2float(Ks[j * head_dim + d]) : 0.0f;
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float acc = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc = fmaf(qreg[g][i], kv[i], acc);
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
                if (lane == 0) sc[g * kAttnMaxChunk + j] = __fmul_rn(acc, scale);
            }
        }
    }
    __syncthreads();

    // ---- per head: chunk max, exponentials, chunk sum (one position per lane) ------------------------------
    for (int g = warp; g < G; g += kAttnThreads / 32) {
        const float s = lane < np ? sc[g * kAttnMaxChunk + lane] : -1e30f;
        float m = s;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
        const float e = lane < np ? expf(s - m) : 0.0f;
        if (lane < np) sc[g * kAttnMaxChunk + lane] = e;
        float l = e;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, off);
        if (lane == 0) {
            float* dst = scratch + (static_cast<size_t>(kvh * G + g) * nsplit_max + split) * (head_dim + 2);
            dst[0] = m;
            dst[1] = l;
        }
    }
    __syncthreads();

    // ---- sum_j e[g][j] * V[j][d], positions in order -----------------------------------------------------------
    for (int t = tid; t < G * head_dim; t += kAttnThreads) {
        const int g = t / head_dim, d = t - g * head_dim;
        float o = 0.0f;
        for (int j = 0; j < np; ++j) o = fmaf(sc[g * kAttnMaxChunk + j], __half2float(Vs[j * head_dim + d]), o);
        scratch[(static_cast<size_t>(kvh * G + g) * nsplit_max + split) * (head_dim + 2) + 2 + d] = o;
    }
}

// floats of shared memory attn_merge_group needs: the weight and the sum of every (head, chunk), 1 / sum of every head
__host__ __device__ inline size_t attn_merge_smem_floats(int G, int max_seq_len) {
    return static_cast<size_t>(2 * G) * attn_nsplit_max(max_seq_len) + G;
}

// Merges the chunks of the G query heads of KV head `kvh` with the usual log-sum-exp weights and rounds to half;
// the whole block of kAttnThreads threads works on it.  sm: attn_merge_smem_floats() floats.
//   1. the chunk maxima and sums of every head into shared memory (one round of loads);
//   2. warp g takes head g: M = max, w[s] = exp(m[s] - M) into shared memory, L = sum l[s] * w[s];
//   3. thread t takes (head, dim) pairs t, t + 256, ..: sum_s w[s] * o[s][d] with eight loads in flight.
// With `fan` the result goes out as tagged words (two halves each) to every destination of the fan instead of to
// `out`; word i of a destination holds elements 2 i, 2 i + 1 of the launch's output vector.
template <int G>
__device__ __forceinline__ void attn_merge_group(const float* scratch, __half* out, int kvh, int head_dim,
                                                 int nsplit_max, int nsplit, float* sm, const LlFan* fan = nullptr,
                                                 unsigned ll_tag = 0) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t hstride = static_cast<size_t>(nsplit_max) * (head_dim + 2);
    const float* base = scratch + static_cast<size_t>(kvh) * G * hstride;
    float* w = sm;
    float* lsum = sm + G * nsplit;
    float* inv = sm + 2 * G * nsplit;
    for (int i = tid; i < G * nsplit; i += kAttnThreads) {
        const int g = i / nsplit, s = i - g * nsplit;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(base + g * hstride + static_cast<size_t>(s) * (head_dim + 2)));
        w[i] = ml.x;
        lsum[i] = ml.y;
    }
    __syncthreads();
    for (int g = warp; g < G; g += kAttnThreads / 32) {
        float M = -1e30f;
        for (int s = lane; s < nsplit; s += 32) M = fmaxf(M, w[g * nsplit + s]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, off));
        float L = 0.0f;
        for (int s = lane; s < nsplit; s += 32) {
            const float e = expf(w[g * nsplit + s] - M);
            w[g * nsplit + s] = e;
            L = fmaf(lsum[g * nsplit + s], e, L);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xFFFFFFFFu, L, off);
        if (lane == 0) inv[g] = 1.0f / L;
    }
    __syncthreads();
    // Eight loads in flight per output; a chunk index past the end is clamped (a valid address) and weighted 0.
    // (Requesting the partial rows of all of a thread's outputs at once, 32 loads in flight, was measured no faster:
    // 750 against 761 tok/s on the 2B-4T decode.)
    for (int t = tid; t < G * head_dim; t += kAttnThreads) {
        const int g = t / head_dim, d = t - g * head_dim;
        const float* ob = base + g * hstride + 2 + d;
        const float* wg = w + g * nsplit;
        float o = 0.0f;
        for (int s = 0; s < nsplit; s += 8) {
            float v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __ldcg(ob + static_cast<size_t>(min(s + k, nsplit - 1)) * (head_dim + 2));
#pragma unroll
            for (int k = 0; k < 8; ++k) o = fmaf(v[k], s + k < nsplit ? wg[s + k] : 0.0f, o);
        }
        const __half h = __float2half_rn(__fmul_rn(o, inv[g]));
        if (!fan) {
            out[(static_cast<size_t>(kvh) * G + g) * head_dim + d] = h;
        } else {  // the even dim of a pair stores both (G * head_dim is a multiple of 16: a pair is active together)
            const uint32_t mine = __half_as_ushort(h);
            const uint32_t next = __shfl_down_sync(__activemask(), mine, 1);
            if ((d & 1) == 0) ll_fan_write(*fan, ((static_cast<size_t>(kvh) * G + g) * head_dim + d) >> 1, mine | (next << 16), ll_tag);
        }
    }
}

}  // namespace spb
