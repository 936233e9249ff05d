// Magnitude 2:4 pruning + ternary sign extraction + packing of a float32 weight matrix on the GPU,
// byte-identical to the reference's converter (python/convert_model.py:88-138 generate_24_mask and
// quantize_ternary_absmean, :270-283 the zero-at-mask fix, :141-207 pack_sparse_ternary).
//
// What the converter's five steps come to, per group of four consecutive weights of a row:
//   * kept positions = the two largest |w|; on equal magnitudes the HIGHER index is kept (a stable ascending
//     argsort leaves equal elements in index order and the top two are taken from its end);
//   * a kept weight packs as -1 exactly when w < 0: RoundClip(w / gamma) of a negative weight is -1 or 0, a
//     kept 0 is forced to the sign of w, and w >= 0 (including -0.0) packs as +1 — so the packed bits do not
//     depend on gamma at all;
//   * gamma = mean |w| goes to the manifest only.  It is accumulated here in double precision (optional);
//     numpy's float32 pairwise sum can differ from it in the last bits, so a caller that needs the manifest
//     byte-identical computes gamma with numpy.
// A thread packs 16 groups (64 weights): two bitmap words and one sign word.
#include "spb_common.cuh"

namespace spb {

constexpr int kPackThreads = 256;

__global__ void __launch_bounds__(kPackThreads) prune_pack_kernel(const float* __restrict__ w, int rows, int cols,
                                                                  size_t w_row_stride, uint32_t* __restrict__ meta,
                                                                  uint32_t* __restrict__ values, int meta_stride,
                                                                  int values_stride, double* __restrict__ abs_sum) {
    grid_dep_launch();
    grid_dep_wait();
    const int groups = cols >> 2, tpr = (groups + 15) >> 4;  // threads per row
    const long long t = static_cast<long long>(blockIdx.x) * kPackThreads + threadIdx.x;
    double local = 0.0;
    if (t < static_cast<long long>(rows) * tpr) {
        const int row = static_cast<int>(t / tpr), tc = static_cast<int>(t - static_cast<long long>(row) * tpr);
        const float* src = w + static_cast<size_t>(row) * w_row_stride + static_cast<size_t>(tc) * 64;
        const int ng = min(16, groups - tc * 16);
        uint32_t m0 = 0, m1 = 0, sg = 0;
        const bool vec = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
#pragma unroll 4
        for (int g = 0; g < ng; ++g) {
            float v[4];
            if (vec) {
                const float4 f = *reinterpret_cast<const float4*>(src + 4 * g);
                v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = src[4 * g + i];
            }
            float a[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = fabsf(v[i]);
                local += static_cast<double>(a[i]);
            }
            // rank of element i in the stable ascending order = how many elements sort before it
            uint32_t bitmap = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int before = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) before += (a[j] < a[i]) || (a[j] == a[i] && j < i);
                if (before >= 2) bitmap |= 1u << i;  // the last two of the order are kept
            }
            // sign pair: bit 0 = lower kept index, bit 1 = higher kept index; 1 = negative
            uint32_t signs = 0;
            int seen = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (bitmap & (1u << i)) {
                    if (v[i] < 0.0f) signs |= 1u << seen;
                    ++seen;
                }
            }
            if (g < 8) m0 |= bitmap << (4 * g); else m1 |= bitmap << (4 * (g - 8));
            sg |= signs << (2 * g);
        }
        uint32_t* mrow = meta + static_cast<size_t>(row) * meta_stride + 2 * tc;
        mrow[0] = m0;
        if (ng > 8) mrow[1] = m1;
        values[static_cast<size_t>(row) * values_stride + tc] = sg;
    }
    if (abs_sum) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) local += __shfl_xor_sync(0xFFFFFFFFu, local, off);
        if ((threadIdx.x & 31) == 0 && local != 0.0) atomicAdd(abs_sum, local);
    }
}

}  // namespace spb

using namespace spb;

extern "C" int spb_prune_pack_gpu(const float* weights, int rows, int cols, size_t weights_row_stride, uint32_t* meta,
                                  uint32_t* values, int meta_row_stride, int values_row_stride, double* abs_sum,
                                  void* stream) {
    const char* name = "spb_prune_pack_gpu";
    if (rows < 0 || cols < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    if (rows == 0 || cols == 0) return SPB_OK;
    if (cols % 4 != 0) return fail(SPB_E_INVALID, "%s: cols=%d is not a multiple of 4", name, cols);
    if (!weights || !meta || !values) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (weights_row_stride < static_cast<size_t>(cols)) return fail(SPB_E_INVALID, "%s: row stride shorter than a row", name);
    if (meta_row_stride < (cols / 4 + 7) / 8 || values_row_stride < (cols / 4 + 15) / 16)
        return fail(SPB_E_INVALID, "%s: row stride shorter than a row", name);
    const long long threads = static_cast<long long>(rows) * ((cols / 4 + 15) / 16);
    const unsigned grid = static_cast<unsigned>((threads + kPackThreads - 1) / kPackThreads);
    return launch(name, prune_pack_kernel, dim3(grid), dim3(kPackThreads), 0, stream, weights, rows, cols, weights_row_stride,
                  meta, values, meta_row_stride, values_row_stride, abs_sum);
}
