// sparse_ternary_unpack_gpu for sm_100a (reference: src/kernels/sparse_ternary.cu:58-102,
// 240-254): compressed -> dense int8, row-major.  One thread expands one meta word
// (8 groups, 32 columns) into two 16-byte stores when the output rows allow it; a
// thread-per-group path with 4-byte stores covers every other layout.
#include "spb_common.cuh"

namespace spb {

__global__ void __launch_bounds__(256) unpack_words_kernel(const uint32_t* __restrict__ meta,
                                                           const uint32_t* __restrict__ values,
                                                           int8_t* __restrict__ out, int rows, int cols,
                                                           int meta_stride, int values_stride) {
    grid_dep_launch();
    grid_dep_wait();
    const int wpr = cols >> 5;  // meta words per row (cols % 32 == 0 on this path)
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= static_cast<long long>(rows) * wpr) return;
    const int row = static_cast<int>(t / wpr), w = static_cast<int>(t % wpr);
    const uint32_t m = meta[static_cast<size_t>(row) * meta_stride + w];
    const uint32_t vv = values[static_cast<size_t>(row) * values_stride + (w >> 1)];
    const uint32_t sg = (w & 1) ? (vv >> 16) : vv;
    uint32_t o[8];
#pragma unroll
    for (int g = 0; g < 8; ++g)
        o[g] = c_group_lut.w[((m >> (4 * g)) & 0xFu) | (((sg >> (2 * g)) & 0x3u) << 4)];
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * cols + (static_cast<size_t>(w) << 5));
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

__global__ void __launch_bounds__(256) unpack_groups_kernel(const uint32_t* __restrict__ meta,
                                                            const uint32_t* __restrict__ values,
                                                            int8_t* __restrict__ out, int rows, int cols,
                                                            int meta_stride, int values_stride,
                                                            int word_stores) {
    grid_dep_launch();
    grid_dep_wait();
    const int gpr = cols >> 2;
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= static_cast<long long>(rows) * gpr) return;
    const int row = static_cast<int>(t / gpr), g = static_cast<int>(t % gpr);
    const uint32_t bitmap = (meta[static_cast<size_t>(row) * meta_stride + (g >> 3)] >> ((g & 7) * 4)) & 0xFu;
    const uint32_t signs = (values[static_cast<size_t>(row) * values_stride + (g >> 4)] >> ((g & 15) * 2)) & 0x3u;
    const uint32_t word = c_group_lut.w[bitmap | (signs << 4)];
    int8_t* dst = out + static_cast<size_t>(row) * cols + (static_cast<size_t>(g) << 2);
    if (word_stores) {
        *reinterpret_cast<uint32_t*>(dst) = word;
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = static_cast<int8_t>(word >> (8 * i));
    }
}

}  // namespace spb

using namespace spb;

extern "C" int spb_sparse_ternary_unpack(const uint32_t* meta, const uint32_t* values, int8_t* out,
                                         int rows, int cols, int meta_row_stride,
                                         int values_row_stride, void* stream) {
    const char* name = "spb_sparse_ternary_unpack";
    if (rows < 0 || cols < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    if (rows == 0 || cols == 0) return SPB_OK;
    if (cols % 4 != 0) return fail(SPB_E_INVALID, "%s: cols=%d is not a multiple of 4", name, cols);
    if (!meta || !values || !out) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (meta_row_stride < (cols / 4 + 7) / 8 || values_row_stride < (cols / 4 + 15) / 16)
        return fail(SPB_E_INVALID, "%s: row stride shorter than a row", name);
    const uintptr_t o = reinterpret_cast<uintptr_t>(out);
    if (cols % 32 == 0 && (o & 15) == 0) {
        const long long n = static_cast<long long>(rows) * (cols / 32);
        return launch(name, unpack_words_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0,
                      stream, meta, values, out, rows, cols, meta_row_stride, values_row_stride);
    }
    const long long n = static_cast<long long>(rows) * (cols / 4);
    return launch(name, unpack_groups_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0,
                  stream, meta, values, out, rows, cols, meta_row_stride, values_row_stride,
                  static_cast<int>((o & 3) == 0));
}
