#pragma once
// Drop-in replacement for the reference's include/spbitnet/sparse_ternary_kernels.h:
// the same three functions in namespace spbitnet with the same signatures, forwarding to
// the sm_100a library through its C-ABI.  Link with -lspbitnet_b200 instead of the
// reference's spbitnet_kernels.
#include <cstddef>
#include <cstdint>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "b200_check.h"

namespace spbitnet {

// reference sparse_ternary_kernels.h:16-19
inline void sparse_ternary_unpack_gpu(const uint32_t* meta, const uint32_t* values, int8_t* out, int rows,
                                      int cols, int meta_row_stride, int values_row_stride,
                                      cudaStream_t stream = nullptr) {
    SPB200_CHECK(spb_sparse_ternary_unpack(meta, values, out, rows, cols, meta_row_stride, values_row_stride, stream));
}

// reference sparse_ternary_kernels.h:29-33
inline void sparse_ternary_gemv_gpu(const uint32_t* meta, const uint32_t* values, const int8_t* x, int32_t* y,
                                    int rows, int cols, int meta_row_stride, int values_row_stride,
                                    cudaStream_t stream = nullptr) {
    SPB200_CHECK(spb_sparse_ternary_gemv(meta, values, x, y, rows, cols, meta_row_stride, values_row_stride, stream));
}

// reference sparse_ternary_kernels.h:43-48
inline void fused_sparse_bitlinear_gpu(const uint32_t* meta, const uint32_t* values, const half* x, half* output,
                                       const float* d_absmax, float gamma, int rows, int cols,
                                       int meta_row_stride, int values_row_stride, cudaStream_t stream = nullptr) {
    SPB200_CHECK(spb_fused_sparse_bitlinear(meta, values, x, output, d_absmax, gamma, rows, cols, meta_row_stride,
                                            values_row_stride, stream));
}

// Batched form; the reference names it (README.md:44) but ships no such function.  Operand
// layout of CuSparseLtGemm::execute (reference include/spbitnet/cusparselt_backend.h:47-50).
inline void sparse_ternary_gemm_gpu(const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y,
                                    int rows, int cols, int n, int meta_row_stride, int values_row_stride,
                                    cudaStream_t stream = nullptr) {
    SPB200_CHECK(spb_sparse_ternary_gemm(meta, values, X, Y, rows, cols, n, meta_row_stride, values_row_stride, stream));
}

}  // namespace spbitnet
