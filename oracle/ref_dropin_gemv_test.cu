// ref_dropin_gemv_test.cu -- a C++ program written against the reference's own API only: the reference's
// SparseTernaryTensor header (packing, CPU unpack) and the kernel wrapper spbitnet::sparse_ternary_gemv_gpu,
// the latter taken from THIS repository's drop-in header (the include path puts it first) and linked with
// libspbitnet_b200.so.  It replays the flow of the reference's exact-equality GEMV tests
// (tests/test_sparse_ternary.cu:252-324 and :330-402): seeded weights and mask from testgen.cpp, pack with the
// reference header, GPU GEMV through the drop-in wrapper with default arguments (null stream), compare every row
// with unpack_to_int8 + int32 dot.  Exit code 0 = every row equal.  TEST INFRASTRUCTURE ONLY.
#include <cstdint>
#include <cstdio>
#include <vector>

#include <cuda_runtime.h>

#include "spbitnet/sparse_ternary_kernels.h"
#include "spbitnet/sparse_ternary_tensor.h"

extern "C" void testgen_gemv_case(unsigned seed, int rows, int cols, int xlo, int xhi, int8_t* weights,
                                  uint8_t* mask, int8_t* x);

static int run_case(unsigned seed, int rows, int cols) {
    std::vector<int8_t> w(static_cast<size_t>(rows) * cols), x(cols);
    std::vector<uint8_t> mask(w.size());
    testgen_gemv_case(seed, rows, cols, -5, 5, w.data(), mask.data(), x.data());
    auto t = spbitnet::SparseTernaryTensor::pack_from_dense(w.data(), mask.data(), rows, cols);
    std::vector<int8_t> dense(w.size());
    t.unpack_to_int8(dense.data());
    uint32_t *d_meta = nullptr, *d_values = nullptr;
    int8_t* d_x = nullptr;
    int32_t* d_y = nullptr;
    const size_t mb = t.meta_size() * sizeof(uint32_t), vb = t.values_size() * sizeof(uint32_t);
    if (cudaMalloc(&d_meta, mb) || cudaMalloc(&d_values, vb) || cudaMalloc(&d_x, cols) || cudaMalloc(&d_y, 4 * rows)) return 2;
    cudaMemcpy(d_meta, t.meta_data(), mb, cudaMemcpyHostToDevice);
    cudaMemcpy(d_values, t.values_data(), vb, cudaMemcpyHostToDevice);
    cudaMemcpy(d_x, x.data(), cols, cudaMemcpyHostToDevice);
    cudaMemset(d_y, 0, 4 * rows);
    spbitnet::sparse_ternary_gemv_gpu(d_meta, d_values, d_x, d_y, rows, cols, static_cast<int>(t.meta_row_stride()),
                                      static_cast<int>(t.values_row_stride()));
    if (cudaDeviceSynchronize() != cudaSuccess) return 3;
    std::vector<int32_t> y(rows);
    cudaMemcpy(y.data(), d_y, 4 * rows, cudaMemcpyDeviceToHost);
    int bad = 0;
    for (int r = 0; r < rows; ++r) {
        int32_t sum = 0;
        for (int c = 0; c < cols; ++c) sum += static_cast<int32_t>(dense[static_cast<size_t>(r) * cols + c]) * x[c];
        if (sum != y[r] && bad++ < 5) std::fprintf(stderr, "seed %u row %d: expected %d, got %d\n", seed, r, sum, y[r]);
    }
    cudaFree(d_meta); cudaFree(d_values); cudaFree(d_x); cudaFree(d_y);
    std::printf("seed %u %dx%d: %s\n", seed, rows, cols, bad ? "MISMATCH" : "exact");
    return bad ? 1 : 0;
}

int main() {
    int rc = run_case(42u, 64, 256);
    rc |= run_case(77u, 2048, 2048);
    return rc;
}
