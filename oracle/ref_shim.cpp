// ref_shim.cpp -- extern "C" doorway onto the UNMODIFIED reference header
// include/spbitnet/sparse_ternary_tensor.h, compiled where it lies (the
// Makefile passes -I<reference>/include).  TEST INFRASTRUCTURE ONLY: it exists
// so the restatement in spb_oracle.c can be pinned against the reference's own
// code, and so the bench can time the reference's CPU path.  Output goes to
// oracle/_ref/ and is never linked into the shipped library.
#include "spbitnet/sparse_ternary_tensor.h"

#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

using spbitnet::SparseTernaryTensor;

extern "C" {

int ref_meta_stride(int cols) {
    SparseTernaryTensor t(1, cols);
    return static_cast<int>(t.meta_row_stride());
}
int ref_values_stride(int cols) {
    SparseTernaryTensor t(1, cols);
    return static_cast<int>(t.values_row_stride());
}

// SparseTernaryTensor::pack_from_dense; copies the packed words out.
void ref_pack_from_dense(const int8_t* w, const uint8_t* mask, int rows, int cols,
                         uint32_t* meta, uint32_t* values) {
    auto t = SparseTernaryTensor::pack_from_dense(w, mask, rows, cols);
    std::memcpy(meta, t.meta_data(), t.meta_size() * sizeof(uint32_t));
    std::memcpy(values, t.values_data(), t.values_size() * sizeof(uint32_t));
}

// SparseTernaryTensor::pack_with_pruning.
void ref_pack_with_pruning(const float* latent, int rows, int cols,
                           uint32_t* meta, uint32_t* values) {
    auto t = SparseTernaryTensor::pack_with_pruning(latent, rows, cols);
    std::memcpy(meta, t.meta_data(), t.meta_size() * sizeof(uint32_t));
    std::memcpy(values, t.values_data(), t.values_size() * sizeof(uint32_t));
}

// pack_from_dense followed by unpack_to_int8: the effective dense matrix.
void ref_roundtrip(const int8_t* w, const uint8_t* mask, int rows, int cols,
                   int8_t* out) {
    auto t = SparseTernaryTensor::pack_from_dense(w, mask, rows, cols);
    t.unpack_to_int8(out);
}

// The reference's CPU GEMV as its tests run it (tests/test_sparse_ternary.cu:17-33):
// unpack_to_int8 of the packed tensor, then a row-major int32 dot product.
// The tensor can only be built through the packers, so the inputs are the
// dense ternary weights and the keep-mask.  threads > 1 splits the row loop of
// the dot product into contiguous slices (no algorithmic change).
void ref_cpu_sparse_gemv(const int8_t* w, const uint8_t* mask, int rows, int cols,
                         const int8_t* x, int32_t* y, int threads, int repeats) {
    auto t = SparseTernaryTensor::pack_from_dense(w, mask, rows, cols);
    for (int rep = 0; rep < repeats; ++rep) {
        std::vector<int8_t> dense(static_cast<size_t>(rows) * cols);
        t.unpack_to_int8(dense.data());
        auto body = [&](int r0, int r1) {
            for (int r = r0; r < r1; ++r) {
                int32_t sum = 0;
                for (int c = 0; c < cols; ++c)
                    sum += static_cast<int32_t>(dense[static_cast<size_t>(r) * cols + c]) *
                           static_cast<int32_t>(x[c]);
                y[r] = sum;
            }
        };
        if (threads <= 1) {
            body(0, rows);
        } else {
            std::vector<std::thread> pool;
            for (int i = 0; i < threads; ++i)
                pool.emplace_back(body, static_cast<int>(static_cast<long>(rows) * i / threads),
                                  static_cast<int>(static_cast<long>(rows) * (i + 1) / threads));
            for (auto& th : pool) th.join();
        }
    }
}

}  // extern "C"
