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

// The same CPU GEMV with the row range cut into `slices` contiguous parts, one thread each, every part a
// SparseTernaryTensor of its own (packed once, outside any timing) that its thread unpacks with the reference's
// unpack_to_int8 and multiplies with the loop of tests/test_sparse_ternary.cu:24-32.  No algorithmic change:
// slices = 1 is the function above without the repeated allocation.
//   mode 0: every repeat unpacks and multiplies (the reference's cpu_sparse_gemv, partitioned);
//   mode 1: the slices are unpacked once up front and every repeat only multiplies (dot product only).
struct RefGemvCtx {
    int rows, cols;
    std::vector<SparseTernaryTensor> part;
    std::vector<int> r0;
    std::vector<std::vector<int8_t>> dense;
};

void* ref_gemv_ctx_create(const int8_t* w, const uint8_t* mask, int rows, int cols, int slices) {
    if (slices < 1) slices = 1;
    if (slices > rows) slices = rows;
    auto* ctx = new RefGemvCtx{rows, cols, {}, {}, {}};
    for (int i = 0; i < slices; ++i) {
        const int a = static_cast<int>(static_cast<long>(rows) * i / slices);
        const int b = static_cast<int>(static_cast<long>(rows) * (i + 1) / slices);
        ctx->r0.push_back(a);
        ctx->part.push_back(SparseTernaryTensor::pack_from_dense(w + static_cast<size_t>(a) * cols,
                                                                 mask + static_cast<size_t>(a) * cols, b - a, cols));
        ctx->dense.emplace_back(static_cast<size_t>(b - a) * cols);
    }
    ctx->r0.push_back(rows);
    return ctx;
}

void ref_gemv_ctx_destroy(void* p) { delete static_cast<RefGemvCtx*>(p); }

void ref_gemv_ctx_run(void* p, const int8_t* x, int32_t* y, int repeats, int mode) {
    RefGemvCtx* ctx = static_cast<RefGemvCtx*>(p);
    const int cols = ctx->cols, slices = static_cast<int>(ctx->part.size());
    auto body = [&](int i) {
        int8_t* dense = ctx->dense[i].data();
        const int nrows = ctx->r0[i + 1] - ctx->r0[i];
        if (mode == 1) ctx->part[i].unpack_to_int8(dense);
        for (int rep = 0; rep < repeats; ++rep) {
            if (mode == 0) ctx->part[i].unpack_to_int8(dense);
            for (int r = 0; r < nrows; ++r) {
                int32_t sum = 0;
                for (int c = 0; c < cols; ++c)
                    sum += static_cast<int32_t>(dense[static_cast<size_t>(r) * cols + c]) * static_cast<int32_t>(x[c]);
                y[ctx->r0[i] + r] = sum;
            }
        }
    };
    if (slices == 1) {
        body(0);
        return;
    }
    std::vector<std::thread> pool;
    for (int i = 0; i < slices; ++i) pool.emplace_back(body, i);
    for (auto& th : pool) th.join();
}

}  // extern "C"
