// cslt_shim.cpp -- the reference's batched path (cuSPARSELt SpMMA) behind a plain C interface.
// TEST / BENCH INFRASTRUCTURE ONLY: the comparison arm of the batched product; never linked into the product.
//
// It follows the reference class spbitnet::CuSparseLtGemm step by step (src/cusparselt_backend.cu):
//   cslt_create   = the constructor, :38-106: structured A [k, m] column-major ld = k (i.e. the row-major
//                   [m, k] weight matrix) used transposed, dense B [k, n] column-major ld = k, dense C = D
//                   [m, n] column-major ld = m int32, CUSPARSE_COMPUTE_32I, default algorithm, plan, workspace;
//   cslt_prepare  = prepare(), :125-179: prune (strip), prune check, compressed size, compress;
//   cslt_execute  = execute(), :186-207: one cusparseLtMatmul, alpha = 1, beta = 0;
//   cslt_pruned   = get_pruned_weights(), :209-217.
// The reference source itself does not compile against the cuSPARSELt 0.7.1 of this image (it calls
// cusparseLtMatmulAlgSelectionDestroy, which that version does not have), hence this restatement.  Unlike
// the reference, which exits the process on a library error, every call returns 0 or the failing status.
#include <cuda_runtime.h>
#include <cusparseLt.h>

#include <cstdint>
#include <cstdio>

namespace {

struct Cslt {
    int m, k, n;
    bool prepared = false;
    cusparseLtHandle_t handle;
    cusparseLtMatDescriptor_t a, b, c;
    cusparseLtMatmulDescriptor_t matmul;
    cusparseLtMatmulAlgSelection_t alg;
    cusparseLtMatmulPlan_t plan;
    int8_t* pruned = nullptr;
    void* compressed = nullptr;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
};

char g_error[256] = "";

int lt_fail(const char* what, cusparseStatus_t st) {
    snprintf(g_error, sizeof g_error, "%s: cusparseStatus_t %d", what, static_cast<int>(st));
    return 100 + static_cast<int>(st);
}
int cu_fail(const char* what, cudaError_t e) {
    snprintf(g_error, sizeof g_error, "%s: %s", what, cudaGetErrorString(e));
    return 1000 + static_cast<int>(e);
}

#define LT(call)                                                         \
    do {                                                                 \
        cusparseStatus_t st__ = (call);                                  \
        if (st__ != CUSPARSE_STATUS_SUCCESS) return lt_fail(#call, st__); \
    } while (0)
#define CU(call)                                              \
    do {                                                      \
        cudaError_t e__ = (call);                             \
        if (e__ != cudaSuccess) return cu_fail(#call, e__);   \
    } while (0)

}  // namespace

extern "C" {

const char* cslt_last_error(void) { return g_error; }

int cslt_version(void) { return CUSPARSELT_VERSION; }  // of the header this file was compiled against

int cslt_create(int m, int k, int n, void** out) {
    if (!out || m <= 0 || k <= 0 || n < 16) {  // the reference refuses n < 16 (:41-45)
        snprintf(g_error, sizeof g_error, "cslt_create: bad arguments (n must be >= 16)");
        return 1;
    }
    Cslt* h = new Cslt();
    h->m = m; h->k = k; h->n = n;
    LT(cusparseLtInit(&h->handle));
    LT(cusparseLtStructuredDescriptorInit(&h->handle, &h->a, k, m, k, 16, CUDA_R_8I, CUSPARSE_ORDER_COL,
                                          CUSPARSELT_SPARSITY_50_PERCENT));
    LT(cusparseLtDenseDescriptorInit(&h->handle, &h->b, k, n, k, 16, CUDA_R_8I, CUSPARSE_ORDER_COL));
    LT(cusparseLtDenseDescriptorInit(&h->handle, &h->c, m, n, m, 16, CUDA_R_32I, CUSPARSE_ORDER_COL));
    LT(cusparseLtMatmulDescriptorInit(&h->handle, &h->matmul, CUSPARSE_OPERATION_TRANSPOSE,
                                      CUSPARSE_OPERATION_NON_TRANSPOSE, &h->a, &h->b, &h->c, &h->c,
                                      CUSPARSE_COMPUTE_32I));
    LT(cusparseLtMatmulAlgSelectionInit(&h->handle, &h->alg, &h->matmul, CUSPARSELT_MATMUL_ALG_DEFAULT));
    LT(cusparseLtMatmulPlanInit(&h->handle, &h->plan, &h->matmul, &h->alg));
    LT(cusparseLtMatmulGetWorkspace(&h->handle, &h->plan, &h->workspace_bytes));
    if (h->workspace_bytes) CU(cudaMalloc(&h->workspace, h->workspace_bytes));
    *out = h;
    return 0;
}

void cslt_destroy(void* p) {
    Cslt* h = static_cast<Cslt*>(p);
    if (!h) return;
    cudaFree(h->pruned);
    cudaFree(h->compressed);
    cudaFree(h->workspace);
    cusparseLtMatmulPlanDestroy(&h->plan);
    cusparseLtMatDescriptorDestroy(&h->a);
    cusparseLtMatDescriptorDestroy(&h->b);
    cusparseLtMatDescriptorDestroy(&h->c);
    cusparseLtDestroy(&h->handle);
    delete h;
}

// d_weights: dense int8 [m, k] row-major.  Returns 2 when the pruned matrix fails the library's 2:4 check.
int cslt_prepare(void* p, const int8_t* d_weights, void* stream_) {
    Cslt* h = static_cast<Cslt*>(p);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const size_t bytes = static_cast<size_t>(h->m) * h->k;
    if (!h->pruned) CU(cudaMalloc(reinterpret_cast<void**>(&h->pruned), bytes));
    LT(cusparseLtSpMMAPrune(&h->handle, &h->matmul, d_weights, h->pruned, CUSPARSELT_PRUNE_SPMMA_STRIP, stream));
    int* d_valid = nullptr;
    CU(cudaMalloc(reinterpret_cast<void**>(&d_valid), sizeof(int)));
    LT(cusparseLtSpMMAPruneCheck(&h->handle, &h->matmul, h->pruned, d_valid, stream));
    int valid = 0;
    CU(cudaMemcpyAsync(&valid, d_valid, sizeof(int), cudaMemcpyDeviceToHost, stream));
    CU(cudaStreamSynchronize(stream));
    cudaFree(d_valid);
    if (valid != 0) {
        snprintf(g_error, sizeof g_error, "cslt_prepare: the pruned matrix is not 2:4");
        return 2;
    }
    size_t csize = 0, cbuf = 0;
    LT(cusparseLtSpMMACompressedSize(&h->handle, &h->plan, &csize, &cbuf));
    cudaFree(h->compressed);
    h->compressed = nullptr;
    CU(cudaMalloc(&h->compressed, csize));
    void* tmp = nullptr;
    if (cbuf) CU(cudaMalloc(&tmp, cbuf));
    LT(cusparseLtSpMMACompress(&h->handle, &h->plan, h->pruned, h->compressed, tmp, stream));
    CU(cudaStreamSynchronize(stream));
    cudaFree(tmp);
    h->prepared = true;
    return 0;
}

// d_B: int8 [k, n] column-major (n activation rows of k); d_D: int32 [m, n] column-major (n rows of m).
int cslt_execute(void* p, const int8_t* d_B, int32_t* d_D, void* stream_) {
    Cslt* h = static_cast<Cslt*>(p);
    if (!h->prepared) {
        snprintf(g_error, sizeof g_error, "cslt_execute: prepare() has not run");
        return 3;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const float alpha = 1.0f, beta = 0.0f;
    LT(cusparseLtMatmul(&h->handle, &h->plan, &alpha, h->compressed, d_B, &beta, d_D, d_D, h->workspace, &stream, 1));
    return 0;
}

int cslt_pruned(void* p, int8_t* d_out, void* stream_) {
    Cslt* h = static_cast<Cslt*>(p);
    if (!h->prepared) return 3;
    CU(cudaMemcpyAsync(d_out, h->pruned, static_cast<size_t>(h->m) * h->k, cudaMemcpyDeviceToDevice,
                       static_cast<cudaStream_t>(stream_)));
    return 0;
}

}  // extern "C"
