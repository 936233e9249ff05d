// Batched sparse-ternary product Y[n, rows] = X[n, cols] * W^T for sm_100a.
//
// The reference has no kernel of its own for this; its batched path hands a dense
// int8 copy of the weights to cuSPARSELt (src/cusparselt_backend.cu:186-207).  Here
// the compressed format is consumed directly.  This file holds the SIMT form used
// for small batches: every thread decodes its unit (128 columns of one row) once
// into 32 packed int8x4 weight words held in registers and replays them against
// kBatchTile activation rows staged in shared memory, so the weight stream is read
// from HBM once per kBatchTile rows.
#include "spb_common.cuh"

namespace spb {

constexpr int kGemmThreads = 256;
constexpr int kBatchTile = 8;

struct GemmArgs {
    const uint32_t* meta;
    const uint32_t* values;
    const int8_t* X;  // [n, cols]
    int32_t* Y;       // [n, rows]
    int rows, cols, n;
    int meta_stride, values_stride;
    int upr, rpc;
};

template <int U>
__global__ void __launch_bounds__(kGemmThreads) gemm_units_kernel(const GemmArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem);
    int* rowacc = reinterpret_cast<int*>(smem + kLutBytes);  // [rpc][kBatchTile]
    uint4* xs = reinterpret_cast<uint4*>(smem + kLutBytes + ((a.rpc * kBatchTile * 4 + 15) & ~15));

    const int tid = threadIdx.x, lane = tid & 31;
    const int r_lo = blockIdx.x * a.rpc;
    const int nrows = min(a.rpc, a.rows - r_lo);
    const int nunits = nrows * a.upr;
    const int j_lo = blockIdx.y * kBatchTile;
    const int nb = min(kBatchTile, a.n - j_lo);
    const int chunks_per_row = a.cols >> 4;

    grid_dep_launch();

    uint4 m[U];
    uint2 v[U];
    int rl[U], cb[U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
        const int u = tid + i * kGemmThreads;
        if (u < nunits) {
            rl[i] = u / a.upr;
            cb[i] = u - rl[i] * a.upr;
            const size_t row = static_cast<size_t>(r_lo + rl[i]);
            m[i] = ld_stream_v4(a.meta + row * a.meta_stride + cb[i] * 4);
            v[i] = ld_stream_v2(a.values + row * a.values_stride + cb[i] * 2);
        } else {
            rl[i] = -1;
            cb[i] = a.upr;
            m[i] = make_uint4(0, 0, 0, 0);
            v[i] = make_uint2(0, 0);
        }
    }
    fill_lane_lut(lut, tid, kGemmThreads);
    for (int e = tid; e < nrows * kBatchTile; e += kGemmThreads) rowacc[e] = 0;

    grid_dep_wait();
    for (int q = tid; q < nb * chunks_per_row; q += kGemmThreads) {
        const int jj = q / chunks_per_row, qq = q - jj * chunks_per_row;
        const int c = qq >> 3, i = qq & 7;
        xs[jj * chunks_per_row + (c << 3) + (i ^ (c & 7))] =
            reinterpret_cast<const uint4*>(a.X + static_cast<size_t>(j_lo + jj) * a.cols)[qq];
    }
    __syncthreads();

    const uint32_t* lutp = lut + lane;
#pragma unroll
    for (int i = 0; i < U; ++i) {
        // decode the unit once
        uint32_t wt[32];
        const uint32_t mw[4] = {m[i].x, m[i].y, m[i].z, m[i].w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t vv = (w < 2) ? v[i].x : v[i].y;
            const uint32_t sg = (w & 1) ? (vv >> 16) : vv;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const uint32_t idx = ((mw[w] >> (4 * g)) & 0xFu) | (((sg >> (2 * g)) & 0x3u) << 4);
                wt[w * 8 + g] = lutp[idx * 32];
            }
        }
        const int sw = cb[i] & 7;
        for (int jj = 0; jj < nb; ++jj) {
            int part = 0;
            if (rl[i] >= 0) {
                const uint4* xb = xs + jj * chunks_per_row + (cb[i] << 3);
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    const uint4 xv = xb[ch ^ sw];
                    part = __dp4a(static_cast<int>(wt[ch * 4 + 0]), static_cast<int>(xv.x), part);
                    part = __dp4a(static_cast<int>(wt[ch * 4 + 1]), static_cast<int>(xv.y), part);
                    part = __dp4a(static_cast<int>(wt[ch * 4 + 2]), static_cast<int>(xv.z), part);
                    part = __dp4a(static_cast<int>(wt[ch * 4 + 3]), static_cast<int>(xv.w), part);
                }
            }
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int other = __shfl_down_sync(0xFFFFFFFFu, part, off);
                if (lane + off < 32 && cb[i] + off < a.upr) part += other;
            }
            if (rl[i] >= 0 && (cb[i] == 0 || lane == 0)) atomicAdd(&rowacc[rl[i] * kBatchTile + jj], part);
        }
    }
    __syncthreads();
    for (int t = tid; t < nrows * nb; t += kGemmThreads) {
        const int jj = t / nrows, r = t - jj * nrows;
        a.Y[static_cast<size_t>(j_lo + jj) * a.rows + r_lo + r] = rowacc[r * kBatchTile + jj];
    }
}

// Any layout: a warp per (row, batch row).  Correctness path only.
__global__ void __launch_bounds__(kGemmThreads) gemm_generic_kernel(const GemmArgs a) {
    grid_dep_launch();
    grid_dep_wait();
    const int lane = threadIdx.x & 31;
    const long long wid = (static_cast<long long>(blockIdx.x) * kGemmThreads + threadIdx.x) >> 5;
    if (wid >= static_cast<long long>(a.rows) * a.n) return;
    const int j = static_cast<int>(wid / a.rows), row = static_cast<int>(wid % a.rows);
    const uint32_t* mrow = a.meta + static_cast<size_t>(row) * a.meta_stride;
    const uint32_t* vrow = a.values + static_cast<size_t>(row) * a.values_stride;
    const int8_t* x = a.X + static_cast<size_t>(j) * a.cols;
    int acc = 0;
    for (int g = lane; g < (a.cols >> 2); g += 32) {
        const uint32_t bitmap = (mrow[g >> 3] >> ((g & 7) * 4)) & 0xFu;
        const uint32_t signs = (vrow[g >> 4] >> ((g & 15) * 2)) & 0x3u;
        const uint32_t wt = c_group_lut.w[bitmap | (signs << 4)];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc += static_cast<int8_t>(wt >> (8 * i)) * static_cast<int>(x[4 * g + i]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    if (lane == 0) a.Y[static_cast<size_t>(j) * a.rows + row] = acc;
}

int gemm_tcsp_ws_launch(const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y, int rows, int cols,
                        int n, int meta_stride, int values_stride, void* stream, const GemmEpilogue* ep);
// prefill.cu
int dequantize_rows(const int32_t* acc, void* out, const float* d_absmax, float gamma, int rows, int vectors,
                    void* stream);
bool gemm_mmasp_supported(const uint32_t* meta, const uint32_t* values, const int8_t* X, int rows, int cols, int n,
                          int meta_stride, int values_stride, int max_n);
int gemm_mmasp_launch(const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y, int rows, int cols,
                      int n, int meta_stride, int values_stride, void* stream, const GemmEpilogue* ep);

// 0 automatic (up to 32 batch rows: warp-level sparse MMA form; above: tcgen05 sparse form; SIMT where the layout
// allows neither), 1 SIMT form, 3 tcgen05 sparse form, 4 warp-level sparse MMA form (3 and 4 whenever the layout
// allows)
static int g_gemm_variant = 0;
constexpr int kMmaSpAutoMaxN = 32;

}  // namespace spb

using namespace spb;

extern "C" int spb_set_gemm_variant(int variant) {
    const int old = g_gemm_variant;
    g_gemm_variant = variant;
    return old;
}

// The batched product.  With `ep` the output is the scaled half matrix: the two default forms write it from their
// own epilogues (Y unused); every other form leaves the sums in Y, which must then be a workspace of n * rows
// int32, and a per-row dequantise follows on the same stream.
static int gemm_dispatch(const char* name, const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y,
                         int rows, int cols, int n, int meta_row_stride, int values_row_stride, void* stream,
                         const GemmEpilogue* ep);
static int gemm_dispatch_int(const char* name, const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y,
                             int rows, int cols, int n, int meta_row_stride, int values_row_stride, void* stream,
                             bool fast);

extern "C" int spb_sparse_ternary_gemm(const uint32_t* meta, const uint32_t* values, const int8_t* X,
                                       int32_t* Y, int rows, int cols, int n, int meta_row_stride,
                                       int values_row_stride, void* stream) {
    const char* name = "spb_sparse_ternary_gemm";
    if (rows < 0 || cols < 0 || n < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    if (rows == 0 || cols == 0 || n == 0) return SPB_OK;
    if (!Y) return fail(SPB_E_INVALID, "%s: null pointer", name);
    return gemm_dispatch(name, meta, values, X, Y, rows, cols, n, meta_row_stride, values_row_stride, stream, nullptr);
}

extern "C" int spb_sparse_bitlinear_gemm(const uint32_t* meta, const uint32_t* values, const int8_t* Xq, void* output,
                                         const float* d_absmax, float gamma, int32_t* acc_workspace, int rows,
                                         int cols, int n, int meta_row_stride, int values_row_stride, void* stream) {
    const char* name = "spb_sparse_bitlinear_gemm";
    if (rows < 0 || cols < 0 || n < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    if (rows == 0 || cols == 0 || n == 0) return SPB_OK;
    if (!output || !d_absmax) return fail(SPB_E_INVALID, "%s: null pointer", name);
    const GemmEpilogue ep{static_cast<__half*>(output), d_absmax, gamma};
    return gemm_dispatch(name, meta, values, Xq, acc_workspace, rows, cols, n, meta_row_stride, values_row_stride,
                         stream, &ep);
}

static int gemm_dispatch(const char* name, const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y,
                         int rows, int cols, int n, int meta_row_stride, int values_row_stride, void* stream,
                         const GemmEpilogue* ep) {
    if (cols % 4 != 0) return fail(SPB_E_INVALID, "%s: cols=%d is not a multiple of 4", name, cols);
    if (!meta || !values || !X) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (meta_row_stride < (cols / 4 + 7) / 8 || values_row_stride < (cols / 4 + 15) / 16)
        return fail(SPB_E_INVALID, "%s: row stride shorter than a row", name);
    auto al = [](const void* p, size_t k) { return (reinterpret_cast<uintptr_t>(p) & (k - 1)) == 0; };
    const bool fast = cols % 128 == 0 && cols / 128 <= 512 && meta_row_stride % 4 == 0 &&
                      values_row_stride % 2 == 0 && al(meta, 16) && al(values, 8) && al(X, 16);
    // up to 32 batch rows the warp-level form always wins; up to 64 it still does when the tcgen05 form, with
    // its tiles of 128 weight rows, would leave most SMs idle (measured at 2560x6912: 18.8 against 30.1 us)
    const int mma_auto_max_n = (rows + 127) / 128 < sm_count() / 4 ? 64 : kMmaSpAutoMaxN;
    if ((g_gemm_variant == 0 || g_gemm_variant == 4) &&
        gemm_mmasp_supported(meta, values, X, rows, cols, n, meta_row_stride, values_row_stride,
                             g_gemm_variant == 4 ? 4096 : mma_auto_max_n))
        return gemm_mmasp_launch(meta, values, X, Y, rows, cols, n, meta_row_stride, values_row_stride, stream, ep);
    if (fast && g_gemm_variant != 1) {  // warp-specialised tcgen05 sparse form
        const int rc = gemm_tcsp_ws_launch(meta, values, X, Y, rows, cols, n, meta_row_stride, values_row_stride, stream, ep);
        if (rc != SPB_E_UNSUPPORTED) return rc;  // no tensor map of X on this system: the SIMT form below
    }
    if (ep) {  // the SIMT forms write int32 sums: run them into the workspace, then scale row by row
        if (!Y) return fail(SPB_E_UNSUPPORTED, "%s: this layout needs acc_workspace (n * rows int32)", name);
        const int rc = gemm_dispatch_int(name, meta, values, X, Y, rows, cols, n, meta_row_stride, values_row_stride, stream,
                                         fast);
        if (rc) return rc;
        return dequantize_rows(Y, ep->out, ep->absmax, ep->gamma, rows, n, stream);
    }
    return gemm_dispatch_int(name, meta, values, X, Y, rows, cols, n, meta_row_stride, values_row_stride, stream, fast);
}

// The SIMT forms (no fused epilogue).
static int gemm_dispatch_int(const char* name, const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y,
                             int rows, int cols, int n, int meta_row_stride, int values_row_stride, void* stream,
                             bool fast) {
    GemmArgs a{meta, values, X, Y, rows, cols, n, meta_row_stride, values_row_stride, 0, 0};
    const size_t x_bytes = static_cast<size_t>(kBatchTile) * cols;
    if (!fast) {
        const long long warps = static_cast<long long>(rows) * n;
        const unsigned grid = static_cast<unsigned>((warps * 32 + kGemmThreads - 1) / kGemmThreads);
        return launch(name, gemm_generic_kernel, dim3(grid), dim3(kGemmThreads), 0, stream, a);
    }
    const int sms = sm_count();
    a.upr = cols / 128;
    const int rpc_cap = max(1, 512 / a.upr);
    const int fill = max(1, kGemmThreads / a.upr);
    int rpc = max((rows + 4 * sms - 1) / (4 * sms), min(fill, (rows + sms - 1) / sms));
    a.rpc = max(1, min(rpc, rpc_cap));
    const int passes = (a.rpc * a.upr + kGemmThreads - 1) / kGemmThreads;
    if (x_bytes > 160 * 1024) {
        const long long warps = static_cast<long long>(rows) * n;
        const unsigned grid1 = static_cast<unsigned>((warps * 32 + kGemmThreads - 1) / kGemmThreads);
        return launch(name, gemm_generic_kernel, dim3(grid1), dim3(kGemmThreads), 0, stream, a);
    }
    const dim3 grid((rows + a.rpc - 1) / a.rpc, (n + kBatchTile - 1) / kBatchTile);
    const size_t smem = kLutBytes + ((a.rpc * kBatchTile * 4 + 15) & ~15) + x_bytes;
    auto kernel = passes <= 1 ? gemm_units_kernel<1> : gemm_units_kernel<2>;
    if (int rc = ensure_dynamic_smem(name, kernel, smem)) return rc;
    return launch(name, kernel, dim3(grid), dim3(kGemmThreads), smem, stream, a);
}
