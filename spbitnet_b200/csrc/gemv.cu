// Sparse-ternary GEMV / BitLinear for sm_100a.
//
// Replaces sparse_ternary_gemv_gpu and fused_sparse_bitlinear_gpu of the reference
// (src/kernels/sparse_ternary.cu:116-234,256-291).  The reference walks one group
// per lane per step with scalar word loads, a lane-divergent constant-memory table
// and byte gathers from global memory.  This kernel instead
//   * reads the two weight streams with one 128-bit (meta: 32 groups) and one
//     64-bit (values: 32 groups) load per thread, issued before anything else so
//     that they are in flight while the block sets up and, under programmatic
//     dependent launch, while the previous kernel on the stream drains;
//   * stages the activation vector once per block in shared memory as int8
//     (quantising it on the way when the input is half), in 16-byte chunks whose
//     position is XOR-swizzled so that the per-thread 128-byte reads are
//     conflict free;
//   * turns (bitmap, sign pair) into the four int8 weights of a group with a
//     64-entry table replicated once per lane in shared memory (bank = lane, no
//     conflicts) and consumes a group with one dp4a;
//   * reduces the per-thread partials of a row with a segmented shuffle scan.
// A "unit" is 128 consecutive columns of one row: 16 B of meta + 8 B of values.
#include "spb_common.cuh"

namespace spb {

enum { IN_I8 = 0, IN_F16 = 1 };
enum { OUT_I32 = 0, OUT_F32 = 1, OUT_F16 = 2 };

struct GemvArgs {
    const uint32_t* meta;
    const uint32_t* values;
    const void* x;         // int8 (IN_I8) or half (IN_F16), cols elements
    void* y;               // int32 / float / half, rows elements
    int32_t* y_acc;        // optional int32 copy of the accumulators (OUT_F32)
    const float* d_absmax; // device scalar; read after the dependency wait
    float gamma;
    int rows, cols;
    int meta_stride, values_stride;  // uint32 words
    int upr;                         // units per row = cols / 128
    int rpc;                         // rows per block
};

constexpr int kThreads = 256;

__device__ __forceinline__ void store_out(const GemvArgs& a, int row, int acc, float dq, int out_mode) {
    if (out_mode == OUT_I32) {
        static_cast<int32_t*>(a.y)[row] = acc;
    } else if (out_mode == OUT_F32) {
        static_cast<float*>(a.y)[row] = __fmul_rn(static_cast<float>(acc), dq);
        if (a.y_acc) a.y_acc[row] = acc;
    } else {
        static_cast<__half*>(a.y)[row] = __float2half_rn(__fmul_rn(static_cast<float>(acc), dq));
    }
}

// One unit: 32 groups.  xs_blk points at the unit's eight 16-byte activation chunks,
// chunk i stored at index i ^ sw.  lutp = table base + lane.
__device__ __forceinline__ int decode_unit(const uint4& m, const uint2& v, const uint4* xs_blk,
                                           int sw, const uint32_t* lutp) {
    const uint32_t mw[4] = {m.x, m.y, m.z, m.w};
    int acc = 0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const uint32_t vv = (w < 2) ? v.x : v.y;
        const uint32_t sg = (w & 1) ? (vv >> 16) : vv;  // 16 sign bits of this meta word
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 xv = xs_blk[(2 * w + h) ^ sw];
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int g = 4 * h + j;
                const uint32_t idx = ((mw[w] >> (4 * g)) & 0xFu) | (((sg >> (2 * g)) & 0x3u) << 4);
                const uint32_t wt = lutp[idx * 32];
                acc = __dp4a(static_cast<int>(wt), static_cast<int>(xw[j]), acc);
            }
        }
    }
    return acc;
}

template <int U, int IN, int OUT>
__global__ void __launch_bounds__(kThreads) gemv_units_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem);
    int* rowacc = reinterpret_cast<int*>(smem + kLutBytes);
    uint4* xs = reinterpret_cast<uint4*>(smem + kLutBytes + ((a.rpc * 4 + 15) & ~15));

    const int tid = threadIdx.x, lane = tid & 31;
    const int r_lo = blockIdx.x * a.rpc;
    const int nrows = min(a.rpc, a.rows - r_lo);
    const int nunits = nrows * a.upr;

    grid_dep_launch();

    // 1. weight loads first: nothing below depends on a predecessor until the wait.
    uint4 m[U];
    uint2 v[U];
    int rl[U], cb[U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
        const int u = tid + i * kThreads;
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

    // 2. per-lane copies of the group table; zero the row accumulators.
    fill_lane_lut(lut, tid, kThreads);
    for (int e = tid; e < nrows; e += kThreads) rowacc[e] = 0;

    // 3. activations: only now may a predecessor's output be read.
    grid_dep_wait();
    const int nchunks = a.cols >> 4;
    float absmax = 0.0f;
    if (IN == IN_F16 || OUT != OUT_I32) absmax = *a.d_absmax;
    if (IN == IN_I8) {
        const uint4* xg = static_cast<const uint4*>(a.x);
        for (int q = tid; q < nchunks; q += kThreads) {
            const int c = q >> 3, i = q & 7;
            xs[(c << 3) + (i ^ (c & 7))] = xg[q];
        }
    } else {
        const float scale = quant_scale(absmax);
        const uint4* xg = static_cast<const uint4*>(a.x);
        for (int q = tid; q < nchunks; q += kThreads) {
            const uint4 lo = xg[2 * q], hi = xg[2 * q + 1];
            const uint32_t hw[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            uint32_t out[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t packed = 0;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const __half2 h2 = *reinterpret_cast<const __half2*>(&hw[2 * k + e]);
                    const int q0 = quantize_one(__low2float(h2), scale);
                    const int q1 = quantize_one(__high2float(h2), scale);
                    packed |= (static_cast<uint32_t>(q0) & 0xFFu) << (16 * e);
                    packed |= (static_cast<uint32_t>(q1) & 0xFFu) << (16 * e + 8);
                }
                out[k] = packed;
            }
            const int c = q >> 3, i = q & 7;
            xs[(c << 3) + (i ^ (c & 7))] = make_uint4(out[0], out[1], out[2], out[3]);
        }
    }
    __syncthreads();

    // 4. decode + segmented reduction over the lanes that share a row.
    const uint32_t* lutp = lut + lane;
#pragma unroll
    for (int i = 0; i < U; ++i) {
        int part = 0;
        if (rl[i] >= 0) part = decode_unit(m[i], v[i], xs + (cb[i] << 3), cb[i] & 7, lutp);
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int other = __shfl_down_sync(0xFFFFFFFFu, part, off);
            if (lane + off < 32 && cb[i] + off < a.upr) part += other;
        }
        if (rl[i] >= 0 && (cb[i] == 0 || lane == 0)) atomicAdd(&rowacc[rl[i]], part);
    }
    __syncthreads();

    // 5. epilogue.
    const float dq = (OUT != OUT_I32) ? dequant_scale(a.gamma, absmax) : 0.0f;
    for (int t = tid; t < nrows; t += kThreads) store_out(a, r_lo + t, rowacc[t], dq, OUT);
}

// Any cols % 4 == 0, any stride, any alignment: a warp per row, a group per lane per
// step, activations straight from global memory.  Correctness path for layouts the
// unit kernel does not take; not tuned.
template <int IN, int OUT>
__global__ void __launch_bounds__(kThreads) gemv_generic_kernel(const GemvArgs a) {
    grid_dep_launch();
    grid_dep_wait();
    const int lane = threadIdx.x & 31;
    const int row = (blockIdx.x * kThreads + threadIdx.x) >> 5;
    if (row >= a.rows) return;
    const uint32_t* mrow = a.meta + static_cast<size_t>(row) * a.meta_stride;
    const uint32_t* vrow = a.values + static_cast<size_t>(row) * a.values_stride;
    float absmax = 0.0f;
    if (IN == IN_F16 || OUT != OUT_I32) absmax = *a.d_absmax;
    const float scale = quant_scale(absmax);
    const int groups = a.cols >> 2;
    int acc = 0;
    for (int g = lane; g < groups; g += 32) {
        const uint32_t bitmap = (mrow[g >> 3] >> ((g & 7) * 4)) & 0xFu;
        const uint32_t signs = (vrow[g >> 4] >> ((g & 15) * 2)) & 0x3u;
        const uint32_t wt = c_group_lut.w[bitmap | (signs << 4)];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int w = static_cast<int8_t>(wt >> (8 * i));
            if (w != 0) {
                int xv;
                if (IN == IN_I8)
                    xv = static_cast<const int8_t*>(a.x)[4 * g + i];
                else
                    xv = quantize_one(__half2float(static_cast<const __half*>(a.x)[4 * g + i]), scale);
                acc += w * xv;
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    if (lane == 0) store_out(a, row, acc, dequant_scale(a.gamma, absmax), OUT);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
template <typename K>
static int ensure_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return SPB_OK;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(bytes));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "cudaFuncSetAttribute(%zu B): %s", bytes, cudaGetErrorString(err));
    }
    return SPB_OK;
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

template <int IN, int OUT>
static int run_gemv(const char* name, GemvArgs a, void* stream) {
    if (a.rows < 0 || a.cols < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    if (a.rows == 0 || a.cols == 0) return SPB_OK;
    if (a.cols % 4 != 0) return fail(SPB_E_INVALID, "%s: cols=%d is not a multiple of 4", name, a.cols);
    if (!a.meta || !a.values || !a.x || !a.y) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if ((IN == IN_F16 || OUT != OUT_I32) && !a.d_absmax)
        return fail(SPB_E_INVALID, "%s: d_absmax is null", name);
    if (a.meta_stride < (a.cols / 4 + 7) / 8 || a.values_stride < (a.cols / 4 + 15) / 16)
        return fail(SPB_E_INVALID, "%s: row stride shorter than a row", name);

    const bool fast = a.cols % 128 == 0 && a.cols / 128 <= 1024 && a.meta_stride % 4 == 0 &&
                      a.values_stride % 2 == 0 && aligned(a.meta, 16) && aligned(a.values, 8) &&
                      aligned(a.x, 16) && a.cols <= 196608;
    if (!fast) {
        const int grid = (a.rows + 7) / 8;
        return launch(name, gemv_generic_kernel<IN, OUT>, dim3(grid), dim3(kThreads), 0, stream, a);
    }

    const int sms = sm_count();
    a.upr = a.cols / 128;
    const int rpc_cap = max(1, 1024 / a.upr);
    const int fill = max(1, kThreads / a.upr);                 // rows that fill one pass of the block
    const int spread = (a.rows + sms - 1) / sms;               // rows per block at one block per SM
    int rpc = max((a.rows + 4 * sms - 1) / (4 * sms), min(fill, spread));
    rpc = max(1, min(rpc, rpc_cap));
    a.rpc = rpc;
    const int units = rpc * a.upr;
    const int passes = (units + kThreads - 1) / kThreads;
    const int grid = (a.rows + rpc - 1) / rpc;
    const size_t smem = kLutBytes + ((rpc * 4 + 15) & ~15) + static_cast<size_t>(a.cols);

    int rc;
    if (passes <= 1) {
        if ((rc = ensure_smem(gemv_units_kernel<1, IN, OUT>, smem))) return rc;
        return launch(name, gemv_units_kernel<1, IN, OUT>, dim3(grid), dim3(kThreads), smem, stream, a);
    } else if (passes <= 2) {
        if ((rc = ensure_smem(gemv_units_kernel<2, IN, OUT>, smem))) return rc;
        return launch(name, gemv_units_kernel<2, IN, OUT>, dim3(grid), dim3(kThreads), smem, stream, a);
    } else {
        if ((rc = ensure_smem(gemv_units_kernel<4, IN, OUT>, smem))) return rc;
        return launch(name, gemv_units_kernel<4, IN, OUT>, dim3(grid), dim3(kThreads), smem, stream, a);
    }
}

}  // namespace spb

using namespace spb;

extern "C" int spb_sparse_ternary_gemv(const uint32_t* meta, const uint32_t* values, const int8_t* x,
                                       int32_t* y, int rows, int cols, int meta_row_stride,
                                       int values_row_stride, void* stream) {
    GemvArgs a{meta, values, x, y, nullptr, nullptr, 0.0f, rows, cols, meta_row_stride, values_row_stride, 0, 0};
    return run_gemv<IN_I8, OUT_I32>("spb_sparse_ternary_gemv", a, stream);
}

extern "C" int spb_sparse_ternary_gemv_scaled(const uint32_t* meta, const uint32_t* values,
                                              const int8_t* x, float* y, int32_t* y_acc,
                                              const float* d_absmax, float gamma, int rows, int cols,
                                              int meta_row_stride, int values_row_stride, void* stream) {
    GemvArgs a{meta, values, x, y, y_acc, d_absmax, gamma, rows, cols, meta_row_stride, values_row_stride, 0, 0};
    return run_gemv<IN_I8, OUT_F32>("spb_sparse_ternary_gemv_scaled", a, stream);
}

extern "C" int spb_fused_sparse_bitlinear(const uint32_t* meta, const uint32_t* values, const void* x,
                                          void* output, const float* d_absmax, float gamma, int rows,
                                          int cols, int meta_row_stride, int values_row_stride,
                                          void* stream) {
    GemvArgs a{meta, values, x, output, nullptr, d_absmax, gamma, rows, cols, meta_row_stride, values_row_stride, 0, 0};
    return run_gemv<IN_F16, OUT_F16>("spb_fused_sparse_bitlinear", a, stream);
}

extern "C" int spb_sparse_bitlinear_q8(const uint32_t* meta, const uint32_t* values, const int8_t* xq,
                                       void* output, const float* d_absmax, float gamma, int rows,
                                       int cols, int meta_row_stride, int values_row_stride,
                                       void* stream) {
    GemvArgs a{meta, values, xq, output, nullptr, d_absmax, gamma, rows, cols, meta_row_stride, values_row_stride, 0, 0};
    return run_gemv<IN_I8, OUT_F16>("spb_sparse_bitlinear_q8", a, stream);
}
