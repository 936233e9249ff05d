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

constexpr int kMaxMats = 3;

// One weight matrix of a launch.  Up to kMaxMats matrices that consume the same
// activation vector (q/k/v, gate/up) share one launch; blocks [blk_begin, next blk_begin)
// work on matrix i.
struct GemvMat {
    const uint32_t* meta;
    const uint32_t* values;
    void* y;          // int32 / float / half, rows elements
    int32_t* y_acc;   // optional int32 copy of the accumulators (OUT_F32)
    float gamma;
    int rows;
    int meta_stride, values_stride;  // uint32 words
    int blk_begin;
};

struct GemvArgs {
    GemvMat mat[kMaxMats];
    int nmat;
    const void* x;          // int8 (IN_I8) or half (IN_F16), cols elements
    const float* d_absmax;  // device scalar; read after the dependency wait
    int cols;
    int upr;  // units per row = cols / 128
    int rpc;  // rows per block
};

constexpr int kThreads = 256;

__device__ __forceinline__ void store_out(const GemvMat& m, int row, int acc, float dq, int out_mode) {
    if (out_mode == OUT_I32) {
        static_cast<int32_t*>(m.y)[row] = acc;
    } else if (out_mode == OUT_F32) {
        static_cast<float*>(m.y)[row] = __fmul_rn(static_cast<float>(acc), dq);
        if (m.y_acc) m.y_acc[row] = acc;
    } else {
        static_cast<__half*>(m.y)[row] = __float2half_rn(__fmul_rn(static_cast<float>(acc), dq));
    }
}

// Block = rpc rows of one matrix = rpc * upr units, one unit per thread.
//   phase A (independent of any predecessor): stream the unit's 24 bytes of weights, build the
//            per-lane table, expand the unit to 32 packed int8x4 weight words in registers;
//   phase B (after the dependency wait): stage x, 8 x LDS.128 + 32 x dp4a, reduce, store.
template <int IN, int OUT>
__global__ void __launch_bounds__(kThreads) gemv_units_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem);
    int* rowacc = reinterpret_cast<int*>(smem + kLutBytes);
    uint4* xs = reinterpret_cast<uint4*>(smem + kLutBytes + ((a.rpc * 4 + 15) & ~15));

    const int tid = threadIdx.x, lane = tid & 31;
    int mi = 0;
    if (a.nmat > 1 && static_cast<int>(blockIdx.x) >= a.mat[1].blk_begin) mi = 1;
    if (a.nmat > 2 && static_cast<int>(blockIdx.x) >= a.mat[2].blk_begin) mi = 2;
    const GemvMat& M = a.mat[mi];
    const int r_lo = (blockIdx.x - M.blk_begin) * a.rpc;
    const int nrows = min(a.rpc, M.rows - r_lo);
    const int nunits = nrows * a.upr;

    grid_dep_launch();

    // ---- phase A ------------------------------------------------------------------------
    const bool valid = tid < nunits;
    int rl = -1, cb = a.upr;
    uint4 m = make_uint4(0, 0, 0, 0);
    uint2 v = make_uint2(0, 0);
    if (valid) {
        rl = tid / a.upr;
        cb = tid - rl * a.upr;
        const size_t row = static_cast<size_t>(r_lo + rl);
        m = ld_stream_v4(M.meta + row * M.meta_stride + cb * 4);
        v = ld_stream_v2(M.values + row * M.values_stride + cb * 2);
    }
    fill_lane_lut(lut, tid, kThreads);
    for (int e = tid; e < nrows; e += kThreads) rowacc[e] = 0;
    __syncthreads();

    uint32_t wt[32];
    {
        const uint32_t* lutp = lut + lane;
        const uint32_t mw[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t vv = (w < 2) ? v.x : v.y;
            const uint32_t sg = (w & 1) ? (vv >> 16) : vv;  // the 16 sign bits of this meta word
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const uint32_t idx = ((mw[w] >> (4 * g)) & 0xFu) | (((sg >> (2 * g)) & 0x3u) << 4);
                wt[w * 8 + g] = lutp[idx * 32];
            }
        }
    }

    // ---- phase B ------------------------------------------------------------------------
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

    int part = 0;
    if (valid) {
        const uint4* xb = xs + (cb << 3);
        const int sw = cb & 7;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
            const uint4 xv = xb[ch ^ sw];
            part = __dp4a(static_cast<int>(wt[ch * 4 + 0]), static_cast<int>(xv.x), part);
            part = __dp4a(static_cast<int>(wt[ch * 4 + 1]), static_cast<int>(xv.y), part);
            part = __dp4a(static_cast<int>(wt[ch * 4 + 2]), static_cast<int>(xv.z), part);
            part = __dp4a(static_cast<int>(wt[ch * 4 + 3]), static_cast<int>(xv.w), part);
        }
    }
    // segmented reduction: the units of a row sit in consecutive lanes
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int other = __shfl_down_sync(0xFFFFFFFFu, part, off);
        if (lane + off < 32 && cb + off < a.upr) part += other;
    }
    if (valid && (cb == 0 || lane == 0)) atomicAdd(&rowacc[rl], part);
    __syncthreads();

    const float dq = (OUT != OUT_I32) ? dequant_scale(M.gamma, absmax) : 0.0f;
    for (int t = tid; t < nrows; t += kThreads) store_out(M, r_lo + t, rowacc[t], dq, OUT);
}

// ---------------------------------------------------------------------------
// Pair kernel (the default).
//
// Same block/unit mapping and the same two phases as the kernel above, but two groups (one
// meta byte, one sign nibble) are consumed at a time:
//   sel = sel_lut[meta byte & 0x77] : PRMT selector that gathers the four non-zero columns
//   sgn = sgn_lut[sign nibble]      : their four signs as int8 +-1
//   acc = dp4a(prmt(x_lo, x_hi, sel), sgn, acc)
// i.e. one dp4a per two groups.  Three bits of a bitmap with exactly two of four bits set
// determine the fourth, so the selector table is indexed by 3+3 bits.  Both tables are
// replicated once per lane (bank = lane, no conflicts) and copied from a constant image in
// global memory (L2-resident) with 128-bit loads.  The dependency wait sits between the table
// copy and the expansion: the x chunks are requested right after it and land while the
// weights are expanded to 16 selectors and 16 sign words in registers; the arithmetic is then
// 8 x LDS.128 + 16 x (PRMT, dp4a).  Per-thread partial sums meet in a transposed shared array
// and one thread per row folds them.
// Bitmaps must be valid (spb_validate_packed); others decode as some valid bitmap.
// ---------------------------------------------------------------------------
constexpr int kSelEntries = 120;  // (meta byte & 0x77) <= 0x77
constexpr int kSelBytes = kSelEntries * 32 * 4;  // 15360
constexpr int kSgnBytes = 16 * 32 * 4;           // 2048
constexpr int kWindow = 16384;

struct PairLutImage {
    uint32_t sel[kSelEntries * 32];
    uint32_t sgn[16 * 32];
};

constexpr uint32_t pair_selector(int b) {
    // b = (meta byte & 0x77): the low three bits of each nibble; the fourth bit is implied
    uint32_t sel = 0;
    for (int half = 0; half < 2; ++half) {
        int n = (b >> (4 * half)) & 7;
        const int cnt = (n & 1) + ((n >> 1) & 1) + ((n >> 2) & 1);
        if (cnt == 1) n |= 8;
        int bits = 0, p0 = 0, p1 = 0;
        for (int i = 0; i < 4; ++i)
            if (n & (1 << i)) {
                if (bits == 0) p0 = i;
                if (bits == 1) p1 = i;
                ++bits;
            }
        if (bits != 2) { p0 = 0; p1 = 0; }
        sel |= static_cast<uint32_t>((4 * half + p0) | ((4 * half + p1) << 4)) << (8 * half);
    }
    return sel;
}

constexpr PairLutImage make_pair_lut_image() {
    PairLutImage t{};
    for (int e = 0; e < kSelEntries; ++e)
        for (int l = 0; l < 32; ++l) t.sel[e * 32 + l] = pair_selector(e);
    for (int n = 0; n < 16; ++n) {
        uint32_t w = 0;
        for (int i = 0; i < 4; ++i) w |= ((n >> i) & 1 ? 0xFFu : 0x01u) << (8 * i);
        for (int l = 0; l < 32; ++l) t.sgn[n * 32 + l] = w;
    }
    return t;
}

__device__ __align__(128) const PairLutImage g_pair_lut = make_pair_lut_image();

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

template <int IN, int OUT>
__global__ void __launch_bounds__(kThreads, 4) gemv_pairs_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) uint8_t psmem[];
    // [sel 15360][sgn 2048][partials upr*pitch ints (16-aligned)][x cols bytes]
    const uint32_t win_s = smem_u32(psmem);
    uint8_t* win = psmem;
    const int pitch = a.rpc | 1;
    int* partial = reinterpret_cast<int*>(win + kSelBytes + kSgnBytes);
    uint4* xs = reinterpret_cast<uint4*>(win + kSelBytes + kSgnBytes + ((a.upr * pitch * 4 + 15) & ~15));

    const int tid = threadIdx.x, lane = tid & 31;
    int mi = 0;
    if (a.nmat > 1 && static_cast<int>(blockIdx.x) >= a.mat[1].blk_begin) mi = 1;
    if (a.nmat > 2 && static_cast<int>(blockIdx.x) >= a.mat[2].blk_begin) mi = 2;
    const GemvMat& M = a.mat[mi];
    const int r_lo = (blockIdx.x - M.blk_begin) * a.rpc;
    const int nrows = min(a.rpc, M.rows - r_lo);
    const int nunits = nrows * a.upr;

    grid_dep_launch();

    // ---- phase A: weights, tables, expansion to selectors and signs ---------------------------
    const bool valid = tid < nunits;
    int rl = 0, cb = 0;
    uint4 m = make_uint4(0, 0, 0, 0);
    uint2 v = make_uint2(0, 0);
    if (valid) {
        rl = tid / a.upr;
        cb = tid - rl * a.upr;
        const size_t row = static_cast<size_t>(r_lo + rl);
        m = ld_stream_v4(M.meta + row * M.meta_stride + cb * 4);
        v = ld_stream_v2(M.values + row * M.values_stride + cb * 2);
    }
    {
        const uint4* src = reinterpret_cast<const uint4*>(&g_pair_lut);
        uint4* dst = reinterpret_cast<uint4*>(win);
        for (int q = tid; q < (kSelBytes + kSgnBytes) / 16; q += kThreads) dst[q] = __ldg(src + q);
    }

    // ---- phase B starts: only now may a predecessor's output be read.  The first two x chunks
    // of every thread are requested here, so that their latency overlaps the expansion below
    // (and, when no predecessor is pending, the weight loads above).
    grid_dep_wait();
    const int nchunks = a.cols >> 4;
    float absmax = 0.0f;
    if (IN == IN_F16 || OUT != OUT_I32) absmax = *a.d_absmax;
    const float qscale = quant_scale(absmax);
    auto load_chunk = [&](int q, uint4& lo, uint4& hi) {
        const uint4* xg = static_cast<const uint4*>(a.x);
        if (IN == IN_I8) {
            lo = xg[q];
        } else {
            lo = xg[2 * q];
            hi = xg[2 * q + 1];
        }
    };
    auto store_chunk = [&](int q, const uint4& lo, const uint4& hi) {
        uint4 out = lo;
        if (IN == IN_F16) {
            const uint32_t hw[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t packed = 0;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const __half2 h2 = *reinterpret_cast<const __half2*>(&hw[2 * k + e]);
                    const int q0 = quantize_one(__low2float(h2), qscale);
                    const int q1 = quantize_one(__high2float(h2), qscale);
                    packed |= (static_cast<uint32_t>(q0) & 0xFFu) << (16 * e);
                    packed |= (static_cast<uint32_t>(q1) & 0xFFu) << (16 * e + 8);
                }
                o[k] = packed;
            }
            out = make_uint4(o[0], o[1], o[2], o[3]);
        }
        const int c = q >> 3, i = q & 7;
        xs[(c << 3) + (i ^ (c & 7))] = out;
    };
    uint4 xa_lo = make_uint4(0, 0, 0, 0), xa_hi = xa_lo, xb_lo = xa_lo, xb_hi = xa_lo;
    if (tid < nchunks) load_chunk(tid, xa_lo, xa_hi);
    if (tid + kThreads < nchunks) load_chunk(tid + kThreads, xb_lo, xb_hi);

    __syncthreads();  // tables complete

    uint32_t sel[16], sgn[16];
    {
        // produced by a volatile statement after the barrier, so that no table load can be
        // scheduled above it
        uint32_t sel_lane;
        asm volatile("add.u32 %0, %1, %2;" : "=r"(sel_lane) : "r"(win_s), "r"(lane * 4) : "memory");
        const uint32_t sgn_lane = sel_lane + kSelBytes;
        const uint32_t mw[4] = {m.x, m.y, m.z, m.w};
        const uint32_t vw[2] = {v.x, v.y};
#pragma unroll
        for (int p = 0; p < 16; ++p) {  // groups 2p and 2p+1: meta byte p, sign nibble p
            const int ms = 8 * (p & 3) - 7, ss = 4 * (p & 7) - 7;
            sel[p] = lds32(((ms >= 0 ? (mw[p >> 2] >> ms) : (mw[p >> 2] << -ms)) & (0x77u << 7)) + sel_lane);
            sgn[p] = lds32(((ss >= 0 ? (vw[p >> 3] >> ss) : (vw[p >> 3] << -ss)) & (0xFu << 7)) + sgn_lane);
        }
    }

    if (tid < nchunks) store_chunk(tid, xa_lo, xa_hi);
    if (tid + kThreads < nchunks) store_chunk(tid + kThreads, xb_lo, xb_hi);
    for (int q = tid + 2 * kThreads; q < nchunks; q += kThreads) {  // wide matrices
        uint4 lo, hi = make_uint4(0, 0, 0, 0);
        load_chunk(q, lo, hi);
        store_chunk(q, lo, hi);
    }
    __syncthreads();

    if (valid) {
        const uint4* xb = xs + (cb << 3);
        const int sw = cb & 7;
        int acc = 0;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {  // 16 columns = 4 groups = 2 pairs per chunk
            const uint4 xv = xb[ch ^ sw];
            acc = __dp4a(static_cast<int>(__byte_perm(xv.x, xv.y, sel[2 * ch])), static_cast<int>(sgn[2 * ch]), acc);
            acc = __dp4a(static_cast<int>(__byte_perm(xv.z, xv.w, sel[2 * ch + 1])), static_cast<int>(sgn[2 * ch + 1]), acc);
        }
        partial[cb * pitch + rl] = acc;
    }
    __syncthreads();

    // one thread per row folds its partials (consecutive rows -> consecutive banks)
    const float dq = (OUT != OUT_I32) ? dequant_scale(M.gamma, absmax) : 0.0f;
    for (int lr = tid; lr < nrows; lr += kThreads) {
        int s = 0;
        for (int c = 0; c < a.upr; ++c) s += partial[c * pitch + lr];
        store_out(M, r_lo + lr, s, dq, OUT);
    }
}

// Any cols % 4 == 0, any stride, any alignment: a warp per row, a group per lane per
// step, activations straight from global memory.  Correctness path for layouts the
// unit kernel does not take; not tuned.
template <int IN, int OUT>
__global__ void __launch_bounds__(kThreads) gemv_generic_kernel(const GemvArgs a) {
    grid_dep_launch();
    grid_dep_wait();
    const int lane = threadIdx.x & 31;
    int mi = 0;
    if (a.nmat > 1 && static_cast<int>(blockIdx.x) >= a.mat[1].blk_begin) mi = 1;
    if (a.nmat > 2 && static_cast<int>(blockIdx.x) >= a.mat[2].blk_begin) mi = 2;
    const GemvMat& M = a.mat[mi];
    const int row = ((blockIdx.x - M.blk_begin) * kThreads + threadIdx.x) >> 5;
    if (row >= M.rows) return;
    const uint32_t* mrow = M.meta + static_cast<size_t>(row) * M.meta_stride;
    const uint32_t* vrow = M.values + static_cast<size_t>(row) * M.values_stride;
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
    if (lane == 0) store_out(M, row, acc, dequant_scale(M.gamma, absmax), OUT);
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

struct MatDesc {
    const uint32_t* meta;
    const uint32_t* values;
    void* y;
    int32_t* y_acc;
    float gamma;
    int rows, meta_stride, values_stride;
};

static int g_gemv_variant = 0;  // 0/1 pair kernel (default), 2 per-group table kernel

// Launches up to kMaxMats matrices that share x (and d_absmax) as one grid.
template <int IN, int OUT>
static int run_gemv(const char* name, const MatDesc* mats, int nmat, const void* x, const float* d_absmax,
                    int cols, void* stream) {
    if (nmat < 1 || nmat > kMaxMats) return fail(SPB_E_INVALID, "%s: %d matrices in one launch", name, nmat);
    if (cols < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    int total_rows = 0;
    for (int i = 0; i < nmat; ++i) {
        if (mats[i].rows < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
        total_rows += mats[i].rows;
    }
    if (total_rows == 0 || cols == 0) return SPB_OK;
    if (cols % 4 != 0) return fail(SPB_E_INVALID, "%s: cols=%d is not a multiple of 4", name, cols);
    if (!x) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if ((IN == IN_F16 || OUT != OUT_I32) && !d_absmax) return fail(SPB_E_INVALID, "%s: d_absmax is null", name);
    bool fast = cols % 128 == 0 && cols / 128 <= kThreads && aligned(x, 16) && cols <= 196608;
    int max_rows = 0;
    for (int i = 0; i < nmat; ++i) {
        const MatDesc& m = mats[i];
        if (m.rows == 0) continue;
        if (!m.meta || !m.values || !m.y) return fail(SPB_E_INVALID, "%s: null pointer", name);
        if (m.meta_stride < (cols / 4 + 7) / 8 || m.values_stride < (cols / 4 + 15) / 16)
            return fail(SPB_E_INVALID, "%s: row stride shorter than a row", name);
        fast = fast && m.meta_stride % 4 == 0 && m.values_stride % 2 == 0 && aligned(m.meta, 16) &&
               aligned(m.values, 8);
        max_rows = max(max_rows, m.rows);
    }

    GemvArgs a{};
    a.nmat = nmat;
    a.x = x;
    a.d_absmax = d_absmax;
    a.cols = cols;
    const int sms = sm_count();
    int rpc = 8;  // generic path: a warp per row, 8 rows per block
    if (fast) {
        a.upr = cols / 128;
        const int fill = max(1, kThreads / a.upr);       // rows that fill the block
        const int spread = (total_rows + sms - 1) / sms;  // rows per block at one block per SM
        rpc = max(1, min(fill, spread));
    }
    a.rpc = rpc;
    int blocks = 0;
    for (int i = 0; i < nmat; ++i) {
        const MatDesc& m = mats[i];
        a.mat[i] = GemvMat{m.meta, m.values, m.y, m.y_acc, m.gamma, m.rows, m.meta_stride, m.values_stride, blocks};
        blocks += (m.rows + rpc - 1) / rpc;
    }
    if (!fast) return launch(name, gemv_generic_kernel<IN, OUT>, dim3(blocks), dim3(kThreads), 0, stream, a);
    int rc;
    if (g_gemv_variant == 2) {  // the per-group table kernel, kept for comparison
        const size_t smem = kLutBytes + ((rpc * 4 + 15) & ~15) + static_cast<size_t>(cols);
        if ((rc = ensure_smem(gemv_units_kernel<IN, OUT>, smem))) return rc;
        return launch(name, gemv_units_kernel<IN, OUT>, dim3(blocks), dim3(kThreads), smem, stream, a);
    }
    const size_t smem = kSelBytes + kSgnBytes + ((a.upr * (rpc | 1) * 4 + 15) & ~15) + static_cast<size_t>(cols);
    if ((rc = ensure_smem(gemv_pairs_kernel<IN, OUT>, smem))) return rc;
    return launch(name, gemv_pairs_kernel<IN, OUT>, dim3(blocks), dim3(kThreads), smem, stream, a);
}

// Engine-internal: several BitLinear layers on the same pre-quantised activation in one launch.
int bitlinear_q8_group(const uint32_t* const* meta, const uint32_t* const* values, void* const* out,
                       const float* gamma, const int* rows, const int* ms, const int* vs, int nmat,
                       const int8_t* xq, const float* d_absmax, int cols, void* stream) {
    MatDesc d[kMaxMats];
    if (nmat > kMaxMats) return fail(SPB_E_INVALID, "bitlinear_q8_group: too many matrices");
    for (int i = 0; i < nmat; ++i) d[i] = MatDesc{meta[i], values[i], out[i], nullptr, gamma[i], rows[i], ms[i], vs[i]};
    return run_gemv<IN_I8, OUT_F16>("bitlinear_q8_group", d, nmat, xq, d_absmax, cols, stream);
}

}  // namespace spb

using namespace spb;

extern "C" int spb_set_gemv_variant(int variant) {
    const int old = g_gemv_variant;
    g_gemv_variant = variant;
    return old;
}

extern "C" int spb_sparse_ternary_gemv(const uint32_t* meta, const uint32_t* values, const int8_t* x,
                                       int32_t* y, int rows, int cols, int meta_row_stride,
                                       int values_row_stride, void* stream) {
    MatDesc d{meta, values, y, nullptr, 0.0f, rows, meta_row_stride, values_row_stride};
    return run_gemv<IN_I8, OUT_I32>("spb_sparse_ternary_gemv", &d, 1, x, nullptr, cols, stream);
}

extern "C" int spb_sparse_ternary_gemv_scaled(const uint32_t* meta, const uint32_t* values,
                                              const int8_t* x, float* y, int32_t* y_acc,
                                              const float* d_absmax, float gamma, int rows, int cols,
                                              int meta_row_stride, int values_row_stride, void* stream) {
    MatDesc d{meta, values, y, y_acc, gamma, rows, meta_row_stride, values_row_stride};
    return run_gemv<IN_I8, OUT_F32>("spb_sparse_ternary_gemv_scaled", &d, 1, x, d_absmax, cols, stream);
}

extern "C" int spb_fused_sparse_bitlinear(const uint32_t* meta, const uint32_t* values, const void* x,
                                          void* output, const float* d_absmax, float gamma, int rows,
                                          int cols, int meta_row_stride, int values_row_stride,
                                          void* stream) {
    MatDesc d{meta, values, output, nullptr, gamma, rows, meta_row_stride, values_row_stride};
    return run_gemv<IN_F16, OUT_F16>("spb_fused_sparse_bitlinear", &d, 1, x, d_absmax, cols, stream);
}

extern "C" int spb_sparse_bitlinear_q8(const uint32_t* meta, const uint32_t* values, const int8_t* xq,
                                       void* output, const float* d_absmax, float gamma, int rows,
                                       int cols, int meta_row_stride, int values_row_stride,
                                       void* stream) {
    MatDesc d{meta, values, output, nullptr, gamma, rows, meta_row_stride, values_row_stride};
    return run_gemv<IN_I8, OUT_F16>("spb_sparse_bitlinear_q8", &d, 1, xq, d_absmax, cols, stream);
}
