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
// "Column-owner" kernel: the throughput form.
//
// A thread owns one 128-column block of x for the whole launch (32 registers) and walks
// down the rows of its block, so the activation bytes cost no shared-memory bandwidth in
// the inner loop.  Two groups (one meta byte, one sign nibble) are consumed by
//   sel = sel_lut[meta byte & 0x77] : PRMT selector that gathers the four non-zero columns
//   sgn = sgn_lut[sign nibble]      : their four signs as int8 +-1
//   acc = dp4a(prmt(x_lo, x_hi, sel), sgn, acc)
// i.e. one dp4a per two groups.  Three bits of a bitmap with exactly two of four bits set
// determine the fourth, so the table is indexed by 3+3 bits; both tables are replicated
// once per lane (bank = lane, no conflicts) and arrive in shared memory by one bulk
// asynchronous copy (TMA) from a constant image in global memory.  Bitmaps must be valid
// (spb_validate_packed); others decode as some valid bitmap.
// One block of 512 threads per SM takes a contiguous range of rows of one matrix; the
// per-thread partial sums of a row meet in shared memory and a warp folds each row.
// ---------------------------------------------------------------------------
constexpr int kColsThreads = 512;
constexpr int kSelEntries = 120;  // (meta byte & 0x77) <= 0x77
constexpr int kSgnEntries = 16;
constexpr int kLaneLutWords = (kSelEntries + kSgnEntries) * 32;
constexpr int kLaneLutBytes = kLaneLutWords * 4;  // 17408
constexpr int kSelLutBytes = kSelEntries * 32 * 4;
constexpr int kDepth = 4;  // units whose weights are in flight per thread

struct LaneLutImage {
    uint32_t w[kLaneLutWords];
};

constexpr uint32_t pair_selector(int b) {
    // b = (meta byte & 0x77): low three bits of each nibble; the fourth bit is implied
    uint32_t sel = 0;
    for (int half = 0; half < 2; ++half) {
        int n = (b >> (4 * half)) & 7;
        int cnt = (n & 1) + ((n >> 1) & 1) + ((n >> 2) & 1);
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

constexpr LaneLutImage make_lane_lut_image() {
    LaneLutImage t{};
    for (int e = 0; e < kSelEntries; ++e)
        for (int l = 0; l < 32; ++l) t.w[e * 32 + l] = pair_selector(e);
    for (int n = 0; n < kSgnEntries; ++n) {
        uint32_t w = 0;
        for (int i = 0; i < 4; ++i) w |= ((n >> i) & 1 ? 0xFFu : 0x01u) << (8 * i);
        for (int l = 0; l < 32; ++l) t.w[(kSelEntries + n) * 32 + l] = w;
    }
    return t;
}

__device__ __align__(128) const LaneLutImage g_lane_lut = make_lane_lut_image();

struct ColsArgs {
    GemvMat mat[kMaxMats];  // blk_begin = first block of the matrix
    int nmat;
    const void* x;
    const float* d_absmax;
    int cols, upr;
    int rs;   // row slots per block = kColsThreads / upr
    int rpc;  // rows per block
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// One unit against the thread's 32 x words.  lut_lane = shared address of the table + lane*4.
__device__ __forceinline__ int mac_unit(const uint4& m, const uint2& v, const uint32_t (&xr)[32],
                                        uint32_t lut_lane) {
    const uint32_t mw[4] = {m.x, m.y, m.z, m.w};
    const uint32_t vw[2] = {v.x, v.y};
    int acc = 0;
#pragma unroll
    for (int p = 0; p < 16; ++p) {  // groups 2p and 2p+1
        const int ms = 8 * (p & 3) - 7;  // meta byte p of its word, scaled by 128 (entry stride)
        const uint32_t mb = (ms >= 0 ? (mw[p >> 2] >> ms) : (mw[p >> 2] << -ms)) & (0x77u << 7);
        const int ss = 4 * (p & 7) - 7;  // sign nibble p of its word, scaled by 128
        const uint32_t sn = (ss >= 0 ? (vw[p >> 3] >> ss) : (vw[p >> 3] << -ss)) & (0xFu << 7);
        uint32_t sel, sg;
        asm("ld.shared.u32 %0, [%1];" : "=r"(sel) : "r"(lut_lane + mb));
        asm("ld.shared.u32 %0, [%1+%2];" : "=r"(sg) : "r"(lut_lane + sn), "n"(kSelLutBytes));
        acc = __dp4a(static_cast<int>(__byte_perm(xr[2 * p], xr[2 * p + 1], sel)), static_cast<int>(sg), acc);
    }
    return acc;
}

template <int IN, int OUT>
__global__ void __launch_bounds__(kColsThreads, 1) gemv_cols_kernel(const ColsArgs a) {
    extern __shared__ __align__(128) uint8_t csmem[];
    uint8_t* const smem = csmem;
    // layout: [lane tables 17408][mbarrier 16][partials rpc*upr*4 (16-aligned)][xs cols (IN_F16)]
    uint64_t* mbar = reinterpret_cast<uint64_t*>(smem + kLaneLutBytes);
    int* partial = reinterpret_cast<int*>(smem + kLaneLutBytes + 16);
    uint4* xs = reinterpret_cast<uint4*>(smem + kLaneLutBytes + 16 + ((a.rpc * a.upr * 4 + 15) & ~15));

    const int tid = threadIdx.x, lane = tid & 31;
    int mi = 0;
    if (a.nmat > 1 && static_cast<int>(blockIdx.x) >= a.mat[1].blk_begin) mi = 1;
    if (a.nmat > 2 && static_cast<int>(blockIdx.x) >= a.mat[2].blk_begin) mi = 2;
    const GemvMat& M = a.mat[mi];
    const int r_lo = (blockIdx.x - M.blk_begin) * a.rpc;
    const int nrows = min(a.rpc, M.rows - r_lo);
    const int rs = tid / a.upr, cb = tid - rs * a.upr;
    const bool active = rs < a.rs;
    const int niter = (nrows + a.rs - 1) / a.rs;

    grid_dep_launch();

    // ---- tables: one bulk copy global -> shared, completion on an mbarrier -----------------
    const uint32_t mbar_s = smem_u32(mbar);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_s));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar_s), "n"(kLaneLutBytes) : "memory");
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem)),
            "l"(&g_lane_lut), "n"(kLaneLutBytes), "r"(mbar_s)
            : "memory");
    }

    // ---- weights of the first kDepth units: independent of any predecessor -----------------
    const uint32_t* mp = M.meta + static_cast<size_t>(r_lo + rs) * M.meta_stride + cb * 4;
    const uint32_t* vp = M.values + static_cast<size_t>(r_lo + rs) * M.values_stride + cb * 2;
    const size_t m_step = static_cast<size_t>(a.rs) * M.meta_stride;
    const size_t v_step = static_cast<size_t>(a.rs) * M.values_stride;
    uint4 m[kDepth];
    uint2 v[kDepth];
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
        if (active && d * a.rs + rs < nrows) {
            m[d] = ld_stream_v4(mp + d * m_step);
            v[d] = ld_stream_v2(vp + d * v_step);
        } else {
            m[d] = make_uint4(0, 0, 0, 0);
            v[d] = make_uint2(0, 0);
        }
    }

    // ---- activations: only now may a predecessor's output be read --------------------------
    grid_dep_wait();
    float absmax = 0.0f;
    if (IN == IN_F16 || OUT != OUT_I32) absmax = *a.d_absmax;
    uint32_t xr[32];
    if (IN == IN_I8) {
        const uint4* xg = static_cast<const uint4*>(a.x) + (active ? (cb << 3) : 0);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
            const uint4 t = __ldg(xg + ch);
            xr[4 * ch + 0] = t.x; xr[4 * ch + 1] = t.y; xr[4 * ch + 2] = t.z; xr[4 * ch + 3] = t.w;
        }
    } else {
        const float scale = quant_scale(absmax);
        const uint4* xg = static_cast<const uint4*>(a.x);
        const int nchunks = a.cols >> 4;
        for (int q = tid; q < nchunks; q += kColsThreads) {
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
        __syncthreads();
        const uint4* xb = xs + (active ? (cb << 3) : 0);
        const int sw = active ? (cb & 7) : 0;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
            const uint4 t = xb[ch ^ sw];
            xr[4 * ch + 0] = t.x; xr[4 * ch + 1] = t.y; xr[4 * ch + 2] = t.z; xr[4 * ch + 3] = t.w;
        }
    }

    // ---- wait for the tables (bounded); on expiry fill them with plain loads instead ----------
    {
        uint32_t done = 0;
        for (int spin = 0; spin < 4096 && !done; ++spin) {
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(done)
                : "r"(mbar_s)
                : "memory");
        }
        if (!__syncthreads_and(done != 0)) {
            uint32_t* lut = reinterpret_cast<uint32_t*>(smem);
            for (int e = tid; e < kLaneLutWords; e += kColsThreads) lut[e] = g_lane_lut.w[e];
            __syncthreads();
        }
    }

    // ---- main loop: consume unit `it`, refill its slot with unit `it + kDepth` -----------------
    // The table address is produced after the wait by a volatile statement, so that no table
    // load can be scheduled above the wait.
    uint32_t lut_lane;
    asm volatile("add.u32 %0, %1, %2;" : "=r"(lut_lane) : "r"(smem_u32(smem)), "r"(lane * 4) : "memory");
    int* my_partial = partial + rs * a.upr + cb;
    for (int it0 = 0; it0 < niter; it0 += kDepth) {
#pragma unroll
        for (int d = 0; d < kDepth; ++d) {
            const int it = it0 + d;
            if (it >= niter) break;  // uniform across the block
            const int lr = it * a.rs + rs;
            if (active && lr < nrows) {
                my_partial[it * a.rs * a.upr] = mac_unit(m[d], v[d], xr, lut_lane);
                const int nx = it + kDepth;
                if (nx * a.rs + rs < nrows) {
                    m[d] = ld_stream_v4(mp + nx * m_step);
                    v[d] = ld_stream_v2(vp + nx * v_step);
                }
            }
        }
    }
    __syncthreads();

    // ---- a warp folds each row ------------------------------------------------------------------
    const float dq = (OUT != OUT_I32) ? dequant_scale(M.gamma, absmax) : 0.0f;
    for (int lr = tid >> 5; lr < nrows; lr += kColsThreads / 32) {
        int s = 0;
        for (int c = lane; c < a.upr; c += 32) s += partial[lr * a.upr + c];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
        if (lane == 0) store_out(M, r_lo + lr, s, dq, OUT);
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

static int g_gemv_variant = 0;  // 0 auto, 1 unit kernel (latency form), 2 column-owner kernel (throughput form)

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

    if (fast && g_gemv_variant != 1 && cols / 128 <= kColsThreads) {
        ColsArgs c{};
        c.nmat = nmat;
        c.x = x;
        c.d_absmax = d_absmax;
        c.cols = cols;
        c.upr = cols / 128;
        c.rs = kColsThreads / c.upr;
        const int sms_ = sm_count();
        // rows per block: one block per SM, but never more partial sums than shared memory holds
        int rpc = max(1, (total_rows + sms_ - 1) / sms_);
        const int rpc_cap = max(1, (150 * 1024) / (c.upr * 4));
        rpc = min(rpc, rpc_cap);
        c.rpc = rpc;
        int blocks = 0;
        for (int i = 0; i < nmat; ++i) {
            const MatDesc& m = mats[i];
            c.mat[i] = GemvMat{m.meta, m.values, m.y, m.y_acc, m.gamma, m.rows, m.meta_stride, m.values_stride, blocks};
            blocks += (m.rows + rpc - 1) / rpc;
        }
        const size_t smem = kLaneLutBytes + 16 + ((rpc * c.upr * 4 + 15) & ~15) + (IN == IN_F16 ? static_cast<size_t>(cols) : 0);
        int rc;
        if ((rc = ensure_smem(gemv_cols_kernel<IN, OUT>, smem))) return rc;
        return launch(name, gemv_cols_kernel<IN, OUT>, dim3(blocks), dim3(kColsThreads), smem, stream, c);
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
    const size_t smem = kLutBytes + ((rpc * 4 + 15) & ~15) + static_cast<size_t>(cols);
    int rc;
    if ((rc = ensure_smem(gemv_units_kernel<IN, OUT>, smem))) return rc;
    return launch(name, gemv_units_kernel<IN, OUT>, dim3(blocks), dim3(kThreads), smem, stream, a);
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
