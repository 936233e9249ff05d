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
//   * gathers the four non-zero x bytes of two groups with one PRMT whose selector comes from a
//     per-lane table indexed by the two bitmaps, takes their signs from a second per-lane table
//     and consumes two groups with one dp4a (the pair kernel below);
//   * reduces the per-thread partials of a row with a segmented shuffle scan.
// A "unit" is 128 consecutive columns of one row: 16 B of meta + 8 B of values.
#include "fused_ops.cuh"
#include "producers.cuh"

namespace spb {

// The activation producers (IN_*) and output kinds (OUT_*) live in producers.cuh.

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
    const void* x;          // int8 (IN_I8), half (IN_F16*), residual x_in (IN_RESNORM), gate (IN_RELU2)
    const void* x2;         // delta (IN_RESNORM, may be null), up (IN_RELU2)
    const float* w_sub;     // sub-norm weights (IN_RESNORM on delta, IN_RELU2), may be null
    const float* w_norm;    // norm weights (IN_RESNORM)
    void* x_out;            // updated residual stream (IN_RESNORM)
    float eps;
    const float* d_absmax;  // device scalar (IN_I8 with scaled output, IN_F16); read after the dependency wait
    int cols;
    int upr;  // units per row = cols / 128
    int rpc;  // rows per block
    RopeScatter rope;  // d_pos set: the launch is q, k, v and rotates / scatters its rows (pair kernel, OUT_F16)
};

constexpr int kThreads = kProdThreads;

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

// ---------------------------------------------------------------------------
// Pair kernel (the default).
//
// Block = rpc rows of one matrix = rpc * upr units, one unit per thread, two phases:
//   phase A (independent of any predecessor): stream the unit's 24 bytes of weights, copy the tables;
//   phase B (after the dependency wait): stage x, expand, multiply-add, reduce, store.
// Two groups (one meta byte, one sign nibble) are consumed at a time:
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
__global__ void __launch_bounds__(kThreads, (IN >= IN_RESNORM) ? 2 : 4) gemv_pairs_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) uint8_t psmem[];
    // [sel 15360][sgn 2048][red 64 floats][partials upr*pitch ints (16-aligned)][x cols bytes]
    // [half scratch 2*cols bytes, only for the producers that normalise][their norm weights: cols floats each]
    const uint32_t win_s = smem_u32(psmem);
    uint8_t* win = psmem;
    const int pitch = a.rpc | 1;
    float* red = reinterpret_cast<float*>(win + kSelBytes + kSgnBytes);
    int* partial = reinterpret_cast<int*>(win + kSelBytes + kSgnBytes + 256);
    uint4* xs = reinterpret_cast<uint4*>(win + kSelBytes + kSgnBytes + 256 + ((a.upr * pitch * 4 + 15) & ~15));

    const int tid = threadIdx.x, lane = tid & 31;
    int mi = 0;
    if (a.nmat > 1 && static_cast<int>(blockIdx.x) >= a.mat[1].blk_begin) mi = 1;
    if (a.nmat > 2 && static_cast<int>(blockIdx.x) >= a.mat[2].blk_begin) mi = 2;
    const GemvMat& M = a.mat[mi];
    const int r_lo = (blockIdx.x - M.blk_begin) * a.rpc;
    const int nrows = min(a.rpc, M.rows - r_lo);
    const int nunits = nrows * a.upr;

    grid_dep_launch();

    // The norm weights of the normalising producers are constants: they start towards shared memory now, so that
    // the producer does not go to L2 for them between its reductions.
    ProducerArgs pa{a.x, a.x2, a.w_sub, a.w_norm, a.x_out, a.eps, a.d_absmax, a.cols};
    if (IN >= IN_RESNORM) {
        float* wbuf = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xs) + 3 * a.cols);
        auto stage = [&](const float* src, float* dst) {
            for (int q = tid; q < (a.cols >> 2); q += kThreads)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst + 4 * q)), "l"(src + 4 * q) : "memory");
        };
        if (IN == IN_RESNORM) {
            stage(a.w_norm, wbuf);
            pa.w_norm = wbuf;
            wbuf += a.cols;
        }
        if (a.w_sub) {
            stage(a.w_sub, wbuf);
            pa.w_sub = wbuf;
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    // ---- phase A: weights of the first pass, tables, expansion to selectors and signs ---------
    const int npass = (nunits + kThreads - 1) / kThreads;
    uint4 m = make_uint4(0, 0, 0, 0);
    uint2 v = make_uint2(0, 0);
    auto load_unit = [&](int u, uint4& mm, uint2& vv) {
        if (u < nunits) {
            const int r = u / a.upr, c = u - r * a.upr;
            const size_t row = static_cast<size_t>(r_lo + r);
            mm = ld_stream_v4(M.meta + row * M.meta_stride + c * 4);
            vv = ld_stream_v2(M.values + row * M.values_stride + c * 2);
        }
    };
    load_unit(tid, m, v);
    {
        const uint4* src = reinterpret_cast<const uint4*>(&g_pair_lut);
        uint4* dst = reinterpret_cast<uint4*>(win);
        for (int q = tid; q < (kSelBytes + kSgnBytes) / 16; q += kThreads) dst[q] = __ldg(src + q);
    }
    __syncthreads();  // tables complete

    // produced by a volatile statement after the barrier, so that no table load can be
    // scheduled above it
    uint32_t sel_lane;
    asm volatile("add.u32 %0, %1, %2;" : "=r"(sel_lane) : "r"(win_s), "r"(lane * 4) : "memory");
    const uint32_t sgn_lane = sel_lane + kSelBytes;
    uint32_t sel[16], sgn[16];
    auto expand = [&](const uint4& mm, const uint2& vv) {
        const uint32_t mw[4] = {mm.x, mm.y, mm.z, mm.w};
        const uint32_t vw[2] = {vv.x, vv.y};
#pragma unroll
        for (int p = 0; p < 16; ++p) {  // groups 2p and 2p+1: meta byte p, sign nibble p
            const int ms = 8 * (p & 3) - 7, ss = 4 * (p & 7) - 7;
            sel[p] = lds32(((ms >= 0 ? (mw[p >> 2] >> ms) : (mw[p >> 2] << -ms)) & (0x77u << 7)) + sel_lane);
            sgn[p] = lds32(((ss >= 0 ? (vw[p >> 3] >> ss) : (vw[p >> 3] << -ss)) & (0xFu << 7)) + sgn_lane);
        }
    };
    expand(m, v);

    // ---- phase B: activations (only now may a predecessor's output be read) ------------------
    grid_dep_wait();
    // the position of the fused rotation is asked for now, not in the epilogue where it would be a trip to L2 on the
    // critical path (volatile: the load stays here)
    int rope_pos = 0;
    if (OUT == OUT_F16 && a.rope.d_pos) asm volatile("ld.global.s32 %0, [%1];" : "=r"(rope_pos) : "l"(a.rope.d_pos));
    if (IN >= IN_RESNORM) asm volatile("cp.async.wait_group 0;" ::: "memory");  // (each weight is first read after a block-wide reduction)
    const float absmax = produce_x<IN, OUT>(pa, xs, reinterpret_cast<__half*>(xs) + (a.cols >> 1), red,
                                             blockIdx.x == 0);
    __syncthreads();

    for (int pass = 0; pass < npass; ++pass) {
        const int u = pass * kThreads + tid;
        uint4 mn = make_uint4(0, 0, 0, 0);
        uint2 vn = make_uint2(0, 0);
        if (pass + 1 < npass) load_unit(u + kThreads, mn, vn);  // next pass's weights in flight
        if (pass > 0) expand(m, v);
        if (u < nunits) {
            const int rl = u / a.upr, cb = u - rl * a.upr;
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
        m = mn;
        v = vn;
    }
    __syncthreads();

    // one thread per row folds its partials (consecutive rows -> consecutive banks)
    const float dq = (OUT != OUT_I32) ? dequant_scale(M.gamma, absmax) : 0.0f;
    if (OUT == OUT_F16 && a.rope.d_pos) {
        // q, k, v: a thread takes the two rows of a rotation pair (blocks start on even rows and hold an even number)
        const int pos = rope_pos, hd = a.rope.head_dim;
        for (int pr = tid; 2 * pr < nrows; pr += kThreads) {
            int s0 = 0, s1 = 0;
            for (int c = 0; c < a.upr; ++c) {
                s0 += partial[c * pitch + 2 * pr];
                s1 += partial[c * pitch + 2 * pr + 1];
            }
            const int row = r_lo + 2 * pr, head = row / hd, d = row - head * hd;
            const __half h0 = __float2half_rn(__fmul_rn(static_cast<float>(s0), dq));
            const __half h1 = __float2half_rn(__fmul_rn(static_cast<float>(s1), dq));
            __half2 outv = __halves2half2(h0, h1);
            if (mi < 2) {
                __half y0, y1;
                rope_rotate(__half2float(h0), __half2float(h1), pos, d >> 1, hd, a.rope.theta, y0, y1);
                outv = __halves2half2(y0, y1);
            }
            __half* dst = mi == 0 ? static_cast<__half*>(M.y) + row
                                  : static_cast<__half*>(mi == 1 ? a.rope.kcache : a.rope.vcache) +
                                        (static_cast<size_t>(head) * a.rope.max_seq_len + pos) * hd + d;
            *reinterpret_cast<__half2*>(dst) = outv;
        }
        return;
    }
    for (int lr = tid; lr < nrows; lr += kThreads) {
        int s = 0;
        for (int c = 0; c < a.upr; ++c) s += partial[c * pitch + lr];
        store_out(M, r_lo + lr, s, dq, OUT);
    }
}

// ---------------------------------------------------------------------------------------------------
// The tensor-core form with the activation producers in front (see gemv_mmasp.cu for the scheme and the
// operand layouts of mma.sp m16n8k64): up to kMaxMats matrices per launch, any IN_* producer, any OUT_*.
// A block owns 16 * rb rows of one matrix and the whole K extent; its raw slab arrives by 16-byte
// cp.async before the dependency wait; after it the block produces the int8 activation vector exactly as
// the SIMT kernel does (produce_x), re-orders it for the B registers and runs the step loop.
struct MmaGeom {
    int steps;    // cols / 64
    int ks;       // warps per row block (power of two <= 8)
    int ks_log2;
    int rb;       // row blocks per thread block = 8 / ks
    int spw;      // steps per warp
    int mpitch;   // shared-memory row pitch of the bitmap words, in words (an odd multiple of 4)
    int vpitch;   // same for the sign words
};

__device__ __forceinline__ uint32_t mma_index_pairs(uint32_t m) {
    // eight bitmaps (two of four bits set each) -> eight index pairs {low index | high index << 2}
    const uint32_t mr = m >> 1, ml = m << 1;
    const uint32_t t1 = (0x11111111u & (~m & mr)) | (~0x11111111u & (mr | ~m));
    const uint32_t t2 = (0x22222222u & (~ml & ~m)) | (~0x22222222u & (m | ml));
    return (t1 & 0x55555555u) | (t2 & 0xAAAAAAAAu);
}

template <int IN, int OUT>
__global__ void __launch_bounds__(kThreads, (IN >= IN_RESNORM) ? 2 : 4) gemv_mma_kernel(const GemvArgs a, const MmaGeom geo) {
    __shared__ __align__(16) uint32_t sgn_tab[16 * 32];  // entry (nibble n, lane l) at word n * 32 + l
    __shared__ int redi[8 * 16];
    // dynamic: [x int8, swizzled as produce_x writes it: cols][half scratch of the normalising producers: 2 cols]
    //          [red: 64 floats][x in B-register order: cols][bitmap rows][sign rows]
    extern __shared__ __align__(128) uint8_t msmem[];
    const int hb = (IN >= IN_RESNORM) ? 2 * a.cols : 0;
    uint4* xs_sw = reinterpret_cast<uint4*>(msmem);
    float* red = reinterpret_cast<float*>(msmem + a.cols + hb);
    const uint32_t dyn_s = smem_u32(msmem);
    const uint32_t tab_s = smem_u32(sgn_tab);
    const uint32_t xs_s = dyn_s + static_cast<uint32_t>(a.cols + hb) + 256u;
    const uint32_t ms_s = xs_s + static_cast<uint32_t>(a.cols);
    const int nrows_blk = 16 * geo.rb;
    const uint32_t vs_s = ms_s + static_cast<uint32_t>(nrows_blk * geo.mpitch) * 4u;

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);  // through a shuffle: known to be uniform over the warp
    int mi = 0;
    if (a.nmat > 1 && static_cast<int>(blockIdx.x) >= a.mat[1].blk_begin) mi = 1;
    if (a.nmat > 2 && static_cast<int>(blockIdx.x) >= a.mat[2].blk_begin) mi = 2;
    const GemvMat& M = a.mat[mi];
    const int row0 = (blockIdx.x - M.blk_begin) * nrows_blk;
    const int valid = min(nrows_blk, M.rows - row0);

    // the raw slab: a warp per row, consecutive lanes on consecutive 16-byte chunks (bitmaps, then signs)
    {
        const int mch = a.cols >> 7, cpr = mch + (a.cols >> 8);
        for (int k = lane; k < cpr; k += 32) {
            const bool is_m = k < mch;
            const uint8_t* src = is_m ? reinterpret_cast<const uint8_t*>(M.meta) + k * 16
                                      : reinterpret_cast<const uint8_t*>(M.values) + (k - mch) * 16;
            const size_t src_pitch = static_cast<size_t>(is_m ? M.meta_stride : M.values_stride) * 4u;
            const uint32_t dst = is_m ? ms_s + static_cast<uint32_t>(k) * 16u : vs_s + static_cast<uint32_t>(k - mch) * 16u;
            const uint32_t dst_pitch = static_cast<uint32_t>(is_m ? geo.mpitch : geo.vpitch) * 4u;
            src += static_cast<size_t>(row0 + warp) * src_pitch;
            for (int r = warp; r < valid; r += 8) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + static_cast<uint32_t>(r) * dst_pitch), "l"(src)
                             : "memory");
                src += 8 * src_pitch;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {  // byte b of an entry = -1 if bit b of the nibble is set, else +1
        const uint32_t i = tid + j * kThreads;
        const uint32_t t = ((i >> 5) * 0x00204081u) & 0x01010101u;
        sgn_tab[i] = (t * 0xFEu) | 0x01010101u;
    }

    const int g = lane >> 2, tig = lane & 3;
    const int rbi = warp >> geo.ks_log2, kq = warp & (geo.ks - 1);
    const int s_begin = kq * geo.spw, s_end = min(geo.steps, s_begin + geo.spw);
    const uint32_t lane_or = static_cast<uint32_t>(lane) << 2;
    const uint32_t rot_lo = (static_cast<uint32_t>(tig) * 4u + 25u) & 31u, rot_hi = (static_cast<uint32_t>(tig) * 4u + 9u) & 31u;
    uint32_t me_p = ms_s + static_cast<uint32_t>((rbi * 16 + g + 8 * (tig & 1)) * geo.mpitch + (tig >> 1) + 2 * s_begin) * 4u;
    uint32_t v0_p = vs_s + static_cast<uint32_t>((rbi * 16 + g) * geo.vpitch + s_begin) * 4u;
    const uint32_t v_half = static_cast<uint32_t>(8 * geo.vpitch) * 4u;
    uint32_t xq_p = xs_s + static_cast<uint32_t>(tig) * 16u + static_cast<uint32_t>(s_begin) * 64u;

    // ---- after the dependency: the activation vector --------------------------------------------------
    grid_dep_wait();
    grid_dep_launch();  // the successor is let in only now (see gemv_mmasp.cu)
    const float absmax = produce_x<IN, OUT>(a, xs_sw, reinterpret_cast<__half*>(xs_sw) + (a.cols >> 1), red,
                                             blockIdx.x == 0);
    __syncthreads();
    // x in B-register order: xs[step][tig][j][0..3] = x[64 step + 16 j + 4 tig ..+3]
    for (int q = tid; q < (a.cols >> 4); q += kThreads) {
        const int c = q >> 3, i = q & 7;
        const uint4 xv = xs_sw[(c << 3) + (i ^ (c & 7))];
        const uint32_t d = xs_s + (static_cast<uint32_t>(q) >> 2) * 64u + (static_cast<uint32_t>(q) & 3u) * 4u;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d), "r"(xv.x) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 16u), "r"(xv.y) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 32u), "r"(xv.z) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 48u), "r"(xv.w) : "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // the slab, the table and x are visible

    int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
    auto step = [&](uint32_t w0, uint32_t w1, uint32_t me_off, uint32_t x_off) {
        const uint32_t e = mma_index_pairs(lds32(me_p + me_off));
        const uint32_t a0 = lds32(tab_s + ((__funnelshift_r(w0, w0, rot_lo) & 0x780u) | lane_or));
        const uint32_t a1 = lds32(tab_s + ((__funnelshift_r(w1, w1, rot_lo) & 0x780u) | lane_or));
        const uint32_t a2 = lds32(tab_s + ((__funnelshift_r(w0, w0, rot_hi) & 0x780u) | lane_or));
        const uint32_t a3 = lds32(tab_s + ((__funnelshift_r(w1, w1, rot_hi) & 0x780u) | lane_or));
        uint32_t b0, b1, b2, b3;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(xq_p + x_off));
        asm volatile(
            "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
            "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
            : "+r"(c0), "+r"(c1), "+r"(c2), "+r"(c3)
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(b2), "r"(b3), "r"(e));
    };
    auto advance = [&](uint32_t steps) {
        me_p += 8u * steps;
        v0_p += 4u * steps;
        xq_p += 64u * steps;
    };
    int st = s_begin;
    for (; st < s_end && (st & 3) != 0; ++st) {
        step(lds32(v0_p), lds32(v0_p + v_half), 0u, 0u);
        advance(1u);
    }
    for (; st + 4 <= s_end; st += 4) {  // four steps share one 16-byte read of each row's sign words
        uint4 w0, w1;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w0.x), "=r"(w0.y), "=r"(w0.z), "=r"(w0.w) : "r"(v0_p));
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w1.x), "=r"(w1.y), "=r"(w1.z), "=r"(w1.w) : "r"(v0_p + v_half));
        step(w0.x, w1.x, 0u, 0u);
        step(w0.y, w1.y, 8u, 64u);
        step(w0.z, w1.z, 16u, 128u);
        step(w0.w, w1.w, 24u, 192u);
        advance(4u);
    }
    for (; st < s_end; ++st) {
        step(lds32(v0_p), lds32(v0_p + v_half), 0u, 0u);
        advance(1u);
    }
    if (tig == 0) {  // column 0 of the tile: rows g (c0) and g + 8 (c2)
        redi[warp * 16 + g] = c0;
        redi[warp * 16 + g + 8] = c2;
    }
    __syncthreads();
    const float dq = (OUT != OUT_I32) ? dequant_scale(M.gamma, absmax) : 0.0f;
    if (tid < valid) {
        const int rblk = tid >> 4, r = tid & 15;
        int acc = 0;
        for (int k = 0; k < geo.ks; ++k) acc += redi[((rblk << geo.ks_log2) + k) * 16 + r];
        store_out(M, row0 + tid, acc, dq, OUT);
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
    return ensure_dynamic_smem("sparse-ternary GEMV", kernel, bytes);
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

// 0 automatic (warp-level sparse MMA kernel where the layout allows it, else the pair kernel), 1 pair kernel,
// 4 warp-level sparse MMA kernel (also for the fused-producer forms)
static int g_gemv_variant = 0;

bool gemv_mmasp_supported(const uint32_t* meta, const uint32_t* values, const int8_t* x, int rows, int cols,
                          int meta_stride, int values_stride);
int gemv_mmasp_launch(const char* name, const uint32_t* meta, const uint32_t* values, const int8_t* x, void* y,
                      int32_t* y_acc, const float* d_absmax, float gamma, int out_mode, int rows, int cols,
                      int meta_stride, int values_stride, void* stream);

// Where the activation vector of a launch comes from (see the IN_* producers).
struct XDesc {
    const void* x = nullptr;
    const void* x2 = nullptr;
    const float* w_sub = nullptr;
    const float* w_norm = nullptr;
    void* x_out = nullptr;
    float eps = 0.0f;
    const float* d_absmax = nullptr;
    const RopeScatter* rope = nullptr;
};

// Launches up to kMaxMats matrices that share the activation vector as one grid.
template <int IN, int OUT>
static int run_gemv(const char* name, const MatDesc* mats, int nmat, const XDesc& xd, int cols, void* stream) {
    if (nmat < 1 || nmat > kMaxMats) return fail(SPB_E_INVALID, "%s: %d matrices in one launch", name, nmat);
    if (cols < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    int total_rows = 0;
    for (int i = 0; i < nmat; ++i) {
        if (mats[i].rows < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
        total_rows += mats[i].rows;
    }
    if (total_rows == 0 || cols == 0) return SPB_OK;
    if (cols % 4 != 0) return fail(SPB_E_INVALID, "%s: cols=%d is not a multiple of 4", name, cols);
    if (!xd.x) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if ((IN == IN_F16 || (IN == IN_I8 && OUT != OUT_I32)) && !xd.d_absmax)
        return fail(SPB_E_INVALID, "%s: d_absmax is null", name);
    if (IN == IN_RESNORM && (!xd.w_norm || !xd.x_out)) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (IN == IN_RELU2 && !xd.x2) return fail(SPB_E_INVALID, "%s: null pointer", name);
    bool fast = cols % 128 == 0 && cols / 128 <= kThreads && aligned(xd.x, 16) && cols <= 65536;
    for (int i = 0; i < nmat; ++i) {
        const MatDesc& m = mats[i];
        if (m.rows == 0) continue;
        if (!m.meta || !m.values || !m.y) return fail(SPB_E_INVALID, "%s: null pointer", name);
        if (m.meta_stride < (cols / 4 + 7) / 8 || m.values_stride < (cols / 4 + 15) / 16)
            return fail(SPB_E_INVALID, "%s: row stride shorter than a row", name);
        fast = fast && m.meta_stride % 4 == 0 && m.values_stride % 2 == 0 && aligned(m.meta, 16) &&
               aligned(m.values, 8);
    }
    if (!fast && IN >= IN_F16_AMAX)
        return fail(SPB_E_UNSUPPORTED, "%s: this layout has no fused-producer kernel (cols %% 128, strides, alignment)", name);

    GemvArgs a{};
    a.nmat = nmat;
    a.x = xd.x;
    a.x2 = xd.x2;
    a.w_sub = xd.w_sub;
    a.w_norm = xd.w_norm;
    a.x_out = xd.x_out;
    a.eps = xd.eps;
    a.d_absmax = xd.d_absmax;
    a.cols = cols;
    const int sms = sm_count();
    int rpc = 8;  // generic path: a warp per row, 8 rows per block
    if (fast) {
        a.upr = cols / 128;
        const int fill = max(1, kThreads / a.upr);       // rows that fill the block
        const int spread = (total_rows + sms - 1) / sms;  // rows per block at one block per SM
        rpc = max(1, min(fill, spread));
        if (IN >= IN_F16_AMAX) {
            // every block recomputes the activation vector: use about two fat blocks per SM, each
            // making several passes over its rows, instead of many thin ones
            const int want = (total_rows + 2 * sms - 1) / (2 * sms);
            const int cap = max(fill, (32 * 1024 / 4) / a.upr);
            rpc = max(rpc, min(cap, (want + fill - 1) / fill * fill));
        }
    }
    if (xd.rope) {
        if (OUT != OUT_F16 || nmat != 3 || !fast || mats[0].rows % 2 || mats[1].rows % 2 || mats[2].rows % 2 ||
            xd.rope->head_dim % 2 || !aligned(mats[0].y, 4) || !aligned(xd.rope->kcache, 4) || !aligned(xd.rope->vcache, 4))
            return fail(SPB_E_UNSUPPORTED, "%s: this q/k/v group cannot take the fused rotation", name);
        a.rope = *xd.rope;
        rpc += rpc & 1;  // rotation pairs never straddle two blocks
    }
    a.rpc = rpc;
    int blocks = 0;
    for (int i = 0; i < nmat; ++i) {
        const MatDesc& m = mats[i];
        a.mat[i] = GemvMat{m.meta, m.values, m.y, m.y_acc, m.gamma, m.rows, m.meta_stride, m.values_stride, blocks};
        blocks += (m.rows + rpc - 1) / rpc;
    }
    int rc;
    // tensor-core form with producers: every matrix must have 16-byte aligned rows in both arrays
    // (opt-in: in a dependent chain, which is what a decode step is, the SIMT kernel is quicker because it expands
    // its weights before the dependency wait; measured 530 against 614 tok/s)
    bool mma_ok = fast && g_gemv_variant == 4 && cols % 256 == 0 && cols <= 16384 && !(IN == IN_I8 && nmat == 1) && !xd.rope;
    for (int i = 0; i < nmat && mma_ok; ++i)
        mma_ok = mats[i].rows == 0 || (mats[i].meta_stride % 4 == 0 && mats[i].values_stride % 4 == 0 &&
                                       aligned(mats[i].meta, 16) && aligned(mats[i].values, 16));
    if (mma_ok) {
        MmaGeom geo{};
        geo.steps = cols / 64;
        int row_blocks = 0;
        for (int i = 0; i < nmat; ++i) row_blocks += (mats[i].rows + 15) / 16;
        geo.ks = 8;
        while (geo.ks > 1 && geo.steps / geo.ks < 16) geo.ks >>= 1;
        while (geo.ks < 8 && row_blocks * geo.ks < 2 * sms && geo.steps / (2 * geo.ks) >= 8) geo.ks <<= 1;
        while (geo.ks > geo.steps) geo.ks >>= 1;
        geo.rb = 8 / geo.ks;
        geo.ks_log2 = geo.ks == 8 ? 3 : geo.ks == 4 ? 2 : geo.ks == 2 ? 1 : 0;
        geo.spw = (geo.steps + geo.ks - 1) / geo.ks;
        auto pitch = [](int words) { return words % 8 == 4 ? words : words + ((4 - words % 8) + 8) % 8; };
        geo.mpitch = pitch(cols / 32);
        geo.vpitch = pitch(cols / 64);
        a.rpc = 16 * geo.rb;
        int nblk = 0;
        for (int i = 0; i < nmat; ++i) {
            a.mat[i].blk_begin = nblk;
            nblk += (mats[i].rows + a.rpc - 1) / a.rpc;
        }
        const size_t msmem = static_cast<size_t>(cols) * (IN >= IN_RESNORM ? 3 : 1) + 256 + cols +
                             static_cast<size_t>(16 * geo.rb) * (geo.mpitch + geo.vpitch) * 4;
        if (msmem <= 200 * 1024) {
            if ((rc = ensure_smem(gemv_mma_kernel<IN, OUT>, msmem))) return rc;
            return launch(name, gemv_mma_kernel<IN, OUT>, dim3(nblk), dim3(kThreads), msmem, stream, a, geo);
        }
        a.rpc = rpc;  // does not fit: back to the SIMT form
        for (int i = 0, b = 0; i < nmat; ++i) {
            a.mat[i].blk_begin = b;
            b += (mats[i].rows + rpc - 1) / rpc;
        }
    }
    if constexpr (IN == IN_I8) {
        if (fast && nmat == 1 && (g_gemv_variant == 0 || g_gemv_variant == 4) &&
            gemv_mmasp_supported(mats[0].meta, mats[0].values, static_cast<const int8_t*>(xd.x), mats[0].rows, cols,
                                 mats[0].meta_stride, mats[0].values_stride)) {
            return gemv_mmasp_launch(name, mats[0].meta, mats[0].values, static_cast<const int8_t*>(xd.x), mats[0].y,
                                     mats[0].y_acc, xd.d_absmax, mats[0].gamma, OUT, mats[0].rows, cols,
                                     mats[0].meta_stride, mats[0].values_stride, stream);
        }
    }
    if constexpr (IN <= IN_F16) {
        if (!fast) return launch(name, gemv_generic_kernel<IN, OUT>, dim3(blocks), dim3(kThreads), 0, stream, a);
    }
    const size_t smem = kSelBytes + kSgnBytes + 256 + ((a.upr * (a.rpc | 1) * 4 + 15) & ~15) +
                        static_cast<size_t>(cols) * (IN == IN_RESNORM ? 3 + 8 : IN == IN_RELU2 ? 3 + 4 : 1);
    if ((rc = ensure_smem(gemv_pairs_kernel<IN, OUT>, smem))) return rc;
    return launch(name, gemv_pairs_kernel<IN, OUT>, dim3(blocks), dim3(kThreads), smem, stream, a);
}

// gemv_prepared.cu
bool prepared_group_fused_supported(const int* rows, int nmat, int cols);
int prepared_group_fused(int in, const void* const* prep, void* const* out_half, const float* gamma, const int* rows, int nmat,
                         const ProducerArgs& p, const RopeScatter* rope, void* stream);

// The group on prepared copies of its matrices, when it has them all and fits; 1 = not applicable.
static int try_prepared(int in, const BitLinearGroup& g, const XDesc& xd, void* stream) {
    for (int i = 0; i < g.nmat; ++i)
        if (!g.prep[i]) return 1;
    if (g_gemv_variant != 0 || !prepared_group_fused_supported(g.rows, g.nmat, g.cols)) return 1;
    if (!aligned(xd.x, 16) || (xd.x2 && !aligned(xd.x2, 16)) || (xd.w_norm && !aligned(xd.w_norm, 16)) ||
        (xd.w_sub && !aligned(xd.w_sub, 16)))
        return 1;
    ProducerArgs p{};
    p.x = xd.x; p.x2 = xd.x2; p.w_sub = xd.w_sub; p.w_norm = xd.w_norm; p.x_out = xd.x_out; p.eps = xd.eps;
    p.d_absmax = xd.d_absmax; p.cols = g.cols;
    return prepared_group_fused(in, g.prep, g.out, g.gamma, g.rows, g.nmat, p, xd.rope, stream);
}

static int fill_mats(MatDesc* d, const BitLinearGroup& g) {
    if (g.nmat < 1 || g.nmat > kMaxMats) return fail(SPB_E_INVALID, "bitlinear group: %d matrices", g.nmat);
    for (int i = 0; i < g.nmat; ++i)
        d[i] = MatDesc{g.meta[i], g.values[i], g.out[i], nullptr, g.gamma[i], g.rows[i], g.ms[i], g.vs[i]};
    return SPB_OK;
}

// Engine-internal launchers: several BitLinear layers on one activation vector in one launch.
int bitlinear_q8_group(const BitLinearGroup& g, const int8_t* xq, const float* d_absmax, void* stream) {
    MatDesc d[kMaxMats];
    if (int rc = fill_mats(d, g)) return rc;
    XDesc xd;
    xd.x = xq;
    xd.d_absmax = d_absmax;
    return run_gemv<IN_I8, OUT_F16>("bitlinear_q8_group", d, g.nmat, xd, g.cols, stream);
}

int bitlinear_amax_group(const BitLinearGroup& g, const void* x_half, void* stream) {
    MatDesc d[kMaxMats];
    if (int rc = fill_mats(d, g)) return rc;
    XDesc xd;
    xd.x = x_half;
    if (const int rc = try_prepared(IN_F16_AMAX, g, xd, stream); rc != 1) return rc;
    return run_gemv<IN_F16_AMAX, OUT_F16>("bitlinear_amax_group", d, g.nmat, xd, g.cols, stream);
}

int bitlinear_resnorm_group(const BitLinearGroup& g, const void* x_in, const void* delta, const float* w_sub,
                            const float* w_norm, void* x_out, float eps, void* stream, const RopeScatter* rope) {
    MatDesc d[kMaxMats];
    if (int rc = fill_mats(d, g)) return rc;
    XDesc xd;
    xd.x = x_in;
    xd.x2 = delta;
    xd.w_sub = w_sub;
    xd.w_norm = w_norm;
    xd.x_out = x_out;
    xd.eps = eps;
    xd.rope = rope;
    if (const int rc = try_prepared(IN_RESNORM, g, xd, stream); rc != 1) return rc;
    return run_gemv<IN_RESNORM, OUT_F16>("bitlinear_resnorm_group", d, g.nmat, xd, g.cols, stream);
}

int bitlinear_relu2_group(const BitLinearGroup& g, const void* gate, const void* up, const float* w_sub, float eps,
                          void* stream) {
    MatDesc d[kMaxMats];
    if (int rc = fill_mats(d, g)) return rc;
    XDesc xd;
    xd.x = gate;
    xd.x2 = up;
    xd.w_sub = w_sub;
    xd.eps = eps;
    if (const int rc = try_prepared(IN_RELU2, g, xd, stream); rc != 1) return rc;
    return run_gemv<IN_RELU2, OUT_F16>("bitlinear_relu2_group", d, g.nmat, xd, g.cols, stream);
}

// True when a BitLinear group can take the fused-producer kernels.
bool bitlinear_group_is_fast(const BitLinearGroup& g) {
    if (g.cols % 128 != 0 || g.cols / 128 > kThreads || g.cols > 65536) return false;
    for (int i = 0; i < g.nmat; ++i)
        if (g.ms[i] % 4 || g.vs[i] % 2 || !aligned(g.meta[i], 16) || !aligned(g.values[i], 8)) return false;
    return true;
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
    XDesc xd;
    xd.x = x;
    return run_gemv<IN_I8, OUT_I32>("spb_sparse_ternary_gemv", &d, 1, xd, cols, stream);
}

extern "C" int spb_sparse_ternary_gemv_scaled(const uint32_t* meta, const uint32_t* values,
                                              const int8_t* x, float* y, int32_t* y_acc,
                                              const float* d_absmax, float gamma, int rows, int cols,
                                              int meta_row_stride, int values_row_stride, void* stream) {
    MatDesc d{meta, values, y, y_acc, gamma, rows, meta_row_stride, values_row_stride};
    XDesc xd;
    xd.x = x;
    xd.d_absmax = d_absmax;
    return run_gemv<IN_I8, OUT_F32>("spb_sparse_ternary_gemv_scaled", &d, 1, xd, cols, stream);
}

extern "C" int spb_fused_sparse_bitlinear(const uint32_t* meta, const uint32_t* values, const void* x,
                                          void* output, const float* d_absmax, float gamma, int rows,
                                          int cols, int meta_row_stride, int values_row_stride,
                                          void* stream) {
    MatDesc d{meta, values, output, nullptr, gamma, rows, meta_row_stride, values_row_stride};
    XDesc xd;
    xd.x = x;
    xd.d_absmax = d_absmax;
    return run_gemv<IN_F16, OUT_F16>("spb_fused_sparse_bitlinear", &d, 1, xd, cols, stream);
}

extern "C" int spb_sparse_bitlinear_q8(const uint32_t* meta, const uint32_t* values, const int8_t* xq,
                                       void* output, const float* d_absmax, float gamma, int rows,
                                       int cols, int meta_row_stride, int values_row_stride,
                                       void* stream) {
    MatDesc d{meta, values, output, nullptr, gamma, rows, meta_row_stride, values_row_stride};
    XDesc xd;
    xd.x = xq;
    xd.d_absmax = d_absmax;
    return run_gemv<IN_I8, OUT_F16>("spb_sparse_bitlinear_q8", &d, 1, xd, cols, stream);
}
