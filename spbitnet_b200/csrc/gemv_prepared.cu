// Sparse-ternary GEMV on weights re-laid once for the warp-level sparse MMA ("prepared" weights), sm_100a.
//
// The GEMV on the packed format (gemv_mmasp.cu) tops out near 3 TB/s whatever the matrix size: per 64-column step
// of 16 rows a warp issues about 23 instructions and 12 shared-memory wavefronts to turn 192 bytes of bitmaps and
// sign bits into the operands of one mma.sp.  An engine that owns its weights (it uploads them once) can pay that
// conversion once instead.  The prepared form keeps 1.5 bits per weight and holds, per tile of 16 rows and "quad"
// of four steps (256 columns), 768 contiguous bytes in the order the lanes consume them:
//
//   [lane 0..31][4 words]   the metadata operand of steps 4q .. 4q+3: the index pairs of bitmap word
//                           2 s + (tig >> 1) of row 16 t + g + 8 (tig & 1)            (g = lane / 4, tig = lane % 4)
//   [lane 0..31][64 bits]   the sign bits of the lane's four A registers of those steps, 16 bits a step:
//                           bit 4 k + r = sign of byte k of register r
//                           (r = 0: row g, compressed columns 4 tig..; 1: row g + 8, same; 2, 3: columns 16 + 4 tig..)
//
// so a warp reads its weights straight from global memory with one 16-byte and one 8-byte load per lane and quad,
// fully coalesced, and nothing of them passes through shared memory.  A register of four sign bytes comes out of
// ONE byte permute: the 16-bit field is the selector, and the permute's source is a constant whose byte i is 0xFF
// when bit r of i is set, so byte k of the result is 0xFF (-1) or 0x00 according to bit r of selector nibble k (the
// nibble's top bit asks for sign replication, which leaves 0x00 / 0xFF as they are; register 3 takes the selector
// shifted by one).  With A in {0, -1} the step needs a second MMA with A = 1 on the same metadata and activations:
//   y = sum over kept x  +  2 * sum of (A * x)   =   S + 2 R.
// A step is about ten instructions and one shared-memory wavefront (the activation registers; only the four lanes
// of output column 0 load them).  (Turning 0x00 / 0xFF into +1 / -1 with an "or" per register and issuing a single MMA
// was measured slower, 9.5 against 8.9 us at 28672 x 8192: the four extra logic instructions cost more than the MMA.)
//
// Measured (one B200, graphs of launches over weight copies larger than L2, eight branches): 28672 x 8192 in 9.0 us =
// 4.9 TB/s against 13.9 us = 3.2 TB/s for the packed-format kernel, 8192 x 28672 9.7 against 15.6 us, 8192 x 8192 3.7
// against 4.0 us; at the 2B-4T shapes (a few MB per matrix, a handful of quads per warp) the packed-format kernel is
// the faster one (6912 x 2560: 0.94 against 1.22 us), so this form is meant for matrices of tens of megabytes.
// Two forms that cut the work by bytes instead of by row tiles (equal contiguous runs of quads, partial tiles summed
// through atomics into a workspace and finished by whoever completes a tile's count) balanced the SMs exactly and
// were slower everywhere: per block with a block-wide reduction per piece, 17.1 against 14.7 us at 28672 x 8192 as a
// chain of launches; per warp with no block-wide step, 16.5 against 14.6 us (14.0 against 8.9 us in the graph of eight
// branches): the fence and the round trip of the counting atomic drain the warp's prefetch at every hand-over.
// Also measured and dropped: asking L2 for the rest of a warp's run of quads before the dependency wait (one bulk
// prefetch per warp, or a prefetch per 128 bytes): the 70B-shape decode step got 3 - 4 % slower both ways.
#include "fused_ops.cuh"
#include "producers.cuh"
#include "spb_common.cuh"

namespace spb {

constexpr int kGpThreads = 256;
constexpr int kGpWarps = kGpThreads / 32;
constexpr int kGpQuadBytes = 768;
constexpr int kGpBlocksPerSm = 4;  // 64 registers a thread

enum { GP_OUT_I32 = 0, GP_OUT_F32 = 1, GP_OUT_F16 = 2 };

// One launch multiplies up to three matrices of the same width on one activation vector (q, k, v or gate, up): the
// tiles of the matrices are numbered through.
constexpr int kGpMaxMats = 3;
struct GpMat {
    const uint8_t* prep;
    void* y;
    float gamma;
    int rows;
    int tile0;  // the matrix's first tile in the launch's numbering
};
struct GpArgs {
    GpMat mat[kGpMaxMats];
    int nmat;
    const int8_t* x;
    int32_t* y_acc;
    const float* d_absmax;
    int out_mode;
    int cols;
    int ntiles, nquads;  // tiles of all matrices
    int ks, ks_log2;     // warps per tile (power of two <= 8); a block holds 8 / ks tiles
    int qpw;             // quads per warp
    RopeScatter rope;    // d_pos set: the matrices are q, k, v; q and k rows are rotated, k and v rows go to the cache
    LlFan fan[2];        // ndst > 0: the rows of matrix 0 / 1 go out as tagged words (half outputs, no rotation)
};

// Eight bitmaps (two of four bits set each) -> eight index pairs {low index | high index << 2}.
__device__ __forceinline__ uint32_t gp_index_pairs(uint32_t m) {
    const uint32_t mr = m >> 1, ml = m << 1;
    const uint32_t t1 = (0x11111111u & (~m & mr)) | (~0x11111111u & (mr | ~m));
    const uint32_t t2 = (0x22222222u & (~ml & ~m)) | (~0x22222222u & (m | ml));
    return (t1 & 0x55555555u) | (t2 & 0xAAAAAAAAu);
}

// One thread per (tile, quad, lane): reads the packed rows, writes the lane's 24 bytes of the prepared block.
__global__ void __launch_bounds__(256) gemv_prepare_kernel(const uint32_t* __restrict__ meta, const uint32_t* __restrict__ values,
                                                           int rows, int cols, int meta_stride, int values_stride, int ntiles,
                                                           int nquads, uint8_t* __restrict__ prep) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<long long>(ntiles) * nquads * 32) return;
    const int lane = static_cast<int>(i & 31);
    const long long tq = i >> 5;
    const int q = static_cast<int>(tq % nquads), t = static_cast<int>(tq / nquads);
    const int g = lane >> 2, tig = lane & 3;
    const int mrow = 16 * t + g + 8 * (tig & 1);
    uint32_t mw[4];
    unsigned long long sg = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int s = 4 * q + j;
        mw[j] = mrow < rows ? gp_index_pairs(meta[static_cast<size_t>(mrow) * meta_stride + 2 * s + (tig >> 1)]) : 0x44444444u;
        const int r0 = 16 * t + g, r1 = r0 + 8;
        const uint32_t w0 = r0 < rows ? values[static_cast<size_t>(r0) * values_stride + s] : 0u;
        const uint32_t w1 = r1 < rows ? values[static_cast<size_t>(r1) * values_stride + s] : 0u;
        const uint32_t nib[4] = {(w0 >> (4 * tig)) & 15u, (w1 >> (4 * tig)) & 15u, (w0 >> (16 + 4 * tig)) & 15u,
                                 (w1 >> (16 + 4 * tig)) & 15u};
        uint32_t field = 0;
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int k = 0; k < 4; ++k) field |= ((nib[r] >> k) & 1u) << (4 * k + r);
        sg |= static_cast<unsigned long long>(field) << (16 * j);
    }
    uint8_t* blk = prep + static_cast<size_t>(tq) * kGpQuadBytes;
    reinterpret_cast<uint4*>(blk)[lane] = make_uint4(mw[0], mw[1], mw[2], mw[3]);
    reinterpret_cast<uint2*>(blk + 512)[lane] = make_uint2(static_cast<uint32_t>(sg), static_cast<uint32_t>(sg >> 32));
}

// Streaming loads of one quad of a tile: the lane's four metadata words and its 64 sign bits.
__device__ __forceinline__ void gp_load_quad(const uint8_t* tile_base, int q, int lane, uint4& m, uint2& s) {
    const uint8_t* blk = tile_base + static_cast<size_t>(q) * kGpQuadBytes;
    m = ld_stream_v4(reinterpret_cast<const uint32_t*>(blk) + 4 * lane);
    s = ld_stream_v2(reinterpret_cast<const uint32_t*>(blk + 512) + 2 * lane);
}

// Quads [q_begin, q_end) of one tile times the staged activation vector; the first three quads are already in
// (m0, s0), (m1, s1), (m2, s2) (zeros past q_end).  Returns S + 2 R of output column 0 for rows g (c_lo) and g + 8
// (c_hi), meaningful in the lanes with tig == 0.
__device__ __forceinline__ void gp_run_quads(const uint8_t* tile_base, int q_begin, int q_end, uint4 m0, uint2 s0, uint4 m1,
                                             uint2 s1, uint4 m2, uint2 s2, uint32_t xs_s, int lane, int& c_lo, int& c_hi) {
    const int g = lane >> 2, tig = lane & 3;
    // R: A in {0, -1} from the sign bits; S: A = 1.  Two sets of each on alternate steps.
    int r0 = 0, r1 = 0, r2 = 0, r3 = 0, t0 = 0, t1 = 0, t2 = 0, t3 = 0;
    int u0 = 0, u1 = 0, u2 = 0, u3 = 0, v0 = 0, v1 = 0, v2 = 0, v3 = 0;
    const bool bcol = g == 0;  // the lanes that hold output column 0 of the activation operand
    uint32_t xq_p = xs_s + static_cast<uint32_t>(tig) * 16u + static_cast<uint32_t>(q_begin) * 256u;
    auto step = [&](int& c0, int& c1, int& c2, int& c3, int& d0, int& d1, int& d2, int& d3, uint32_t e, uint32_t sel, uint32_t x_off) {
        const uint32_t a0 = __byte_perm(0xFF00FF00u, 0xFF00FF00u, sel);
        const uint32_t a1 = __byte_perm(0xFFFF0000u, 0xFFFF0000u, sel);
        const uint32_t a2 = __byte_perm(0x00000000u, 0xFFFFFFFFu, sel);
        const uint32_t a3 = __byte_perm(0x00000000u, 0xFFFFFFFFu, sel >> 1);
        uint32_t b0 = 0, b1 = 0, b2 = 0, b3 = 0;
        if (bcol) asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(xq_p + x_off));
        asm volatile(
            "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
            "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
            : "+r"(c0), "+r"(c1), "+r"(c2), "+r"(c3)
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(b2), "r"(b3), "r"(e));
        asm volatile(
            "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
            "{%0, %1, %2, %3}, {%4, %4, %4, %4}, {%5, %6, %7, %8}, {%0, %1, %2, %3}, %9, 0x0;"
            : "+r"(d0), "+r"(d1), "+r"(d2), "+r"(d3)
            : "r"(0x01010101u), "r"(b0), "r"(b1), "r"(b2), "r"(b3), "r"(e));
    };
    for (int q = q_begin; q < q_end; ++q) {
        uint4 mn = make_uint4(0, 0, 0, 0);
        uint2 sn = make_uint2(0, 0);
        if (q + 3 < q_end) gp_load_quad(tile_base, q + 3, lane, mn, sn);
        step(r0, r1, r2, r3, u0, u1, u2, u3, m0.x, s0.x, 0u);
        step(t0, t1, t2, t3, v0, v1, v2, v3, m0.y, s0.x >> 16, 64u);
        step(r0, r1, r2, r3, u0, u1, u2, u3, m0.z, s0.y, 128u);
        step(t0, t1, t2, t3, v0, v1, v2, v3, m0.w, s0.y >> 16, 192u);
        xq_p += 256u;
        m0 = m1; s0 = s1;
        m1 = m2; s1 = s2;
        m2 = mn; s2 = sn;
    }
    c_lo = (u0 + v0) + 2 * (r0 + t0);
    c_hi = (u2 + v2) + 2 * (r2 + t2);
}

__global__ void __launch_bounds__(kGpThreads, kGpBlocksPerSm) gemv_prepared_kernel(const GpArgs a) {
    __shared__ int red[kGpWarps * 16];
    extern __shared__ __align__(16) uint8_t gp_raw[];  // x in B-register order: xs[step][tig][j][0..3] = x[64 step + 16 j + 4 tig ..+3]
    const uint32_t xs_s = static_cast<uint32_t>(__cvta_generic_to_shared(gp_raw));
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
    const int tiles_blk = kGpWarps >> a.ks_log2;
    const int tile = blockIdx.x * tiles_blk + (warp >> a.ks_log2), kq = warp & (a.ks - 1);
    const bool live = tile < a.ntiles;
    const int q_begin = live ? min(a.nquads, kq * a.qpw) : 0, q_end = live ? min(a.nquads, q_begin + a.qpw) : 0;
    const int g = lane >> 2, tig = lane & 3;

    // which matrix a tile belongs to (selects, not an indexed read of the parameter array)
    auto mat_of = [&](int t) { return (a.nmat > 2 && t >= a.mat[2].tile0) ? 2 : (a.nmat > 1 && t >= a.mat[1].tile0) ? 1 : 0; };
    const int wm = mat_of(live ? tile : 0);
    const uint8_t* wprep = wm == 2 ? a.mat[2].prep : wm == 1 ? a.mat[1].prep : a.mat[0].prep;
    const int wtile0 = wm == 2 ? a.mat[2].tile0 : wm == 1 ? a.mat[1].tile0 : 0;
    const uint8_t* tp = wprep + (static_cast<size_t>(live ? tile - wtile0 : 0) * a.nquads) * kGpQuadBytes;
    auto load_quad = [&](int q, uint4& m, uint2& s) {
        if (q < q_end) gp_load_quad(tp, q, lane, m, s);
    };
    // weights never depend on a predecessor: the first quads are requested before the dependency wait
    uint4 m0 = make_uint4(0, 0, 0, 0), m1 = m0, m2 = m0;
    uint2 s0 = make_uint2(0, 0), s1 = s0, s2 = s0;
    load_quad(q_begin, m0, s0);
    load_quad(q_begin + 1, m1, s1);
    load_quad(q_begin + 2, m2, s2);

    grid_dep_wait();
    float absmax_early = 0.0f;  // asked for now: in the epilogue the load would be a trip to L2 on the critical path
    int rope_pos = 0;
    if (a.out_mode != GP_OUT_I32) asm volatile("ld.global.f32 %0, [%1];" : "=f"(absmax_early) : "l"(a.d_absmax));
    if (a.rope.d_pos) asm volatile("ld.global.s32 %0, [%1];" : "=r"(rope_pos) : "l"(a.rope.d_pos));
    unsigned fan_tag = 0;  // both matrices of a launch belong to the same exchange
    if (a.fan[0].ndst) asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(fan_tag) : "l"(a.fan[0].seq));
    fan_tag += 1u;
    grid_dep_launch();
    for (int q = tid; q < (a.cols >> 4); q += kGpThreads) {
        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(a.x) + q);
        const uint32_t d = xs_s + (static_cast<uint32_t>(q) >> 2) * 64u + (static_cast<uint32_t>(q) & 3u) * 4u;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d), "r"(xv.x) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 16u), "r"(xv.y) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 32u), "r"(xv.z) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 48u), "r"(xv.w) : "memory");
    }
    __syncthreads();

    int c_lo = 0, c_hi = 0;
    gp_run_quads(tp, q_begin, q_end, m0, s0, m1, s1, m2, s2, xs_s, lane, c_lo, c_hi);
    // column 0 of the tile: lanes with tig == 0 hold rows g (register 0) and g + 8 (register 2)
    if (tig == 0) {
        red[warp * 16 + g] = c_lo;
        red[warp * 16 + g + 8] = c_hi;
    }
    __syncthreads();
    // one thread per row of the block's tiles; whole warps take part (the rotation exchanges values between lanes)
    if (tid < ((16 * tiles_blk + 31) & ~31)) {
        const int tl = tid >> 4, r = tid & 15;
        const int t = blockIdx.x * tiles_blk + tl;
        const bool in_tile = tl < tiles_blk && t < a.ntiles;
        const int mi = mat_of(in_tile ? t : 0);
        const int row = ((in_tile ? t : 0) - (mi == 2 ? a.mat[2].tile0 : mi == 1 ? a.mat[1].tile0 : 0)) * 16 + r;
        const int mrows = mi == 2 ? a.mat[2].rows : mi == 1 ? a.mat[1].rows : a.mat[0].rows;
        const bool valid = in_tile && row < mrows;
        void* y = mi == 2 ? a.mat[2].y : mi == 1 ? a.mat[1].y : a.mat[0].y;
        int acc = 0;
        if (in_tile)
            for (int k = 0; k < a.ks; ++k) acc += red[((tl << a.ks_log2) + k) * 16 + r];
        if (a.out_mode == GP_OUT_I32) {
            if (valid) static_cast<int32_t*>(y)[row] = acc;
        } else {
            const float gamma = mi == 2 ? a.mat[2].gamma : mi == 1 ? a.mat[1].gamma : a.mat[0].gamma;
            const float f = __fmul_rn(static_cast<float>(acc), dequant_scale(gamma, absmax_early));
            if (a.out_mode == GP_OUT_F32) {
                if (valid) {
                    static_cast<float*>(y)[row] = f;
                    if (a.y_acc) a.y_acc[row] = acc;
                }
            } else if (a.fan[0].ndst) {
                // rows 2 i, 2 i + 1 are neighbours in the warp: the even one stores both halves and the tag, once per
                // destination (the peers' staging areas over NVLink, this GPU's own among them)
                const uint32_t lo = __half_as_ushort(__float2half_rn(f));
                const uint32_t hi = __shfl_down_sync(0xFFFFFFFFu, lo, 1);
                if (valid && !(r & 1)) ll_fan_write(mi == 1 ? a.fan[1] : a.fan[0], static_cast<size_t>(row >> 1), lo | (hi << 16), fan_tag);
            } else if (!a.rope.d_pos) {
                if (valid) static_cast<__half*>(y)[row] = __float2half_rn(f);
            } else {
                // rows 2 i, 2 i + 1 of a head are a rotation pair and neighbours in the warp (head_dim is even, tiles
                // start at multiples of 16 rows)
                const __half hv = __float2half_rn(f);
                const float v = __half2float(hv);
                const float pv = __shfl_xor_sync(0xFFFFFFFFu, v, 1);
                const int hd = a.rope.head_dim;
                const int head = row / hd, d = row - head * hd;
                __half out = hv;
                if (mi != 2) {
                    __half y0, y1;
                    rope_rotate((r & 1) ? pv : v, (r & 1) ? v : pv, rope_pos, d >> 1, hd, a.rope.theta, y0, y1);
                    out = (r & 1) ? y1 : y0;
                }
                if (valid) {
                    if (mi == 0)
                        static_cast<__half*>(y)[row] = out;
                    else
                        static_cast<__half*>(mi == 1 ? a.rope.kcache : a.rope.vcache)[(static_cast<size_t>(head) * a.rope.max_seq_len + rope_pos) * hd + d] = out;
                }
            }
        }
    }
}

// ---- the same multiplication with the activation producer in front (the decode chain of the single-GPU engine) -------
// A decode step is a chain of dependent launches, and what a launch can do BEFORE its dependency resolves is free.
// With prepared weights that is everything except the activation: a block keeps 16 / 32 / 64 rows (8 / 4 / 2 warps
// per tile) and every warp requests ALL of its quads (at most kGpFusedQuads: the launch is one wave of at most two
// blocks per SM) into registers before the wait, and the norm weights go to shared memory by cp.async.  After the
// wait the block forms the int8 activation vector exactly as the SIMT kernels of gemv.cu do (produce_x: same sums,
// same rounding points), re-orders it for the B registers and multiplies out of registers: nothing of the weight
// path is left on the critical path.  Epilogue as above (half outputs; RoPE and the KV scatter for q, k, v).
constexpr int kGpFusedQuads = 6;
constexpr int kGpFusedBlocksPerSm = 2;  // two blocks of up to 128 registers fill an SM's register file.  (Held to 80 registers
                                        // so that a block of the NEXT launch fits beside them and requests its weights while
                                        // these compute, the same decode step ran at 789 instead of 924 tok/s.)
struct GpFusedArgs {
    GpMat mat[kGpMaxMats];
    int nmat;
    ProducerArgs p;
    int ntiles, nquads;
    int ks, ks_log2, qpw;
    RopeScatter rope;
};

__device__ __forceinline__ void gp_step(int& c0, int& c1, int& c2, int& c3, int& d0, int& d1, int& d2, int& d3, uint32_t e,
                                        uint32_t sel, uint32_t x_addr, bool bcol) {
    const uint32_t a0 = __byte_perm(0xFF00FF00u, 0xFF00FF00u, sel);
    const uint32_t a1 = __byte_perm(0xFFFF0000u, 0xFFFF0000u, sel);
    const uint32_t a2 = __byte_perm(0x00000000u, 0xFFFFFFFFu, sel);
    const uint32_t a3 = __byte_perm(0x00000000u, 0xFFFFFFFFu, sel >> 1);
    uint32_t b0 = 0, b1 = 0, b2 = 0, b3 = 0;
    if (bcol) asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(x_addr));
    asm volatile(
        "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
        : "+r"(c0), "+r"(c1), "+r"(c2), "+r"(c3)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(b2), "r"(b3), "r"(e));
    asm volatile(
        "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
        "{%0, %1, %2, %3}, {%4, %4, %4, %4}, {%5, %6, %7, %8}, {%0, %1, %2, %3}, %9, 0x0;"
        : "+r"(d0), "+r"(d1), "+r"(d2), "+r"(d3)
        : "r"(0x01010101u), "r"(b0), "r"(b1), "r"(b2), "r"(b3), "r"(e));
}

template <int IN>
__global__ void __launch_bounds__(kGpThreads, kGpFusedBlocksPerSm) gemv_prepared_fused_kernel(const GpFusedArgs a) {
    __shared__ int red[kGpWarps * 16];
    __shared__ float redf[64];
    // x in B-register order (cols bytes) | x as the producer writes it, swizzled 16-byte chunks (cols bytes) |
    // norm weights (cols floats) | sub-norm weights (cols floats)
    extern __shared__ __align__(16) uint8_t gpf_raw[];
    const int cols = a.p.cols;
    const uint32_t xs_s = static_cast<uint32_t>(__cvta_generic_to_shared(gpf_raw));
    uint4* xs_sw = reinterpret_cast<uint4*>(gpf_raw + cols);
    float* wbuf = reinterpret_cast<float*>(gpf_raw + 2 * cols);
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
    const int tiles_blk = kGpWarps >> a.ks_log2;
    const int tile = blockIdx.x * tiles_blk + (warp >> a.ks_log2), kq = warp & (a.ks - 1);
    const bool live = tile < a.ntiles;
    const int q_begin = live ? min(a.nquads, kq * a.qpw) : 0, q_end = live ? min(a.nquads, q_begin + a.qpw) : 0;
    const int g = lane >> 2, tig = lane & 3;
    auto mat_of = [&](int t) { return (a.nmat > 2 && t >= a.mat[2].tile0) ? 2 : (a.nmat > 1 && t >= a.mat[1].tile0) ? 1 : 0; };
    const int wm = mat_of(live ? tile : 0);
    const uint8_t* wprep = wm == 2 ? a.mat[2].prep : wm == 1 ? a.mat[1].prep : a.mat[0].prep;
    const int wtile0 = wm == 2 ? a.mat[2].tile0 : wm == 1 ? a.mat[1].tile0 : 0;
    const uint8_t* tp = wprep + (static_cast<size_t>(live ? tile - wtile0 : 0) * a.nquads) * kGpQuadBytes;

    // ---- before the dependency wait: all weights of the warp, the norm weights ----
    uint4 m[kGpFusedQuads];
    uint2 s[kGpFusedQuads];
#pragma unroll
    for (int i = 0; i < kGpFusedQuads; ++i) {
        m[i] = make_uint4(0, 0, 0, 0);
        s[i] = make_uint2(0, 0);
        if (q_begin + i < q_end) gp_load_quad(tp, q_begin + i, lane, m[i], s[i]);
    }
    ProducerArgs pa = a.p;
    if (IN >= IN_RESNORM) {
        auto stage = [&](const float* src, float* dst) {
            for (int q = tid; q < (cols >> 2); q += kGpThreads)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst + 4 * q))), "l"(src + 4 * q) : "memory");
        };
        if (IN == IN_RESNORM) {
            stage(a.p.w_norm, wbuf);
            pa.w_norm = wbuf;
            if (a.p.w_sub) {
                stage(a.p.w_sub, wbuf + cols);
                pa.w_sub = wbuf + cols;
            }
        } else if (a.p.w_sub) {
            stage(a.p.w_sub, wbuf);
            pa.w_sub = wbuf;
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    grid_dep_wait();
    grid_dep_launch();
    int rope_pos = 0;
    if (a.rope.d_pos) asm volatile("ld.global.s32 %0, [%1];" : "=r"(rope_pos) : "l"(a.rope.d_pos));
    if (IN >= IN_RESNORM) asm volatile("cp.async.wait_group 0;" ::: "memory");  // (each weight is first read after a block-wide reduction)
    const float absmax = produce_x<IN, OUT_F16>(pa, xs_sw, static_cast<__half*>(nullptr), redf, blockIdx.x == 0);
    __syncthreads();
    for (int q = tid; q < (cols >> 4); q += kGpThreads) {
        const int c = q >> 3, i = q & 7;
        const uint4 xv = xs_sw[(c << 3) + (i ^ (c & 7))];
        const uint32_t d = xs_s + (static_cast<uint32_t>(q) >> 2) * 64u + (static_cast<uint32_t>(q) & 3u) * 4u;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d), "r"(xv.x) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 16u), "r"(xv.y) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 32u), "r"(xv.z) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 48u), "r"(xv.w) : "memory");
    }
    __syncthreads();

    // ---- the multiplication, out of registers ----
    int r0 = 0, r1 = 0, r2 = 0, r3 = 0, t0 = 0, t1 = 0, t2 = 0, t3 = 0;
    int u0 = 0, u1 = 0, u2 = 0, u3 = 0, v0 = 0, v1 = 0, v2 = 0, v3 = 0;
    const bool bcol = g == 0;
    const uint32_t xq0 = xs_s + static_cast<uint32_t>(tig) * 16u + static_cast<uint32_t>(q_begin) * 256u;
#pragma unroll
    for (int i = 0; i < kGpFusedQuads; ++i) {
        if (q_begin + i < q_end) {  // uniform over the warp
            const uint32_t xq = xq0 + static_cast<uint32_t>(i) * 256u;
            gp_step(r0, r1, r2, r3, u0, u1, u2, u3, m[i].x, s[i].x, xq, bcol);
            gp_step(t0, t1, t2, t3, v0, v1, v2, v3, m[i].y, s[i].x >> 16, xq + 64u, bcol);
            gp_step(r0, r1, r2, r3, u0, u1, u2, u3, m[i].z, s[i].y, xq + 128u, bcol);
            gp_step(t0, t1, t2, t3, v0, v1, v2, v3, m[i].w, s[i].y >> 16, xq + 192u, bcol);
        }
    }
    if (tig == 0) {
        red[warp * 16 + g] = (u0 + v0) + 2 * (r0 + t0);
        red[warp * 16 + g + 8] = (u2 + v2) + 2 * (r2 + t2);
    }
    __syncthreads();
    if (tid < ((16 * tiles_blk + 31) & ~31)) {
        const int tl = tid >> 4, r = tid & 15;
        const int t = blockIdx.x * tiles_blk + tl;
        const bool in_tile = tl < tiles_blk && t < a.ntiles;
        const int mi = mat_of(in_tile ? t : 0);
        const int row = ((in_tile ? t : 0) - (mi == 2 ? a.mat[2].tile0 : mi == 1 ? a.mat[1].tile0 : 0)) * 16 + r;
        const int mrows = mi == 2 ? a.mat[2].rows : mi == 1 ? a.mat[1].rows : a.mat[0].rows;
        const bool valid = in_tile && row < mrows;
        void* y = mi == 2 ? a.mat[2].y : mi == 1 ? a.mat[1].y : a.mat[0].y;
        const float gamma = mi == 2 ? a.mat[2].gamma : mi == 1 ? a.mat[1].gamma : a.mat[0].gamma;
        int acc = 0;
        if (in_tile)
            for (int k = 0; k < a.ks; ++k) acc += red[((tl << a.ks_log2) + k) * 16 + r];
        const __half hv = __float2half_rn(__fmul_rn(static_cast<float>(acc), dequant_scale(gamma, absmax)));
        if (!a.rope.d_pos) {
            if (valid) static_cast<__half*>(y)[row] = hv;
        } else {
            const float v = __half2float(hv);
            const float pv = __shfl_xor_sync(0xFFFFFFFFu, v, 1);
            const int hd = a.rope.head_dim;
            const int head = row / hd, d = row - head * hd;
            __half out = hv;
            if (mi != 2) {
                __half y0, y1;
                rope_rotate((r & 1) ? pv : v, (r & 1) ? v : pv, rope_pos, d >> 1, hd, a.rope.theta, y0, y1);
                out = (r & 1) ? y1 : y0;
            }
            if (valid) {
                if (mi == 0)
                    static_cast<__half*>(y)[row] = out;
                else
                    static_cast<__half*>(mi == 1 ? a.rope.kcache : a.rope.vcache)[(static_cast<size_t>(head) * a.rope.max_seq_len + rope_pos) * hd + d] = out;
            }
        }
    }
}

static bool gp_shape_ok(int rows, int cols) { return rows > 0 && cols > 0 && cols % 256 == 0 && cols <= 65536; }
static size_t gp_weight_bytes(int rows, int cols) { return static_cast<size_t>((rows + 15) / 16) * (cols / 256) * kGpQuadBytes; }

struct GpMatDesc {
    const void* prep;
    void* y;
    float gamma;
    int rows;
};

static int gp_launch(const char* name, const GpMatDesc* mats, int nmat, const int8_t* x, int32_t* y_acc, const float* d_absmax,
                     int out_mode, int cols, const RopeScatter* rope, void* stream, const LlFan* fans = nullptr) {
    if (nmat < 1 || nmat > kGpMaxMats) return fail(SPB_E_INVALID, "%s: %d matrices", name, nmat);
    if (cols < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    GpArgs a{};
    int tiles = 0;
    for (int i = 0; i < nmat; ++i) {
        if (mats[i].rows < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
        if (mats[i].rows == 0 || cols == 0) {
            if (nmat == 1) return SPB_OK;
            return fail(SPB_E_INVALID, "%s: an empty matrix in a group", name);
        }
        if (!mats[i].prep || !mats[i].y) return fail(SPB_E_INVALID, "%s: null pointer", name);
        if (reinterpret_cast<uintptr_t>(mats[i].prep) & 15u) return fail(SPB_E_INVALID, "%s: prepared weights must be 16-byte aligned", name);
        a.mat[i] = GpMat{static_cast<const uint8_t*>(mats[i].prep), mats[i].y, mats[i].gamma, mats[i].rows, tiles};
        tiles += (mats[i].rows + 15) / 16;
    }
    if (!x) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (out_mode != GP_OUT_I32 && !d_absmax) return fail(SPB_E_INVALID, "%s: d_absmax is null", name);
    if (!gp_shape_ok(mats[0].rows, cols)) return fail(SPB_E_UNSUPPORTED, "%s: cols=%d is not a multiple of 256 up to 65536", name, cols);
    if (reinterpret_cast<uintptr_t>(x) & 15u) return fail(SPB_E_INVALID, "%s: x must be 16-byte aligned", name);
    if (rope) {
        if (nmat != 3 || out_mode != GP_OUT_F16 || rope->head_dim < 2 || rope->head_dim % 2 || mats[0].rows % rope->head_dim ||
            mats[1].rows % rope->head_dim || mats[1].rows != mats[2].rows || !rope->d_pos || !rope->kcache || !rope->vcache)
            return fail(SPB_E_INVALID, "%s: rotation wants q, k, v with whole heads and half outputs", name);
        a.rope = *rope;
    }
    if (fans) {
        if (nmat > 2 || rope || out_mode != GP_OUT_F16) return fail(SPB_E_INVALID, "%s: a fan-out wants one or two matrices with half outputs", name);
        for (int i = 0; i < nmat; ++i) {
            if (mats[i].rows % 2 || fans[i].ndst < 1 || fans[i].ndst > kLlMaxDest || !fans[i].seq || fans[i].seq != fans[0].seq)
                return fail(SPB_E_INVALID, "%s: bad fan-out", name);
            a.fan[i] = fans[i];
        }
    }
    a.nmat = nmat;
    a.x = x; a.y_acc = y_acc; a.d_absmax = d_absmax; a.out_mode = out_mode;
    a.cols = cols;
    a.ntiles = tiles;
    a.nquads = cols / 256;
    // Warps per tile (1, 2, 4 or 8; a block is 8 warps).  A launch runs in waves of sm_count x 4 blocks, and a wave
    // lasts as long as a warp's run of quads plus a fixed part (start, activation vector into shared memory, the
    // sum over the tile's warps: about three quads' worth), so the choice minimises waves x (quads per warp + 3):
    // 512 tiles of 112 quads (8192 x 28672) run as one wave of 512 blocks with 14 quads per warp, where a rule that
    // only filled the SMs ran the same blocks in two waves.  Ties go to the longer runs.
    const int slots = sm_count() * kGpBlocksPerSm;
    long long best = 0;
    a.ks = 1;
    for (int ks = 1; ks <= 8; ks <<= 1) {
        const int qpw = (a.nquads + ks - 1) / ks;
        if (ks > 1 && qpw < 2) break;
        const int nblocks = (a.ntiles + kGpWarps / ks - 1) / (kGpWarps / ks);
        const long long cost = static_cast<long long>((nblocks + slots - 1) / slots) * (qpw + 3);
        if (ks == 1 || cost < best) {
            best = cost;
            a.ks = ks;
        }
    }
    a.ks_log2 = a.ks == 8 ? 3 : a.ks == 4 ? 2 : a.ks == 2 ? 1 : 0;
    a.qpw = (a.nquads + a.ks - 1) / a.ks;
    const int tiles_blk = kGpWarps / a.ks;
    const unsigned blocks = static_cast<unsigned>((a.ntiles + tiles_blk - 1) / tiles_blk);
    const size_t smem = static_cast<size_t>(cols);
    if (int rc = ensure_dynamic_smem(name, gemv_prepared_kernel, smem)) return rc;
    return launch(name, gemv_prepared_kernel, dim3(blocks), dim3(kGpThreads), smem, stream, a);
}

static int gp_launch(const char* name, const void* prep, const int8_t* x, void* y, int32_t* y_acc, const float* d_absmax,
                     float gamma, int out_mode, int rows, int cols, void* stream) {
    if (rows < 0 || cols < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    if (rows == 0 || cols == 0) return SPB_OK;
    if (!prep || !x || !y) return fail(SPB_E_INVALID, "%s: null pointer", name);
    const GpMatDesc m{prep, y, gamma, rows};
    return gp_launch(name, &m, 1, x, y_acc, d_absmax, out_mode, cols, nullptr, stream);
}

// Whether a group of BitLinears with prepared copies can run as ONE wave of gemv_prepared_fused_kernel, and how.
static bool gp_fused_plan(const int* rows, int nmat, int cols, GpFusedArgs& a) {
    if (nmat < 1 || nmat > kGpMaxMats || cols <= 0 || cols % 256 || cols > 8192) return false;
    int tiles = 0;
    for (int i = 0; i < nmat; ++i) {
        if (rows[i] <= 0) return false;
        a.mat[i].tile0 = tiles;
        a.mat[i].rows = rows[i];
        tiles += (rows[i] + 15) / 16;
    }
    a.nmat = nmat;
    a.ntiles = tiles;
    a.nquads = cols / 256;
    const int slots = sm_count() * kGpFusedBlocksPerSm;
    for (int ks = 8; ks >= 1; ks >>= 1) {  // as many warps per tile as one wave allows: the shortest run of quads per warp
        const int qpw = (a.nquads + ks - 1) / ks;
        const int nblocks = (tiles + kGpWarps / ks - 1) / (kGpWarps / ks);
        if (nblocks <= slots && qpw <= kGpFusedQuads) {
            a.ks = ks;
            a.ks_log2 = ks == 8 ? 3 : ks == 4 ? 2 : ks == 2 ? 1 : 0;
            a.qpw = qpw;
            return true;
        }
    }
    return false;
}

bool prepared_group_fused_supported(const int* rows, int nmat, int cols) {
    GpFusedArgs a{};
    return gp_fused_plan(rows, nmat, cols, a);
}

// engine-internal: the BitLinears of a group on prepared weights with the activation producer `in` (IN_F16_AMAX,
// IN_RESNORM, IN_RELU2) in front, one launch; p as for the SIMT kernels of gemv.cu; half outputs; with `rope` the
// group is q, k, v.
int prepared_group_fused(int in, const void* const* prep, void* const* out_half, const float* gamma, const int* rows, int nmat,
                         const ProducerArgs& p, const RopeScatter* rope, void* stream) {
    const char* name = "prepared_group_fused";
    GpFusedArgs a{};
    if (!gp_fused_plan(rows, nmat, p.cols, a)) return fail(SPB_E_UNSUPPORTED, "%s: shape outside the one-wave form", name);
    for (int i = 0; i < nmat; ++i) {
        if (!prep[i] || !out_half[i] || (reinterpret_cast<uintptr_t>(prep[i]) & 15u)) return fail(SPB_E_INVALID, "%s: bad pointer", name);
        a.mat[i].prep = static_cast<const uint8_t*>(prep[i]);
        a.mat[i].y = out_half[i];
        a.mat[i].gamma = gamma[i];
    }
    if (!p.x || (reinterpret_cast<uintptr_t>(p.x) & 15u) || (p.x2 && (reinterpret_cast<uintptr_t>(p.x2) & 15u)))
        return fail(SPB_E_INVALID, "%s: activation vectors must be 16-byte aligned", name);
    if ((p.w_norm && (reinterpret_cast<uintptr_t>(p.w_norm) & 15u)) || (p.w_sub && (reinterpret_cast<uintptr_t>(p.w_sub) & 15u)))
        return fail(SPB_E_UNSUPPORTED, "%s: norm weights must be 16-byte aligned", name);
    if (in == IN_RESNORM && (!p.w_norm || !p.x_out)) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (in == IN_RELU2 && !p.x2) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (rope) {
        if (nmat != 3 || rope->head_dim < 2 || rope->head_dim % 2 || rows[0] % rope->head_dim || rows[1] % rope->head_dim ||
            rows[1] != rows[2] || !rope->d_pos || !rope->kcache || !rope->vcache)
            return fail(SPB_E_INVALID, "%s: rotation wants q, k, v with whole heads", name);
        a.rope = *rope;
    }
    a.p = p;
    const int tiles_blk = kGpWarps / a.ks;
    const unsigned blocks = static_cast<unsigned>((a.ntiles + tiles_blk - 1) / tiles_blk);
    const size_t smem = static_cast<size_t>(p.cols) * (2 + (in == IN_RESNORM ? 8 : in == IN_RELU2 ? 4 : 0));
    int rc;
    switch (in) {
        case IN_F16_AMAX:
            if ((rc = ensure_dynamic_smem(name, gemv_prepared_fused_kernel<IN_F16_AMAX>, smem))) return rc;
            return launch(name, gemv_prepared_fused_kernel<IN_F16_AMAX>, dim3(blocks), dim3(kGpThreads), smem, stream, a);
        case IN_RESNORM:
            if ((rc = ensure_dynamic_smem(name, gemv_prepared_fused_kernel<IN_RESNORM>, smem))) return rc;
            return launch(name, gemv_prepared_fused_kernel<IN_RESNORM>, dim3(blocks), dim3(kGpThreads), smem, stream, a);
        case IN_RELU2:
            if ((rc = ensure_dynamic_smem(name, gemv_prepared_fused_kernel<IN_RELU2>, smem))) return rc;
            return launch(name, gemv_prepared_fused_kernel<IN_RELU2>, dim3(blocks), dim3(kGpThreads), smem, stream, a);
        default:
            return fail(SPB_E_INVALID, "%s: producer %d", name, in);
    }
}

// engine-internal: BitLinear on prepared weights, quantised activation, scaled half output
int prepared_bitlinear_q8(const void* prep, const int8_t* xq, void* out_half, const float* d_absmax, float gamma, int rows,
                          int cols, void* stream) {
    return gp_launch("prepared_bitlinear_q8", prep, xq, out_half, nullptr, d_absmax, gamma, GP_OUT_F16, rows, cols, stream);
}

// engine-internal: up to three BitLinears of the same width on one quantised activation in one launch; with `rope`
// they are q, k, v: q and k rows are rotated for the position in *rope->d_pos, k and v rows go to the cache rows of
// that position (out[1], out[2] are not written)
int prepared_bitlinear_q8_group(const void* const* prep, void* const* out_half, const float* gamma, const int* rows, int n,
                                const int8_t* xq, const float* d_absmax, int cols, const RopeScatter* rope, void* stream,
                                const LlFan* fans) {
    GpMatDesc m[kGpMaxMats];
    if (n < 1 || n > kGpMaxMats) return fail(SPB_E_INVALID, "prepared_bitlinear_q8_group: %d matrices", n);
    for (int i = 0; i < n; ++i) m[i] = GpMatDesc{prep[i], out_half[i], gamma[i], rows[i]};
    return gp_launch("prepared_bitlinear_q8_group", m, n, xq, nullptr, d_absmax, GP_OUT_F16, cols, rope, stream, fans);
}

}  // namespace spb

using namespace spb;

extern "C" size_t spb_prepared_weights_bytes(int rows, int cols) {
    if (!gp_shape_ok(rows, cols)) return 0;
    return gp_weight_bytes(rows, cols);
}

extern "C" int spb_prepare_weights(const uint32_t* d_meta, const uint32_t* d_values, int rows, int cols, int meta_row_stride,
                                   int values_row_stride, void* d_prepared, void* stream) {
    const char* name = "spb_prepare_weights";
    if (rows < 0 || cols < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    if (rows == 0 || cols == 0) return SPB_OK;
    if (!d_meta || !d_values || !d_prepared) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (!gp_shape_ok(rows, cols)) return fail(SPB_E_UNSUPPORTED, "%s: cols=%d is not a multiple of 256 up to 65536", name, cols);
    if (meta_row_stride < cols / 32 || values_row_stride < cols / 64) return fail(SPB_E_INVALID, "%s: row stride shorter than a row", name);
    if (reinterpret_cast<uintptr_t>(d_prepared) & 15u) return fail(SPB_E_INVALID, "%s: the prepared buffer must be 16-byte aligned", name);
    const int ntiles = (rows + 15) / 16, nquads = cols / 256;
    const long long threads = static_cast<long long>(ntiles) * nquads * 32;
    const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
    return launch(name, gemv_prepare_kernel, dim3(blocks), dim3(256), 0, stream, d_meta, d_values, rows, cols, meta_row_stride,
                  values_row_stride, ntiles, nquads, static_cast<uint8_t*>(d_prepared));
}

extern "C" int spb_prepared_gemv(const void* d_prepared, const int8_t* d_x, int32_t* d_y, int rows, int cols, void* stream) {
    return gp_launch("spb_prepared_gemv", d_prepared, d_x, d_y, nullptr, nullptr, 0.0f, GP_OUT_I32, rows, cols, stream);
}

extern "C" int spb_prepared_bitlinear_q8(const void* d_prepared, const int8_t* d_xq, void* d_out_half, const float* d_absmax,
                                         float gamma, int rows, int cols, void* stream) {
    return prepared_bitlinear_q8(d_prepared, d_xq, d_out_half, d_absmax, gamma, rows, cols, stream);
}
