// Sparse-ternary GEMV on the warp-level sparse MMA (mma.sp m16n8k64, int8), sm_100a.
//
//   y[r] = sum_c W[r, c] * x[c]          W: rows x cols compressed 2:4 ternary, x: int8
//
// Decoding this format on the SIMT pipes costs several hundred issued instructions per unit of
// 128 weights.  The sparse MMA takes the format almost as it is stored: per group of four columns
// it wants the two kept values (+1 / -1 as int8) and their two column indices as 2-bit numbers.
// So the SIMT side only re-encodes, about a quarter of the instructions of a full decode:
//   * a bitmap word (8 groups) becomes a word of index pairs with five logical operations,
//   * a sign nibble (2 groups) becomes four bytes of +1 / -1 through a 16-entry per-lane table,
// and the gather and the multiply-add are the tensor core's.  No tensor memory is involved (its
// allocation alone costs about a microsecond per block, which rules tcgen05 out for a kernel that
// lives three microseconds), and the re-encoded operands never leave registers.
//
// Work split: a block of eight warps owns RB row blocks of 16 rows and the whole K extent, KS warps
// per row block, each with a contiguous range of 64-column steps (RB * KS = 8).  The block's raw
// weight slab (16 * RB rows, 3/16 byte per weight) arrives by 16-byte asynchronous copies (cp.async,
// a warp per row) into padded shared-memory rows (conflict-free word reads), so every byte of the
// block is in flight from its first instructions and nothing is held in registers meanwhile (a
// cp.async.bulk per row was measured to take about a microsecond longer to issue).  Weights never
// depend on a predecessor kernel: the copies are issued before the dependency wait, x is staged
// after it.  Operand registers of a lane (g = lane / 4, tig = lane % 4), as the instruction defines
// them: A = four sign nibbles -> compressed columns 4 tig.. and 16 + 4 tig.. of rows g and g + 8;
// metadata = the index pairs of one whole bitmap word (word tig / 2 of the step, row g + 8 (tig & 1));
// B = x[64 s + 16 j + 4 tig ..] in register j, the same in all N = 8 columns (only column 0 is
// read).  Partial sums of the KS warps meet in shared memory.  There is no spin-wait in the kernel.
// Tried and dropped (slower): a form in which a warp keeps the x slices of four steps in registers and
// walks over the row blocks (fewer shared-memory reads, but thin warps); a two-deep software pipeline
// of the step loop; cp.async.bulk for the slab.  What pays is long step ranges per warp.
#include "spb_common.cuh"

namespace spb {

constexpr int kGmThreads = 256;
constexpr int kGmWarps = kGmThreads / 32;
// Blocks per SM the register allocation is held to: 48 registers; shared memory (38 KB per block of 64 rows at
// 2560 columns) allows the same five.
#ifndef SPB_GEMV_MMA_MIN_BLOCKS
#define SPB_GEMV_MMA_MIN_BLOCKS 5
#endif

enum { GM_OUT_I32 = 0, GM_OUT_F32 = 1, GM_OUT_F16 = 2 };

struct GmArgs {
    const uint32_t* meta;
    const uint32_t* values;
    const int8_t* x;
    void* y;
    int32_t* y_acc;
    const float* d_absmax;
    float gamma;
    int out_mode;
    int rows, cols;
    int meta_stride, values_stride;
    int steps;      // cols / 64
    int ks;         // warps per row block (power of two <= 8)
    int ks_log2;
    int rb;         // row blocks per thread block = 8 / ks
    int spw;        // steps per warp
    int mpitch;     // shared-memory row pitch of the bitmap words, in words (an odd multiple of 4)
    int vpitch;     // same for the sign words
};

// Eight bitmaps (two of four bits set each) -> eight index pairs {low index | high index << 2}.
//   low  = first set bit:  bit0 = ~b0 & b1,  bit1 = ~b0 & ~b1
//   high = last set bit:   bit0 = b3 | ~b2,  bit1 = b3 | b2
__device__ __forceinline__ uint32_t gm_index_pairs(uint32_t m) {
    const uint32_t mr = m >> 1, ml = m << 1;
    const uint32_t t1 = (0x11111111u & (~m & mr)) | (~0x11111111u & (mr | ~m));
    const uint32_t t2 = (0x22222222u & (~ml & ~m)) | (~0x22222222u & (m | ml));
    return (t1 & 0x55555555u) | (t2 & 0xAAAAAAAAu);
}

__device__ __forceinline__ uint32_t gm_lds(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// table read: `off` = (nibble << 7) | (lane << 2); the table's own address is added by the load instruction
__device__ __forceinline__ uint32_t gm_tab(uint32_t tab_s, uint32_t off) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(tab_s + off));
    return v;
}

__global__ void __launch_bounds__(kGmThreads, SPB_GEMV_MMA_MIN_BLOCKS) gemv_mmasp_kernel(const GmArgs a) {
    // static: the sign table (entry (nibble n, lane l) at word n * 32 + l), the partial sums of the eight warps
    __shared__ __align__(16) uint32_t sgn_tab[16 * 32];
    __shared__ int red[kGmWarps * 16];
    // dynamic: [x, permuted: cols bytes][bitmap rows: 16 rb x mpitch words][sign rows: 16 rb x vpitch words]
    extern __shared__ __align__(16) uint8_t gm_raw[];
    const uint32_t tab_s = static_cast<uint32_t>(__cvta_generic_to_shared(sgn_tab));
    const uint32_t xs_s = static_cast<uint32_t>(__cvta_generic_to_shared(gm_raw));
    const uint32_t ms_s = xs_s + static_cast<uint32_t>(a.cols);
    const int nrows_blk = 16 * a.rb;
    const uint32_t vs_s = ms_s + static_cast<uint32_t>(nrows_blk * a.mpitch) * 4u;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = blockIdx.x * nrows_blk;
    const int valid = min(nrows_blk, a.rows - row0);  // rows of this block inside the matrix
    const uint32_t mbytes = static_cast<uint32_t>(a.cols >> 3), vbytes = static_cast<uint32_t>(a.cols >> 4);
    // The raw slab: 16-byte asynchronous copies, a warp per row (bitmap chunks first, then sign chunks), so
    // that a row's bytes are fetched by consecutive lanes.
    {
        const int mch = static_cast<int>(mbytes >> 4), cpr = mch + static_cast<int>(vbytes >> 4);  // 16-byte chunks of a row
        for (int k = lane; k < cpr; k += 32) {  // one pass for up to 32 chunks per row (cols <= 2560), else several
            const bool is_m = k < mch;
            const uint8_t* src = is_m ? reinterpret_cast<const uint8_t*>(a.meta) + k * 16
                                      : reinterpret_cast<const uint8_t*>(a.values) + (k - mch) * 16;
            const size_t src_pitch = static_cast<size_t>(is_m ? a.meta_stride : a.values_stride) * 4u;
            const uint32_t dst = is_m ? ms_s + static_cast<uint32_t>(k) * 16u : vs_s + static_cast<uint32_t>(k - mch) * 16u;
            const uint32_t dst_pitch = static_cast<uint32_t>(is_m ? a.mpitch : a.vpitch) * 4u;
            src += static_cast<size_t>(row0 + warp) * src_pitch;
            for (int r = warp; r < valid; r += kGmWarps) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + static_cast<uint32_t>(r) * dst_pitch), "l"(src)
                             : "memory");
                src += kGmWarps * src_pitch;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // sign table under the copy latency: entry (nibble n, lane l) at n * 128 + l * 4, byte b = -1 if bit b of n
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const uint32_t i = tid + j * kGmThreads;
        const uint32_t t = ((i >> 5) * 0x00204081u) & 0x01010101u;
        sgn_tab[i] = (t * 0xFEu) | 0x01010101u;
    }

    const int g = lane >> 2, tig = lane & 3;
    // the warp index through a shuffle, so that everything derived from it (the step range, the loop) is
    // known to be uniform over the warp
    const int warp_u = __shfl_sync(0xFFFFFFFFu, warp, 0);
    const int rbi = warp_u >> a.ks_log2, kq = warp_u & (a.ks - 1);
    const int s_begin = kq * a.spw, s_end = min(a.steps, s_begin + a.spw);
    const uint32_t lane_or = static_cast<uint32_t>(lane) << 2;  // byte offset of the lane's column of the table
    // rotations that bring sign nibble tig (compressed columns 4 tig..) and nibble 4 + tig (16 + 4 tig..) of a
    // sign word to bits 7..10, where they index the table
    const uint32_t rot_lo = (static_cast<uint32_t>(tig) * 4u + 25u) & 31u, rot_hi = (static_cast<uint32_t>(tig) * 4u + 9u) & 31u;
    // running addresses: the lane's bitmap word, the sign words of rows g and g + 8 of the row block, the x slice
    uint32_t me_p = ms_s + static_cast<uint32_t>((rbi * 16 + g + 8 * (tig & 1)) * a.mpitch + (tig >> 1) + 2 * s_begin) * 4u;
    uint32_t v0_p = vs_s + static_cast<uint32_t>((rbi * 16 + g) * a.vpitch + s_begin) * 4u;
    const uint32_t v_half = static_cast<uint32_t>(8 * a.vpitch) * 4u;
    uint32_t xq_p = xs_s + static_cast<uint32_t>(tig) * 16u + static_cast<uint32_t>(s_begin) * 64u;

    // ---- after the dependency: x, permuted so that a lane's four B registers of a step are 16 contiguous bytes:
    //      xs[step][tig][j][0..3] = x[64 step + 16 j + 4 tig + 0..3] -------------------------------------------
    grid_dep_wait();
    // the activation scale of the scaled outputs is asked for now, not in the epilogue where the load would be a trip
    // to L2 on the critical path (volatile: it stays here)
    float absmax_early = 0.0f;
    if (a.out_mode != GM_OUT_I32) asm volatile("ld.global.f32 %0, [%1];" : "=f"(absmax_early) : "l"(a.d_absmax));
    // The successor on the stream is let in only now: it then loads and waits while this grid computes, and
    // no deeper queue of waiting grids builds up (measured: a deep queue slows a long chain of launches).
    grid_dep_launch();
    for (int q = tid; q < (a.cols >> 4); q += kGmThreads) {
        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(a.x) + q);
        const uint32_t s = static_cast<uint32_t>(q) >> 2, j = static_cast<uint32_t>(q) & 3u;
        const uint32_t d = xs_s + s * 64u + j * 4u;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d), "r"(xv.x) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 16u), "r"(xv.y) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 32u), "r"(xv.z) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 48u), "r"(xv.w) : "memory");
    }
    // the weights have landed, the table and x are visible
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    // One step = 64 columns of 16 rows.  Metadata register of lane (g, tig): the index pairs of bitmap word
    // 2 s + (tig >> 1) of row g + 8 (tig & 1).  `off` is a compile-time byte offset from the running addresses.
    int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
    auto step = [&](uint32_t w0, uint32_t w1, uint32_t me_off, uint32_t x_off) {
        const uint32_t e = gm_index_pairs(gm_lds(me_p + me_off));
        const uint32_t a0 = gm_tab(tab_s, (__funnelshift_r(w0, w0, rot_lo) & 0x780u) | lane_or);
        const uint32_t a1 = gm_tab(tab_s, (__funnelshift_r(w1, w1, rot_lo) & 0x780u) | lane_or);
        const uint32_t a2 = gm_tab(tab_s, (__funnelshift_r(w0, w0, rot_hi) & 0x780u) | lane_or);
        const uint32_t a3 = gm_tab(tab_s, (__funnelshift_r(w1, w1, rot_hi) & 0x780u) | lane_or);
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
    for (; st < s_end && (st & 3) != 0; ++st) {  // up to the next multiple of four steps
        step(gm_lds(v0_p), gm_lds(v0_p + v_half), 0u, 0u);
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
        step(gm_lds(v0_p), gm_lds(v0_p + v_half), 0u, 0u);
        advance(1u);
    }
    // column 0 of the tile: lanes with tig == 0 hold rows g (c0) and g + 8 (c2)
    if (tig == 0) {
        red[warp_u * 16 + g] = c0;
        red[warp_u * 16 + g + 8] = c2;
    }
    __syncthreads();
    if (tid < nrows_blk && tid < valid) {
        const int rblk = tid >> 4, r = tid & 15;
        int acc = 0;
        for (int k = 0; k < a.ks; ++k) acc += red[((rblk << a.ks_log2) + k) * 16 + r];
        const int row = row0 + tid;
        if (a.out_mode == GM_OUT_I32) {
            static_cast<int32_t*>(a.y)[row] = acc;
        } else {
            const float f = __fmul_rn(static_cast<float>(acc), dequant_scale(a.gamma, absmax_early));
            if (a.out_mode == GM_OUT_F32) {
                static_cast<float*>(a.y)[row] = f;
                if (a.y_acc) a.y_acc[row] = acc;
            } else {
                static_cast<__half*>(a.y)[row] = __float2half_rn(f);
            }
        }
    }
}

// The same kernel for rows too long to hold whole in shared memory (cols > 16384, e.g. a 28672-column down
// projection): the K extent is cut into chunks of `csteps` steps whose raw slabs alternate between two buffers,
// chunk c + 1 being copied while chunk c is multiplied; the accumulators live across chunks, x is staged whole.
// Inside a chunk the work split is the one above (KS warps per row block, contiguous step ranges).
struct GmChunkArgs {
    GmArgs g;
    int csteps;      // steps per chunk (a multiple of 4 * ks)
    int nchunks;
    int slab_bytes;  // one buffer: 16 rb x (mpitch + vpitch) words
};

__global__ void __launch_bounds__(kGmThreads, 2) gemv_mmasp_chunked_kernel(const GmChunkArgs ca) {
    const GmArgs& a = ca.g;
    __shared__ __align__(16) uint32_t sgn_tab[16 * 32];
    __shared__ int red[kGmWarps * 16];
    extern __shared__ __align__(16) uint8_t gm_raw[];  // [x, permuted: cols bytes][slab 0][slab 1]
    const uint32_t tab_s = static_cast<uint32_t>(__cvta_generic_to_shared(sgn_tab));
    const uint32_t xs_s = static_cast<uint32_t>(__cvta_generic_to_shared(gm_raw));
    const uint32_t slab0_s = xs_s + static_cast<uint32_t>(a.cols);
    const int nrows_blk = 16 * a.rb;
    const uint32_t v_in_slab = static_cast<uint32_t>(nrows_blk * a.mpitch) * 4u;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = blockIdx.x * nrows_blk;
    const int valid = min(nrows_blk, a.rows - row0);
    const int mch = ca.csteps >> 1, vch = ca.csteps >> 2;  // 16-byte pieces of a row's chunk: 8 / 4 bytes per step

    auto issue_chunk = [&](int c) {
        const int steps_here = min(ca.csteps, a.steps - c * ca.csteps);
        const int m_here = (steps_here + 1) >> 1, v_here = (steps_here + 3) >> 2, cpr = m_here + v_here;
        const uint32_t ms_s = slab0_s + static_cast<uint32_t>(c & 1) * ca.slab_bytes, vs_s = ms_s + v_in_slab;
        const size_t m_col = static_cast<size_t>(c) * mch * 16, v_col = static_cast<size_t>(c) * vch * 16;
        for (int k = lane; k < cpr; k += 32) {
            const bool is_m = k < m_here;
            const uint8_t* src = is_m ? reinterpret_cast<const uint8_t*>(a.meta) + m_col + k * 16
                                      : reinterpret_cast<const uint8_t*>(a.values) + v_col + (k - m_here) * 16;
            const size_t src_pitch = static_cast<size_t>(is_m ? a.meta_stride : a.values_stride) * 4u;
            const uint32_t dst = is_m ? ms_s + static_cast<uint32_t>(k) * 16u : vs_s + static_cast<uint32_t>(k - m_here) * 16u;
            const uint32_t dst_pitch = static_cast<uint32_t>(is_m ? a.mpitch : a.vpitch) * 4u;
            src += static_cast<size_t>(row0 + warp) * src_pitch;
            for (int r = warp; r < valid; r += kGmWarps) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + static_cast<uint32_t>(r) * dst_pitch), "l"(src)
                             : "memory");
                src += kGmWarps * src_pitch;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue_chunk(0);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const uint32_t i = tid + j * kGmThreads;
        const uint32_t t = ((i >> 5) * 0x00204081u) & 0x01010101u;
        sgn_tab[i] = (t * 0xFEu) | 0x01010101u;
    }
    const int g = lane >> 2, tig = lane & 3;
    const int warp_u = __shfl_sync(0xFFFFFFFFu, warp, 0);
    const int rbi = warp_u >> a.ks_log2, kq = warp_u & (a.ks - 1);
    const uint32_t lane_or = static_cast<uint32_t>(lane) << 2;
    const uint32_t rot_lo = (static_cast<uint32_t>(tig) * 4u + 25u) & 31u, rot_hi = (static_cast<uint32_t>(tig) * 4u + 9u) & 31u;
    const uint32_t v_half = static_cast<uint32_t>(8 * a.vpitch) * 4u;

    grid_dep_wait();
    // the activation scale of the scaled outputs is asked for now, not in the epilogue where the load would be a trip
    // to L2 on the critical path (volatile: it stays here)
    float absmax_early = 0.0f;
    if (a.out_mode != GM_OUT_I32) asm volatile("ld.global.f32 %0, [%1];" : "=f"(absmax_early) : "l"(a.d_absmax));
    grid_dep_launch();
    for (int q = tid; q < (a.cols >> 4); q += kGmThreads) {
        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(a.x) + q);
        const uint32_t st = static_cast<uint32_t>(q) >> 2, j = static_cast<uint32_t>(q) & 3u;
        const uint32_t d = xs_s + st * 64u + j * 4u;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d), "r"(xv.x) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 16u), "r"(xv.y) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 32u), "r"(xv.z) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 48u), "r"(xv.w) : "memory");
    }
    int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
    for (int c = 0; c < ca.nchunks; ++c) {
        if (c + 1 < ca.nchunks) {
            issue_chunk(c + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // chunk c has landed for every thread (and, at c == 0, the table and x are visible)
        const int steps_here = min(ca.csteps, a.steps - c * ca.csteps);
        const int s_begin = kq * a.spw, s_end = min(steps_here, s_begin + a.spw);  // within the chunk; spw % 4 == 0
        const uint32_t ms_s = slab0_s + static_cast<uint32_t>(c & 1) * ca.slab_bytes, vs_s = ms_s + v_in_slab;
        uint32_t me_p = ms_s + static_cast<uint32_t>((rbi * 16 + g + 8 * (tig & 1)) * a.mpitch + (tig >> 1) + 2 * s_begin) * 4u;
        uint32_t v0_p = vs_s + static_cast<uint32_t>((rbi * 16 + g) * a.vpitch + s_begin) * 4u;
        uint32_t xq_p = xs_s + static_cast<uint32_t>(tig) * 16u + static_cast<uint32_t>(c * ca.csteps + s_begin) * 64u;
        auto step = [&](uint32_t w0, uint32_t w1, uint32_t me_off, uint32_t x_off) {
            const uint32_t e = gm_index_pairs(gm_lds(me_p + me_off));
            const uint32_t a0 = gm_tab(tab_s, (__funnelshift_r(w0, w0, rot_lo) & 0x780u) | lane_or);
            const uint32_t a1 = gm_tab(tab_s, (__funnelshift_r(w1, w1, rot_lo) & 0x780u) | lane_or);
            const uint32_t a2 = gm_tab(tab_s, (__funnelshift_r(w0, w0, rot_hi) & 0x780u) | lane_or);
            const uint32_t a3 = gm_tab(tab_s, (__funnelshift_r(w1, w1, rot_hi) & 0x780u) | lane_or);
            uint32_t b0, b1, b2, b3;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(xq_p + x_off));
            asm volatile(
                "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
                "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
                : "+r"(c0), "+r"(c1), "+r"(c2), "+r"(c3)
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(b2), "r"(b3), "r"(e));
        };
        int st = s_begin;
        for (; st + 4 <= s_end; st += 4) {
            uint4 w0, w1;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w0.x), "=r"(w0.y), "=r"(w0.z), "=r"(w0.w) : "r"(v0_p));
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w1.x), "=r"(w1.y), "=r"(w1.z), "=r"(w1.w) : "r"(v0_p + v_half));
            step(w0.x, w1.x, 0u, 0u);
            step(w0.y, w1.y, 8u, 64u);
            step(w0.z, w1.z, 16u, 128u);
            step(w0.w, w1.w, 24u, 192u);
            me_p += 32u; v0_p += 16u; xq_p += 256u;
        }
        for (; st < s_end; ++st) {  // a last chunk whose step count is not a multiple of four
            step(gm_lds(v0_p), gm_lds(v0_p + v_half), 0u, 0u);
            me_p += 8u; v0_p += 4u; xq_p += 64u;
        }
        __syncthreads();  // everybody is done with this buffer before chunk c + 2 is copied into it
    }
    if (tig == 0) {
        red[warp_u * 16 + g] = c0;
        red[warp_u * 16 + g + 8] = c2;
    }
    __syncthreads();
    if (tid < nrows_blk && tid < valid) {
        const int rblk = tid >> 4, r = tid & 15;
        int acc = 0;
        for (int k = 0; k < a.ks; ++k) acc += red[((rblk << a.ks_log2) + k) * 16 + r];
        const int row = row0 + tid;
        if (a.out_mode == GM_OUT_I32) {
            static_cast<int32_t*>(a.y)[row] = acc;
        } else {
            const float f = __fmul_rn(static_cast<float>(acc), dequant_scale(a.gamma, absmax_early));
            if (a.out_mode == GM_OUT_F32) {
                static_cast<float*>(a.y)[row] = f;
                if (a.y_acc) a.y_acc[row] = acc;
            } else {
                static_cast<__half*>(a.y)[row] = __float2half_rn(f);
            }
        }
    }
}

// Whether the layout can take this kernel: whole 16-byte sign rows (cols % 256 == 0), 16-byte aligned
// rows in both arrays and x, and a slab that fits in shared memory.
bool gemv_mmasp_supported(const uint32_t* meta, const uint32_t* values, const int8_t* x, int rows, int cols,
                          int meta_stride, int values_stride) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return rows > 0 && cols > 0 && cols % 256 == 0 && cols <= 65536 && meta_stride % 4 == 0 && values_stride % 4 == 0 &&
           al16(meta) && al16(values) && al16(x);
}

int gemv_mmasp_launch(const char* name, const uint32_t* meta, const uint32_t* values, const int8_t* x, void* y,
                      int32_t* y_acc, const float* d_absmax, float gamma, int out_mode, int rows, int cols,
                      int meta_stride, int values_stride, void* stream) {
    // smallest pitch >= words that is an odd multiple of four words: eight consecutive rows then start on eight
    // different groups of four banks, and rows stay 16-byte aligned
    auto pitch = [](int words) { return words % 8 == 4 ? words : words + ((4 - words % 8) + 8) % 8; };
    GmArgs a{};
    a.meta = meta; a.values = values; a.x = x; a.y = y; a.y_acc = y_acc; a.d_absmax = d_absmax; a.gamma = gamma;
    a.out_mode = out_mode; a.rows = rows; a.cols = cols; a.meta_stride = meta_stride; a.values_stride = values_stride;
    a.steps = cols / 64;
    if (cols > 16384) {  // rows too long for one slab: chunks of 64 steps (4096 columns), four warps per row block
        GmChunkArgs ca{};
        a.ks = 4; a.ks_log2 = 2; a.rb = 2;
        ca.csteps = 64;
        a.spw = ca.csteps / a.ks;
        a.mpitch = pitch(ca.csteps * 2);
        a.vpitch = pitch(ca.csteps);
        ca.nchunks = (a.steps + ca.csteps - 1) / ca.csteps;
        ca.slab_bytes = 16 * a.rb * (a.mpitch + a.vpitch) * 4;
        ca.g = a;
        const size_t smem = static_cast<size_t>(cols) + 2 * static_cast<size_t>(ca.slab_bytes);
        if (int rc = ensure_dynamic_smem(name, gemv_mmasp_chunked_kernel, smem)) return rc;
        const unsigned blocks = static_cast<unsigned>((rows + 16 * a.rb - 1) / (16 * a.rb));
        return launch(name, gemv_mmasp_chunked_kernel, dim3(blocks), dim3(kGmThreads), smem, stream, ca);
    }
    // Warps per row block: long step ranges per warp amortise a warp's fixed cost (measured: about 20 steps
    // per warp is best at 6912 x 2560), but a small matrix still has to give every SM a few warps.
    const int row_blocks = (rows + 15) / 16;
    a.ks = 8;
    while (a.ks > 1 && a.steps / a.ks < 16) a.ks >>= 1;
    while (a.ks < 8 && row_blocks * a.ks < 2 * sm_count() && a.steps / (2 * a.ks) >= 8) a.ks <<= 1;
    while (a.ks > a.steps) a.ks >>= 1;
    a.rb = kGmWarps / a.ks;
    a.ks_log2 = a.ks == 8 ? 3 : a.ks == 4 ? 2 : a.ks == 2 ? 1 : 0;
    a.spw = (a.steps + a.ks - 1) / a.ks;
    a.mpitch = pitch(cols / 32);
    a.vpitch = pitch(cols / 64);
    const size_t smem = static_cast<size_t>(cols) +
                        static_cast<size_t>(16 * a.rb) * (a.mpitch + a.vpitch) * 4;
    if (int rc = ensure_dynamic_smem(name, gemv_mmasp_kernel, smem)) return rc;
    const unsigned blocks = static_cast<unsigned>((rows + 16 * a.rb - 1) / (16 * a.rb));
    return launch(name, gemv_mmasp_kernel, dim3(blocks), dim3(kGmThreads), smem, stream, a);
}


}  // namespace spb
