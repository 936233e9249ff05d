// Small-batch sparse-ternary product on the warp-level sparse MMA (mma.sp m16n8k64, int8), sm_100a.
//
//   Y[j, r] = sum_c W[r, c] * X[j, c]      W: rows x cols compressed 2:4 ternary, X: n x cols int8, n <= 32
//
// The same scheme as the GEMV on this instruction (gemv_mmasp.cu): the raw weight slab of a block comes
// in by 16-byte asynchronous copies, bitmap words are turned into index pairs and sign nibbles into
// +1 / -1 bytes in registers, and the N = 8 columns of the instruction, which the GEMV fills with copies
// of one vector, carry eight different activation rows here.  A warp re-encodes a step (64 columns of 16
// rows) once and issues one MMA per tile of eight activation rows, so 8, 16, 24 or 32 rows cost little
// more than one.  The reference has no kernel of its own for this (its batched path hands a dense copy
// to cuSPARSELt, src/cusparselt_backend.cu:186-207).
//
// Work split: a block of eight warps owns RB row blocks of 16 weight rows x KS warps, each warp a range of
// steps (RB * KS = 8); blockIdx.y selects the tiles of activation rows (NT tiles of 8 per block, as many
// as fit in shared memory next to the slab).  Activations are staged after the dependency wait, permuted
// so that a lane's four B registers of a step are 16 contiguous bytes; row pitch = cols + 64 bytes, which
// keeps the 16-byte reads of a quarter warp (two activation rows x four lanes) on distinct banks.
#include "spb_common.cuh"

namespace spb {

constexpr int kGqThreads = 256;
constexpr int kGqWarps = kGqThreads / 32;
constexpr int kGqSignLutBytes = 16 * 32 * 4;  // 2 KB on a 2 KB boundary
constexpr int kGqMaxTiles = 4;

struct GqArgs {
    const uint32_t* meta;
    const uint32_t* values;
    const int8_t* X;  // [n, cols]
    int32_t* Y;       // [n, rows]
    int rows, cols, n;
    int meta_stride, values_stride;
    int steps;    // cols / 64
    int ks;       // warps per row block (power of two <= 8)
    int ks_log2;
    int rb;       // row blocks per thread block = 8 / ks
    int spw;      // steps per warp
    int mpitch;   // shared-memory row pitch of the bitmap words, in words (= 4 mod 32)
    int vpitch;   // same for the sign words
    int xpitch;   // shared-memory pitch of an activation row, bytes (cols + 64)
    GemmEpilogue ep;  // ep.out set: scaled half output instead of Y
};

__device__ __forceinline__ uint32_t gq_index_pairs(uint32_t m) {
    // eight bitmaps (two of four bits set each) -> eight index pairs {low index | high index << 2}
    const uint32_t mr = m >> 1, ml = m << 1;
    const uint32_t t1 = (0x11111111u & (~m & mr)) | (~0x11111111u & (mr | ~m));
    const uint32_t t2 = (0x22222222u & (~ml & ~m)) | (~0x22222222u & (m | ml));
    return (t1 & 0x55555555u) | (t2 & 0xAAAAAAAAu);
}

__device__ __forceinline__ uint32_t gq_lds(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// NT = tiles of eight activation rows per block.
// HALF_OUT: the epilogue writes the scaled half output (a.ep) instead of the int32 sums
template <int NT, bool HALF_OUT>
__global__ void __launch_bounds__(kGqThreads, 2) gemm_mmasp_kernel(const GqArgs a) {
    extern __shared__ uint8_t gq_raw[];
    // 2 KB-aligned: [sign table 2 KB][bitmap rows: 16 rb x mpitch words][sign rows: 16 rb x vpitch words]
    //               [activations, permuted: 8 NT rows x xpitch bytes; reused for the partial sums at the end]
    const uint32_t raw_s = static_cast<uint32_t>(__cvta_generic_to_shared(gq_raw));
    const uint32_t base_s = (raw_s + 2047u) & ~2047u;
    uint8_t* base = gq_raw + (base_s - raw_s);
    const int nrows_blk = 16 * a.rb;
    const uint32_t ms_s = base_s + kGqSignLutBytes;
    const uint32_t vs_s = ms_s + static_cast<uint32_t>(nrows_blk * a.mpitch) * 4u;
    const uint32_t xs_s = vs_s + static_cast<uint32_t>(nrows_blk * a.vpitch) * 4u;
    volatile int* red = reinterpret_cast<volatile int*>(base + (xs_s - base_s));  // [warp][16 rows][8 NT] after the loop

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);  // through a shuffle: known to be uniform over the warp
    const int row0 = blockIdx.x * nrows_blk;
    const int valid = min(nrows_blk, a.rows - row0);
    const int j0 = blockIdx.y * 8 * NT;                       // first activation row of this block
    const uint32_t mbytes = static_cast<uint32_t>(a.cols >> 3), vbytes = static_cast<uint32_t>(a.cols >> 4);

    // the raw slab: 16-byte asynchronous copies, a warp per row, consecutive lanes on consecutive chunks
    {
        const int mch = static_cast<int>(mbytes >> 4), cpr = mch + static_cast<int>(vbytes >> 4);
        for (int k = lane; k < cpr; k += 32) {
            const bool is_m = k < mch;
            const uint8_t* src = is_m ? reinterpret_cast<const uint8_t*>(a.meta) + k * 16
                                      : reinterpret_cast<const uint8_t*>(a.values) + (k - mch) * 16;
            const size_t src_pitch = static_cast<size_t>(is_m ? a.meta_stride : a.values_stride) * 4u;
            const uint32_t dst = is_m ? ms_s + static_cast<uint32_t>(k) * 16u : vs_s + static_cast<uint32_t>(k - mch) * 16u;
            const uint32_t dst_pitch = static_cast<uint32_t>(is_m ? a.mpitch : a.vpitch) * 4u;
            src += static_cast<size_t>(row0 + warp) * src_pitch;
            for (int r = warp; r < valid; r += kGqWarps) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + static_cast<uint32_t>(r) * dst_pitch), "l"(src)
                             : "memory");
                src += kGqWarps * src_pitch;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // sign table: entry (nibble n, lane l) at n * 128 + l * 4, byte b = -1 if bit b of n is set, else +1
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const uint32_t i = tid + j * kGqThreads;
        const uint32_t t = ((i >> 5) * 0x00204081u) & 0x01010101u;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(base_s + i * 4u), "r"((t * 0xFEu) | 0x01010101u) : "memory");
    }

    const int g = lane >> 2, tig = lane & 3;
    const int rbi = warp >> a.ks_log2, kq = warp & (a.ks - 1);
    const int s_begin = kq * a.spw, s_end = min(a.steps, s_begin + a.spw);
    const uint32_t lane_or = base_s | (static_cast<uint32_t>(lane) << 2);
    const uint32_t rot_lo = (static_cast<uint32_t>(tig) * 4u + 25u) & 31u, rot_hi = (static_cast<uint32_t>(tig) * 4u + 9u) & 31u;
    uint32_t me_p = ms_s + static_cast<uint32_t>((rbi * 16 + g + 8 * (tig & 1)) * a.mpitch + (tig >> 1) + 2 * s_begin) * 4u;
    uint32_t v0_p = vs_s + static_cast<uint32_t>((rbi * 16 + g) * a.vpitch + s_begin) * 4u;
    const uint32_t v_half = static_cast<uint32_t>(8 * a.vpitch) * 4u;
    // B registers of a step for tile t: 16 bytes at activation row 8 t + g, step s, lane slot tig
    uint32_t xq_p = xs_s + static_cast<uint32_t>(g) * static_cast<uint32_t>(a.xpitch) + static_cast<uint32_t>(tig) * 16u +
                    static_cast<uint32_t>(s_begin) * 64u;
    const uint32_t x_tile = 8u * static_cast<uint32_t>(a.xpitch);

    // ---- after the dependency: activations, permuted: xs[row][step][tig][j][0..3] = X[row][64 step + 16 j + 4 tig ..+3];
    //      rows past n are zero ---------------------------------------------------------------------------------------
    grid_dep_wait();
    grid_dep_launch();
    {
        const int cpr = a.cols >> 4;  // 16-byte chunks per activation row
        for (int q = tid; q < 8 * NT * cpr; q += kGqThreads) {
            const int jr = q / cpr, c = q - jr * cpr;
            uint4 xv = make_uint4(0, 0, 0, 0);
            if (j0 + jr < a.n) xv = __ldg(reinterpret_cast<const uint4*>(a.X + static_cast<size_t>(j0 + jr) * a.cols) + c);
            const uint32_t s = static_cast<uint32_t>(c) >> 2, j = static_cast<uint32_t>(c) & 3u;
            const uint32_t d = xs_s + static_cast<uint32_t>(jr) * static_cast<uint32_t>(a.xpitch) + s * 64u + j * 4u;
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(d), "r"(xv.x) : "memory");
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 16u), "r"(xv.y) : "memory");
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 32u), "r"(xv.z) : "memory");
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 48u), "r"(xv.w) : "memory");
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // the slab, the table and the activations are visible

    int acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[t][i] = 0;
    // One step = 64 columns of 16 weight rows: re-encode once, one MMA per tile of activation rows.  Metadata
    // register of lane (g, tig): the index pairs of bitmap word 2 s + (tig >> 1) of row g + 8 (tig & 1).
    auto step = [&](uint32_t w0, uint32_t w1, uint32_t me_off, uint32_t x_off) {
        const uint32_t e = gq_index_pairs(gq_lds(me_p + me_off));
        const uint32_t a0 = gq_lds((__funnelshift_r(w0, w0, rot_lo) & 0x780u) | lane_or);
        const uint32_t a1 = gq_lds((__funnelshift_r(w1, w1, rot_lo) & 0x780u) | lane_or);
        const uint32_t a2 = gq_lds((__funnelshift_r(w0, w0, rot_hi) & 0x780u) | lane_or);
        const uint32_t a3 = gq_lds((__funnelshift_r(w1, w1, rot_hi) & 0x780u) | lane_or);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            uint32_t b0, b1, b2, b3;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                         : "r"(xq_p + x_off + static_cast<uint32_t>(t) * x_tile));
            asm volatile(
                "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
                "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
                : "+r"(acc[t][0]), "+r"(acc[t][1]), "+r"(acc[t][2]), "+r"(acc[t][3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(b2), "r"(b3), "r"(e));
        }
    };
    auto advance = [&](uint32_t steps) {
        me_p += 8u * steps;
        v0_p += 4u * steps;
        xq_p += 64u * steps;
    };
    int st = s_begin;
    for (; st < s_end && (st & 3) != 0; ++st) {
        step(gq_lds(v0_p), gq_lds(v0_p + v_half), 0u, 0u);
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
        step(gq_lds(v0_p), gq_lds(v0_p + v_half), 0u, 0u);
        advance(1u);
    }

    // Partial sums of the KS warps meet in shared memory (the activation area is free once everybody is done
    // with it): red[warp][row 0..15][column 0..8 NT).  Lane (g, tig) holds rows g, g + 8 x columns 2 tig, 2 tig + 1.
    __syncthreads();
    constexpr int NC = 8 * NT;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        volatile int* r0 = red + (warp * 16 + g) * NC + 8 * t + 2 * tig;
        r0[0] = acc[t][0];
        r0[1] = acc[t][1];
        r0[8 * NC] = acc[t][2];
        r0[8 * NC + 1] = acc[t][3];
    }
    __syncthreads();
    for (int o = tid; o < NC * nrows_blk; o += kGqThreads) {
        const int jc = o / nrows_blk, r = o - jc * nrows_blk;  // consecutive threads on consecutive weight rows
        if (r < valid && j0 + jc < a.n) {
            const int rblk = r >> 4, rr = r & 15;
            int sum = 0;
            for (int k = 0; k < a.ks; ++k) sum += red[(((rblk << a.ks_log2) + k) * 16 + rr) * NC + jc];
            const size_t o = static_cast<size_t>(j0 + jc) * a.rows + row0 + r;
            if (HALF_OUT)
                a.ep.out[o] = __float2half_rn(__fmul_rn(static_cast<float>(sum), dequant_scale(a.ep.gamma, a.ep.absmax[j0 + jc])));
            else
                a.Y[o] = sum;
        }
    }
}

// Whether the small-batch form applies: up to max_n activation rows, whole 16-byte sign rows (cols % 256 == 0),
// 16-byte aligned rows everywhere.
bool gemm_mmasp_supported(const uint32_t* meta, const uint32_t* values, const int8_t* X, int rows, int cols, int n,
                          int meta_stride, int values_stride, int max_n) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return rows > 0 && n > 0 && n <= max_n && cols > 0 && cols % 256 == 0 && cols <= 16384 &&
           meta_stride % 4 == 0 && values_stride % 4 == 0 && al16(meta) && al16(values) && al16(X);
}

int gemm_mmasp_launch(const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y, int rows, int cols,
                      int n, int meta_stride, int values_stride, void* stream, const GemmEpilogue* ep) {
    const char* name = "spb_sparse_ternary_gemm(mma.sp)";
    GqArgs a{};
    a.meta = meta; a.values = values; a.X = X; a.Y = Y;
    if (ep) a.ep = *ep;
    a.rows = rows; a.cols = cols; a.n = n;
    a.meta_stride = meta_stride; a.values_stride = values_stride;
    a.steps = cols / 64;
    const int row_blocks = (rows + 15) / 16;
    a.ks = 8;
    while (a.ks > 1 && a.steps / a.ks < 16) a.ks >>= 1;
    while (a.ks < 8 && row_blocks * a.ks < 2 * sm_count() && a.steps / (2 * a.ks) >= 8) a.ks <<= 1;
    while (a.ks > a.steps) a.ks >>= 1;
    a.rb = kGqWarps / a.ks;
    a.ks_log2 = a.ks == 8 ? 3 : a.ks == 4 ? 2 : a.ks == 2 ? 1 : 0;
    a.spw = (a.steps + a.ks - 1) / a.ks;
    auto pitch = [](int words) { return words + ((4 - words % 32) + 32) % 32; };  // smallest >= words that is 4 mod 32
    a.mpitch = pitch(cols / 32);
    a.vpitch = pitch(cols / 64);
    a.xpitch = cols + 64;
    // tiles of eight activation rows per block: all of them if the activations (and, later, the partial sums)
    // fit in about 100 KB next to the slab, else fewer and more blocks along y
    const int tiles = (n + 7) / 8;
    const size_t slab = static_cast<size_t>(16 * a.rb) * (a.mpitch + a.vpitch) * 4;
    int nt = tiles < kGqMaxTiles ? tiles : kGqMaxTiles;
    auto xbytes = [&](int t) {
        const size_t act = static_cast<size_t>(8 * t) * a.xpitch, part = static_cast<size_t>(kGqWarps) * 16 * 8 * t * 4;
        return act > part ? act : part;
    };
    while (nt > 1 && (nt == 3 || 2048 + kGqSignLutBytes + slab + xbytes(nt) > 110 * 1024)) --nt;
    const size_t smem = 2048 + kGqSignLutBytes + slab + xbytes(nt);
    if (smem > 200 * 1024) return fail(SPB_E_UNSUPPORTED, "%s: %d columns do not fit", name, cols);
    void (*kernel)(GqArgs) = nt == 1 ? gemm_mmasp_kernel<1, false> : nt == 2 ? gemm_mmasp_kernel<2, false> : gemm_mmasp_kernel<4, false>;
    if (a.ep.out) kernel = nt == 1 ? gemm_mmasp_kernel<1, true> : nt == 2 ? gemm_mmasp_kernel<2, true> : gemm_mmasp_kernel<4, true>;
    if (int rc = ensure_dynamic_smem(name, kernel, smem)) return rc;
    const dim3 grid((rows + 16 * a.rb - 1) / (16 * a.rb), (tiles + nt - 1) / nt);
    return launch(name, kernel, grid, dim3(kGqThreads), smem, stream, a);
}

}  // namespace spb
