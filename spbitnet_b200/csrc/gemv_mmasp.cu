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
// weight slab (16 * RB rows, 3/16 byte per weight) arrives by one cp.async.bulk per row and array
// into padded shared-memory rows (conflict-free word reads), so every byte of the block is in
// flight from its first instructions and nothing is held in registers meanwhile.  Weights never
// depend on a predecessor kernel: the copies are issued before the dependency wait, x is staged
// after it.  Operand registers of a lane (g = lane / 4, tig = lane % 4), as the instruction defines
// them: A = four sign nibbles -> compressed columns 4 tig.. and 16 + 4 tig.. of rows g and g + 8;
// metadata = the index pairs of one whole bitmap word (word tig / 2 of the step, row g + 8 (tig & 1));
// B = x[64 s + 16 j + 4 tig ..] in register j, the same in all N = 8 columns (only column 0 is
// read).  Partial sums of the KS warps meet in shared memory.
// The wait for the copies is bounded; a block whose wait runs out records it and returns without
// storing.
#include "spb_common.cuh"

namespace spb {

constexpr int kGmThreads = 256;
constexpr int kGmWarps = kGmThreads / 32;
constexpr int kGmSignLutBytes = 16 * 32 * 4;  // 2 KB on a 2 KB boundary
constexpr unsigned kGmWaitLimit = 1u << 22;

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
    int rb;         // row blocks per thread block = 8 / ks
    int spw;        // steps per warp
    int mpitch;     // shared-memory row pitch of the bitmap words, in words (= 4 mod 32)
    int vpitch;     // same for the sign words
};

// Number of blocks whose bounded wait ran out since the library was loaded (0 in a healthy run).
__device__ int g_gemv_mma_timeouts = 0;

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

__global__ void __launch_bounds__(kGmThreads, 4) gemv_mmasp_kernel(const GmArgs a) {
    extern __shared__ uint8_t gm_raw[];
    // 2 KB-aligned: [sign table 2 KB][mbarrier 16 B][partial sums 8 warps x 16 ints][x, permuted: cols bytes]
    //               [bitmap rows: 16 rb x mpitch words][sign rows: 16 rb x vpitch words]
    const uint32_t raw_s = static_cast<uint32_t>(__cvta_generic_to_shared(gm_raw));
    const uint32_t base_s = (raw_s + 2047u) & ~2047u;
    uint8_t* base = gm_raw + (base_s - raw_s);
    const uint32_t bar_s = base_s + kGmSignLutBytes;
    volatile int* red = reinterpret_cast<volatile int*>(base + kGmSignLutBytes + 16);
    const uint32_t xs_s = base_s + kGmSignLutBytes + 16 + kGmWarps * 16 * 4;
    const uint32_t ms_s = xs_s + static_cast<uint32_t>(a.cols);
    const int nrows_blk = 16 * a.rb;
    const uint32_t vs_s = ms_s + static_cast<uint32_t>(nrows_blk * a.mpitch) * 4u;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = blockIdx.x * nrows_blk;
    const int valid = min(nrows_blk, a.rows - row0);  // rows of this block inside the matrix
    const uint32_t mbytes = static_cast<uint32_t>(a.cols >> 3), vbytes = static_cast<uint32_t>(a.cols >> 4);

    grid_dep_launch();
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_s));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_s),
                     "r"(static_cast<uint32_t>(valid) * (mbytes + vbytes))
                     : "memory");
    }
    __syncthreads();
    // one bulk copy per (row, array): thread t < rows copies bitmap row t, thread 32.. the sign rows
    {
        const int r = tid & 63, which = tid >> 6;  // which: 0 bitmaps, 1 signs (rows <= 64)
        if (which < 2 && r < valid) {
            const size_t grow = static_cast<size_t>(row0 + r);
            const void* src = which == 0 ? static_cast<const void*>(a.meta + grow * a.meta_stride)
                                         : static_cast<const void*>(a.values + grow * a.values_stride);
            const uint32_t dst = which == 0 ? ms_s + static_cast<uint32_t>(r * a.mpitch) * 4u
                                            : vs_s + static_cast<uint32_t>(r * a.vpitch) * 4u;
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                         "l"(src), "r"(which == 0 ? mbytes : vbytes), "r"(bar_s)
                         : "memory");
        }
    }
    // sign table under the copy latency: entry (nibble n, lane l) at n * 128 + l * 4, byte b = -1 if bit b of n
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const uint32_t i = tid + j * kGmThreads;
        const uint32_t t = ((i >> 5) * 0x00204081u) & 0x01010101u;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(base_s + i * 4u), "r"((t * 0xFEu) | 0x01010101u) : "memory");
    }

    const int g = lane >> 2, tig = lane & 3;
    const int rbi = warp / a.ks, kq = warp - rbi * a.ks;
    const int s_begin = kq * a.spw, s_end = min(a.steps, s_begin + a.spw);
    const uint32_t lane_or = base_s | (static_cast<uint32_t>(lane) << 2);
    const uint32_t sh = static_cast<uint32_t>(tig) * 4u;
    // word addresses at step 0: the lane's bitmap word, the sign words of rows g and g + 8 of the row block
    const uint32_t me_s = ms_s + static_cast<uint32_t>((rbi * 16 + g + 8 * (tig & 1)) * a.mpitch + (tig >> 1)) * 4u;
    const uint32_t v0_s = vs_s + static_cast<uint32_t>((rbi * 16 + g) * a.vpitch) * 4u;
    const uint32_t v1_s = v0_s + static_cast<uint32_t>(8 * a.vpitch) * 4u;
    const uint32_t xq_s = xs_s + static_cast<uint32_t>(tig) * 16u;

    // ---- after the dependency: x, permuted so that a lane's four B registers of a step are 16 contiguous bytes:
    //      xs[step][tig][j][0..3] = x[64 step + 16 j + 4 tig + 0..3] -------------------------------------------
    grid_dep_wait();
    for (int q = tid; q < (a.cols >> 4); q += kGmThreads) {
        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(a.x) + q);
        const uint32_t s = static_cast<uint32_t>(q) >> 2, j = static_cast<uint32_t>(q) & 3u;
        const uint32_t d = xs_s + s * 64u + j * 4u;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d), "r"(xv.x) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 16u), "r"(xv.y) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 32u), "r"(xv.z) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 48u), "r"(xv.w) : "memory");
    }
    // the weights have landed (bounded wait), the table and x are visible
    bool ok = false;
    for (unsigned spin = 0; spin < kGmWaitLimit && !ok; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar_s), "r"(0u)
            : "memory");
        ok = done != 0;
    }
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (!ok) {
        if (tid == 0) atomicAdd(&g_gemv_mma_timeouts, 1);
        return;
    }

    int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
    for (int s = s_begin; s < s_end; ++s) {
        const uint32_t so = static_cast<uint32_t>(s);
        // metadata register of lane (g, tig): the eight groups of bitmap word 2 s + (tig >> 1) of row g + 8 (tig & 1)
        const uint32_t e = gm_index_pairs(gm_lds(me_s + so * 8u));
        const uint32_t t0 = gm_lds(v0_s + so * 4u) >> sh, t1 = gm_lds(v1_s + so * 4u) >> sh;
        const uint32_t a0 = gm_lds(((t0 << 7) & 0x780u) | lane_or), a1 = gm_lds(((t1 << 7) & 0x780u) | lane_or);
        const uint32_t a2 = gm_lds(((t0 >> 9) & 0x780u) | lane_or), a3 = gm_lds(((t1 >> 9) & 0x780u) | lane_or);
        uint32_t b0, b1, b2, b3;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(xq_s + so * 64u));
        asm volatile(
            "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
            "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
            : "+r"(c0), "+r"(c1), "+r"(c2), "+r"(c3)
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(b2), "r"(b3), "r"(e));
    }
    // column 0 of the tile: lanes with tig == 0 hold rows g (c0) and g + 8 (c2)
    if (tig == 0) {
        red[warp * 16 + g] = c0;
        red[warp * 16 + g + 8] = c2;
    }
    __syncthreads();
    if (tid < nrows_blk && tid < valid) {
        const int rblk = tid >> 4, r = tid & 15;
        int acc = 0;
        for (int k = 0; k < a.ks; ++k) acc += red[(rblk * a.ks + k) * 16 + r];
        const int row = row0 + tid;
        if (a.out_mode == GM_OUT_I32) {
            static_cast<int32_t*>(a.y)[row] = acc;
        } else {
            const float f = __fmul_rn(static_cast<float>(acc), dequant_scale(a.gamma, *a.d_absmax));
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
    return rows > 0 && cols > 0 && cols % 256 == 0 && cols <= 16384 && meta_stride % 4 == 0 && values_stride % 4 == 0 &&
           al16(meta) && al16(values) && al16(x);
}

int gemv_mmasp_launch(const char* name, const uint32_t* meta, const uint32_t* values, const int8_t* x, void* y,
                      int32_t* y_acc, const float* d_absmax, float gamma, int out_mode, int rows, int cols,
                      int meta_stride, int values_stride, void* stream) {
    GmArgs a{};
    a.meta = meta; a.values = values; a.x = x; a.y = y; a.y_acc = y_acc; a.d_absmax = d_absmax; a.gamma = gamma;
    a.out_mode = out_mode; a.rows = rows; a.cols = cols; a.meta_stride = meta_stride; a.values_stride = values_stride;
    a.steps = cols / 64;
    a.ks = 8;
    while (a.ks > a.steps) a.ks >>= 1;
    a.rb = kGmWarps / a.ks;
    a.spw = (a.steps + a.ks - 1) / a.ks;
    auto pitch = [](int words) { return words + ((4 - words % 32) + 32) % 32; };  // smallest >= words that is 4 mod 32
    a.mpitch = pitch(cols / 32);
    a.vpitch = pitch(cols / 64);
    const size_t smem = 2048 + kGmSignLutBytes + 16 + kGmWarps * 16 * 4 + static_cast<size_t>(cols) +
                        static_cast<size_t>(16 * a.rb) * (a.mpitch + a.vpitch) * 4;
    cudaError_t err = cudaFuncSetAttribute(gemv_mmasp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "%s: %s", name, cudaGetErrorString(err));
    }
    const unsigned blocks = static_cast<unsigned>((rows + 16 * a.rb - 1) / (16 * a.rb));
    return launch(name, gemv_mmasp_kernel, dim3(blocks), dim3(kGmThreads), smem, stream, a);
}

int gemv_mmasp_timeouts() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_mma_timeouts, sizeof v) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return v;
}

}  // namespace spb
