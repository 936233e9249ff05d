// Sparse-ternary GEMV on the sparse tensor-core path (tcgen05.mma.sp.kind::i8, sm_100a).
//
//   y[r] = sum_c W[r, c] * x[c]          W: rows x cols compressed 2:4 ternary, x: int8
//
// Decoding this format on the SIMT pipes costs about eight issued instructions per group of four
// weights, which caps a B200 far below its HBM bandwidth.  Here the SIMT side only re-encodes:
// per unit (128 columns of a row = 16 B of bitmaps + 8 B of signs) a thread turns the four
// bitmap words into four words of 2-bit index pairs (five logical operations per word) that go
// to tensor memory with tcgen05.st, and the 64 sign bits into 64 bytes of +1 / -1 (sign nibble
// -> four bytes through a 16-entry per-lane table) that go to shared memory as the compressed
// A operand.  The multiply-add itself is done by tcgen05.mma.sp with M = 128 rows, N = 8
// (row 0 of the N operand carries x; the other seven rows are never initialised and only feed
// accumulator columns that are never read), K = 64 columns per instruction.
//
// Work split: a block owns 128 rows x up to 1024 columns (one to four units per thread, all loaded
// up front so that a block has its whole weight slab in flight at once).  Every unit has its own
// accumulator in tensor memory and its MMAs are issued by a warp of its own, so issue is spread
// over the block.  The column slabs of a row tile form a thread-block cluster; ranks 1.. send
// their int32 partial sums to rank 0 with st.async (data + completion on rank 0's mbarrier), and
// rank 0 adds them, applies the output scaling and stores.  Weights never depend on a predecessor
// kernel, so loading and re-encoding run before the dependency wait; only the x slab, the MMAs and
// the epilogue come after it.
// Every mbarrier wait is bounded (rank 0's wait for its peers longer than the peers' own waits, and
// a peer sends its partial sums even when its own wait ran out, so rank 0 never leaves while data
// for it can still be in flight); a block whose wait runs out records it, frees its tensor memory
// and returns.
#include <cstdlib>

#include "spb_common.cuh"

namespace spb {

constexpr int kGtThreads = 256;
constexpr int kGtTileM = 128;
constexpr int kGtMaxUnitsPerThread = 4;                      // a block covers at most 8 units = 1024 columns
constexpr int kGtMaxUnits = 2 * kGtMaxUnitsPerThread;
constexpr int kGtMaxSplit = 8;                               // portable cluster size
constexpr int kGtSignLutBytes = 16 * 32 * 4;                 // 2 KB, placed on a 2 KB boundary
constexpr int kGtHeadBytes = 6144;                           // table, barriers, partial sums of the peers
constexpr int kGtATileBytes = kGtTileM * 128;                // two units of 128 rows: 128 x 128 B
constexpr unsigned kGtWaitLimit = 1u << 22;
constexpr unsigned kGtPeerWaitLimit = 1u << 24;

enum { GT_OUT_I32 = 0, GT_OUT_F32 = 1, GT_OUT_F16 = 2 };

struct GtArgs {
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
    int upr;        // units per row
    int upc;        // units per block (column slab), at most 2 * UPT
    int ksplit;     // blocks per row tile = cluster size
    int tmem_cols;  // power of two >= 24 * UPT
};

// Number of blocks whose bounded wait ran out since the library was loaded (0 in a healthy run).
__device__ int g_gemv_tc_timeouts = 0;

// Development aid, compiled out unless SPB_GT_TRACE is defined: per-block cycle stamps of the phases.
#ifdef SPB_GT_TRACE
// slot = (launch id taken from gamma) * 512 + linear block index; entries 0 and 15 are globaltimer, the rest clock64
__device__ long long g_gt_trace[4 * 512 * 16];
__device__ __forceinline__ unsigned long long gt_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define GT_STAMP(k)                                                                                          \
    do {                                                                                                     \
        if (threadIdx.x == 0)                                                                                \
            g_gt_trace[((static_cast<int>(a.gamma) & 3) * 512 + (blockIdx.y * gridDim.x + blockIdx.x) % 512) * 16 + (k)] = \
                ((k) == 0 || (k) == 15) ? static_cast<long long>(gt_globaltimer()) : clock64();              \
    } while (0)
#else
#define GT_STAMP(k)
#endif

// K-major operand tile with 128-byte swizzle: 8-row groups of 1024 B, 16-byte leading offset.
__device__ __forceinline__ uint64_t gt_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Eight bitmaps (two of four bits set each) -> eight index pairs {low index | high index << 2}.
//   low  = first set bit:  bit0 = ~b0 & b1,  bit1 = ~b0 & ~b1
//   high = last set bit:   bit0 = b3 | ~b2,  bit1 = b3 | b2
__device__ __forceinline__ uint32_t gt_index_pairs(uint32_t m) {
    const uint32_t mr = m >> 1, ml = m << 1;
    const uint32_t t1 = (0x11111111u & (~m & mr)) | (~0x11111111u & (mr | ~m));
    const uint32_t t2 = (0x22222222u & (~ml & ~m)) | (~0x22222222u & (m | ml));
    return (t1 & 0x55555555u) | (t2 & 0xAAAAAAAAu);
}

__device__ __forceinline__ bool gt_wait(uint32_t mbar, uint32_t parity, unsigned limit) {
    for (unsigned spin = 0; spin < limit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(mbar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// UPT = units per thread; the block covers up to 2 * UPT units of its 128 rows.
template <int UPT>
__global__ void __launch_bounds__(kGtThreads, 4) gemv_tcsp_kernel(const GtArgs a) {
    extern __shared__ uint8_t gt_raw[];
    // 2 KB-aligned: [sign table 2 KB][mbarriers, tmem slot: 64 B][partial sums of ranks 1..7: 3.5 KB] pad to 6 KB
    //               [x slab: upc sub-tiles of 8 rows x 128 B][A tiles: ceil(upc/2) x 16 KB]
    const uint32_t raw_s = static_cast<uint32_t>(__cvta_generic_to_shared(gt_raw));
    const uint32_t base_s = (raw_s + 2047u) & ~2047u;
    uint8_t* base = gt_raw + (base_s - raw_s);
    const uint32_t bar_done_s = base_s + kGtSignLutBytes, bar_red_s = bar_done_s + 8;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base + kGtSignLutBytes + 16);
    const volatile int* red = reinterpret_cast<const volatile int*>(base + kGtSignLutBytes + 64);
    const uint32_t red_s = base_s + kGtSignLutBytes + 64;
    const uint32_t sb_s = base_s + kGtHeadBytes;
    const uint32_t sa_s = sb_s + static_cast<uint32_t>(a.upc) * 1024u;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int krank = blockIdx.x;  // == rank in the cluster: the cluster spans the whole x extent
    const int row0 = blockIdx.y * kGtTileM;
    const int u0 = krank * a.upc;
    const int cnt = min(a.upc, a.upr - u0);  // units of this block, >= 1
    constexpr uint32_t kECol0 = 16 * UPT;     // metadata columns behind the 2 * UPT accumulators of 8 columns

    grid_dep_launch();
    GT_STAMP(0);
    GT_STAMP(1);
    // Tensor memory first: the allocation permit is given back before anything slow happens.
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base_s + kGtSignLutBytes + 16),
                     "r"(static_cast<uint32_t>(a.tmem_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_done_s), "r"(cnt));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_red_s));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (krank == 0 && a.ksplit > 1)  // the peers' partial sums: 128 ints from each
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_red_s),
                         "r"(static_cast<uint32_t>((a.ksplit - 1) * kGtTileM * 4))
                         : "memory");
    }
    // "this block is running and its barriers exist" (made visible by the fence above): peers wait for it
    // before they send to rank 0.
    if (a.ksplit > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    GT_STAMP(2);

    // ---- weights of this thread: row (tid & 127), units thalf, thalf + 2, ... of the slab.  Rows past the
    //      end of the matrix re-read the last row; their results are never stored. ------------------------
    const int trow = tid & (kGtTileM - 1), thalf = tid >> 7;
    const int wrow = row0 + trow;
    const int lrow = min(wrow, a.rows - 1);
    const uint32_t* mrow = a.meta + static_cast<size_t>(lrow) * a.meta_stride + (u0 + thalf) * 4;
    const uint32_t* vrow = a.values + static_cast<size_t>(lrow) * a.values_stride + (u0 + thalf) * 2;
    uint4 m[UPT];
    uint2 v[UPT];
#pragma unroll
    for (int i = 0; i < UPT; ++i) {
        if (thalf + 2 * i < cnt) {
            m[i] = ld_stream_v4(mrow + 8 * i);
            v[i] = ld_stream_v2(vrow + 4 * i);
        }
    }
    // ---- set-up under the load latency: sign table, tensor memory ------------------------------------
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        // entry (sign nibble n, lane l) at n * 128 + l * 4: byte b = 0xFF (-1) if bit b of n is set, else 0x01
        const uint32_t i = tid + j * kGtThreads;
        const uint32_t t = ((i >> 5) * 0x00204081u) & 0x01010101u;
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(base_s + i * 4u), "r"((t * 0xFEu) | 0x01010101u) : "memory");
    }
    GT_STAMP(5);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;
    GT_STAMP(3);
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;

    // ---- re-encode: index pairs -> tensor memory, sign bytes -> the swizzled A tiles ---------------
    const uint32_t lane_or = base_s | (static_cast<uint32_t>(lane) << 2);
    const uint32_t x7 = static_cast<uint32_t>(trow & 7);
    const uint32_t rowbase = sa_s + static_cast<uint32_t>(trow >> 3) * 1024u + x7 * 128u;
    uint32_t st_addr[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) st_addr[c] = rowbase + (((static_cast<uint32_t>(thalf) * 4u + c) ^ x7) << 4);
#pragma unroll
    for (int i = 0; i < UPT; ++i) {
        const int u = thalf + 2 * i;
        if (u < cnt) {  // uniform over a warp
            const uint32_t e0 = gt_index_pairs(m[i].x), e1 = gt_index_pairs(m[i].y);
            const uint32_t e2 = gt_index_pairs(m[i].z), e3 = gt_index_pairs(m[i].w);
            const uint32_t eaddr = tmem_d + lane_base + kECol0 + static_cast<uint32_t>(u * 4);
            asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(eaddr), "r"(e0), "r"(e1),
                         "r"(e2), "r"(e3)
                         : "memory");
            const uint32_t vw[2] = {v[i].x, v[i].y};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int nibble = 4 * c + q, sh = 4 * (nibble & 7);
                    const uint32_t word = vw[nibble >> 3];
                    const uint32_t t = sh >= 7 ? (word >> (sh - 7)) : (word << (7 - sh));  // nibble at bits 7..10
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[q]) : "r"((t & 0x780u) | lane_or));
                }
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(st_addr[c] + i * kGtATileBytes), "r"(w[0]),
                             "r"(w[1]), "r"(w[2]), "r"(w[3])
                             : "memory");
            }
        }
    }
    GT_STAMP(4);
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");

    // Warp (h, j) issues the two MMAs of unit h + 2j into that unit's own accumulator; everything the
    // instructions need is prepared here, ahead of the dependency wait.
    constexpr uint32_t kIdesc = (1u << 2) | (2u << 4) | (1u << 7) | (1u << 10) | (1u << 17) |
                                (static_cast<uint32_t>(kGtTileM >> 4) << 24);  // sparse, S32, S8 x S8, N 8, M 128
    const int mma_j = warp & 3, mma_u = (warp >> 2) + 2 * mma_j;
    const bool issuer = mma_j < UPT && mma_u < cnt && lane == 0;
    const uint64_t mma_da = gt_smem_desc(sa_s + static_cast<uint32_t>(mma_j) * kGtATileBytes) + static_cast<uint64_t>(4 * (mma_u & 1));
    const uint64_t mma_db = gt_smem_desc(sb_s + static_cast<uint32_t>(mma_u) * 1024u);
    const uint32_t mma_td = tmem_d + static_cast<uint32_t>(8 * mma_u);
    const uint32_t mma_te = tmem_d + kECol0 + static_cast<uint32_t>(4 * mma_u);

    // ---- after the dependency: x slab, MMAs, epilogue -----------------------------------------------
    grid_dep_wait();
    GT_STAMP(6);
    if (tid < cnt * 8) {  // row 0 of a sub-tile is not swizzled
        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(u0) * 128) + tid);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sb_s + (tid >> 3) * 1024u + (tid & 7) * 16u),
                     "r"(xv.x), "r"(xv.y), "r"(xv.z), "r"(xv.w)
                     : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    GT_STAMP(7);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (issuer) {
        asm volatile(  // columns 0..63 of the unit: overwrite the accumulator
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.sp.cta_group::1.kind::i8 [%0], %1, %2, [%4], %3, {%5, %5, %5, %5}, p;\n\t}"
            :
            : "r"(mma_td), "l"(mma_da), "l"(mma_db), "r"(kIdesc), "r"(mma_te), "r"(0u), "r"(0u)
            : "memory");
        asm volatile(  // columns 64..127: accumulate
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.sp.cta_group::1.kind::i8 [%0], %1, %2, [%4], %3, {%5, %5, %5, %5}, p;\n\t}"
            :
            : "r"(mma_td), "l"(mma_da + 2), "l"(mma_db + 4), "r"(kIdesc), "r"(mma_te + 2), "r"(0u), "r"(1u)
            : "memory");
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_done_s)
                     : "memory");
    }
    GT_STAMP(8);
    int part = 0;
    bool ok = true;
    if (warp < 4) {  // column 0 of every accumulator: lane = row
        ok = __all_sync(0xFFFFFFFFu, gt_wait(bar_done_s, 0, kGtWaitLimit) ? 1 : 0) != 0;
        GT_STAMP(9);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            uint32_t r[2 * UPT];
#pragma unroll
            for (int u = 0; u < 2 * UPT; ++u) {
                r[u] = 0;
                if (u < cnt)
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];"
                                 : "=r"(r[u])
                                 : "r"(tmem_d + lane_base + static_cast<uint32_t>(8 * u))
                                 : "memory");
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int u = 0; u < 2 * UPT; ++u) part += static_cast<int>(r[u]);
        } else if (lane == 0) {
            atomicAdd(&g_gemv_tc_timeouts, 1);
        }
    }
    GT_STAMP(10);
    if (a.ksplit > 1) {
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        GT_STAMP(11);  // rank 0 runs and its barrier exists
        if (warp < 4) {
            if (krank != 0) {
                uint32_t rdata, rbar;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rdata) : "r"(red_s + ((krank - 1) * kGtTileM + tid) * 4u), "r"(0));
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(bar_red_s), "r"(0));
                asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(rdata),
                             "r"(part), "r"(rbar)
                             : "memory");
            } else {
                const bool got = __all_sync(0xFFFFFFFFu, gt_wait(bar_red_s, 0, kGtPeerWaitLimit) ? 1 : 0) != 0;
                if (!got && ok && lane == 0) atomicAdd(&g_gemv_tc_timeouts, 1);
                ok = ok && got;
                for (int r = 0; r < a.ksplit - 1; ++r) part += red[r * kGtTileM + tid];
            }
        }
    }
    GT_STAMP(12);
    if (krank == 0 && warp < 4 && wrow < a.rows && ok) {
        if (a.out_mode == GT_OUT_I32) {
            static_cast<int32_t*>(a.y)[wrow] = part;
        } else {
            const float dq = dequant_scale(a.gamma, *a.d_absmax);
            const float f = __fmul_rn(static_cast<float>(part), dq);
            if (a.out_mode == GT_OUT_F32) {
                static_cast<float*>(a.y)[wrow] = f;
                if (a.y_acc) a.y_acc[wrow] = part;
            } else {
                static_cast<__half*>(a.y)[wrow] = __float2half_rn(f);
            }
        }
    }
    GT_STAMP(13);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    GT_STAMP(14);
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                     "r"(static_cast<uint32_t>(a.tmem_cols))
                     : "memory");
    GT_STAMP(15);
}

// Whether the layout can take the tensor-core GEMV (the caller has checked pointers and strides for the
// ordinary fast path: cols % 128 == 0, 16/8-byte aligned rows, 16-byte aligned x).
bool gemv_tcsp_supported(int rows, int cols) {
    return rows > 0 && cols % 128 == 0 && cols / 128 <= kGtMaxUnits * kGtMaxSplit;
}

int gemv_tcsp_launch(const char* name, const uint32_t* meta, const uint32_t* values, const int8_t* x, void* y,
                     int32_t* y_acc, const float* d_absmax, float gamma, int out_mode, int rows, int cols,
                     int meta_stride, int values_stride, void* stream) {
    GtArgs a{};
    a.meta = meta; a.values = values; a.x = x; a.y = y; a.y_acc = y_acc; a.d_absmax = d_absmax; a.gamma = gamma;
    a.out_mode = out_mode; a.rows = rows; a.cols = cols; a.meta_stride = meta_stride; a.values_stride = values_stride;
    a.upr = cols / 128;
    const int mtiles = (rows + kGtTileM - 1) / kGtTileM;
    // Column split: enough blocks for about two per SM, slabs of at most kGtMaxUnits units.
    int ksplit = (a.upr + kGtMaxUnits - 1) / kGtMaxUnits;
    static const int per_sm = [] {
        const char* e = getenv("SPB_GEMV_TC_BLOCKS_PER_SM");
        const int v = e ? atoi(e) : 0;
        return v > 0 ? v : 2;
    }();
    const int want = (per_sm * sm_count() + mtiles - 1) / mtiles;
    ksplit = max(ksplit, min(want, kGtMaxSplit));
    ksplit = min(ksplit, min(a.upr, kGtMaxSplit));
    a.upc = (a.upr + ksplit - 1) / ksplit;
    a.ksplit = (a.upr + a.upc - 1) / a.upc;
    const int upt = (a.upc + 1) / 2;
    a.tmem_cols = 32;
    while (a.tmem_cols < 24 * upt) a.tmem_cols <<= 1;
    const size_t smem = 2048 + kGtHeadBytes + static_cast<size_t>(a.upc) * 1024 + static_cast<size_t>(upt) * kGtATileBytes;
    void (*kernel)(GtArgs) = upt == 1 ? gemv_tcsp_kernel<1> : upt == 2 ? gemv_tcsp_kernel<2>
                           : upt == 3 ? gemv_tcsp_kernel<3> : gemv_tcsp_kernel<4>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "%s: %s", name, cudaGetErrorString(err));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.ksplit, mtiles);
    cfg.blockDim = dim3(kGtThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (a.ksplit > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = a.ksplit;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    err = cudaLaunchKernelEx(&cfg, kernel, a);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "%s: launch failed: %s", name, cudaGetErrorString(err));
    }
    return SPB_OK;
}

#ifdef SPB_GT_TRACE
extern "C" int spb_debug_gt_trace(long long* out) {
    return cudaMemcpyFromSymbol(out, g_gt_trace, sizeof(long long) * 4 * 512 * 16) == cudaSuccess ? 0 : -1;
}
#endif

int gemv_tcsp_timeouts() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_tc_timeouts, sizeof v) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return v;
}

}  // namespace spb
