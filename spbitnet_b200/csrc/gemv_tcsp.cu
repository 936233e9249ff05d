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
// (column 0 carries x, the rest is zero), K = 64 columns per instruction.
//
// Work split: a block owns 128 rows x up to 1024 columns (one to four units per thread, all loaded
// up front so that a block has its whole weight slab in flight at once); the column slabs of a
// row tile form a thread-block cluster and reduce their int32 partial sums through distributed
// shared memory in rank 0, which applies the output scaling and stores.  Weights never depend on
// a predecessor kernel, so loading and re-encoding run before the dependency wait; only the x
// slab, the MMAs and the epilogue come after it.
// Every mbarrier wait is bounded; a block whose wait runs out records it, still takes part in the
// cluster barriers, frees its tensor memory and returns.
#include "spb_common.cuh"

namespace spb {

constexpr int kGtThreads = 256;
constexpr int kGtTileM = 128;
constexpr int kGtMaxUnitsPerThread = 4;                      // a block covers at most 8 units = 1024 columns
constexpr int kGtMaxUnits = 2 * kGtMaxUnitsPerThread;
constexpr int kGtMaxSplit = 8;                               // portable cluster size
constexpr int kGtSignLutBytes = 16 * 32 * 4;
constexpr int kGtRedBytes = kGtMaxSplit * kGtTileM * 4;
constexpr int kGtHeadBytes = kGtSignLutBytes + 64 + kGtRedBytes;
constexpr int kGtATileBytes = kGtTileM * 128;                // two units of 128 rows: 128 x 128 B
constexpr int kGtECol0 = 16;                                 // metadata columns start behind the accumulator
constexpr unsigned kGtWaitLimit = 1u << 22;

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
    int upc;        // units per block (column slab), at most kGtMaxUnits
    int ksplit;     // blocks per row tile = cluster size
    int tmem_cols;  // power of two >= kGtECol0 + 4 * upc
};

// Number of blocks whose bounded wait ran out since the library was loaded (0 in a healthy run).
__device__ int g_gemv_tc_timeouts = 0;

__device__ __forceinline__ uint32_t gt_smem(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

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

__device__ __forceinline__ uint32_t gt_swz(int r, int c) {
    return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

// Eight bitmaps (two of four bits set each) -> eight index pairs {low index | high index << 2}.
__device__ __forceinline__ uint32_t gt_index_pairs(uint32_t m) {
    const uint32_t mr = m >> 1, ml = m << 1;
    const uint32_t t1 = (0x11111111u & (~m & mr)) | (~0x11111111u & (mr | ~m));
    const uint32_t t2 = (0x22222222u & (~ml & ~m)) | (~0x22222222u & (m | ml));
    return (t1 & 0x55555555u) | (t2 & 0xAAAAAAAAu);
}

__device__ __forceinline__ void gt_cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void gt_cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(kGtThreads, 3) gemv_tcsp_kernel(const GtArgs a) {
    extern __shared__ uint8_t gt_raw[];
    // [sign table 2 KB][done barrier, tmem slot: 64 B][partial sums of the cluster 4 KB] ...
    // 1024-aligned: [x slab: upc sub-tiles of 8 rows x 128 B][A tiles: ceil(upc/2) x 16 KB]
    uint32_t* sgn = reinterpret_cast<uint32_t*>(gt_raw);
    uint64_t* bar_done = reinterpret_cast<uint64_t*>(gt_raw + kGtSignLutBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gt_raw + kGtSignLutBytes + 16);
    int* red = reinterpret_cast<int*>(gt_raw + kGtSignLutBytes + 64);
    const uint32_t raw_s = gt_smem(gt_raw);
    const uint32_t tiles_s = (raw_s + kGtHeadBytes + 1023) & ~1023u;
    uint8_t* sb = gt_raw + (tiles_s - raw_s);
    uint8_t* sa = sb + a.upc * 1024;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int krank = blockIdx.x;  // == rank in the cluster: the cluster spans the whole x extent
    const int row0 = blockIdx.y * kGtTileM;
    const int u0 = krank * a.upc;
    const int cnt = min(a.upc, a.upr - u0);  // units of this block, >= 1

    grid_dep_launch();
    // ---- prologue: table, barrier, tensor memory, zero rows 1..7 of the x sub-tiles ----------------
    for (int i = tid; i < 16 * 32; i += kGtThreads) {
        const int nib = i >> 5;
        uint32_t w = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) w |= (((nib >> b) & 1) ? 0xFFu : 0x01u) << (8 * b);
        sgn[i] = w;
    }
    for (int i = tid; i < a.upc * 64; i += kGtThreads)  // 64 16-byte chunks per sub-tile, first 8 = row 0
        if ((i & 63) >= 8) reinterpret_cast<uint4*>(sb)[i] = make_uint4(0, 0, 0, 0);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gt_smem(bar_done)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gt_smem(tmem_slot)),
                     "r"(static_cast<uint32_t>(a.tmem_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // ---- weights of this thread: row (tid & 127), units thalf, thalf + 2, ... of the slab -----------
    const int trow = tid & (kGtTileM - 1), thalf = tid >> 7;
    const int wrow = row0 + trow;
    const bool wvalid = wrow < a.rows;
    uint4 m[kGtMaxUnitsPerThread];
    uint2 v[kGtMaxUnitsPerThread];
#pragma unroll
    for (int i = 0; i < kGtMaxUnitsPerThread; ++i) {
        const int u = thalf + 2 * i;
        m[i] = make_uint4(0x33333333u, 0x33333333u, 0x33333333u, 0x33333333u);
        v[i] = make_uint2(0, 0);
        if (wvalid && u < cnt) {
            m[i] = ld_stream_v4(a.meta + static_cast<size_t>(wrow) * a.meta_stride + (u0 + u) * 4);
            v[i] = ld_stream_v2(a.values + static_cast<size_t>(wrow) * a.values_stride + (u0 + u) * 2);
        }
    }
    if (a.ksplit > 1) gt_cluster_arrive();  // "this block is running": peers wait for it before remote stores

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;

    // ---- re-encode: index pairs -> tensor memory, sign bytes -> the swizzled A tiles ---------------
    const uint8_t* sgn_lane = reinterpret_cast<const uint8_t*>(sgn + lane);
#pragma unroll
    for (int i = 0; i < kGtMaxUnitsPerThread; ++i) {
        const int u = thalf + 2 * i;
        if (u < cnt) {  // uniform over a warp
            const uint32_t e0 = gt_index_pairs(m[i].x), e1 = gt_index_pairs(m[i].y);
            const uint32_t e2 = gt_index_pairs(m[i].z), e3 = gt_index_pairs(m[i].w);
            const uint32_t eaddr = tmem_d + lane_base + static_cast<uint32_t>(kGtECol0 + u * 4);
            asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(eaddr), "r"(e0), "r"(e1),
                         "r"(e2), "r"(e3)
                         : "memory");
            uint8_t* tile = sa + i * kGtATileBytes;
            const uint32_t vw[2] = {v[i].x, v[i].y};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int nibble = 4 * c + q;
                    const uint32_t nib = (vw[nibble >> 3] >> (4 * (nibble & 7))) & 0xFu;
                    w[q] = wvalid ? *reinterpret_cast<const uint32_t*>(sgn_lane + nib * 128) : 0u;
                }
                *reinterpret_cast<uint4*>(tile + gt_swz(trow, thalf * 4 + c)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");

    // ---- after the dependency: x slab, MMAs, epilogue -----------------------------------------------
    grid_dep_wait();
    if (tid < cnt * 8) {
        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(u0) * 128) + tid);
        *reinterpret_cast<uint4*>(sb + (tid >> 3) * 1024 + (tid & 7) * 16) = xv;  // row 0 of a sub-tile is not swizzled
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t idesc = (1u << 2) | (2u << 4) | (1u << 7) | (1u << 10) | (1u << 17) |
                               (static_cast<uint32_t>(kGtTileM >> 4) << 24);  // sparse, S32, S8 x S8, N = 8, M = 128
        for (int u = 0; u < cnt; ++u) {
            const uint64_t da = gt_smem_desc(gt_smem(sa + (u >> 1) * kGtATileBytes)) + static_cast<uint64_t>(4 * (u & 1));
            const uint64_t db = gt_smem_desc(gt_smem(sb + u * 1024));
#pragma unroll
            for (int k = 0; k < 2; ++k) {  // 64 columns each: 32 B of A, 64 B of x, two metadata columns
                const uint32_t acc = (u > 0 || k > 0) ? 1u : 0u;
                const uint32_t te = tmem_d + static_cast<uint32_t>(kGtECol0 + u * 4 + 2 * k);
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.sp.cta_group::1.kind::i8 [%0], %1, %2, [%9], %3, {%5, %6, %7, %8}, p;\n\t}"
                    :
                    : "r"(tmem_d), "l"(da + 2 * k), "l"(db + 4 * k), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u),
                      "r"(0u), "r"(te)
                    : "memory");
            }
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(gt_smem(bar_done))
                     : "memory");
    }
    bool ok = false;
    for (unsigned spin = 0; spin < kGtWaitLimit && !ok; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(gt_smem(bar_done)), "r"(0u)
            : "memory");
        ok = done != 0;
    }
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!ok && tid == 0) atomicAdd(&g_gemv_tc_timeouts, 1);

    int part = 0;
    if (warp < 4) {  // column 0 of the accumulator: lane = row
        uint32_t r0 = 0;
        if (ok) {
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r0) : "r"(tmem_d + lane_base) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        }
        part = static_cast<int>(r0);
    }
    if (a.ksplit > 1) {
        gt_cluster_wait();  // every block of the cluster is running: rank 0's shared memory may be written
        if (warp < 4) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(gt_smem(red + krank * kGtTileM + tid)), "r"(0));
            asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(remote), "r"(part) : "memory");
        }
        gt_cluster_arrive();
        gt_cluster_wait();
        if (krank == 0 && warp < 4) {
            part = 0;
            for (int r = 0; r < a.ksplit; ++r) part += red[r * kGtTileM + tid];
        }
    }
    if (krank == 0 && warp < 4 && wvalid && ok) {
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
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                     "r"(static_cast<uint32_t>(a.tmem_cols))
                     : "memory");
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
    const int want = (2 * sm_count() + mtiles - 1) / mtiles;
    ksplit = max(ksplit, min(want, kGtMaxSplit));
    ksplit = min(ksplit, min(a.upr, kGtMaxSplit));
    a.upc = (a.upr + ksplit - 1) / ksplit;
    a.ksplit = (a.upr + a.upc - 1) / a.upc;
    a.tmem_cols = 32;
    while (a.tmem_cols < kGtECol0 + 4 * a.upc) a.tmem_cols <<= 1;
    const size_t smem = kGtHeadBytes + 1024 + static_cast<size_t>(a.upc) * 1024 +
                        static_cast<size_t>((a.upc + 1) / 2) * kGtATileBytes;
    cudaError_t err = cudaFuncSetAttribute(gemv_tcsp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
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
    err = cudaLaunchKernelEx(&cfg, gemv_tcsp_kernel, a);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "%s: launch failed: %s", name, cudaGetErrorString(err));
    }
    return SPB_OK;
}

int gemv_tcsp_timeouts() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_tc_timeouts, sizeof v) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return v;
}

}  // namespace spb
