// Batched sparse-ternary product on the 5th-generation tensor cores (tcgen05, sm_100a).
//
//   Y[j, r] = sum_c W[r, c] * X[j, c]      W: rows x cols compressed 2:4 ternary, X: n x cols int8
//
// A block owns 128 weight rows and up to 256 batch rows.  Per 128-column step of K it
//   * expands its 128 units (two threads per unit: 16 B meta + 8 B values -> 128 int8 through
//     the per-lane 64-entry group table) straight into shared memory in the canonical K-major
//     128-byte-swizzled operand layout (the A operand),
//   * brings the matching 128-byte slices of up to 256 activation rows into the same layout with
//     16-byte asynchronous copies issued one step ahead (the B operand),
//   * and one thread issues four tcgen05.mma.kind::i8 (M=128, N=batch tile, K=32 each) that
//     accumulate int32 in tensor memory.  tcgen05.commit signals an mbarrier when the MMAs that
//     read a stage are done, which is what lets the next expansion reuse it: expansion of step
//     k+1 overlaps the MMAs of step k through a ring of three stages.
// The epilogue reads the accumulators with tcgen05.ld (a warp owns 32 TMEM lanes = 32 weight
// rows) and stores Y with 128-byte coalesced writes.
// The weights stay in the reference's compressed format in HBM (1.5 bit/weight); the int8
// expansion exists only in shared memory.  The 2:4 structure is not yet handed to the sparse
// MMA (tcgen05.mma.sp needs the bitmaps re-encoded as index pairs in tensor memory); this is
// the dense kind::i8 form.
// Every wait is bounded; on expiry the block records it, frees its tensor memory and returns.
#include "spb_common.cuh"

namespace spb {

constexpr int kTcThreads = 256;
constexpr int kTileM = 128;
constexpr int kTileK = 128;
constexpr int kTcStages = 3;
constexpr unsigned kTcWaitLimit = 1u << 24;

struct TcArgs {
    const uint32_t* meta;
    const uint32_t* values;
    const int8_t* X;
    int32_t* Y;
    int rows, cols, n;
    int meta_stride, values_stride;
    int nt;         // batch rows per block: multiple of 16, at most 256
    int tmem_cols;  // power of two >= max(32, nt)
};

// Number of blocks whose bounded wait ran out since the library was loaded (0 in a healthy run).
__device__ int g_tc_timeouts = 0;

__device__ __forceinline__ uint32_t tc_smem(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// K-major, 128-byte swizzle: 8-row groups of 1024 B (SBO), 16-byte leading offset (LBO = 1).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);  // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                  // leading byte offset
    d |= static_cast<uint64_t>(1024 >> 4) << 32;          // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                  // descriptor version (sm_100)
    d |= static_cast<uint64_t>(2) << 61;                  // SWIZZLE_128B
    return d;
}

// kind::i8 instruction descriptor: S32 accumulate, signed 8-bit A and B, both K-major.
__device__ __forceinline__ uint32_t tc_idesc(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ bool tc_wait(uint32_t mbar, uint32_t parity) {
    for (unsigned spin = 0; spin < kTcWaitLimit; ++spin) {
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

// byte offset of 16-byte chunk c of row r inside a K-major SWIZZLE_128B tile (rows of 128 B)
__device__ __forceinline__ uint32_t tc_swz(int r, int c) {
    return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

__global__ void __launch_bounds__(kTcThreads, 1) gemm_tc_kernel(const TcArgs a) {
    extern __shared__ uint8_t tc_raw[];
    // [group table 8 KB][barriers + tmem slot 64 B] ... 1024-aligned: [stage: A 16 KB | B nt*128] x kTcStages
    uint32_t* lut = reinterpret_cast<uint32_t*>(tc_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tc_raw + kLutBytes);  // empty[0..S), done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tc_raw + kLutBytes + 8 * (kTcStages + 1));
    const uint32_t raw_s = tc_smem(tc_raw);
    const uint32_t stage0_s = (raw_s + kLutBytes + 64 + 1023) & ~1023u;
    uint8_t* stage0 = tc_raw + (stage0_s - raw_s);
    const int b_bytes = a.nt * 128;
    const int stage_bytes = kTileM * 128 + b_bytes;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = blockIdx.x * kTileM;
    const int n0 = blockIdx.y * a.nt;
    const int nchunks = a.cols / kTileK;

    grid_dep_launch();
    fill_lane_lut(lut, tid, kTcThreads);
    if (tid == 0) {
        for (int s = 0; s <= kTcStages; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(bars + s)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {  // tensor memory for the accumulator: one warp allocates
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(tmem_slot)),
                     "r"(static_cast<uint32_t>(a.tmem_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;

    // Expansion: thread t and thread t+128 share weight row (t & 127) of the tile; each expands
    // one half of the row's unit (64 columns = 16 groups = four 16-byte chunks) per step.
    const int trow = tid & (kTileM - 1), thalf = tid >> 7;
    const int wrow = row0 + trow;
    const bool wvalid = wrow < a.rows;
    uint2 m = make_uint2(0, 0);  // the two meta words of this half
    uint32_t v = 0;              // its 32 sign bits
    auto load_half = [&](int kc, uint2& mm, uint32_t& vv) {
        mm = ld_stream_v2(a.meta + static_cast<size_t>(wrow) * a.meta_stride + kc * 4 + thalf * 2);
        vv = __ldg(a.values + static_cast<size_t>(wrow) * a.values_stride + kc * 2 + thalf);
    };
    if (wvalid) load_half(0, m, v);

    grid_dep_wait();  // X may be a predecessor's output

    // Activations: 16-byte asynchronous copies (cp.async) into the swizzled B tile, issued one
    // step ahead of their use; rows beyond n are zero-filled by a zero source size.
    auto issue_b = [&](int kc) {
        uint8_t* sb = stage0 + static_cast<size_t>(kc % kTcStages) * stage_bytes + kTileM * 128;
        for (int i = tid; i < a.nt * 8; i += kTcThreads) {
            const int j = i >> 3, c = i & 7;
            const bool in = n0 + j < a.n;
            const int8_t* src = a.X + static_cast<size_t>(in ? n0 + j : 0) * a.cols + kc * kTileK + c * 16;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(tc_smem(sb + tc_swz(j, c))), "l"(src),
                         "r"(in ? 16 : 0)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue_b(0);

    const uint32_t idesc = tc_idesc(kTileM, a.nt);
    bool ok = true;
    for (int kc = 0; kc < nchunks; ++kc) {
        const int s = kc % kTcStages;
        uint8_t* sa = stage0 + static_cast<size_t>(s) * stage_bytes;
        uint8_t* sb = sa + kTileM * 128;
        // Stage of the NEXT step: the MMAs that read it last must be done before anything is written
        // to it (the outcome is made uniform across the block so that nobody is left at a barrier).
        if (kc + 1 < nchunks) {
            const int use_next = (kc + 1) / kTcStages;
            if (use_next > 0)
                ok = __syncthreads_and(tc_wait(tc_smem(bars + (kc + 1) % kTcStages), (use_next - 1) & 1) ? 1 : 0) != 0;
            if (!ok) break;
            issue_b(kc + 1);
        } else {
            asm volatile("cp.async.commit_group;" ::: "memory");  // keeps the group count uniform
        }
        {
            // next half-unit in flight while this one is expanded
            uint2 mn = make_uint2(0, 0);
            uint32_t vn = 0;
            if (wvalid && kc + 1 < nchunks) load_half(kc + 1, mn, vn);
            const uint32_t* lutp = lut + lane;
            const uint32_t mw[2] = {m.x, m.y};
#pragma unroll
            for (int c = 0; c < 4; ++c) {  // 16-byte chunk = 4 groups
                uint32_t w[4];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int grp = 4 * c + g;  // group inside this half (0..15)
                    const uint32_t idx = ((mw[grp >> 3] >> (4 * (grp & 7))) & 0xFu) | (((v >> (2 * grp)) & 0x3u) << 4);
                    w[g] = wvalid ? lutp[idx * 32] : 0u;
                }
                *reinterpret_cast<uint4*>(sa + tc_swz(trow, thalf * 4 + c)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            m = mn;
            v = vn;
        }
        // this step's activations have landed (all groups but the newest are complete)
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        // generic-proxy writes -> visible to the tensor core (async proxy), then hand over
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = tc_smem_desc(tc_smem(sa)), db = tc_smem_desc(tc_smem(sb));
#pragma unroll
            for (int k = 0; k < kTileK / 32; ++k) {
                const uint32_t acc = (kc > 0 || k > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                    :
                    : "r"(tmem_d), "l"(da + 2 * k), "l"(db + 2 * k), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
                    : "memory");
            }
            // arrives on the stage's barrier when the MMAs issued so far have completed
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(bars + s))
                         : "memory");
            if (kc == nchunks - 1)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 tc_smem(bars + kTcStages))
                             : "memory");
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- epilogue: accumulators -> Y ---------------------------------------------------------
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (ok) ok = tc_wait(tc_smem(bars + kTcStages), 0);
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        // warp w reads TMEM lanes 32*(w%4)..+31 (weight rows) and the column half w/4
        const int quarter = warp & 3, half = warp >> 2;
        const int row = row0 + quarter * 32 + lane;
        for (int c0 = half * 32; c0 < a.nt; c0 += 64) {
            uint32_t r[32];
            const uint32_t taddr = tmem_d + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(c0);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                  "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                  "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < a.rows) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int j = n0 + c0 + i;
                    if (c0 + i < a.nt && j < a.n) a.Y[static_cast<size_t>(j) * a.rows + row] = static_cast<int32_t>(r[i]);
                }
            }
        }
    } else if (tid == 0) {
        atomicAdd(&g_tc_timeouts, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                     "r"(static_cast<uint32_t>(a.tmem_cols))
                     : "memory");
}

// Launch of the tensor-core form; the caller has checked the layout.
int gemm_tc_launch(const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y, int rows, int cols,
                   int n, int meta_stride, int values_stride, void* stream) {
    TcArgs a{};
    a.meta = meta; a.values = values; a.X = X; a.Y = Y;
    a.rows = rows; a.cols = cols; a.n = n;
    a.meta_stride = meta_stride; a.values_stride = values_stride;
    a.nt = min(256, (n + 15) / 16 * 16);
    a.tmem_cols = 32;
    while (a.tmem_cols < a.nt) a.tmem_cols <<= 1;
    const size_t smem = kLutBytes + 64 + 1024 + static_cast<size_t>(kTcStages) * (kTileM * 128 + a.nt * 128);
    cudaError_t err = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "gemm_tc: %s", cudaGetErrorString(err));
    }
    const dim3 grid((rows + kTileM - 1) / kTileM, (n + a.nt - 1) / a.nt);
    return launch("spb_sparse_ternary_gemm(tcgen05)", gemm_tc_kernel, grid, dim3(kTcThreads), smem, stream, a);
}

int gemm_tcsp_timeouts();
int gemv_tcsp_timeouts();
int gemm_tcsp_ws_timeouts();

}  // namespace spb

extern "C" int spb_gemm_tc_timeouts(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, spb::g_tc_timeouts, sizeof v) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    const int w = spb::gemm_tcsp_timeouts(), g = spb::gemv_tcsp_timeouts(), s = spb::gemm_tcsp_ws_timeouts();
    return (w < 0 || g < 0 || s < 0) ? -1 : v + w + g + s;
}
