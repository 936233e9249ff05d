// Batched sparse-ternary product on the sparse tensor-core path (tcgen05.mma.sp, sm_100a).
//
//   Y[j, r] = sum_c W[r, c] * X[j, c]      W: rows x cols compressed 2:4 ternary, X: n x cols int8
//
// The 2:4 structure of the reference format is handed to the hardware instead of being expanded
// to a dense int8 tile: per group of four columns the tensor core wants the two kept values
// (here +1 / -1 as int8, the A operand in shared memory, half as wide as the dense tile) and
// the two column indices as a pair of 2-bit numbers (the metadata, in tensor memory).
// Per unit (128 columns of a row) a thread
//   * turns the four bitmap words into four index-pair words with five logical operations each
//     (bit-parallel over the eight groups of a word) and stores them with tcgen05.st into the
//     tensor-memory lane of its row,
//   * turns the 64 sign bits into 64 bytes of +1 / -1 through a 16-entry per-lane table
//     (sign nibble -> four bytes) and writes them as four 16-byte chunks of the K-major
//     128-byte-swizzled A tile.
// One thread then issues four tcgen05.mma.sp.kind::i8 (M=128, N=batch tile, K=64 each) per
// 256-column step; accumulators are int32 in tensor memory.  The activation tiles of a step
// arrive one step ahead by two tensor-map bulk copies (cp.async.bulk.tensor.2d, box 128 bytes x
// batch tile, 128-byte swizzle and zero fill past n done by the copy engine, completion on a
// "full" mbarrier per stage); the tensor map of X is encoded on the host per call through the
// driver entry point, and 16-byte cp.async by all threads remain as the fall-back.  The weight
// words of a thread are loaded four steps ahead.  A ring of stages (operand tiles + metadata
// slots) is recycled through tcgen05.commit on one mbarrier per stage.
// Every wait is bounded; on expiry the block records it, frees its tensor memory and returns.
#include <cuda.h>

#include <cstring>

#include "spb_common.cuh"

namespace spb {

constexpr int kSpThreads = 256;
constexpr int kSpTileM = 128;
constexpr int kSpStepK = 256;          // logical columns per step: two units per row
constexpr int kSpABytes = kSpTileM * 128;  // compressed A tile: 128 rows x 128 bytes
constexpr int kSpMaxStages = 4;
constexpr int kSpSignLutBytes = 16 * 32 * 4;
constexpr unsigned kSpWaitLimit = 1u << 24;

struct SpArgs {
    const uint32_t* meta;
    const uint32_t* values;
    const int8_t* X;
    int32_t* Y;
    int rows, cols, n;
    int meta_stride, values_stride;
    int nt;         // batch rows per block: multiple of 16, at most 256
    int stages;     // ring depth (2..kSpMaxStages)
    int tmem_cols;  // power of two >= nt + 8 * stages
};

// Number of blocks of this kernel whose bounded wait ran out since the library was loaded.
__device__ int g_tcsp_timeouts = 0;

__device__ __forceinline__ uint32_t sp_smem(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// K-major, 128-byte swizzle: 8-row groups of 1024 B (SBO), 16-byte leading offset.
__device__ __forceinline__ uint64_t sp_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// kind::i8 instruction descriptor with the sparse flag: S32 accumulate, signed 8-bit A and B, K-major.
__device__ __forceinline__ uint32_t sp_idesc(int m, int n) {
    return (1u << 2) | (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ bool sp_wait(uint32_t mbar, uint32_t parity) {
    for (unsigned spin = 0; spin < kSpWaitLimit; ++spin) {
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

__device__ __forceinline__ uint32_t sp_swz(int r, int c) {
    return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

// Eight bitmaps (two of four bits set each) -> eight index pairs {low index, high index << 2}.
//   low  = first set bit:  bit0 = ~b0 & b1,  bit1 = ~b0 & ~b1
//   high = last set bit:   bit0 = b3 | ~b2,  bit1 = b3 | b2
__device__ __forceinline__ uint32_t sp_index_pairs(uint32_t m) {
    const uint32_t mr = m >> 1, ml = m << 1;
    const uint32_t t1 = (0x11111111u & (~m & mr)) | (~0x11111111u & (mr | ~m));   // bit 0 and bit 2 of a nibble
    const uint32_t t2 = (0x22222222u & (~ml & ~m)) | (~0x22222222u & (m | ml));   // bit 1 and bit 3
    return (t1 & 0x55555555u) | (t2 & 0xAAAAAAAAu);
}

// TMAB: the activation tiles come in by two tensor-map bulk copies per step (cp.async.bulk.tensor, 128-byte
// swizzle written by the copy engine, rows past n zero-filled by it) issued by one thread, instead of 16-byte
// cp.async by everybody (4096 of them per step at 256 batch rows: they kept the load/store unit busy for about
// 3000 cycles per step).
template <bool TMAB>
__global__ void __launch_bounds__(kSpThreads, 1) gemm_tcsp_kernel(const SpArgs a, const __grid_constant__ CUtensorMap tmap_x) {
    extern __shared__ uint8_t sp_raw[];
    // [sign table 2 KB][barriers + tmem slot 128 B] ... 1024-aligned: [stage: A 16 KB | B0 nt*128 | B1 nt*128] x stages
    uint32_t* sgn = reinterpret_cast<uint32_t*>(sp_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sp_raw + kSpSignLutBytes);  // free[0..4), done, full[5..9)
    uint64_t* full = bars + kSpMaxStages + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sp_raw + kSpSignLutBytes + 96);
    const uint32_t raw_s = sp_smem(sp_raw);
    const uint32_t stage0_s = (raw_s + kSpSignLutBytes + 128 + 1023) & ~1023u;
    uint8_t* stage0 = sp_raw + (stage0_s - raw_s);
    const int b_bytes = a.nt * 128;  // one of the two activation sub-tiles
    const int stage_bytes = kSpABytes + 2 * b_bytes;
    const int S = a.stages;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = blockIdx.x * kSpTileM;
    const int n0 = blockIdx.y * a.nt;
    const int upr = a.cols >> 7;
    const int nsteps = (upr + 1) >> 1;

    grid_dep_launch();
    for (int i = tid; i < 16 * 32; i += kSpThreads) {
        const int nib = i >> 5;
        uint32_t w = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) w |= (((nib >> b) & 1) ? 0xFFu : 0x01u) << (8 * b);
        sgn[i] = w;
    }
    if (tid == 0) {
        for (int s = 0; s < 2 * kSpMaxStages + 1; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sp_smem(bars + s)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sp_smem(tmem_slot)),
                     "r"(static_cast<uint32_t>(a.tmem_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;
    const uint32_t tmem_e = tmem_d + static_cast<uint32_t>(a.nt);  // metadata slots behind the accumulator

    // Thread t and thread t+128 share weight row (t & 127) of the tile; per step the first expands
    // the even unit, the second the odd unit.  A warp's rows are the tensor-memory lanes it may access.
    const int trow = tid & (kSpTileM - 1), thalf = tid >> 7;
    const int wrow = row0 + trow;
    const bool wvalid = wrow < a.rows;
    uint4 m = make_uint4(0, 0, 0, 0);
    uint2 v = make_uint2(0, 0);
    bool uvalid = false;
    auto load_unit = [&](int step, uint4& mm, uint2& vv, bool& valid) {
        const int u = 2 * step + thalf;
        valid = wvalid && u < upr;
        if (valid) {
            mm = ld_stream_v4(a.meta + static_cast<size_t>(wrow) * a.meta_stride + u * 4);
            vv = ld_stream_v2(a.values + static_cast<size_t>(wrow) * a.values_stride + u * 2);
        }
    };
    load_unit(0, m, v, uvalid);
    // three more steps in flight: a step takes about as long as one trip to DRAM, so a single step of
    // look-ahead left every step waiting for its weights
    uint4 m1 = make_uint4(0, 0, 0, 0), m2 = m1, m3 = m1;
    uint2 v1 = make_uint2(0, 0), v2 = v1, v3 = v1;
    bool u1 = false, u2 = false, u3 = false;
    if (1 < nsteps) load_unit(1, m1, v1, u1);
    if (2 < nsteps) load_unit(2, m2, v2, u2);
    if (3 < nsteps) load_unit(3, m3, v3, u3);

    grid_dep_wait();  // X may be a predecessor's output

    // Activations: 16-byte asynchronous copies into the two swizzled sub-tiles of a stage, one step
    // ahead of their use; rows beyond n and columns beyond cols are zero-filled (zero source size).
    auto issue_b = [&](int step) {
        uint8_t* sb = stage0 + static_cast<size_t>(step % S) * stage_bytes + kSpABytes;
        if constexpr (TMAB) {
            if (tid == 0) {
                const uint32_t fb = sp_smem(full + step % S);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb),
                             "r"(static_cast<uint32_t>(2 * b_bytes))
                             : "memory");
#pragma unroll
                for (int h = 0; h < 2; ++h)  // columns [256 step + 128 h, +128) of batch rows [n0, n0 + nt)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                            sp_smem(sb + h * b_bytes)),
                        "l"(reinterpret_cast<uint64_t>(&tmap_x)), "r"(step * kSpStepK + 128 * h), "r"(n0), "r"(fb)
                        : "memory");
            }
        } else {
            for (int i = tid; i < a.nt * 16; i += kSpThreads) {
                const int j = i >> 4, c = i & 15;
                const int col = step * kSpStepK + c * 16;
                const bool in = n0 + j < a.n && col < a.cols;
                const int8_t* src = a.X + static_cast<size_t>(in ? n0 + j : 0) * a.cols + (in ? col : 0);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                                 sp_smem(sb + (c >> 3) * b_bytes + sp_swz(j, c & 7))),
                             "l"(src), "r"(in ? 16 : 0)
                             : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
    };
    issue_b(0);

    const uint32_t idesc = sp_idesc(kSpTileM, a.nt);
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint8_t* sgn_lane = reinterpret_cast<const uint8_t*>(sgn + lane);
    bool ok = true;
    for (int kc = 0; kc < nsteps; ++kc) {
        const int s = kc % S;
        uint8_t* sa = stage0 + static_cast<size_t>(s) * stage_bytes;
        uint8_t* sb = sa + kSpABytes;
        {
            uint4 mn = make_uint4(0, 0, 0, 0);
            uint2 vn = make_uint2(0, 0);
            bool nvalid = false;
            if (kc + 4 < nsteps) load_unit(kc + 4, mn, vn, nvalid);
            // metadata: index pairs of this unit's 32 groups -> four tensor-memory columns of the row
            uint32_t e0 = 0x44444444u, e1 = 0x44444444u, e2 = 0x44444444u, e3 = 0x44444444u;
            if (uvalid) {
                e0 = sp_index_pairs(m.x);
                e1 = sp_index_pairs(m.y);
                e2 = sp_index_pairs(m.z);
                e3 = sp_index_pairs(m.w);
            }
            const uint32_t eaddr = tmem_e + lane_base + static_cast<uint32_t>(s * 8 + thalf * 4);
            asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(eaddr), "r"(e0), "r"(e1),
                         "r"(e2), "r"(e3)
                         : "memory");
            // values: sign nibble -> four bytes of +1 / -1; a unit is four 16-byte chunks of the row
            const uint32_t vw[2] = {v.x, v.y};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int nibble = 4 * c + q;  // 0..15 over the 64 sign bits
                    const uint32_t nib = (vw[nibble >> 3] >> (4 * (nibble & 7))) & 0xFu;
                    w[q] = uvalid ? *reinterpret_cast<const uint32_t*>(sgn_lane + nib * 128) : 0u;
                }
                *reinterpret_cast<uint4*>(sa + sp_swz(trow, thalf * 4 + c)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            m = m1; v = v1; uvalid = u1;
            m1 = m2; v1 = v2; u1 = u2;
            m2 = m3; v2 = v3; u2 = u3;
            m3 = mn; v3 = vn; u3 = nvalid;
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        // The stage of the NEXT step must have been released by the MMAs that read it last before its
        // activations are copied in and, one iteration later, its weights expanded (the outcome is made
        // uniform so that nobody is left at a barrier).  Waiting here, after the expansion, lets the
        // MMAs of the previous step run under this step's expansion even with two stages.
        if (kc + 1 < nsteps) {
            const int use_next = (kc + 1) / S;
            if (use_next > 0)
                ok = __syncthreads_and(sp_wait(sp_smem(bars + (kc + 1) % S), (use_next - 1) & 1) ? 1 : 0) != 0;
            if (!ok) break;
            issue_b(kc + 1);
        } else if constexpr (!TMAB) {
            asm volatile("cp.async.commit_group;" ::: "memory");  // keeps the group count uniform
        }
        if constexpr (!TMAB) asm volatile("cp.async.wait_group 1;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            bool landed = true;
            if constexpr (TMAB) landed = sp_wait(sp_smem(full + s), static_cast<uint32_t>(kc / S) & 1u);  // this step's activations
            if (!landed) atomicAdd(&g_tcsp_timeouts, 1);
            const uint64_t da = sp_smem_desc(sp_smem(sa));
            const uint64_t db0 = sp_smem_desc(sp_smem(sb)), db1 = sp_smem_desc(sp_smem(sb + b_bytes));
#pragma unroll
            for (int k = 0; k < 4 && landed; ++k) {  // 64 logical columns each: 32 B of A, 64 B of X, two metadata columns
                const uint32_t acc = (kc > 0 || k > 0) ? 1u : 0u;
                const uint64_t db = ((k & 2) ? db1 : db0) + static_cast<uint64_t>(4 * (k & 1));
                const uint32_t te = tmem_e + static_cast<uint32_t>(s * 8 + 2 * k);
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.sp.cta_group::1.kind::i8 [%0], %1, %2, [%9], %3, {%5, %6, %7, %8}, p;\n\t}"
                    :
                    : "r"(tmem_d), "l"(da + 2 * k), "l"(db), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u),
                      "r"(te)
                    : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sp_smem(bars + s))
                         : "memory");
            if (kc == nsteps - 1)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 sp_smem(bars + kSpMaxStages))
                             : "memory");
        }
    }
    if constexpr (!TMAB) asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- epilogue: accumulators -> Y ---------------------------------------------------------
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (ok) ok = sp_wait(sp_smem(bars + kSpMaxStages), 0);
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        const int quarter = warp & 3, half = warp >> 2;
        const int row = row0 + quarter * 32 + lane;
        for (int c0 = half * 32; c0 < a.nt; c0 += 64) {
            uint32_t r[32];
            const uint32_t taddr = tmem_d + lane_base + static_cast<uint32_t>(c0);
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
        atomicAdd(&g_tcsp_timeouts, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                     "r"(static_cast<uint32_t>(a.tmem_cols))
                     : "memory");
}

// Launch of the sparse tensor-core form; the caller has checked the layout (cols % 128 == 0, aligned rows).
int gemm_tcsp_launch(const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y, int rows, int cols,
                     int n, int meta_stride, int values_stride, void* stream) {
    SpArgs a{};
    a.meta = meta; a.values = values; a.X = X; a.Y = Y;
    a.rows = rows; a.cols = cols; a.n = n;
    a.meta_stride = meta_stride; a.values_stride = values_stride;
    a.nt = min(256, (n + 15) / 16 * 16);
    const int stage_bytes = kSpABytes + 2 * a.nt * 128;
    a.stages = max(2, min(kSpMaxStages, (200 * 1024) / stage_bytes));
    a.tmem_cols = 32;
    while (a.tmem_cols < a.nt + 8 * a.stages) a.tmem_cols <<= 1;
    const size_t smem = kSpSignLutBytes + 128 + 1024 + static_cast<size_t>(a.stages) * stage_bytes;
    // tensor map of X for the activation tiles: uint8 [n rows][cols], box 128 bytes x nt rows, 128-byte swizzle
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static const EncodeFn encode = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            p = nullptr;
        }
        return reinterpret_cast<EncodeFn>(p);
    }();
    alignas(64) CUtensorMap tmap;
    bool use_tma = encode != nullptr && cols % 128 == 0;
    if (use_tma) {
        const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(n)};
        const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(cols)};
        const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(a.nt)};
        const cuuint32_t estr[2] = {1u, 1u};
        use_tma = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(X), gdim, gstride, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    if (!use_tma) memset(&tmap, 0, sizeof tmap);
    void (*kernel)(SpArgs, CUtensorMap) = use_tma ? gemm_tcsp_kernel<true> : gemm_tcsp_kernel<false>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "gemm_tcsp: %s", cudaGetErrorString(err));
    }
    const dim3 grid((rows + kSpTileM - 1) / kSpTileM, (n + a.nt - 1) / a.nt);
    return launch("spb_sparse_ternary_gemm(tcgen05.sp)", kernel, grid, dim3(kSpThreads), smem, stream, a, tmap);
}

int gemm_tcsp_timeouts() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tcsp_timeouts, sizeof v) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return v;
}

}  // namespace spb
