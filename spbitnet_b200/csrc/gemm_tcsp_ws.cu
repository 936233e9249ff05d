// Batched sparse-ternary product on tcgen05.mma.sp, warp-specialised form (sm_100a).
//
//   Y[j, r] = sum_c W[r, c] * X[j, c]      W: rows x cols compressed 2:4 ternary, X: n x cols int8
//
// Operands: the sign bytes (+1 / -1) of a tile as the compressed A operand in shared memory (K-major, 128-byte
// swizzle), the index pairs as metadata in tensor memory (one byte per 8 columns, lane = weight row), the
// activation tiles by tensor-map bulk copies, int32 accumulators in tensor memory.  A first form in which one
// thread issued the copies and the MMAs between two block-wide barriers per step cost about 2450 cycles per
// step of which the re-encoding was 500 (the rest: that thread's serial chain with 255 threads parked).  Here
// the block has three roles that only meet at mbarriers:
//   warps 0-7 and 12-19      re-encode, as two groups of 256 threads that take alternate steps: wait for a
//                            free stage, write the A tile and the metadata of a step, arrive on the
//                            stage's "a_full" barrier;
//   warp 8     (one lane)    issues the MMAs: waits for a_full and b_full of a stage, issues four
//                            tcgen05.mma.sp, commits to the stage's "free" barrier;
//   warp 9     (one lane)    feeds the activations: waits for a free stage, expect_tx + two tensor-map
//                            bulk copies onto the stage's "b_full" barrier.
// So the re-encoding of step k + 1 runs under the MMAs of step k, and nobody waits at a block barrier
// inside the loop.  The epilogue (tcgen05.ld, stores) is done by the re-encoding warps after the last commit.
// Every wait is bounded; a role whose wait runs out records it and leaves its loop, the others then run
// out of their own bounds, the copy warp waits (bounded) for its copies in flight, tensor memory is freed
// and the block returns.
#include <cuda.h>

#include <cstring>

#include "spb_common.cuh"

namespace spb {

constexpr int kWsExpanders = 256;
// warps 0-7: re-encoding group 0 (even steps); 8: MMA; 9: copy; 10-11: idle (a warp may only touch the tensor-memory
// lanes 32 * (warp % 4) .. + 31, so the second group starts at a multiple of four); 12-19: re-encoding group 1 (odd steps)
constexpr int kWsGroup1Warp = 12;
constexpr int kWsThreads = 32 * (kWsGroup1Warp + 8);
constexpr int kWsTileM = 128;
constexpr int kWsStepK = 256;                  // logical columns per step: two units per row
constexpr int kWsABytes = kWsTileM * 128;      // compressed A tile: 128 rows x 128 bytes
constexpr int kWsMaxStages = 4;
constexpr int kWsSignLutBytes = 16 * 32 * 4;
constexpr long long kWsWaitCycles = 40000000;

struct WsArgs {
    const uint32_t* meta;
    const uint32_t* values;
    int32_t* Y;
    int rows, cols, n;
    int meta_stride, values_stride;
    int nt;         // batch rows per block: multiple of 16, at most 256
    int stages;     // ring depth (2..kWsMaxStages)
    int tmem_cols;  // power of two >= nt + 8 * stages
    int groups;     // re-encoding groups in use: 2 (alternate steps), or 1 (warps 12-19 idle)
    int mh;         // weight-row halves per block: 1 (128 rows), or 2 (256 rows: group g re-encodes rows 128 g .. of every
                    // step, both halves multiply the same activation tile into their own accumulator)
    GemmEpilogue ep;  // ep.out set: scaled half output instead of Y
    int* timeouts;        // counter of waits that ran out (pinned host memory, system-scope atomics), may be null
    long long wait_cycles;  // bound of every wait in the kernel
};

// 0 automatic, 1 / 2 force one / two weight-row halves per block (spb_set_gemm_row_halves; testing and measurement)
static int g_ws_mh = 0;

__device__ __forceinline__ void ws_count_timeout(int* counter) {
    if (counter) atomicAdd_system(counter, 1);
}

__device__ __forceinline__ uint32_t ws_smem(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// K-major, 128-byte swizzle: 8-row groups of 1024 B (SBO), 16-byte leading offset.
__device__ __forceinline__ uint64_t ws_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// kind::i8 instruction descriptor with the sparse flag: S32 accumulate, signed 8-bit A and B, K-major.
__device__ __forceinline__ uint32_t ws_idesc(int m, int n) {
    return (1u << 2) | (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}
// Bounded by time, not by polls (a poll may suspend for a while): kWsWaitCycles is about 20 ms at 2 GHz.
__device__ __forceinline__ bool ws_wait(uint32_t mbar, uint32_t parity, long long limit) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(mbar), "r"(parity)
            : "memory");
        if (done) return true;
        if (clock64() - t0 > limit) return false;
    }
}
__device__ __forceinline__ uint32_t ws_swz(int r, int c) {
    return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}
// Eight bitmaps (two of four bits set each) -> eight index pairs {low index | high index << 2}.
__device__ __forceinline__ uint32_t ws_index_pairs(uint32_t m) {
    const uint32_t mr = m >> 1, ml = m << 1;
    const uint32_t t1 = (0x11111111u & (~m & mr)) | (~0x11111111u & (mr | ~m));
    const uint32_t t2 = (0x22222222u & (~ml & ~m)) | (~0x22222222u & (m | ml));
    return (t1 & 0x55555555u) | (t2 & 0xAAAAAAAAu);
}

// HALF_OUT: the epilogue writes the scaled half output (a.ep) instead of the int32 sums
template <bool HALF_OUT>
__global__ void __launch_bounds__(kWsThreads, 1) gemm_tcsp_ws_kernel(const WsArgs a, const __grid_constant__ CUtensorMap tmap_x) {
    extern __shared__ uint8_t ws_raw[];
    // [sign table 2 KB][barriers + tmem slot 128 B] ... 1024-aligned: [stage: A 16 KB x mh | B0 nt*128 | B1 nt*128] x stages
    uint32_t* sgn = reinterpret_cast<uint32_t*>(ws_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ws_raw + kWsSignLutBytes);
    uint64_t* a_full = bars;                      // [stage]: 256 arrivals, the re-encoded tile and its metadata are written
    uint64_t* b_full = bars + kWsMaxStages;       // [stage]: the two activation tiles have landed
    uint64_t* free_b = bars + 2 * kWsMaxStages;   // [stage]: the MMAs that read the stage are done
    uint64_t* done_b = bars + 3 * kWsMaxStages;   // all MMAs of the block are done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ws_raw + kWsSignLutBytes + 112);
    const uint32_t raw_s = ws_smem(ws_raw);
    const uint32_t stage0_s = (raw_s + kWsSignLutBytes + 128 + 1023) & ~1023u;
    uint8_t* stage0 = ws_raw + (stage0_s - raw_s);
    const int b_bytes = a.nt * 128;  // one of the two activation sub-tiles
    const int a_bytes = a.mh * kWsABytes;
    const int stage_bytes = a_bytes + 2 * b_bytes;
    const int S = a.stages;

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
    const int row0 = blockIdx.x * kWsTileM * a.mh;
    const int n0 = blockIdx.y * a.nt;
    const int upr = a.cols >> 7;
    const int nsteps = (upr + 1) >> 1;

    grid_dep_launch();
    for (int i = tid; i < 16 * 32; i += kWsThreads) {  // byte b of an entry = -1 if bit b of the nibble is set, else +1
        const uint32_t t = ((static_cast<uint32_t>(i) >> 5) * 0x00204081u) & 0x01010101u;
        sgn[i] = (t * 0xFEu) | 0x01010101u;
    }
    if (tid == 0) {
        for (int s = 0; s < kWsMaxStages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ws_smem(a_full + s)), "r"(kWsExpanders * a.mh));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(ws_smem(b_full + s)));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(ws_smem(free_b + s)));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(ws_smem(done_b)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ws_smem(tmem_slot)),
                     "r"(static_cast<uint32_t>(a.tmem_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    const uint32_t tmem_e = tmem_d + static_cast<uint32_t>(a.nt * a.mh);  // metadata slots behind the accumulators
    bool ok = true;

    if (warp == 9) {
        // ---- copy warp: activation tiles of every step, as soon as their stage is free ----------------------
        if (lane == 0) {
            grid_dep_wait();  // X may be a predecessor's output
            int issued = 0;
            for (int kc = 0; kc < nsteps && ok; ++kc) {
                const int s = kc % S;
                if (kc >= S) ok = ws_wait(ws_smem(free_b + s), static_cast<uint32_t>(kc / S - 1) & 1u, a.wait_cycles);
                if (!ok) break;
                const uint32_t fb = ws_smem(b_full + s);
                uint8_t* sb = stage0 + static_cast<size_t>(s) * stage_bytes + a_bytes;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb),
                             "r"(static_cast<uint32_t>(2 * b_bytes))
                             : "memory");
#pragma unroll
                for (int h = 0; h < 2; ++h)  // columns [256 kc + 128 h, +128) of batch rows [n0, n0 + nt)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                            ws_smem(sb + h * b_bytes)),
                        "l"(reinterpret_cast<uint64_t>(&tmap_x)), "r"(kc * kWsStepK + 128 * h), "r"(n0), "r"(fb)
                        : "memory");
                issued = kc + 1;
            }
            // nothing of this block's copies may be in flight when it leaves: the last S issued steps
            for (int kc = max(0, issued - S); kc < issued; ++kc)
                if (!ws_wait(ws_smem(b_full + kc % S), static_cast<uint32_t>(kc / S) & 1u, a.wait_cycles)) ok = false;
            if (!ok) ws_count_timeout(a.timeouts);
        }
    } else if (warp == 8) {
        // ---- MMA warp: four tcgen05.mma.sp per step, as soon as both operands of the stage are there ----------
        if (lane == 0) {
            const uint32_t idesc = ws_idesc(kWsTileM, a.nt);
            for (int kc = 0; kc < nsteps; ++kc) {
                const int s = kc % S;
                const uint32_t par = static_cast<uint32_t>(kc / S) & 1u;
                ok = ws_wait(ws_smem(a_full + s), par, a.wait_cycles) && ws_wait(ws_smem(b_full + s), par, a.wait_cycles);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = stage0_s + static_cast<uint32_t>(s) * stage_bytes;
                const uint64_t db0 = ws_smem_desc(sa + a_bytes), db1 = ws_smem_desc(sa + a_bytes + b_bytes);
                for (int h = 0; h < a.mh; ++h) {  // each half of the weight rows into its own accumulator
                    const uint64_t da = ws_smem_desc(sa + static_cast<uint32_t>(h) * kWsABytes);
                    const uint32_t td = tmem_d + static_cast<uint32_t>(h * a.nt);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {  // 64 logical columns each: 32 B of A, 64 B of X, two metadata columns
                        const uint32_t acc = (kc > 0 || k > 0) ? 1u : 0u;
                        const uint64_t db = ((k & 2) ? db1 : db0) + static_cast<uint64_t>(4 * (k & 1));
                        const uint32_t te = tmem_e + static_cast<uint32_t>((s * a.mh + h) * 8 + 2 * k);
                        asm volatile(
                            "{\n\t.reg .pred p;\n\t"
                            "setp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.sp.cta_group::1.kind::i8 [%0], %1, %2, [%9], %3, {%5, %6, %7, %8}, p;\n\t}"
                            :
                            : "r"(td), "l"(da + 2 * k), "l"(db), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u),
                              "r"(te)
                            : "memory");
                    }
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ws_smem(free_b + s))
                             : "memory");
                if (kc == nsteps - 1)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ws_smem(done_b))
                                 : "memory");
            }
            if (!ok) ws_count_timeout(a.timeouts);
        }
    } else if (warp < 8 || (warp >= kWsGroup1Warp && a.groups == 2)) {
        // ---- re-encoding warps, two groups of eight that take alternate steps (a step's re-encoding is a chain of
        //      dependent loads, table reads and stores: two steps in flight hide its latency).  In a group, thread t
        //      and thread t + 128 share weight row (t & 127) of the tile; per step the first takes the even unit, the
        //      second the odd unit.  A warp's rows are the tensor-memory lanes it may access.
        const int grp = warp < 8 ? 0 : 1;
        const int ewarp = warp < 8 ? warp : warp - kWsGroup1Warp + 8;  // 0..15 over both groups
        const int etid = (ewarp & 7) * 32 + lane;                        // 0..255 within the group
        const int trow = etid & (kWsTileM - 1), thalf = etid >> 7;
        const int mhalf = a.mh == 2 ? grp : 0;  // which 128 rows of the block this group serves
        const int wrow = row0 + mhalf * kWsTileM + trow;
        const bool wvalid = wrow < a.rows;
        auto load_unit = [&](int step, uint4& mm, uint2& vv, bool& valid) {
            const int u = 2 * step + thalf;
            valid = wvalid && u < upr;
            if (valid) {
                mm = ld_stream_v4(a.meta + static_cast<size_t>(wrow) * a.meta_stride + u * 4);
                vv = ld_stream_v2(a.values + static_cast<size_t>(wrow) * a.values_stride + u * 2);
            }
        };
        // the weight words of four steps are in flight
        uint4 m0 = make_uint4(0, 0, 0, 0), m1 = m0, m2 = m0, m3 = m0;
        uint2 v0 = make_uint2(0, 0), v1 = v0, v2 = v0, v3 = v0;
        bool u0 = false, u1 = false, u2 = false, u3 = false;
        const int gs = a.mh == 2 ? 1 : a.groups;  // step stride of a group (with two row halves every group takes every step)
        const int k_first = a.mh == 2 ? 0 : grp;
        if (k_first < nsteps) load_unit(k_first, m0, v0, u0);
        if (k_first + gs < nsteps) load_unit(k_first + gs, m1, v1, u1);
        if (k_first + 2 * gs < nsteps) load_unit(k_first + 2 * gs, m2, v2, u2);
        if (k_first + 3 * gs < nsteps) load_unit(k_first + 3 * gs, m3, v3, u3);
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t sgn_s = raw_s + (static_cast<uint32_t>(lane) << 2);
        for (int kc = k_first; kc < nsteps; kc += gs) {
            const int s = kc % S;
            uint4 mn = make_uint4(0, 0, 0, 0);
            uint2 vn = make_uint2(0, 0);
            bool nvalid = false;
            if (kc + 4 * gs < nsteps) load_unit(kc + 4 * gs, mn, vn, nvalid);
            if (kc >= S) ok = ws_wait(ws_smem(free_b + s), static_cast<uint32_t>(kc / S - 1) & 1u, a.wait_cycles);
            ok = __all_sync(0xFFFFFFFFu, ok ? 1 : 0) != 0;  // tcgen05.st below is warp-wide
            if (!ok) break;
            // metadata: index pairs of this unit's 32 groups -> four tensor-memory columns of the row
            uint32_t e0 = 0x44444444u, e1 = 0x44444444u, e2 = 0x44444444u, e3 = 0x44444444u;
            if (u0) {
                e0 = ws_index_pairs(m0.x);
                e1 = ws_index_pairs(m0.y);
                e2 = ws_index_pairs(m0.z);
                e3 = ws_index_pairs(m0.w);
            }
            const uint32_t eaddr = tmem_e + lane_base + static_cast<uint32_t>((s * a.mh + mhalf) * 8 + thalf * 4);
            asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(eaddr), "r"(e0), "r"(e1), "r"(e2),
                         "r"(e3)
                         : "memory");
            // values: sign nibble -> four bytes of +1 / -1; a unit is four 16-byte chunks of the row
            const uint32_t sa = stage0_s + static_cast<uint32_t>(s) * stage_bytes + static_cast<uint32_t>(mhalf) * kWsABytes;
            const uint32_t vw[2] = {v0.x, v0.y};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int nibble = 4 * c + q, sh = 4 * (nibble & 7);
                    const uint32_t word = vw[nibble >> 3];
                    const uint32_t t = sh >= 7 ? (word >> (sh - 7)) : (word << (7 - sh));  // nibble at bits 7..10
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[q]) : "r"(sgn_s + (t & 0x780u)));
                    if (!u0) w[q] = 0u;
                }
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sa + ws_swz(trow, thalf * 4 + c)), "r"(w[0]),
                             "r"(w[1]), "r"(w[2]), "r"(w[3])
                             : "memory");
            }
            m0 = m1; v0 = v1; u0 = u1;
            m1 = m2; v1 = v2; u1 = u2;
            m2 = m3; v2 = v3; u2 = u3;
            m3 = mn; v3 = vn; u3 = nvalid;
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ws_smem(a_full + s)) : "memory");
        }
        // ---- epilogue: accumulators -> Y -------------------------------------------------------------
        if (ok) ok = ws_wait(ws_smem(done_b), 0, a.wait_cycles);
        ok = __all_sync(0xFFFFFFFFu, ok ? 1 : 0) != 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            grid_dep_wait();  // Y may still be read by a predecessor
            // warp w reads TMEM lanes 32 * (w % 4) .. + 31 (weight rows); the warps that serve the same rows share the
            // columns (all sixteen with one row half, the eight of a group with two)
            const int quarter = ewarp & 3;
            const int csel = a.mh == 2 ? ((ewarp >> 2) & 1) : (ewarp >> 2);
            const int cstep = a.mh == 2 ? 64 : 64 * a.groups;
            const int row = row0 + mhalf * kWsTileM + quarter * 32 + lane;
            for (int c0 = csel * 32; c0 < a.nt; c0 += cstep) {
                uint32_t r[32];
                const uint32_t taddr = tmem_d + lane_base + static_cast<uint32_t>(mhalf * a.nt + c0);
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
                        if (c0 + i < a.nt && j < a.n) {
                            const size_t o = static_cast<size_t>(j) * a.rows + row;
                            if (HALF_OUT)
                                a.ep.out[o] = __float2half_rn(__fmul_rn(static_cast<float>(static_cast<int32_t>(r[i])),
                                                                        dequant_scale(a.ep.gamma, a.ep.absmax[j])));
                            else
                                a.Y[o] = static_cast<int32_t>(r[i]);
                        }
                    }
                }
            }
        } else if (lane == 0) {
            ws_count_timeout(a.timeouts);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                     "r"(static_cast<uint32_t>(a.tmem_cols))
                     : "memory");
}

// One block that allocates tensor memory, waits with ws_wait on a barrier nobody arrives at, reports the run-out
// like the product kernel does, frees the tensor memory and returns.  No copy is in flight at any time.
__global__ void __launch_bounds__(128, 1) ws_wait_selftest_kernel(int* timeouts, long long limit) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(ws_smem(&bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ws_smem(&tmem_slot)), "r"(32u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
    if (threadIdx.x == 0 && !ws_wait(ws_smem(&bar), 0u, limit)) ws_count_timeout(timeouts);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32u) : "memory");
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeFn tensor_map_encoder() {
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
    return encode;
}

// Everything the launchers look up or allocate lazily on the host (driver entry point, the pinned timeout counter,
// the SM count), done now: an engine calls this at creation so that none of it first happens inside a stream
// capture, where allocations and look-ups are not allowed.
void prepare_host_state() {
    tensor_map_encoder();
    timeout_counter();
    sm_count();
}

// Launch of the warp-specialised form; the caller has checked the layout (cols % 128 == 0, aligned rows and X).
// Returns SPB_E_UNSUPPORTED when the tensor map of X cannot be made (the caller then takes the plain form).
int gemm_tcsp_ws_launch(const uint32_t* meta, const uint32_t* values, const int8_t* X, int32_t* Y, int rows, int cols,
                        int n, int meta_stride, int values_stride, void* stream, const GemmEpilogue* ep) {
    WsArgs a{};
    a.meta = meta; a.values = values; a.Y = Y;
    if (ep) a.ep = *ep;
    a.rows = rows; a.cols = cols; a.n = n;
    a.meta_stride = meta_stride; a.values_stride = values_stride;
    // batch rows per block: 256, or 128 / 64 when the wider tile would leave more than half of the SMs without a
    // block (a step costs about the same whatever the tile width, so more, narrower blocks finish sooner)
    const int mtiles = (rows + kWsTileM - 1) / kWsTileM;
    int nt = 256;
    while (nt > 64 && mtiles * ((n + nt - 1) / nt) < sm_count() / 2) nt >>= 1;
    a.nt = min(nt, (n + 15) / 16 * 16);
    // Two row halves per block (256 weight rows on one activation tile, one re-encoding group per half, two
    // accumulators).  A step then costs about twice as much (the MMA warp issues eight MMAs, each group re-encodes
    // every step), so it only pays by saving a wave.  Both accumulators and the metadata slots must fit the 512
    // tensor-memory columns: 240 batch rows.
    a.mh = 1;
    if (g_ws_mh != 1 && n > 128) {
        // automatic: only where the 128-row blocks need a second wave and the 256-row blocks fit into one
        // (measured: 6912x2560 at n = 1024, 25.2 -> 22.1 us; everywhere else the 128-row form is faster)
        const int mt2 = (rows + 2 * kWsTileM - 1) / (2 * kWsTileM), nt2 = 240;
        const int items1 = mtiles * ((n + a.nt - 1) / a.nt), items2 = mt2 * ((n + nt2 - 1) / nt2);
        if (g_ws_mh == 2 || (items1 > sm_count() && items2 <= sm_count() && items2 >= (3 * sm_count()) / 4)) {
            a.mh = 2;
            a.nt = min(nt2, (n + 15) / 16 * 16);
        }
    }
    const int stage_bytes = a.mh * kWsABytes + 2 * a.nt * 128;
    a.stages = max(2, min(kWsMaxStages, (200 * 1024) / stage_bytes));
    // two groups pay off except at 128 batch rows per block (measured at 6912x2560, n = 256: 12.4 against 11.9 us)
    a.groups = a.mh == 2 ? 2 : a.nt == 128 ? 1 : 2;
    // A group must not run more than one ring revolution ahead of the MMA warp, or its parity wait on a stage's
    // "free" barrier would be satisfied by the previous completion of the same parity.  A group's wait for step k
    // confirms the commit of step k - stages; its next step is k + groups, whose wait needs the commit of
    // k + groups - 2 * stages to be over: true when groups <= stages.  (Three groups on two stages were tried and
    // ran into exactly this.)
    a.groups = min(a.groups, a.stages);
    a.tmem_cols = 32;
    while (a.tmem_cols < a.mh * (a.nt + 8 * a.stages)) a.tmem_cols <<= 1;
    if (a.tmem_cols > 512) return fail(SPB_E_UNSUPPORTED, "gemm_tcsp_ws: %d tensor-memory columns", a.tmem_cols);
    const size_t smem = kWsSignLutBytes + 128 + 1024 + static_cast<size_t>(a.stages) * stage_bytes;
    const EncodeFn encode = tensor_map_encoder();
    if (!encode) return SPB_E_UNSUPPORTED;
    // tensor map of X: uint8 [n rows][cols], box 128 bytes x nt rows, 128-byte swizzle, zero fill past n
    alignas(64) CUtensorMap tmap;
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(n)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(cols)};
    const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(a.nt)};
    const cuuint32_t estr[2] = {1u, 1u};
    if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(X), gdim, gstride, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return SPB_E_UNSUPPORTED;
    void (*kernel)(WsArgs, CUtensorMap) = a.ep.out ? gemm_tcsp_ws_kernel<true> : gemm_tcsp_ws_kernel<false>;
    if (int rc = ensure_dynamic_smem("gemm_tcsp_ws", kernel, smem)) return rc;
    a.timeouts = timeout_counter();
    a.wait_cycles = kWsWaitCycles;
    const dim3 grid((rows + a.mh * kWsTileM - 1) / (a.mh * kWsTileM), (n + a.nt - 1) / a.nt);
    return launch("spb_sparse_ternary_gemm(tcgen05.sp, warp-specialised)", kernel, grid, dim3(kWsThreads), smem,
                  stream, a, tmap);
}

}  // namespace spb

extern "C" int spb_debug_bounded_wait_selftest(long long limit_cycles, void* stream) {
    using namespace spb;
    int* counter = timeout_counter();
    if (!counter) return fail(SPB_E_CUDA, "spb_debug_bounded_wait_selftest: no timeout counter");
    const long long limit = limit_cycles < 1000 ? 1000 : limit_cycles > kWsWaitCycles ? kWsWaitCycles : limit_cycles;
    const int before = timeouts_now();
    ws_wait_selftest_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(counter, limit);
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail(SPB_E_CUDA, "spb_debug_bounded_wait_selftest: %s", cudaGetErrorString(err));
    if (timeouts_now() != before)
        return fail(SPB_E_TIMEOUT, "spb_debug_bounded_wait_selftest: the wait ran out after %lld cycles, as it must", limit);
    return SPB_OK;
}

extern "C" int spb_set_gemm_row_halves(int halves) {
    const int old = spb::g_ws_mh;
    spb::g_ws_mh = halves == 1 || halves == 2 ? halves : 0;
    return old;
}
