// One decode token's layers as ONE persistent kernel (sm_100a): a block per SM, grid-wide barriers between the
// stages of a layer, every layer's weight slabs prefetched into shared memory several stages ahead.
//
// The chain-of-kernels step (engine.cu, enqueue_token) runs a layer as five dependent launches, each of which
// fetches its activation vector from L2, reduces it, multiplies and drains.  The work itself is small (13 MB of
// weights per layer at the 2B-4T shape, 2 us of HBM time).  Here the blocks stay resident for the whole token:
//
//   stage 1  x = quantise(rms_norm(residual + down))            q, k, v rows of this block; RoPE; K, V -> cache
//   stage 2  split-KV attention, (KV head, chunk of 16 or 32 positions) per block; the last block of a KV head merges
//   stage 3  x = quantise(attn)                                   o rows of this block
//   stage 4  x = quantise(rms_norm(residual + sub_norm(o)))       gate and up rows of this block
//   stage 5  x = quantise(sub_norm(relu(gate)^2 * up))            down rows of this block
//
// with a grid barrier after every stage (five per layer).  Every block forms the (short) activation vector of a
// stage itself, with the producers of the GEMV kernels (producers.cuh): same sums in the same order, same
// rounding points, so a token computed here equals the chain-of-kernels token bit for bit.  The matrix rows are
// dealt out as tiles of 16 rows (tile t of a stage goes to block t mod grid); a tile is multiplied by the
// warp-level sparse MMA exactly as in gemv_mmasp.cu (bitmaps -> index pairs, sign nibbles -> +-1 bytes, mma.sp
// m16n8k64), its K extent split over the warps of the block.
//
// Weight slabs never depend on activations, so they are copied four stages before their use: each of the four
// kinds of slab (q/k/v, o, gate/up, down) has its own shared-memory region, refilled for the next layer as soon
// as the stage that read it is over, by one bulk copy (cp.async.bulk) per row and stream that reports to the
// kind's mbarrier; the layer's norm weights travel with them when they fit, and the layer table (pointers,
// strides, scales) of this layer and the next is kept in shared memory too, because every global read after a
// barrier is a trip to L2 (about 0.8 us) on the block's critical path.
//
// The grid barrier is a counter in global memory: arrive = fence + atomic add; the block whose arrival completes
// the count publishes the target on a second word, which the others poll.  Every wait (grid barrier, slab
// mbarrier) is bounded in time; a block whose wait runs out marks the barrier state broken, bumps the library's
// timeout counter, waits (bounded) for its own copies in flight and returns; the other blocks run out of their
// own bounds.  The kernel is launched cooperatively (all blocks resident).
//
// Where the time goes (2B-4T shape, position ~150, one B200): a layer takes 43 us against 37 us for the chain of
// five kernels.  A stage is a chain of dependent round trips that the persistent form does not remove: barrier
// arrival (atomic) -> flag seen by the pollers -> activation vector from L2 -> two or three block-wide reductions ->
// rows -> stores, 6 - 9 us in all, of which the barrier itself is 1.5 - 3 us.  Hence an opt-in mode.
#include "decode_persistent.cuh"

#include <algorithm>

#include "attention_body.cuh"
#include "fused_ops.cuh"
#include "producers.cuh"

namespace spb {
namespace {

constexpr int kPdThreads = kProdThreads;  // the producers are written for this block size
constexpr int kPdWarps = kPdThreads / 32;
constexpr long long kPdWaitCycles = 2000000000LL;  // about a second
constexpr size_t kPdStaticSmem = 5 * 1024;            // the kernel's static shared memory, rounded up
constexpr int kPdTraceWords = 4096;                   // marks per traced block (spb_debug_set_decode_trace)
constexpr int kPdMarksPerLayer = 20;

// Shared-memory geometry, worked out on the host.
struct PdGeom {
    int mp_h, vp_h;  // row pitches (words) of the bitmap / sign rows of a slab with cols = H (q k v gate up)
    int mp_q, vp_q;  // cols = heads * head_dim (o)
    int mp_i, vp_i;  // cols = intermediate size (down)
    int t_qkv, t_o, t_gu, t_dn;  // tile slots per block and kind
    uint32_t off_sw, off_x, off_qkv, off_o, off_gu, off_dn, off_attn;  // byte offsets in dynamic shared memory
    uint32_t off_res;      // barrier-free form: the block's copy of the residual stream (H halves)
    uint32_t off_norm[4];  // the layer's norm weights (input_ln, post_attn_ln, attn_sub_norm, ffn_sub_norm), if staged
    int norms;             // 1: the norm weights travel with the slabs into shared memory; 0: read from global memory
    long long wait_cycles;
    int* timeouts;
    unsigned long long* trace;  // stage timing (spb_debug_set_decode_trace), or null
};

using PdProd = ProducerArgs;

// Producer operands of the barrier-free form: vectors that other blocks publish as tagged words (attention_body.cuh).
struct PdProdLl : ProducerArgs {
    const uint2* ll_x;   // tagged words behind x (attention output; gate and up)
    const uint2* ll_x2;  // tagged words behind x2 (the delta of a residual add)
    unsigned tag;
    long long limit;
    int* fail;
};
// x = the block's own copy of the residual stream (shared memory), x2 = delta as tagged words
struct LoadsResidualLl {
    static __device__ __forceinline__ uint4 x(const PdProdLl& a, int q) { return *(static_cast<const uint4*>(a.x) + q); }
    static __device__ __forceinline__ uint4 x2(const PdProdLl& a, int q) { return ll_read4(a.ll_x2 + 4 * q, a.tag, a.limit, a.fail); }
};
// x = a half vector as tagged words
struct LoadsVectorLl {
    static __device__ __forceinline__ uint4 x(const PdProdLl& a, int q) { return ll_read4(a.ll_x + 4 * q, a.tag, a.limit, a.fail); }
    static __device__ __forceinline__ uint4 x2(const PdProdLl& a, int q) { return x(a, q); }
};
// x = gate, x2 = up: word i holds gate[i] in its low and up[i] in its high half
struct LoadsGateUpLl {
    static __device__ __forceinline__ uint4 pick(const PdProdLl& a, int q, uint32_t sel) {
        const uint4 lo = ll_read4(a.ll_x + 8 * q, a.tag, a.limit, a.fail), hi = ll_read4(a.ll_x + 8 * q + 4, a.tag, a.limit, a.fail);
        return make_uint4(__byte_perm(lo.x, lo.y, sel), __byte_perm(lo.z, lo.w, sel), __byte_perm(hi.x, hi.y, sel),
                          __byte_perm(hi.z, hi.w, sel));
    }
    static __device__ __forceinline__ uint4 x(const PdProdLl& a, int q) { return pick(a, q, 0x5410u); }
    static __device__ __forceinline__ uint4 x2(const PdProdLl& a, int q) { return pick(a, q, 0x7632u); }
};

__device__ __forceinline__ uint32_t pd_smem(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint32_t pd_lds(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// eight bitmaps (two of four bits set each) -> eight index pairs {low index | high index << 2}
__device__ __forceinline__ uint32_t pd_index_pairs(uint32_t m) {
    const uint32_t mr = m >> 1, ml = m << 1;
    const uint32_t t1 = (0x11111111u & (~m & mr)) | (~0x11111111u & (mr | ~m));
    const uint32_t t2 = (0x22222222u & (~ml & ~m)) | (~0x22222222u & (m | ml));
    return (t1 & 0x55555555u) | (t2 & 0xAAAAAAAAu);
}
__device__ __forceinline__ unsigned pd_ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Words of the synchronisation array (PdModel::sync), each group on its own 128-byte line.
constexpr int kSyncCount = 0;    // arrivals at grid barriers, ever
constexpr int kSyncGen = 1;      // the count when the previous launch ended
constexpr int kSyncBroken = 2;   // a wait ran out: the counters no longer mean anything
constexpr int kSyncEpoch = 3;    // barrier-free form: launches so far (the tags of a launch's words derive from it)
constexpr int kSyncDone = 4;     // barrier-free form: blocks of the current launch that have finished
constexpr int kSyncFlag = 32;    // the last barrier every block has arrived at (its target count)
constexpr int kSyncKv = 64;      // per KV head: chunks of the current attention stage that are written

__device__ __forceinline__ unsigned pd_ld_relaxed(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Grid barrier number k of this launch (target = generation + k * blocks).  Arrivals are counted on one word;
// the block whose arrival completes the count publishes the target on another word, which is the one the others
// poll (with a pause between polls: a block that still works, like the one merging the attention chunks, shares
// the memory system with 147 pollers).  Returns false when the wait ran out (or ran out in an earlier barrier of
// this block).
__device__ __forceinline__ bool pd_barrier(unsigned* sync, unsigned target, long long limit, int* timeouts,
                                           int* s_abort) {
    __syncthreads();
    if (threadIdx.x == 0 && *s_abort == 0) {
        __threadfence();
        if (atomicAdd(sync + kSyncCount, 1u) + 1u == target) {
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(sync + kSyncFlag), "r"(target) : "memory");
        } else {
            const long long t0 = clock64();
            while (static_cast<int>(pd_ld_relaxed(sync + kSyncFlag) - target) < 0) {
                if (clock64() - t0 > limit) {
                    *s_abort = 1;
                    if (atomicExch(sync + kSyncBroken, 1u) == 0u && timeouts) atomicAdd_system(timeouts, 1);
                    break;
                }
                __nanosleep(40);
            }
        }
        __threadfence();
    }
    __syncthreads();
    return *s_abort == 0;
}

// One bulk copy (global -> shared, 16-byte aligned, a multiple of 16 bytes) that reports its bytes to `mbar`.
__device__ __forceinline__ void pd_bulk(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(mbar)
                 : "memory");
}
// Row r of a tile: its bitmap words (which = 0) or its sign words (which = 1) into the tile slot's padded rows.
__device__ __forceinline__ void pd_bulk_row(const PdLinear& L, int row, int r, int which, int cols, uint32_t ms_s, uint32_t vs_s,
                                            int mp, int vp, uint32_t mbar) {
    if (which == 0)
        pd_bulk(ms_s + static_cast<uint32_t>(r * mp) * 4u, L.meta + static_cast<size_t>(row) * L.ms, static_cast<uint32_t>(cols >> 3), mbar);
    else
        pd_bulk(vs_s + static_cast<uint32_t>(r * vp) * 4u, L.values + static_cast<size_t>(row) * L.vs, static_cast<uint32_t>(cols >> 4), mbar);
}
// Waits (bounded) for phase `parity` of a copy barrier.
__device__ __forceinline__ bool pd_wait(uint32_t mbar, uint32_t parity, long long limit) {
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

// The T (<= 8) tiles of a slab times the staged activation vector.  ks warps share a tile (contiguous ranges of
// 64-column steps), their partial sums meet in redi, and thread 16 * tile + r hands row r of tile `tile` to
// epi(active, tile, r, sum).  epi is called by every thread of the block (it may shuffle).
template <class Epi>
__device__ __forceinline__ void pd_tiles(uint32_t ms_s, int tcap, int T, int mp, int vp, int steps, uint32_t xs_s,
                                         uint32_t tab_s, int* redi, int tid, int lane, int warp, Epi epi) {
    const int ks_log2 = T <= 1 ? 3 : T == 2 ? 2 : T <= 4 ? 1 : 0;
    const int ks = 1 << ks_log2;
    const int tile = warp >> ks_log2, kq = warp & (ks - 1);
    const int spw = (steps + ks - 1) >> ks_log2;
    const int s_begin = tile < T ? min(steps, kq * spw) : 0, s_end = tile < T ? min(steps, s_begin + spw) : 0;
    const uint32_t vs_s = ms_s + static_cast<uint32_t>(16 * tcap * mp) * 4u;
    const int g = lane >> 2, tig = lane & 3;
    const uint32_t lane_or = static_cast<uint32_t>(lane) << 2;
    const uint32_t rot_lo = (static_cast<uint32_t>(tig) * 4u + 25u) & 31u, rot_hi = (static_cast<uint32_t>(tig) * 4u + 9u) & 31u;
    uint32_t me_p = ms_s + static_cast<uint32_t>((tile * 16 + g + 8 * (tig & 1)) * mp + (tig >> 1) + 2 * s_begin) * 4u;
    uint32_t v0_p = vs_s + static_cast<uint32_t>((tile * 16 + g) * vp + s_begin) * 4u;
    const uint32_t v_half = static_cast<uint32_t>(8 * vp) * 4u;
    uint32_t xq_p = xs_s + static_cast<uint32_t>(tig) * 16u + static_cast<uint32_t>(s_begin) * 64u;

    // two sets of accumulators on alternate steps: consecutive MMAs do not wait for one another
    int c0 = 0, c1 = 0, c2 = 0, c3 = 0, e0 = 0, e1 = 0, e2 = 0, e3 = 0;
    auto step = [&](int& c0, int& c1, int& c2, int& c3, uint32_t w0, uint32_t w1, uint32_t me_off, uint32_t x_off) {
        const uint32_t e = pd_index_pairs(pd_lds(me_p + me_off));
        const uint32_t a0 = pd_lds(tab_s + ((__funnelshift_r(w0, w0, rot_lo) & 0x780u) | lane_or));
        const uint32_t a1 = pd_lds(tab_s + ((__funnelshift_r(w1, w1, rot_lo) & 0x780u) | lane_or));
        const uint32_t a2 = pd_lds(tab_s + ((__funnelshift_r(w0, w0, rot_hi) & 0x780u) | lane_or));
        const uint32_t a3 = pd_lds(tab_s + ((__funnelshift_r(w1, w1, rot_hi) & 0x780u) | lane_or));
        uint32_t b0, b1, b2, b3;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(xq_p + x_off));
        asm volatile(
            "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
            "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
            : "+r"(c0), "+r"(c1), "+r"(c2), "+r"(c3)
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(b2), "r"(b3), "r"(e));
    };
    auto advance = [&](uint32_t n) {
        me_p += 8u * n;
        v0_p += 4u * n;
        xq_p += 64u * n;
    };
    int st = s_begin;
    for (; st < s_end && (st & 3) != 0; ++st) {  // up to the next multiple of four steps
        step(c0, c1, c2, c3, pd_lds(v0_p), pd_lds(v0_p + v_half), 0u, 0u);
        advance(1u);
    }
    for (; st + 4 <= s_end; st += 4) {  // four steps share one 16-byte read of each row's sign words
        uint4 w0, w1;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w0.x), "=r"(w0.y), "=r"(w0.z), "=r"(w0.w) : "r"(v0_p));
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w1.x), "=r"(w1.y), "=r"(w1.z), "=r"(w1.w) : "r"(v0_p + v_half));
        step(c0, c1, c2, c3, w0.x, w1.x, 0u, 0u);
        step(e0, e1, e2, e3, w0.y, w1.y, 8u, 64u);
        step(c0, c1, c2, c3, w0.z, w1.z, 16u, 128u);
        step(e0, e1, e2, e3, w0.w, w1.w, 24u, 192u);
        advance(4u);
    }
    for (; st < s_end; ++st) {
        step(c0, c1, c2, c3, pd_lds(v0_p), pd_lds(v0_p + v_half), 0u, 0u);
        advance(1u);
    }
    if (tig == 0) {  // column 0 of the tile: rows g (c0) and g + 8 (c2)
        redi[warp * 16 + g] = c0 + e0;
        redi[warp * 16 + g + 8] = c2 + e2;
    }
    __syncthreads();
    const bool active = tid < 16 * T;
    int acc = 0;
    if (active) {
        const int tl = tid >> 4, r = tid & 15;
        for (int k = 0; k < ks; ++k) acc += redi[((tl << ks_log2) + k) * 16 + r];
    }
    epi(active, tid >> 4, tid & 15, acc);
}

template <int G, bool LL>
__global__ void __launch_bounds__(kPdThreads, 1) decode_persistent_kernel(const PdModel m, const PdGeom geo) {
    __shared__ __align__(16) uint32_t sgn_tab[16 * 32];  // entry (nibble n, lane l) at word n * 32 + l
    __shared__ int redi[kPdWarps * 16];
    __shared__ float redf[64];
    __shared__ int s_flag[2];  // [0] a barrier wait of this block ran out, [1] this block merges the chunks of a KV head
    __shared__ float2 rope_cs[128];  // cos, sin of this token's position for every pair of a head
    __shared__ __align__(16) PdLayer s_layer[2];  // the tables of this layer and the next (a global read after a barrier is a trip to L2)
    __shared__ __align__(8) uint64_t copy_bar[4];  // q/k/v, o, gate/up, down: the slab of that kind (and the norm weights beside it) has landed
    extern __shared__ __align__(128) uint8_t pd_raw[];

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);  // through a shuffle: known to be uniform over the warp
    const int nb = static_cast<int>(gridDim.x), b = static_cast<int>(blockIdx.x);
    const uint32_t raw_s = pd_smem(pd_raw), tab_s = pd_smem(sgn_tab);
    const volatile unsigned* vsync = m.sync;
    if (vsync[kSyncBroken] != 0u) return;  // an earlier launch gave up at a barrier: the counters no longer mean anything
    const unsigned bar_base = vsync[kSyncGen];
    unsigned bar_n = 0;  // barriers passed so far
    // barrier-free form: the words of layer l of this launch carry tag_base + l (never 0, which is what the buffer
    // is cleared to); the regions of the stage outputs follow one another in m.ll
    const unsigned tag_base = LL ? vsync[kSyncEpoch] * static_cast<unsigned>(m.nlayers + 1) + 1u : 0u;

    if (tid < 2) s_flag[tid] = 0;
    if (tid == 0) {
        for (int i = 0; i < 4; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pd_smem(copy_bar + i)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {  // byte b of an entry = -1 if bit b of the nibble is set, else +1
        const uint32_t i = tid + j * kPdThreads;
        const uint32_t t = ((i >> 5) * 0x00204081u) & 0x01010101u;
        sgn_tab[i] = (t * 0xFEu) | 0x01010101u;
    }

    constexpr int kLayerWords = static_cast<int>(sizeof(PdLayer) / 4);
    static_assert(sizeof(PdLayer) % 4 == 0 && 2 * kLayerWords <= kPdThreads, "layer table copy");
    if (tid < 2 * kLayerWords && tid / kLayerWords < m.nlayers)
        reinterpret_cast<uint32_t*>(s_layer)[tid] = __ldg(reinterpret_cast<const uint32_t*>(m.layers) + tid);
    const int pos = *m.d_pos;
    if (tid < (m.hd >> 1)) {
        float c, s;
        rope_angle(pos, tid, m.hd, m.theta, c, s);
        rope_cs[tid] = make_float2(c, s);
    }
    const int token = (m.d_prompt && pos < m.n_prompt) ? m.d_prompt[pos] : *m.d_next;
    const int qdim = m.nh * m.hd, kvdim = m.nkv * m.hd;
    const int nt_q = qdim >> 4, nt_kv = kvdim >> 4, nt_qkv = nt_q + 2 * nt_kv, nt_h = m.H >> 4, np_gu = m.inter >> 4;
    auto mine = [&](int n) { return b < n ? (n - b + nb - 1) / nb : 0; };
    const int T_qkv = mine(nt_qkv), T_h = mine(nt_h), T_gu = 2 * mine(np_gu);

    uint4* xs_sw = reinterpret_cast<uint4*>(pd_raw + geo.off_sw);
    const uint32_t xs_s = raw_s + geo.off_x;
    const uint32_t qkv_s = raw_s + geo.off_qkv, o_s = raw_s + geo.off_o, gu_s = raw_s + geo.off_gu, dn_s = raw_s + geo.off_dn;
    uint8_t* attn_sm = pd_raw + geo.off_attn;
    __half* res_sm = reinterpret_cast<__half*>(pd_raw + geo.off_res);
    uint2* const ll_q = m.ll;
    uint2* const ll_k = ll_q + (qdim >> 1);
    uint2* const ll_v = ll_k + (kvdim >> 1);
    uint2* const ll_a = ll_v + (kvdim >> 1);
    uint2* const ll_o = ll_a + (qdim >> 1);
    uint2* const ll_gu = ll_o + (m.H >> 1);
    uint2* const ll_d = ll_gu + m.inter;

    // ---- slab copies -------------------------------------------------------------------------------------------
    // One bulk copy per row and stream (bitmaps, signs), spread over the threads; thread 0 announces the byte count.
    // A region is only rewritten after the stage that read it (a grid barrier lies between): the proxy fence orders
    // those generic reads before the asynchronous writes.
    const uint32_t bar_s = pd_smem(copy_bar);
    auto announce = [&](int kind, uint32_t bytes) {
        if (tid == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_s + 8u * kind), "r"(bytes) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    };
    auto norm_bytes = [&](const float* src, int n) { return (geo.norms && src) ? static_cast<uint32_t>(n) * 4u : 0u; };
    auto issue_norm = [&](const float* src, int i, int n, int kind, int who) {  // n floats of norm weights beside a slab
        if (geo.norms && src && tid == who) pd_bulk(raw_s + geo.off_norm[i], src, static_cast<uint32_t>(n) * 4u, bar_s + 8u * kind);
    };
    auto norm_ptr = [&](const float* global, int i) -> const float* {
        return (global && geo.norms) ? reinterpret_cast<const float*>(pd_raw + geo.off_norm[i]) : global;
    };
    auto issue_qkv = [&](int l) {
        if (l >= m.nlayers || T_qkv == 0) return;
        const PdLayer& Ly = s_layer[l & 1];
        const uint32_t vs_s = qkv_s + static_cast<uint32_t>(16 * geo.t_qkv * geo.mp_h) * 4u;
        announce(0, static_cast<uint32_t>(T_qkv) * 16u * static_cast<uint32_t>((m.H >> 3) + (m.H >> 4)) + norm_bytes(Ly.norm[0], m.H));
        for (int i = tid; i < T_qkv * 32; i += kPdThreads) {
            const int k = i >> 5, r = (i >> 1) & 15, t = b + k * nb;
            const int mi = t < nt_q ? 0 : t < nt_q + nt_kv ? 1 : 2;
            const int row0 = 16 * (t - (mi == 0 ? 0 : mi == 1 ? nt_q : nt_q + nt_kv));
            pd_bulk_row(Ly.lin[mi], row0 + r, r, i & 1, m.H, qkv_s + static_cast<uint32_t>(k * 16 * geo.mp_h) * 4u,
                        vs_s + static_cast<uint32_t>(k * 16 * geo.vp_h) * 4u, geo.mp_h, geo.vp_h, bar_s);
        }
        issue_norm(Ly.norm[0], 0, m.H, 0, kPdThreads - 1);
    };
    auto issue_rows = [&](int l, int which, int cols, uint32_t slab_s, int tcap, int mp, int vp) {  // o (kind 1) or down (kind 3)
        if (l >= m.nlayers || T_h == 0) return;
        const PdLayer& Ly = s_layer[l & 1];
        const int kind = which == 3 ? 1 : 3;
        const uint32_t vs_s = slab_s + static_cast<uint32_t>(16 * tcap * mp) * 4u;
        announce(kind, static_cast<uint32_t>(T_h) * 16u * static_cast<uint32_t>((cols >> 3) + (cols >> 4)) +
                           (which == 6 ? norm_bytes(Ly.norm[3], m.inter) : 0u));
        for (int i = tid; i < T_h * 32; i += kPdThreads) {
            const int k = i >> 5, r = (i >> 1) & 15;
            pd_bulk_row(Ly.lin[which], 16 * (b + k * nb) + r, r, i & 1, cols, slab_s + static_cast<uint32_t>(k * 16 * mp) * 4u,
                        vs_s + static_cast<uint32_t>(k * 16 * vp) * 4u, mp, vp, bar_s + 8u * kind);
        }
        if (which == 6) issue_norm(Ly.norm[3], 3, m.inter, 3, kPdThreads - 1);
    };
    auto issue_gu = [&](int l) {  // tile pair p: gate rows 16 p.. in slot 2 k, up rows 16 p.. in slot 2 k + 1
        if (l >= m.nlayers || T_gu == 0) return;
        const PdLayer& Ly = s_layer[l & 1];
        const uint32_t vs_s = gu_s + static_cast<uint32_t>(16 * geo.t_gu * geo.mp_h) * 4u;
        announce(2, static_cast<uint32_t>(T_gu) * 16u * static_cast<uint32_t>((m.H >> 3) + (m.H >> 4)) + norm_bytes(Ly.norm[1], m.H) +
                        norm_bytes(Ly.norm[2], m.H));
        for (int i = tid; i < T_gu * 32; i += kPdThreads) {
            const int k = i >> 5, r = (i >> 1) & 15;  // slot k: pair k / 2, gate (even) or up (odd)
            pd_bulk_row(Ly.lin[4 + (k & 1)], 16 * (b + (k >> 1) * nb) + r, r, i & 1, m.H, gu_s + static_cast<uint32_t>(k * 16 * geo.mp_h) * 4u,
                        vs_s + static_cast<uint32_t>(k * 16 * geo.vp_h) * 4u, geo.mp_h, geo.vp_h, bar_s + 16u);
        }
        issue_norm(Ly.norm[1], 1, m.H, 2, kPdThreads - 1);
        issue_norm(Ly.norm[2], 2, m.H, 2, kPdThreads - 2);
    };
    // The slab of `kind` for layer l has landed (bounded wait; false when it ran out for any thread of the block).
    auto slab_ready = [&](int kind, int l) {
        const bool ok = pd_wait(bar_s + 8u * kind, static_cast<uint32_t>(l) & 1u, geo.wait_cycles);
        if (!__syncthreads_and(ok ? 1 : 0)) {
            if (tid == 0) {
                s_flag[0] = 1;
                if (atomicExch(m.sync + kSyncBroken, 1u) == 0u && geo.timeouts) atomicAdd_system(geo.timeouts, 1);
            }
            return false;
        }
        return true;
    };
    // Before the block returns early: nothing of its copies may still be in flight (bounded).  Kind k was last issued
    // for layer `upto[k]`.
    int issued[4] = {-1, -1, -1, -1}, consumed[4] = {-1, -1, -1, -1};
    auto leave = [&]() {
        const int tiles[4] = {T_qkv, T_h, T_gu, T_h};
        for (int k = 0; k < 4; ++k)
            for (int l = consumed[k] + 1; l <= issued[k] && tiles[k] > 0; ++l)
                pd_wait(bar_s + 8u * k, static_cast<uint32_t>(l) & 1u, geo.wait_cycles);
    };
    // The activation vector of a stage: produced (swizzled int8, as the SIMT kernel wants it), then re-ordered for
    // the B registers: xs[step][tig][j][0..3] = x[64 step + 16 j + 4 tig ..+3].
    auto reorder_x = [&](int cols) {
        __syncthreads();
        for (int q = tid; q < (cols >> 4); q += kPdThreads) {
            const int c = q >> 3, i = q & 7;
            const uint4 xv = xs_sw[(c << 3) + (i ^ (c & 7))];
            const uint32_t d = xs_s + (static_cast<uint32_t>(q) >> 2) * 64u + (static_cast<uint32_t>(q) & 3u) * 4u;
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(d), "r"(xv.x) : "memory");
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 16u), "r"(xv.y) : "memory");
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 32u), "r"(xv.z) : "memory");
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(d + 48u), "r"(xv.w) : "memory");
        }
    };
    // Stage timing for spb_debug_set_decode_trace: thread 0 of the first and of the last block write the global
    // nanosecond timer at up to kPdMarksPerLayer points of every layer, in this order:
    //   stage 1: slab and norm weights there, x produced, tiles done, barrier passed        (0 .. 3)
    //   stage 2: next q/k/v slab issued, chunks (and merge) done, barrier passed            (4 .. 6)
    //   stages 3, 4, 5: as stage 1                                                          (7 .. 10, 11 .. 14, 15 .. 18)
    int layer_now = 0;
    auto mark = [&](int k) {
        const int i = layer_now * kPdMarksPerLayer + k;
        if (geo.trace && (b == 0 || b == nb - 1) && tid == 0 && i < kPdTraceWords) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            geo.trace[(b ? kPdTraceWords : 0) + i] = t;
        }
    };
    // Between two stages: the grid barrier, or (barrier-free form) a block barrier that also collects a poll that
    // ran out somewhere in the block.
    auto barrier = [&]() {
        if (LL) {
            if (__syncthreads_or(s_flag[0])) {
                if (tid == 0 && atomicExch(m.sync + kSyncBroken, 1u) == 0u && geo.timeouts) atomicAdd_system(geo.timeouts, 1);
                return false;
            }
            return true;
        }
        ++bar_n;
        return pd_barrier(m.sync, bar_base + bar_n * static_cast<unsigned>(nb), geo.wait_cycles, geo.timeouts, &s_flag[0]);
    };
    // two halves that neighbouring lanes hold -> one tagged word, stored by the even lane
    auto ll_pair = [&](uint2* dst, int index, __half mine, bool writer, unsigned tag) {
        const uint32_t lo = __half_as_ushort(mine);
        const uint32_t hi = __shfl_down_sync(0xFFFFFFFFu, lo, 1);
        if (writer) ll_write(dst + (index >> 1), lo | (hi << 16), tag);
    };

    if (LL)  // every block keeps its own copy of the residual stream; it starts as the token's embedding row
        for (int q = tid; q < (m.H >> 3); q += kPdThreads)
            reinterpret_cast<uint4*>(res_sm)[q] = __ldg(reinterpret_cast<const uint4*>(m.embed + static_cast<size_t>(token) * m.H) + q);
    __syncthreads();  // the table, the flags, the copy barriers
    issue_qkv(0);
    issue_rows(0, 3, qdim, o_s, geo.t_o, geo.mp_q, geo.vp_q);
    issue_gu(0);
    issued[0] = issued[1] = issued[2] = 0;

    const int seq_len = pos + 1;
    const int nsplit = attn_nsplit(seq_len);
    const int nsplit_max = attn_nsplit_max(m.max_seq);

    uint32_t next_word = 0;  // a word of layer l + 2's table, on its way to shared memory
    for (int l = 0; l < m.nlayers; ++l) {
        if (l >= 1 && l + 1 < m.nlayers && tid < kLayerWords) reinterpret_cast<uint32_t*>(&s_layer[(l + 1) & 1])[tid] = next_word;
        const PdLayer& Ly = s_layer[l & 1];
        layer_now = l;
        // ---- stage 1: residual + input norm -> q k v, RoPE, cache --------------------------------------------
        issue_rows(l, 6, m.inter, dn_s, geo.t_dn, geo.mp_i, geo.vp_i);
        issued[3] = l;
        const unsigned tag = tag_base + static_cast<unsigned>(l);
        if (T_qkv > 0) {
            PdProdLl pa{};
            pa.x = l == 0 ? static_cast<const void*>(m.embed + static_cast<size_t>(token) * m.H) : static_cast<const void*>(m.xa);
            pa.x2 = l == 0 ? nullptr : m.down;
            pa.w_sub = nullptr;
            pa.w_norm = norm_ptr(Ly.norm[0], 0);
            pa.x_out = m.xb;
            pa.eps = m.eps;
            pa.cols = m.H;
            if (LL) {  // residual: the block's copy, updated in place; delta: the previous layer's down projection
                pa.x = res_sm;
                pa.x_out = res_sm;
                pa.ll_x2 = ll_d;
                pa.tag = tag - 1u;
                pa.limit = geo.wait_cycles;
                pa.fail = &s_flag[0];
            }
            if (!slab_ready(0, l)) return leave();
            consumed[0] = l;
            mark(0);
            const float absmax = LL ? produce_x<IN_RESNORM, OUT_F16, PdProdLl, LoadsResidualLl>(pa, xs_sw, static_cast<__half*>(nullptr), redf, true)
                                    : produce_x<IN_RESNORM, OUT_F16>(pa, xs_sw, static_cast<__half*>(nullptr), redf, b == 0);
            reorder_x(m.H);
            __syncthreads();
            mark(1);
            const float dq_q = dequant_scale(Ly.lin[0].gamma, absmax), dq_k = dequant_scale(Ly.lin[1].gamma, absmax);
            const float dq_v = dequant_scale(Ly.lin[2].gamma, absmax);
            pd_tiles(qkv_s, geo.t_qkv, T_qkv, geo.mp_h, geo.vp_h, m.H >> 6, xs_s, tab_s, redi, tid, lane, warp,
                     [&](bool active, int tl, int r, int acc) {
                         const int t = b + tl * nb;  // the tile's number among the q, k, v tiles
                         const int mi = t < nt_q ? 0 : t < nt_q + nt_kv ? 1 : 2;
                         const int row = 16 * (t - (mi == 0 ? 0 : mi == 1 ? nt_q : nt_q + nt_kv)) + r;
                         const float dq = mi == 0 ? dq_q : mi == 1 ? dq_k : dq_v;
                         const __half hv = __float2half_rn(__fmul_rn(static_cast<float>(acc), dq));
                         const float v = __half2float(hv);
                         const float p = __shfl_xor_sync(0xFFFFFFFFu, v, 1);  // the other element of the RoPE pair
                         const int head = row / m.hd, d = row - head * m.hd;
                         __half y = hv;
                         if (mi != 2) {
                             __half y0, y1;
                             const float2 cs = rope_cs[(d >> 1) & 127];
                             rope_apply((r & 1) ? p : v, (r & 1) ? v : p, cs.x, cs.y, y0, y1);
                             y = (r & 1) ? y1 : y0;
                         }
                         if (LL) ll_pair(mi == 0 ? ll_q : mi == 1 ? ll_k : ll_v, row, y, active && (r & 1) == 0, tag);
                         if (!active) return;
                         if (mi == 0) {
                             if (!LL) m.q[row] = y;
                         } else {
                             (mi == 1 ? Ly.kc : Ly.vc)[(static_cast<size_t>(head) * m.max_seq + pos) * m.hd + d] = y;
                         }
                     });
        }
        mark(2);
        if (!barrier()) return leave();
        mark(3);

        // ---- stage 2: attention ------------------------------------------------------------------------------
        issue_qkv(l + 1);
        if (l + 1 < m.nlayers) issued[0] = l + 1;
        mark(4);
        for (int item = b; item < m.nkv * nsplit; item += nb) {
            const int kvh = item / nsplit, split = item - kvh * nsplit;
            const LlSource lls{ll_q, ll_k, ll_v, tag, pos, geo.wait_cycles, &s_flag[0]};
            attn_chunk_block<G>(m.q, Ly.kc, Ly.vc, m.scratch, kvh, split, m.hd, m.max_seq, nsplit_max, m.attn_scale, seq_len,
                                attn_sm, LL ? &lls : nullptr);
            __syncthreads();
            if (tid == 0) {
                __threadfence();  // cumulative: the block's partial results, then the count
                const unsigned old = atomicAdd(m.sync + kSyncKv + kvh, 1u);
                const int last = old + 1u == static_cast<unsigned>(nsplit);
                if (last) atomicExch(m.sync + kSyncKv + kvh, 0u);
                __threadfence();
                s_flag[1] = last;
            }
            __syncthreads();
            if (s_flag[1]) {  // every chunk of this KV head is written: merge them for its G query heads
                LlFan fan{};
                fan.dst[0] = ll_a;
                fan.ndst = 1;
                attn_merge_group<G>(m.scratch, m.attn, kvh, m.hd, nsplit_max, nsplit, reinterpret_cast<float*>(attn_sm),
                                    LL ? &fan : nullptr, tag);
            }
            __syncthreads();
        }
        mark(5);
        if (!barrier()) return leave();
        mark(6);

        // ---- stage 3: o projection ---------------------------------------------------------------------------
        if (T_h > 0) {
            PdProdLl pa{};
            pa.x = m.attn;
            pa.cols = qdim;
            pa.ll_x = ll_a;
            pa.tag = tag;
            pa.limit = geo.wait_cycles;
            pa.fail = &s_flag[0];
            if (!slab_ready(1, l)) return leave();
            consumed[1] = l;
            mark(7);
            const float absmax = LL ? produce_x<IN_F16_AMAX, OUT_F16, PdProdLl, LoadsVectorLl>(pa, xs_sw, static_cast<__half*>(nullptr), redf, true)
                                    : produce_x<IN_F16_AMAX, OUT_F16>(pa, xs_sw, static_cast<__half*>(nullptr), redf, b == 0);
            reorder_x(qdim);
            __syncthreads();
            mark(8);
            const float dq = dequant_scale(Ly.lin[3].gamma, absmax);
            pd_tiles(o_s, geo.t_o, T_h, geo.mp_q, geo.vp_q, qdim >> 6, xs_s, tab_s, redi, tid, lane, warp,
                     [&](bool active, int tl, int r, int acc) {
                         const int row = 16 * (b + tl * nb) + r;
                         const __half hv = __float2half_rn(__fmul_rn(static_cast<float>(acc), dq));
                         if (LL) ll_pair(ll_o, row, hv, active && (r & 1) == 0, tag);
                         else if (active) m.o[row] = hv;
                     });
        }
        mark(9);
        if (!barrier()) return leave();
        mark(10);

        // ---- stage 4: sub-norm(o) + residual + post-attention norm -> gate, up --------------------------------
        issue_rows(l + 1, 3, qdim, o_s, geo.t_o, geo.mp_q, geo.vp_q);
        if (l + 1 < m.nlayers) issued[1] = l + 1;
        if (T_gu > 0) {
            PdProdLl pa{};
            pa.x = m.xb;
            pa.x2 = m.o;
            pa.w_sub = norm_ptr(Ly.norm[2], 2);
            pa.w_norm = norm_ptr(Ly.norm[1], 1);
            pa.x_out = m.xa;
            pa.eps = m.eps;
            pa.cols = m.H;
            if (LL) {
                pa.x = res_sm;
                pa.x_out = res_sm;
                pa.ll_x2 = ll_o;
                pa.tag = tag;
                pa.limit = geo.wait_cycles;
                pa.fail = &s_flag[0];
            }
            if (!slab_ready(2, l)) return leave();
            consumed[2] = l;
            mark(11);
            const float absmax = LL ? produce_x<IN_RESNORM, OUT_F16, PdProdLl, LoadsResidualLl>(pa, xs_sw, static_cast<__half*>(nullptr), redf, true)
                                    : produce_x<IN_RESNORM, OUT_F16>(pa, xs_sw, static_cast<__half*>(nullptr), redf, b == 0);
            reorder_x(m.H);
            __syncthreads();
            mark(12);
            const float dq_g = dequant_scale(Ly.lin[4].gamma, absmax), dq_u = dequant_scale(Ly.lin[5].gamma, absmax);
            pd_tiles(gu_s, geo.t_gu, T_gu, geo.mp_h, geo.vp_h, m.H >> 6, xs_s, tab_s, redi, tid, lane, warp,
                     [&](bool active, int tl, int r, int acc) {
                         const int row = 16 * (b + (tl >> 1) * nb) + r;
                         const __half hv = __float2half_rn(__fmul_rn(static_cast<float>(acc), (tl & 1) ? dq_u : dq_g));
                         if (LL) {  // a gate row's thread and its up row's thread are 16 lanes apart: one word for both
                             const uint32_t lo = __half_as_ushort(hv);
                             const uint32_t hi = __shfl_down_sync(0xFFFFFFFFu, lo, 16);
                             if (active && !(tl & 1)) ll_write(ll_gu + row, lo | (hi << 16), tag);
                             return;
                         }
                         if (!active) return;
                         if (tl & 1) m.up[row] = hv;
                         else m.gate[row] = hv;
                     });
        }
        mark(13);
        if (!barrier()) return leave();
        mark(14);

        // ---- stage 5: relu(gate)^2 * up, sub-norm -> down -----------------------------------------------------
        if (l + 2 < m.nlayers && tid < kLayerWords)
            next_word = __ldg(reinterpret_cast<const uint32_t*>(m.layers + l + 2) + tid);
        issue_gu(l + 1);
        if (l + 1 < m.nlayers) issued[2] = l + 1;
        if (T_h > 0) {
            PdProdLl pa{};
            pa.x = m.gate;
            pa.x2 = m.up;
            pa.w_sub = norm_ptr(Ly.norm[3], 3);
            pa.eps = m.eps;
            pa.cols = m.inter;
            pa.ll_x = ll_gu;
            pa.tag = tag;
            pa.limit = geo.wait_cycles;
            pa.fail = &s_flag[0];
            if (!slab_ready(3, l)) return leave();
            consumed[3] = l;
            mark(15);
            const float absmax = LL ? produce_x<IN_RELU2, OUT_F16, PdProdLl, LoadsGateUpLl>(pa, xs_sw, static_cast<__half*>(nullptr), redf, true)
                                    : produce_x<IN_RELU2, OUT_F16>(pa, xs_sw, static_cast<__half*>(nullptr), redf, b == 0);
            reorder_x(m.inter);
            __syncthreads();
            mark(16);
            const float dq = dequant_scale(Ly.lin[6].gamma, absmax);
            pd_tiles(dn_s, geo.t_dn, T_h, geo.mp_i, geo.vp_i, m.inter >> 6, xs_s, tab_s, redi, tid, lane, warp,
                     [&](bool active, int tl, int r, int acc) {
                         const int row = 16 * (b + tl * nb) + r;
                         const __half hv = __float2half_rn(__fmul_rn(static_cast<float>(acc), dq));
                         if (LL) ll_pair(ll_d, row, hv, active && (r & 1) == 0, tag);
                         if (active && (!LL || l + 1 == m.nlayers)) m.down[row] = hv;  // the last layer's goes to the kernels that follow
                     });
        }
        mark(17);
        if (l + 1 < m.nlayers && !barrier()) return leave();
        mark(18);
    }
    if (LL) {
        // the residual stream goes back to global memory for the kernels that follow; the last block to finish
        // opens the next launch's range of tags
        if (b == 0)
            for (int q = tid; q < (m.H >> 3); q += kPdThreads) reinterpret_cast<uint4*>(m.xa)[q] = reinterpret_cast<const uint4*>(res_sm)[q];
        __syncthreads();
        if (tid == 0 && atomicAdd(m.sync + kSyncDone, 1u) + 1u == static_cast<unsigned>(nb)) {
            atomicExch(m.sync + kSyncDone, 0u);
            atomicAdd(m.sync + kSyncEpoch, 1u);
        }
        return;
    }
    // Arrive only: the kernel boundary orders the rest.  The last block to arrive publishes the count as the
    // next launch's generation.
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        ++bar_n;
        const unsigned old = atomicAdd(m.sync + kSyncCount, 1u);
        if (old + 1u == bar_base + bar_n * static_cast<unsigned>(nb)) atomicExch(m.sync + kSyncGen, old + 1u);
    }
}

// Two blocks at a barrier that expects three: both waits run out, the state is marked broken, the timeout is
// counted once, both blocks return.
__global__ void __launch_bounds__(32) pd_barrier_selftest_kernel(unsigned* sync, long long limit, int* timeouts) {
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = 0;
    pd_barrier(sync, 3u, limit, timeouts, &s_abort);
}

int pitch_words(int words) { return words % 8 == 4 ? words : words + ((4 - words % 8) + 8) % 8; }

// Fills the geometry for `blocks` blocks; returns the dynamic shared memory it needs.
size_t make_geom(const PdModel& m, int blocks, PdGeom& g) {
    const int qdim = m.nh * m.hd, kvdim = m.nkv * m.hd;
    auto per_block = [&](int n) { return (n + blocks - 1) / blocks; };
    g.mp_h = pitch_words(m.H / 32);
    g.vp_h = pitch_words(m.H / 64);
    g.mp_q = pitch_words(qdim / 32);
    g.vp_q = pitch_words(qdim / 64);
    g.mp_i = pitch_words(m.inter / 32);
    g.vp_i = pitch_words(m.inter / 64);
    g.t_qkv = per_block((qdim + 2 * kvdim) / 16);
    g.t_o = per_block(m.H / 16);
    g.t_gu = 2 * per_block(m.inter / 16);
    g.t_dn = per_block(m.H / 16);
    const int maxcols = std::max(std::max(m.H, qdim), m.inter);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off = (off + bytes + 127) / 128 * 128;
        return static_cast<uint32_t>(o);
    };
    g.off_sw = take(maxcols);
    g.off_x = take(maxcols);
    g.off_qkv = take(static_cast<size_t>(16) * g.t_qkv * (g.mp_h + g.vp_h) * 4);
    g.off_o = take(static_cast<size_t>(16) * g.t_o * (g.mp_q + g.vp_q) * 4);
    g.off_gu = take(static_cast<size_t>(16) * g.t_gu * (g.mp_h + g.vp_h) * 4);
    g.off_dn = take(static_cast<size_t>(16) * g.t_dn * (g.mp_i + g.vp_i) * 4);
    const int G = m.nh / m.nkv;
    g.off_attn = take(std::max(attn_smem_bytes(G, m.hd), sizeof(float) * attn_merge_smem_floats(G, m.max_seq)));
    g.off_res = take(sizeof(__half) * m.H);
    // The norm weights of a layer beside its slabs, if there is room: a producer then finds them without another
    // round trip to L2 after its reduction.
    int dev = 0, max_optin = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const size_t without = off;
    for (int i = 0; i < 3; ++i) g.off_norm[i] = take(sizeof(float) * m.H);
    g.off_norm[3] = take(sizeof(float) * m.inter);
    g.norms = off + kPdStaticSmem <= static_cast<size_t>(max_optin) ? 1 : 0;
    if (!g.norms) off = without;
    return off;
}

unsigned long long* g_pd_trace = nullptr;  // spb_debug_set_decode_trace
using PdKernel = void (*)(PdModel, PdGeom);
PdKernel kernel_for(int G, bool ll = false) {
    switch (G) {
        case 1: return ll ? decode_persistent_kernel<1, true> : decode_persistent_kernel<1, false>;
        case 2: return ll ? decode_persistent_kernel<2, true> : decode_persistent_kernel<2, false>;
        case 4: return ll ? decode_persistent_kernel<4, true> : decode_persistent_kernel<4, false>;
        case 8: return ll ? decode_persistent_kernel<8, true> : decode_persistent_kernel<8, false>;
        default: return nullptr;
    }
}

bool cooperative_ok() {
    int dev = 0, coop = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return coop != 0;
}

}  // namespace

bool decode_persistent_supported(const PdModel& m, const PdLinear* lin, const char** why) {
    auto no = [&](const char* w) {
        if (why) *why = w;
        return false;
    };
    if (m.nlayers < 1) return no("no layers");
    if (m.nh % m.nkv) return no("query heads not a multiple of KV heads");
    const int G = m.nh / m.nkv, qdim = m.nh * m.hd, kvdim = m.nkv * m.hd;
    if (!kernel_for(G)) return no("GQA group size other than 1, 2, 4, 8");
    if (m.hd % 2 || m.hd > 256 || m.hd % 16) return no("head_dim");
    if (m.H % 256 || qdim % 256 || m.inter % 256) return no("a matrix width is not a multiple of 256 columns");
    if (kvdim % 16) return no("KV rows not a multiple of 16");
    if (std::max(std::max(m.H, qdim), m.inter) > 8192) return no("a vector longer than 8192 elements");
    if (lin)
        for (int i = 0; i < 7; ++i) {
            auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
            if (lin[i].ms % 4 || lin[i].vs % 4 || !al16(lin[i].meta) || !al16(lin[i].values))
                return no("weight rows not 16-byte aligned");
        }
    if (!cooperative_ok()) return no("no cooperative launch on this device");
    PdGeom g{};
    const size_t smem = make_geom(m, sm_count(), g);
    int dev = 0, max_optin = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (g.t_qkv > 8 || g.t_o > 8 || g.t_gu > 8 || g.t_dn > 8) return no("more than eight tiles per block and stage");
    if (smem + kPdStaticSmem > static_cast<size_t>(max_optin)) return no("weight slabs of a layer do not fit in shared memory");
    if (m.barrier_free) {
        // every block keeps the residual stream itself, so every block must own rows of every projection
        const int nb = sm_count();
        if ((qdim + 2 * kvdim) / 16 < nb || m.H / 16 < nb || m.inter / 16 < nb)
            return no("barrier-free form: fewer row tiles than blocks in a projection");
        if (!m.ll) return no("barrier-free form: no buffer of tagged words");
    }
    return true;
}

size_t decode_persistent_ll_words(int H, int inter, int nh, int nkv, int hd) {
    // q, k, v, attention output, o, gate|up, down: two halves per word (gate and up of a row share one)
    return static_cast<size_t>(nh) * hd + static_cast<size_t>(nkv) * hd + static_cast<size_t>(H) + static_cast<size_t>(inter);
}

int decode_persistent_launch(const PdModel& m, long long wait_cycles, void* stream) {
    const char* name = "decode step (persistent)";
    PdKernel kernel = kernel_for(m.nh / m.nkv, m.barrier_free != 0);
    if (!kernel) return fail(SPB_E_UNSUPPORTED, "%s: group size", name);
    PdGeom g{};
    const int blocks = sm_count();
    const size_t smem = make_geom(m, blocks, g);
    g.wait_cycles = wait_cycles > 0 ? wait_cycles : kPdWaitCycles;
    g.timeouts = timeout_counter();
    g.trace = g_pd_trace;
    if (int rc = ensure_dynamic_smem(name, kernel, smem)) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(kPdThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, m, g);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "%s: launch failed: %s", name, cudaGetErrorString(err));
    }
    return SPB_OK;
}

}  // namespace spb

using namespace spb;

extern "C" int spb_debug_grid_barrier_selftest(long long limit_cycles, void* stream) {
    const char* name = "spb_debug_grid_barrier_selftest";
    int* counter = timeout_counter();
    if (!counter) return fail(SPB_E_CUDA, "%s: no timeout counter", name);
    const long long limit = limit_cycles < 1000 ? 1000 : limit_cycles > kPdWaitCycles ? kPdWaitCycles : limit_cycles;
    unsigned* sync = nullptr;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMalloc(&sync, kPdSyncWords * sizeof(unsigned));
    if (err == cudaSuccess) err = cudaMemsetAsync(sync, 0, kPdSyncWords * sizeof(unsigned), s);
    const int before = timeouts_now();
    unsigned state[4] = {0, 0, 0, 0};
    if (err == cudaSuccess) {
        pd_barrier_selftest_kernel<<<2, 32, 0, s>>>(sync, limit, counter);
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) err = cudaMemcpyAsync(state, sync, sizeof(state), cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    if (sync) cudaFree(sync);
    if (err != cudaSuccess) return fail(SPB_E_CUDA, "%s: %s", name, cudaGetErrorString(err));
    if (timeouts_now() != before && state[kSyncBroken] == 1u && state[kSyncCount] == 2u)
        return fail(SPB_E_TIMEOUT, "%s: both waits ran out after %lld cycles, as they must", name, limit);
    return fail(SPB_E_CUDA, "%s: the barrier did not report the run-out (count %u, broken %u)", name, state[kSyncCount],
                state[kSyncBroken]);
}

extern "C" void spb_debug_set_decode_trace(void* d_trace) { spb::g_pd_trace = static_cast<unsigned long long*>(d_trace); }
