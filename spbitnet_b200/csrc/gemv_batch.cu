// Persistent work-list form of the sparse-ternary GEMV for sm_100a.
//
// One launch walks a device-resident list of GEMVs (weights, x, y per item).  The grid is a
// fixed number of blocks per SM that stay resident for the whole list, so everything that
// costs a fixed amount per launch (table set-up, launch and drain latency, the DRAM latency
// of the first load) is paid once per list instead of once per 3 MB matrix.  Every block
// takes the same slice of rows of every item; a thread owns one 128-column block of x per
// item (32 registers) and walks down the rows of its slice:
//   sel = sel_lut[meta byte & 0x77]   PRMT selector gathering the four non-zero columns of two groups
//   sgn = sgn_lut[sign nibble]        their signs as int8 +-1
//   acc = dp4a(prmt(x_lo, x_hi, sel), sgn, acc)
// Weight loads (16 B meta + 8 B values per unit) run two units ahead of the arithmetic and
// cross item boundaries, the next item's x block is prefetched into L1, and the per-row
// partial sums meet in a double-buffered shared array that one thread per row folds.
// The tables reach shared memory by bulk asynchronous copies (TMA) into a 16 KB-aligned
// window so that a table address is (index bits | lane bits | window) - one LOP3.
#include "spb_common.cuh"

namespace spb {

constexpr int kBThreads = 256;
constexpr int kBSelEntries = 120;  // (meta byte & 0x77) <= 0x77
constexpr int kBSelBytes = kBSelEntries * 32 * 4;  // 15360
constexpr int kBSgnBytes = 16 * 32 * 4;           // 2048
constexpr int kBWindow = 16384;

struct BatchLutImage {
    uint32_t sel[kBSelEntries * 32];
    uint32_t sgn[16 * 32];
};

constexpr uint32_t batch_pair_selector(int b) {
    uint32_t sel = 0;
    for (int half = 0; half < 2; ++half) {
        int n = (b >> (4 * half)) & 7;
        const int cnt = (n & 1) + ((n >> 1) & 1) + ((n >> 2) & 1);
        if (cnt == 1) n |= 8;  // exactly two of four bits are set: the fourth bit is implied
        int bits = 0, p0 = 0, p1 = 0;
        for (int i = 0; i < 4; ++i)
            if (n & (1 << i)) {
                if (bits == 0) p0 = i;
                if (bits == 1) p1 = i;
                ++bits;
            }
        if (bits != 2) { p0 = 0; p1 = 0; }
        sel |= static_cast<uint32_t>((4 * half + p0) | ((4 * half + p1) << 4)) << (8 * half);
    }
    return sel;
}

constexpr BatchLutImage make_batch_lut_image() {
    BatchLutImage t{};
    for (int e = 0; e < kBSelEntries; ++e)
        for (int l = 0; l < 32; ++l) t.sel[e * 32 + l] = batch_pair_selector(e);
    for (int n = 0; n < 16; ++n) {
        uint32_t w = 0;
        for (int i = 0; i < 4; ++i) w |= ((n >> i) & 1 ? 0xFFu : 0x01u) << (8 * i);
        for (int l = 0; l < 32; ++l) t.sgn[n * 32 + l] = w;
    }
    return t;
}

__device__ __align__(128) const BatchLutImage g_batch_lut = make_batch_lut_image();

__device__ __forceinline__ uint32_t s_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// sel_lane = window | lane*4 (window 16 KB aligned); sgn_lane = sel_lane + kBWindow.
__device__ __forceinline__ int mac_unit_b(const uint4& m, const uint2& v, const uint32_t (&xr)[32],
                                          uint32_t sel_lane, uint32_t sgn_lane) {
    const uint32_t mw[4] = {m.x, m.y, m.z, m.w};
    const uint32_t vw[2] = {v.x, v.y};
    int acc = 0;
#pragma unroll
    for (int p = 0; p < 16; ++p) {  // groups 2p and 2p+1: meta byte p, sign nibble p
        const int ms = 8 * (p & 3) - 7;
        const uint32_t ma = ((ms >= 0 ? (mw[p >> 2] >> ms) : (mw[p >> 2] << -ms)) & (0x77u << 7)) | sel_lane;
        const int ss = 4 * (p & 7) - 7;
        const uint32_t sa = ((ss >= 0 ? (vw[p >> 3] >> ss) : (vw[p >> 3] << -ss)) & (0xFu << 7)) | sgn_lane;
        uint32_t sel, sg;
        asm("ld.shared.u32 %0, [%1];" : "=r"(sel) : "r"(ma));
        asm("ld.shared.u32 %0, [%1];" : "=r"(sg) : "r"(sa));
        acc = __dp4a(static_cast<int>(__byte_perm(xr[2 * p], xr[2 * p + 1], sel)), static_cast<int>(sg), acc);
    }
    return acc;
}

// Position of a thread in the flattened (item, iteration) sequence.
struct Cursor {
    int j;       // item
    int it;      // iteration inside the item
    int niter;   // iterations of the item for this block
    int nrows;   // rows of the item in this block's slice
    int rs_cnt;  // row slots
    int rs, cb;  // this thread's slot and column block
    bool active;
    const uint32_t* mp;
    const uint32_t* vp;
    size_t m_step, v_step;
};

__device__ __forceinline__ void cursor_open(Cursor& c, const spb_gemv_item* items, int n, int j, int tid) {
    c.j = j;
    c.it = 0;
    if (j >= n) {
        c.niter = 0;
        c.nrows = 0;
        c.active = false;
        return;
    }
    const spb_gemv_item I = items[j];
    const int upr = I.cols >> 7;
    const int rpc = (I.rows + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    const int r_lo = static_cast<int>(blockIdx.x) * rpc;
    c.nrows = max(0, min(rpc, I.rows - r_lo));
    c.rs_cnt = kBThreads / upr;
    c.rs = tid / upr;
    c.cb = tid - c.rs * upr;
    c.active = c.rs < c.rs_cnt;
    c.niter = (c.nrows + c.rs_cnt - 1) / c.rs_cnt;
    c.mp = I.meta + static_cast<size_t>(r_lo + c.rs) * I.meta_row_stride + c.cb * 4;
    c.vp = I.values + static_cast<size_t>(r_lo + c.rs) * I.values_row_stride + c.cb * 2;
    c.m_step = static_cast<size_t>(c.rs_cnt) * I.meta_row_stride;
    c.v_step = static_cast<size_t>(c.rs_cnt) * I.values_row_stride;
}

// Skips items in which this block has no rows; returns false at the end of the list.
__device__ __forceinline__ bool cursor_settle(Cursor& c, const spb_gemv_item* items, int n, int tid) {
    while (c.j < n && c.it >= c.niter) cursor_open(c, items, n, c.j + 1, tid);
    return c.j < n;
}

__device__ __forceinline__ bool cursor_has_unit(const Cursor& c) {
    return c.active && c.it * c.rs_cnt + c.rs < c.nrows;
}

__global__ void __launch_bounds__(kBThreads, 2) gemv_batch_kernel(const spb_gemv_item* __restrict__ items,
                                                                   int n, int partial_words) {
    extern __shared__ __align__(128) uint8_t braw[];
    const uint32_t raw_s = s_addr(braw);
    const uint32_t win_s = (raw_s + kBWindow - 1) & ~static_cast<uint32_t>(kBWindow - 1);
    uint8_t* win = braw + (win_s - raw_s);
    // window: [sel 16 KB][sgn 2 KB][mbarrier 16 B][partials: 2 buffers of partial_words ints]
    uint64_t* mbar = reinterpret_cast<uint64_t*>(win + kBWindow + kBSgnBytes);
    int* partial = reinterpret_cast<int*>(win + kBWindow + kBSgnBytes + 16);

    const int tid = threadIdx.x, lane = tid & 31;
    grid_dep_launch();

    const uint32_t mbar_s = s_addr(mbar);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_s));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar_s), "n"(kBSelBytes + kBSgnBytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(win_s),
                     "l"(__cvta_generic_to_global(g_batch_lut.sel)), "n"(kBSelBytes), "r"(mbar_s)
                     : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(win_s + kBWindow),
                     "l"(__cvta_generic_to_global(g_batch_lut.sgn)), "n"(kBSgnBytes), "r"(mbar_s)
                     : "memory");
    }
    __syncthreads();  // nobody polls the barrier before it is initialised

    // The work list and the weights are not produced by a predecessor kernel; x and y are.
    Cursor cur, ahead;
    cursor_open(cur, items, n, 0, tid);
    bool more = cursor_settle(cur, items, n, tid);
    ahead = cur;

    // two units of weights in flight
    uint4 m[2];
    uint2 v[2];
#pragma unroll
    for (int d = 0; d < 2; ++d) {
        m[d] = make_uint4(0, 0, 0, 0);
        v[d] = make_uint2(0, 0);
        if (ahead.j < n) {
            if (cursor_has_unit(ahead)) {
                m[d] = ld_stream_v4(ahead.mp + ahead.it * ahead.m_step);
                v[d] = ld_stream_v2(ahead.vp + ahead.it * ahead.v_step);
            }
            ahead.it++;
            cursor_settle(ahead, items, n, tid);
        }
    }

    grid_dep_wait();

    // tables: bounded wait, plain-load fill if the copy did not land
    {
        uint32_t done = 0;
        for (int spin = 0; spin < (1 << 20) && !done; ++spin) {
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(done)
                : "r"(mbar_s)
                : "memory");
        }
        if (!__syncthreads_and(done != 0)) {
            uint32_t* sel = reinterpret_cast<uint32_t*>(win);
            uint32_t* sgn = reinterpret_cast<uint32_t*>(win + kBWindow);
            for (int e = tid; e < kBSelEntries * 32; e += kBThreads) sel[e] = g_batch_lut.sel[e];
            for (int e = tid; e < 16 * 32; e += kBThreads) sgn[e] = g_batch_lut.sgn[e];
            __syncthreads();
        }
    }
    uint32_t sel_lane;
    asm volatile("or.b32 %0, %1, %2;" : "=r"(sel_lane) : "r"(win_s), "r"(lane * 4) : "memory");
    const uint32_t sgn_lane = sel_lane + kBWindow;

    uint32_t xr[32];
    int slot = 0;
    int buf = 0;  // partial buffer of the item being processed; alternates per processed item
    while (more) {
        // ---- one item --------------------------------------------------------------------
        const int j = cur.j;
        const spb_gemv_item I = items[j];
        const int upr = I.cols >> 7;
        const int pitch = ((I.rows + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)) | 1;
        int* pbuf = partial + buf * partial_words;
        buf ^= 1;
        if (cur.active) {
            const uint4* xg = reinterpret_cast<const uint4*>(I.x) + (cur.cb << 3);
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                const uint4 t = __ldg(xg + ch);
                xr[4 * ch + 0] = t.x; xr[4 * ch + 1] = t.y; xr[4 * ch + 2] = t.z; xr[4 * ch + 3] = t.w;
            }
            if (j + 1 < n) {  // next item's x block into L1
                const spb_gemv_item N = items[j + 1];
                if ((cur.cb << 7) < N.cols)
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const uint8_t*>(N.x) + (cur.cb << 7)));
            }
        }
        const int niter = cur.niter;
        for (int it = 0; it < niter; ++it) {
            // consume slot, refill it with the unit two steps ahead (possibly of a later item)
            const bool has = cursor_has_unit(cur);
            int part = 0;
            if (slot == 0) {
                if (has) part = mac_unit_b(m[0], v[0], xr, sel_lane, sgn_lane);
                if (ahead.j < n) {
                    if (cursor_has_unit(ahead)) {
                        m[0] = ld_stream_v4(ahead.mp + ahead.it * ahead.m_step);
                        v[0] = ld_stream_v2(ahead.vp + ahead.it * ahead.v_step);
                    }
                    ahead.it++;
                    cursor_settle(ahead, items, n, tid);
                }
            } else {
                if (has) part = mac_unit_b(m[1], v[1], xr, sel_lane, sgn_lane);
                if (ahead.j < n) {
                    if (cursor_has_unit(ahead)) {
                        m[1] = ld_stream_v4(ahead.mp + ahead.it * ahead.m_step);
                        v[1] = ld_stream_v2(ahead.vp + ahead.it * ahead.v_step);
                    }
                    ahead.it++;
                    cursor_settle(ahead, items, n, tid);
                }
            }
            slot ^= 1;
            if (has) pbuf[cur.cb * pitch + it * cur.rs_cnt + cur.rs] = part;
            cur.it++;
        }
        __syncthreads();
        // one thread per row folds the partials of its row and stores y
        {
            const int rpc = (I.rows + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
            const int r_lo = static_cast<int>(blockIdx.x) * rpc;
            for (int lr = tid; lr < cur.nrows; lr += kBThreads) {
                int s = 0;
                for (int c = 0; c < upr; ++c) s += pbuf[c * pitch + lr];
                I.y[r_lo + lr] = s;
            }
        }
        more = cursor_settle(cur, items, n, tid);
    }
}

}  // namespace spb

using namespace spb;

extern "C" int spb_gemv_batch_check(const spb_gemv_item* h_items, int n) {
    if (n < 0 || (n > 0 && !h_items)) return fail(SPB_E_INVALID, "spb_gemv_batch_check: bad list");
    for (int i = 0; i < n; ++i) {
        const spb_gemv_item& I = h_items[i];
        auto al = [](const void* p, size_t k) { return (reinterpret_cast<uintptr_t>(p) & (k - 1)) == 0; };
        if (I.rows <= 0 || I.cols <= 0 || I.cols % 128 != 0 || I.cols > 128 * kBThreads)
            return fail(SPB_E_UNSUPPORTED, "item %d: %dx%d (cols must be a multiple of 128, at most %d)", i, I.rows,
                        I.cols, 128 * kBThreads);
        if (!I.meta || !I.values || !I.x || !I.y) return fail(SPB_E_INVALID, "item %d: null pointer", i);
        if (I.meta_row_stride < I.cols / 32 || I.values_row_stride < I.cols / 64 || I.meta_row_stride % 4 ||
            I.values_row_stride % 2)
            return fail(SPB_E_UNSUPPORTED, "item %d: row strides must cover a row and be multiples of 4 / 2 words", i);
        if (!al(I.meta, 16) || !al(I.values, 8) || !al(I.x, 16) || !al(I.y, 4))
            return fail(SPB_E_UNSUPPORTED, "item %d: meta/values/x must be 16/8/16-byte aligned", i);
    }
    return SPB_OK;
}

extern "C" int spb_sparse_ternary_gemv_batch(const spb_gemv_item* d_items, int n, int max_rows, int max_cols,
                                             void* stream) {
    const char* name = "spb_sparse_ternary_gemv_batch";
    if (n < 0 || max_rows < 0 || max_cols < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    if (n == 0 || max_rows == 0 || max_cols == 0) return SPB_OK;
    if (!d_items) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (max_cols % 128 != 0 || max_cols > 128 * kBThreads)
        return fail(SPB_E_UNSUPPORTED, "%s: max_cols=%d (multiple of 128, at most %d)", name, max_cols, 128 * kBThreads);
    const int grid = 2 * sm_count();
    const int rpc = (max_rows + grid - 1) / grid;
    const int partial_words = ((max_cols / 128) * (rpc | 1) + 3) & ~3;
    const size_t smem = kBWindow /*alignment slack*/ + kBWindow + kBSgnBytes + 16 + 2 * sizeof(int) * partial_words;
    if (smem > 110 * 1024) return fail(SPB_E_UNSUPPORTED, "%s: %d rows x %d cols per block exceed shared memory", name, rpc, max_cols);
    cudaError_t err = cudaFuncSetAttribute(gemv_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "%s: %s", name, cudaGetErrorString(err));
    }
    return launch(name, gemv_batch_kernel, dim3(grid), dim3(kBThreads), smem, stream, d_items, n, partial_words);
}
