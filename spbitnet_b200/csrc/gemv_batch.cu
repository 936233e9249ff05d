// Persistent work-list form of the sparse-ternary GEMV for sm_100a.
//
// One launch walks a device-resident list of GEMVs (weights, x, y per item).  The grid is a
// fixed two blocks per SM that stay resident for the whole list, so everything that costs a
// fixed amount per launch (table set-up, launch and drain latency, the DRAM latency of the
// first load) is paid once per list instead of once per 3 MB matrix, and the weight stream
// never stops: every block takes the same slice of rows of every item and brings it into
// shared memory with bulk asynchronous copies (TMA, cp.async.bulk + mbarrier transaction
// counts) through a ring of stages, so several items' worth of bytes are in flight per block
// regardless of how many registers or threads there are.
// Per item and block:
//   producer (thread 0)  : one bulk copy for the block's meta rows, one for its values rows,
//                          one 128-byte copy per column block of x (pitch 144 B, so that the
//                          per-thread 128-byte reads hit different banks);
//   consumers (all)      : wait for the stage, take their x block into 32 registers, then per
//                          unit (128 columns of a row): LDS.128 meta + LDS.64 values and
//                            sel = sel_lut[meta byte & 0x77]   PRMT selector for two groups
//                            sgn = sgn_lut[sign nibble]        their signs as int8 +-1
//                            acc = dp4a(prmt(x_lo, x_hi, sel), sgn, acc)
//                          partial sums meet in a double-buffered transposed shared array,
//                          one block barrier per item, one thread per row folds and stores y.
// The barrier that ends an item also hands its stage back to the producer.  A block never
// leaves with a copy of its own in flight: every copy it issues is waited for by the item
// that consumes it, and items are only issued for list entries that will be consumed.
#include "spb_common.cuh"

namespace spb {

int gemv_variant_setting();
int gemv_batch_mma_launch(const spb_gemv_item* d_items, int n, int max_rows, int max_cols, void* stream);

constexpr int kBThreads = 256;
constexpr int kMaxStages = 4;
constexpr int kMaxItems = 256;  // descriptors held in shared memory per launch
constexpr int kBSelEntries = 120;  // (meta byte & 0x77) <= 0x77
constexpr int kBSelBytes = kBSelEntries * 32 * 4;  // 15360
constexpr int kBSgnBytes = 16 * 32 * 4;            // 2048
constexpr int kXPitch = 144;                       // bytes between the x blocks of a stage
constexpr unsigned kWaitLimit = 1u << 26;          // polls of one barrier before giving up

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
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(mbar)
                 : "memory");
}
// Bounded wait for the phase with the given parity.  Returns false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
    for (unsigned spin = 0; spin < kWaitLimit; ++spin) {
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

// tab_lane = shared address of the tables + lane*4; the sign table follows the selector table.
__device__ __forceinline__ int mac_unit_b(const uint4& m, const uint2& v, const uint32_t (&xr)[32],
                                          uint32_t tab_lane) {
    const uint32_t mw[4] = {m.x, m.y, m.z, m.w};
    const uint32_t vw[2] = {v.x, v.y};
    int acc = 0;
#pragma unroll
    for (int p = 0; p < 16; ++p) {  // groups 2p and 2p+1: meta byte p, sign nibble p
        const int ms = 8 * (p & 3) - 7, ss = 4 * (p & 7) - 7;
        const uint32_t sel = lds_u32(((ms >= 0 ? (mw[p >> 2] >> ms) : (mw[p >> 2] << -ms)) & (0x77u << 7)) + tab_lane);
        const uint32_t sg =
            lds_u32(((ss >= 0 ? (vw[p >> 3] >> ss) : (vw[p >> 3] << -ss)) & (0xFu << 7)) + tab_lane + kBSelBytes);
        acc = __dp4a(static_cast<int>(__byte_perm(xr[2 * p], xr[2 * p + 1], sel)), static_cast<int>(sg), acc);
    }
    return acc;
}

struct BatchGeom {
    int nstages;        // stages of the ring
    int stage_bytes;    // bytes of one stage
    int values_off;     // offset of the values rows inside a stage
    int x_off;          // offset of the x blocks inside a stage
    int partial_words;  // ints of one partial buffer
};

// The slice of item I that this block owns.
__device__ __forceinline__ void item_slice(const spb_gemv_item& I, int& r_lo, int& nrows) {
    const int G = static_cast<int>(gridDim.x);
    const int rpc = (I.rows + G - 1) / G;
    r_lo = static_cast<int>(blockIdx.x) * rpc;
    nrows = max(0, min(rpc, I.rows - r_lo));
}

__global__ void __launch_bounds__(kBThreads, 2) gemv_batch_kernel(const spb_gemv_item* __restrict__ items,
                                                                   int n, const BatchGeom geom) {
    extern __shared__ __align__(128) uint8_t braw[];
    // [tables 17408][barriers (64)][descriptors kMaxItems*48][partials 2 buffers][stages]
    uint8_t* tables = braw;
    uint64_t* full = reinterpret_cast<uint64_t*>(braw + kBSelBytes + kBSgnBytes);
    spb_gemv_item* desc = reinterpret_cast<spb_gemv_item*>(braw + kBSelBytes + kBSgnBytes + 64);
    int* partial = reinterpret_cast<int*>(braw + kBSelBytes + kBSgnBytes + 64 + kMaxItems * sizeof(spb_gemv_item));
    uint8_t* stages = reinterpret_cast<uint8_t*>(partial + 2 * geom.partial_words);
    const int S = geom.nstages;

    const int tid = threadIdx.x, lane = tid & 31;
    grid_dep_launch();

    // The work list, the weights and the tables are not produced by a predecessor kernel.
    for (int q = tid; q < (kBSelBytes + kBSgnBytes) / 16; q += kBThreads)
        reinterpret_cast<uint4*>(tables)[q] = __ldg(reinterpret_cast<const uint4*>(&g_batch_lut) + q);
    {
        const uint4* src = reinterpret_cast<const uint4*>(items);
        uint4* dst = reinterpret_cast<uint4*>(desc);
        for (int q = tid; q < n * 3; q += kBThreads) dst[q] = __ldg(src + q);  // 48-byte descriptors
    }
    if (tid == 0) {
        for (int s = 0; s < S; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_addr(full + s)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // x is an output of a predecessor: nothing of an item is requested before the wait.
    grid_dep_wait();

    // Producer: fills stage (j % S) with item j.  Thread 0 only.
    auto produce = [&](int j) {
        const spb_gemv_item& I = desc[j];
        int r_lo, nrows;
        item_slice(I, r_lo, nrows);
        const uint32_t bar = s_addr(full + (j % S));
        const uint32_t base = s_addr(stages + static_cast<size_t>(j % S) * geom.stage_bytes);
        if (nrows == 0) {
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
            return;
        }
        const uint32_t mrow = static_cast<uint32_t>(I.cols) >> 3, vrow = static_cast<uint32_t>(I.cols) >> 4;
        const uint32_t total = nrows * (mrow + vrow) + I.cols;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(total) : "memory");
        if (I.meta_row_stride * 4 == static_cast<int>(mrow)) {
            bulk_g2s(base, I.meta + static_cast<size_t>(r_lo) * I.meta_row_stride, nrows * mrow, bar);
        } else {
            for (int r = 0; r < nrows; ++r)
                bulk_g2s(base + r * mrow, I.meta + static_cast<size_t>(r_lo + r) * I.meta_row_stride, mrow, bar);
        }
        if (I.values_row_stride * 4 == static_cast<int>(vrow)) {
            bulk_g2s(base + geom.values_off, I.values + static_cast<size_t>(r_lo) * I.values_row_stride, nrows * vrow, bar);
        } else {
            for (int r = 0; r < nrows; ++r)
                bulk_g2s(base + geom.values_off + r * vrow, I.values + static_cast<size_t>(r_lo + r) * I.values_row_stride,
                         vrow, bar);
        }
        const int upr = I.cols >> 7;
        for (int c = 0; c < upr; ++c) bulk_g2s(base + geom.x_off + c * kXPitch, I.x + (c << 7), 128, bar);
    };
    if (tid == 0)
        for (int j = 0; j < min(n, S); ++j) produce(j);

    const uint32_t tab_lane = s_addr(tables) + lane * 4;
    int buf = 0;
    for (int j = 0; j < n; ++j) {
        const spb_gemv_item I = desc[j];
        int r_lo, nrows;
        item_slice(I, r_lo, nrows);
        const int stage = j % S;
        // If the limit runs out the data is not there: leave the item's outputs untouched
        // rather than compute on garbage (the copy is still awaited by nobody else, so the
        // limit is set far beyond any legitimate delay).
        const bool landed = mbar_wait(s_addr(full + stage), (j / S) & 1);
        const uint8_t* sb = stages + static_cast<size_t>(stage) * geom.stage_bytes;
        int* pbuf = partial + buf * geom.partial_words;
        const int upr = I.cols >> 7;
        const int pitch = ((I.rows + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)) | 1;
        if (nrows > 0 && landed) {
            const int rs_cnt = kBThreads / upr;
            const int rs = tid / upr, cb = tid - rs * upr;
            if (rs < rs_cnt) {
                uint32_t xr[32];
                const uint4* xb = reinterpret_cast<const uint4*>(sb + geom.x_off + cb * kXPitch);
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    const uint4 t = xb[ch];
                    xr[4 * ch + 0] = t.x; xr[4 * ch + 1] = t.y; xr[4 * ch + 2] = t.z; xr[4 * ch + 3] = t.w;
                }
                const uint32_t mrow = static_cast<uint32_t>(I.cols) >> 3, vrow = static_cast<uint32_t>(I.cols) >> 4;
                for (int rl = rs; rl < nrows; rl += rs_cnt) {
                    const uint4 m = *reinterpret_cast<const uint4*>(sb + rl * mrow + cb * 16);
                    const uint2 v = *reinterpret_cast<const uint2*>(sb + geom.values_off + rl * vrow + cb * 8);
                    pbuf[cb * pitch + rl] = mac_unit_b(m, v, xr, tab_lane);
                }
            }
        }
        __syncthreads();  // partials complete; the stage is free again
        if (tid == 0 && j + S < n) produce(j + S);
        if (landed) {
            for (int lr = tid; lr < nrows; lr += kBThreads) {
                int s = 0;
                for (int c = 0; c < upr; ++c) s += pbuf[c * pitch + lr];
                I.y[r_lo + lr] = s;
            }
        }
        buf ^= 1;
    }
}

}  // namespace spb

using namespace spb;

extern "C" int spb_gemv_batch_check(const spb_gemv_item* h_items, int n) {
    if (n < 0 || (n > 0 && !h_items)) return fail(SPB_E_INVALID, "spb_gemv_batch_check: bad list");
    for (int i = 0; i < n; ++i) {
        const spb_gemv_item& I = h_items[i];
        auto al = [](const void* p, size_t k) { return (reinterpret_cast<uintptr_t>(p) & (k - 1)) == 0; };
        if (I.rows <= 0 || I.cols <= 0 || I.cols % 256 != 0 || I.cols > 128 * kBThreads)
            return fail(SPB_E_UNSUPPORTED, "item %d: %dx%d (cols must be a multiple of 256, at most %d)", i, I.rows,
                        I.cols, 128 * kBThreads);
        if (!I.meta || !I.values || !I.x || !I.y) return fail(SPB_E_INVALID, "item %d: null pointer", i);
        if (I.meta_row_stride < I.cols / 32 || I.values_row_stride < I.cols / 64 || I.meta_row_stride % 4 ||
            I.values_row_stride % 4)
            return fail(SPB_E_UNSUPPORTED, "item %d: row strides must cover a row and be multiples of 4 words", i);
        if (!al(I.meta, 16) || !al(I.values, 16) || !al(I.x, 16) || !al(I.y, 4))
            return fail(SPB_E_UNSUPPORTED, "item %d: meta, values and x must be 16-byte aligned", i);
    }
    return SPB_OK;
}

extern "C" int spb_sparse_ternary_gemv_batch(const spb_gemv_item* d_items, int n, int max_rows, int max_cols,
                                             void* stream) {
    const char* name = "spb_sparse_ternary_gemv_batch";
    if (n < 0 || max_rows < 0 || max_cols < 0) return fail(SPB_E_INVALID, "%s: negative size", name);
    if (n == 0 || max_rows == 0 || max_cols == 0) return SPB_OK;
    if (!d_items) return fail(SPB_E_INVALID, "%s: null pointer", name);
    if (max_cols % 256 != 0 || max_cols > 128 * kBThreads)
        return fail(SPB_E_UNSUPPORTED, "%s: max_cols=%d (multiple of 256, at most %d)", name, max_cols, 128 * kBThreads);
    if ((reinterpret_cast<uintptr_t>(d_items) & 15) != 0) return fail(SPB_E_INVALID, "%s: d_items must be 16-byte aligned", name);
    // automatic: the tensor-core form (gemv_batch_mma.cu); the SIMT form below when a SIMT GEMV kernel is selected
    if (gemv_variant_setting() == 0 || gemv_variant_setting() >= 3)
        return gemv_batch_mma_launch(d_items, n, max_rows, max_cols, stream);
    const int grid = 2 * sm_count();
    const int rpc = (max_rows + grid - 1) / grid;
    BatchGeom g{};
    const int meta_area = (rpc * (max_cols / 8) + 127) & ~127;
    const int values_area = (rpc * (max_cols / 16) + 127) & ~127;
    const int x_area = ((max_cols / 128) * kXPitch + 127) & ~127;
    g.values_off = meta_area;
    g.x_off = meta_area + values_area;
    g.stage_bytes = meta_area + values_area + x_area;
    g.partial_words = ((max_cols / 128) * (rpc | 1) + 31) & ~31;
    const size_t fixed = kBSelBytes + kBSgnBytes + 64 + kMaxItems * sizeof(spb_gemv_item) + 2 * sizeof(int) * g.partial_words;
    size_t budget = 110 * 1024;  // two blocks per SM
    if (fixed + 2 * static_cast<size_t>(g.stage_bytes) > budget) budget = 200 * 1024;  // one block per SM
    if (fixed + 2 * static_cast<size_t>(g.stage_bytes) > budget)
        return fail(SPB_E_UNSUPPORTED, "%s: %d rows x %d cols per block need more shared memory than a block may take", name,
                    rpc, max_cols);
    g.nstages = static_cast<int>((budget - fixed) / g.stage_bytes);
    if (g.nstages > kMaxStages) g.nstages = kMaxStages;
    const size_t smem = fixed + static_cast<size_t>(g.nstages) * g.stage_bytes;
    cudaError_t err = cudaFuncSetAttribute(gemv_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "%s: %s", name, cudaGetErrorString(err));
    }
    for (int first = 0; first < n; first += kMaxItems) {
        const int count = min(kMaxItems, n - first);
        int rc = launch(name, gemv_batch_kernel, dim3(grid), dim3(kBThreads), smem, stream, d_items + first, count, g);
        if (rc) return rc;
    }
    return SPB_OK;
}
