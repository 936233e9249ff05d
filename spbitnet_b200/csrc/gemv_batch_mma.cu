// Persistent work-list GEMV on the warp-level sparse MMA (mma.sp m16n8k64), sm_100a.
//
// One launch walks a device-resident list of GEMVs.  The scheme per tile is the one of gemv_mmasp.cu
// (raw slab by 16-byte cp.async into padded shared-memory rows, bitmap words re-encoded to index pairs
// and sign nibbles to +1 / -1 bytes in registers, one mma.sp per 64 columns of 16 rows); what the list
// form adds is that nothing is paid per GEMV any more: blocks stay resident, the sign table is built
// once, and while a block computes tile t the slab and the x vector of tile t + 1 are already on their
// way into the other half of a double buffer, so the weight stream never stops and there is no launch,
// no block start-up and no cold DRAM latency between two GEMVs.
//
// Tiles: item i is cut into tiles of 16 * rb_i rows, rb_i = 8 / ks_i row blocks with ks_i warps each
// (ks_i = the largest of 8, 4, 2, 1 that leaves a warp at least 16 steps of 64 columns).  Tile number g
// of the whole list belongs to block g mod gridDim.x.
// There is no spin-wait in the kernel (cp.async groups and block barriers only).
#include "spb_common.cuh"

namespace spb {

constexpr int kBmThreads = 256;
constexpr int kBmWarps = 8;
constexpr int kBmMaxItems = 256;  // descriptors held in shared memory per launch

struct BmGeom {
    int stage_bytes;  // one half of the double buffer: slab + x, 16-byte aligned
    int x_off;        // offset of the x vector inside a stage
    int max_cols;     // the stages are sized for items of up to this many columns; wider items are skipped
};

struct BmTile {
    int item;   // index into the descriptor array, or -1 past the end of the list
    int row0;   // first row of the tile
    int ks_log2;
};

__device__ __forceinline__ int bm_ks_log2(int cols) {
    const int steps = cols >> 6;
    return steps >= 128 ? 3 : steps >= 64 ? 2 : steps >= 32 ? 1 : 0;
}
__host__ __device__ __forceinline__ int bm_pitch(int words) {
    // smallest pitch >= words that is an odd multiple of four words (rows stay 16-byte aligned and eight
    // consecutive rows start on eight different groups of four banks)
    return words % 8 == 4 ? words : words + ((4 - words % 8) + 8) % 8;
}

__device__ __forceinline__ uint32_t bm_index_pairs(uint32_t m) {
    // eight bitmaps (two of four bits set each) -> eight index pairs {low index | high index << 2}
    const uint32_t mr = m >> 1, ml = m << 1;
    const uint32_t t1 = (0x11111111u & (~m & mr)) | (~0x11111111u & (mr | ~m));
    const uint32_t t2 = (0x22222222u & (~ml & ~m)) | (~0x22222222u & (m | ml));
    return (t1 & 0x55555555u) | (t2 & 0xAAAAAAAAu);
}
__device__ __forceinline__ uint32_t bm_lds(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__global__ void __launch_bounds__(kBmThreads, 3) gemv_batch_mma_kernel(const spb_gemv_item* __restrict__ items, int n,
                                                                       const BmGeom geo) {
    __shared__ __align__(16) uint32_t sgn_tab[16 * 32];  // entry (nibble v, lane l) at word v * 32 + l
    __shared__ int red[kBmWarps * 16];
    __shared__ __align__(16) spb_gemv_item desc[kBmMaxItems];
    extern __shared__ __align__(16) uint8_t bm_raw[];     // two stages: [slab: bitmap rows | sign rows][x]
    const uint32_t tab_s = static_cast<uint32_t>(__cvta_generic_to_shared(sgn_tab));
    const uint32_t dyn_s = static_cast<uint32_t>(__cvta_generic_to_shared(bm_raw));

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);  // through a shuffle: known to be uniform over the warp
    const int g = lane >> 2, tig = lane & 3;

    grid_dep_launch();
    grid_dep_wait();  // descriptors, weights and activations may all come from a predecessor
    {
        const uint4* src = reinterpret_cast<const uint4*>(items);
        uint4* dst = reinterpret_cast<uint4*>(desc);
        for (int q = tid; q < n * 3; q += kBmThreads) dst[q] = __ldg(src + q);  // 48-byte descriptors
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {  // byte b of an entry = -1 if bit b of the nibble is set, else +1
        const uint32_t i = tid + j * kBmThreads;
        const uint32_t t = ((i >> 5) * 0x00204081u) & 0x01010101u;
        sgn_tab[i] = (t * 0xFEu) | 0x01010101u;
    }
    __syncthreads();

    // ---- the block's tile sequence: global tile number blockIdx.x, + gridDim.x, ... -------------------------
    int walk_item = 0, walk_base = 0;  // first item not yet passed, global number of its first tile
    auto locate = [&](int gt) {        // gt is non-decreasing over calls
        BmTile t{-1, 0, 0};
        while (walk_item < n) {
            const int kl = bm_ks_log2(desc[walk_item].cols), tr = 128 >> kl;
            // an item wider than the stages were sized for has no tiles: it is skipped, never copied
            const int nt = desc[walk_item].cols > geo.max_cols ? 0 : (desc[walk_item].rows + tr - 1) / tr;
            if (gt < walk_base + nt) {
                t.item = walk_item;
                t.row0 = (gt - walk_base) * tr;
                t.ks_log2 = kl;
                break;
            }
            walk_base += nt;
            ++walk_item;
        }
        return t;
    };
    // issues the copies of a tile (its slab and its x) into stage `st`, one commit group
    auto fetch = [&](const BmTile& t, int st) {
        if (t.item >= 0) {
            const spb_gemv_item& I = desc[t.item];
            const int tr = 128 >> t.ks_log2, valid = min(tr, I.rows - t.row0);
            const int mp = bm_pitch(I.cols >> 5), vp = bm_pitch(I.cols >> 6);
            const uint32_t ms_s = dyn_s + static_cast<uint32_t>(st) * geo.stage_bytes;
            const uint32_t vs_s = ms_s + static_cast<uint32_t>(tr * mp) * 4u;
            const int mch = I.cols >> 7, cpr = mch + (I.cols >> 8);  // 16-byte chunks of a row: bitmaps, then signs
            for (int k = lane; k < cpr; k += 32) {
                const bool is_m = k < mch;
                const uint8_t* src = is_m ? reinterpret_cast<const uint8_t*>(I.meta) + k * 16
                                          : reinterpret_cast<const uint8_t*>(I.values) + (k - mch) * 16;
                const size_t src_pitch = static_cast<size_t>(is_m ? I.meta_row_stride : I.values_row_stride) * 4u;
                const uint32_t dst = is_m ? ms_s + static_cast<uint32_t>(k) * 16u : vs_s + static_cast<uint32_t>(k - mch) * 16u;
                const uint32_t dst_pitch = static_cast<uint32_t>(is_m ? mp : vp) * 4u;
                src += static_cast<size_t>(t.row0 + warp) * src_pitch;
                for (int r = warp; r < valid; r += kBmWarps) {
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + static_cast<uint32_t>(r) * dst_pitch),
                                 "l"(src)
                                 : "memory");
                    src += kBmWarps * src_pitch;
                }
            }
            const uint32_t xs_s = ms_s + static_cast<uint32_t>(geo.x_off);
            for (int q = tid; q < (I.cols >> 4); q += kBmThreads)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(xs_s + static_cast<uint32_t>(q) * 16u),
                             "l"(I.x + static_cast<size_t>(q) * 16)
                             : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // also for an empty tile: keeps the group count uniform
    };

    const uint32_t lane_or = static_cast<uint32_t>(lane) << 2;
    const uint32_t rot_lo = (static_cast<uint32_t>(tig) * 4u + 25u) & 31u, rot_hi = (static_cast<uint32_t>(tig) * 4u + 9u) & 31u;

    int gt = blockIdx.x;
    BmTile cur = locate(gt);
    fetch(cur, 0);
    for (int it = 0; cur.item >= 0; ++it) {
        gt += gridDim.x;
        const BmTile nxt = locate(gt);
        fetch(nxt, (it + 1) & 1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the newest group: this tile has landed
        __syncthreads();

        const spb_gemv_item& I = desc[cur.item];
        const int ks = 1 << cur.ks_log2, tr = 128 >> cur.ks_log2;
        const int steps = I.cols >> 6, spw = (steps + ks - 1) >> cur.ks_log2;
        const int mp = bm_pitch(I.cols >> 5), vp = bm_pitch(I.cols >> 6);
        const uint32_t ms_s = dyn_s + static_cast<uint32_t>(it & 1) * geo.stage_bytes;
        const uint32_t vs_s = ms_s + static_cast<uint32_t>(tr * mp) * 4u;
        const uint32_t xs_s = ms_s + static_cast<uint32_t>(geo.x_off);
        const int rbi = warp >> cur.ks_log2, kq = warp & (ks - 1);
        const int s_begin = kq * spw, s_end = min(steps, s_begin + spw);
        // running addresses: the lane's bitmap word, the sign words of rows g and g + 8 of the row block, x
        uint32_t me_p = ms_s + static_cast<uint32_t>((rbi * 16 + g + 8 * (tig & 1)) * mp + (tig >> 1) + 2 * s_begin) * 4u;
        uint32_t v0_p = vs_s + static_cast<uint32_t>((rbi * 16 + g) * vp + s_begin) * 4u;
        const uint32_t v_half = static_cast<uint32_t>(8 * vp) * 4u;
        uint32_t xq_p = xs_s + static_cast<uint32_t>(tig) * 4u + static_cast<uint32_t>(s_begin) * 64u;

        // One step = 64 columns of 16 rows.  Metadata register of lane (g, tig): the index pairs of bitmap word
        // 2 s + (tig >> 1) of row g + 8 (tig & 1); B register j: x[64 s + 16 j + 4 tig ..+3] (x is not re-ordered
        // here: four 4-byte reads, each the same word for the eight lanes of equal tig).
        int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
        auto step = [&](uint32_t w0, uint32_t w1, uint32_t me_off, uint32_t x_off) {
            const uint32_t e = bm_index_pairs(bm_lds(me_p + me_off));
            const uint32_t a0 = bm_lds(tab_s + ((__funnelshift_r(w0, w0, rot_lo) & 0x780u) | lane_or));
            const uint32_t a1 = bm_lds(tab_s + ((__funnelshift_r(w1, w1, rot_lo) & 0x780u) | lane_or));
            const uint32_t a2 = bm_lds(tab_s + ((__funnelshift_r(w0, w0, rot_hi) & 0x780u) | lane_or));
            const uint32_t a3 = bm_lds(tab_s + ((__funnelshift_r(w1, w1, rot_hi) & 0x780u) | lane_or));
            const uint32_t b0 = bm_lds(xq_p + x_off), b1 = bm_lds(xq_p + x_off + 16u);
            const uint32_t b2 = bm_lds(xq_p + x_off + 32u), b3 = bm_lds(xq_p + x_off + 48u);
            asm volatile(
                "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
                "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
                : "+r"(c0), "+r"(c1), "+r"(c2), "+r"(c3)
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(b2), "r"(b3), "r"(e));
        };
        auto advance = [&](uint32_t k) {
            me_p += 8u * k;
            v0_p += 4u * k;
            xq_p += 64u * k;
        };
        int st = s_begin;
        for (; st < s_end && (st & 3) != 0; ++st) {
            step(bm_lds(v0_p), bm_lds(v0_p + v_half), 0u, 0u);
            advance(1u);
        }
        for (; st + 4 <= s_end; st += 4) {
            // Four steps at a time, written phase by phase so that all independent shared-memory reads are in
            // flight together: raw words (sign words of four steps are one 16-byte read per row), then the
            // table reads, then the four MMAs.
            uint32_t w0[4], w1[4], mw[4], B[4][4], A[4][4];
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w0[0]), "=r"(w0[1]), "=r"(w0[2]), "=r"(w0[3]) : "r"(v0_p));
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w1[0]), "=r"(w1[1]), "=r"(w1[2]), "=r"(w1[3])
                         : "r"(v0_p + v_half));
#pragma unroll
            for (int i = 0; i < 4; ++i) mw[i] = bm_lds(me_p + 8u * i);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) B[i][j] = bm_lds(xq_p + 64u * i + 16u * j);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                A[i][0] = bm_lds(tab_s + ((__funnelshift_r(w0[i], w0[i], rot_lo) & 0x780u) | lane_or));
                A[i][1] = bm_lds(tab_s + ((__funnelshift_r(w1[i], w1[i], rot_lo) & 0x780u) | lane_or));
                A[i][2] = bm_lds(tab_s + ((__funnelshift_r(w0[i], w0[i], rot_hi) & 0x780u) | lane_or));
                A[i][3] = bm_lds(tab_s + ((__funnelshift_r(w1[i], w1[i], rot_hi) & 0x780u) | lane_or));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t e = bm_index_pairs(mw[i]);
                asm volatile(
                    "mma.sp::ordered_metadata.sync.aligned.m16n8k64.row.col.s32.s8.s8.s32 "
                    "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
                    : "+r"(c0), "+r"(c1), "+r"(c2), "+r"(c3)
                    : "r"(A[i][0]), "r"(A[i][1]), "r"(A[i][2]), "r"(A[i][3]), "r"(B[i][0]), "r"(B[i][1]), "r"(B[i][2]),
                      "r"(B[i][3]), "r"(e));
            }
            advance(4u);
        }
        for (; st < s_end; ++st) {
            step(bm_lds(v0_p), bm_lds(v0_p + v_half), 0u, 0u);
            advance(1u);
        }
        if (tig == 0) {  // column 0 of the tile: rows g (c0) and g + 8 (c2)
            red[warp * 16 + g] = c0;
            red[warp * 16 + g + 8] = c2;
        }
        __syncthreads();  // partial sums complete; everybody is done reading this stage
        const int valid = min(tr, I.rows - cur.row0);
        if (tid < valid) {
            const int rblk = tid >> 4, r = tid & 15;
            int acc = 0;
            for (int k = 0; k < ks; ++k) acc += red[((rblk << cur.ks_log2) + k) * 16 + r];
            I.y[cur.row0 + tid] = acc;
        }
        cur = nxt;
        // the next iteration writes `red` only after its own barrier, and that barrier comes after these reads
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Launch for a list whose items passed spb_gemv_batch_check; max_cols bounds the columns of any item.
int gemv_batch_mma_launch(const spb_gemv_item* d_items, int n, int max_rows, int max_cols, void* stream) {
    const char* name = "spb_sparse_ternary_gemv_batch(mma.sp)";
    (void)max_rows;
    // the largest slab any item of up to max_cols columns can have: check max_cols and the widest matrix of
    // every smaller ks class
    size_t slab = 0;
    auto consider = [&](int cols) {
        if (cols < 256 || cols > max_cols) return;
        const int steps = cols / 64, kl = steps >= 128 ? 3 : steps >= 64 ? 2 : steps >= 32 ? 1 : 0;
        const size_t b = static_cast<size_t>(128 >> kl) * (bm_pitch(cols / 32) + bm_pitch(cols / 64)) * 4;
        if (b > slab) slab = b;
    };
    consider(max_cols);
    consider(1792);  // widest multiples of 256 below 32, 64 and 128 steps
    consider(3840);
    consider(7936);
    BmGeom geo{};
    geo.x_off = static_cast<int>((slab + 15) & ~static_cast<size_t>(15));
    geo.stage_bytes = geo.x_off + max_cols;
    geo.max_cols = max_cols;
    const size_t smem = 2 * static_cast<size_t>(geo.stage_bytes);
    if (smem > 200 * 1024) return fail(SPB_E_UNSUPPORTED, "%s: %d columns need more shared memory than a block may take", name, max_cols);
    if (int rc = ensure_dynamic_smem(name, gemv_batch_mma_kernel, smem)) return rc;
    const size_t per_block = smem + 16 * 1024;  // + static shared memory (table, descriptors) and the reserve
    int per_sm = static_cast<int>((227 * 1024) / per_block);
    per_sm = per_sm < 1 ? 1 : per_sm > 3 ? 3 : per_sm;
    const int grid = per_sm * sm_count();
    for (int first = 0; first < n; first += kBmMaxItems) {
        const int count = n - first < kBmMaxItems ? n - first : kBmMaxItems;
        int rc = launch(name, gemv_batch_mma_kernel, dim3(grid), dim3(kBmThreads), smem, stream, d_items + first, count, geo);
        if (rc) return rc;
    }
    return SPB_OK;
}

}  // namespace spb

using namespace spb;

extern "C" int spb_gemv_batch_check(const spb_gemv_item* h_items, int n) {
    if (n < 0 || (n > 0 && !h_items)) return fail(SPB_E_INVALID, "spb_gemv_batch_check: bad list");
    for (int i = 0; i < n; ++i) {
        const spb_gemv_item& I = h_items[i];
        auto al = [](const void* p, size_t k) { return (reinterpret_cast<uintptr_t>(p) & (k - 1)) == 0; };
        if (I.rows <= 0 || I.cols <= 0 || I.cols % 256 != 0 || I.cols > 32768)
            return fail(SPB_E_UNSUPPORTED, "item %d: %dx%d (cols must be a multiple of 256, at most 32768)", i, I.rows,
                        I.cols);
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
    if (max_cols % 256 != 0 || max_cols > 32768)
        return fail(SPB_E_UNSUPPORTED, "%s: max_cols=%d (multiple of 256, at most 32768)", name, max_cols);
    if ((reinterpret_cast<uintptr_t>(d_items) & 15) != 0) return fail(SPB_E_INVALID, "%s: d_items must be 16-byte aligned", name);
    return gemv_batch_mma_launch(d_items, n, max_rows, max_cols, stream);
}
