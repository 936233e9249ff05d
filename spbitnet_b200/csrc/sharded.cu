// Row-sharded decode engine: one rank of a tensor-parallel group, one process per GPU.
//
// The reference is single-GPU (src/inference.cu); this is the one way its decode step partitions without a
// reduction, so that every integer accumulator and every half output stays bit-identical to the unsharded
// step: rank r owns a contiguous slice of the output rows of every ternary matrix (q/k/v by whole KV heads,
// so that RoPE, the KV cache and attention are local; o / gate / up / down by rows; the LM head by vocabulary
// rows), computes its slice with the ordinary kernels on the full activation vector, and the slices are
// concatenated on every rank.  Vector ops (norms, quantisation, residual adds) are replicated.  Four
// exchanges per layer (attention output, o_proj output, gate and up, down output) plus one per token for the
// arg-max candidates.
//
// The exchange is not a library collective.  Every rank exports one device buffer (CUDA IPC) and maps its
// peers'; an exchange is ONE kernel that
//   1. copies the rank's slice into the same place of every rank's buffer with ordinary stores through the
//      peer mappings (NVLink / NVSwitch), its own included,
//   2. fences (system scope) and, in the last block to finish, stores the exchange's sequence number into
//      its flag word on every peer,
//   3. waits until the local flag words of all peers have reached that sequence number, bounded by time:
//      when the bound runs out the kernel raises a status word that the host reads at its next
//      synchronisation (SPB_E_TIMEOUT), and every later exchange of the engine skips its wait.
// Slices of up to 96 KB per sender (every exchange of a batch-1 step) take a second form without the fence round
// trip: every 4 bytes travel as one 8-byte store {data, sequence number} into a per-sender staging area, the
// receiver polls each word until it carries the current number and moves the data into place (exchange_ll_kernel).
// In the single-sequence step of a wide model (hidden >= 4096) that second form needs no kernel of its own: the
// kernel that computes a slice (attention merge, prepared GEMV) stores the tagged words from its epilogue into every
// rank's staging area, its own included, and the kernel that consumes the gathered vector polls its local staging
// area as it loads (ll_gather8), so compute and exchange are one kernel on each side and the NVLink crossing
// overlaps the producer's tail (spb_shard_engine_set_exchange_fold; form 1 lets the consumer do the whole exchange).
// No multicast, no bulk-copy engine, no library kernel ever sees a peer pointer; remote data always lands in
// the consumer's own memory before anything reads it.  Sequence numbers only grow, so flags are never reset.
// A buffer is reused once per layer: a rank that writes exchange n into a peer has passed its wait of
// exchange n - 1, so that peer has issued everything up to exchange n - 1, which comes after its last read
// of this buffer's previous contents (four exchanges earlier).
//
// batch = 1 runs the fused GEMV launches of the single-GPU engine on the row slices (wide models: one vector kernel
// per activation, a cluster of eight blocks, and every matrix through the tensor-core GEMV, q / k / v and gate / up
// as one launch each on prepared copies of the slices); batch > 1 decodes that
// many independent sequences in lock step (same position, own KV caches) with the batched product
// (spb_sparse_bitlinear_gemm) and the row-batched vector kernels.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <new>
#include <vector>

#include "fused_ops.cuh"

namespace spb {

namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxBatch = 64;
enum { X_ATTN = 0, X_O = 1, X_GU = 2, X_DOWN = 3, X_AMAX = 4, X_KINDS = 5 };
constexpr size_t kFlagBytesPerKind = 64;

struct XSeg {
    const uint8_t* src;   // local compact slice: rows x len bytes
    uint32_t dst_off;     // byte offset of the slice inside every rank's exchange buffer (row 0)
    uint32_t dst_pitch;   // bytes between rows of the gathered array
    uint32_t len;         // bytes per row of this rank's slice (a multiple of 4)
};

struct XArgs {
    uint8_t* peer[kMaxWorld];  // exchange buffers of all ranks, peer[rank] = the local one
    XSeg seg[2];
    int nseg, rows, world, rank;
    uint32_t flag_off;              // byte offset of this kind's flag words in the exchange buffer
    unsigned* seqno;                // local: sequence number of this kind's last exchange
    unsigned* done;                 // local: blocks of the running exchange that have finished copying
    int* status;                    // pinned host word: 0 healthy, 1 a wait ran out
    int* broken;                    // the same fact in device memory (read by every later exchange)
    unsigned long long timeout_ns;  // bound of the wait
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <typename T>
__device__ __forceinline__ void xcopy(const XArgs& a, int tid_global, int nthreads) {
    constexpr int kUnroll = 4;  // loads of four pieces in flight per thread before the first store
    for (int s = 0; s < a.nseg; ++s) {
        const XSeg& g = a.seg[s];
        const uint32_t per_row = g.len / sizeof(T);
        const uint32_t total = per_row * static_cast<uint32_t>(a.rows);
        for (uint32_t i0 = tid_global; i0 < total; i0 += kUnroll * nthreads) {
            T v[kUnroll];
            size_t o[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const uint32_t i = i0 + u * nthreads;
                if (i < total) {
                    const uint32_t row = a.rows == 1 ? 0u : i / per_row, c = i - row * per_row;
                    v[u] = reinterpret_cast<const T*>(g.src + static_cast<size_t>(row) * g.len)[c];
                    o[u] = static_cast<size_t>(g.dst_off) + static_cast<size_t>(row) * g.dst_pitch + static_cast<size_t>(c) * sizeof(T);
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u)
                if (i0 + u * nthreads < total)
                    for (int p = 0; p < a.world; ++p) *reinterpret_cast<T*>(a.peer[p] + o[u]) = v[u];
        }
    }
}

// WIDE: every length, offset and pitch is a multiple of 16 bytes (16-byte copies), else 4-byte copies.
template <bool WIDE>
__global__ void __launch_bounds__(256) exchange_kernel(const XArgs a) {
    __shared__ unsigned s_last, s_seq;
    grid_dep_launch();
    grid_dep_wait();  // the slice was written by the predecessor
    const int tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
    if (WIDE) xcopy<uint4>(a, tid, nthreads);
    else xcopy<uint32_t>(a, tid, nthreads);
    __threadfence_system();  // every thread's stores are ordered before what follows its barrier arrival
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned ticket = gridDim.x == 1 ? 0u : atomicAdd(a.done, 1u);
        s_last = ticket == gridDim.x - 1 ? 1u : 0u;
        if (s_last) {
            if (gridDim.x > 1) {
                *a.done = 0;
                __threadfence();  // the other blocks' stores (ordered before their tickets) before the flags below
            }
            s_seq = *a.seqno + 1;
            *a.seqno = s_seq;
        }
    }
    __syncthreads();
    if (!s_last) return;
    const unsigned seq = s_seq;
    const int p = threadIdx.x;
    if (p < a.world && p != a.rank) {
        st_release_sys(reinterpret_cast<unsigned*>(a.peer[p] + a.flag_off) + a.rank, seq);
        const unsigned* mine = reinterpret_cast<const unsigned*>(a.peer[a.rank] + a.flag_off) + p;
        if (*reinterpret_cast<volatile int*>(a.broken) == 0) {
            const unsigned long long t0 = globaltimer_ns();
            for (;;) {
                // sequence numbers only grow; the subtraction keeps the comparison right across a wrap
                if (static_cast<int>(ld_acquire_sys(mine) - seq) >= 0) break;
                if (globaltimer_ns() - t0 > a.timeout_ns) {
                    *reinterpret_cast<volatile int*>(a.broken) = 1;
                    atomicExch_system(a.status, 1);
                    break;
                }
                __nanosleep(64);
            }
        }
    }
}

// The small-message form of the exchange.  The fenced form above pays a system-scope fence round trip between
// the data and the flag; for slices of a few kilobytes that round trip is most of the exchange.  Here every
// 4 bytes of data travel as ONE 8-byte store {data, sequence number} into a per-sender staging area of the
// receiver's buffer (8-byte stores arrive whole), so the data is its own flag: the receiver polls each word until
// it carries the current sequence number and moves the data into the gathered array.  One NVLink crossing, no
// fence, twice the bytes.  Sequence numbers grow by one per exchange of a kind, so a slot's previous contents
// (number - 1, or 0 after allocation) never look current.  The poll is bounded by time like the flag wait.
struct LSeg {
    const uint8_t* src;       // local compact slice: rows x len[rank] bytes
    uint32_t dst_region;      // byte offset of the gathered array in the exchange buffer
    uint32_t dst_pitch;       // bytes between its rows
    uint32_t off[kMaxWorld];  // byte offset of every rank's slice inside a row
    uint32_t len[kMaxWorld];  // bytes per row of every rank's slice (multiples of 4)
    uint32_t ll_off;          // byte offset of this segment's staging area in the exchange buffer
    uint32_t ll_stride;       // bytes of staging per sending rank
};
struct LArgs {
    uint8_t* peer[kMaxWorld];
    LSeg seg[2];
    int nseg, rows, world, rank;
    int direct;                     // the producers already stored the words into the staging areas (their epilogues):
                                    // the consumer reads its vector from there (ll_gather8), nothing is sent or copied
    const uint8_t* self;            // this rank's exchange buffer (peer[rank])
    unsigned* seqno;
    unsigned* done;
    int* status;
    int* broken;
    unsigned long long timeout_ns;
};

// Send and receive of one small-message exchange by `nthreads` threads (this one is number `tid`).  A thread keeps
// eight words in flight, both ways: one word at a time, every poll would be a dependent trip to L2.
__device__ __forceinline__ void exchange_ll_run(const LArgs& a, uint32_t tid, uint32_t nthreads, unsigned seq) {
    constexpr int kU = 8;
    // send: this rank's words, to its own gathered array directly and to every peer's staging area with the number
    for (int s = 0; s < a.nseg; ++s) {
        const LSeg& g = a.seg[s];
        const uint32_t wpr = g.len[a.rank] >> 2, words = wpr * static_cast<uint32_t>(a.rows);
        for (uint32_t j0 = tid; j0 < words; j0 += kU * nthreads) {
            uint32_t v[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const uint32_t j = j0 + u * nthreads;
                v[u] = j < words ? reinterpret_cast<const uint32_t*>(g.src)[j] : 0u;
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const uint32_t j = j0 + u * nthreads;
                if (j >= words) continue;
                const uint32_t row = a.rows == 1 ? 0u : j / wpr, c = j - row * wpr;
                *reinterpret_cast<uint32_t*>(a.peer[a.rank] + g.dst_region + static_cast<size_t>(row) * g.dst_pitch + g.off[a.rank] + 4u * c) = v[u];
                const size_t slot = static_cast<size_t>(g.ll_off) + static_cast<size_t>(a.rank) * g.ll_stride + 8u * static_cast<size_t>(j);
                for (int p = 0; p < a.world; ++p)
                    if (p != a.rank)
                        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(a.peer[p] + slot), "r"(v[u]), "r"(seq) : "memory");
            }
        }
    }
    // receive: every peer's words out of the local staging area
    bool alive = *reinterpret_cast<volatile int*>(a.broken) == 0;
    unsigned long long t0 = 0;
    for (int s = 0; s < a.nseg && alive; ++s) {
        const LSeg& g = a.seg[s];
        for (int p = 0; p < a.world && alive; ++p) {
            if (p == a.rank) continue;
            const uint32_t wpr = g.len[p] >> 2, words = wpr * static_cast<uint32_t>(a.rows);
            const uint8_t* stage = a.peer[a.rank] + g.ll_off + static_cast<size_t>(p) * g.ll_stride;
            for (uint32_t j0 = tid; j0 < words && alive; j0 += kU * nthreads) {
                unsigned pending = 0;
#pragma unroll
                for (int u = 0; u < kU; ++u)
                    if (j0 + u * nthreads < words) pending |= 1u << u;
                unsigned spins = 0;
                while (pending) {
                    uint32_t v[kU], n[kU];
#pragma unroll
                    for (int u = 0; u < kU; ++u)
                        if ((pending >> u) & 1u)
                            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v[u]), "=r"(n[u]) : "l"(stage + 8u * static_cast<size_t>(j0 + u * nthreads)) : "memory");
#pragma unroll
                    for (int u = 0; u < kU; ++u)
                        if (((pending >> u) & 1u) && n[u] == seq) {
                            const uint32_t j = j0 + u * nthreads;
                            const uint32_t row = a.rows == 1 ? 0u : j / wpr, c = j - row * wpr;
                            *reinterpret_cast<uint32_t*>(a.peer[a.rank] + g.dst_region + static_cast<size_t>(row) * g.dst_pitch + g.off[p] + 4u * c) = v[u];
                            pending &= ~(1u << u);
                        }
                    if (pending && (++spins & 255u) == 0) {
                        const unsigned long long now = globaltimer_ns();
                        if (t0 == 0) t0 = now;
                        if (now - t0 > a.timeout_ns || *reinterpret_cast<volatile int*>(a.broken) != 0) {
                            *reinterpret_cast<volatile int*>(a.broken) = 1;
                            atomicExch_system(a.status, 1);
                            alive = false;
                            break;
                        }
                    }
                }
            }
        }
    }
}

__global__ void __launch_bounds__(256) exchange_ll_kernel(const LArgs a) {
    grid_dep_launch();
    grid_dep_wait();  // the slice was written by the predecessor
    const unsigned seq = *reinterpret_cast<volatile unsigned*>(a.seqno) + 1u;
    exchange_ll_run(a, blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x, seq);
    // the last block to finish advances the sequence number (every block has read it by then)
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned ticket = gridDim.x == 1 ? 0u : atomicAdd(a.done, 1u);
        if (ticket == gridDim.x - 1) {
            if (gridDim.x > 1) *a.done = 0;
            *a.seqno = seq;
        }
    }
}

// Direct form (a.direct): elements 8 run .. 8 run + 7 of gathered vector `seg`, read as four tagged words from the
// staging area of the rank that owns them (slices are multiples of 8 elements, so a run has one owner).  The poll is
// bounded like every wait for a peer; when it runs out the status is raised and the data is whatever was there.
__device__ __forceinline__ uint4 ll_gather8(const LArgs& a, int seg, int run, unsigned seq, bool& alive) {
    const LSeg& g = a.seg[seg];
    const uint32_t byte = 16u * static_cast<uint32_t>(run);
    uint32_t owner = 0, first = 0;
#pragma unroll
    for (int p = 0; p < kMaxWorld; ++p)
        if (p < a.world && byte >= g.off[p] && byte < g.off[p] + g.len[p]) {
            owner = p;
            first = g.off[p];
        }
    const uint8_t* src = a.self + g.ll_off + static_cast<size_t>(owner) * g.ll_stride + 2u * static_cast<size_t>(byte - first);
    uint32_t d0, t0, d1, t1, d2, t2, d3, t3;
    unsigned spins = 0;
    unsigned long long started = 0;
    for (;;) {
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(d0), "=r"(t0), "=r"(d1), "=r"(t1) : "l"(src) : "memory");
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(d2), "=r"(t2), "=r"(d3), "=r"(t3) : "l"(src + 16) : "memory");
        if ((t0 == seq && t1 == seq && t2 == seq && t3 == seq) || !alive) break;
        if ((++spins & 255u) == 0) {
            const unsigned long long now = globaltimer_ns();
            if (started == 0) started = now;
            if (now - started > a.timeout_ns || *reinterpret_cast<volatile int*>(a.broken) != 0) {
                *reinterpret_cast<volatile int*>(a.broken) = 1;
                atomicExch_system(a.status, 1);
                alive = false;
            }
        }
    }
    return make_uint4(d0, d1, d2, d3);
}
// What a kernel that consumes gathered vectors does first: nothing (one rank, or an exchange launch ran before it),
// the whole exchange (a.world > 1, single block), or only the bookkeeping of the direct form.  Returns the sequence
// number of the exchange.
__device__ __forceinline__ unsigned consumer_exchange_begin(const LArgs& a, bool& alive) {
    if (a.world <= 1) return 0u;
    const unsigned seq = *reinterpret_cast<volatile unsigned*>(a.seqno) + 1u;
    if (a.direct) {
        alive = *reinterpret_cast<volatile int*>(a.broken) == 0;
        return seq;
    }
    exchange_ll_run(a, threadIdx.x, blockDim.x, seq);
    __syncthreads();
    if (threadIdx.x == 0) *a.seqno = seq;
    return seq;
}

// token of sequence b: prompt[pos * batch + b] while pos < n_prompt, else next[b]; row copy of the embedding
__global__ void __launch_bounds__(256) shard_embed_kernel(const __half* __restrict__ embed, __half* __restrict__ x,
                                                          int hidden, const int* __restrict__ d_prompt, int n_prompt,
                                                          const int* __restrict__ d_next, const int* __restrict__ d_pos,
                                                          int batch) {
    grid_dep_launch();
    grid_dep_wait();
    const int b = blockIdx.y, pos = *d_pos;
    const int token = (d_prompt && pos < n_prompt) ? d_prompt[pos * batch + b] : d_next[b];
    const uint4* row = reinterpret_cast<const uint4*>(embed + static_cast<size_t>(token) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(x + static_cast<size_t>(b) * hidden);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden / 8; i += gridDim.x * blockDim.x) dst[i] = row[i];
}

// First maximum of the rank's logits (std::max_element order), two stages.  Stage 1: block (x, b) scans a strided
// share of sequence b's row and leaves one candidate (value, local index).  Stage 2: block b folds the candidates of
// sequence b into (value, global index).
__device__ __forceinline__ void argmax_take(float& a, int& ai, float b, int bi) {
    if (bi != 0x7FFFFFFF && (ai == 0x7FFFFFFF || b > a || (b == a && bi < ai))) { a = b; ai = bi; }
}
__device__ __forceinline__ void argmax_block_fold(float& best, int& besti, float* sv, int* si) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
        argmax_take(best, besti, __shfl_xor_sync(0xFFFFFFFFu, best, off), __shfl_xor_sync(0xFFFFFFFFu, besti, off));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = besti; }
    __syncthreads();
    if (warp == 0) {
        best = lane < nw ? sv[lane] : -INFINITY;
        besti = lane < nw ? si[lane] : 0x7FFFFFFF;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
            argmax_take(best, besti, __shfl_xor_sync(0xFFFFFFFFu, best, off), __shfl_xor_sync(0xFFFFFFFFu, besti, off));
    }
}
__global__ void __launch_bounds__(1024) shard_argmax1_kernel(const float* __restrict__ logits, int n, float* __restrict__ cand) {
    __shared__ float sv[32];
    __shared__ int si[32];
    grid_dep_launch();
    grid_dep_wait();
    const float* v = logits + static_cast<size_t>(blockIdx.y) * n;
    float best = -INFINITY;
    int besti = 0x7FFFFFFF;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float x = v[i];
        if (besti == 0x7FFFFFFF || x > best) {  // i grows: a later equal value never replaces an earlier one
            best = x;
            besti = i;
        }
    }
    argmax_block_fold(best, besti, sv, si);
    if (threadIdx.x == 0) {
        float* c = cand + 2 * (static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x);
        c[0] = best;
        reinterpret_cast<int*>(c)[1] = besti;
    }
}
__global__ void __launch_bounds__(128) shard_argmax2_kernel(const float* __restrict__ cand, int nblocks, int index0,
                                                            float* __restrict__ out_pairs) {
    __shared__ float sv[32];
    __shared__ int si[32];
    grid_dep_launch();
    grid_dep_wait();
    const float* c = cand + 2 * static_cast<size_t>(blockIdx.x) * nblocks;
    float best = -INFINITY;
    int besti = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < nblocks; i += blockDim.x) argmax_take(best, besti, c[2 * i], reinterpret_cast<const int*>(c)[2 * i + 1]);
    argmax_block_fold(best, besti, sv, si);
    if (threadIdx.x == 0) {
        out_pairs[2 * blockIdx.x] = best;
        reinterpret_cast<int*>(out_pairs)[2 * blockIdx.x + 1] = besti == 0x7FFFFFFF ? besti : besti + index0;
    }
}

// Thread b: the first maximum over the ranks' candidates of sequence b (ranks hold ascending vocabulary ranges, so
// the lowest rank wins ties), published as the next token; thread 0 then advances the position.
__global__ void __launch_bounds__(kMaxBatch) shard_pick_kernel(const float* __restrict__ pairs, int world, int batch,
                                                               int* __restrict__ d_next, int* __restrict__ d_out,
                                                               int* __restrict__ d_pos) {
    grid_dep_launch();
    grid_dep_wait();
    const int b = threadIdx.x, pos = *d_pos;
    if (b < batch) {
        float best = -INFINITY;
        int besti = 0x7FFFFFFF;
        for (int r = 0; r < world; ++r) {
            const float v = pairs[(static_cast<size_t>(b) * world + r) * 2];
            const int i = reinterpret_cast<const int*>(pairs)[(static_cast<size_t>(b) * world + r) * 2 + 1];
            if (i != 0x7FFFFFFF && (besti == 0x7FFFFFFF || v > best)) { best = v; besti = i; }
        }
        d_next[b] = besti;
        if (d_out) d_out[static_cast<size_t>(pos) * batch + b] = besti;
    }
    __syncthreads();
    if (b == 0) *d_pos = pos + 1;
}

// LM head for a batch: logits[b][r] = sum_k W[r][k] * x[b][k], fp16 inputs, fp32 accumulation on the warp-level
// tensor-core MMA (m16n8k16).  A warp owns 16 rows of W and all NT * 8 batch columns; per 32 columns every lane
// reads 16 bytes of its two rows and of each batch column it serves.  Which four of a lane's eight values go
// into which MMA step is the same for W and x, so the products pair up correctly (a dot product does not care
// about the order of its terms; the fp32 sums differ from a sequential loop in the last bits only).
template <int NT>
__global__ void __launch_bounds__(128) half_gemm_rows_kernel(const __half* __restrict__ W, const __half* __restrict__ x,
                                                             float* __restrict__ y, int rows, int cols, int batch) {
    grid_dep_launch();
    grid_dep_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tig = lane & 3;
    const int row0 = (blockIdx.x * 4 + warp) * 16;
    if (row0 >= rows) return;
    const int ra = row0 + g, rb = row0 + g + 8;
    const uint4* wa = reinterpret_cast<const uint4*>(W + static_cast<size_t>(min(ra, rows - 1)) * cols) + tig;
    const uint4* wb = reinterpret_cast<const uint4*>(W + static_cast<size_t>(min(rb, rows - 1)) * cols) + tig;
    const uint4* xp[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) xp[j] = reinterpret_cast<const uint4*>(x + static_cast<size_t>(min(8 * j + g, batch - 1)) * cols) + tig;
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    for (int k = 0; k < cols / 32; ++k) {
        const uint4 a = ld_stream_v4(reinterpret_cast<const uint32_t*>(wa + 4 * k));
        const uint4 b = ld_stream_v4(reinterpret_cast<const uint32_t*>(wb + 4 * k));
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const uint4 v = __ldg(xp[j] + 4 * k);
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3])
                         : "r"(a.x), "r"(b.x), "r"(a.y), "r"(b.y), "r"(v.x), "r"(v.y));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3])
                         : "r"(a.z), "r"(b.z), "r"(a.w), "r"(b.w), "r"(v.z), "r"(v.w));
        }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int n0 = 8 * j + 2 * tig;
        if (n0 < batch) {
            if (ra < rows) y[static_cast<size_t>(n0) * rows + ra] = acc[j][0];
            if (rb < rows) y[static_cast<size_t>(n0) * rows + rb] = acc[j][2];
        }
        if (n0 + 1 < batch) {
            if (ra < rows) y[static_cast<size_t>(n0 + 1) * rows + ra] = acc[j][1];
            if (rb < rows) y[static_cast<size_t>(n0 + 1) * rows + rb] = acc[j][3];
        }
    }
}

// ---- vector ops for wide models -------------------------------------------------------------------------
// The same arithmetic as residual_norm_quant / relu2_norm_quant / absmax_quantize_rows (fused_ops.cu, prefill.cu:
// every rounding point of the reference's op sequence), laid out for vectors of 4096 .. 32768 elements: one block
// of 1024 threads per vector, every thread keeps its elements (up to four runs of eight) in registers, all loads
// are issued before the first reduction, so a kernel costs one memory round trip plus two or three block
// reductions instead of five passes over shared memory.  Only the order in which the squares are summed differs
// from the narrow kernels (both are fp32 sums of the same terms).
constexpr int kWideThreads = 1024;
constexpr int kWideRuns = 4;  // runs of eight elements per thread: vectors of up to 32768

// Block-wide sum / maximum over 1024 threads.  The 1024 threads are either one block (CL = 1) or a cluster of CL
// blocks of 1024 / CL threads, in which a thread's number is rank * (1024 / CL) + threadIdx.x; the arithmetic is the
// same in both forms (warp tree, then a tree over the 32 warp results in warp order), so the results are too.  In the
// cluster form every warp stores its result into slot (its number among the 32 warps) of `sh` in EVERY block of the
// cluster (distributed shared memory) and a cluster barrier stands where the block barrier stood.  `sh` is used once
// per kernel: nothing is overwritten while a slower block still reads.
__device__ __forceinline__ uint32_t wide_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
template <int CL>
__device__ __forceinline__ int wide_tid() {
    return CL == 1 ? static_cast<int>(threadIdx.x) : static_cast<int>(wide_cluster_rank() * (kWideThreads / CL) + threadIdx.x);
}
template <int CL>
__device__ __forceinline__ void wide_share(float v, float* sh) {
    if (CL == 1) {
        __syncthreads();
        if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
        __syncthreads();
    } else {
        if ((threadIdx.x & 31) == 0) {
            const uint32_t slot = wide_cluster_rank() * (kWideThreads / CL / 32) + (threadIdx.x >> 5);
            const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(sh + slot));
#pragma unroll
            for (int c = 0; c < CL; ++c) {
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(c));
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
}
template <int CL>
__device__ __forceinline__ float wide_bsum(float v, float* sh) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    wide_share<CL>(v, sh);
    v = sh[threadIdx.x & 31];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}
template <int CL>
__device__ __forceinline__ float wide_bmax(float v, float* sh) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    wide_share<CL>(v, sh);
    v = sh[threadIdx.x & 31];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    return v;
}
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ void load8f(const float* p, float* f) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void quantise_store8(const float* v, float qs, int8_t* dst) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        lo |= (static_cast<uint32_t>(quantize_one(v[i], qs)) & 0xFFu) << (8 * i);
        hi |= (static_cast<uint32_t>(quantize_one(v[4 + i], qs)) & 0xFFu) << (8 * i);
    }
    *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
}

// residual_norm_quant for one vector per block (blockIdx.x = vector): x += [rms_norm(sub_w)](delta) in half, then
// xn = rms_norm(w)(x) in half (to xn_out when given), absmax, int8.  n % 8 == 0, n <= 8192: one run of eight
// elements per thread, everything in registers.
template <int CL>
__global__ void __launch_bounds__(kWideThreads / CL) wide_residual_norm_quant_kernel(
    const __half* delta, const float* __restrict__ sub_w, __half* __restrict__ x, const float* __restrict__ w,
    __half* __restrict__ xn_out, int8_t* __restrict__ xq, float* __restrict__ d_absmax, int n, float eps, const LArgs xin) {
    __shared__ float sh[3][32];
    const int vt = wide_tid<CL>(), vec = blockIdx.x / CL;
    grid_dep_launch();
    grid_dep_wait();
    bool alive = true;
    const unsigned xseq = consumer_exchange_begin(xin, alive);  // delta is gathered from the ranks' slices
    const bool direct = xin.world > 1 && xin.direct;
    const size_t off = static_cast<size_t>(vec) * n;
    const int runs = n >> 3;
    constexpr int kRuns = 1;
    float v[kRuns][8], wv[kRuns][8];
    float s = 0.0f;
    if (delta) {
        float d[kRuns][8], sw[kRuns][8];
#pragma unroll
        for (int k = 0; k < kRuns; ++k) {
            const int r = vt + k * kWideThreads;
            if (r < runs) {
                unpack8(direct ? ll_gather8(xin, 0, r, xseq, alive) : *reinterpret_cast<const uint4*>(delta + off + 8 * r), d[k]);
                unpack8(*reinterpret_cast<const uint4*>(x + off + 8 * r), v[k]);
                load8f(w + 8 * r, wv[k]);
                if (sub_w) load8f(sub_w + 8 * r, sw[k]);
#pragma unroll
                for (int i = 0; i < 8; ++i) s += d[k][i] * d[k][i];
            }
        }
        float sub_scale = 1.0f;
        if (sub_w) sub_scale = rsqrtf(wide_bsum<CL>(s, sh[0]) / static_cast<float>(n) + eps);
        s = 0.0f;
#pragma unroll
        for (int k = 0; k < kRuns; ++k) {
            const int r = vt + k * kWideThreads;
            if (r < runs) {
                __half2 out[4];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float dd = d[k][i];
                    if (sub_w) dd = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(dd, sub_scale), sw[k][i])));
                    const __half h = __float2half_rn(dd + v[k][i]);
                    reinterpret_cast<__half*>(out)[i] = h;
                    v[k][i] = __half2float(h);
                    s += v[k][i] * v[k][i];
                }
                *reinterpret_cast<uint4*>(x + off + 8 * r) = *reinterpret_cast<const uint4*>(out);
            }
        }
    } else {
#pragma unroll
        for (int k = 0; k < kRuns; ++k) {
            const int r = vt + k * kWideThreads;
            if (r < runs) {
                unpack8(*reinterpret_cast<const uint4*>(x + off + 8 * r), v[k]);
                load8f(w + 8 * r, wv[k]);
#pragma unroll
                for (int i = 0; i < 8; ++i) s += v[k][i] * v[k][i];
            }
        }
    }
    const float scale = rsqrtf(wide_bsum<CL>(s, sh[1]) / static_cast<float>(n) + eps);
    float m = 0.0f;
#pragma unroll
    for (int k = 0; k < kRuns; ++k) {
        const int r = vt + k * kWideThreads;
        if (r < runs) {
            __half2 out[4];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const __half h = __float2half_rn(__fmul_rn(__fmul_rn(v[k][i], scale), wv[k][i]));
                reinterpret_cast<__half*>(out)[i] = h;
                v[k][i] = __half2float(h);
                m = fmaxf(m, fabsf(v[k][i]));
            }
            if (xn_out) *reinterpret_cast<uint4*>(xn_out + off + 8 * r) = *reinterpret_cast<const uint4*>(out);
        }
    }
    const float absmax = wide_bmax<CL>(m, sh[2]);
    if (vt == 0) d_absmax[vec] = absmax;
    if (direct && vt == 0) *xin.seqno = xseq;  // every thread read the number before the reduction above
    const float qs = quant_scale(absmax);
#pragma unroll
    for (int k = 0; k < kRuns; ++k) {
        const int r = vt + k * kWideThreads;
        if (r < runs) quantise_store8(v[k], qs, xq + off + 8 * r);
    }
}

// relu2_norm_quant for one vector per block: m = relu(gate)^2 * up in fp32, h = half(m * rsqrt(mean m^2 + eps) * sub_w)
// (or half(m) without sub_w), absmax, int8.
template <int CL>
__global__ void __launch_bounds__(kWideThreads / CL) wide_relu2_norm_quant_kernel(
    const __half* gate, const __half* up, const float* __restrict__ sub_w, int8_t* __restrict__ hq,
    float* __restrict__ d_absmax, int n, float eps, const LArgs xin) {
    __shared__ float sh[2][32];
    const int vt = wide_tid<CL>(), vec = blockIdx.x / CL;
    grid_dep_launch();
    const int runs = n >> 3;
    // sub_w is read after the reduction, when it is needed (no registers to hold it until then); it is constant, so its
    // lines are brought into L1 before the dependency wait and the later read does not go to L2
    if (sub_w)
#pragma unroll
        for (int k = 0; k < kWideRuns; ++k) {
            const int r = vt + k * kWideThreads;
            if (r < runs) asm volatile("prefetch.global.L1 [%0];" ::"l"(sub_w + 8 * r));
        }
    grid_dep_wait();
    bool alive = true;
    const unsigned xseq = consumer_exchange_begin(xin, alive);  // gate and up are gathered from the ranks' slices
    const bool direct = xin.world > 1 && xin.direct;
    const size_t off = static_cast<size_t>(vec) * n;
    float v[kWideRuns][8];  // the products stay in registers
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < kWideRuns; ++k) {
        const int r = vt + k * kWideThreads;
        if (r < runs) {
            float g[8], u[8];
            unpack8(direct ? ll_gather8(xin, 0, r, xseq, alive) : *reinterpret_cast<const uint4*>(gate + off + 8 * r), g);
            unpack8(direct ? ll_gather8(xin, 1, r, xseq, alive) : *reinterpret_cast<const uint4*>(up + off + 8 * r), u);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float t = fmaxf(0.0f, g[i]);
                v[k][i] = __fmul_rn(__fmul_rn(t, t), u[i]);
                s += v[k][i] * v[k][i];
            }
        }
    }
    float scale = 1.0f;
    if (sub_w) scale = rsqrtf(wide_bsum<CL>(s, sh[0]) / static_cast<float>(n) + eps);
    float m = 0.0f;
#pragma unroll
    for (int k = 0; k < kWideRuns; ++k) {
        const int r = vt + k * kWideThreads;
        if (r < runs) {
            float sw[8];
            if (sub_w) load8f(sub_w + 8 * r, sw);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const __half h = sub_w ? __float2half_rn(__fmul_rn(__fmul_rn(v[k][i], scale), sw[i])) : __float2half_rn(v[k][i]);
                v[k][i] = __half2float(h);
                m = fmaxf(m, fabsf(v[k][i]));
            }
        }
    }
    const float absmax = wide_bmax<CL>(m, sh[1]);
    if (vt == 0) d_absmax[vec] = absmax;
    if (direct && vt == 0) *xin.seqno = xseq;  // every thread read the number before the reduction above
    const float qs = quant_scale(absmax);
#pragma unroll
    for (int k = 0; k < kWideRuns; ++k) {
        const int r = vt + k * kWideThreads;
        if (r < runs) quantise_store8(v[k], qs, hq + off + 8 * r);
    }
}

// absmax_quantize_gpu for one vector per block.
template <int CL>
__global__ void __launch_bounds__(kWideThreads / CL) wide_absmax_quantize_kernel(const __half* in, int8_t* __restrict__ out,
                                                                            float* __restrict__ d_absmax, int n, const LArgs xin) {
    __shared__ float sh[32];
    const int vt = wide_tid<CL>(), vec = blockIdx.x / CL;
    grid_dep_launch();
    grid_dep_wait();
    bool alive = true;
    const unsigned xseq = consumer_exchange_begin(xin, alive);
    const bool direct = xin.world > 1 && xin.direct;
    const size_t off = static_cast<size_t>(vec) * n;
    const int runs = n >> 3;
    float v[kWideRuns][8];
    float m = 0.0f;
#pragma unroll
    for (int k = 0; k < kWideRuns; ++k) {
        const int r = vt + k * kWideThreads;
        if (r < runs) {
            unpack8(direct ? ll_gather8(xin, 0, r, xseq, alive) : *reinterpret_cast<const uint4*>(in + off + 8 * r), v[k]);
#pragma unroll
            for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[k][i]));
        }
    }
    const float absmax = wide_bmax<CL>(m, sh);
    if (vt == 0) d_absmax[vec] = absmax;
    if (direct && vt == 0) *xin.seqno = xseq;  // every thread read the number before the reduction above
    const float qs = quant_scale(absmax);
#pragma unroll
    for (int k = 0; k < kWideRuns; ++k) {
        const int r = vt + k * kWideThreads;
        if (r < runs) quantise_store8(v[k], qs, out + off + 8 * r);
    }
}

// launch() with thread-block clusters of `cluster` blocks along x (and programmatic dependent launch as usual)
template <typename... KArgs, typename... Args>
int launch_clustered(const char* name, void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster, void* stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "%s: launch failed: %s", name, cudaGetErrorString(err));
    }
    return SPB_OK;
}
constexpr int kWideCluster = 8;  // blocks that share one vector of the single-sequence step

int half_gemm_rows(const __half* W, const __half* x, float* y, int rows, int cols, int batch, void* stream) {
    if (cols % 32 || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(x) & 15))
        return fail(SPB_E_UNSUPPORTED, "batched lm_head: hidden size must be a multiple of 32 and rows 16-byte aligned");
    const dim3 grid((rows + 63) / 64), block(128);
    const int nt = (batch + 7) / 8;
    if (nt <= 1) return launch("half_gemm_rows", half_gemm_rows_kernel<1>, grid, block, 0, stream, W, x, y, rows, cols, batch);
    if (nt <= 2) return launch("half_gemm_rows", half_gemm_rows_kernel<2>, grid, block, 0, stream, W, x, y, rows, cols, batch);
    if (nt <= 4) return launch("half_gemm_rows", half_gemm_rows_kernel<4>, grid, block, 0, stream, W, x, y, rows, cols, batch);
    return launch("half_gemm_rows", half_gemm_rows_kernel<8>, grid, block, 0, stream, W, x, y, rows, cols, batch);
}

struct Linear {
    const uint32_t* meta = nullptr;
    const uint32_t* values = nullptr;
    float gamma = 0.0f;
    int rows = 0, cols = 0, ms = 0, vs = 0;
    void* prep = nullptr;  // the slice re-laid for the tensor-core GEMV (gemv_prepared.cu), owned by the engine; or null
};
struct Layer {
    Linear lin[7];              // q k v o gate up down: this rank's row slices
    const float* norm[4] = {};  // input_ln, post_attn_ln, attn_sub_norm, ffn_sub_norm (full vectors)
};

void split_range(int units, int world, int rank, int multiple, int* start, int* stop) {
    const int n = units / multiple, base = n / world, extra = n % world;
    const int a = rank * base + std::min(rank, extra);
    *start = a * multiple;
    *stop = (a + base + (rank < extra ? 1 : 0)) * multiple;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int cuda_fail(const char* what, cudaError_t err) {
    cudaGetLastError();
    return fail(SPB_E_CUDA, "%s: %s", what, cudaGetErrorString(err));
}
#define SPB_CUDA(call)                                            \
    do {                                                          \
        cudaError_t err__ = (call);                               \
        if (err__ != cudaSuccess) return cuda_fail(#call, err__); \
    } while (0)

BitLinearGroup make_group(const Linear* const* L, __half* const* out, int n) {
    BitLinearGroup g{};
    g.nmat = n;
    g.cols = L[0]->cols;
    for (int i = 0; i < n; ++i) {
        g.meta[i] = L[i]->meta; g.values[i] = L[i]->values; g.out[i] = out[i]; g.gamma[i] = L[i]->gamma;
        g.rows[i] = L[i]->rows; g.ms[i] = L[i]->ms; g.vs[i] = L[i]->vs;
    }
    return g;
}

}  // namespace
}  // namespace spb

using namespace spb;

struct spb_shard_engine {
    spb_model_config cfg{};
    int rank = 0, world = 1, batch = 1, device = 0;
    std::vector<Layer> layers;
    const __half* embed = nullptr;
    const __half* lm_head_loc = nullptr;  // this rank's vocabulary rows
    const float* final_norm = nullptr;

    // the split: [start, stop) per rank
    int kv0[kMaxWorld + 1] = {}, hrow[kMaxWorld + 1] = {}, irow[kMaxWorld + 1] = {}, vrow[kMaxWorld + 1] = {};
    int group_heads = 1;
    int nkv_loc = 0, nh_loc = 0, h_loc = 0, i_loc = 0, v_loc = 0;

    cudaStream_t stream = nullptr;
    cudaStream_t side[2] = {nullptr, nullptr};  // parallel branches of the captured step
    cudaEvent_t fork = nullptr, join[2] = {nullptr, nullptr};
    uint8_t* pool = nullptr;
    size_t kv_layer_bytes = 0;  // one layer's K (or V) caches of all sequences
    size_t seq_stride = 0;      // elements between the caches of two sequences
    __half *kcache = nullptr, *vcache = nullptr;
    __half *x = nullptr, *x2 = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *o = nullptr;
    __half *gate = nullptr, *up = nullptr, *down = nullptr, *xfinal = nullptr;
    int8_t* xq = nullptr;
    unsigned* attn_counters = nullptr;  // per local KV head: attention chunks written so far (zero between launches)
    float *absmax = nullptr, *attn_scratch = nullptr, *logits = nullptr, *pairs = nullptr, *cand = nullptr;
    int argmax_blocks = 1;
    int32_t* acc = nullptr;  // three int32 workspaces for the SIMT form of the batched product
    size_t acc_third = 0;
    int *d_pos = nullptr, *d_next = nullptr, *d_prompt = nullptr, *d_out = nullptr;
    unsigned* counters = nullptr;  // [X_KINDS][2]: seqno, done
    int prompt_cap = 0, n_prompt_in_graph = 0, out_cap = 0;
    bool split_attention = false, fused = false, wide = false;
    int use_prepared = 1;  // wide form, one sequence: GEMVs on weights re-laid at set_linear (1 large slices, 2 every slice, 0 none)

    // exchange buffer (exported through CUDA IPC) and the peers' mappings
    uint8_t* xbuf = nullptr;
    size_t xbuf_bytes = 0;
    uint8_t* peer[kMaxWorld] = {};
    bool peers_set = false;
    size_t off_flags = 0, off_attn = 0, off_o = 0, off_gate = 0, off_up = 0, off_down = 0, off_amax = 0;
    size_t ll_off[X_KINDS] = {};   // staging areas of the small-message exchange
    bool ll_ok[X_KINDS] = {};      // the kind's slices are small enough for it
    int fold_exchange = 2;         // wide single-sequence step: 0 exchanges are launches, 1 the consumer kernel of a vector
                                   // performs its exchange, 2 the producer's epilogue sends and the consumer receives
    int ident[kMaxWorld + 1] = {0, 1, 2, 3, 4, 5, 6, 7, 8};
    int* status = nullptr;  // pinned, mapped
    unsigned long long timeout_ns = 5000000000ull;

    cudaGraphExec_t graph = nullptr;
    bool graph_records = false;
    int seq_len = 0;
};

namespace {

// bounds[s]: the split table of segment s (world + 1 entries, in units of unit_bytes[s] bytes per row)
// Arguments of the small-message exchange of `kind` (e->ll_ok[kind]).
void make_ll_args(spb_shard_engine* e, int kind, const XSeg* segs, int nseg, const int* const* bounds, const int* unit_bytes,
                  LArgs& l, size_t* words_out) {
    for (int p = 0; p < e->world; ++p) l.peer[p] = e->peer[p];
    size_t words = 0, ll_at = e->ll_off[kind];
    for (int s = 0; s < nseg; ++s) {
        LSeg& g = l.seg[s];
        g.src = segs[s].src;
        g.dst_pitch = segs[s].dst_pitch;
        g.dst_region = segs[s].dst_off - static_cast<uint32_t>(bounds[s][e->rank]) * unit_bytes[s];
        uint32_t maxlen = 0;
        for (int p = 0; p < e->world; ++p) {
            g.off[p] = static_cast<uint32_t>(bounds[s][p]) * unit_bytes[s];
            g.len[p] = static_cast<uint32_t>(bounds[s][p + 1] - bounds[s][p]) * unit_bytes[s];
            maxlen = std::max(maxlen, g.len[p]);
            words += static_cast<size_t>(g.len[p] / 4) * e->batch;
        }
        g.ll_off = static_cast<uint32_t>(ll_at);
        g.ll_stride = 2 * maxlen * e->batch;
        ll_at += static_cast<size_t>(g.ll_stride) * e->world;
    }
    l.nseg = nseg; l.rows = e->batch; l.world = e->world; l.rank = e->rank;
    l.direct = 0;
    l.self = e->peer[e->rank];
    l.seqno = e->counters + 2 * kind;
    l.done = e->counters + 2 * kind + 1;
    l.status = e->status;
    l.broken = reinterpret_cast<int*>(e->counters + 2 * X_KINDS);
    l.timeout_ns = e->timeout_ns;
    if (words_out) *words_out = words;
}

int exchange(spb_shard_engine* e, int kind, const XSeg* segs, int nseg, const int* const* bounds, const int* unit_bytes) {
    if (e->world == 1) {  // nothing to exchange: the "slice" is the whole vector; copy it into place
        for (int s = 0; s < nseg; ++s)
            SPB_CUDA(cudaMemcpy2DAsync(e->xbuf + segs[s].dst_off, segs[s].dst_pitch, segs[s].src, segs[s].len, segs[s].len,
                                       e->batch, cudaMemcpyDeviceToDevice, e->stream));
        return SPB_OK;
    }
    if (e->ll_ok[kind]) {  // small slices: data and sequence number in one store, no fence
        LArgs l{};
        size_t words = 0;
        make_ll_args(e, kind, segs, nseg, bounds, unit_bytes, l, &words);
        const int blocks = static_cast<int>(std::max<size_t>(1, std::min<size_t>(32, words / 1024)));
        return launch("exchange_ll", exchange_ll_kernel, dim3(blocks), dim3(256), 0, e->stream, l);
    }
    XArgs a{};
    for (int p = 0; p < e->world; ++p) a.peer[p] = e->peer[p];
    bool wide = true;
    size_t bytes = 0;
    for (int s = 0; s < nseg; ++s) {
        a.seg[s] = segs[s];
        wide = wide && segs[s].len % 16 == 0 && segs[s].dst_off % 16 == 0 && segs[s].dst_pitch % 16 == 0 &&
               (reinterpret_cast<uintptr_t>(segs[s].src) & 15) == 0;
        bytes += static_cast<size_t>(segs[s].len) * e->batch;
    }
    a.nseg = nseg; a.rows = e->batch; a.world = e->world; a.rank = e->rank;
    a.flag_off = static_cast<uint32_t>(e->off_flags + kind * kFlagBytesPerKind);
    a.seqno = e->counters + 2 * kind;
    a.done = e->counters + 2 * kind + 1;
    a.status = e->status;
    a.broken = reinterpret_cast<int*>(e->counters + 2 * X_KINDS);
    a.timeout_ns = e->timeout_ns;
    const int blocks = static_cast<int>(std::max<size_t>(1, std::min<size_t>(64, bytes / (8 * 1024))));
    return wide ? launch("exchange", exchange_kernel<true>, dim3(blocks), dim3(256), 0, e->stream, a)
                : launch("exchange", exchange_kernel<false>, dim3(blocks), dim3(256), 0, e->stream, a);
}

XSeg seg_of(const void* src, size_t region, size_t off_bytes, size_t pitch, size_t len) {
    return XSeg{static_cast<const uint8_t*>(src), static_cast<uint32_t>(region + off_bytes), static_cast<uint32_t>(pitch),
                static_cast<uint32_t>(len)};
}

// Enqueues one decode step of all `batch` sequences on e->stream.
int enqueue_step(spb_shard_engine* e, bool record) {
    const spb_model_config& c = e->cfg;
    const int H = c.hidden_size, hd = c.head_dim, inter = c.intermediate_size, B = e->batch, r = e->rank;
    const int qdim = c.num_attention_heads * hd;
    void* s = e->stream;
    int rc;
    __half* cur = e->x;
    __half* other = e->x2;
    __half* attn_full = reinterpret_cast<__half*>(e->xbuf + e->off_attn);
    __half* o_full = reinterpret_cast<__half*>(e->xbuf + e->off_o);
    __half* gate_full = reinterpret_cast<__half*>(e->xbuf + e->off_gate);
    __half* up_full = reinterpret_cast<__half*>(e->xbuf + e->off_up);
    __half* down_full = reinterpret_cast<__half*>(e->xbuf + e->off_down);
    float* amax_full = reinterpret_cast<float*>(e->xbuf + e->off_amax);
    float* am0 = e->absmax;
    float* am1 = e->absmax + B;
    // One rank: a "slice" is the whole vector, so the producing kernels write where the consumers read and there
    // is nothing to exchange.
    const bool alone = e->world == 1;
    // Several ranks, wide single-sequence step: every gathered vector has one consumer, a single-block vector kernel;
    // it sends this rank's slice and collects the peers' itself (small-message form) instead of a launch doing that.
    LArgs pend{};  // the exchange the next vector kernel performs (world == 0: none)
    auto exchange_or_defer = [&](int kind, const XSeg* sg, int nseg, const int* const* bd, const int* ub) -> int {
        if (e->fold_exchange == 1 && e->wide && B == 1 && e->ll_ok[kind]) {
            make_ll_args(e, kind, sg, nseg, bd, ub, pend, nullptr);
            return SPB_OK;
        }
        return exchange(e, kind, sg, nseg, bd, ub);
    };
    auto take_pending = [&]() {
        const LArgs x = pend;
        pend = LArgs{};
        return x;
    };
    // One sequence and no exchange to perform inside: the vector kernels run as a cluster of eight blocks (eight SMs
    // pull the vector and its norm weights instead of one; same arithmetic, same results).
    auto clustered = [&]() { return B == 1 && (pend.world == 0 || pend.direct); };
    // Form 2: the kernel that computes this rank's slice stores it, as tagged words, straight into every rank's staging
    // area (this rank's own included) from its epilogue, and the consumer reads its vector from the local staging
    // area: no exchange launch, no gathered copy, and the NVLink crossing overlaps the producer's tail.  plan_direct
    // prepares both sides of exchange `kind` when the form applies; the producer must then be one that takes a fan.
    auto plan_direct = [&](int kind, const XSeg* sg, int nseg, const int* const* bd, const int* ub, LArgs& x, LlFan* fans) {
        if (e->fold_exchange != 2 || !e->wide || B != 1 || alone || !e->ll_ok[kind]) return false;
        x = LArgs{};
        make_ll_args(e, kind, sg, nseg, bd, ub, x, nullptr);
        x.direct = 1;
        for (int i = 0; i < nseg; ++i) {
            fans[i] = LlFan{};
            for (int q = 0; q < e->world; ++q)
                fans[i].dst[q] = reinterpret_cast<uint2*>(e->peer[q] + x.seg[i].ll_off + static_cast<size_t>(e->rank) * x.seg[i].ll_stride);
            fans[i].ndst = e->world;
            fans[i].seq = x.seqno;
        }
        return true;
    };
    __half* attn_out = alone ? attn_full : e->attn;
    __half* o_out = alone ? o_full : e->o;
    __half* gate_out = alone ? gate_full : e->gate;
    __half* up_out = alone ? up_full : e->up;
    __half* down_out = alone ? down_full : e->down;
    if ((rc = launch("shard_embed", shard_embed_kernel, dim3(std::max(1, H / 8 / 256), B), dim3(256), 0, s, e->embed, cur, H,
                     static_cast<const int*>(e->d_prompt), e->n_prompt_in_graph, static_cast<const int*>(e->d_next),
                     static_cast<const int*>(e->d_pos), B))) return rc;
    const float attn_scale = 1.0f / sqrtf(static_cast<float>(hd));
    auto linear_b = [&](const Linear& L, const float* am, __half* out, int32_t* ws) {
        return spb_sparse_bitlinear_gemm(L.meta, L.values, e->xq, out, am, L.gamma, ws, L.rows, L.cols, B, L.ms, L.vs, s);
    };
    // one matrix per launch on the quantised vector: takes the tensor-core GEMV wherever the layout allows
    auto linear_1 = [&](const Linear& L, const float* am, __half* out, void* on = nullptr) {
        if (L.prep) return prepared_bitlinear_q8(L.prep, e->xq, out, am, L.gamma, L.rows, L.cols, on ? on : s);
        return spb_sparse_bitlinear_q8(L.meta, L.values, e->xq, out, am, L.gamma, L.rows, L.cols, L.ms, L.vs, on ? on : s);
    };
    // Matrices that read the same quantised vector (q / k / v, gate / up) do not depend on one another: the first
    // goes on the engine's stream, the others on side streams between a fork and a join event, which the capture
    // turns into parallel branches of the graph.  k and v are latency bound on their own; side by side they cost
    // one GEMV's latency, and two large GEMVs in flight get more of the memory system than one.
    auto linear_side_by_side = [&](const Linear* const* L, __half* const* out, int n, const float* am) -> int {
        SPB_CUDA(cudaEventRecord(e->fork, e->stream));
        for (int i = 1; i < n; ++i) {
            SPB_CUDA(cudaStreamWaitEvent(e->side[i - 1], e->fork, 0));
            if (int r2 = linear_1(*L[i], am, out[i], e->side[i - 1])) return r2;
            SPB_CUDA(cudaEventRecord(e->join[i - 1], e->side[i - 1]));
        }
        if (int r2 = linear_1(*L[0], am, out[0])) return r2;
        for (int i = 1; i < n; ++i) SPB_CUDA(cudaStreamWaitEvent(e->stream, e->join[i - 1], 0));
        return SPB_OK;
    };
    // ... unless every matrix of the group has a prepared copy: then the group is one launch (no fork and join, whose
    // graph edges are full dependencies where a stream-ordered launch overlaps its predecessor's tail), and q, k, v
    // rotate and scatter their rows in its epilogue.
    auto all_prepared = [&](const Linear* const* L, int n) {
        for (int i = 0; i < n; ++i)
            if (!L[i]->prep) return false;
        return true;
    };
    auto linear_group_prepared = [&](const Linear* const* L, __half* const* out, int n, const float* am, const RopeScatter* rope,
                                     const LlFan* fans = nullptr) {
        const void* prep[3];
        void* outs[3];
        float gamma[3];
        int rows[3];
        for (int i = 0; i < n; ++i) {
            prep[i] = L[i]->prep; outs[i] = out[i]; gamma[i] = L[i]->gamma; rows[i] = L[i]->rows;
        }
        return prepared_bitlinear_q8_group(prep, outs, gamma, rows, n, e->xq, am, L[0]->cols, rope, s, fans);
    };
    // Wide models (hidden >= 4096): a matrix is tens of megabytes and its GEMV runs for tens of microseconds, so
    // throughput decides, not launch latency: the vector op runs once in a kernel of its own and every matrix goes
    // through the tensor-core GEMV, instead of the SIMT kernels that recompute the vector op in every block.
    const bool fused1 = e->fused && !e->wide;
    // vector ops: the register-resident kernels for wide models, the shared ones of the single-GPU engine otherwise
    auto res_norm_quant = [&](const __half* delta, const float* sub_w, __half* x, const float* w, __half* xn_out, float* am) {
        if (e->wide) {
            if (clustered())
                return launch_clustered("wide_residual_norm_quant", wide_residual_norm_quant_kernel<kWideCluster>, dim3(kWideCluster),
                                        dim3(kWideThreads / kWideCluster), kWideCluster, s, delta, sub_w, x, w, xn_out, e->xq, am, H,
                                        c.rms_norm_eps, take_pending());
            return launch("wide_residual_norm_quant", wide_residual_norm_quant_kernel<1>, dim3(B), dim3(kWideThreads), 0, s, delta, sub_w,
                          x, w, xn_out, e->xq, am, H, c.rms_norm_eps, take_pending());
        }
        return residual_norm_quant(delta, sub_w, x, w, xn_out, e->xq, am, H, c.rms_norm_eps, s, B);
    };
    for (int l = 0; l < c.num_hidden_layers; ++l) {
        const Layer& L = e->layers[l];
        __half* kc = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(e->kcache) + l * e->kv_layer_bytes);
        __half* vc = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(e->vcache) + l * e->kv_layer_bytes);
        const Linear* g3[3] = {&L.lin[0], &L.lin[1], &L.lin[2]};
        __half* o3[3] = {e->q, e->k, e->v};
        const Linear* g1o[1] = {&L.lin[3]};
        __half* o1o[1] = {o_out};
        const Linear* g2[2] = {&L.lin[4], &L.lin[5]};
        __half* o2[2] = {gate_out, up_out};
        const Linear* g1d[1] = {&L.lin[6]};
        __half* o1d[1] = {down_out};
        const __half* delta = l == 0 ? nullptr : down_full;
        bool rope_done = false;  // q, k, v rotated and scattered by the launch that computed them
        // ---- q / k / v on this rank's heads ----
        if (B == 1 && fused1) {
            if ((rc = bitlinear_resnorm_group(make_group(g3, o3, 3), cur, delta, nullptr, L.norm[0], other, c.rms_norm_eps, s))) return rc;
            std::swap(cur, other);
        } else {
            if ((rc = res_norm_quant(delta, nullptr, cur, L.norm[0], nullptr, am0))) return rc;
            if (B == 1 && e->wide) {
                if (all_prepared(g3, 3)) {
                    const RopeScatter rs{e->d_pos, c.rope_theta, hd, c.max_position_embeddings, kc, vc};
                    if ((rc = linear_group_prepared(g3, o3, 3, am0, &rs))) return rc;
                    rope_done = true;
                } else if ((rc = linear_side_by_side(g3, o3, 3, am0))) {
                    return rc;
                }
            } else if (B == 1) {
                if ((rc = bitlinear_q8_group(make_group(g3, o3, 3), e->xq, am0, s))) return rc;
            } else {
                for (int i = 0; i < 3; ++i)
                    if ((rc = linear_b(L.lin[i], am0, o3[i], e->acc + i * e->acc_third))) return rc;
            }
        }
        if (!rope_done && (rc = rope_scatter(e->q, e->k, e->v, kc, vc, e->nh_loc, e->nkv_loc, hd, c.max_position_embeddings, c.rope_theta,
                               e->d_pos, s, B, B > 1 ? e->seq_stride : 0))) return rc;
        const XSeg sg_attn = seg_of(e->attn, e->off_attn, static_cast<size_t>(e->kv0[r]) * e->group_heads * hd * 2,
                                    static_cast<size_t>(qdim) * 2, static_cast<size_t>(e->nh_loc) * hd * 2);
        const int* bd_attn[1] = {e->kv0};
        const int ub_attn[1] = {e->group_heads * hd * 2};
        LArgs xd{};
        LlFan fan[2];
        bool sent = false;  // the producer's epilogue sent the slice (form 2)
        if (B == 1 && e->split_attention) {
            // (a batched form of the split kernel, one block per (KV head, chunk, sequence), was measured slower for
            // 64 sequences than one block per (head, sequence): 54.6 against 51.6 ms per step)
            sent = plan_direct(X_ATTN, &sg_attn, 1, bd_attn, ub_attn, xd, fan);
            if ((rc = decode_attention_split(e->q, kc, vc, attn_out, e->nh_loc, e->nkv_loc, hd, c.max_position_embeddings, 0,
                                             e->d_pos, attn_scale, e->attn_scratch, s, e->attn_counters, sent ? fan : nullptr))) return rc;
        } else if ((rc = decode_attention_pos(e->q, kc, vc, attn_out, e->nh_loc, e->nkv_loc, hd, c.max_position_embeddings,
                                              attn_scale, e->d_pos, s, B, B > 1 ? e->seq_stride : 0))) {
            return rc;
        }
        if (sent) pend = xd;
        else if (!alone && (rc = exchange_or_defer(X_ATTN, &sg_attn, 1, bd_attn, ub_attn))) return rc;
        // ---- o_proj rows ----
        const XSeg sg_o = seg_of(e->o, e->off_o, static_cast<size_t>(e->hrow[r]) * 2, static_cast<size_t>(H) * 2,
                                 static_cast<size_t>(e->h_loc) * 2);
        const int* bd_h[1] = {e->hrow};
        const int ub_h[1] = {2};
        sent = false;
        if (B == 1 && fused1) {
            if ((rc = bitlinear_amax_group(make_group(g1o, o1o, 1), attn_full, s))) return rc;
        } else {
            if (e->wide) {
                if (clustered()) {
                    if ((rc = launch_clustered("wide_absmax_quantize", wide_absmax_quantize_kernel<kWideCluster>, dim3(kWideCluster),
                                               dim3(kWideThreads / kWideCluster), kWideCluster, s, static_cast<const __half*>(attn_full),
                                               e->xq, am1, qdim, take_pending()))) return rc;
                } else if ((rc = launch("wide_absmax_quantize", wide_absmax_quantize_kernel<1>, dim3(B), dim3(kWideThreads), 0, s,
                                        static_cast<const __half*>(attn_full), e->xq, am1, qdim, take_pending()))) {
                    return rc;
                }
            } else if ((rc = absmax_quantize_rows(attn_full, e->xq, am1, qdim, B, s))) {
                return rc;
            }
            if (B == 1) {
                sent = L.lin[3].prep && plan_direct(X_O, &sg_o, 1, bd_h, ub_h, xd, fan);
                if (sent) {
                    if ((rc = linear_group_prepared(g1o, o1o, 1, am1, nullptr, fan))) return rc;
                } else if ((rc = linear_1(L.lin[3], am1, o_out))) {
                    return rc;
                }
            } else if ((rc = linear_b(L.lin[3], am1, o_out, e->acc))) {
                return rc;
            }
        }
        if (sent) pend = xd;
        else if (!alone && (rc = exchange_or_defer(X_O, &sg_o, 1, bd_h, ub_h))) return rc;
        // ---- gate / up rows ----
        const XSeg sg_gu[2] = {seg_of(e->gate, e->off_gate, static_cast<size_t>(e->irow[r]) * 2, static_cast<size_t>(inter) * 2,
                                      static_cast<size_t>(e->i_loc) * 2),
                               seg_of(e->up, e->off_up, static_cast<size_t>(e->irow[r]) * 2, static_cast<size_t>(inter) * 2,
                                      static_cast<size_t>(e->i_loc) * 2)};
        const int* bd_gu[2] = {e->irow, e->irow};
        const int ub_gu[2] = {2, 2};
        sent = false;
        if (B == 1 && fused1) {
            if ((rc = bitlinear_resnorm_group(make_group(g2, o2, 2), cur, o_full, L.norm[2], L.norm[1], other, c.rms_norm_eps, s))) return rc;
            std::swap(cur, other);
        } else {
            if ((rc = res_norm_quant(o_full, L.norm[2], cur, L.norm[1], nullptr, am0))) return rc;
            if (B == 1 && e->wide) {
                if (all_prepared(g2, 2)) {
                    sent = plan_direct(X_GU, sg_gu, 2, bd_gu, ub_gu, xd, fan);
                    if ((rc = linear_group_prepared(g2, o2, 2, am0, nullptr, sent ? fan : nullptr))) return rc;
                } else if ((rc = linear_side_by_side(g2, o2, 2, am0))) {
                    return rc;
                }
            } else if (B == 1) {
                if ((rc = bitlinear_q8_group(make_group(g2, o2, 2), e->xq, am0, s))) return rc;
            } else {
                if ((rc = linear_b(L.lin[4], am0, gate_out, e->acc))) return rc;
                if ((rc = linear_b(L.lin[5], am0, up_out, e->acc + e->acc_third))) return rc;
            }
        }
        if (sent) pend = xd;
        else if (!alone && (rc = exchange_or_defer(X_GU, sg_gu, 2, bd_gu, ub_gu))) return rc;
        // ---- down rows: relu2 * up and ffn_sub_norm need the whole vectors ----
        const XSeg sg_down = seg_of(e->down, e->off_down, static_cast<size_t>(e->hrow[r]) * 2, static_cast<size_t>(H) * 2,
                                    static_cast<size_t>(e->h_loc) * 2);
        sent = false;
        if (B == 1 && fused1) {
            if ((rc = bitlinear_relu2_group(make_group(g1d, o1d, 1), gate_full, up_full, L.norm[3], c.rms_norm_eps, s))) return rc;
        } else {
            if (e->wide) {
                if (clustered()) {
                    if ((rc = launch_clustered("wide_relu2_norm_quant", wide_relu2_norm_quant_kernel<kWideCluster>, dim3(kWideCluster),
                                               dim3(kWideThreads / kWideCluster), kWideCluster, s, static_cast<const __half*>(gate_full),
                                               static_cast<const __half*>(up_full), L.norm[3], e->xq, am1, inter, c.rms_norm_eps,
                                               take_pending()))) return rc;
                } else if ((rc = launch("wide_relu2_norm_quant", wide_relu2_norm_quant_kernel<1>, dim3(B), dim3(kWideThreads), 0, s,
                                        static_cast<const __half*>(gate_full), static_cast<const __half*>(up_full), L.norm[3], e->xq,
                                        am1, inter, c.rms_norm_eps, take_pending()))) {
                    return rc;
                }
            } else if ((rc = relu2_norm_quant(gate_full, up_full, L.norm[3], nullptr, e->xq, am1, inter, c.rms_norm_eps, s, B))) {
                return rc;
            }
            if (B == 1) {
                sent = L.lin[6].prep && plan_direct(X_DOWN, &sg_down, 1, bd_h, ub_h, xd, fan);
                if (sent) {
                    if ((rc = linear_group_prepared(g1d, o1d, 1, am1, nullptr, fan))) return rc;
                } else if ((rc = linear_1(L.lin[6], am1, down_out))) {
                    return rc;
                }
            } else if ((rc = linear_b(L.lin[6], am1, down_out, e->acc))) {
                return rc;
            }
        }
        if (sent) pend = xd;
        else if (!alone && (rc = exchange_or_defer(X_DOWN, &sg_down, 1, bd_h, ub_h))) return rc;
    }
    // last residual add + final norm, LM head on this rank's vocabulary rows, arg-max candidates
    if ((rc = res_norm_quant(c.num_hidden_layers ? down_full : nullptr, nullptr, cur, e->final_norm, e->xfinal, am0))) return rc;
    if (B == 1) {
        if ((rc = spb_half_gemv(e->lm_head_loc, e->xfinal, e->logits, e->v_loc, H, s))) return rc;
    } else if ((rc = half_gemm_rows(e->lm_head_loc, e->xfinal, e->logits, e->v_loc, H, B, s))) {
        return rc;
    }
    if ((rc = launch("shard_argmax1", shard_argmax1_kernel, dim3(e->argmax_blocks, B), dim3(1024), 0, s,
                     static_cast<const float*>(e->logits), e->v_loc, e->cand))) return rc;
    if ((rc = launch("shard_argmax2", shard_argmax2_kernel, dim3(B), dim3(128), 0, s, static_cast<const float*>(e->cand),
                     e->argmax_blocks, e->vrow[r], e->pairs))) return rc;
    {
        const XSeg sg = seg_of(e->pairs, e->off_amax, static_cast<size_t>(r) * 8, static_cast<size_t>(e->world) * 8, 8);
        const int* bd[1] = {e->ident};
        const int ub[1] = {8};
        if ((rc = exchange(e, X_AMAX, &sg, 1, bd, ub))) return rc;
    }
    return launch("shard_pick", shard_pick_kernel, dim3(1), dim3(kMaxBatch), 0, s, static_cast<const float*>(amax_full), e->world,
                  B, e->d_next, record ? e->d_out : nullptr, e->d_pos);
}

int check_ready(const spb_shard_engine* e) {
    if (!e) return fail(SPB_E_INVALID, "sharded engine: null handle");
    if (!e->embed || !e->final_norm || !e->lm_head_loc) return fail(SPB_E_INVALID, "sharded engine: globals not set");
    if (e->world > 1 && !e->peers_set) return fail(SPB_E_INVALID, "sharded engine: peers not set");
    for (const Layer& L : e->layers) {
        for (int i = 0; i < 7; ++i)
            if (!L.lin[i].meta) return fail(SPB_E_INVALID, "sharded engine: a linear layer has no weights attached");
        if (!L.norm[0] || !L.norm[1]) return fail(SPB_E_INVALID, "sharded engine: a layer norm is missing");
    }
    return SPB_OK;
}

void drop_graph(spb_shard_engine* e) {
    if (e->graph) cudaGraphExecDestroy(e->graph);
    e->graph = nullptr;
}

int ensure_graph(spb_shard_engine* e, bool record, int n_prompt) {
    if (e->graph && e->graph_records == record && e->n_prompt_in_graph == n_prompt) return SPB_OK;
    drop_graph(e);
    e->n_prompt_in_graph = n_prompt;
    e->fused = true;
    for (const Layer& L : e->layers) {
        const Linear* all[7] = {&L.lin[0], &L.lin[1], &L.lin[2], &L.lin[3], &L.lin[4], &L.lin[5], &L.lin[6]};
        __half* none[7] = {};
        for (int i = 0; i < 7 && e->fused; ++i) e->fused = bitlinear_group_is_fast(make_group(all + i, none + i, 1));
    }
    SPB_CUDA(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    const int rc = enqueue_step(e, record);
    cudaGraph_t g = nullptr;
    const cudaError_t err = cudaStreamEndCapture(e->stream, &g);
    if (rc) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (err != cudaSuccess) return cuda_fail("cudaStreamEndCapture", err);
    const cudaError_t ierr = cudaGraphInstantiate(&e->graph, g, 0);
    cudaGraphDestroy(g);
    if (ierr != cudaSuccess) return cuda_fail("cudaGraphInstantiate", ierr);
    e->graph_records = record;
    return SPB_OK;
}

int check_status(spb_shard_engine* e, const char* where) {
    if (*static_cast<volatile int*>(e->status) == 0) return SPB_OK;
    return fail(SPB_E_TIMEOUT, "%s: rank %d waited longer than %.0f ms for a peer in an exchange; the engine's outputs are "
                "unspecified and it must be recreated", where, e->rank, e->timeout_ns / 1e6);
}

class DeviceScope {
public:
    explicit DeviceScope(int device) {
        if (cudaGetDevice(&prev_) != cudaSuccess) prev_ = -1;
        if (prev_ != device) switched_ = cudaSetDevice(device) == cudaSuccess;
    }
    ~DeviceScope() {
        if (switched_ && prev_ >= 0) cudaSetDevice(prev_);
    }

private:
    int prev_ = -1;
    bool switched_ = false;
};

}  // namespace

extern "C" spb_shard_engine* spb_shard_engine_create(const spb_model_config* cfg, int rank, int world, int batch) {
    if (!cfg || cfg->hidden_size <= 0 || cfg->num_hidden_layers < 0 || cfg->num_attention_heads <= 0 ||
        cfg->num_key_value_heads <= 0 || cfg->head_dim <= 0 || cfg->head_dim % 8 || cfg->intermediate_size <= 0 ||
        cfg->vocab_size <= 0 || cfg->max_position_embeddings <= 0 || cfg->hidden_size % 8 || cfg->intermediate_size % 8 ||
        cfg->num_attention_heads % cfg->num_key_value_heads) {
        fail(SPB_E_INVALID, "spb_shard_engine_create: bad config (hidden, intermediate and head_dim must be multiples of 8)");
        return nullptr;
    }
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || batch < 1 || batch > kMaxBatch ||
        world > cfg->num_key_value_heads || (world > 1 && cfg->num_hidden_layers < 1)) {
        fail(SPB_E_INVALID, "spb_shard_engine_create: world 1..%d (at most the KV heads; at least one layer when sharded), "
             "batch 1..%d", kMaxWorld, kMaxBatch);
        return nullptr;
    }
    spb_shard_engine* e = new (std::nothrow) spb_shard_engine();
    if (!e) return nullptr;
    prepare_host_state();
    e->cfg = *cfg; e->rank = rank; e->world = world; e->batch = batch;
    e->layers.resize(cfg->num_hidden_layers);
    cudaGetDevice(&e->device);
    const int H = cfg->hidden_size, hd = cfg->head_dim, inter = cfg->intermediate_size, B = batch;
    const int qdim = cfg->num_attention_heads * hd;
    e->group_heads = cfg->num_attention_heads / cfg->num_key_value_heads;
    for (int p = 0; p < world; ++p) {
        int a, b;
        split_range(cfg->num_key_value_heads, world, p, 1, &a, &b);
        e->kv0[p] = a; e->kv0[p + 1] = b;
        split_range(H, world, p, 8, &a, &b);
        e->hrow[p] = a; e->hrow[p + 1] = b;
        split_range(inter, world, p, 8, &a, &b);
        e->irow[p] = a; e->irow[p + 1] = b;
        split_range(cfg->vocab_size, world, p, 1, &a, &b);
        e->vrow[p] = a; e->vrow[p + 1] = b;
    }
    e->nkv_loc = e->kv0[rank + 1] - e->kv0[rank];
    e->nh_loc = e->nkv_loc * e->group_heads;
    e->h_loc = e->hrow[rank + 1] - e->hrow[rank];
    e->i_loc = e->irow[rank + 1] - e->irow[rank];
    e->v_loc = e->vrow[rank + 1] - e->vrow[rank];
    e->split_attention = e->nkv_loc > 0 && decode_attention_split_supported(e->nh_loc, e->nkv_loc, hd);
    e->wide = H >= 4096 && H <= 8 * kWideThreads && inter <= 8 * kWideThreads * kWideRuns && qdim <= 8 * kWideThreads * kWideRuns;
    e->seq_stride = static_cast<size_t>(e->nkv_loc) * cfg->max_position_embeddings * hd;
    e->kv_layer_bytes = align_up(sizeof(__half) * e->seq_stride * B, 256);
    const size_t maxdim = std::max(std::max(H, qdim), inter);
    const size_t max_rows_loc = std::max(std::max(e->nh_loc * hd, e->h_loc), e->i_loc);
    e->acc_third = static_cast<size_t>(B) * max_rows_loc;
    e->out_cap = cfg->max_position_embeddings;

    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
    const size_t o_kc = take(e->kv_layer_bytes * cfg->num_hidden_layers), o_vc = take(e->kv_layer_bytes * cfg->num_hidden_layers);
    const size_t o_x = take(2 * B * H), o_x2 = take(2 * B * H), o_q = take(2 * B * e->nh_loc * hd), o_k = take(2 * B * e->nkv_loc * hd);
    const size_t o_v = take(2 * B * e->nkv_loc * hd), o_attn = take(2 * B * e->nh_loc * hd), o_o = take(2 * B * e->h_loc);
    const size_t o_gate = take(2 * B * e->i_loc), o_up = take(2 * B * e->i_loc), o_down = take(2 * B * e->h_loc), o_xf = take(2 * B * H);
    const size_t o_xq = take(B * maxdim), o_abs = take(4 * 2 * B), o_acc = take(B > 1 ? 3 * 4 * e->acc_third : 16);
    const size_t o_ascr = take(decode_attention_scratch_bytes(std::max(e->nh_loc, 1), hd, cfg->max_position_embeddings));
    const size_t o_actr = take(4 * static_cast<size_t>(std::max(e->nkv_loc, 1)));
    e->argmax_blocks = std::max(1, std::min(128, (e->v_loc + 1023) / 1024));
    const size_t o_logits = take(4 * static_cast<size_t>(B) * e->v_loc), o_pairs = take(8 * B), o_ints = take(4 * (1 + B));
    const size_t o_cand = take(8 * static_cast<size_t>(B) * e->argmax_blocks);
    const size_t o_out = take(4 * static_cast<size_t>(e->out_cap) * B), o_ctr = take(4 * (2 * X_KINDS + 1));
    const size_t pool_bytes = off;
    // exchange buffer
    off = 0;
    e->off_flags = take(kFlagBytesPerKind * X_KINDS);
    e->off_attn = take(2 * static_cast<size_t>(B) * qdim);
    e->off_o = take(2 * static_cast<size_t>(B) * H);
    e->off_gate = take(2 * static_cast<size_t>(B) * inter);
    e->off_up = take(2 * static_cast<size_t>(B) * inter);
    e->off_down = take(2 * static_cast<size_t>(B) * H);
    e->off_amax = take(8 * static_cast<size_t>(B) * world);
    {   // staging of the small-message exchange: per kind, per segment, per sending rank 2 x (largest slice) x batch
        auto maxdiff = [&](const int* b) { int m = 0; for (int p = 0; p < world; ++p) m = std::max(m, b[p + 1] - b[p]); return static_cast<size_t>(m); };
        const size_t slice[X_KINDS] = {maxdiff(e->kv0) * e->group_heads * hd * 2, maxdiff(e->hrow) * 2, maxdiff(e->irow) * 2,
                                       maxdiff(e->hrow) * 2, 8};
        const int nseg[X_KINDS] = {1, 1, 2, 1, 1};
        constexpr size_t kLlMaxSliceBytes = 96 * 1024;  // per segment and sender; larger slices take the fenced form
        for (int k = 0; k < X_KINDS; ++k) {
            e->ll_ok[k] = world > 1 && slice[k] * B <= kLlMaxSliceBytes;
            if (e->ll_ok[k]) e->ll_off[k] = take(2 * slice[k] * B * world * nseg[k]);
        }
    }
    e->xbuf_bytes = off;
    if (cudaMalloc(&e->pool, pool_bytes) != cudaSuccess || cudaMemset(e->pool, 0, pool_bytes) != cudaSuccess ||
        cudaMalloc(&e->xbuf, e->xbuf_bytes) != cudaSuccess || cudaMemset(e->xbuf, 0, e->xbuf_bytes) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess ||  // the fills run on the null stream, the engine on a stream that does not wait for it
        cudaHostAlloc(reinterpret_cast<void**>(&e->status), sizeof(int), cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess ||
        cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess) {
        cuda_fail("spb_shard_engine_create", cudaGetLastError());
        if (e->pool) cudaFree(e->pool);
        if (e->xbuf) cudaFree(e->xbuf);
        if (e->status) cudaFreeHost(e->status);
        delete e;
        return nullptr;
    }
    *e->status = 0;
    cudaEventCreateWithFlags(&e->fork, cudaEventDisableTiming);
    for (int i = 0; i < 2; ++i) {
        cudaStreamCreateWithFlags(&e->side[i], cudaStreamNonBlocking);
        cudaEventCreateWithFlags(&e->join[i], cudaEventDisableTiming);
    }
    cudaDeviceSynchronize();
    uint8_t* p = e->pool;
    e->kcache = reinterpret_cast<__half*>(p + o_kc); e->vcache = reinterpret_cast<__half*>(p + o_vc);
    e->x = reinterpret_cast<__half*>(p + o_x); e->x2 = reinterpret_cast<__half*>(p + o_x2);
    e->q = reinterpret_cast<__half*>(p + o_q); e->k = reinterpret_cast<__half*>(p + o_k); e->v = reinterpret_cast<__half*>(p + o_v);
    e->attn = reinterpret_cast<__half*>(p + o_attn); e->o = reinterpret_cast<__half*>(p + o_o);
    e->gate = reinterpret_cast<__half*>(p + o_gate); e->up = reinterpret_cast<__half*>(p + o_up);
    e->down = reinterpret_cast<__half*>(p + o_down); e->xfinal = reinterpret_cast<__half*>(p + o_xf);
    e->xq = reinterpret_cast<int8_t*>(p + o_xq); e->absmax = reinterpret_cast<float*>(p + o_abs);
    e->acc = reinterpret_cast<int32_t*>(p + o_acc); e->attn_scratch = reinterpret_cast<float*>(p + o_ascr);
    e->attn_counters = reinterpret_cast<unsigned*>(p + o_actr);
    e->logits = reinterpret_cast<float*>(p + o_logits); e->pairs = reinterpret_cast<float*>(p + o_pairs);
    e->cand = reinterpret_cast<float*>(p + o_cand);
    e->d_pos = reinterpret_cast<int*>(p + o_ints); e->d_next = e->d_pos + 1;
    e->d_out = reinterpret_cast<int*>(p + o_out); e->counters = reinterpret_cast<unsigned*>(p + o_ctr);
    e->peer[rank] = e->xbuf;
    return e;
}

// (Re)builds or drops the prepared form of a slice according to the engine's setting.  Only the wide single-sequence
// step multiplies matrix by matrix on the quantised vector, which is where the prepared GEMV applies.
static int prepare_linear(spb_shard_engine* e, Linear& L, int which) {
    if (L.prep) {
        SPB_CUDA(cudaStreamSynchronize(e->stream));
        cudaFree(L.prep);
        L.prep = nullptr;
    }
    const size_t bytes = spb_prepared_weights_bytes(L.rows, L.cols);
    // (measured on the per-rank shapes of the 70B model, one step of eight layers: at 4 ranks 0.72 ms with every slice
    // prepared against 0.79 with only those of 32 M weights and more, at 8 ranks 0.67 against 0.80: with prepared
    // copies q / k / v and gate / up are one launch each and rotate and scatter in the epilogue, which the packed
    // form's launch per matrix does not make up for even where its kernel is the quicker one.)
    // k and v go with q: the group is one launch only with prepared copies of all three
    long long weights = static_cast<long long>(L.rows) * L.cols;
    if (which == 1 || which == 2) weights *= e->group_heads;
    const bool large = e->use_prepared == 2 || weights >= 4LL * 1024 * 1024;
    if (!e->use_prepared || !e->wide || e->batch != 1 || !large || bytes == 0 || L.ms < L.cols / 32 || L.vs < L.cols / 64) return SPB_OK;
    SPB_CUDA(cudaMalloc(&L.prep, bytes));
    return spb_prepare_weights(L.meta, L.values, L.rows, L.cols, L.ms, L.vs, L.prep, e->stream);
}

extern "C" void spb_shard_engine_destroy(spb_shard_engine* e) {
    if (!e) return;
    DeviceScope scope(e->device);
    cudaStreamSynchronize(e->stream);
    drop_graph(e);
    for (int p = 0; p < e->world; ++p)
        if (p != e->rank && e->peer[p]) cudaIpcCloseMemHandle(e->peer[p]);
    if (e->d_prompt) cudaFree(e->d_prompt);
    for (int i = 0; i < 2; ++i) {
        if (e->side[i]) cudaStreamDestroy(e->side[i]);
        if (e->join[i]) cudaEventDestroy(e->join[i]);
    }
    if (e->fork) cudaEventDestroy(e->fork);
    for (Layer& Ly : e->layers)
        for (Linear& L : Ly.lin)
            if (L.prep) cudaFree(L.prep);
    cudaFree(e->pool);
    cudaFree(e->xbuf);
    cudaFreeHost(e->status);
    cudaStreamDestroy(e->stream);
    delete e;
}

extern "C" int spb_shard_engine_row_range(const spb_shard_engine* e, int which, int* start, int* stop) {
    if (!e || !start || !stop || which < 0 || which > 7) return fail(SPB_E_INVALID, "spb_shard_engine_row_range: bad arguments");
    const int hd = e->cfg.head_dim, r = e->rank;
    switch (which) {
        case 0: *start = e->kv0[r] * e->group_heads * hd; *stop = e->kv0[r + 1] * e->group_heads * hd; break;
        case 1: case 2: *start = e->kv0[r] * hd; *stop = e->kv0[r + 1] * hd; break;
        case 3: case 6: *start = e->hrow[r]; *stop = e->hrow[r + 1]; break;
        case 4: case 5: *start = e->irow[r]; *stop = e->irow[r + 1]; break;
        default: *start = e->vrow[r]; *stop = e->vrow[r + 1]; break;
    }
    return SPB_OK;
}

extern "C" int spb_shard_engine_ipc_handle(spb_shard_engine* e, void* handle_out) {
    if (!e || !handle_out) return fail(SPB_E_INVALID, "spb_shard_engine_ipc_handle: null pointer");
    DeviceScope scope(e->device);
    cudaIpcMemHandle_t h;
    SPB_CUDA(cudaIpcGetMemHandle(&h, e->xbuf));
    static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
    std::memcpy(handle_out, &h, sizeof h);
    return SPB_OK;
}

extern "C" int spb_shard_engine_set_peers(spb_shard_engine* e, const void* handles) {
    if (!e || (e->world > 1 && !handles)) return fail(SPB_E_INVALID, "spb_shard_engine_set_peers: null pointer");
    if (e->peers_set) return fail(SPB_E_INVALID, "spb_shard_engine_set_peers: peers already set");
    DeviceScope scope(e->device);
    for (int p = 0; p < e->world; ++p) {
        if (p == e->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const uint8_t*>(handles) + 64 * p, sizeof h);
        void* ptr = nullptr;
        SPB_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        e->peer[p] = static_cast<uint8_t*>(ptr);
    }
    e->peers_set = true;
    drop_graph(e);
    return SPB_OK;
}

extern "C" int spb_shard_engine_set_peer_pointers(spb_shard_engine* e, void* const* buffers) {
    // same-process form (and the failure test's stand-in peer): device pointers that this GPU can already reach
    if (!e || !buffers) return fail(SPB_E_INVALID, "spb_shard_engine_set_peer_pointers: null pointer");
    if (e->peers_set) return fail(SPB_E_INVALID, "spb_shard_engine_set_peer_pointers: peers already set");
    for (int p = 0; p < e->world; ++p)
        if (p != e->rank) {
            if (!buffers[p]) return fail(SPB_E_INVALID, "spb_shard_engine_set_peer_pointers: null buffer for rank %d", p);
            e->peer[p] = static_cast<uint8_t*>(buffers[p]);
        }
    e->peers_set = true;
    drop_graph(e);
    return SPB_OK;
}

extern "C" size_t spb_shard_engine_exchange_bytes(const spb_shard_engine* e) { return e ? e->xbuf_bytes : 0; }

extern "C" int spb_shard_engine_set_timeout_ms(spb_shard_engine* e, int ms) {
    if (!e || ms < 1) return fail(SPB_E_INVALID, "spb_shard_engine_set_timeout_ms: bad arguments");
    e->timeout_ns = static_cast<unsigned long long>(ms) * 1000000ull;
    drop_graph(e);
    return SPB_OK;
}

extern "C" int spb_shard_engine_set_linear(spb_shard_engine* e, int layer, int which, const uint32_t* d_meta,
                                           const uint32_t* d_values, float gamma, int rows, int cols, int meta_stride,
                                           int values_stride) {
    if (!e || layer < 0 || layer >= static_cast<int>(e->layers.size()) || which < 0 || which > 6)
        return fail(SPB_E_INVALID, "spb_shard_engine_set_linear: bad layer/which");
    if (!d_meta || !d_values || rows <= 0 || cols <= 0 || cols % 4) return fail(SPB_E_INVALID, "spb_shard_engine_set_linear: bad tensor");
    int a = 0, b = 0;
    spb_shard_engine_row_range(e, which, &a, &b);
    const spb_model_config& c = e->cfg;
    const int qdim = c.num_attention_heads * c.head_dim;
    const int want_cols[7] = {c.hidden_size, c.hidden_size, c.hidden_size, qdim, c.hidden_size, c.hidden_size, c.intermediate_size};
    if (rows != b - a || cols != want_cols[which])
        return fail(SPB_E_INVALID, "spb_shard_engine_set_linear: layer %d tensor %d is %dx%d, rank %d of %d owns %dx%d", layer, which,
                    rows, cols, e->rank, e->world, b - a, want_cols[which]);
    Linear& L = e->layers[layer].lin[which];
    L.meta = d_meta; L.values = d_values; L.gamma = gamma; L.rows = rows; L.cols = cols; L.ms = meta_stride; L.vs = values_stride;
    drop_graph(e);
    DeviceScope scope(e->device);
    return prepare_linear(e, L, which);
}

extern "C" int spb_shard_engine_set_exchange_fold(spb_shard_engine* e, int on) {
    if (!e) return fail(SPB_E_INVALID, "spb_shard_engine_set_exchange_fold: null handle");
    DeviceScope scope(e->device);
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    drop_graph(e);
    e->fold_exchange = on < 0 ? 0 : on > 2 ? 2 : on;
    return SPB_OK;
}

extern "C" int spb_shard_engine_set_prepared_weights(spb_shard_engine* e, int on) {
    if (!e) return fail(SPB_E_INVALID, "spb_shard_engine_set_prepared_weights: null handle");
    DeviceScope scope(e->device);
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    drop_graph(e);
    e->use_prepared = on < 0 ? 0 : on > 2 ? 2 : on;
    for (Layer& Ly : e->layers)
        for (int which = 0; which < 7; ++which)
            if (Ly.lin[which].meta)
                if (int rc = prepare_linear(e, Ly.lin[which], which)) return rc;
    return SPB_OK;
}

extern "C" int spb_shard_engine_set_norm(spb_shard_engine* e, int layer, int which, const float* d_weight) {
    if (!e || layer < 0 || layer >= static_cast<int>(e->layers.size()) || which < 0 || which > 3)
        return fail(SPB_E_INVALID, "spb_shard_engine_set_norm: bad layer/which");
    e->layers[layer].norm[which] = d_weight;
    drop_graph(e);
    return SPB_OK;
}

extern "C" int spb_shard_engine_set_globals(spb_shard_engine* e, const void* d_embed, const void* d_lm_head_rows,
                                            const float* d_final_norm) {
    if (!e || !d_embed || !d_lm_head_rows || !d_final_norm) return fail(SPB_E_INVALID, "spb_shard_engine_set_globals: null pointer");
    e->embed = static_cast<const __half*>(d_embed);
    e->lm_head_loc = static_cast<const __half*>(d_lm_head_rows);
    e->final_norm = d_final_norm;
    drop_graph(e);
    return SPB_OK;
}

extern "C" int spb_shard_engine_reset(spb_shard_engine* e) {
    if (!e) return fail(SPB_E_INVALID, "spb_shard_engine_reset: null handle");
    DeviceScope scope(e->device);
    const size_t kv_total = e->kv_layer_bytes * e->cfg.num_hidden_layers;
    SPB_CUDA(cudaMemsetAsync(e->kcache, 0, kv_total, e->stream));
    SPB_CUDA(cudaMemsetAsync(e->vcache, 0, kv_total, e->stream));
    SPB_CUDA(cudaMemsetAsync(e->d_pos, 0, 4 * (1 + e->batch), e->stream));
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    e->seq_len = 0;
    return SPB_OK;
}

extern "C" int spb_shard_engine_seq_len(const spb_shard_engine* e) { return e ? e->seq_len : 0; }

extern "C" int spb_shard_engine_step(spb_shard_engine* e, const int* tokens) {
    int rc = check_ready(e);
    if (rc) return rc;
    if (!tokens) return fail(SPB_E_INVALID, "spb_shard_engine_step: null pointer");
    for (int b = 0; b < e->batch; ++b)
        if (tokens[b] < 0 || tokens[b] >= e->cfg.vocab_size) return fail(SPB_E_INVALID, "spb_shard_engine_step: token outside the vocabulary");
    if (e->seq_len >= e->cfg.max_position_embeddings) return fail(SPB_E_INVALID, "spb_shard_engine_step: KV cache full");
    DeviceScope scope(e->device);
    if ((rc = ensure_graph(e, false, 0))) return rc;
    SPB_CUDA(cudaMemcpyAsync(e->d_next, tokens, sizeof(int) * e->batch, cudaMemcpyHostToDevice, e->stream));
    SPB_CUDA(cudaGraphLaunch(e->graph, e->stream));
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    e->seq_len++;
    return check_status(e, "spb_shard_engine_step");
}

extern "C" int spb_shard_engine_copy_logits(spb_shard_engine* e, float* h_logits_rows) {
    if (!e || !h_logits_rows) return fail(SPB_E_INVALID, "spb_shard_engine_copy_logits: null pointer");
    DeviceScope scope(e->device);
    SPB_CUDA(cudaMemcpyAsync(h_logits_rows, e->logits, sizeof(float) * e->batch * e->v_loc, cudaMemcpyDeviceToHost, e->stream));
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    return check_status(e, "spb_shard_engine_copy_logits");
}

extern "C" int spb_shard_engine_generate(spb_shard_engine* e, const int* prompt, int n_prompt, int max_tokens, int* out_tokens) {
    int rc = check_ready(e);
    if (rc) return rc;
    if (!prompt || n_prompt < 1 || max_tokens < 0 || (max_tokens > 0 && !out_tokens))
        return fail(SPB_E_INVALID, "spb_shard_engine_generate: bad arguments");
    const int B = e->batch, start = e->seq_len, steps = n_prompt - 1 + max_tokens;
    if (start + steps > e->cfg.max_position_embeddings || start + steps > e->out_cap)
        return fail(SPB_E_INVALID, "spb_shard_engine_generate: %d positions exceed the KV cache", start + steps);
    for (int i = 0; i < n_prompt * B; ++i)
        if (prompt[i] < 0 || prompt[i] >= e->cfg.vocab_size) return fail(SPB_E_INVALID, "spb_shard_engine_generate: token outside the vocabulary");
    DeviceScope scope(e->device);
    const int need = start + n_prompt;  // the prompt table is indexed by absolute position
    if (need > e->prompt_cap) {
        if (e->d_prompt) cudaFree(e->d_prompt);
        e->d_prompt = nullptr;
        const int cap = std::max(need, 1024);
        SPB_CUDA(cudaMalloc(&e->d_prompt, sizeof(int) * cap * B));
        e->prompt_cap = cap;
        drop_graph(e);
    }
    SPB_CUDA(cudaMemcpyAsync(e->d_prompt + static_cast<size_t>(start) * B, prompt, sizeof(int) * n_prompt * B, cudaMemcpyHostToDevice, e->stream));
    if ((rc = ensure_graph(e, true, need))) return rc;
    for (int s = 0; s < steps; ++s) SPB_CUDA(cudaGraphLaunch(e->graph, e->stream));
    e->seq_len += steps;
    if (max_tokens > 0)
        SPB_CUDA(cudaMemcpyAsync(out_tokens, e->d_out + static_cast<size_t>(start + n_prompt - 1) * B, sizeof(int) * max_tokens * B,
                                 cudaMemcpyDeviceToHost, e->stream));
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    if ((rc = check_status(e, "spb_shard_engine_generate"))) return rc;
    return max_tokens;
}
