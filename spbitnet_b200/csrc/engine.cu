// Host-side decode engine: the B200 counterpart of spbitnet::InferenceEngine
// (include/spbitnet/inference.h:23-70, src/inference.cu).  Same state (KV caches,
// scratch vectors, sequence position), same op order and rounding points as
// InferenceEngine::forward (src/inference.cu:123-283), but
//   * one pooled device allocation instead of ~75 cudaMallocs,
//   * the activation is quantised once per normed vector and shared by q/k/v and by
//     gate/up (the reference recomputes the same absmax 2-3 times, src/inference.cu:106-117),
//   * the small vector ops between GEMVs are fused (fused_ops.cu),
//   * the whole token is a CUDA graph of PDL-chained kernels whose position lives in
//     device memory, replayed once per token on a private stream,
//   * the arg-max of the greedy loop (src/main.cpp:285-287) runs on the device.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <new>
#include <vector>

#include "decode_persistent.cuh"
#include "fused_ops.cuh"

namespace spb {

struct Linear {
    const uint32_t* meta = nullptr;
    const uint32_t* values = nullptr;
    float gamma = 0.0f;
    int rows = 0, cols = 0, ms = 0, vs = 0;
    void* prep = nullptr;  // the engine's prepared copy (spb_prepare_weights), when it keeps one
};

struct Layer {
    Linear lin[7];             // q k v o gate up down
    const float* norm[4] = {};  // input_ln, post_attn_ln, attn_sub_norm, ffn_sub_norm
};

}  // namespace spb

using namespace spb;

struct spb_engine {
    spb_model_config cfg{};
    std::vector<Layer> layers;
    const __half* embed = nullptr;
    const __half* lm_head = nullptr;
    const float* final_norm = nullptr;

    int device = 0;
    cudaStream_t stream = nullptr;
    uint8_t* pool = nullptr;
    size_t pool_bytes = 0;
    size_t kv_bytes_per_layer = 0;
    __half *kcache = nullptr, *vcache = nullptr;
    __half *x = nullptr, *x2 = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *o = nullptr;
    __half *gate = nullptr, *up = nullptr, *down = nullptr, *xfinal = nullptr;
    int8_t* xq = nullptr;   // quantised activation, max(hidden, inter, heads*head_dim)
    float* absmax = nullptr;
    float* attn_scratch = nullptr;  // split-KV partial results
    unsigned* attn_counters = nullptr;  // per KV head: chunks written so far (zero between launches)
    bool split_attention = false;
    float* logits = nullptr;
    float* bval = nullptr;
    int* bidx = nullptr;
    int *d_pos = nullptr, *d_next = nullptr, *d_prompt = nullptr, *d_out = nullptr;
    int prompt_cap = 0;
    int n_prompt_in_graph = 0;
    int argmax_blocks = 0;

    cudaGraphExec_t graph = nullptr;  // one token, position and token read from device memory
    bool graph_generates = false;     // the captured graph records tokens into d_out
    bool fused = false;               // vector ops run inside the BitLinear launches
    bool rope_in_qkv = false;         // ... and rope + KV scatter inside the q/k/v launch
    int use_prepared = 1;             // spb_engine_set_prepared_weights
    int decode_mode = 0;              // spb_engine_set_decode_mode
    bool persistent = false;          // the layers of a token run as the one persistent kernel (decode_persistent.cu)
    PdModel pd{};
    PdLayer* d_pd_layers = nullptr;
    unsigned* d_pd_sync = nullptr;
    uint2* d_pd_ll = nullptr;         // tagged words of the barrier-free form (decode mode 4)
    size_t pd_ll_words = 0;
    int seq_len = 0;
    int timeouts_seen = 0;  // value of the library's bounded-wait counter when the engine last looked

    // batched prefill: buffers for `pf_cap` tokens at a time, allocated by the first call that needs them
    int prefill_chunk = 0;  // 0 = generate() feeds the prompt token by token, as the reference does
    int pf_cap = 0;
    uint8_t* pf_pool = nullptr;
    __half *pf_x = nullptr, *pf_q = nullptr, *pf_k = nullptr, *pf_v = nullptr, *pf_attn = nullptr, *pf_o = nullptr;
    __half *pf_gate = nullptr, *pf_up = nullptr, *pf_down = nullptr;
    int8_t* pf_xq = nullptr;
    int32_t* pf_acc = nullptr;
    float* pf_absmax = nullptr;  // two arrays of pf_cap
    int* pf_tokens = nullptr;
    // a chunk of T tokens replayed as a CUDA graph once the same (T, last) has been asked for twice in a row
    struct PrefillGraph { int T; bool last; cudaGraphExec_t exec; };
    std::vector<PrefillGraph> pf_graphs;
    int pf_prev_T = 0;
    bool pf_prev_last = false;
    // side streams for the products of a layer that do not depend on one another (k, v beside q; up beside gate)
    cudaStream_t pf_side[2] = {nullptr, nullptr};
    cudaEvent_t pf_fork = nullptr, pf_join[2] = {nullptr, nullptr};
};

namespace {

constexpr int kMaxTokensOut = 1 << 16;

int cuda_fail(const char* what, cudaError_t err) {
    cudaGetLastError();
    return fail(SPB_E_CUDA, "%s: %s", what, cudaGetErrorString(err));
}

#define SPB_CUDA(call)                                           \
    do {                                                         \
        cudaError_t err__ = (call);                              \
        if (err__ != cudaSuccess) return cuda_fail(#call, err__); \
    } while (0)

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Makes the engine's device current for the duration of an entry point and restores the caller's afterwards, so
// that launches, late allocations and graph work land on the GPU the engine was created on.
class DeviceScope {
public:
    explicit DeviceScope(int device) {
        if (cudaGetDevice(&prev_) != cudaSuccess) prev_ = -1;
        if (prev_ != device) {
            ok_ = cudaSetDevice(device) == cudaSuccess;
            switched_ = ok_;
        }
    }
    ~DeviceScope() {
        if (switched_ && prev_ >= 0) cudaSetDevice(prev_);
    }
    bool ok() const { return ok_; }

private:
    int prev_ = -1;
    bool ok_ = true, switched_ = false;
};

#define SPB_ON_ENGINE_DEVICE(e)                                                             \
    DeviceScope device_scope__((e)->device);                                                \
    if (!device_scope__.ok()) return fail(SPB_E_CUDA, "engine: cannot make device %d current", (e)->device)

// Called after the engine's stream has been synchronised: a tensor-core block of the batched product whose bounded
// wait ran out has skipped its epilogue, so whatever was computed since the last look is not to be trusted.
int check_timeouts(spb_engine* e, const char* where) {
    const int now = timeouts_now();
    if (now == e->timeouts_seen) return SPB_OK;
    const int n = now - e->timeouts_seen;
    e->timeouts_seen = now;
    return fail(SPB_E_TIMEOUT, "%s: %d bounded device-side wait(s) of the tensor-core product ran out; the outputs of "
                "this call are unspecified", where, n);
}

BitLinearGroup make_group(const Linear* const* L, __half* const* out, int n) {
    BitLinearGroup g{};
    g.nmat = n;
    g.cols = L[0]->cols;
    for (int i = 0; i < n; ++i) {
        g.meta[i] = L[i]->meta; g.values[i] = L[i]->values; g.out[i] = out[i]; g.gamma[i] = L[i]->gamma;
        g.rows[i] = L[i]->rows; g.ms[i] = L[i]->ms; g.vs[i] = L[i]->vs;
        g.prep[i] = L[i]->prep;
    }
    return g;
}

// Enqueues one token's worth of kernels on e->stream.  The first kernel reads the token
// (prompt[pos] while pos < n_prompt, else the previous arg-max) and the last advances pos.
// With layouts the fused-producer GEMV kernels take (every benchmark model), a layer is five
// launches: the vector ops between the BitLinears run inside the consuming launch, RoPE and the
// KV scatter inside the q/k/v launch, the merge of the attention chunks inside the attention
// launch.  In the persistent mode the layers of a token are one cooperative launch.
int enqueue_token(spb_engine* e, bool record_tokens) {
    const spb_model_config& c = e->cfg;
    const int H = c.hidden_size, hd = c.head_dim, nh = c.num_attention_heads, nkv = c.num_key_value_heads;
    const int inter = c.intermediate_size;
    void* s = e->stream;
    int rc;
    __half* cur = e->x;
    __half* other = e->x2;
    const float attn_scale = 1.0f / sqrtf(static_cast<float>(hd));
    if (e->persistent) {
        // embedding gather and every layer in one cooperative launch; the residual stream ends up in e->x
        e->pd.d_prompt = e->d_prompt;
        e->pd.n_prompt = e->n_prompt_in_graph;
        if ((rc = decode_persistent_launch(e->pd, 0, s))) return rc;
    } else if ((rc = embed_token(e->embed, cur, H, e->d_prompt, e->n_prompt_in_graph, e->d_next, e->d_pos, s))) {
        return rc;
    }
    for (int l = 0; l < c.num_hidden_layers && !e->persistent; ++l) {
        const Layer& L = e->layers[l];
        __half* kc = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(e->kcache) + l * e->kv_bytes_per_layer);
        __half* vc = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(e->vcache) + l * e->kv_bytes_per_layer);
        const Linear* g3[3] = {&L.lin[0], &L.lin[1], &L.lin[2]};
        __half* o3[3] = {e->q, e->k, e->v};
        const Linear* g1o[1] = {&L.lin[3]};
        __half* o1o[1] = {e->o};
        const Linear* g2[2] = {&L.lin[4], &L.lin[5]};
        __half* o2[2] = {e->gate, e->up};
        const Linear* g1d[1] = {&L.lin[6]};
        __half* o1d[1] = {e->down};
        if (e->fused) {
            // previous layer's down-projection residual add + input norm + quantise, inside q/k/v
            // ... and rope(q), rope(k), scatter of k and v into the caches as its epilogue
            const RopeScatter rs{e->d_pos, c.rope_theta, hd, c.max_position_embeddings, kc, vc};
            if ((rc = bitlinear_resnorm_group(make_group(g3, o3, 3), cur, l == 0 ? nullptr : e->down, nullptr, L.norm[0],
                                              other, c.rms_norm_eps, s, e->rope_in_qkv ? &rs : nullptr))) return rc;
            std::swap(cur, other);
        } else {
            if ((rc = residual_norm_quant(l == 0 ? nullptr : e->down, nullptr, cur, L.norm[0], nullptr, e->xq, e->absmax,
                                          H, c.rms_norm_eps, s))) return rc;
            if ((rc = bitlinear_q8_group(make_group(g3, o3, 3), e->xq, e->absmax, s))) return rc;
        }
        if (!(e->fused && e->rope_in_qkv) &&
            (rc = rope_scatter(e->q, e->k, e->v, kc, vc, nh, nkv, hd, c.max_position_embeddings, c.rope_theta, e->d_pos, s)))
            return rc;
        if (e->split_attention) {
            if ((rc = decode_attention_split(e->q, kc, vc, e->attn, nh, nkv, hd, c.max_position_embeddings, 0, e->d_pos,
                                             attn_scale, e->attn_scratch, s, e->fused ? e->attn_counters : nullptr))) return rc;
        } else if ((rc = decode_attention_pos(e->q, kc, vc, e->attn, nh, nkv, hd, c.max_position_embeddings,
                                              attn_scale, e->d_pos, s))) {
            return rc;
        }
        if (e->fused) {
            if ((rc = bitlinear_amax_group(make_group(g1o, o1o, 1), e->attn, s))) return rc;
            // attn_sub_norm -> residual add -> post-attention norm -> quantise, inside gate/up
            if ((rc = bitlinear_resnorm_group(make_group(g2, o2, 2), cur, e->o, L.norm[2], L.norm[1], other,
                                              c.rms_norm_eps, s))) return rc;
            std::swap(cur, other);
            // relu2 * up -> ffn_sub_norm -> quantise, inside down
            if ((rc = bitlinear_relu2_group(make_group(g1d, o1d, 1), e->gate, e->up, L.norm[3], c.rms_norm_eps, s))) return rc;
        } else {
            if ((rc = spb_absmax_quantize(e->attn, e->xq, e->absmax + 1, nh * hd, s))) return rc;
            if ((rc = bitlinear_q8_group(make_group(g1o, o1o, 1), e->xq, e->absmax + 1, s))) return rc;
            if ((rc = residual_norm_quant(e->o, L.norm[2], cur, L.norm[1], nullptr, e->xq, e->absmax, H, c.rms_norm_eps, s))) return rc;
            if ((rc = bitlinear_q8_group(make_group(g2, o2, 2), e->xq, e->absmax, s))) return rc;
            if ((rc = relu2_norm_quant(e->gate, e->up, L.norm[3], nullptr, e->xq, e->absmax + 1, inter, c.rms_norm_eps, s))) return rc;
            if ((rc = bitlinear_q8_group(make_group(g1d, o1d, 1), e->xq, e->absmax + 1, s))) return rc;
        }
    }
    // last residual add + final norm
    if ((rc = residual_norm_quant(c.num_hidden_layers ? e->down : nullptr, nullptr, cur, e->final_norm, e->xfinal,
                                  e->xq, e->absmax, H, c.rms_norm_eps, s))) return rc;
    if ((rc = spb_half_gemv(e->lm_head ? e->lm_head : e->embed, e->xfinal, e->logits, c.vocab_size, H, s))) return rc;
    return argmax_advance(e->logits, c.vocab_size, e->bval, e->bidx, e->argmax_blocks, e->d_next,
                          record_tokens ? e->d_out : nullptr, e->d_pos, s);
}

int check_ready(const spb_engine* e) {
    if (!e) return fail(SPB_E_INVALID, "engine: null handle");
    if (!e->embed || !e->final_norm) return fail(SPB_E_INVALID, "engine: globals not set");
    for (const Layer& L : e->layers) {
        for (int i = 0; i < 7; ++i)
            if (!L.lin[i].meta) return fail(SPB_E_INVALID, "engine: a linear layer has no weights attached");
        if (!L.norm[0] || !L.norm[1]) return fail(SPB_E_INVALID, "engine: a layer norm is missing");
    }
    return SPB_OK;
}

void drop_graph(spb_engine* e) {
    if (e->graph) {
        cudaGraphExecDestroy(e->graph);
        e->graph = nullptr;
    }
    for (auto& g : e->pf_graphs) cudaGraphExecDestroy(g.exec);
    e->pf_graphs.clear();
    e->pf_prev_T = 0;
}

// Decides whether the layers of a token run as the persistent kernel and, if so, hands it the model: the layer
// table goes to device memory here, outside any stream capture.
int choose_persistent(spb_engine* e) {
    e->persistent = false;
    if (e->decode_mode != 2 && e->decode_mode != 4) return SPB_OK;  // only on request
    const spb_model_config& c = e->cfg;
    const int qdim = c.num_attention_heads * c.head_dim, kvdim = c.num_key_value_heads * c.head_dim;
    PdModel m{};
    m.nlayers = c.num_hidden_layers;
    m.H = c.hidden_size; m.inter = c.intermediate_size; m.nh = c.num_attention_heads; m.nkv = c.num_key_value_heads;
    m.hd = c.head_dim; m.max_seq = c.max_position_embeddings;
    m.eps = c.rms_norm_eps; m.theta = c.rope_theta; m.attn_scale = 1.0f / sqrtf(static_cast<float>(c.head_dim));
    m.embed = e->embed;
    m.d_next = e->d_next; m.d_pos = e->d_pos;
    m.xa = e->x; m.xb = e->x2; m.q = e->q; m.attn = e->attn; m.o = e->o; m.gate = e->gate; m.up = e->up; m.down = e->down;
    m.scratch = e->attn_scratch;
    m.barrier_free = e->decode_mode == 4 ? 1 : 0;
    if (m.barrier_free) {
        if (!e->d_pd_ll) {
            e->pd_ll_words = decode_persistent_ll_words(m.H, m.inter, m.nh, m.nkv, m.hd);
            SPB_CUDA(cudaMalloc(&e->d_pd_ll, sizeof(uint2) * e->pd_ll_words));
            SPB_CUDA(cudaMemsetAsync(e->d_pd_ll, 0, sizeof(uint2) * e->pd_ll_words, e->stream));
        }
        m.ll = e->d_pd_ll;
    }
    const char* why = "";
    std::vector<PdLayer> host(e->layers.size());
    const int want_rows[7] = {qdim, kvdim, kvdim, c.hidden_size, c.intermediate_size, c.intermediate_size, c.hidden_size};
    const int want_cols[7] = {c.hidden_size, c.hidden_size, c.hidden_size, qdim, c.hidden_size, c.hidden_size, c.intermediate_size};
    bool ok = e->split_attention && !e->layers.empty();
    if (!ok) why = "attention shape";
    for (size_t l = 0; l < e->layers.size() && ok; ++l) {
        const Layer& L = e->layers[l];
        for (int i = 0; i < 7; ++i) {
            if (L.lin[i].rows != want_rows[i] || L.lin[i].cols != want_cols[i]) {
                ok = false;
                why = "a matrix does not have the shape the model config implies";
            }
            host[l].lin[i] = PdLinear{L.lin[i].meta, L.lin[i].values, L.lin[i].gamma, L.lin[i].ms, L.lin[i].vs};
        }
        for (int i = 0; i < 4; ++i) host[l].norm[i] = L.norm[i];
        host[l].kc = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(e->kcache) + l * e->kv_bytes_per_layer);
        host[l].vc = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(e->vcache) + l * e->kv_bytes_per_layer);
        if (ok && !decode_persistent_supported(m, host[l].lin, &why)) ok = false;
    }
    if (!ok) {
        return fail(SPB_E_UNSUPPORTED, "engine: the persistent decode step does not take this model: %s", why);
    }
    // Both transfers go through the engine's own stream (it does not synchronise with the null stream) and are
    // waited for here: the kernel must not start before its tables are in place.
    if (!e->d_pd_layers) SPB_CUDA(cudaMalloc(&e->d_pd_layers, sizeof(PdLayer) * host.size()));
    if (!e->d_pd_sync) {
        SPB_CUDA(cudaMalloc(&e->d_pd_sync, sizeof(unsigned) * (kPdSyncWords + c.num_key_value_heads)));
        SPB_CUDA(cudaMemsetAsync(e->d_pd_sync, 0, sizeof(unsigned) * (kPdSyncWords + c.num_key_value_heads), e->stream));
    }
    SPB_CUDA(cudaMemcpyAsync(e->d_pd_layers, host.data(), sizeof(PdLayer) * host.size(), cudaMemcpyHostToDevice, e->stream));
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    m.layers = e->d_pd_layers;
    m.sync = e->d_pd_sync;
    e->pd = m;
    e->persistent = true;
    return SPB_OK;
}

// The engine's prepared copies of the matrices (the chain of fused launches multiplies on them, gemv_prepared.cu):
// built here, outside any capture, for every matrix the layout takes; dropped when the setting or the mode says so.
int sync_prepared(spb_engine* e, bool want) {
    bool waited = false;
    for (Layer& Ly : e->layers)
        for (Linear& L : Ly.lin) {
            const size_t bytes = want && L.meta ? spb_prepared_weights_bytes(L.rows, L.cols) : 0;
            const bool can = bytes > 0 && L.ms >= L.cols / 32 && L.vs >= L.cols / 64;
            if (L.prep && !can) {
                if (!waited) SPB_CUDA(cudaStreamSynchronize(e->stream));
                waited = true;
                cudaFree(L.prep);
                L.prep = nullptr;
            } else if (!L.prep && can) {
                SPB_CUDA(cudaMalloc(&L.prep, bytes));
                if (int rc = spb_prepare_weights(L.meta, L.values, L.rows, L.cols, L.ms, L.vs, L.prep, e->stream)) return rc;
            }
        }
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    return SPB_OK;
}

int ensure_graph(spb_engine* e, bool record_tokens, int n_prompt) {
    if (e->graph && e->graph_generates == record_tokens && e->n_prompt_in_graph == n_prompt) return SPB_OK;
    drop_graph(e);
    e->n_prompt_in_graph = n_prompt;
    e->fused = e->decode_mode != 3;
    if (int rc = choose_persistent(e)) return rc;
    for (const Layer& L : e->layers) {
        const Linear* all[7] = {&L.lin[0], &L.lin[1], &L.lin[2], &L.lin[3], &L.lin[4], &L.lin[5], &L.lin[6]};
        __half* none[7] = {};
        for (int i = 0; i < 7 && e->fused; ++i) e->fused = bitlinear_group_is_fast(make_group(all + i, none + i, 1));
    }
    if (int rc = sync_prepared(e, e->use_prepared && e->fused && !e->persistent)) return rc;
    e->rope_in_qkv = e->fused && e->cfg.head_dim % 2 == 0;
    SPB_CUDA(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_token(e, record_tokens);
    cudaGraph_t g = nullptr;
    cudaError_t err = cudaStreamEndCapture(e->stream, &g);
    if (rc) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (err != cudaSuccess) return cuda_fail("cudaStreamEndCapture", err);
    err = cudaGraphInstantiate(&e->graph, g, 0);
    cudaGraphDestroy(g);
    if (err != cudaSuccess) return cuda_fail("cudaGraphInstantiate", err);
    e->graph_generates = record_tokens;
    return SPB_OK;
}

// ---- batched prefill -------------------------------------------------------------------------------
// T prompt tokens go through a layer together: the BitLinear layers run as the batched product
// (spb_sparse_ternary_gemm, one activation row per token, integer-exact) followed by a per-row dequantise,
// the vector ops as one block per token, attention as one block per (head, token) over the positions up to
// the token's own.  Every rounding point of the token-serial step is kept, so the integer accumulators and
// the quantised activations are the ones forward() produces token by token; only the attention sums are
// formed in a different order (the split-KV kernel is not used here).

constexpr int kPrefillMaxChunk = 1024;  // larger batches amortise the re-encoding of a weight tile over more activation rows

int ensure_prefill_buffers(spb_engine* e, int cap) {
    if (e->pf_cap >= cap) return SPB_OK;
    if (e->pf_pool) {
        SPB_CUDA(cudaStreamSynchronize(e->stream));
        for (auto& g : e->pf_graphs) cudaGraphExecDestroy(g.exec);  // they hold the old addresses
        e->pf_graphs.clear();
        e->pf_prev_T = 0;
        cudaFree(e->pf_pool);
        e->pf_pool = nullptr;
        e->pf_cap = 0;
    }
    const spb_model_config& c = e->cfg;
    const size_t T = static_cast<size_t>(cap);
    const size_t H = c.hidden_size, qdim = static_cast<size_t>(c.num_attention_heads) * c.head_dim;
    const size_t kvdim = static_cast<size_t>(c.num_key_value_heads) * c.head_dim, inter = c.intermediate_size;
    const size_t maxdim = std::max(std::max(H, qdim), inter);
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
    const size_t o_x = take(2 * T * H), o_q = take(2 * T * qdim), o_k = take(2 * T * kvdim), o_v = take(2 * T * kvdim);
    const size_t o_attn = take(2 * T * qdim), o_o = take(2 * T * H), o_gate = take(2 * T * inter);
    const size_t o_up = take(2 * T * inter), o_down = take(2 * T * H), o_xq = take(T * maxdim);
    const size_t o_acc = take(3 * 4 * T * maxdim), o_abs = take(4 * 2 * T), o_tok = take(4 * T);
    SPB_CUDA(cudaMalloc(&e->pf_pool, off));
    if (!e->pf_fork) {
        SPB_CUDA(cudaEventCreateWithFlags(&e->pf_fork, cudaEventDisableTiming));
        for (int i = 0; i < 2; ++i) {
            SPB_CUDA(cudaStreamCreateWithFlags(&e->pf_side[i], cudaStreamNonBlocking));
            SPB_CUDA(cudaEventCreateWithFlags(&e->pf_join[i], cudaEventDisableTiming));
        }
    }
    uint8_t* p = e->pf_pool;
    e->pf_x = reinterpret_cast<__half*>(p + o_x);
    e->pf_q = reinterpret_cast<__half*>(p + o_q);
    e->pf_k = reinterpret_cast<__half*>(p + o_k);
    e->pf_v = reinterpret_cast<__half*>(p + o_v);
    e->pf_attn = reinterpret_cast<__half*>(p + o_attn);
    e->pf_o = reinterpret_cast<__half*>(p + o_o);
    e->pf_gate = reinterpret_cast<__half*>(p + o_gate);
    e->pf_up = reinterpret_cast<__half*>(p + o_up);
    e->pf_down = reinterpret_cast<__half*>(p + o_down);
    e->pf_xq = reinterpret_cast<int8_t*>(p + o_xq);
    e->pf_acc = reinterpret_cast<int32_t*>(p + o_acc);
    e->pf_absmax = reinterpret_cast<float*>(p + o_abs);
    e->pf_tokens = reinterpret_cast<int*>(p + o_tok);
    e->pf_cap = cap;
    return SPB_OK;
}

// out[t] = BitLinear(L) of the T quantised rows in pf_xq with the row scales `absmax`
int prefill_linear(spb_engine* e, const Linear& L, const float* absmax, __half* out, int T, cudaStream_t stream,
                   int32_t* acc) {
    return spb_sparse_bitlinear_gemm(L.meta, L.values, e->pf_xq, out, absmax, L.gamma, acc, L.rows, L.cols, T, L.ms,
                                     L.vs, stream);
}

// Up to three BitLinear layers on the same quantised rows: the first on the engine's stream, the others on side
// streams between a fork and a join event (graph capture turns these into parallel branches), so that products
// with few row tiles share the machine.  Each gets its own third of the int32 workspace.
int prefill_linear_group(spb_engine* e, const Linear* const* L, __half* const* out, int n, const float* absmax, int T) {
    const spb_model_config& c = e->cfg;
    const size_t maxdim = std::max(std::max(static_cast<size_t>(c.hidden_size),
                                            static_cast<size_t>(c.num_attention_heads) * c.head_dim),
                                   static_cast<size_t>(c.intermediate_size));
    const size_t third = static_cast<size_t>(e->pf_cap) * maxdim;  // pf_acc holds three of these
    SPB_CUDA(cudaEventRecord(e->pf_fork, e->stream));
    for (int i = 1; i < n; ++i) {
        SPB_CUDA(cudaStreamWaitEvent(e->pf_side[i - 1], e->pf_fork, 0));
        if (int rc = prefill_linear(e, *L[i], absmax, out[i], T, e->pf_side[i - 1], e->pf_acc + i * third)) return rc;
        SPB_CUDA(cudaEventRecord(e->pf_join[i - 1], e->pf_side[i - 1]));
    }
    if (int rc = prefill_linear(e, *L[0], absmax, out[0], T, e->stream, e->pf_acc)) return rc;
    for (int i = 1; i < n; ++i) SPB_CUDA(cudaStreamWaitEvent(e->stream, e->pf_join[i - 1], 0));
    return SPB_OK;
}

// Tokens d_tokens[0..T) at positions start..start+T-1 (T <= pf_cap); *d_pos must hold `start`.  With `last`
// the logits of the final token are formed as well.
int enqueue_prefill_chunk(spb_engine* e, int T, bool last) {
    const spb_model_config& c = e->cfg;
    const int H = c.hidden_size, hd = c.head_dim, nh = c.num_attention_heads, nkv = c.num_key_value_heads;
    const int inter = c.intermediate_size;
    void* s = e->stream;
    float* am0 = e->pf_absmax;
    float* am1 = e->pf_absmax + e->pf_cap;
    int rc;
    if ((rc = embed_rows(e->embed, e->pf_tokens, e->pf_x, H, T, s))) return rc;
    const float attn_scale = 1.0f / sqrtf(static_cast<float>(hd));
    for (int l = 0; l < c.num_hidden_layers; ++l) {
        const Layer& L = e->layers[l];
        __half* kc = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(e->kcache) + l * e->kv_bytes_per_layer);
        __half* vc = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(e->vcache) + l * e->kv_bytes_per_layer);
        if ((rc = residual_norm_quant(l == 0 ? nullptr : e->pf_down, nullptr, e->pf_x, L.norm[0], nullptr, e->pf_xq,
                                      am0, H, c.rms_norm_eps, s, T))) return rc;
        {
            const Linear* g[3] = {&L.lin[0], &L.lin[1], &L.lin[2]};
            __half* o[3] = {e->pf_q, e->pf_k, e->pf_v};
            if ((rc = prefill_linear_group(e, g, o, 3, am0, T))) return rc;
        }
        if ((rc = rope_scatter(e->pf_q, e->pf_k, e->pf_v, kc, vc, nh, nkv, hd, c.max_position_embeddings,
                               c.rope_theta, e->d_pos, s, T))) return rc;
        if ((rc = decode_attention_pos(e->pf_q, kc, vc, e->pf_attn, nh, nkv, hd, c.max_position_embeddings,
                                       attn_scale, e->d_pos, s, T))) return rc;
        if ((rc = absmax_quantize_rows(e->pf_attn, e->pf_xq, am1, nh * hd, T, s))) return rc;
        if ((rc = prefill_linear(e, L.lin[3], am1, e->pf_o, T, e->stream, e->pf_acc))) return rc;
        if ((rc = residual_norm_quant(e->pf_o, L.norm[2], e->pf_x, L.norm[1], nullptr, e->pf_xq, am0, H,
                                      c.rms_norm_eps, s, T))) return rc;
        {
            const Linear* g[2] = {&L.lin[4], &L.lin[5]};
            __half* o[2] = {e->pf_gate, e->pf_up};
            if ((rc = prefill_linear_group(e, g, o, 2, am0, T))) return rc;
        }
        if ((rc = relu2_norm_quant(e->pf_gate, e->pf_up, L.norm[3], nullptr, e->pf_xq, am1, inter, c.rms_norm_eps,
                                   s, T))) return rc;
        if ((rc = prefill_linear(e, L.lin[6], am1, e->pf_down, T, e->stream, e->pf_acc))) return rc;
    }
    if (!last) return SPB_OK;
    // only the final token's logits are ever read: last residual add + final norm + lm_head on its row
    const size_t row = static_cast<size_t>(T - 1) * H;
    if ((rc = residual_norm_quant(c.num_hidden_layers ? e->pf_down + row : nullptr, nullptr, e->pf_x + row,
                                  e->final_norm, e->xfinal, e->xq, e->absmax, H, c.rms_norm_eps, s))) return rc;
    return spb_half_gemv(e->lm_head ? e->lm_head : e->embed, e->xfinal, e->logits, c.vocab_size, H, s);
}

// A chunk is some 500 launches; issued one by one the host is slower than the GPU.  All of a chunk's operands sit at
// fixed addresses (batch buffers, device-resident position), so the chunk is captured as a graph when the same
// (T, last) comes twice in a row (full chunks of a long prompt, prompts of one length) and replayed from then on.
int run_prefill_chunk(spb_engine* e, int T, bool last) {
    for (const auto& g : e->pf_graphs)
        if (g.T == T && g.last == last) {
            SPB_CUDA(cudaGraphLaunch(g.exec, e->stream));
            return SPB_OK;
        }
    const bool repeat = e->pf_prev_T == T && e->pf_prev_last == last;
    e->pf_prev_T = T;
    e->pf_prev_last = last;
    if (!repeat) return enqueue_prefill_chunk(e, T, last);
    SPB_CUDA(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    const int rc = enqueue_prefill_chunk(e, T, last);
    cudaGraph_t g = nullptr;
    cudaError_t err = cudaStreamEndCapture(e->stream, &g);
    if (rc) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (err != cudaSuccess) return cuda_fail("cudaStreamEndCapture", err);
    cudaGraphExec_t exec = nullptr;
    err = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (err != cudaSuccess) return cuda_fail("cudaGraphInstantiate", err);
    if (e->pf_graphs.size() >= 4) {
        cudaGraphExecDestroy(e->pf_graphs.front().exec);
        e->pf_graphs.erase(e->pf_graphs.begin());
    }
    e->pf_graphs.push_back({T, last, exec});
    SPB_CUDA(cudaGraphLaunch(exec, e->stream));
    return SPB_OK;
}

// Runs tokens[0..n) (HOST array) through the model from position e->seq_len in chunks; leaves the logits of
// the last one in e->logits, *d_pos = e->seq_len = old + n.  Validated by the caller.
int prefill_tokens(spb_engine* e, const int* tokens, int n) {
    const int chunk = std::min(e->prefill_chunk > 0 ? e->prefill_chunk : kPrefillMaxChunk, kPrefillMaxChunk);
    int rc = ensure_prefill_buffers(e, std::min(chunk, std::max(n, 1)));
    if (rc) return rc;
    const int cap = std::min(chunk, e->pf_cap);
    for (int done = 0; done < n; done += cap) {
        const int T = std::min(cap, n - done);
        // the token ids are consumed by the first kernel of the chunk; the copy is ordered before it on the stream
        SPB_CUDA(cudaMemcpyAsync(e->pf_tokens, tokens + done, sizeof(int) * T, cudaMemcpyHostToDevice, e->stream));
        if ((rc = set_int(e->d_pos, e->seq_len, e->stream))) return rc;
        if ((rc = run_prefill_chunk(e, T, done + T == n))) return rc;
        e->seq_len += T;  // the next chunk's copy into pf_tokens is ordered after this chunk's kernels by the stream
    }
    return set_int(e->d_pos, e->seq_len, e->stream);
}

}  // namespace

extern "C" spb_engine* spb_engine_create(const spb_model_config* cfg) {
    if (!cfg || cfg->hidden_size <= 0 || cfg->num_hidden_layers < 0 || cfg->num_attention_heads <= 0 ||
        cfg->num_key_value_heads <= 0 || cfg->head_dim <= 0 || cfg->head_dim % 2 || cfg->intermediate_size <= 0 ||
        cfg->vocab_size <= 0 || cfg->max_position_embeddings <= 0) {
        fail(SPB_E_INVALID, "spb_engine_create: bad config");
        return nullptr;
    }
    spb_engine* e = new (std::nothrow) spb_engine();
    if (!e) return nullptr;
    e->cfg = *cfg;
    e->layers.resize(cfg->num_hidden_layers);
    cudaGetDevice(&e->device);
    const int H = cfg->hidden_size, qdim = cfg->num_attention_heads * cfg->head_dim;
    const int kvdim = cfg->num_key_value_heads * cfg->head_dim, inter = cfg->intermediate_size;
    const int maxdim = std::max(std::max(H, qdim), inter);
    e->kv_bytes_per_layer = align_up(sizeof(__half) * static_cast<size_t>(kvdim) * cfg->max_position_embeddings, 256);
    e->argmax_blocks = std::max(1, std::min(128, (cfg->vocab_size + 1023) / 1024));

    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
    const size_t o_kc = take(e->kv_bytes_per_layer * cfg->num_hidden_layers);
    const size_t o_vc = take(e->kv_bytes_per_layer * cfg->num_hidden_layers);
    const size_t o_x = take(2 * H), o_x2 = take(2 * H), o_q = take(2 * qdim), o_k = take(2 * kvdim), o_v = take(2 * kvdim);
    const size_t o_attn = take(2 * qdim), o_o = take(2 * H), o_gate = take(2 * inter), o_up = take(2 * inter);
    const size_t o_down = take(2 * H), o_xf = take(2 * H), o_xq = take(maxdim), o_abs = take(16);
    const size_t o_logits = take(4 * static_cast<size_t>(cfg->vocab_size));
    e->split_attention = decode_attention_split_supported(cfg->num_attention_heads, cfg->num_key_value_heads, cfg->head_dim);
    const size_t o_ascr = take(decode_attention_scratch_bytes(cfg->num_attention_heads, cfg->head_dim,
                                                              cfg->max_position_embeddings));
    const size_t o_actr = take(4 * static_cast<size_t>(cfg->num_key_value_heads));
    const size_t o_bval = take(4 * 128), o_bidx = take(4 * 128), o_ints = take(16);
    const size_t o_out = take(4 * static_cast<size_t>(kMaxTokensOut));
    e->pool_bytes = off;
    if (cudaMalloc(&e->pool, e->pool_bytes) != cudaSuccess || cudaMemset(e->pool, 0, e->pool_bytes) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess ||  // the fill runs on the null stream, the engine on a stream that does not wait for it
        cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess) {
        cuda_fail("spb_engine_create", cudaGetLastError());
        if (e->pool) cudaFree(e->pool);
        delete e;
        return nullptr;
    }
    uint8_t* p = e->pool;
    e->kcache = reinterpret_cast<__half*>(p + o_kc);
    e->vcache = reinterpret_cast<__half*>(p + o_vc);
    e->x = reinterpret_cast<__half*>(p + o_x);
    e->x2 = reinterpret_cast<__half*>(p + o_x2);
    e->q = reinterpret_cast<__half*>(p + o_q);
    e->k = reinterpret_cast<__half*>(p + o_k);
    e->v = reinterpret_cast<__half*>(p + o_v);
    e->attn = reinterpret_cast<__half*>(p + o_attn);
    e->o = reinterpret_cast<__half*>(p + o_o);
    e->gate = reinterpret_cast<__half*>(p + o_gate);
    e->up = reinterpret_cast<__half*>(p + o_up);
    e->down = reinterpret_cast<__half*>(p + o_down);
    e->xfinal = reinterpret_cast<__half*>(p + o_xf);
    e->xq = reinterpret_cast<int8_t*>(p + o_xq);
    e->absmax = reinterpret_cast<float*>(p + o_abs);
    e->logits = reinterpret_cast<float*>(p + o_logits);
    e->attn_scratch = reinterpret_cast<float*>(p + o_ascr);
    e->attn_counters = reinterpret_cast<unsigned*>(p + o_actr);
    e->bval = reinterpret_cast<float*>(p + o_bval);
    e->bidx = reinterpret_cast<int*>(p + o_bidx);
    e->d_pos = reinterpret_cast<int*>(p + o_ints);
    e->d_next = e->d_pos + 1;
    e->d_out = reinterpret_cast<int*>(p + o_out);
    prepare_host_state();
    e->timeouts_seen = timeouts_now();
    return e;
}

extern "C" void spb_engine_destroy(spb_engine* e) {
    if (!e) return;
    DeviceScope scope(e->device);
    cudaStreamSynchronize(e->stream);
    drop_graph(e);
    if (e->d_prompt) cudaFree(e->d_prompt);
    if (e->pf_pool) cudaFree(e->pf_pool);
    for (int i = 0; i < 2; ++i) {
        if (e->pf_side[i]) cudaStreamDestroy(e->pf_side[i]);
        if (e->pf_join[i]) cudaEventDestroy(e->pf_join[i]);
    }
    if (e->pf_fork) cudaEventDestroy(e->pf_fork);
    if (e->d_pd_layers) cudaFree(e->d_pd_layers);
    if (e->d_pd_sync) cudaFree(e->d_pd_sync);
    if (e->d_pd_ll) cudaFree(e->d_pd_ll);
    for (Layer& Ly : e->layers)
        for (Linear& L : Ly.lin)
            if (L.prep) cudaFree(L.prep);
    cudaFree(e->pool);
    cudaStreamDestroy(e->stream);
    delete e;
}

extern "C" int spb_engine_set_linear(spb_engine* e, int layer, int which, const uint32_t* d_meta,
                                     const uint32_t* d_values, float gamma, int rows, int cols,
                                     int meta_stride, int values_stride) {
    if (!e || layer < 0 || layer >= static_cast<int>(e->layers.size()) || which < 0 || which > 6)
        return fail(SPB_E_INVALID, "spb_engine_set_linear: bad layer/which");
    if (!d_meta || !d_values || rows <= 0 || cols <= 0 || cols % 4)
        return fail(SPB_E_INVALID, "spb_engine_set_linear: bad tensor");
    const spb_model_config& c = e->cfg;
    const int qdim = c.num_attention_heads * c.head_dim, kvdim = c.num_key_value_heads * c.head_dim;
    const int want_rows[7] = {qdim, kvdim, kvdim, c.hidden_size, c.intermediate_size, c.intermediate_size, c.hidden_size};
    const int want_cols[7] = {c.hidden_size, c.hidden_size, c.hidden_size, qdim, c.hidden_size, c.hidden_size, c.intermediate_size};
    if (rows != want_rows[which] || cols != want_cols[which])
        return fail(SPB_E_INVALID, "spb_engine_set_linear: layer %d tensor %d is %dx%d, config wants %dx%d", layer,
                    which, rows, cols, want_rows[which], want_cols[which]);
    Linear& L = e->layers[layer].lin[which];
    drop_graph(e);
    if (L.prep) {  // a copy of the tensor this one replaces
        SPB_ON_ENGINE_DEVICE(e);
        SPB_CUDA(cudaStreamSynchronize(e->stream));
        cudaFree(L.prep);
        L.prep = nullptr;
    }
    L.meta = d_meta; L.values = d_values; L.gamma = gamma; L.rows = rows; L.cols = cols;
    L.ms = meta_stride; L.vs = values_stride;
    return SPB_OK;
}

extern "C" int spb_engine_set_norm(spb_engine* e, int layer, int which, const float* d_weight) {
    if (!e || layer < 0 || layer >= static_cast<int>(e->layers.size()) || which < 0 || which > 3)
        return fail(SPB_E_INVALID, "spb_engine_set_norm: bad layer/which");
    e->layers[layer].norm[which] = d_weight;
    drop_graph(e);
    return SPB_OK;
}

extern "C" int spb_engine_set_globals(spb_engine* e, const void* d_embed, const void* d_lm_head,
                                      const float* d_final_norm) {
    if (!e || !d_embed || !d_final_norm) return fail(SPB_E_INVALID, "spb_engine_set_globals: null pointer");
    e->embed = static_cast<const __half*>(d_embed);
    e->lm_head = static_cast<const __half*>(d_lm_head);
    e->final_norm = d_final_norm;
    drop_graph(e);
    return SPB_OK;
}

extern "C" int spb_engine_forward(spb_engine* e, int token_id, const float** d_logits) {
    int rc = check_ready(e);
    if (rc) return rc;
    if (token_id < 0 || token_id >= e->cfg.vocab_size) return fail(SPB_E_INVALID, "spb_engine_forward: token %d outside the vocabulary", token_id);
    if (e->seq_len >= e->cfg.max_position_embeddings) return fail(SPB_E_INVALID, "spb_engine_forward: KV cache full (%d)", e->seq_len);
    SPB_ON_ENGINE_DEVICE(e);
    if ((rc = ensure_graph(e, false, 0))) return rc;
    if ((rc = set_int(e->d_next, token_id, e->stream))) return rc;
    SPB_CUDA(cudaGraphLaunch(e->graph, e->stream));
    e->seq_len++;
    if (d_logits) {
        // The reference returns after enqueueing on the null stream; this engine runs on a
        // private stream, so make the result visible to whoever reads it next.
        SPB_CUDA(cudaStreamSynchronize(e->stream));
        *d_logits = e->logits;
    }
    return SPB_OK;
}

extern "C" int spb_engine_prefill(spb_engine* e, const int* tokens, int n, const float** d_logits) {
    int rc = check_ready(e);
    if (rc) return rc;
    if (!tokens || n < 1) return fail(SPB_E_INVALID, "spb_engine_prefill: no tokens");
    if (e->seq_len + n > e->cfg.max_position_embeddings)
        return fail(SPB_E_INVALID, "spb_engine_prefill: %d positions exceed the KV cache (%d)", e->seq_len + n,
                    e->cfg.max_position_embeddings);
    for (int i = 0; i < n; ++i)
        if (tokens[i] < 0 || tokens[i] >= e->cfg.vocab_size)
            return fail(SPB_E_INVALID, "spb_engine_prefill: token %d outside the vocabulary", tokens[i]);
    SPB_ON_ENGINE_DEVICE(e);
    if ((rc = prefill_tokens(e, tokens, n))) return rc;
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    if ((rc = check_timeouts(e, "spb_engine_prefill"))) return rc;
    if (d_logits) *d_logits = e->logits;
    return SPB_OK;
}

extern "C" int spb_engine_set_prefill_chunk(spb_engine* e, int chunk) {
    if (!e) return fail(SPB_E_INVALID, "spb_engine_set_prefill_chunk: null handle");
    if (chunk < 0) return fail(SPB_E_INVALID, "spb_engine_set_prefill_chunk: negative chunk");
    const int prev = e->prefill_chunk;
    e->prefill_chunk = std::min(chunk, kPrefillMaxChunk);
    return prev;
}

extern "C" int spb_engine_reset(spb_engine* e) {
    if (!e) return fail(SPB_E_INVALID, "spb_engine_reset: null handle");
    SPB_ON_ENGINE_DEVICE(e);
    const size_t kv_total = e->kv_bytes_per_layer * e->cfg.num_hidden_layers;
    SPB_CUDA(cudaMemsetAsync(e->kcache, 0, kv_total, e->stream));
    SPB_CUDA(cudaMemsetAsync(e->vcache, 0, kv_total, e->stream));
    SPB_CUDA(cudaMemsetAsync(e->d_pos, 0, 16, e->stream));
    // barrier words of the persistent step: a launch that gave up at a barrier leaves them marked broken
    if (e->d_pd_sync)
        SPB_CUDA(cudaMemsetAsync(e->d_pd_sync, 0, sizeof(unsigned) * (kPdSyncWords + e->cfg.num_key_value_heads), e->stream));
    // the tags of the barrier-free form start over with the launch count: no word of an earlier run may stay
    if (e->d_pd_ll) SPB_CUDA(cudaMemsetAsync(e->d_pd_ll, 0, sizeof(uint2) * e->pd_ll_words, e->stream));
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    e->seq_len = 0;
    return SPB_OK;
}

extern "C" int spb_engine_set_decode_mode(spb_engine* e, int mode) {
    if (!e) return fail(SPB_E_INVALID, "spb_engine_set_decode_mode: null handle");
    if (mode < 0 || mode > 4) return fail(SPB_E_INVALID, "spb_engine_set_decode_mode: mode %d", mode);
    SPB_ON_ENGINE_DEVICE(e);
    if (mode != e->decode_mode) {
        SPB_CUDA(cudaStreamSynchronize(e->stream));
        drop_graph(e);
        e->decode_mode = mode;
    }
    return SPB_OK;
}

extern "C" int spb_engine_set_prepared_weights(spb_engine* e, int on) {
    if (!e) return fail(SPB_E_INVALID, "spb_engine_set_prepared_weights: null handle");
    SPB_ON_ENGINE_DEVICE(e);
    if ((on != 0) != (e->use_prepared != 0)) {
        SPB_CUDA(cudaStreamSynchronize(e->stream));
        drop_graph(e);
        e->use_prepared = on != 0;
    }
    return SPB_OK;
}

extern "C" int spb_engine_decode_is_persistent(const spb_engine* e) { return e && e->persistent ? 1 : 0; }

extern "C" int spb_engine_seq_len(const spb_engine* e) { return e ? e->seq_len : 0; }

extern "C" int spb_engine_copy_logits(spb_engine* e, float* h_logits) {
    if (!e || !h_logits) return fail(SPB_E_INVALID, "spb_engine_copy_logits: null pointer");
    SPB_ON_ENGINE_DEVICE(e);
    SPB_CUDA(cudaMemcpyAsync(h_logits, e->logits, sizeof(float) * e->cfg.vocab_size, cudaMemcpyDeviceToHost, e->stream));
    SPB_CUDA(cudaStreamSynchronize(e->stream));
    return check_timeouts(e, "spb_engine_copy_logits");
}

static int generate_impl(spb_engine* e, const int* prompt, int n_prompt, int max_tokens, int eos_token_id,
                         int* out_tokens);

extern "C" int spb_engine_generate(spb_engine* e, const int* prompt, int n_prompt, int max_tokens,
                                   int eos_token_id, int* out_tokens) {
    int rc = check_ready(e);
    if (rc) return rc;
    SPB_ON_ENGINE_DEVICE(e);
    const int produced = generate_impl(e, prompt, n_prompt, max_tokens, eos_token_id, out_tokens);
    if (produced < 0) return produced;
    // every path of generate_impl ends with the stream synchronised
    if ((rc = check_timeouts(e, "spb_engine_generate"))) return rc;
    return produced;
}

static int generate_impl(spb_engine* e, const int* prompt, int n_prompt, int max_tokens, int eos_token_id,
                         int* out_tokens) {
    int rc;
    if (!prompt || n_prompt < 1 || max_tokens < 0 || (max_tokens > 0 && !out_tokens))
        return fail(SPB_E_INVALID, "spb_engine_generate: bad arguments");
    const int start = e->seq_len;
    const int steps = n_prompt - 1 + max_tokens;
    if (start + steps > e->cfg.max_position_embeddings || start + steps > kMaxTokensOut)
        return fail(SPB_E_INVALID, "spb_engine_generate: %d positions exceed the KV cache", start + steps);
    for (int i = 0; i < n_prompt; ++i)
        if (prompt[i] < 0 || prompt[i] >= e->cfg.vocab_size)
            return fail(SPB_E_INVALID, "spb_engine_generate: prompt token %d outside the vocabulary", prompt[i]);
    // The prompt table is indexed by absolute position.
    const int need = start + n_prompt;
    if (need > e->prompt_cap) {
        if (e->d_prompt) cudaFree(e->d_prompt);
        e->d_prompt = nullptr;
        const int cap = std::max(need, 1024);
        SPB_CUDA(cudaMalloc(&e->d_prompt, sizeof(int) * cap));
        e->prompt_cap = cap;
        drop_graph(e);
    }
    SPB_CUDA(cudaMemcpyAsync(e->d_prompt + start, prompt, sizeof(int) * n_prompt, cudaMemcpyHostToDevice, e->stream));
    if ((rc = ensure_graph(e, true, need))) return rc;
    int produced = 0;
    if (e->prefill_chunk > 0 && n_prompt >= 2) {
        // The prompt as a batch; the first generated token comes from its last logits, the rest from the
        // per-token graph.  Positions and recorded tokens end up where the token-serial loop puts them.
        if (max_tokens == 0) {
            if ((rc = prefill_tokens(e, prompt, n_prompt - 1))) return rc;
            SPB_CUDA(cudaStreamSynchronize(e->stream));
            return 0;
        }
        if ((rc = prefill_tokens(e, prompt, n_prompt))) return rc;
        if ((rc = set_int(e->d_pos, e->seq_len - 1, e->stream))) return rc;
        if ((rc = argmax_advance(e->logits, e->cfg.vocab_size, e->bval, e->bidx, e->argmax_blocks, e->d_next, e->d_out,
                                 e->d_pos, e->stream))) return rc;
        const int first_slot = start + n_prompt - 1;
        if (eos_token_id < 0) {
            for (int s = 1; s < max_tokens; ++s) SPB_CUDA(cudaGraphLaunch(e->graph, e->stream));
            e->seq_len += max_tokens - 1;
            SPB_CUDA(cudaMemcpyAsync(out_tokens, e->d_out + first_slot, sizeof(int) * max_tokens, cudaMemcpyDeviceToHost,
                                     e->stream));
            SPB_CUDA(cudaStreamSynchronize(e->stream));
            return max_tokens;
        }
        for (int t = 0; t < max_tokens; ++t) {
            if (t > 0) {
                SPB_CUDA(cudaGraphLaunch(e->graph, e->stream));
                e->seq_len++;
            }
            SPB_CUDA(cudaMemcpyAsync(out_tokens + t, e->d_out + first_slot + t, sizeof(int), cudaMemcpyDeviceToHost,
                                     e->stream));
            SPB_CUDA(cudaStreamSynchronize(e->stream));
            produced = t + 1;
            if (out_tokens[t] == eos_token_id) break;
        }
        return produced;
    }
    if (eos_token_id < 0) {
        for (int s = 0; s < steps; ++s) SPB_CUDA(cudaGraphLaunch(e->graph, e->stream));
        e->seq_len += steps;
        produced = max_tokens;
        if (produced > 0)
            SPB_CUDA(cudaMemcpyAsync(out_tokens, e->d_out + start + n_prompt - 1, sizeof(int) * produced,
                                     cudaMemcpyDeviceToHost, e->stream));
        SPB_CUDA(cudaStreamSynchronize(e->stream));
    } else {
        for (int s = 0; s < n_prompt - 1; ++s) SPB_CUDA(cudaGraphLaunch(e->graph, e->stream));
        e->seq_len += n_prompt - 1;
        for (int t = 0; t < max_tokens; ++t) {
            SPB_CUDA(cudaGraphLaunch(e->graph, e->stream));
            SPB_CUDA(cudaMemcpyAsync(out_tokens + t, e->d_out + e->seq_len, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
            SPB_CUDA(cudaStreamSynchronize(e->stream));
            e->seq_len++;
            produced = t + 1;
            if (out_tokens[t] == eos_token_id) break;
        }
    }
    return produced;
}
