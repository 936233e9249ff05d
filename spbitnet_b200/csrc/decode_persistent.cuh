// Host interface of the persistent decode-step kernel (decode_persistent.cu); engine-internal.
#pragma once
#include "spb_common.cuh"

namespace spb {

// One BitLinear of a layer as the kernel reads it (rows and cols follow from the model shape).
struct PdLinear {
    const uint32_t* meta;
    const uint32_t* values;
    float gamma;
    int ms, vs;  // row strides in uint32 words
};

struct PdLayer {
    PdLinear lin[7];       // q k v o gate up down
    const float* norm[4];  // input_ln, post_attn_ln, attn_sub_norm, ffn_sub_norm (sub-norms may be null)
    __half* kc;            // this layer's K cache [kv head][max_seq][head_dim]
    __half* vc;
};

// Model shape and the engine's buffers.  All pointers are device memory.
struct PdModel {
    const PdLayer* layers;  // device array of nlayers entries
    int nlayers;
    int H, inter, nh, nkv, hd, max_seq;
    float eps, theta, attn_scale;
    const __half* embed;
    const int* d_prompt;  // may be null
    int n_prompt;
    const int* d_next;
    const int* d_pos;
    __half *xa, *xb;  // residual stream: the kernel leaves the stream after the last layer's attention half in xa
    __half *q, *attn, *o, *gate, *up, *down;
    float* scratch;     // split-attention partials, attn_scratch_floats() floats
    unsigned* sync;     // kPdSyncWords + nkv words, zeroed once (barrier words and the per-KV-head chunk counts)
    uint2* ll;          // decode_persistent_ll_words() tagged words, zeroed once: the stage outputs of the barrier-free form
    int barrier_free;   // 1: stages hand their outputs over as tagged words that the consumers poll; 0: grid barriers
};

constexpr int kPdSyncWords = 64;  // words of PdModel::sync ahead of the per-KV-head counts

// 64-bit words of PdModel::ll: q, new K row, new V row, attention output, o, (gate, up), down of one layer.
size_t decode_persistent_ll_words(int H, int inter, int nh, int nkv, int hd);

// Whether the kernel takes this shape on the current device (layout rules, shared memory, cooperative launch).
// `why` receives a short reason when it does not.
bool decode_persistent_supported(const PdModel& m, const PdLinear* first_layer_lin, const char** why);

// Enqueues the layers of one token (embedding gather to the last down projection) as one cooperative launch.
// wait_cycles bounds every grid-barrier wait (0 = the default of about a second).
int decode_persistent_launch(const PdModel& m, long long wait_cycles, void* stream);

}  // namespace spb
