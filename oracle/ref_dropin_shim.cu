// ref_dropin_shim.cu -- the reference's OWN host engine (spbitnet::Model::load, src/model.cu, and
// spbitnet::InferenceEngine, src/inference.cu, both compiled unchanged where they lie) built against the drop-in
// headers of this repository (include/spbitnet/sparse_ternary_kernels.h, inference_kernels.h) and linked with
// libspbitnet_b200.so instead of the reference's kernel library.  TEST INFRASTRUCTURE ONLY: it proves that the
// reference engine runs unmodified on the sm_100a kernels, and gives the tests a third implementation of the
// forward pass (reference host code over this repository's kernels).
#include <cstdio>
#include <exception>
#include <memory>
#include <string>

#include "spbitnet/inference.h"
#include "spbitnet/model.h"

namespace {
struct DropIn {
    spbitnet::Model model;
    std::unique_ptr<spbitnet::InferenceEngine> engine;
    explicit DropIn(spbitnet::Model&& m) : model(std::move(m)) {}
};
char g_error[512] = "";
}  // namespace

extern "C" {

const char* dropin_last_error(void) { return g_error; }

// Loads a model directory (config.json, manifest.json, weights/) the way the reference CLI does.
void* dropin_create(const char* model_dir) {
    try {
        auto* d = new DropIn(spbitnet::Model::load(model_dir));
        d->engine = std::make_unique<spbitnet::InferenceEngine>(d->model);
        return d;
    } catch (const std::exception& e) {
        snprintf(g_error, sizeof g_error, "%s", e.what());
        return nullptr;
    }
}

void dropin_destroy(void* h) { delete static_cast<DropIn*>(h); }

int dropin_vocab(void* h) { return static_cast<DropIn*>(h)->model.config().vocab_size; }

// InferenceEngine::forward; the logits are copied to host memory as src/main.cpp:280-282 does.
int dropin_forward(void* h, int token, float* h_logits) {
    DropIn* d = static_cast<DropIn*>(h);
    const float* d_logits = d->engine->forward(token);
    const cudaError_t err = cudaMemcpy(h_logits, d_logits, sizeof(float) * d->model.config().vocab_size,
                                       cudaMemcpyDeviceToHost);
    if (err != cudaSuccess) {
        snprintf(g_error, sizeof g_error, "cudaMemcpy: %s", cudaGetErrorString(err));
        return -1;
    }
    return 0;
}

void dropin_reset(void* h) { static_cast<DropIn*>(h)->engine->reset(); }

int dropin_seq_len(void* h) { return static_cast<DropIn*>(h)->engine->seq_len(); }

}  // extern "C"
