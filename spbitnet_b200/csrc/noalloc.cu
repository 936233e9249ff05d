// Split-KV decode attention for callers that cannot hand over a scratch buffer.
//
// The reference's convention is that the caller owns every device buffer and the kernels
// allocate nothing.  Its engine fixes its buffer plan in the constructor (src/inference.cu:16-69)
// and has no slot for the per-chunk partial results the split-KV kernel needs; a drop-in user
// of that engine, code running inside a stream capture, or a serving loop that must not stall
// the device cannot call cudaMalloc between decode steps to make room for one.  For them the
// partial results go to one array that is part of the library image: every GPU that loads the
// library carries kNoAllocScratchBytes of it until the process exits.
#include <mutex>

#include "fused_ops.cuh"

namespace {

constexpr size_t kNoAllocScratchFloats = 512 * 1024;
constexpr size_t kNoAllocScratchBytes = kNoAllocScratchFloats * sizeof(float);  // 2 MiB

static __device__ __align__(256) float g_attention_scratch[kNoAllocScratchFloats];

// In host code `g_attention_scratch` names a host-side handle, not device memory: the device
// address has to be asked for, once per device, with that device current.
constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};
std::mutex g_scratch_mutex;

int scratch_address_for_current_device(float** out) {
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return spb::fail(SPB_E_CUDA, "spb_decode_attention_noalloc: cudaGetDevice: %s", cudaGetErrorString(err));
    }
    if (dev < 0 || dev >= kMaxDevices)
        return spb::fail(SPB_E_UNSUPPORTED, "spb_decode_attention_noalloc: device %d beyond the %d slots of the address table",
                         dev, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_address[dev]) {
        float* p = nullptr;
        err = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attention_scratch);
        if (err != cudaSuccess || !p) {
            cudaGetLastError();
            return spb::fail(SPB_E_CUDA, "spb_decode_attention_noalloc: cudaGetSymbolAddress: %s",
                             cudaGetErrorString(err));
        }
        g_scratch_address[dev] = p;
    }
    *out = g_scratch_address[dev];
    return SPB_OK;
}

}  // namespace

extern "C" size_t spb_decode_attention_noalloc_capacity(void) { return kNoAllocScratchBytes; }

extern "C" int spb_decode_attention_noalloc(const void* Q, const void* K_cache, const void* V_cache, void* output,
                                            int num_heads, int num_kv_heads, int head_dim, int max_seq_len,
                                            int seq_len, float scale, void* stream) {
    const char* name = "spb_decode_attention_noalloc";
    if (num_heads < 0 || num_kv_heads <= 0 || head_dim <= 0 || max_seq_len <= 0)
        return spb::fail(SPB_E_INVALID, "%s: bad shape", name);
    if (seq_len < 1 || seq_len > max_seq_len) return spb::fail(SPB_E_INVALID, "%s: seq_len outside the cache", name);
    if (num_heads == 0) return SPB_OK;
    if (!Q || !K_cache || !V_cache || !output) return spb::fail(SPB_E_INVALID, "%s: null pointer", name);
    const size_t need = spb::decode_attention_scratch_bytes(num_heads, head_dim, max_seq_len);
    if (need > kNoAllocScratchBytes)
        return spb::fail(SPB_E_UNSUPPORTED,
                         "%s: %d heads x head_dim %d x max_seq_len %d needs %zu bytes of partial results, the built-in "
                         "scratch holds %zu; use spb_decode_attention_split with your own buffer",
                         name, num_heads, head_dim, max_seq_len, need, kNoAllocScratchBytes);
    float* scratch = nullptr;
    if (int rc = scratch_address_for_current_device(&scratch)) return rc;
    // Every chunk slot that the merge kernel reads is written by this call's first kernel, so
    // nothing left over from an earlier call needs clearing.
    return spb::decode_attention_split(Q, K_cache, V_cache, output, num_heads, num_kv_heads, head_dim, max_seq_len,
                                       seq_len, nullptr, scale, scratch, stream);
}
