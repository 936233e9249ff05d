// Library-wide state: the per-thread error string, the PDL switch, device facts.
#include "spb_common.cuh"

#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

namespace spb {

static thread_local char t_error[512] = "";
static std::atomic<int> g_pdl{1};

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof t_error, fmt, ap);
    va_end(ap);
    return code;
}

bool pdl_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int ensure_dynamic_smem_impl(const char* name, const void* kernel, size_t bytes) {
    struct Entry { const void* kernel; int device; size_t bytes; };
    static std::mutex mu;
    static std::vector<Entry> seen;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
    std::lock_guard<std::mutex> lock(mu);
    Entry* hit = nullptr;
    for (Entry& e : seen)
        if (e.kernel == kernel && e.device == dev) hit = &e;
    if (hit && hit->bytes >= bytes) return SPB_OK;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "%s: cudaFuncSetAttribute(%zu B of shared memory): %s", name, bytes, cudaGetErrorString(err));
    }
    if (hit) hit->bytes = bytes;
    else seen.push_back(Entry{kernel, dev, bytes});
    return SPB_OK;
}

int* timeout_counter() {
    static int* counter = [] {
        int* p = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void**>(&p), sizeof(int), cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
            cudaGetLastError();
            return static_cast<int*>(nullptr);
        }
        *p = 0;
        return p;
    }();
    return counter;
}

int timeouts_now() {
    int* p = timeout_counter();
    return p ? *static_cast<volatile int*>(p) : 0;
}

}  // namespace spb

extern "C" int spb_gemm_tc_timeouts(void) {
    if (!spb::timeout_counter()) return -1;
    if (cudaDeviceSynchronize() != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return spb::timeouts_now();
}

extern "C" const char* spb_last_error_string(void) { return spb::t_error; }

extern "C" const char* spb_version(void) { return "spbitnet_b200 0.1 sm_100a"; }

extern "C" int spb_set_pdl(int enabled) { return spb::g_pdl.exchange(enabled ? 1 : 0); }
