// Library-wide state: the per-thread error string, the PDL switch, device facts.
#include "spb_common.cuh"

#include <atomic>
#include <cstring>

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

}  // namespace spb

extern "C" const char* spb_last_error_string(void) { return spb::t_error; }

extern "C" const char* spb_version(void) { return "spbitnet_b200 0.1 sm_100a"; }

extern "C" int spb_set_pdl(int enabled) { return spb::g_pdl.exchange(enabled ? 1 : 0); }
