// Shared plumbing for the sm_100a kernels: status codes, the per-thread error
// string, launch helpers (programmatic dependent launch) and small PTX wrappers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/spbitnet_b200.h"

namespace spb {

// Records a formatted message for spb_last_error_string() and returns `code`.
int fail(int code, const char* fmt, ...);

// Whether kernels are launched with the programmatic-stream-serialization
// attribute (spb_set_pdl).
bool pdl_enabled();

// Number of SMs of the current device (cached per device).
int sm_count();

// Raises a kernel's dynamic shared-memory limit to at least `bytes` on the current device.  The attribute is
// per (kernel, device) and only ever grows here, so the largest value set so far is remembered and the runtime
// is called only when a launch needs more.  Returns SPB_OK or SPB_E_CUDA (message recorded under `name`).
int ensure_dynamic_smem_impl(const char* name, const void* kernel, size_t bytes);
template <typename... KArgs>
int ensure_dynamic_smem(const char* name, void (*kernel)(KArgs...), size_t bytes) {
    // no shortcut for small sizes: the default limit of 48 KB covers static + dynamic shared memory together
    return ensure_dynamic_smem_impl(name, reinterpret_cast<const void*>(kernel), bytes);
}

// Counter of bounded device-side waits that ran out (tensor-core kernels).  It lives in pinned host memory
// that every GPU of the process can reach (allocated portable and mapped on first use), so a kernel bumps it
// with a system-scope atomic through the pointer it is given, and the host reads it after a synchronisation
// without another CUDA call.  nullptr when the allocation failed (kernels then skip the count).
int* timeout_counter();
// Current value of the counter (0 when it could not be allocated).
int timeouts_now();
// Performs every lazy host-side look-up and allocation of the launchers (gemm_tcsp_ws.cu); engines call it at
// creation, outside any stream capture.
void prepare_host_state();

// Launches `kernel` on `stream`.  With PDL enabled the launch carries
// cudaLaunchAttributeProgrammaticStreamSerialization, so the grid may start
// while its predecessor on the stream is still draining; every kernel in this
// library therefore executes grid_dep_wait() before it touches anything a
// predecessor may have written, and before its own first store.
template <typename... KArgs, typename... Args>
int launch(const char* name, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
           void* stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(SPB_E_CUDA, "%s: launch failed: %s", name, cudaGetErrorString(err));
    }
    return SPB_OK;
}

// griddepcontrol.launch_dependents: lets the next grid on the stream begin its independent prologue
// (weight prefetch).  Harmless without PDL.  Most kernels call it first thing; the tensor-core GEMV
// calls it after its own dependency wait, which keeps at most one waiting grid per stream resident
// (measured: better for fat blocks, slightly worse for the thin-block SIMT kernels).
__device__ __forceinline__ void grid_dep_launch() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// griddepcontrol.wait: returns once every predecessor grid has completed and its
// writes are visible.  A no-op for a grid launched without the PDL attribute.
__device__ __forceinline__ void grid_dep_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// 128-bit / 64-bit streaming loads of weight words: read once, keep out of L1.
__device__ __forceinline__ uint4 ld_stream_v4(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_v2(const uint32_t* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ int clamp_i8(int q) { return max(-128, min(127, q)); }

// The activation quantiser of the reference (src/kernels/inference_kernels.cu:105-112,
// src/kernels/sparse_ternary.cu:198-217): fp32 multiply, round to nearest even, clamp.
__device__ __forceinline__ int quantize_one(float x, float scale) {
    return clamp_i8(__float2int_rn(__fmul_rn(x, scale)));
}
__device__ __forceinline__ float quant_scale(float absmax) {
    return (absmax > 0.0f) ? __fdiv_rn(127.0f, absmax) : 0.0f;
}
// dequantize_kernel's scale, evaluated left to right (inference_kernels.cu:169).
__device__ __forceinline__ float dequant_scale(float gamma, float absmax) {
    return __fdiv_rn(__fmul_rn(gamma, absmax), 127.0f);
}

// Optional BitLinear epilogue of the batched product: with `out` set, output row j is written as
// half(float(acc) * dequant_scale(gamma, absmax[j])) (dequantize_gpu per activation row) instead of the int32 sums.
struct GemmEpilogue {
    __half* out;          // [n, rows] half, or nullptr
    const float* absmax;  // n row scales
    float gamma;
};


// ---------------------------------------------------------------------------
// (bitmap | signs << 4) -> the four int8 weights of a group, packed little-endian
// for dp4a.  Bitmaps with other than two bits set reproduce the reference GPU table,
// which maps them to positions (0,0) (src/kernels/sparse_ternary.cu:34-51): both
// signed units land on column 0 of the group.
// ---------------------------------------------------------------------------
struct GroupLut {
    uint32_t w[64];
};

constexpr GroupLut make_group_lut() {
    GroupLut t{};
    for (int idx = 0; idx < 64; ++idx) {
        const int n = idx & 15, s = idx >> 4;
        const int s0 = (s & 1) ? -1 : 1, s1 = (s & 2) ? -1 : 1;
        int b[4] = {0, 0, 0, 0};
        int bits = 0, p0 = 0, p1 = 0;
        for (int i = 0; i < 4; ++i)
            if (n & (1 << i)) {
                if (bits == 0) p0 = i;
                if (bits == 1) p1 = i;
                ++bits;
            }
        if (bits != 2) { p0 = 0; p1 = 0; }
        b[p0] += s0;
        b[p1] += s1;
        uint32_t word = 0;
        for (int i = 0; i < 4; ++i) word |= (static_cast<uint32_t>(b[i]) & 0xFFu) << (8 * i);
        t.w[idx] = word;
    }
    return t;
}

// One copy per translation unit (no relocatable device code needed).
static __constant__ GroupLut c_group_lut = make_group_lut();

constexpr int kLutBytes = 64 * 32 * 4;  // the table replicated once per lane

// Fills the per-lane replicated table: entry e of lane l lives at lut[e * 32 + l].
__device__ __forceinline__ void fill_lane_lut(uint32_t* lut, int tid, int nthreads) {
    for (int e = tid; e < 64 * 32; e += nthreads) lut[e] = c_group_lut.w[e >> 5];
}

}  // namespace spb
