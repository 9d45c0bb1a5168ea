// Shared device/host helpers for the rfk kernels (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cfloat>
#include <cstdint>
#include <utility>
#include "rfk.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "rfk kernels are written for sm_100a (Blackwell) only"
#endif

namespace rfk {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

// ---------------------------------------------------------------- host side

extern std::atomic<unsigned long long> g_launches;  // defined in abi.cu; launches may come from any host thread

// Status of the most recent launch on this thread, mapped to the C-ABI convention.
inline int launch_status() {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return RFK_OK;
}

inline cudaStream_t as_stream(rfk_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Programmatic dependent launch. A kernel launched through launch_pdl may be scheduled as soon as every CTA of the
// kernel before it in the stream has called pdl_trigger() (or exited), so its launch latency and its on-chip
// set-up overlap that kernel's tail; it must call pdl_wait() before it touches global memory, which blocks until the
// preceding kernel has completed and its writes are visible. Every kernel launched this way calls pdl_wait() in all
// of its CTAs, so completion of a kernel implies completion of everything before it. Inside a stream capture the
// launches become programmatic edges of the graph. RFK_PDL=0 in the environment turns the attribute off (the
// device-side calls are then no-ops).
extern bool g_pdl_enabled;  // defined in abi.cu
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = g_pdl_enabled ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }

inline unsigned ceil_div(long long a, long long b) { return (unsigned)((a + b - 1) / b); }

// ------------------------------------------------------------- device side

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 8 fp16 values moved as one 128-bit transaction.
struct __align__(16) Half8 {
    __half2 v[4];
};

__device__ __forceinline__ Half8 ld_half8(const __half* p) {
    Half8 r;
    *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
    return r;
}
// Read-only (non-coherent) path for data that is never written by the same kernel.
__device__ __forceinline__ Half8 ldg_half8(const __half* p) {
    Half8 r;
    *reinterpret_cast<uint4*>(&r) = __ldg(reinterpret_cast<const uint4*>(p));
    return r;
}
__device__ __forceinline__ void st_half8(__half* p, const Half8& v) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&v);
}
// Streaming variants: the data is touched once, keep it from displacing reusable lines.
__device__ __forceinline__ Half8 ldcs_half8(const __half* p) {
    Half8 r;
    *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
    return r;
}
__device__ __forceinline__ void stcs_half8(__half* p, const Half8& v) {
    __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&v));
}

__device__ __forceinline__ void unpack8(const Half8& h, float (&f)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h.v[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ Half8 pack8(const float (&f)[8]) {
    Half8 h;
#pragma unroll
    for (int i = 0; i < 4; ++i) h.v[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return h;
}

__device__ __forceinline__ void ld_float8(const float* p, float (&f)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void ldg_float8(const float* p, float (&f)[8]) {
    float4 a = __ldg(reinterpret_cast<const float4*>(p));
    float4 b = __ldg(reinterpret_cast<const float4*>(p + 4));
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void ldcs_float8(const float* p, float (&f)[8]) {
    float4 a = __ldcs(reinterpret_cast<const float4*>(p));
    float4 b = __ldcs(reinterpret_cast<const float4*>(p + 4));
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void st_float8(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

// Typed 8-element accessors so one kernel template serves fp16 and fp32 storage.
__device__ __forceinline__ void load8(const __half* p, float (&f)[8]) { unpack8(ld_half8(p), f); }
__device__ __forceinline__ void load8(const float* p, float (&f)[8]) { ld_float8(p, f); }
__device__ __forceinline__ void store8(__half* p, const float (&f)[8]) { st_half8(p, pack8(f)); }
__device__ __forceinline__ void store8(float* p, const float (&f)[8]) { st_float8(p, f); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// 2^x on the special-function unit (one MUFU.EX2); -inf -> 0, denormal results flush to 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Round through fp16 exactly as a store followed by a load of a `half` would.
__device__ __forceinline__ float round_half(float v) { return __half2float(__float2half_rn(v)); }

}  // namespace rfk

#define RFK_REQUIRE(cond) \
    do {                  \
        if (!(cond)) return RFK_EINVAL; \
    } while (0)
