// Shared helpers for the vtpack_b200 kernels: element types, 16-byte vector access,
// warp reductions, argument checks and the per-thread error string.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/vtpack_b200.h"

namespace vtp {

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------- host side errors
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);

#define VTP_REQUIRE(cond, code, ...)            \
    do {                                        \
        if (!(cond)) return ::vtp::fail((code), __VA_ARGS__); \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t elem_size(int dtype) { return dtype == VTP_BF16 ? 2 : 4; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline long long round_up(long long a, long long b) { return (a + b - 1) / b * b; }

// Number of SMs of the current device (cached per device).
int sm_count();

// True when the environment variable VTP_PDL is set.  Off by default: the tensor-core kernels
// fill an SM's shared memory, so a dependent kernel cannot become resident early and the
// overlap measured on B200 was nil.
bool pdl_enabled();

// Launch `kernel` so that it may overlap the tail of the previous kernel on the stream
// (the kernel must call griddep_wait() before it touches that kernel's results).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the grid cut into clusters of `cluster_x` CTAs (1: no cluster attribute).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), int cluster_x, dim3 grid, dim3 block, size_t smem,
                               cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------- device status word
// Bounded waits OR one of these codes into the device status word (see runtime.h)
// instead of hanging; vtp_device_status reads it back.
enum : int {
    STATUS_GEMM_PRODUCER = 1, STATUS_GEMM_MMA = 2, STATUS_GEMM_EPILOGUE = 4,
    STATUS_ATTN_LOAD = 8, STATUS_ATTN_MMA = 16, STATUS_ATTN_SOFTMAX = 32,
    STATUS_BAD_INDEX = 64,      // a caller-supplied patch row or row offset pointed outside the declared arrays
    STATUS_WAIT_MASK = 63,      // the bounded-wait codes: while one is set, tensor-core launches return at once
};

// Index guards: kernels that follow caller-supplied indices (patch lists, packed-row offsets) check them
// against the declared shapes, skip what does not fit and OR STATUS_BAD_INDEX into the status word.
// Four integer compares per patch row; compile with -DVTP_INDEX_GUARDS=0 to leave them out.
#ifndef VTP_INDEX_GUARDS
#define VTP_INDEX_GUARDS 1
#endif

// ---------------------------------------------------------------- element vectors
// A Vec<T> is 16 bytes of T: 4 floats or 8 bf16.
template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    float4 raw;
    __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = raw; }
    __device__ __forceinline__ void to_float(float* f) const { f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w; }
    __device__ __forceinline__ void from_float(const float* f) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec<bf16> {
    static constexpr int N = 8;
    uint4 raw;
    __device__ __forceinline__ void load(const bf16* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void store(bf16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
    __device__ __forceinline__ void to_float(float* f) const {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
    __device__ __forceinline__ void from_float(const float* f) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    }
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Programmatic dependent launch: a kernel launched with launch_pdl may start while the kernel
// in front of it on the stream is still running.  griddep_wait() blocks until that kernel
// has completed and its writes are visible: everything before it (barrier setup, TMEM
// allocation, descriptor prefetch) overlaps the predecessor's tail.  griddep_launch() lets
// the kernel behind this one begin its own prologue.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float gelu_erf(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}

}  // namespace vtp
