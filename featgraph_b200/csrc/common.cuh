// Shared host/device helpers for the featgraph_b200 kernels.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "featgraph_b200.h"

namespace fg {

// Thread-local error text behind fg_last_error().
char* error_buffer();
int fail(int code, const char* fmt, ...);

#define FG_CUDA_TRY(expr)                                                                  \
    do {                                                                                   \
        cudaError_t fg_err__ = (expr);                                                     \
        if (fg_err__ != cudaSuccess)                                                       \
            return ::fg::fail(FG_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                 \
                              cudaGetErrorString(fg_err__), __FILE__, __LINE__);           \
    } while (0)

// Kernels launched by this library in this process (fg_kernel_launch_count).
void count_launches(int n);

// Compile-time shapes of the hot kernels of each source file, for fg_kernel_signature().
const char* spmm_signature();
const char* sddmm_signature();
const char* sddmm_plan_signature();

// SM count and L2 size of the current device, looked up once per device ordinal (a host thread may
// move between devices; each device keeps its own figures).
constexpr int kMaxDevices = 64;
struct DeviceProps {
    int sm_count = 148;
    int64_t l2_bytes = 64ll << 20;
};
DeviceProps device_props();
// Ordinal of the current device, or -1 if it cannot be had or is beyond kMaxDevices.
int current_device_slot();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int pow2_floor(int v) {
    int p = 1;
    while (p * 2 <= v) p *= 2;
    return p;
}
inline int pow2_ceil(int v) {
    int p = 1;
    while (p < v) p *= 2;
    return p;
}

// 128-bit read-only gather of one feature-row slice.
__device__ __forceinline__ float4 ldg4(const float* p) {
    return __ldg(reinterpret_cast<const float4*>(p));
}

// L2 residency hints, as build-time switches (both OFF by default).  The kernels gather from a slice of
// the feature matrix that is sized to stay in L2 while index arrays and outputs stream past it once per
// pass; the hints ask L2 to evict gathered lines last (FG_HINT_KEEP) and streamed lines first
// (FG_HINT_STREAM).  Measured on B200 with the 233K-node graph they changed nothing that matters: SpMM was
// 1-7 % slower with FG_HINT_KEEP (the policy operand costs an instruction slot per gather), SDDMM within
// +-3 % either way - the slice's hit rate is set by its size against L2, not by the streams.
#ifndef FG_HINT_KEEP
#define FG_HINT_KEEP 0
#endif
#ifndef FG_HINT_STREAM
#define FG_HINT_STREAM 0
#endif
__device__ __forceinline__ uint64_t l2_keep_policy() {
    uint64_t p = 0;
#if FG_HINT_KEEP
    asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
#endif
    return p;
}
// gather with the evict-last policy
__device__ __forceinline__ float4 ldg4_keep(const float* p, uint64_t policy) {
#if FG_HINT_KEEP
    float4 v;
    asm("ld.global.nc.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
        : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
        : "l"(p), "l"(policy));
    return v;
#else
    return ldg4(p);
#endif
}
// streamed (read-once / write-once) data: evict first
template <typename T>
__device__ __forceinline__ T ld_stream(const T* p) {
#if FG_HINT_STREAM
    return __ldcs(p);
#else
    return *p;
#endif
}
template <typename T>
__device__ __forceinline__ void st_stream(T* p, T v) {
#if FG_HINT_STREAM
    __stcs(p, v);
#else
    *p = v;
#endif
}

// acc + a*b with two roundings (never contracted into an FMA).
__device__ __forceinline__ float mul_then_add(float acc, float a, float b) {
    return __fadd_rn(acc, __fmul_rn(a, b));
}

}  // namespace fg
