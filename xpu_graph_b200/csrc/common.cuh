// Shared helpers for the xg_sm100 kernel library: error reporting, dtype traits, 16-byte vectors.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/xg_sm100.h"

namespace xg {

// Thread-local message buffer behind xg_last_error().
char* last_error_buf();
int fail(int code, const char* fmt, ...);

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(XG_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    return XG_OK;
}

inline int num_sms() {
    static thread_local int cached_dev = -1;
    static thread_local int cached = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) cached = n;
        cached_dev = dev;
    }
    return cached;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int dtype_size(int dtype) { return dtype == XG_F32 ? 4 : ((dtype == XG_BF16 || dtype == XG_F16) ? 2 : 0); }

template <typename T>
struct Cvt;
template <>
struct Cvt<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <>
struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Cvt<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};

// GELU (erf form) for epilogues whose result is rounded to a 16-bit type: erfc from Abramowitz & Stegun 7.1.26
// (absolute error <= 1.5e-7, against a 16-bit rounding step of 2^-9 or 2^-11 relative), one reciprocal, one exp2 and
// five FMAs instead of erff's branches; for v < 0 the factor 1 + erf is the formula's erfc term itself, so the tail
// does not cancel. fp32 outputs keep erff.
__device__ __forceinline__ float gelu_erf_16bit(float v) {
    const float x = fabsf(v) * 0.70710678118654752f;
    const float t = __fdividef(1.0f, fmaf(0.3275911f, x, 1.0f));
    float poly = fmaf(1.061405429f, t, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    const float e = poly * t * __expf(-x * x);  // erfc(|v| / sqrt(2))
    return 0.5f * v * (v >= 0.f ? 2.0f - e : e);
}

// 16-byte vector of T (4 floats or 8 half-precision values).
template <typename T>
struct alignas(16) Vec16 {
    static constexpr int N = 16 / sizeof(T);
    T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> ld16(const T* p) {
    Vec16<T> r;
    *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
    return r;
}
// Streaming 16-byte load that does not allocate in L1 (data read exactly once).
template <typename T>
__device__ __forceinline__ Vec16<T> ld16_stream(const T* p) {
    Vec16<T> r;
    uint4 u;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                 : "l"(p));
    *reinterpret_cast<uint4*>(&r) = u;
    return r;
}
template <typename T>
__device__ __forceinline__ void st16(T* p, const Vec16<T>& r) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

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

}  // namespace xg
