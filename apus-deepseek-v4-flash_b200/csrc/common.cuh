// Shared device/host helpers for libapus_b200: numeric format conversions that
// reproduce the reference bit for bit, error plumbing, and the launch counter.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

namespace apus {

// ---- error plumbing ---------------------------------------------------------
void set_error(const char *fmt, ...);          // api.cu
extern unsigned long long g_dispatches;        // api.cu: kernels launched
// Order of the long f32 sums (public: apus_cuda_set_sum_order).
#ifndef APUS_CUDA_SUM_REFERENCE
#define APUS_CUDA_SUM_REFERENCE 0
#define APUS_CUDA_SUM_TREE 1
#endif
int sum_order();                               // api.cu

#define APUS_CUDA_OK(expr)                                                     \
    do {                                                                       \
        cudaError_t e__ = (expr);                                              \
        if (e__ != cudaSuccess) {                                              \
            apus::set_error("%s:%d %s -> %s", __FILE__, __LINE__, #expr,       \
                            cudaGetErrorString(e__));                          \
            return 1;                                                          \
        }                                                                      \
    } while (0)

#define APUS_LAUNCHED()                                                        \
    do {                                                                       \
        apus::g_dispatches++;                                                  \
        cudaError_t e__ = cudaGetLastError();                                  \
        if (e__ != cudaSuccess) {                                              \
            apus::set_error("%s:%d launch -> %s", __FILE__, __LINE__,          \
                            cudaGetErrorString(e__));                          \
            return 1;                                                          \
        }                                                                      \
    } while (0)

#define APUS_REQUIRE(cond, ...)                                                \
    do {                                                                       \
        if (!(cond)) { apus::set_error(__VA_ARGS__); return 1; }               \
    } while (0)

// ---- scalar format helpers (device + host) -------------------------------------

// Round-to-nearest-even to BF16, kept in an f32 (reference c/fp4.h:262-270).
__host__ // e^x and log(1+x) evaluated in double and rounded once to f32.  The reference
// calls the host libm's expf/log1pf; a correctly rounded result agrees with any
// good libm (glibc's expf stays under 0.502 ulp) on all but a vanishing share
// of inputs, while the device's f32 expf may be 2 ulp off and would flip a
// BF16 step downstream far more often.
__device__ __forceinline__ float exp_rn(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float log1p_rn(float x) { return (float)log1p((double)x); }

__device__ __forceinline__ float bf16_round(float x) {
#ifdef __CUDA_ARCH__
    uint32_t u = __float_as_uint(x);
#else
    uint32_t u; memcpy(&u, &x, 4);
#endif
    if ((u & 0x7fffffffu) > 0x7f800000u) return x;
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}

__device__ __forceinline__ uint16_t bf16_bits(float x) {
    return (uint16_t)(__float_as_uint(bf16_round(x)) >> 16);
}
__device__ __forceinline__ float bf16_to_f32(uint16_t b) {
    return __uint_as_float((uint32_t)b << 16);
}

// UE8M0 byte -> f32 power of two (reference c/fp4.h:209-217): byte 0 is the
// subnormal 2^-127, byte 255 is +inf.  max() maps 0 onto 0x00400000 because
// every other b<<23 is >= 0x00800000.
__device__ __forceinline__ float ue8m0_f32(uint32_t b) {
    return __uint_as_float(max(b << 23, 0x00400000u));
}

// E4M3 code -> f32, exact (reference c/fp4.h:255-260); 0x7f/0xff decode to
// +-480 like the reference, not NaN.
__device__ __forceinline__ float e4m3_to_f32(uint32_t c) {
    uint32_t e = (c >> 3) & 15u, m = c & 7u;
    float mag = e ? __uint_as_float(((e + 120u) << 23) | (m << 20))
                  : (float)m * 0.001953125f;
    return (c & 0x80u) ? -mag : mag;
}

// Two f32 -> two E4M3 codes (lo = a, hi = b), RNE with saturation to +-448:
// the hardware conversion implements exactly the rule of reference
// c/fp4.h:229-253 for finite inputs (checked bitwise in the tests).
__device__ __forceinline__ uint16_t e4m3x2_from_f32(float a, float b) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(a), "f"(b));
    return r;
}

// 2^ceil(log2(p)) for positive normal p (reference c/fp4.h:306-317).
__device__ __forceinline__ float ceil_pow2(float p) {
    uint32_t b = __float_as_uint(p);
    uint32_t e = ((b >> 23) & 0xffu) + ((b & 0x7fffffu) ? 1u : 0u);
    return __uint_as_float(e << 23);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

}  // namespace apus
