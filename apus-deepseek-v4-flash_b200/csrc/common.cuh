// Shared device/host helpers for libapus_b200: numeric format conversions that
// reproduce the reference bit for bit, error plumbing, and the launch counter.
#pragma once
#include <string.h>
#include <utility>
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
int sum_order();                               // api.cu: TREE only when every operator class is in tree order
unsigned long long sum_order_epoch();          // api.cu: changes whenever the order does, or a workspace buffer moved
int chunk_rows();                              // api.cu: rows (positions x sequences) one chunk of a s > 1 call may hold; 0 = one step per position
bool chunks_enabled();
// Operator classes whose long f32 sums may leave the reference's loop order (public:
// apus_cuda_set_tree_ops).  sum_tree(op) = this class currently sums in tree / tensor-core order.
#ifndef APUS_CUDA_TREE_MHC_MAPS
#define APUS_CUDA_TREE_MHC_MAPS 1
#define APUS_CUDA_TREE_NORMS 2
#define APUS_CUDA_TREE_HEAD 4
#define APUS_CUDA_TREE_WO_A 8
#define APUS_CUDA_TREE_ROUTER 16
#define APUS_CUDA_TREE_COMPRESSOR 32
#define APUS_CUDA_TREE_IDX_WPROJ 64
#define APUS_CUDA_TREE_LINEAR 128
#define APUS_CUDA_TREE_FP8_SPLITK 256
#define APUS_CUDA_TREE_ALL 511
#endif
int tree_ops();                                // api.cu
static inline bool sum_tree(int op) { return (tree_ops() & op) != 0; }
// dense-linear callers name their operator class in bits 8..15 of `flags` (0 = the generic class)
#define APUS_LIN_CLASS(op) ((op) << 8)
// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-DEVICE setting of a kernel: raises it to
// `bytes` for `func` on the current device unless a size at least as large was set there
// before (sizes up to 48 KB need no setting).  Thread-safe.  Nonzero + message on failure.
int ensure_dyn_smem(const void *func, size_t bytes);    // api.cu

#define APUS_CUDA_OK(expr)                                                     \
    do {                                                                       \
        cudaError_t e__ = (expr);                                              \
        if (e__ != cudaSuccess) {                                              \
            apus::set_error("%s:%d %s -> %s", __FILE__, __LINE__, #expr,       \
                            cudaGetErrorString(e__));                          \
            return 1;                                                          \
        }                                                                      \
    } while (0)

// ---- programmatic dependent launch ----------------------------------------------------------
// A step is a chain of short kernels; each launch_k'd kernel may be scheduled while the one before it
// on the stream is still running (its blocks are placed, parameters read, prologue run) and then
// waits in APUS_PDL_WAIT until that kernel has completed and its writes are visible.  Rule: a kernel
// launched through launch_k executes APUS_PDL_WAIT before it touches global memory at all (also
// before it overwrites anything: the kernel before it may still be reading it).  APUS_PDL_GO lets
// the kernel after this one be scheduled; both are no-ops when there is nothing to wait for.
// APUS_PDL=0 in the environment launches everything fully serialised (the two instructions are then no-ops).
#define APUS_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")
#define APUS_PDL_GO() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
bool pdl_enabled();                             // api.cu
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                   Args &&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    // Measurement aid (off unless APUS_DUP is set): every kernel whose name contains $APUS_DUP is launched
    // twice.  The growth of a replayed step is then that kernel's cost ON the step's critical path, launch gap
    // included, which a profiler's serialised per-kernel times do not show (a kernel on a side chain with
    // slack costs nothing; doubling it gives an upper bound).  Only for kernels that may run twice: not the
    // ones that advance the position or the sampler state.
    static const char *dup = getenv("APUS_DUP");
    if (dup && dup[0]) {
        const char *name = nullptr;
        if (cudaFuncGetName(&name, (const void *)kernel) == cudaSuccess && name && strstr(name, dup))
            cudaLaunchKernelEx(&cfg, kernel, args...);
    }
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

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

// acc + s[0] + s[1] + ... + s[n-1], one accumulator, index ascending, every add
// rounded: the order of the reference's scalar loops.  `s` is shared memory,
// 16-byte aligned.  The adds form one dependent chain (about four cycles each),
// so the loads are issued a batch of sixteen values ahead of the adds that
// consume them; left to itself the compiler keeps each load next to its add
// and the chain then pays the shared-memory latency per element.
__device__ __forceinline__ float seq_add4(float acc, const float4 &v) {
    acc = __fadd_rn(acc, v.x); acc = __fadd_rn(acc, v.y);
    acc = __fadd_rn(acc, v.z); acc = __fadd_rn(acc, v.w);
    return acc;
}
__device__ __forceinline__ float seq_sum_smem(const float *s, int n, float acc) {
    const float4 *p = reinterpret_cast<const float4 *>(s);
    const int n4 = n >> 2;
    int i = 0;
    float4 c0, c1, c2, c3;
    c0 = c1 = c2 = c3 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (n4 >= 4) { c0 = p[0]; c1 = p[1]; c2 = p[2]; c3 = p[3]; }
    for (; i + 4 <= n4; i += 4) {
        const float4 d0 = c0, d1 = c1, d2 = c2, d3 = c3;
        if (i + 8 <= n4) { c0 = p[i + 4]; c1 = p[i + 5]; c2 = p[i + 6]; c3 = p[i + 7]; }
        acc = seq_add4(acc, d0); acc = seq_add4(acc, d1);
        acc = seq_add4(acc, d2); acc = seq_add4(acc, d3);
    }
    for (; i < n4; i++) acc = seq_add4(acc, p[i]);
    for (int k = n4 * 4; k < n; k++) acc = __fadd_rn(acc, s[k]);
    return acc;
}

// e^x and log(1+x) evaluated in double and rounded once to f32.  The reference
// calls the host libm's expf/log1pf; a correctly rounded result agrees with any
// good libm (glibc's expf stays under 0.502 ulp) on all but a vanishing share
// of inputs, while the device's f32 expf may be 2 ulp off and would flip a
// BF16 step downstream far more often.
__device__ __forceinline__ float exp_rn(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float log1p_rn(float x) { return (float)log1p((double)x); }

// Round-to-nearest-even to BF16, kept in an f32 (reference c/fp4.h:262-270).
__host__ __device__ __forceinline__ float bf16_round(float x) {
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
