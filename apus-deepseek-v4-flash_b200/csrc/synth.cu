// Counter-based synthetic tensors (include/apus_synth.h): one element function,
// compiled for the device and for the host, so that a random-init model
// generated in HBM can be regenerated tensor by tensor on a CPU.  Only integer
// arithmetic and single, explicitly rounded f32 operations are used (no libm,
// no contraction into FMA), which makes the two builds agree bit for bit.
#include <thread>
#include <vector>

#include "apus_synth.h"
#include "common.cuh"

namespace {

#ifdef __CUDA_ARCH__
#define SY_MUL(a, b) __fmul_rn((a), (b))
#define SY_ADD(a, b) __fadd_rn((a), (b))
#else
// host: separate statements keep the compiler from contracting (x86-64 without -mfma has no FMA anyway)
static inline float sy_mul(float a, float b) { volatile float r = a * b; return r; }
static inline float sy_add(float a, float b) { volatile float r = a + b; return r; }
#define SY_MUL(a, b) sy_mul((a), (b))
#define SY_ADD(a, b) sy_add((a), (b))
#endif

__host__ __device__ __forceinline__ uint64_t sy_mix(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ __forceinline__ uint64_t sy_hash(uint64_t key, uint64_t i) {
    return sy_mix(key + (i + 1) * 0x9E3779B97F4A7C15ull);
}
__host__ __device__ __forceinline__ uint32_t sy_f2u(float f) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
__host__ __device__ __forceinline__ float sy_u2f(uint32_t u) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}
// a + b * z with z = (sum of four 16-bit uniforms - 131070) / 37837.23: mean 0, variance 1,
// support +-3.46
__host__ __device__ __forceinline__ float sy_normal(uint64_t h, float a, float b) {
    const int s = (int)(h & 0xffff) + (int)((h >> 16) & 0xffff) + (int)((h >> 32) & 0xffff) + (int)(h >> 48) - 131070;
    const float z = SY_MUL((float)s, 2.64289963e-5f);
    return SY_ADD(a, SY_MUL(b, z));
}
__host__ __device__ __forceinline__ uint32_t sy_bf16_bits(float x) {
    uint32_t u = sy_f2u(x);
    u = (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
    return u;
}
// RNE to E4M3 with saturation at +-448 (the rule of reference c/fp4.h:229-253) in integer arithmetic
__host__ __device__ __forceinline__ uint32_t sy_e4m3(float x) {
    const uint32_t u = sy_f2u(x), sign = (u >> 24) & 0x80u;
    uint32_t a = u & 0x7fffffffu;
    if (a >= 0x43e00000u) return sign | 0x7eu;                 // |x| >= 448 (inf/nan never occur here)
    uint32_t code;
    if (a < 0x3c800000u) {                                      // below 2^-6: multiples of 2^-9
        const float t = SY_MUL(sy_u2f(a), 512.0f);              // exact scaling, t < 8
        const float r = SY_ADD(SY_ADD(t, 12582912.0f), -12582912.0f);   // RNE to an integer
        code = (uint32_t)(int)r;                                // 8 is the smallest normal, code 0x08
    } else {
        uint32_t e = (a >> 23) - 127u + 7u, m = (a >> 20) & 7u;
        const uint32_t rem = a & 0xfffffu;
        if (rem > 0x80000u || (rem == 0x80000u && (m & 1u))) m++;
        if (m == 8u) { m = 0; e++; }
        code = (e << 3) | m;
        if (code > 0x7eu) code = 0x7eu;
    }
    return sign | code;
}
// element j of row r of the subset table: k distinct values in [0, n_vals), drawn in order with rejection
__host__ __device__ __forceinline__ long long sy_subset(uint64_t key, uint64_t r, int j, uint32_t n_vals) {
    uint32_t got[16];
    int n = 0;
    for (uint32_t c = 0; n <= j; c++) {
        uint32_t e = (uint32_t)(sy_hash(key, r * 64 + (c & 63u)) % n_vals);
        if (c >= 64u) e = (e + c) % n_vals;                     // never reached for k << n_vals; keeps the loop finite
        bool dup = false;
        for (int q = 0; q < n; q++) dup |= got[q] == e;
        if (!dup) got[n++] = e;
    }
    return (long long)got[j];
}

__host__ __device__ __forceinline__ uint64_t sy_key(uint64_t seed, uint32_t layer, uint32_t tensor, uint32_t expert) {
    uint64_t k = sy_mix(seed ^ 0xA5A5F00DDEADBEEFull);
    k = sy_mix(k + 0x9E3779B97F4A7C15ull * ((uint64_t)layer + 1));
    k = sy_mix(k + 0xC2B2AE3D27D4EB4Full * ((uint64_t)tensor + 1));
    k = sy_mix(k + 0x165667B19E3779F9ull * ((uint64_t)expert + 1));
    return k;
}

struct SyArgs { void *dst; int kind; uint64_t n, key; float a, b; };

// elements [lo, hi) of the tensor; lo is a multiple of 8 for the byte kinds
__host__ __device__ __forceinline__ void sy_fill_range(const SyArgs &p, uint64_t lo, uint64_t hi, uint64_t step) {
    switch (p.kind) {
    case APUS_SYNTH_U8: case APUS_SYNTH_U8_RANGE: {
        uint8_t *d = (uint8_t *)p.dst;
        const uint32_t base = (uint32_t)p.a, span = (uint32_t)p.b - (uint32_t)p.a + 1u;
        for (uint64_t w = lo; w < hi; w += step) {              // w counts 8-byte words
            uint64_t h = sy_hash(p.key, w);
            if (p.kind == APUS_SYNTH_U8_RANGE) {
                uint64_t o = 0;
                for (int k = 0; k < 8; k++) o |= (uint64_t)(base + ((((h >> (8 * k)) & 0xff) * span) >> 8)) << (8 * k);
                h = o;
            }
            const uint64_t i = w * 8;
            if (i + 8 <= p.n) *(uint64_t *)(d + i) = h;
            else for (uint64_t k = 0; i + k < p.n; k++) d[i + k] = (uint8_t)(h >> (8 * k));
        }
        break;
    }
    case APUS_SYNTH_F32: case APUS_SYNTH_F32_BF16:
        for (uint64_t i = lo; i < hi; i += step) {
            const float v = sy_normal(sy_hash(p.key, i), p.a, p.b);
            ((float *)p.dst)[i] = p.kind == APUS_SYNTH_F32 ? v : sy_u2f(sy_bf16_bits(v) << 16);
        }
        break;
    case APUS_SYNTH_BF16:
        for (uint64_t i = lo; i < hi; i += step)
            ((uint16_t *)p.dst)[i] = (uint16_t)sy_bf16_bits(sy_normal(sy_hash(p.key, i), p.a, p.b));
        break;
    case APUS_SYNTH_E4M3:
        for (uint64_t i = lo; i < hi; i += step)
            ((uint8_t *)p.dst)[i] = (uint8_t)sy_e4m3(sy_normal(sy_hash(p.key, i), p.a, p.b));
        break;
    case APUS_SYNTH_I64_MOD:
        for (uint64_t i = lo; i < hi; i += step)
            ((long long *)p.dst)[i] = (long long)(sy_hash(p.key, i) % (uint64_t)p.a);
        break;
    case APUS_SYNTH_I64_SUBSET: {
        const int k = (int)p.b;
        for (uint64_t i = lo; i < hi; i += step)
            ((long long *)p.dst)[i] = sy_subset(p.key, i / k, (int)(i % k), (uint32_t)p.a);
        break;
    }
    }
}

__global__ void synth_fill_kernel(SyArgs p, uint64_t units) {
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    sy_fill_range(p, t, units, (uint64_t)gridDim.x * blockDim.x);
}

// n_seg consecutive tensors of n elements each (an expert-major slab): blockIdx.y = segment, whose
// key is that of expert first_expert + segment -- the bytes of n_seg separate fills, in one launch
__global__ void synth_fill_slab_kernel(SyArgs p, uint64_t units, uint64_t seg_bytes, uint64_t seed, uint32_t layer,
                                       uint32_t tensor, uint32_t first_expert) {
    p.dst = (char *)p.dst + seg_bytes * blockIdx.y;
    p.key = sy_key(seed, layer, tensor, first_expert + blockIdx.y);
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    sy_fill_range(p, t, units, (uint64_t)gridDim.x * blockDim.x);
}

int sy_check(const void *dst, int kind, uint64_t n, double a, double b, uint64_t *units) {
    APUS_REQUIRE(dst || !n, "synth_fill: NULL destination");
    APUS_REQUIRE(kind >= APUS_SYNTH_U8 && kind <= APUS_SYNTH_I64_SUBSET, "synth_fill: unknown kind %d", kind);
    if (kind == APUS_SYNTH_U8) { a = 0; b = 255; }
    if (kind == APUS_SYNTH_U8_RANGE) APUS_REQUIRE(a >= 0 && b <= 255 && a <= b, "synth_fill: byte range [%g, %g]", a, b);
    if (kind == APUS_SYNTH_I64_MOD || kind == APUS_SYNTH_I64_SUBSET) APUS_REQUIRE(a >= 1 && a < 4294967296.0, "synth_fill: modulus %g", a);
    if (kind == APUS_SYNTH_I64_SUBSET)
        APUS_REQUIRE(b >= 1 && b <= 16 && b <= a && n % (uint64_t)b == 0, "synth_fill: subsets of %g out of %g, %llu elements", b, a,
                     (unsigned long long)n);
    *units = kind <= APUS_SYNTH_U8_RANGE ? (n + 7) / 8 : n;
    return 0;
}

}  // namespace

extern "C" {

uint64_t apus_synth_key(uint64_t seed, uint32_t layer, uint32_t tensor, uint32_t expert) {
    return sy_key(seed, layer, tensor, expert);
}

int apus_synth_fill_slab_dev(void *dst, int kind, uint64_t n, uint32_t n_seg, uint64_t seed, uint32_t layer,
                             uint32_t tensor, uint32_t first_expert, double a, double b, void *stream) {
    uint64_t units = 0;
    if (sy_check(dst, kind, n, a, b, &units)) return 1;
    APUS_REQUIRE(kind <= APUS_SYNTH_E4M3 && n_seg <= 65535, "synth_fill_slab: kind %d / %u segments", kind, n_seg);
    if (!units || !n_seg) return 0;
    if (kind == APUS_SYNTH_U8) { a = 0; b = 255; }
    static const uint64_t esz[] = {1, 1, 4, 4, 2, 1};
    APUS_REQUIRE((n * esz[kind]) % 8 == 0, "synth_fill_slab: segments must be a multiple of 8 bytes");
    SyArgs p = {dst, kind, n, 0, (float)a, (float)b};
    uint64_t blocks = (units + 255) / 256;
    if (blocks > 148 * 2) blocks = 148 * 2;
    synth_fill_slab_kernel<<<dim3((unsigned)blocks, n_seg), 256, 0, (cudaStream_t)stream>>>(p, units, n * esz[kind], seed,
                                                                                            layer, tensor, first_expert);
    APUS_LAUNCHED();
    return 0;
}

int apus_synth_fill_host(void *dst, int kind, uint64_t n, uint64_t key, double a, double b, int threads) {
    uint64_t units = 0;
    if (sy_check(dst, kind, n, a, b, &units)) return 1;
    if (kind == APUS_SYNTH_U8) { a = 0; b = 255; }
    SyArgs p = {dst, kind, n, key, (float)a, (float)b};
    unsigned nt = threads > 0 ? (unsigned)threads : std::thread::hardware_concurrency();
    if (nt < 1) nt = 1;
    if (nt > 32) nt = 32;
    if (units < (1u << 16)) nt = 1;
    if (nt == 1) { sy_fill_range(p, 0, units, 1); return 0; }
    std::vector<std::thread> th;
    const uint64_t per = (units + nt - 1) / nt;
    for (unsigned t = 0; t < nt; t++) {
        const uint64_t lo = t * per, hi = lo + per < units ? lo + per : units;
        if (lo >= hi) break;
        th.emplace_back([=] { sy_fill_range(p, lo, hi, 1); });
    }
    for (auto &t : th) t.join();
    return 0;
}

int apus_synth_fill_dev(void *dst, int kind, uint64_t n, uint64_t key, double a, double b, void *stream) {
    uint64_t units = 0;
    if (sy_check(dst, kind, n, a, b, &units)) return 1;
    if (!units) return 0;
    if (kind == APUS_SYNTH_U8) { a = 0; b = 255; }
    SyArgs p = {dst, kind, n, key, (float)a, (float)b};
    uint64_t blocks = (units + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    synth_fill_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p, units);
    APUS_LAUNCHED();
    return 0;
}

uint64_t apus_fnv1a(const void *data, uint64_t nbytes, uint64_t h) {
    const unsigned char *p = (const unsigned char *)data;
    for (uint64_t i = 0; i < nbytes; i++) { h ^= p[i]; h *= 0x100000001b3ull; }
    return h;
}

}  // extern "C"
