// mHC (manifold-constrained hyper-connections): per-token pre/post/comb maps,
// Sinkhorn normalisation, and the collapse fused with the adjacent RMSNorm.
//
// Reference: c/mhc.h:159-285 (maps, Sinkhorn order, collapse/apply/head) and
// c/layer.h:401-468 (where the BF16 rounds sit).  Two kernels per hc_pre:
//   1. mhc_mix_kernel: the (2+n)*n dots of the f32 map matrix fn [nmix, n*d]
//      with the token state, plus the sum of squares, one CTA per (mix, token);
//   2. mhc_pre_finish_kernel: one CTA per token turns the raw dots into
//      pre/post/comb (rsqrt applied AFTER the dot, sigmoid gates, Sinkhorn with
//      the reference's eps placement), collapses the n streams with `pre`,
//      BF16-rounds and, when a norm weight is given, applies RMSNorm to the
//      collapsed row in the same kernel (reference c/attn.h:371-378).
// Bytes per token: fn (nmix*n*d*4, L2-resident across tokens) + 2 reads of the
// n*d state.
#include "common.cuh"
#include "kernels.cuh"

namespace apus {

__device__ __forceinline__ float block_sum(float v, float *red) {
    v = warp_sum(v);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[0] = t;
    }
    __syncthreads();
    return red[0];
}

// grid (nmix + 1, rows): blockIdx.x < nmix -> raw[row, j] = fn_j . x ;
// blockIdx.x == nmix -> raw[row, nmix] = sum x^2.
__global__ void __launch_bounds__(256)
mhc_mix_kernel(const float *__restrict__ x4, const float *__restrict__ fn, int nx, int nmix,
               float *__restrict__ raw) {
    __shared__ float red[32];
    const int j = blockIdx.x, row = blockIdx.y;
    const float *x = x4 + (size_t)row * nx;
    float acc = 0.f;
    if (j < nmix) {
        const float *f = fn + (size_t)j * nx;
        for (int i = threadIdx.x * 4; i < nx; i += blockDim.x * 4) {
            float4 a = __ldg(reinterpret_cast<const float4 *>(f + i));
            float4 b = *reinterpret_cast<const float4 *>(x + i);
            acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
            acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
        }
    } else {
        for (int i = threadIdx.x * 4; i < nx; i += blockDim.x * 4) {
            float4 b = *reinterpret_cast<const float4 *>(x + i);
            acc = fmaf(b.x, b.x, acc); acc = fmaf(b.y, b.y, acc);
            acc = fmaf(b.z, b.z, acc); acc = fmaf(b.w, b.w, acc);
        }
    }
    float tot = block_sum(acc, red);
    if (threadIdx.x == 0) raw[(size_t)row * (nmix + 1) + j] = tot;
}

// The same dots in the reference's summation order (c/mhc.h:159-176: one f32
// accumulator per dot, products rounded before each add, index ascending).
// That order is a chain of n*d dependent adds per dot, so the kernel is bound
// by add latency, not bandwidth: 256 producer threads stage rounded products
// of a tile in shared memory while one lane per dot (the consumer warps) walks
// the previous tile.  One CTA per token; chain c < nmix is fn_c . x, chain
// nmix is sum x^2.
__global__ void __launch_bounds__(320)
mhc_mix_seq_kernel(const float *__restrict__ x4, const float *__restrict__ fn, int nx, int nmix,
                   int MIX_TI, float *__restrict__ raw) {
    extern __shared__ __align__(16) float s_prod[];
    const int C = nmix + 1, stride = MIX_TI + 4, tid = threadIdx.x;
    const int row = blockIdx.x, nt = (nx + MIX_TI - 1) / MIX_TI;
    const float *x = x4 + (size_t)row * nx;
    const bool consumer = tid >= 256;
    float acc0 = 0.f, acc1 = 0.f;             // a consumer lane owns chains c0 and c0 + 64
    const int c0 = tid - 256;
    auto produce = [&](int t) {
        float *dst = s_prod + (size_t)(t & 1) * C * stride;
        const int q = MIX_TI / 4;
        for (int idx = tid; idx < C * q; idx += 256) {
            const int c = idx / q, i4 = idx - c * q, gi = t * MIX_TI + 4 * i4;
            float4 xv = make_float4(0.f, 0.f, 0.f, 0.f), fv;
            if (gi < nx) xv = *reinterpret_cast<const float4 *>(x + gi);
            fv = xv;
            if (c < nmix && gi < nx) fv = __ldg(reinterpret_cast<const float4 *>(fn + (size_t)c * nx + gi));
            float4 p = make_float4(__fmul_rn(fv.x, xv.x), __fmul_rn(fv.y, xv.y), __fmul_rn(fv.z, xv.z),
                                   __fmul_rn(fv.w, xv.w));
            *reinterpret_cast<float4 *>(dst + (size_t)c * stride + 4 * i4) = p;
        }
    };
    auto chain = [&](const float *src, float acc) {
        const float4 *p = reinterpret_cast<const float4 *>(src);
#pragma unroll 8
        for (int i4 = 0; i4 < MIX_TI / 4; i4++) {
            float4 v = p[i4];
            acc = __fadd_rn(acc, v.x); acc = __fadd_rn(acc, v.y);
            acc = __fadd_rn(acc, v.z); acc = __fadd_rn(acc, v.w);
        }
        return acc;
    };
    if (!consumer) produce(0);
    __syncthreads();
    for (int t = 0; t < nt; t++) {
        if (!consumer) {
            if (t + 1 < nt) produce(t + 1);
        } else {
            const float *src = s_prod + (size_t)(t & 1) * C * stride;
            if (c0 < C) acc0 = chain(src + (size_t)c0 * stride, acc0);
            if (c0 + 64 < C) acc1 = chain(src + (size_t)(c0 + 64) * stride, acc1);
        }
        __syncthreads();
    }
    if (consumer) {
        if (c0 < C) raw[(size_t)row * C + c0] = acc0;
        if (c0 + 64 < C) raw[(size_t)row * C + c0 + 64] = acc1;
    }
}

__device__ __forceinline__ float sigm(float x) { return __fdiv_rn(1.0f, 1.0f + exp_rn(-x)); }

// Sinkhorn on an n x n matrix held by one thread (reference c/mhc.h:181-218).
__device__ void sinkhorn(float *c, int n, int iters, float eps) {
    for (int j = 0; j < n; j++) {
        float *r = c + j * n, mx = r[0], sum = 0.f;
        for (int k = 1; k < n; k++) mx = fmaxf(mx, r[k]);
        for (int k = 0; k < n; k++) { r[k] = exp_rn(r[k] - mx); sum = __fadd_rn(sum, r[k]); }
        for (int k = 0; k < n; k++) r[k] = __fadd_rn(__fdiv_rn(r[k], sum), eps);
    }
    for (int it = 0; it < iters; it++) {
        if (it) for (int j = 0; j < n; j++) {
            float sum = 0.f;
            for (int k = 0; k < n; k++) sum = __fadd_rn(sum, c[j * n + k]);
            float den = __fadd_rn(sum, eps);
            for (int k = 0; k < n; k++) c[j * n + k] = __fdiv_rn(c[j * n + k], den);
        }
        for (int k = 0; k < n; k++) {
            float sum = 0.f;
            for (int j = 0; j < n; j++) sum = __fadd_rn(sum, c[j * n + k]);
            float den = __fadd_rn(sum, eps);
            for (int j = 0; j < n; j++) c[j * n + k] = __fdiv_rn(c[j * n + k], den);
        }
    }
}

#define MHC_MAX_N 8

// One CTA per token. head_mode: only `pre` gates (scalar scale), no post/comb.
__global__ void __launch_bounds__(256)
mhc_pre_finish_kernel(const float *__restrict__ x4, const float *__restrict__ raw, int d, int n,
                      int nmix, const float *__restrict__ scale, float head_scale,
                      const float *__restrict__ base, float norm_eps, float hc_eps, int iters,
                      int head_mode, const float *__restrict__ norm_w, float rms_eps,
                      float *__restrict__ pre_out, float *__restrict__ post_out,
                      float *__restrict__ comb_out, float *__restrict__ y,
                      float *__restrict__ y_normed, int seq) {
    extern __shared__ float s_sq[];           // seq: d squares of the collapsed row
    __shared__ float s_pre[MHC_MAX_N];
    __shared__ float red[32];
    const int row = blockIdx.x;
    const float *rw = raw + (size_t)row * (nmix + 1);
    if (threadIdx.x == 0) {
        float mean = __fdiv_rn(rw[nmix], (float)(n * d));
        float r = __fdiv_rn(1.0f, sqrtf(__fadd_rn(mean, norm_eps)));
        if (head_mode) {
            for (int j = 0; j < n; j++) {
                float m = __fmul_rn(rw[j], r);
                s_pre[j] = __fadd_rn(sigm(__fadd_rn(__fmul_rn(m, head_scale), base[j])), hc_eps);
            }
        } else {
            float comb[MHC_MAX_N * MHC_MAX_N];
            for (int j = 0; j < n; j++) {
                float m = __fmul_rn(rw[j], r);
                s_pre[j] = __fadd_rn(sigm(__fadd_rn(__fmul_rn(m, scale[0]), base[j])), hc_eps);
                float m2 = __fmul_rn(rw[n + j], r);
                float po = __fmul_rn(2.0f, sigm(__fadd_rn(__fmul_rn(m2, scale[1]), base[n + j])));
                if (post_out) post_out[(size_t)row * n + j] = po;
            }
            for (int i = 0; i < n * n; i++) {
                float m = __fmul_rn(rw[2 * n + i], r);
                comb[i] = __fadd_rn(__fmul_rn(m, scale[2]), base[2 * n + i]);
            }
            sinkhorn(comb, n, iters, hc_eps);
            if (comb_out)
                for (int i = 0; i < n * n; i++) comb_out[(size_t)row * n * n + i] = comb[i];
        }
        if (pre_out) for (int j = 0; j < n; j++) pre_out[(size_t)row * n + j] = s_pre[j];
    }
    __syncthreads();
    if (!y) return;
    // collapse: y[i] = sum_j pre[j] * X[j,i], j ascending, mul then add; BF16 round
    const float *x = x4 + (size_t)row * n * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < n; j++) acc = __fadd_rn(acc, __fmul_rn(s_pre[j], x[(size_t)j * d + i]));
        acc = bf16_round(acc);
        y[(size_t)row * d + i] = acc;
        if (seq) s_sq[i] = __fmul_rn(acc, acc);
        else ss = fmaf(acc, acc, ss);
    }
    if (!y_normed) return;
    float tot;
    if (seq) {                                // reference order: one accumulator, index ascending
        __syncthreads();
        if (threadIdx.x == 0) {
            float a = 0.f;
#pragma unroll 8
            for (int i = 0; i < d; i++) a = __fadd_rn(a, s_sq[i]);
            red[0] = a;
        }
        __syncthreads();
        tot = red[0];
    } else {
        tot = block_sum(ss, red);
    }
    float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(tot, (float)d), rms_eps)));
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = y[(size_t)row * d + i];
        y_normed[(size_t)row * d + i] = bf16_round(__fmul_rn(norm_w[i], __fmul_rn(v, inv)));
    }
}

// Y[j,i] = bf16(post[j]*f[i] + sum_k comb[k,j]*R[k,i]) (reference c/mhc.h:259-270,
// c/layer.h:445-456).
__global__ void mhc_post_kernel(const float *__restrict__ f, const float *__restrict__ res,
                                const float *__restrict__ post, const float *__restrict__ comb,
                                float *__restrict__ y4, int d, int n) {
    const int row = blockIdx.y;
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d) return;
    const float *R = res + (size_t)row * n * d;
    const float *po = post + (size_t)row * n, *cb = comb + (size_t)row * n * n;
    float fv = f[(size_t)row * d + i];
    float rv[MHC_MAX_N];
    for (int k = 0; k < n; k++) rv[k] = R[(size_t)k * d + i];
    for (int j = 0; j < n; j++) {
        float acc = __fmul_rn(po[j], fv);
        for (int k = 0; k < n; k++) acc = __fadd_rn(acc, __fmul_rn(cb[k * n + j], rv[k]));
        y4[((size_t)row * n + j) * d + i] = bf16_round(acc);
    }
}

static float *g_raw = nullptr;
static size_t g_raw_cap = 0;
static int ensure_raw(size_t floats) {
    if (floats <= g_raw_cap) return 0;
    if (g_raw) cudaFree(g_raw);
    g_raw = nullptr; g_raw_cap = 0;
    APUS_CUDA_OK(cudaMalloc(&g_raw, floats * sizeof(float)));
    g_raw_cap = floats;
    return 0;
}

// raw[row, 0..nmix] for `rows` tokens in the sum order now in force.
static int launch_mix(const float *x4, const float *fn, int nx, int nmix, float *raw, int rows,
                      cudaStream_t st) {
    if (sum_order() == APUS_CUDA_SUM_TREE) {
        mhc_mix_kernel<<<dim3(nmix + 1, rows), 256, 0, st>>>(x4, fn, nx, nmix, raw);
        APUS_LAUNCHED();
        return 0;
    }
    const int C = nmix + 1, ti = C <= 48 ? 512 : 128;
    const size_t smem = (size_t)2 * C * (ti + 4) * sizeof(float);
    static bool attr_set = false;
    if (!attr_set) {
        APUS_CUDA_OK(cudaFuncSetAttribute(mhc_mix_seq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        APUS_CUDA_OK(cudaFuncSetAttribute(mhc_pre_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
        attr_set = true;
    }
    mhc_mix_seq_kernel<<<rows, 320, smem, st>>>(x4, fn, nx, nmix, ti, raw);
    APUS_LAUNCHED();
    return 0;
}
static inline int finish_seq() { return sum_order() == APUS_CUDA_SUM_TREE ? 0 : 1; }
static inline size_t finish_smem(int d) { return finish_seq() ? (size_t)d * sizeof(float) : 0; }

int mhc_pre(const float *x4, int d, int n, const float *fn, const float *scale,
            const float *base, float norm_eps, float hc_eps, int iters,
            const float *norm_w, float rms_eps, float *pre, float *post,
            float *comb, float *y, float *y_normed, int rows, cudaStream_t st) {
    APUS_REQUIRE(n >= 1 && n <= MHC_MAX_N && (n * d) % 4 == 0, "mhc: n=%d d=%d unsupported", n, d);
    if (rows <= 0) return 0;
    int nmix = (2 + n) * n;
    if (ensure_raw((size_t)rows * (nmix + 1))) return 1;
    if (launch_mix(x4, fn, n * d, nmix, g_raw, rows, st)) return 1;
    mhc_pre_finish_kernel<<<rows, 256, finish_smem(d), st>>>(x4, g_raw, d, n, nmix, scale, 0.f, base,
                                                norm_eps, hc_eps, iters, 0, norm_w, rms_eps,
                                                pre, post, comb, y, norm_w ? y_normed : nullptr, finish_seq());
    APUS_LAUNCHED();
    return 0;
}

int mhc_head(const float *x4, int d, int n, const float *fn, float scale,
             const float *base, float norm_eps, float hc_eps, float *y,
             int rows, cudaStream_t st) {
    APUS_REQUIRE(n >= 1 && n <= MHC_MAX_N && (n * d) % 4 == 0, "mhc: n=%d d=%d unsupported", n, d);
    if (rows <= 0) return 0;
    if (ensure_raw((size_t)rows * (n + 1))) return 1;
    if (launch_mix(x4, fn, n * d, n, g_raw, rows, st)) return 1;
    mhc_pre_finish_kernel<<<rows, 256, finish_smem(d), st>>>(x4, g_raw, d, n, n, nullptr, scale, base,
                                                norm_eps, hc_eps, 0, 1, nullptr, 0.f,
                                                nullptr, nullptr, nullptr, y, nullptr, finish_seq());
    APUS_LAUNCHED();
    return 0;
}

int mhc_post(const float *f, const float *res4, const float *post,
             const float *comb, float *y4, int d, int n, int rows,
             cudaStream_t st) {
    APUS_REQUIRE(n >= 1 && n <= MHC_MAX_N, "mhc: n=%d unsupported", n);
    if (rows <= 0) return 0;
    mhc_post_kernel<<<dim3(ceil_div(d, 256), rows), 256, 0, st>>>(f, res4, post, comb, y4, d, n);
    APUS_LAUNCHED();
    return 0;
}

// ---- entry point that allocates nothing ------------------------------------------------
//
// Some hosts of this library may not allocate device memory at the moment they
// call in: an engine that has handed all of HBM to its own arena, a caller
// inside a region where the driver forbids allocation, or a real-time loop
// that must not take the allocator's lock.  For them the scratch of the mHC
// pre step (the raw map dots, (2+n)*n+1 floats per token) lives in a fixed
// file-scope device array instead of a grown buffer.  Every GPU that loads the
// library carries the array (MHC_NOALLOC_MAX_ROWS * 65 floats = 66,560 bytes)
// until the process exits.
#define MHC_NOALLOC_MAX_ROWS 256
#define MHC_NOALLOC_MAX_DEVICES 64
static __device__ __align__(256) float g_mhc_static_raw[MHC_NOALLOC_MAX_ROWS * (MHC_MAX_N * (MHC_MAX_N + 2) + 1)];
// In host code the array's name is only a handle for the runtime, not a device
// address; the address each device gives it is looked up once per device.
static float *g_mhc_static_ptr[MHC_NOALLOC_MAX_DEVICES];

static int mhc_static_scratch(float **out) {
    int dev = 0;
    APUS_CUDA_OK(cudaGetDevice(&dev));
    APUS_REQUIRE(dev >= 0 && dev < MHC_NOALLOC_MAX_DEVICES, "hc_pre_noalloc: device %d out of range", dev);
    if (!g_mhc_static_ptr[dev]) {
        void *p = nullptr;
        APUS_CUDA_OK(cudaGetSymbolAddress(&p, g_mhc_static_raw));
        g_mhc_static_ptr[dev] = static_cast<float *>(p);
    }
    *out = g_mhc_static_ptr[dev];
    return 0;
}

int mhc_pre_noalloc(const float *x4, int d, int n, const float *fn, const float *scale,
                    const float *base, float norm_eps, float hc_eps, int iters,
                    const float *norm_w, float rms_eps, float *post, float *comb, float *y,
                    float *y_normed, int rows, cudaStream_t st) {
    APUS_REQUIRE(n >= 1 && n <= MHC_MAX_N && (n * d) % 4 == 0, "hc_pre_noalloc: n=%d d=%d unsupported", n, d);
    APUS_REQUIRE(rows <= MHC_NOALLOC_MAX_ROWS,
                 "hc_pre_noalloc: %d rows exceed the fixed scratch of %d rows; split the call or use "
                 "apus_cuda_hc_pre", rows, MHC_NOALLOC_MAX_ROWS);
    APUS_REQUIRE(y != nullptr, "hc_pre_noalloc: y must not be NULL");
    if (rows <= 0) return 0;
    float *raw = nullptr;
    if (mhc_static_scratch(&raw)) return 1;
    const int nmix = (2 + n) * n;
    // every raw[row, 0..nmix] slot read by the finish kernel is written by the mix
    // kernel of the same call, so nothing left over from an earlier call is used
    if (launch_mix(x4, fn, n * d, nmix, raw, rows, st)) return 1;
    mhc_pre_finish_kernel<<<rows, 256, finish_smem(d), st>>>(x4, raw, d, n, nmix, scale, 0.f, base, norm_eps,
                                                hc_eps, iters, 0, norm_w, rms_eps, nullptr, post,
                                                comb, y, norm_w ? y_normed : nullptr, finish_seq());
    APUS_LAUNCHED();
    return 0;
}

}  // namespace apus

// The mHC pre step for callers that cannot allocate device memory (see the
// comment above g_mhc_static_raw).  All pointers are device pointers owned by
// the caller; the kernels run on `stream`.  The first call on each device looks
// up the device address of the fixed scratch array (cudaGetSymbolAddress), so
// make that first call outside any stream capture.  Calls share the one scratch
// array per device: two calls whose kernels can overlap on the GPU (different
// streams without an ordering between them) race on it.  rows > 256 is
// rejected with an error.
extern "C" int apus_cuda_hc_pre_noalloc_dev(const float *x4, size_t d, size_t n, const float *fn,
                                            const float *scale, const float *base, float norm_eps,
                                            float hc_eps, int iters, const float *norm_w,
                                            float rms_eps, float *y, float *y_normed, float *post,
                                            float *comb, int rows, void *stream) {
    return apus::mhc_pre_noalloc(x4, (int)d, (int)n, fn, scale, base, norm_eps, hc_eps, iters, norm_w,
                                 rms_eps, post, comb, y, y_normed, rows, (cudaStream_t)stream);
}
