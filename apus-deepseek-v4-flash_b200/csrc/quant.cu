// Activation quantisation and RMSNorm.
#include "common.cuh"
#include "kernels.cuh"

namespace apus {

// One warp per (row, 128-group): BF16-round, amax (floored at 1e-4), power-of-
// two scale 2^ceil(log2(amax/448)), E4M3 codes by hardware RNE conversion
// (reference c/attn.h:393-402 + c/fp4.h:293-321).  K % 128 == 0.
__global__ void act_quant_kernel(const float *__restrict__ x, const int *__restrict__ arow,
                                 int M, int K, uint8_t *__restrict__ codes,
                                 float *__restrict__ scales, const int *m_dev) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    int nab = K >> 7;
    if (m_dev) M = min(M, *m_dev);
    long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (wid >= (long long)M * nab) return;
    int m = (int)(wid / nab), b = (int)(wid % nab);
    int src = arow ? arow[m] : m;
    float4 v = *reinterpret_cast<const float4 *>(x + (size_t)src * K + b * 128 + lane * 4);
    v.x = bf16_round(v.x); v.y = bf16_round(v.y);
    v.z = bf16_round(v.z); v.w = bf16_round(v.w);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = warp_max(amax);
    amax = fmaxf(amax, 1e-4f);
    float s = ceil_pow2(__fmul_rn(amax, 1.0f / 448.0f));
    // x / s with s a power of two is exact, and equals x * (1/s)
    float inv = __uint_as_float(0x7f000000u - __float_as_uint(s));
    uint32_t lo = e4m3x2_from_f32(v.x * inv, v.y * inv);
    uint32_t hi = e4m3x2_from_f32(v.z * inv, v.w * inv);
    *reinterpret_cast<uint32_t *>(codes + (size_t)m * K + b * 128 + lane * 4) = lo | (hi << 16);
    if (lane == 0) scales[(size_t)m * nab + b] = s;
}

int act_quant(const float *x, const int *arow, int M, int K, uint8_t *codes,
              float *scales, const int *m_dev, cudaStream_t st) {
    APUS_REQUIRE(K % 128 == 0, "act_quant: K=%d must be a multiple of 128", K);
    if (M <= 0) return 0;
    long long warps = (long long)M * (K / 128);
    launch_k(act_quant_kernel, ceil_div(warps * 32, 256), 256, 0, st, x, arow, M, K, codes,
                                                              scales, m_dev);
    APUS_LAUNCHED();
    return 0;
}

// One CTA per row: y = bf16(w * (x * 1/sqrt(mean(x^2)+eps))) (reference
// c/attn.h:371-378).  seq: the sum of squares walks the row in index order with
// one accumulator and rounded squares, as the reference's loop does; otherwise
// it is a tree reduction.
__global__ void rms_norm_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                float eps, float *__restrict__ y, int64_t n, int seq) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ __align__(16) float s_sq[];
    const float *xr = x + (size_t)blockIdx.x * n;
    float *yr = y + (size_t)blockIdx.x * n;
    __shared__ float red[32];
    if (seq) {
        for (int64_t i = threadIdx.x; i < n; i += blockDim.x) s_sq[i] = __fmul_rn(xr[i], xr[i]);
        __syncthreads();
        if (threadIdx.x == 0) red[0] = seq_sum_smem(s_sq, (int)n, 0.f);
    } else {
        float ss = 0.f;
        for (int64_t i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x < 32) {
            float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
            v = warp_sum(v);
            if (threadIdx.x == 0) red[0] = v;
        }
    }
    __syncthreads();
    float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(red[0], (float)n), eps)));
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x)
        yr[i] = bf16_round(__fmul_rn(w[i], __fmul_rn(xr[i], inv)));
}

int rms_norm(const float *x, const float *w, float eps, float *y, int64_t n,
             int64_t rows, cudaStream_t st) {
    if (rows <= 0) return 0;
    int threads = n >= 1024 ? 256 : 128;
    const int seq = sum_tree(APUS_CUDA_TREE_NORMS) ? 0 : 1;
    const size_t smem = seq ? (size_t)n * sizeof(float) : 0;
    APUS_REQUIRE(smem <= 200 * 1024, "rms_norm: row of %lld elements exceeds the staging buffer", (long long)n);
    if (smem > 48 * 1024 && ensure_dyn_smem((const void *)rms_norm_kernel, 200 * 1024)) return 1;
    launch_k(rms_norm_kernel, (unsigned)rows, threads, smem, st, x, w, eps, y, n, seq);
    APUS_LAUNCHED();
    return 0;
}

}  // namespace apus
