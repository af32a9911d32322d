// Dense f32 / bf16-weight linears: router gate, compressor projections, index
// head weights, grouped o-projection and the LM head (reference
// c/attn.h:460-666, c/attn.h:1439-1492, c/model.h:528-647).
//
// out[m,o] = sum_k x[m,k] * w[o,k] in f32.  One warp per output row streams the
// weight row once (16-byte loads) for up to 8 activation rows at a time; the
// per-lane partial sums are combined by a shuffle tree, so the summation order
// differs from the reference's sequential-k loop (same products, f32
// accumulate).  HBM-bound for small M: bytes = O*K*sizeof(w).
#include "common.cuh"
#include "kernels.cuh"
#include "apus_b200.h"

namespace apus {

template <bool WBF16, int MT>
__global__ void __launch_bounds__(256)
f32_linear_kernel(const void *__restrict__ wv, const float *__restrict__ x,
                  float *__restrict__ out, int M, int K, int O, int flags) {
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long o = (long long)blockIdx.x * 8 + warp;
    int m0 = blockIdx.y * MT;
    if (o >= O) return;
    int mc = min(MT, M - m0);
    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; i++) acc[i] = 0.f;
    const bool rin = flags & APUS_CUDA_R_IN;
    for (int k = lane * 4; k < K; k += 128) {
        float4 w;
        if (WBF16) {
            uint2 raw = __ldg(reinterpret_cast<const uint2 *>(
                reinterpret_cast<const uint16_t *>(wv) + (size_t)o * K + k));
            w.x = __uint_as_float(raw.x << 16); w.y = __uint_as_float(raw.x & 0xffff0000u);
            w.z = __uint_as_float(raw.y << 16); w.w = __uint_as_float(raw.y & 0xffff0000u);
        } else {
            w = __ldg(reinterpret_cast<const float4 *>(
                reinterpret_cast<const float *>(wv) + (size_t)o * K + k));
        }
#pragma unroll
        for (int i = 0; i < MT; i++) {
            if (i < mc) {
                float4 xv = *reinterpret_cast<const float4 *>(x + (size_t)(m0 + i) * K + k);
                if (rin) {
                    xv.x = bf16_round(xv.x); xv.y = bf16_round(xv.y);
                    xv.z = bf16_round(xv.z); xv.w = bf16_round(xv.w);
                }
                acc[i] = fmaf(xv.x, w.x, acc[i]);
                acc[i] = fmaf(xv.y, w.y, acc[i]);
                acc[i] = fmaf(xv.z, w.z, acc[i]);
                acc[i] = fmaf(xv.w, w.w, acc[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MT; i++) {
        float v = warp_sum(acc[i]);
        if (lane == 0 && i < mc)
            out[(size_t)(m0 + i) * O + o] = (flags & APUS_CUDA_R_OUT) ? bf16_round(v) : v;
    }
}

int f32_linear(const void *w, const float *x, float *out, int M, int K, int O,
               int flags, cudaStream_t st) {
    APUS_REQUIRE(K % 4 == 0, "f32_linear: K=%d must be a multiple of 4", K);
    if (M <= 0 || O <= 0) return 0;
    const bool wb = flags & APUS_CUDA_W_BF16;
    if (M == 1) {
        dim3 grid((unsigned)ceil_div(O, 8), 1);
        if (wb) f32_linear_kernel<true, 1><<<grid, 256, 0, st>>>(w, x, out, M, K, O, flags);
        else    f32_linear_kernel<false, 1><<<grid, 256, 0, st>>>(w, x, out, M, K, O, flags);
    } else {
        dim3 grid((unsigned)ceil_div(O, 8), (unsigned)ceil_div(M, 8));
        if (wb) f32_linear_kernel<true, 8><<<grid, 256, 0, st>>>(w, x, out, M, K, O, flags);
        else    f32_linear_kernel<false, 8><<<grid, 256, 0, st>>>(w, x, out, M, K, O, flags);
    }
    APUS_LAUNCHED();
    return 0;
}

}  // namespace apus
