// Dense f32 / bf16-weight linears: router gate, compressor projections, index
// head weights, grouped o-projection and the LM head (reference
// c/attn.h:460-666, c/attn.h:1439-1492, c/model.h:528-647).
//
// out[m,o] = sum_k x[m,k] * w[o,k] in f32.  A CTA of 8 warps owns OT output rows
// and up to MT activation rows; the warps split K into eight contiguous ranges,
// every lane keeps OT*MT partial sums, and the partials are combined by a
// shuffle tree and a fixed-order sum over the warps (deterministic; the
// summation order differs from the reference's sequential-k loop, the
// products are the same f32 products).  All loads of a K step are issued
// before its FMAs so that a thread keeps OT+MT 16-byte loads in flight.
// HBM-bound for small M: bytes = O*K*sizeof(w).
#include "common.cuh"
#include "kernels.cuh"
#include "apus_b200.h"

namespace apus {

template <bool WBF16>
__device__ __forceinline__ float4 load_w4(const void *wv, size_t idx) {
    if (WBF16) {
        uint2 raw = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(wv) + idx));
        return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                           __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
    }
    return __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(wv) + idx));
}

template <bool WBF16, int OT, int MT>
__global__ void __launch_bounds__(256)
f32_linear_kernel(const void *__restrict__ wv, const float *__restrict__ x,
                  float *__restrict__ out, int M, int K, int O, int flags, long long w_stride,
                  long long x_stride, int x_ld, long long out_stride, int out_ld) {
    __shared__ float part[8][OT * MT];
    wv = WBF16 ? (const void *)(reinterpret_cast<const uint16_t *>(wv) + blockIdx.z * w_stride)
               : (const void *)(reinterpret_cast<const float *>(wv) + blockIdx.z * w_stride);
    x += blockIdx.z * x_stride;
    out += blockIdx.z * out_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int o0 = blockIdx.x * OT, m0 = blockIdx.y * MT;
    const int oc = min(OT, O - o0), mc = min(MT, M - m0);
    // K range of this warp, in units of 128 elements (one float4 per lane)
    const int steps = (K + 127) / 128;
    const int s0 = (steps * warp) / 8, s1 = (steps * (warp + 1)) / 8;
    const bool rin = flags & APUS_CUDA_R_IN;
    float acc[OT][MT];
#pragma unroll
    for (int a = 0; a < OT; a++)
#pragma unroll
        for (int b = 0; b < MT; b++) acc[a][b] = 0.f;
    for (int s = s0; s < s1; s++) {
        const int k = s * 128 + lane * 4;
        if (k >= K) continue;
        float4 wr[OT], xr[MT];
#pragma unroll
        for (int a = 0; a < OT; a++)
            wr[a] = a < oc ? load_w4<WBF16>(wv, (size_t)(o0 + a) * K + k) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int b = 0; b < MT; b++)
            xr[b] = b < mc ? __ldg(reinterpret_cast<const float4 *>(x + (size_t)(m0 + b) * x_ld + k))
                           : make_float4(0.f, 0.f, 0.f, 0.f);
        if (rin) {
#pragma unroll
            for (int b = 0; b < MT; b++) {
                xr[b].x = bf16_round(xr[b].x); xr[b].y = bf16_round(xr[b].y);
                xr[b].z = bf16_round(xr[b].z); xr[b].w = bf16_round(xr[b].w);
            }
        }
#pragma unroll
        for (int a = 0; a < OT; a++)
#pragma unroll
            for (int b = 0; b < MT; b++) {
                acc[a][b] = fmaf(xr[b].x, wr[a].x, acc[a][b]);
                acc[a][b] = fmaf(xr[b].y, wr[a].y, acc[a][b]);
                acc[a][b] = fmaf(xr[b].z, wr[a].z, acc[a][b]);
                acc[a][b] = fmaf(xr[b].w, wr[a].w, acc[a][b]);
            }
    }
#pragma unroll
    for (int a = 0; a < OT; a++)
#pragma unroll
        for (int b = 0; b < MT; b++) {
            float v = warp_sum(acc[a][b]);
            if (lane == 0) part[warp][a * MT + b] = v;
        }
    __syncthreads();
    const int t = threadIdx.x;
    if (t < OT * MT) {
        const int a = t / MT, b = t % MT;
        if (a < oc && b < mc) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) v += part[w][t];
            out[(size_t)(m0 + b) * out_ld + o0 + a] = (flags & APUS_CUDA_R_OUT) ? bf16_round(v) : v;
        }
    }
}

template <bool WBF16>
static void launch_linear(const void *w, long long ws, const float *x, long long xs, int x_ld, float *out,
                          long long os, int out_ld, int batch, int M, int K, int O, int flags,
                          cudaStream_t st) {
    if (M == 1) {
        dim3 grid((unsigned)ceil_div(O, 8), 1, (unsigned)batch);
        f32_linear_kernel<WBF16, 8, 1><<<grid, 256, 0, st>>>(w, x, out, M, K, O, flags, ws, xs, x_ld, os, out_ld);
    } else if (M <= 4) {
        dim3 grid((unsigned)ceil_div(O, 4), 1, (unsigned)batch);
        f32_linear_kernel<WBF16, 4, 4><<<grid, 256, 0, st>>>(w, x, out, M, K, O, flags, ws, xs, x_ld, os, out_ld);
    } else {
        dim3 grid((unsigned)ceil_div(O, 4), (unsigned)ceil_div(M, 8), (unsigned)batch);
        f32_linear_kernel<WBF16, 4, 8><<<grid, 256, 0, st>>>(w, x, out, M, K, O, flags, ws, xs, x_ld, os, out_ld);
    }
}

int f32_linear_batched(const void *w, long long w_stride, const float *x, long long x_stride, int x_ld,
                       float *out, long long out_stride, int out_ld, int batch, int M, int K, int O,
                       int flags, cudaStream_t st) {
    APUS_REQUIRE(K % 4 == 0 && x_ld % 4 == 0 && x_stride % 4 == 0 && w_stride % 4 == 0,
                 "f32_linear: K=%d and the strides must be multiples of 4", K);
    if (M <= 0 || O <= 0 || batch <= 0) return 0;
    if (flags & APUS_CUDA_W_BF16)
        launch_linear<true>(w, w_stride, x, x_stride, x_ld, out, out_stride, out_ld, batch, M, K, O, flags, st);
    else
        launch_linear<false>(w, w_stride, x, x_stride, x_ld, out, out_stride, out_ld, batch, M, K, O, flags, st);
    APUS_LAUNCHED();
    return 0;
}

int f32_linear(const void *w, const float *x, float *out, int M, int K, int O,
               int flags, cudaStream_t st) {
    return f32_linear_batched(w, 0, x, 0, K, out, 0, O, 1, M, K, O, flags, st);
}

}  // namespace apus
