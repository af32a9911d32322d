// Dense f32 / bf16-weight linears: router gate, compressor projections, index
// head weights, grouped o-projection and the LM head (reference
// c/attn.h:460-666, c/attn.h:1439-1492, c/model.h:528-647).
//
// Two kernels: `f32_linear_seq_kernel` keeps the reference's summation order
// (the default, see apus_cuda_set_sum_order) and `f32_linear_kernel` is the
// split-K variant of the tree order, described here:
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


// ---- the reference's summation order -------------------------------------------------------
// out[m,o] = (((x[m,0]*w[o,0]) + x[m,1]*w[o,1]) + ...), every product and every
// add rounded to f32, k ascending (reference c/attn.h:460-465, 621-666,
// 1439-1492; c/model.h:585-636) -- bit for bit what the CPU path computes.
// Each output is a chain of K dependent adds, so the kernel is organised
// around the chains: one warp owns 32 output rows, a lane keeps MTT
// accumulators (tokens) of its row; MG such warps per CTA cover MG*MTT
// tokens.  All 256 threads of the CTA keep a three-deep ring of K tiles (32
// rows x 128 of w, BF16 kept as BF16 and widened exactly at use; the tokens' x)
// in flight with 16-byte asynchronous copies while the compute warps walk the
// current tile, so the weight stream is read once per CTA.  FP32-pipe bound at batch 32
// (2*O*K*M separately rounded operations), HBM-bound at batch 1.
//
// One fused multiply-add per term where that is the same number: when x and w both
// carry BF16 values (8 significant bits each) the product has at most 16 significant
// bits, so the f32 multiply is exact and round(acc + x*w) is what the separate add
// returns.  That also needs the product to be a normal number or an exact zero, so a
// tile takes the fused walk only if every operand in it is +-0 or a BF16 value with
// 2^-60 <= |v| < 2^60 (checked while the tile is staged; the whole CTA agrees on it);
// any other tile -- true f32 operands, subnormals, huge values, NaN -- takes the
// two-instruction walk.  BF16 weights with BF16 activations (o-projection, LM head,
// router, compressor projections) therefore run at half the instruction count with
// bit-identical sums.
constexpr int SQ_KT = 128;
constexpr int SQ_WP_F32 = (SQ_KT + 4) * 4;               // bytes per staged weight row, f32 (+16 B: conflict-free 16-byte reads)
constexpr int SQ_WP_BF16 = (SQ_KT + 8) * 2;              // ... BF16 rows stay BF16 in shared memory

__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                    // 0 source bytes = zero fill
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

// +-0, or a BF16 value with 67 <= biased exponent < 187
__device__ __forceinline__ bool fma_ok_f32(float v) {
    const uint32_t u = __float_as_uint(v), a = u & 0x7fffffffu;
    return a == 0u || ((u & 0xffffu) == 0u && a - (67u << 23) < (120u << 23));
}
__device__ __forceinline__ bool fma_ok_bf16x2(uint32_t p) {
    const uint32_t lo = p & 0x7fffu, hi = (p >> 16) & 0x7fffu;
    return (lo == 0u || lo - (67u << 7) < (120u << 7)) && (hi == 0u || hi - (67u << 7) < (120u << 7));
}

// Eight consecutive k of one output row against MTT token rows: acc[j] = acc[j] + x*w,
// k ascending.  FUSED: one FMA per term (only for tiles whose products are exact).
template <int MTT, bool FUSED>
__device__ __forceinline__ void seq_walk8(float (&acc)[MTT], const float4 &wa, const float4 &wb4,
                                          const float4 *xrow, int k8) {
#pragma unroll
    for (int j = 0; j < MTT; j++) {
        const float4 xa = xrow[j * (SQ_KT / 4) + 2 * k8], xb = xrow[j * (SQ_KT / 4) + 2 * k8 + 1];
        float a = acc[j];
        if (FUSED) {
            a = __fmaf_rn(xa.x, wa.x, a); a = __fmaf_rn(xa.y, wa.y, a);
            a = __fmaf_rn(xa.z, wa.z, a); a = __fmaf_rn(xa.w, wa.w, a);
            a = __fmaf_rn(xb.x, wb4.x, a); a = __fmaf_rn(xb.y, wb4.y, a);
            a = __fmaf_rn(xb.z, wb4.z, a); a = __fmaf_rn(xb.w, wb4.w, a);
        } else {
            a = __fadd_rn(a, __fmul_rn(xa.x, wa.x)); a = __fadd_rn(a, __fmul_rn(xa.y, wa.y));
            a = __fadd_rn(a, __fmul_rn(xa.z, wa.z)); a = __fadd_rn(a, __fmul_rn(xa.w, wa.w));
            a = __fadd_rn(a, __fmul_rn(xb.x, wb4.x)); a = __fadd_rn(a, __fmul_rn(xb.y, wb4.y));
            a = __fadd_rn(a, __fmul_rn(xb.z, wb4.z)); a = __fadd_rn(a, __fmul_rn(xb.w, wb4.w));
        }
        acc[j] = a;
    }
}

template <bool WBF16, int MTT, bool FUSED>
__device__ __forceinline__ void seq_walk_tile(float (&acc)[MTT], const unsigned char *wrow, const float4 *xrow) {
#pragma unroll 2
    for (int k8 = 0; k8 < SQ_KT / 8; k8++) {
        float4 wa, wb4;                                   // eight consecutive k of this lane's row
        if (WBF16) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(wrow + k8 * 16);
            wa = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                             __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
            wb4 = make_float4(__uint_as_float(raw.z << 16), __uint_as_float(raw.z & 0xffff0000u),
                              __uint_as_float(raw.w << 16), __uint_as_float(raw.w & 0xffff0000u));
        } else {
            wa = *reinterpret_cast<const float4 *>(wrow + k8 * 32);
            wb4 = *reinterpret_cast<const float4 *>(wrow + k8 * 32 + 16);
        }
        seq_walk8<MTT, FUSED>(acc, wa, wb4, xrow, k8);
    }
}

template <bool WBF16, int MTT, int MG, int SQ_NST>
__global__ void __launch_bounds__(256)
f32_linear_seq_kernel(const void *__restrict__ wv, const float *__restrict__ x, float *__restrict__ out,
                      int M, int K, int O, int flags, long long w_stride, long long x_stride, int x_ld,
                      long long out_stride, int out_ld) {
    constexpr int TPC = MTT * MG;                        // tokens per CTA
    constexpr int WP = WBF16 ? SQ_WP_BF16 : SQ_WP_F32;   // weight row pitch, bytes
    constexpr int W_BYTES = 32 * WP, X_BYTES = TPC * SQ_KT * 4, STAGE = W_BYTES + X_BYTES;
    extern __shared__ __align__(16) unsigned char sq_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int o0 = blockIdx.x * 32, m0 = blockIdx.y * TPC;
    const unsigned char *wbase = reinterpret_cast<const unsigned char *>(wv) +
                                 (size_t)blockIdx.z * w_stride * (WBF16 ? 2 : 4);
    x += blockIdx.z * x_stride;
    out += blockIdx.z * out_stride;
    const bool rin = flags & APUS_CUDA_R_IN;
    const int nt = (K + SQ_KT - 1) / SQ_KT;
    constexpr int ESZ = WBF16 ? 2 : 4, W_CH = SQ_KT * ESZ / 16;      // 16-byte chunks per weight row of a tile

    // all 256 threads issue the asynchronous 16-byte copies of tile t into stage t % SQ_NST
    auto issue = [&](int t) {
        unsigned char *st = sq_smem + (size_t)(t % SQ_NST) * STAGE;
        const int k0 = t * SQ_KT;
        for (int idx = tid; idx < 32 * W_CH; idx += 256) {
            const int r = idx / W_CH, c = idx - r * W_CH, k = k0 + c * (16 / ESZ);
            const bool ok = o0 + r < O && k < K;
            const unsigned char *src = wbase + ((size_t)(ok ? o0 + r : 0) * K + (ok ? k : 0)) * ESZ;
            cp_async16(st + (size_t)r * WP + c * 16, src, ok);
        }
        for (int idx = tid; idx < TPC * (SQ_KT / 4); idx += 256) {
            const int r = idx / (SQ_KT / 4), c = idx - r * (SQ_KT / 4), k = k0 + c * 4;
            const bool ok = m0 + r < M && k < K;
            const float *src = x + (size_t)(ok ? m0 + r : 0) * x_ld + (ok ? k : 0);
            cp_async16(st + W_BYTES + ((size_t)r * SQ_KT + c * 4) * 4, src, ok);
        }
    };

    float acc[MTT];
#pragma unroll
    for (int j = 0; j < MTT; j++) acc[j] = 0.f;
#pragma unroll
    for (int t = 0; t < SQ_NST - 1; t++) {
        if (t < nt) issue(t);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int t = 0; t < nt; t++) {
        if (t + SQ_NST - 1 < nt) issue(t + SQ_NST - 1);   // into the stage consumed at t - 1 (all passed its barrier)
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(SQ_NST - 1) : "memory");
        __syncthreads();                                  // tile t of every thread has landed
        unsigned char *st = sq_smem + (size_t)(t % SQ_NST) * STAGE;
        float *xs = reinterpret_cast<float *>(st + W_BYTES);
        // one pass over the staged tile: round the input (bf16_linear) and decide whether
        // every product of this tile is exact (see the head of this section)
        bool exact = true;
        for (int idx = tid; idx < TPC * SQ_KT; idx += 256) {
            float v = xs[idx];
            if (rin) { v = bf16_round(v); xs[idx] = v; }
            exact &= fma_ok_f32(v);
        }
        if (WBF16) {
            for (int idx = tid; idx < 32 * (SQ_KT / 8); idx += 256) {
                const int r = idx / (SQ_KT / 8), c = idx - r * (SQ_KT / 8);
                const uint4 raw = *reinterpret_cast<const uint4 *>(st + (size_t)r * WP + c * 16);
                exact &= fma_ok_bf16x2(raw.x) && fma_ok_bf16x2(raw.y) && fma_ok_bf16x2(raw.z) && fma_ok_bf16x2(raw.w);
            }
        } else {
            for (int idx = tid; idx < 32 * (SQ_KT / 4); idx += 256) {
                const int r = idx / (SQ_KT / 4), c = idx - r * (SQ_KT / 4);
                const float4 v = *reinterpret_cast<const float4 *>(st + (size_t)r * WP + c * 16);
                exact &= fma_ok_f32(v.x) && fma_ok_f32(v.y) && fma_ok_f32(v.z) && fma_ok_f32(v.w);
            }
        }
        const bool fused = __syncthreads_and(exact);
        if (warp < MG) {
            const unsigned char *wrow = st + (size_t)lane * WP;
            const float4 *xrow = reinterpret_cast<const float4 *>(xs + (size_t)warp * MTT * SQ_KT);
            if (fused) seq_walk_tile<WBF16, MTT, true>(acc, wrow, xrow);
            else seq_walk_tile<WBF16, MTT, false>(acc, wrow, xrow);
        }
        __syncthreads();                                  // stage t % SQ_NST may be refilled
    }
    if (warp < MG && o0 + lane < O) {
#pragma unroll
        for (int j = 0; j < MTT; j++) {
            const int m = m0 + warp * MTT + j;
            if (m < M) out[(size_t)m * out_ld + o0 + lane] = (flags & APUS_CUDA_R_OUT) ? bf16_round(acc[j]) : acc[j];
        }
    }
}

template <bool WBF16, int MTT, int MG>
static cudaError_t seq_launch(dim3 grid, cudaStream_t st, const void *w, const float *x, float *out, int M, int K,
                              int O, int flags, long long ws, long long xs, int x_ld, long long os, int out_ld) {
    constexpr int WP = WBF16 ? SQ_WP_BF16 : SQ_WP_F32;
    // ring depth: few tokens per CTA leave shared memory for a deeper ring, which a
    // CTA that is alone on its SM (small O) needs to cover the memory latency
    constexpr int SQ_NST = MTT * MG <= 8 ? 6 : 3;
    constexpr int smem = SQ_NST * (32 * WP + MTT * MG * SQ_KT * 4);
    auto kern = f32_linear_seq_kernel<WBF16, MTT, MG, SQ_NST>;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    kern<<<grid, 256, smem, st>>>(w, x, out, M, K, O, flags, ws, xs, x_ld, os, out_ld);
    return cudaSuccess;
}

template <bool WBF16>
static int launch_linear_seq(const void *w, long long ws, const float *x, long long xs, int x_ld, float *out,
                             long long os, int out_ld, int batch, int M, int K, int O, int flags,
                             cudaStream_t st) {
    const unsigned gx = (unsigned)ceil_div(O, 32);
#define SEQ_LAUNCH(MTT, MG)                                                                              \
    APUS_CUDA_OK((seq_launch<WBF16, MTT, MG>(dim3(gx, (unsigned)ceil_div(M, (MTT) * (MG)), (unsigned)batch), st, w, x, \
                                              out, M, K, O, flags, ws, xs, x_ld, os, out_ld)))
    // tokens per CTA: as many as keep enough CTAs in flight, at most 32
    const long long ctas32 = (long long)gx * batch * ceil_div(M, 32);
    if (M == 1) SEQ_LAUNCH(1, 1);
    else if (M <= 2) SEQ_LAUNCH(1, 2);
    else if (M <= 4) SEQ_LAUNCH(1, 4);
    else if (M <= 8 || ctas32 < 64) SEQ_LAUNCH(1, 8);          // 8 tokens per CTA, one per warp
    else if (M <= 16 || ctas32 < 148) SEQ_LAUNCH(2, 8);        // 16 tokens per CTA
    else SEQ_LAUNCH(4, 8);                                     // 32 tokens per CTA
#undef SEQ_LAUNCH
    return 0;
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
    if (sum_order() != APUS_CUDA_SUM_TREE) {
        APUS_REQUIRE(K % 8 == 0 && (w_stride * ((flags & APUS_CUDA_W_BF16) ? 2 : 4)) % 16 == 0,
                     "f32_linear: K=%d must be a multiple of 8", K);
        if ((flags & APUS_CUDA_W_BF16)
                ? launch_linear_seq<true>(w, w_stride, x, x_stride, x_ld, out, out_stride, out_ld, batch, M, K, O, flags, st)
                : launch_linear_seq<false>(w, w_stride, x, x_stride, x_ld, out, out_stride, out_ld, batch, M, K, O, flags, st))
            return 1;
        APUS_LAUNCHED();
        return 0;
    }
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
