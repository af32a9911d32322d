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
    APUS_PDL_WAIT();
    APUS_PDL_GO();
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
// around the chains: a lane owns R output rows (rows lane, lane + 32, ...) and
// MTT tokens, i.e. R*MTT accumulators; MG such warps per CTA cover MG*MTT
// tokens of the same 32*R rows.  A second set of warps keeps a ring of K tiles
// (the rows' weights as stored and the tokens' x) in flight with 16-byte
// asynchronous copies, so the weight stream is read once per CTA.  BF16
// weights are widened to f32 once per CTA and tile (into a second buffer) and
// not once per warp; the walk then reads f32 rows for either storage.
// Issue-bound at batch 32 (one multiply-add per term and the shared-memory reads
// that feed it), add-latency bound for small grids, HBM-bound at batch 1.
//
// One fused multiply-add per term where that is the same number: when x and w both
// carry BF16 values (8 significant bits each) the product has at most 16 significant
// bits, so the f32 multiply is exact and round(acc + x*w) is what the separate add
// returns.  That also needs the product to be a normal number or an exact zero, so a
// tile takes the fused walk only if every operand in it is +-0 or a BF16 value with
// 2^-60 <= |v| < 2^60 (checked while the tile is staged; the whole CTA agrees on it);
// any other tile -- true f32 operands, subnormals, huge values, NaN -- takes the
// two-instruction walk.  BF16-stored weights with BF16 activations (o-projection, LM
// head) therefore run at half the instruction count with bit-identical sums; f32-stored
// weights always take the two-instruction walk (those projections are latency bound).
constexpr int SQ_KT = 128;
constexpr int SQ_WP = (SQ_KT + 4) * 4;                   // f32 weight row pitch, bytes (+16 B: conflict-free 16-byte reads)

template <bool WBF16, int R, int MTT, int MG, int NST>
struct SeqCfg {
    static constexpr int ROWS = 32 * R;                  // output rows per CTA
    static constexpr int TPC = MTT * MG;                 // tokens per CTA
    static constexpr int ESZ = WBF16 ? 2 : 4;
    static constexpr int WP_RAW = SQ_KT * ESZ + 16;      // pitch of a staged weight row as stored (272 / 528 bytes)
    static constexpr int W_RAW = ROWS * WP_RAW;
    static constexpr int X_BYTES = TPC * SQ_KT * 4;
    static constexpr int STAGE = W_RAW + X_BYTES;
    static constexpr int WIDE = WBF16 ? ROWS * SQ_WP : 0;  // the widened copy of the current tile
    static constexpr int SMEM = NST * STAGE + 2 * WIDE + 16;   // ring, two widened halves, the tiles' exactness flags
};

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
// The same test on two BF16 values at once, per 16-bit half h = |value| bits: with
// bit 15 set first no subtraction borrows across the halves, and bit 15 of
// (h | 0x8000) - c then says h >= c.  Returns bit 15 / 31 set for a half that is
// neither zero nor inside the window.
__device__ __forceinline__ uint32_t fma_bad_bf16x2(uint32_t p) {
    const uint32_t a = (p & 0x7fff7fffu) | 0x80008000u;
    const uint32_t ge_lo = a - 0x21802180u;              // 67 << 7
    const uint32_t ge_hi = a - 0x5d805d80u;              // 187 << 7
    const uint32_t nz = a - 0x00010001u;
    return nz & ~(ge_lo & ~ge_hi);
}

// Eight consecutive k of one output row against one token: acc = acc + x*w, k ascending.
template <bool FUSED>
__device__ __forceinline__ float seq_walk8(float a, const float4 &wa, const float4 &wb, const float4 &xa,
                                           const float4 &xb) {
    if (FUSED) {
        a = __fmaf_rn(xa.x, wa.x, a); a = __fmaf_rn(xa.y, wa.y, a);
        a = __fmaf_rn(xa.z, wa.z, a); a = __fmaf_rn(xa.w, wa.w, a);
        a = __fmaf_rn(xb.x, wb.x, a); a = __fmaf_rn(xb.y, wb.y, a);
        a = __fmaf_rn(xb.z, wb.z, a); a = __fmaf_rn(xb.w, wb.w, a);
    } else {
        a = __fadd_rn(a, __fmul_rn(xa.x, wa.x)); a = __fadd_rn(a, __fmul_rn(xa.y, wa.y));
        a = __fadd_rn(a, __fmul_rn(xa.z, wa.z)); a = __fadd_rn(a, __fmul_rn(xa.w, wa.w));
        a = __fadd_rn(a, __fmul_rn(xb.x, wb.x)); a = __fadd_rn(a, __fmul_rn(xb.y, wb.y));
        a = __fadd_rn(a, __fmul_rn(xb.z, wb.z)); a = __fadd_rn(a, __fmul_rn(xb.w, wb.w));
    }
    return a;
}

// The operands of one step of eight k: R weight rows and MTT token rows.
template <int R, int MTT>
struct SeqOps {
    float4 wa[R], wb[R], xa[MTT], xb[MTT];
    __device__ __forceinline__ void load(const unsigned char *wrow, const float4 *xrow, int k8) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const float4 *p = reinterpret_cast<const float4 *>(wrow + (size_t)r * 32 * SQ_WP) + 2 * k8;
            wa[r] = p[0]; wb[r] = p[1];
        }
#pragma unroll
        for (int j = 0; j < MTT; j++) {
            xa[j] = xrow[j * (SQ_KT / 4) + 2 * k8]; xb[j] = xrow[j * (SQ_KT / 4) + 2 * k8 + 1];
        }
    }
    template <bool FUSED>
    __device__ __forceinline__ void walk(float (&acc)[R][MTT]) const {
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int j = 0; j < MTT; j++) acc[r][j] = seq_walk8<FUSED>(acc[r][j], wa[r], wb[r], xa[j], xb[j]);
    }
};

// One K tile: the operands of the next step are read from shared memory while the
// current step's chain runs (two register sets, alternating), so the chains do not
// wait for the loads.
template <int R, int MTT, bool FUSED>
__device__ __forceinline__ void seq_walk_tile(float (&acc)[R][MTT], const unsigned char *wrow, const float4 *xrow) {
    SeqOps<R, MTT> A, B;
    A.load(wrow, xrow, 0);
#pragma unroll 1
    for (int k8 = 0; k8 < SQ_KT / 8; k8 += 2) {
        B.load(wrow, xrow, k8 + 1);
        A.template walk<FUSED>(acc);
        if (k8 + 2 < SQ_KT / 8) A.load(wrow, xrow, k8 + 2);
        B.template walk<FUSED>(acc);
    }
}

// 512 threads: warps 0..7 walk the chains (warp w < MG owns MTT tokens), warps 8..15
// stage.  While the chain warps walk tile t, the staging warps issue the copies of
// tile t + NST - 1, wait for tile t + 1 and make their pass over it (round the input,
// widen BF16 weights into the other half of the widened buffer, decide exactness), so
// the chain warps execute nothing but the walk; one __syncthreads per tile hands tile
// t + 1 over.  Every thread runs the same number of loop iterations and barriers.
constexpr int SQ_THREADS = 512, SQ_STAGERS = 256;

template <bool WBF16, int R, int MTT, int MG, int NST>
__global__ void __launch_bounds__(SQ_THREADS, 1)
f32_linear_seq_kernel(const void *__restrict__ wv, const float *__restrict__ x, float *__restrict__ out,
                      int M, int K, int O, int flags, long long w_stride, long long x_stride, int x_ld,
                      long long out_stride, int out_ld) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    using Cf = SeqCfg<WBF16, R, MTT, MG, NST>;
    constexpr int ROWS = Cf::ROWS, TPC = Cf::TPC, ESZ = Cf::ESZ, WP_RAW = Cf::WP_RAW, STAGE = Cf::STAGE;
    constexpr int W_CH = SQ_KT * ESZ / 16;               // 16-byte chunks per stored weight row of a tile
    constexpr int NWC = ROWS * W_CH / SQ_STAGERS;        // weight chunks per staging thread and tile
    constexpr int NXC = (TPC * (SQ_KT / 4) + SQ_STAGERS - 1) / SQ_STAGERS;
    static_assert(ROWS * W_CH % SQ_STAGERS == 0, "weight chunks must divide among the staging threads");
    extern __shared__ __align__(16) unsigned char sq_smem[];
    unsigned char *wide = sq_smem + (size_t)NST * STAGE; // [2][ROWS * SQ_WP] when WBF16
    int *s_bad = reinterpret_cast<int *>(sq_smem + (size_t)NST * STAGE + 2 * Cf::WIDE);   // [2]: tile parity
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool stager = tid >= SQ_THREADS - SQ_STAGERS;
    const int sid = tid - (SQ_THREADS - SQ_STAGERS);
    const int o0 = blockIdx.x * ROWS, m0 = blockIdx.y * TPC;
    const unsigned char *wbase = reinterpret_cast<const unsigned char *>(wv) + (size_t)blockIdx.z * w_stride * ESZ;
    x += blockIdx.z * x_stride;
    out += blockIdx.z * out_stride;
    const bool rin = flags & APUS_CUDA_R_IN;
    const int nt = (K + SQ_KT - 1) / SQ_KT;

    // a staging thread copies the same chunks of every tile: their sources are kept as
    // pointers that only advance by a tile per iteration
    const unsigned char *wsrc[NWC];
    const float *xsrc[NXC];
    unsigned row_ok = 0;                                  // bit j: weight chunk j, bit 16 + j: x chunk j
    if (stager) {
#pragma unroll
        for (int j = 0; j < NWC; j++) {
            const int id = sid + SQ_STAGERS * j, r = id / W_CH, c = id - r * W_CH;
            const bool ok = o0 + r < O;
            wsrc[j] = wbase + ((size_t)(ok ? o0 + r : 0) * K) * ESZ + c * 16;
            row_ok |= ok ? 1u << j : 0u;
        }
#pragma unroll
        for (int j = 0; j < NXC; j++) {
            const int id = sid + SQ_STAGERS * j, r = id / (SQ_KT / 4), c = id - r * (SQ_KT / 4);
            const bool ok = id < TPC * (SQ_KT / 4) && m0 + r < M;
            xsrc[j] = x + (size_t)(ok ? m0 + r : 0) * x_ld + c * 4;
            row_ok |= ok ? 1u << (16 + j) : 0u;
        }
    }
    auto issue = [&](int t) {                             // staging threads: tile t into stage t % NST
        unsigned char *st = sq_smem + (size_t)(t % NST) * STAGE;
        const int k0 = t * SQ_KT;
#pragma unroll
        for (int j = 0; j < NWC; j++) {
            const int id = sid + SQ_STAGERS * j, r = id / W_CH, c = id - r * W_CH;
            const bool ok = (row_ok >> j & 1u) && k0 + c * (16 / ESZ) < K;
            cp_async16(st + (size_t)r * WP_RAW + c * 16, ok ? wsrc[j] + (size_t)k0 * ESZ : wbase, ok);
        }
#pragma unroll
        for (int j = 0; j < NXC; j++) {
            const int id = sid + SQ_STAGERS * j, r = id / (SQ_KT / 4), c = id - r * (SQ_KT / 4);
            if (id < TPC * (SQ_KT / 4)) {
                const bool ok = (row_ok >> (16 + j) & 1u) && k0 + c * 4 < K;
                cp_async16(st + Cf::W_RAW + ((size_t)r * SQ_KT + c * 4) * 4, ok ? xsrc[j] + k0 : x, ok);
            }
        }
    };
    // staging threads: round the input of tile t (bf16_linear), widen its BF16 weights into
    // half t & 1 of the widened buffer, and note whether every product of the tile is exact
    auto pass = [&](int t) {
        unsigned char *st = sq_smem + (size_t)(t % NST) * STAGE;
        float4 *xs4 = reinterpret_cast<float4 *>(st + Cf::W_RAW);
        bool exact = true;
        if (!WBF16) {
            // f32 weight storage: these are the small, add-latency bound projections (router,
            // compressors); the chain is as long either way, so the tile is not examined and
            // takes the two-instruction walk -- the staging warps then only copy (and round)
            if (rin)
                for (int idx = sid; idx < TPC * (SQ_KT / 4); idx += SQ_STAGERS) {
                    float4 v = xs4[idx];
                    v.x = bf16_round(v.x); v.y = bf16_round(v.y); v.z = bf16_round(v.z); v.w = bf16_round(v.w);
                    xs4[idx] = v;
                }
            return;
        }
        for (int idx = sid; idx < TPC * (SQ_KT / 4); idx += SQ_STAGERS) {
            float4 v = xs4[idx];
            if (rin) {
                v.x = bf16_round(v.x); v.y = bf16_round(v.y); v.z = bf16_round(v.z); v.w = bf16_round(v.w);
                xs4[idx] = v;
            }
            exact &= fma_ok_f32(v.x) && fma_ok_f32(v.y) && fma_ok_f32(v.z) && fma_ok_f32(v.w);
        }
        if (WBF16) {
            unsigned char *wd = wide + (size_t)(t & 1) * Cf::WIDE;
            uint32_t bad = 0;
#pragma unroll
            for (int j = 0; j < NWC; j++) {
                const int id = sid + SQ_STAGERS * j, r = id / W_CH, c = id - r * W_CH;
                const uint4 raw = *reinterpret_cast<const uint4 *>(st + (size_t)r * WP_RAW + c * 16);
                bad |= fma_bad_bf16x2(raw.x) | fma_bad_bf16x2(raw.y) | fma_bad_bf16x2(raw.z) | fma_bad_bf16x2(raw.w);
                float4 *dst = reinterpret_cast<float4 *>(wd + (size_t)r * SQ_WP + c * 32);
                dst[0] = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                     __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                dst[1] = make_float4(__uint_as_float(raw.z << 16), __uint_as_float(raw.z & 0xffff0000u),
                                     __uint_as_float(raw.w << 16), __uint_as_float(raw.w & 0xffff0000u));
            }
            exact &= (bad & 0x80008000u) == 0u;
        }
        if (!exact) s_bad[t & 1] = 1;                     // every writer stores the same value
    };
    // the staging threads' own barrier (hardware barrier 1; barrier 0 is __syncthreads)
    auto stagers_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(SQ_STAGERS) : "memory"); };

    float acc[R][MTT];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int j = 0; j < MTT; j++) acc[r][j] = 0.f;
    if (tid < 2) s_bad[tid] = 0;
    __syncthreads();
    if (stager) {
#pragma unroll
        for (int t = 0; t < NST - 1; t++) {
            if (t < nt) issue(t);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        asm volatile("cp.async.wait_group %0;" ::"n"(NST - 2) : "memory");
        stagers_sync();                                   // tile 0 of every staging thread has landed
        pass(0);
    }
    __syncthreads();                                      // tile 0 is staged
    for (int t = 0; t < nt; t++) {
        if (stager) {
            // stage (t - 1) % NST was walked in the last iteration and is free again
            if (t + NST - 1 < nt) issue(t + NST - 1);
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (sid == 0) s_bad[(t + 1) & 1] = 0;         // read last at tile t - 1
            asm volatile("cp.async.wait_group %0;" ::"n"(NST - 2) : "memory");
            stagers_sync();                               // tile t + 1 of every staging thread has landed
            if (t + 1 < nt) pass(t + 1);
        } else if (warp < MG) {
            const unsigned char *stg = sq_smem + (size_t)(t % NST) * STAGE;
            const unsigned char *wrow = (WBF16 ? wide + (size_t)(t & 1) * Cf::WIDE : stg) + (size_t)lane * SQ_WP;
            const float4 *xrow = reinterpret_cast<const float4 *>(stg + Cf::W_RAW) + (size_t)warp * MTT * (SQ_KT / 4);
            if (!WBF16 || s_bad[t & 1]) seq_walk_tile<R, MTT, false>(acc, wrow, xrow);
            else seq_walk_tile<R, MTT, true>(acc, wrow, xrow);
        }
        __syncthreads();                                  // tile t + 1 is staged; tile t's buffers are free
    }
    if (!stager && warp < MG) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int o = o0 + lane + 32 * r;
#pragma unroll
            for (int j = 0; j < MTT; j++) {
                const int m = m0 + warp * MTT + j;
                if (o < O && m < M)
                    out[(size_t)m * out_ld + o] = (flags & APUS_CUDA_R_OUT) ? bf16_round(acc[r][j]) : acc[r][j];
            }
        }
    }
}

template <bool WBF16, int R, int MTT, int MG, int NST>
static cudaError_t seq_launch(cudaStream_t st, int batch, const void *w, const float *x, float *out, int M, int K,
                              int O, int flags, long long ws, long long xs, int x_ld, long long os, int out_ld) {
    using Cf = SeqCfg<WBF16, R, MTT, MG, NST>;
    auto kern = f32_linear_seq_kernel<WBF16, R, MTT, MG, NST>;
    if (ensure_dyn_smem((const void *)kern, Cf::SMEM)) return cudaErrorInvalidValue;
    const dim3 grid((unsigned)ceil_div(O, Cf::ROWS), (unsigned)ceil_div(M, Cf::TPC), (unsigned)batch);
    launch_k(kern, grid, SQ_THREADS, Cf::SMEM, st, w, x, out, M, K, O, flags, ws, xs, x_ld, os, out_ld);
    return cudaSuccess;
}

template <bool WBF16>
static int launch_linear_seq(const void *w, long long ws, const float *x, long long xs, int x_ld, float *out,
                             long long os, int out_ld, int batch, int M, int K, int O, int flags,
                             cudaStream_t st) {
#define SEQ_LAUNCH(R, MTT, MG, NST)                                                                          \
    APUS_CUDA_OK((seq_launch<WBF16, R, MTT, MG, NST>(st, batch, w, x, out, M, K, O, flags, ws, xs, x_ld, os, out_ld)))
    // Tokens per CTA: as many as keep enough CTAs in flight, at most 32.  Few tokens per
    // CTA leave shared memory for a deep ring, which a CTA that is alone on its SM (small
    // O) needs to cover the memory latency; the 64-row tile (R = 2) halves the staging and
    // the x reads per term once there are CTAs enough to fill the GPU with it.
    const long long ctas32 = (long long)ceil_div(O, 32) * batch * ceil_div(M, 32);
    // Every chain warp reads the whole weight tile from shared memory, so two tokens per
    // warp (half as many warps re-reading it) keep the small shapes off the shared-memory
    // pipe: with one token per warp the 8-token CTA spent 3/4 of a tile's time on it.
    if (M == 1) SEQ_LAUNCH(1, 1, 1, 6);
    else if (M <= 2) SEQ_LAUNCH(1, 2, 1, 6);
    else if (M <= 4) SEQ_LAUNCH(1, 2, 2, 6);
    // few output rows (router gate, indexer head weights): the launch is a handful of CTAs, each a chain of K
    // adds per accumulator; one token per warp halves the walk of a warp and doubles the CTAs
    else if (M > 8 && ctas32 < 32) SEQ_LAUNCH(1, 1, 4, 6);      // 4 tokens per CTA, one per warp
    else if (M <= 8 || ctas32 < 64) SEQ_LAUNCH(1, 2, 4, 6);     // 8 tokens per CTA, two per warp
    else if (M <= 16 || ctas32 < 148) SEQ_LAUNCH(1, 2, 8, 3);   // 16 tokens per CTA
    else if constexpr (WBF16) SEQ_LAUNCH(2, 4, 8, 3);           // 32 tokens x 64 rows per CTA
    else SEQ_LAUNCH(1, 4, 8, 3);                                // 32 tokens per CTA
#undef SEQ_LAUNCH
    return 0;
}

template <bool WBF16>
static void launch_linear(const void *w, long long ws, const float *x, long long xs, int x_ld, float *out,
                          long long os, int out_ld, int batch, int M, int K, int O, int flags,
                          cudaStream_t st) {
    if (M == 1) {
        dim3 grid((unsigned)ceil_div(O, 8), 1, (unsigned)batch);
        launch_k(f32_linear_kernel<WBF16, 8, 1>, grid, 256, 0, st, w, x, out, M, K, O, flags, ws, xs, x_ld, os, out_ld);
    } else if (M <= 4) {
        dim3 grid((unsigned)ceil_div(O, 4), 1, (unsigned)batch);
        launch_k(f32_linear_kernel<WBF16, 4, 4>, grid, 256, 0, st, w, x, out, M, K, O, flags, ws, xs, x_ld, os, out_ld);
    } else {
        dim3 grid((unsigned)ceil_div(O, 4), (unsigned)ceil_div(M, 8), (unsigned)batch);
        launch_k(f32_linear_kernel<WBF16, 4, 8>, grid, 256, 0, st, w, x, out, M, K, O, flags, ws, xs, x_ld, os, out_ld);
    }
}

// BF16 weights [batch*O, K] on the tcgen05 kernel (gemm_tcbf.cu): the activations [M, x_ld] are
// copied as BF16 (exact for BF16-valued rows; APUS_CUDA_R_IN asks for that rounding anyway) into
// the stream's scratch, which also holds the K-split partial sums.
static int linear_tcbf(const void *w, const float *x, int x_koff, int x_ld, float *out, int out_ld, int batch, int M,
                       int K, int O, int flags, cudaStream_t st, LinCodes *codes) {
    const int S = tcbf_ksplit(O, K, batch, M);
    const size_t xb = (((size_t)M * x_ld * 2) + 255) & ~(size_t)255;
    const size_t pb = S > 1 ? (size_t)S * M * batch * O * 4 : 0;
    const size_t n_cnt = (size_t)(O / 128) * batch * ((M + 31) / 32);
    void *ws = nullptr;
    int *cnt = nullptr;
    if (stream_scratch(st, xb + pb, &ws, n_cnt, &cnt)) return 1;
    uint16_t *xh = (uint16_t *)ws;
    if (f32_to_bf16(x, xh, (long long)M * x_ld, st)) return 1;
    alignas(64) unsigned char map_w[128], map_x[128];
    if (tcbf_make_weight_map(map_w, w, (long long)batch * O, K) || tcbf_make_act_map(map_x, xh, M, x_ld)) return 1;
    TcbfArgs a = {};
    a.map_w = map_w; a.map_x = map_x;
    a.M = M; a.O = O; a.K = K; a.batch = batch; a.x_koff = x_koff;
    a.out_ld = out_ld; a.round_out = (flags & APUS_CUDA_R_OUT) ? 1 : 0; a.out = out;
    a.ksplit = S; a.part = (float *)((char *)ws + xb); a.counters = cnt;
    if (codes && S > 1 && out_ld % 128 == 0 && out_ld == batch * O) { a.q_out = codes->q; a.qs_out = codes->s; codes->written = 1; }
    return gemm_tcbf(a, st);
}

int f32_linear_batched(const void *w, long long w_stride, const float *x, long long x_stride, int x_ld,
                       float *out, long long out_stride, int out_ld, int batch, int M, int K, int O,
                       int flags, cudaStream_t st, LinCodes *codes) {
    if (codes) codes->written = 0;
    APUS_REQUIRE(K % 4 == 0 && x_ld % 4 == 0 && x_stride % 4 == 0 && w_stride % 4 == 0,
                 "f32_linear: K=%d and the strides must be multiples of 4", K);
    if (M <= 0 || O <= 0 || batch <= 0) return 0;
    const int op = (flags >> 8) & 0xff;
    flags &= 0xff;
    const bool tree = sum_tree(op ? op : APUS_CUDA_TREE_LINEAR);
    // BF16 weights in tree order: the tensor-core kernel, when the problems are laid out as it reads them
    if (tree && (flags & APUS_CUDA_W_BF16) && O % 128 == 0 && K % 64 == 0 && x_ld % 8 == 0 && ((uintptr_t)w & 15) == 0 &&
        (batch == 1 || (w_stride == (long long)O * K && out_stride == O)) && x_stride * (long long)(batch - 1) + K <= x_ld)
        return linear_tcbf(w, x, (int)x_stride, x_ld, out, out_ld, batch, M, K, O, flags, st, codes);
    if (!tree) {
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
