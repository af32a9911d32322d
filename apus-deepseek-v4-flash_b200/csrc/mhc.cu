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
#include <cooperative_groups.h>
#include <map>
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
    APUS_PDL_WAIT();
    APUS_PDL_GO();
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
// by add latency (about 35 us at 4 x 4096), not bandwidth: 256 producer threads
// stage rounded products of a tile in shared memory while one lane per dot (the
// consumer warp) walks the previous tile.  One CTA per (token, group of
// MIX_CPG chains): the chains of a token are independent, so spreading them
// over CTAs divides the producers' load without lengthening any chain.
// Chain c < nmix is fn_c . x, chain nmix is sum x^2.
#define MIX_CPG 4
// TOK tokens share one CTA (and one read of the fn tile): consumer lane
// l = token * MIX_CPG + chain, TOK * MIX_CPG <= 32.
template <int TOK>
__global__ void __launch_bounds__(288)
mhc_mix_seq_kernel(const float *__restrict__ x4, const float *__restrict__ fn, int nx, int nmix,
                   int MIX_TI, int rows, float *__restrict__ raw) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ __align__(16) float s_prod[];
    const int C = nmix + 1, stride = MIX_TI + 4, tid = threadIdx.x;
    const int row0 = blockIdx.x * TOK, c_lo = blockIdx.y * MIX_CPG, Cl = min(MIX_CPG, C - c_lo);
    const int ntok = min(TOK, rows - row0);
    const int nt = (nx + MIX_TI - 1) / MIX_TI;
    const bool consumer = tid >= 256;
    float acc = 0.f;
    const int cl = tid - 256;                 // consumer lane
    const int my_tok = cl / MIX_CPG, my_c = cl - my_tok * MIX_CPG;
    const bool live = consumer && my_tok < ntok && my_c < Cl;
    // Producer thread p owns the 16-byte word p of every tile when a tile has at
    // most 256 words per chain group (TOK > 1: MIX_TI = 256), and keeps the fn
    // word of the NEXT tile it will multiply in a register, loaded one whole
    // iteration ahead; with a single token per CTA (large tiles) it loops.
    const int q = MIX_TI / 4, total = Cl * q;
    const bool one_word = TOK > 1;
    const int pc = tid / q, pi4 = tid - pc * q;          // one_word: this thread's (chain, word)
    const bool p_on = one_word && !consumer && tid < total;
    const bool p_sq = c_lo + pc >= nmix;
    float4 f_next = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 x_next[TOK];
#pragma unroll
    for (int tk = 0; tk < TOK; tk++) x_next[tk] = make_float4(0.f, 0.f, 0.f, 0.f);
    // the words of tile t: fn (one per thread) and the tokens' x, issued a whole
    // iteration before they are multiplied
    auto fetch_fn = [&](int t) {
        const int gi = t * MIX_TI + 4 * pi4;
        f_next = make_float4(0.f, 0.f, 0.f, 0.f);
        const bool in = p_on && t < nt && gi < nx;
        if (in && !p_sq) f_next = __ldg(reinterpret_cast<const float4 *>(fn + (size_t)(c_lo + pc) * nx + gi));
#pragma unroll
        for (int tk = 0; tk < TOK; tk++) {
            x_next[tk] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (in && tk < ntok) x_next[tk] = *reinterpret_cast<const float4 *>(x4 + (size_t)(row0 + tk) * nx + gi);
        }
    };
    auto produce = [&](int t) {
        float *dst = s_prod + (size_t)(t & 1) * (TOK * MIX_CPG) * stride;
        if (one_word) {
            const float4 fcur = f_next;
            float4 xv[TOK];
#pragma unroll
            for (int tk = 0; tk < TOK; tk++) xv[tk] = x_next[tk];
            fetch_fn(t + 1);                              // lands while tile t is multiplied and t - 1 consumed
            if (!p_on) return;
#pragma unroll
            for (int tk = 0; tk < TOK; tk++) {
                const float4 f = p_sq ? xv[tk] : fcur;
                *reinterpret_cast<float4 *>(dst + (size_t)(tk * MIX_CPG + pc) * stride + 4 * pi4) =
                    make_float4(__fmul_rn(f.x, xv[tk].x), __fmul_rn(f.y, xv[tk].y), __fmul_rn(f.z, xv[tk].z),
                                __fmul_rn(f.w, xv[tk].w));
            }
            return;
        }
        // eight 16-byte loads of fn (and the matching x words) in flight per thread
        const float *x = x4 + (size_t)row0 * nx;
        for (int base = tid; base < total; base += 256 * 8) {
            float4 fv[8], xv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int idx = base + u * 256;
                const int c = idx / q, i4 = idx - c * q, gi = t * MIX_TI + 4 * i4;
                const bool ok = idx < total && gi < nx;
                xv[u] = ok ? *reinterpret_cast<const float4 *>(x + gi) : make_float4(0.f, 0.f, 0.f, 0.f);
                fv[u] = (ok && c_lo + c < nmix) ? __ldg(reinterpret_cast<const float4 *>(fn + (size_t)(c_lo + c) * nx + gi))
                                                : xv[u];
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int idx = base + u * 256;
                if (idx >= total) continue;
                const int c = idx / q, i4 = idx - c * q;
                *reinterpret_cast<float4 *>(dst + (size_t)c * stride + 4 * i4) =
                    make_float4(__fmul_rn(fv[u].x, xv[u].x), __fmul_rn(fv[u].y, xv[u].y),
                                __fmul_rn(fv[u].z, xv[u].z), __fmul_rn(fv[u].w, xv[u].w));
            }
        }
    };
    if (one_word) fetch_fn(0);
    if (!consumer) produce(0);
    __syncthreads();
    for (int t = 0; t < nt; t++) {
        if (!consumer) {
            if (t + 1 < nt) produce(t + 1);
        } else if (live) {
            acc = seq_sum_smem(s_prod + (size_t)(t & 1) * (TOK * MIX_CPG) * stride + (size_t)cl * stride, MIX_TI, acc);
        }
        __syncthreads();
    }
    if (live) raw[(size_t)(row0 + my_tok) * C + c_lo + my_c] = acc;
}

__device__ __forceinline__ float sigm(float x) { return __fdiv_rn(1.0f, 1.0f + exp_rn(-x)); }

// Sinkhorn on an n x n matrix held by one thread (reference c/mhc.h:181-218).
// N > 0 fixes the size at compile time so that the matrix stays in registers
// and the loops unroll (N = 4 is the model's hc_mult); N = 0 is the generic
// form on a local array.
template <int N>
__device__ __forceinline__ void sinkhorn(float *c, int n_rt, int iters, float eps) {
    const int n = N ? N : n_rt;
#pragma unroll
    for (int j = 0; j < n; j++) {
        float *r = c + j * n, mx = r[0], sum = 0.f;
#pragma unroll
        for (int k = 1; k < n; k++) mx = fmaxf(mx, r[k]);
#pragma unroll
        for (int k = 0; k < n; k++) { r[k] = exp_rn(r[k] - mx); sum = __fadd_rn(sum, r[k]); }
#pragma unroll
        for (int k = 0; k < n; k++) r[k] = __fadd_rn(__fdiv_rn(r[k], sum), eps);
    }
    for (int it = 0; it < iters; it++) {
        if (it) {
#pragma unroll
            for (int j = 0; j < n; j++) {
                float sum = 0.f;
#pragma unroll
                for (int k = 0; k < n; k++) sum = __fadd_rn(sum, c[j * n + k]);
                float den = __fadd_rn(sum, eps);
#pragma unroll
                for (int k = 0; k < n; k++) c[j * n + k] = __fdiv_rn(c[j * n + k], den);
            }
        }
#pragma unroll
        for (int k = 0; k < n; k++) {
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < n; j++) sum = __fadd_rn(sum, c[j * n + k]);
            float den = __fadd_rn(sum, eps);
#pragma unroll
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
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ __align__(16) float s_sq[];   // seq: d squares of the collapsed row
    __shared__ float s_pre[MHC_MAX_N];
    __shared__ float red[32];
    const int row = blockIdx.x;
    const float *rw = raw + (size_t)row * (nmix + 1);
    const float mean = __fdiv_rn(rw[nmix], (float)(n * d));
    const float r = __fdiv_rn(1.0f, sqrtf(__fadd_rn(mean, norm_eps)));
    // the gates that the collapse needs first (thread 0); post / comb / Sinkhorn,
    // which nothing in this kernel waits for, run on another warp's lane while
    // thread 0 walks the sum of squares
    if (threadIdx.x == 0) {
        for (int j = 0; j < n; j++) {
            float m = __fmul_rn(rw[j], r);
            float sc = head_mode ? head_scale : scale[0];
            s_pre[j] = __fadd_rn(sigm(__fadd_rn(__fmul_rn(m, sc), base[j])), hc_eps);
            if (pre_out) pre_out[(size_t)row * n + j] = s_pre[j];
        }
    }
    __syncthreads();
    const float *x = x4 + (size_t)row * n * d;
    float ss = 0.f;
    if (y) {
        // collapse: y[i] = sum_j pre[j] * X[j,i], j ascending, mul then add; BF16 round
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float acc = 0.f;
            for (int j = 0; j < n; j++) acc = __fadd_rn(acc, __fmul_rn(s_pre[j], x[(size_t)j * d + i]));
            acc = bf16_round(acc);
            y[(size_t)row * d + i] = acc;
            if (seq) s_sq[i] = __fmul_rn(acc, acc);
            else ss = fmaf(acc, acc, ss);
        }
    }
    __syncthreads();
    if ((threadIdx.x >> 5) == 1 && !head_mode && n * n <= 32) {
        // warp 1: lane l < n holds post[l]; lane l < n*n holds comb[l / n][l % n].  Every
        // lane gathers the n values of its row (column) with shuffles and adds them in
        // index order, so each sum is the reference's, computed n*n times in parallel.
        const int l = threadIdx.x & 31;
        if (l < n) {
            float m2 = __fmul_rn(rw[n + l], r);
            float po = __fmul_rn(2.0f, sigm(__fadd_rn(__fmul_rn(m2, scale[1]), base[n + l])));
            if (post_out) post_out[(size_t)row * n + l] = po;
        }
        const bool on = l < n * n;
        const int j = on ? l / n : 0, k = on ? l - j * n : 0;
        float c = on ? __fadd_rn(__fmul_rn(__fmul_rn(rw[2 * n + l], r), scale[2]), base[2 * n + l]) : 0.f;
        // row softmax with eps added per element (reference c/mhc.h:181-190)
        float mx = __shfl_sync(0xffffffffu, c, j * n);
        for (int q = 1; q < n; q++) mx = fmaxf(mx, __shfl_sync(0xffffffffu, c, j * n + q));
        c = exp_rn(c - mx);
        float sum = 0.f;
        for (int q = 0; q < n; q++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, c, j * n + q));
        c = __fadd_rn(__fdiv_rn(c, sum), hc_eps);
        for (int it = 0; it < iters; it++) {
            if (it) {
                float s2 = 0.f;
                for (int q = 0; q < n; q++) s2 = __fadd_rn(s2, __shfl_sync(0xffffffffu, c, j * n + q));
                c = __fdiv_rn(c, __fadd_rn(s2, hc_eps));
            }
            float s3 = 0.f;
            for (int q = 0; q < n; q++) s3 = __fadd_rn(s3, __shfl_sync(0xffffffffu, c, q * n + k));
            c = __fdiv_rn(c, __fadd_rn(s3, hc_eps));
        }
        if (on && comb_out) comb_out[(size_t)row * n * n + l] = c;
    } else if (threadIdx.x == 32 && !head_mode) {
        for (int j = 0; j < n; j++) {
            float m2 = __fmul_rn(rw[n + j], r);
            float po = __fmul_rn(2.0f, sigm(__fadd_rn(__fmul_rn(m2, scale[1]), base[n + j])));
            if (post_out) post_out[(size_t)row * n + j] = po;
        }
        {
            float comb[MHC_MAX_N * MHC_MAX_N];
            for (int i = 0; i < n * n; i++)
                comb[i] = __fadd_rn(__fmul_rn(__fmul_rn(rw[2 * n + i], r), scale[2]), base[2 * n + i]);
            sinkhorn<0>(comb, n, iters, hc_eps);
            if (comb_out)
                for (int i = 0; i < n * n; i++) comb_out[(size_t)row * n * n + i] = comb[i];
        }
    }
    if (!y || !y_normed) return;
    float tot;
    if (seq) {                                // reference order: one accumulator, index ascending
        if (threadIdx.x == 0) red[0] = seq_sum_smem(s_sq, d, 0.f);
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

// post gates and the Sinkhorn-normalised comb matrix of one token (reference c/mhc.h:181-234), one warp.
__device__ __forceinline__ void mhc_gates_warp(const float *__restrict__ rw, float r, int n, const float *__restrict__ scale,
                                               const float *__restrict__ base, float hc_eps, int iters, size_t row,
                                               float *__restrict__ post_out, float *__restrict__ comb_out, int tid) {
    const int l = tid & 31;
    if (l < n) {
        const float m2 = __fmul_rn(rw[n + l], r);
        const float po = __fmul_rn(2.0f, sigm(__fadd_rn(__fmul_rn(m2, scale[1]), base[n + l])));
        if (post_out) post_out[(size_t)row * n + l] = po;
    }
    const bool on = l < n * n;
    const int j = on ? l / n : 0, k = on ? l - j * n : 0;
    float c = on ? __fadd_rn(__fmul_rn(__fmul_rn(rw[2 * n + l], r), scale[2]), base[2 * n + l]) : 0.f;
    float mx = __shfl_sync(0xffffffffu, c, j * n);
    for (int q = 1; q < n; q++) mx = fmaxf(mx, __shfl_sync(0xffffffffu, c, j * n + q));
    c = exp_rn(c - mx);
    float sum = 0.f;
    for (int q = 0; q < n; q++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, c, j * n + q));
    c = __fadd_rn(__fdiv_rn(c, sum), hc_eps);
    for (int it = 0; it < iters; it++) {
        if (it) {
            float s2 = 0.f;
            for (int q = 0; q < n; q++) s2 = __fadd_rn(s2, __shfl_sync(0xffffffffu, c, j * n + q));
            c = __fdiv_rn(c, __fadd_rn(s2, hc_eps));
        }
        float s3 = 0.f;
        for (int q = 0; q < n; q++) s3 = __fadd_rn(s3, __shfl_sync(0xffffffffu, c, q * n + k));
        c = __fdiv_rn(c, __fadd_rn(s3, hc_eps));
    }
    if (on && comb_out) comb_out[(size_t)row * n * n + l] = c;
}

// The same step with a token spread over a cluster of MHC_CL CTAs: one CTA walking a
// 4 x 4096 state alone takes ~30 us, most of it latency (gates -> 64 KB of loads through one
// SM -> sum of squares -> second pass), and at small batches that chain sits twice in every
// layer.  Here every CTA of the cluster collapses its slice of the row and each CTA normalises
// its own slice; the Sinkhorn part, which nothing in this kernel waits for, runs on one warp
// of the last CTA while rank 0 walks the sum of squares (after the row is out when the sum is a tree).  The sum of squares of the norm meets through distributed shared
// memory: in tree order the slices' sums are added in rank order (the same total in every
// CTA); in the reference's order (seq) every CTA stores its squares into rank 0's shared
// memory and one lane there adds all d of them in index order -- the reference's chain, about
// 8 us at d = 4096, without the rest of the kernel queued behind one SM.
#define MHC_CL 8
__global__ void __cluster_dims__(MHC_CL, 1, 1) __launch_bounds__(128)
mhc_pre_finish_cl_kernel(const float *__restrict__ x4, const float *__restrict__ raw, int d, int n,
                         int nmix, const float *__restrict__ scale, float head_scale,
                         const float *__restrict__ base, float norm_eps, float hc_eps, int iters,
                         int head_mode, const float *__restrict__ norm_w, float rms_eps,
                         float *__restrict__ pre_out, float *__restrict__ post_out,
                         float *__restrict__ comb_out, float *__restrict__ y,
                         float *__restrict__ y_normed, int seq, uint8_t *__restrict__ xq, float *__restrict__ xs) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ __align__(16) float s_sq[];   // seq: the d squares of the collapsed row (rank 0's copy is used)
    __shared__ float s_pre[MHC_MAX_N];
    __shared__ float red[32];
    __shared__ float s_part;
    const int row = blockIdx.x / MHC_CL, rank = (int)cluster.block_rank();
    const int tid = threadIdx.x;
    const float *rw = raw + (size_t)row * (nmix + 1);
    const float mean = __fdiv_rn(rw[nmix], (float)(n * d));
    const float r = __fdiv_rn(1.0f, sqrtf(__fadd_rn(mean, norm_eps)));
    if (tid < n) {
        const float m = __fmul_rn(rw[tid], r);
        const float sc = head_mode ? head_scale : scale[0];
        s_pre[tid] = __fadd_rn(sigm(__fadd_rn(__fmul_rn(m, sc), base[tid])), hc_eps);
        if (pre_out && rank == 0) pre_out[(size_t)row * n + tid] = s_pre[tid];
    }
    __syncthreads();
    // this CTA's slice of the row: [i0, i1), a multiple of 4 wide
    const int per = ((d + MHC_CL * 4 - 1) / (MHC_CL * 4)) * 4;
    const int i0 = min(d, rank * per), i1 = min(d, i0 + per);
    const float *x = x4 + (size_t)row * n * d;
    float ss = 0.f;
    // Shared memory of another CTA of the cluster may only be touched once that CTA runs: the CTAs of a
    // cluster are placed together but need not have started together, and a store into rank 0's window
    // before rank 0 has started is a fault (seen as sporadic "unspecified launch failure" once the grid
    // held thousands of clusters).  The loop below stores into rank 0, so the cluster meets first.
    if (y && y_normed && seq) cluster.sync();
    if (y) {
        for (int i = i0 + tid * 4; i < i1; i += blockDim.x * 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < n; j++) {
                const float4 v = *reinterpret_cast<const float4 *>(x + (size_t)j * d + i);
                const float p = s_pre[j];
                acc.x = __fadd_rn(acc.x, __fmul_rn(p, v.x)); acc.y = __fadd_rn(acc.y, __fmul_rn(p, v.y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(p, v.z)); acc.w = __fadd_rn(acc.w, __fmul_rn(p, v.w));
            }
            acc.x = bf16_round(acc.x); acc.y = bf16_round(acc.y); acc.z = bf16_round(acc.z); acc.w = bf16_round(acc.w);
            *reinterpret_cast<float4 *>(y + (size_t)row * d + i) = acc;
            if (seq && y_normed) {
                float *sq0 = cluster.map_shared_rank(s_sq, 0);
                *reinterpret_cast<float4 *>(sq0 + i) = make_float4(__fmul_rn(acc.x, acc.x), __fmul_rn(acc.y, acc.y),
                                                                   __fmul_rn(acc.z, acc.z), __fmul_rn(acc.w, acc.w));
            } else {
                ss = fmaf(acc.x, acc.x, ss); ss = fmaf(acc.y, acc.y, ss); ss = fmaf(acc.z, acc.z, ss); ss = fmaf(acc.w, acc.w, ss);
            }
        }
    }
    // The gates are needed only by the post step, far downstream: one warp of the last rank works them
    // out (a few microseconds of dependent shuffles and divisions) while rank 0 walks the sum of
    // squares, instead of after the normalised row is out, where the next kernel would wait for them.
    const bool gates_warp = !head_mode && rank == MHC_CL - 1 && (tid >> 5) == 1;
    bool gates_done = false;
    if (y && y_normed) {
        float tot = 0.f;
        if (seq) {
            cluster.sync();                        // every slice's squares have landed in rank 0
            if (rank == 0 && tid == 0) s_part = seq_sum_smem(s_sq, d, 0.f);
            if (gates_warp) { mhc_gates_warp(rw, r, n, scale, base, hc_eps, iters, (size_t)row, post_out, comb_out, tid); gates_done = true; }
            cluster.sync();
            tot = *cluster.map_shared_rank(&s_part, 0);
        } else {
            const float mine = block_sum(ss, red);
            if (tid == 0) s_part = mine;
            cluster.sync();
            for (int q = 0; q < MHC_CL; q++) tot = __fadd_rn(tot, *cluster.map_shared_rank(&s_part, q));
        }
        cluster.sync();                            // nobody leaves while its shared memory may still be read
        const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(tot, (float)d), rms_eps)));
        for (int i = i0 + tid * 4; i < i1; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4 *>(y + (size_t)row * d + i);
            const float4 w = __ldg(reinterpret_cast<const float4 *>(norm_w + i));
            float4 o;
            o.x = bf16_round(__fmul_rn(w.x, __fmul_rn(v.x, inv))); o.y = bf16_round(__fmul_rn(w.y, __fmul_rn(v.y, inv)));
            o.z = bf16_round(__fmul_rn(w.z, __fmul_rn(v.z, inv))); o.w = bf16_round(__fmul_rn(w.w, __fmul_rn(v.w, inv)));
            *reinterpret_cast<float4 *>(y_normed + (size_t)row * d + i) = o;
            if (xq) {
                // activation codes of the normalised row (the arithmetic of act_quant_kernel): the launcher
                // passes xq only when every slice is a whole number of 128-groups, so a group is one warp
                float amax = fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w)));
                amax = fmaxf(warp_max(amax), 1e-4f);
                const float s = ceil_pow2(__fmul_rn(amax, 1.0f / 448.0f));
                const float iv = __uint_as_float(0x7f000000u - __float_as_uint(s));
                const uint32_t lo = e4m3x2_from_f32(o.x * iv, o.y * iv), hi = e4m3x2_from_f32(o.z * iv, o.w * iv);
                *reinterpret_cast<uint32_t *>(xq + (size_t)row * d + i) = lo | (hi << 16);
                if ((tid & 31) == 0) xs[(size_t)row * (d >> 7) + (i >> 7)] = s;
            }
        }
    }
    if (!gates_done && gates_warp)
        mhc_gates_warp(rw, r, n, scale, base, hc_eps, iters, (size_t)row, post_out, comb_out, tid);
}

// Y[j,i] = bf16(post[j]*f[i] + sum_k comb[k,j]*R[k,i]) (reference c/mhc.h:259-270,
// c/layer.h:445-456).
__global__ void mhc_post_kernel(const float *__restrict__ f, const float *__restrict__ res,
                                const float *__restrict__ post, const float *__restrict__ comb,
                                float *__restrict__ y4, int d, int n) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
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

// Scratch between the two kernels of a call: the caller's (a model object keeps its
// own, so that models stepping side by side on different streams do not share one),
// else one buffer of the library, which only grows.
static float *g_raw = nullptr;
static size_t g_raw_cap = 0;
static float *ensure_raw(size_t floats, float *callers) {
    if (callers) return callers;
    if (floats <= g_raw_cap) return g_raw;
    if (g_raw) { cudaDeviceSynchronize(); cudaFree(g_raw); }
    g_raw = nullptr; g_raw_cap = 0;
    if (cudaMalloc(&g_raw, floats * sizeof(float)) != cudaSuccess) {
        set_error("mhc: scratch of %zu floats", floats);
        g_raw = nullptr;
        return nullptr;
    }
    g_raw_cap = floats;
    return g_raw;
}

// raw[row, 0..nmix] for `rows` tokens in the sum order now in force.
static int launch_mix(const float *x4, const float *fn, int nx, int nmix, float *raw, int rows,
                      cudaStream_t st) {
    if (sum_tree(APUS_CUDA_TREE_MHC_MAPS)) {
        launch_k(mhc_mix_kernel, dim3(nmix + 1, rows), 256, 0, st, x4, fn, nx, nmix, raw);
        APUS_LAUNCHED();
        return 0;
    }
    const int C = nmix + 1;
    if (ensure_dyn_smem((const void *)mhc_mix_seq_kernel<1>, 100 * 1024) ||
        ensure_dyn_smem((const void *)mhc_mix_seq_kernel<2>, 100 * 1024) ||
        ensure_dyn_smem((const void *)mhc_pre_finish_kernel, 128 * 1024))
        return 1;
    const unsigned gy = (unsigned)((C + MIX_CPG - 1) / MIX_CPG);
    if (rows >= 2) {
        // two tokens share a CTA and its read of fn (measured at batch 32: 2 tokens per CTA
        // beat 1, 4 and 8 by a few percent -- more tokens per CTA load the shared-memory
        // pipe with products and slow every chain down)
        const int tok = 2, ti = 256;
        const size_t smem = (size_t)2 * tok * MIX_CPG * (ti + 4) * sizeof(float);
        const dim3 grid((unsigned)((rows + tok - 1) / tok), gy);
        launch_k(mhc_mix_seq_kernel<2>, grid, 288, smem, st, x4, fn, nx, nmix, ti, rows, raw);
    } else {
        const int ti = 1024;
        const size_t smem = (size_t)2 * MIX_CPG * (ti + 4) * sizeof(float);
        launch_k(mhc_mix_seq_kernel<1>, dim3((unsigned)rows, gy), 288, smem, st, x4, fn, nx, nmix, ti, rows, raw);
    }
    APUS_LAUNCHED();
    return 0;
}
static inline int finish_seq() { return sum_tree(APUS_CUDA_TREE_NORMS) ? 0 : 1; }
static inline size_t finish_smem(int d) { return finish_seq() ? (size_t)d * sizeof(float) : 0; }

// pre/post/comb + collapse (+ RMSNorm) of `rows` tokens from the raw dots: the cluster kernel in
// tree order (when the shapes fit its layout), else one CTA per token.
static int launch_finish(const float *x4, const float *raw, int d, int n, int nmix, const float *scale,
                         float head_scale, const float *base, float norm_eps, float hc_eps, int iters, int head_mode,
                         const float *norm_w, float rms_eps, float *pre, float *post, float *comb, float *y,
                         float *y_normed, int rows, cudaStream_t st, uint8_t *xq = nullptr, float *xs = nullptr,
                         int *codes_written = nullptr) {
    if (codes_written) *codes_written = 0;
    if (d % 4 == 0 && n * n <= 32 && y && (size_t)d * sizeof(float) <= 48 * 1024) {
        // codes beside the normalised row when a CTA's slice (d / MHC_CL) is a whole number of 128-groups
        const bool codes = xq && xs && y_normed && d % (MHC_CL * 128) == 0;
        launch_k(mhc_pre_finish_cl_kernel, rows * MHC_CL, 128, finish_smem(d), st, x4, raw, d, n, nmix, scale, head_scale, base,
                 norm_eps, hc_eps, iters, head_mode, norm_w, rms_eps, pre, post, comb, y, y_normed, finish_seq(),
                 codes ? xq : (uint8_t *)nullptr, codes ? xs : (float *)nullptr);
        if (codes && codes_written) *codes_written = 1;
    } else {
        launch_k(mhc_pre_finish_kernel, rows, 256, finish_smem(d), st, x4, raw, d, n, nmix, scale, head_scale, base, norm_eps,
                                                                 hc_eps, iters, head_mode, norm_w, rms_eps, pre, post,
                                                                 comb, y, y_normed, finish_seq());
    }
    APUS_LAUNCHED();
    return 0;
}

int mhc_pre(const float *x4, int d, int n, const float *fn, const float *scale,
            const float *base, float norm_eps, float hc_eps, int iters,
            const float *norm_w, float rms_eps, float *pre, float *post,
            float *comb, float *y, float *y_normed, int rows, cudaStream_t st, float *raw_in, uint8_t *xq, float *xs,
            int *codes_written) {
    if (codes_written) *codes_written = 0;
    APUS_REQUIRE(n >= 1 && n <= MHC_MAX_N && (n * d) % 4 == 0, "mhc: n=%d d=%d unsupported", n, d);
    if (rows <= 0) return 0;
    int nmix = (2 + n) * n;
    float *raw = ensure_raw((size_t)rows * (nmix + 1), raw_in);
    if (!raw) return 1;
    if (launch_mix(x4, fn, n * d, nmix, raw, rows, st)) return 1;
    return launch_finish(x4, raw, d, n, nmix, scale, 0.f, base, norm_eps, hc_eps, iters, 0, norm_w, rms_eps, pre, post,
                         comb, y, norm_w ? y_normed : nullptr, rows, st, xq, xs, codes_written);
}

int mhc_head(const float *x4, int d, int n, const float *fn, float scale,
             const float *base, float norm_eps, float hc_eps, float *y,
             int rows, cudaStream_t st, float *raw_in) {
    APUS_REQUIRE(n >= 1 && n <= MHC_MAX_N && (n * d) % 4 == 0, "mhc: n=%d d=%d unsupported", n, d);
    if (rows <= 0) return 0;
    float *raw = ensure_raw((size_t)rows * (n + 1), raw_in);
    if (!raw) return 1;
    if (launch_mix(x4, fn, n * d, n, raw, rows, st)) return 1;
    return launch_finish(x4, raw, d, n, n, nullptr, scale, base, norm_eps, hc_eps, 0, 1, nullptr, 0.f, nullptr, nullptr,
                         nullptr, y, nullptr, rows, st);
}

int mhc_post(const float *f, const float *res4, const float *post,
             const float *comb, float *y4, int d, int n, int rows,
             cudaStream_t st) {
    APUS_REQUIRE(n >= 1 && n <= MHC_MAX_N, "mhc: n=%d unsupported", n);
    if (rows <= 0) return 0;
    launch_k(mhc_post_kernel, dim3(ceil_div(d, 256), rows), 256, 0, st, f, res4, post, comb, y4, d, n);
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
// library carries the array (MHC_NOALLOC_MAX_ROWS * (MHC_MAX_N * (MHC_MAX_N + 2) + 1) = 256 * 81 floats = 82,944 bytes)
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
    return launch_finish(x4, raw, d, n, nmix, scale, 0.f, base, norm_eps, hc_eps, iters, 0, norm_w, rms_eps, nullptr,
                         post, comb, y, norm_w ? y_normed : nullptr, rows, st);
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
