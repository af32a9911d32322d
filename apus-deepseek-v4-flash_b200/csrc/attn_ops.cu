// Row-wise numerics helpers of the attention sublayer and the compressor /
// indexer steps.  Every kernel reproduces the reference's per-element
// operation sequence (separately rounded multiply and add where the reference
// is built without contraction, BF16 rounds at the same points); the sums of
// squares follow the reference's loop order unless the tree order is selected.
//
// Reference: c/attn.h:290-299 (RoPE), 301-311 (Hadamard), 325-369 (FP8 / FP4
// quant-dequant), 371-378 (RMSNorm), 797-819 (compressor finish), 892-1011
// (compressor decode step), 1027-1067 (indexer q prep and scores),
// 1356-1388 (q norm + RoPE, window KV finish), 692-737 (index sets).
#include <cooperative_groups.h>
#include "common.cuh"
#include "kernels.cuh"

namespace apus {

// ---- one row per CTA: [bf16 in] -> [rms] -> [rope] -> [hadamard] -> [qat] -> [bf16 out] ----
__device__ __forceinline__ float fp4_qat_value(float y) {
    // E2M1 round-to-nearest-even of |y| <= 6 (reference c/attn.h:342-348)
    float a = fabsf(y);
    const float T[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
    const float V[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    int mag = 0;
#pragma unroll
    for (int j = 0; j < 7; j++) mag += (a > T[j]) || (a == T[j] && (j & 1));
    float v = V[mag];
    return (signbit(y) && mag) ? -v : v;      // the table entry of code 8 is +0
}

__global__ void __launch_bounds__(1024)
row_ops_kernel(const float *__restrict__ x, int x_stride, float *__restrict__ y, int y_stride, int n,
               int flags, const float *__restrict__ norm_w, float eps, int rd,
               const float *__restrict__ cs, int rows_per_cs, int cs_stride, const RowDyn dyn,
               uint8_t *__restrict__ q_codes, float *__restrict__ q_scales) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    if (dyn.pos) {                             // position read on the device (see RowDyn)
        const long long p = *dyn.pos;
        if (dyn.gate_ratio > 0) {
            if ((p + 1) % dyn.gate_ratio != 0) return;
            y += ((p + 1) / dyn.gate_ratio - 1) * dyn.y_step;
        }
        if (cs) {
            long long r = p + dyn.cs_bias;
            cs += (r > 0 ? r : 0) * rd;
        }
    }
    extern __shared__ __align__(16) float s_v[];   // [n] row, then [n/32 + 32] scratch
    float *s_red = s_v + n;
    const int row = blockIdx.x, i = threadIdx.x;
    const bool on = i < n;
    float v = on ? x[(size_t)row * x_stride + i] : 0.f;
    if (flags & ROW_BF16_IN) v = bf16_round(v);
    if (flags & (ROW_RMS_W | ROW_RMS_PLAIN)) {
        if (flags & ROW_SEQ_SUM) {             // the reference's loop order: one accumulator, index ascending
            if (on) s_v[i] = __fmul_rn(v, v);
            __syncthreads();
            if (i == 0) s_red[0] = seq_sum_smem(s_v, n, 0.f);
        } else {
            float ss = warp_sum(on ? __fmul_rn(v, v) : 0.f);
            if ((i & 31) == 0) s_red[i >> 5] = ss;
            __syncthreads();
            if (i < 32) {
                float t = i < (int)(blockDim.x >> 5) ? s_red[i] : 0.f;
                t = warp_sum(t);
                if (i == 0) s_red[0] = t;
            }
        }
        __syncthreads();
        float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(s_red[0], (float)n), eps)));
        if (flags & ROW_RMS_W) v = bf16_round(__fmul_rn(norm_w[on ? i : 0], __fmul_rn(v, inv)));
        else v = bf16_round(__fmul_rn(v, inv));
        __syncthreads();
    }
    s_v[on ? i : 0] = on ? v : s_v[0];
    __syncthreads();
    if (flags & (ROW_ROPE | ROW_ROPE_INV)) {
        const int half = rd >> 1;
        if (i < half) {
            const float *c = cs + (size_t)(row / rows_per_cs) * cs_stride;
            float co = c[i], si = c[half + i];
            if (flags & ROW_ROPE_INV) si = -si;
            float x1 = s_v[n - rd + 2 * i], x2 = s_v[n - rd + 2 * i + 1];
            s_v[n - rd + 2 * i] = bf16_round(__fsub_rn(__fmul_rn(x1, co), __fmul_rn(x2, si)));
            s_v[n - rd + 2 * i + 1] = bf16_round(__fadd_rn(__fmul_rn(x1, si), __fmul_rn(x2, co)));
        }
        __syncthreads();
    }
    if (flags & ROW_HADAMARD) {
        for (int len = 1; len < n; len <<= 1) {
            float a = 0.f, b = 0.f;
            const bool lo = on && !(i & len);
            if (lo) { a = s_v[i]; b = s_v[i + len]; }
            __syncthreads();
            if (lo) { s_v[i] = __fadd_rn(a, b); s_v[i + len] = __fsub_rn(a, b); }
            __syncthreads();
        }
        const float inv = (float)pow((double)n, -0.5);
        if (on) s_v[i] = bf16_round(__fmul_rn(s_v[i], inv));
        __syncthreads();
    }
    v = on ? s_v[i] : 0.f;
    if (flags & ROW_FP8QAT) {
        // groups of 64 over the first n - rd elements
        const int lim = n - rd;
        unsigned *s_amax = reinterpret_cast<unsigned *>(s_red);
        if (i < (lim + 63) / 64) s_amax[i] = 0u;
        __syncthreads();
        if (i < lim) atomicMax(&s_amax[i >> 6], __float_as_uint(fabsf(v)));
        __syncthreads();
        if (i < lim) {
            float amax = fmaxf(__uint_as_float(s_amax[i >> 6]), 1e-4f);
            float s = ceil_pow2(__fmul_rn(amax, 1.0f / 448.0f));
            uint16_t c2 = e4m3x2_from_f32(__fdiv_rn(v, s), 0.f);
            v = __fmul_rn(e4m3_to_f32(c2 & 0xffu), s);
        }
    }
    if (flags & ROW_FP4QAT) {
        float amax = warp_max(on ? fabsf(v) : 0.f);     // 32-element groups = warps
        amax = fmaxf(amax, 7.05484372e-38f);
        float s = ceil_pow2(__fmul_rn(amax, 1.0f / 6.0f));
        float q = __fdiv_rn(v, s);
        q = fminf(fmaxf(q, -6.0f), 6.0f);
        v = __fmul_rn(fp4_qat_value(q), s);
    }
    if (flags & ROW_BF16_OUT) v = bf16_round(v);
    if (on) y[(size_t)row * y_stride + i] = v;
    if (q_codes) {
        // activation codes of the finished row (the arithmetic of act_quant_kernel): a 128-group is four warps
        const float vb = bf16_round(v);
        const float m = warp_max(on ? fabsf(vb) : 0.f);
        __syncthreads();
        if ((i & 31) == 0) s_red[i >> 5] = m;
        __syncthreads();
        if (on) {
            const int g = i >> 7;
            float amax = fmaxf(fmaxf(s_red[4 * g], s_red[4 * g + 1]), fmaxf(s_red[4 * g + 2], s_red[4 * g + 3]));
            amax = fmaxf(amax, 1e-4f);
            const float s = ceil_pow2(__fmul_rn(amax, 1.0f / 448.0f));
            const float inv = __uint_as_float(0x7f000000u - __float_as_uint(s));
            q_codes[(size_t)row * n + i] = (uint8_t)(e4m3x2_from_f32(vb * inv, 0.f) & 0xffu);
            if ((i & 127) == 0) q_scales[(size_t)row * (n >> 7) + g] = s;
        }
    }
}

// Two frequent shapes of the row pipeline on MANY rows (every head of every sequence) get kernels
// of their own; same operations, same order, same bits as row_ops_kernel.
// (a) RoPE only, in place: only the last rd elements of a row change -- one thread per pair.
__global__ void __launch_bounds__(256)
rope_rows_kernel(float *__restrict__ y, int stride, int n, int rows, int inverse, int rd, const float *__restrict__ cs,
                 int rows_per_cs, int cs_stride, const RowDyn dyn) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    if (dyn.pos && cs) {
        const long long r = *dyn.pos + dyn.cs_bias;
        cs += (r > 0 ? r : 0) * rd;
    }
    const int half = rd >> 1;
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)rows * half) return;
    const int row = (int)(t / half), i = (int)(t - (long long)row * half);
    const float *c = cs + (size_t)(row / rows_per_cs) * cs_stride;
    const float co = c[i], si = inverse ? -c[half + i] : c[half + i];
    float2 *p = reinterpret_cast<float2 *>(y + (size_t)row * stride + n - rd) + i;
    const float2 v = *p;
    *p = make_float2(bf16_round(__fsub_rn(__fmul_rn(v.x, co), __fmul_rn(v.y, si))),
                     bf16_round(__fadd_rn(__fmul_rn(v.x, si), __fmul_rn(v.y, co))));
}
// (b) weight-free RMSNorm + RoPE (the per-head q rows, c/attn.h:1356-1370): one warp per row, eight
// rows per CTA; the sum of squares in the reference's order is one lane's walk over the warp's
// squares in shared memory, otherwise a warp reduction.
template <int NV>                                  // NV float4 per lane: n = 128 * NV
__global__ void __launch_bounds__(256)
qnorm_rope_rows_kernel(const float *__restrict__ x, int x_stride, float *__restrict__ y, int y_stride, int rows,
                       float eps, int rd, int seq, const float *__restrict__ cs, int rows_per_cs, int cs_stride,
                       const RowDyn dyn) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    constexpr int N = 128 * NV;
    __shared__ __align__(16) float s_sq[8][N];
    if (dyn.pos && cs) {
        const long long r = *dyn.pos + dyn.cs_bias;
        cs += (r > 0 ? r : 0) * rd;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + warp;
    if (row >= rows) return;
    float4 v[NV];
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * x_stride);
#pragma unroll
    for (int j = 0; j < NV; j++) v[j] = xr[lane + 32 * j];
    float tot;
    if (seq) {
        float4 *sq = reinterpret_cast<float4 *>(s_sq[warp]);
#pragma unroll
        for (int j = 0; j < NV; j++)
            sq[lane + 32 * j] = make_float4(__fmul_rn(v[j].x, v[j].x), __fmul_rn(v[j].y, v[j].y),
                                            __fmul_rn(v[j].z, v[j].z), __fmul_rn(v[j].w, v[j].w));
        __syncwarp();
        tot = lane == 0 ? seq_sum_smem(s_sq[warp], N, 0.f) : 0.f;
        tot = __shfl_sync(0xffffffffu, tot, 0);
    } else {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NV; j++)
            ss += __fmul_rn(v[j].x, v[j].x) + __fmul_rn(v[j].y, v[j].y) + __fmul_rn(v[j].z, v[j].z) + __fmul_rn(v[j].w, v[j].w);
        tot = warp_sum(ss);
    }
    const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(tot, (float)N), eps)));
#pragma unroll
    for (int j = 0; j < NV; j++) {
        v[j].x = bf16_round(__fmul_rn(v[j].x, inv)); v[j].y = bf16_round(__fmul_rn(v[j].y, inv));
        v[j].z = bf16_round(__fmul_rn(v[j].z, inv)); v[j].w = bf16_round(__fmul_rn(v[j].w, inv));
    }
    // RoPE on the last rd elements: element e = 4 * (lane + 32 * j) + c; a float4 holds two pairs
    const int half = rd >> 1;
    const float *c = cs + (size_t)(row / rows_per_cs) * cs_stride;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        const int e = 4 * (lane + 32 * j) - (N - rd);          // offset inside the rotated tail
        if (e >= 0) {
            const int i0 = e >> 1;
            const float c0 = c[i0], s0 = c[half + i0], c1 = c[i0 + 1], s1 = c[half + i0 + 1];
            const float4 w = v[j];
            v[j].x = bf16_round(__fsub_rn(__fmul_rn(w.x, c0), __fmul_rn(w.y, s0)));
            v[j].y = bf16_round(__fadd_rn(__fmul_rn(w.x, s0), __fmul_rn(w.y, c0)));
            v[j].z = bf16_round(__fsub_rn(__fmul_rn(w.z, c1), __fmul_rn(w.w, s1)));
            v[j].w = bf16_round(__fadd_rn(__fmul_rn(w.z, s1), __fmul_rn(w.w, c1)));
        }
    }
    float4 *yr = reinterpret_cast<float4 *>(y + (size_t)row * y_stride);
#pragma unroll
    for (int j = 0; j < NV; j++) yr[lane + 32 * j] = v[j];
}

int row_ops(const float *x, int x_stride, float *y, int y_stride, int rows, int n, int flags,
            const float *norm_w, float eps, int rd, const float *cs, int rows_per_cs, int cs_stride,
            cudaStream_t st, const RowDyn *dyn, uint8_t *q_codes, float *q_scales) {
    APUS_REQUIRE(n >= 32 && n <= 1024 && n % 32 == 0, "row_ops: n=%d unsupported", n);
    APUS_REQUIRE(!q_codes || (n % 128 == 0 && q_scales && (!dyn || dyn->gate_ratio == 0)), "row_ops: codes need n %% 128 == 0 (n=%d)", n);
    APUS_REQUIRE(!(flags & ROW_HADAMARD) || (n & (n - 1)) == 0, "row_ops: Hadamard needs a power of two, n=%d", n);
    if (rows <= 0) return 0;
    size_t smem = (size_t)(n + 64) * sizeof(float);
    if (!sum_tree(APUS_CUDA_TREE_NORMS)) flags |= ROW_SEQ_SUM;
    const RowDyn none = {nullptr, 0, 0, 0};
    const bool no_gate = !dyn || dyn->gate_ratio == 0;
    const int base = flags & ~ROW_SEQ_SUM;
    if (!q_codes && rows >= 32 && no_gate && cs && rd % 4 == 0 && rd <= n && (base == ROW_ROPE || base == ROW_ROPE_INV) && x == y &&
        x_stride == y_stride && x_stride % 2 == 0 && (n - rd) % 2 == 0) {
        const long long pairs = (long long)rows * (rd / 2);
        launch_k(rope_rows_kernel, (unsigned)((pairs + 255) / 256), 256, 0, st, y, y_stride, n, rows, base == ROW_ROPE_INV, rd, cs,
                                                                         rows_per_cs > 0 ? rows_per_cs : 1, cs_stride,
                                                                         dyn ? *dyn : none);
        APUS_LAUNCHED();
        return 0;
    }
    if (!q_codes && rows >= 32 && no_gate && cs && base == (ROW_RMS_PLAIN | ROW_ROPE) && (n == 512 || n == 256 || n == 128) &&
        rd % 4 == 0 && rd <= n && x_stride % 4 == 0 && y_stride % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0) {
        const unsigned g = (unsigned)((rows + 7) / 8);
        const int seq = (flags & ROW_SEQ_SUM) ? 1 : 0, rpc = rows_per_cs > 0 ? rows_per_cs : 1;
        const RowDyn d = dyn ? *dyn : none;
        if (n == 512) launch_k(qnorm_rope_rows_kernel<4>, g, 256, 0, st, x, x_stride, y, y_stride, rows, eps, rd, seq, cs, rpc, cs_stride, d);
        else if (n == 256) launch_k(qnorm_rope_rows_kernel<2>, g, 256, 0, st, x, x_stride, y, y_stride, rows, eps, rd, seq, cs, rpc, cs_stride, d);
        else launch_k(qnorm_rope_rows_kernel<1>, g, 256, 0, st, x, x_stride, y, y_stride, rows, eps, rd, seq, cs, rpc, cs_stride, d);
        APUS_LAUNCHED();
        return 0;
    }
    launch_k(row_ops_kernel, rows, n, smem, st, x, x_stride, y, y_stride, n, flags, norm_w, eps, rd, cs,
                                          rows_per_cs > 0 ? rows_per_cs : 1, cs_stride, dyn ? *dyn : none, q_codes, q_scales);
    APUS_LAUNCHED();
    return 0;
}

// ---- compressor decode step (reference c/attn.h:960-1008) ---------------------------------
// One CTA per sequence, one thread per state column (cd = coff*d).
//   write: state row (overlap ? ratio + slot : slot) <- kv_new, score_new + ape[slot]
//   pool (when the block completes): per channel c < d a softmax over the ne
//     candidate rows (sequential, in row order), weighted sum -> pooled[c]
//   shift (overlap only): rows [ratio, 2*ratio) -> [0, ratio)
__global__ void __launch_bounds__(1024)
comp_step_kernel(float *__restrict__ kv_state, float *__restrict__ sc_state, long long state_stride,
                 const float *__restrict__ kv_new, const float *__restrict__ sc_new, int new_stride,
                 const float *__restrict__ ape, int ratio, int overlap, int d, int slot, int should,
                 float *__restrict__ pooled, int pooled_stride, const long long *__restrict__ dyn_pos) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    if (dyn_pos) {
        const long long p = *dyn_pos;
        slot = (int)(p % ratio);
        should = (p + 1) % ratio == 0;
    }
    const int seq = blockIdx.x, c = threadIdx.x;
    const int cd = (1 + overlap) * d;
    float *kvs = kv_state + (size_t)seq * state_stride;
    float *scs = sc_state + (size_t)seq * state_stride;
    const int wrow = overlap ? ratio + slot : slot;
    if (c < cd) {
        kvs[(size_t)wrow * cd + c] = kv_new[(size_t)seq * new_stride + c];
        scs[(size_t)wrow * cd + c] = __fadd_rn(sc_new[(size_t)seq * new_stride + c], ape[(size_t)slot * cd + c]);
    }
    if (!should) return;
    __syncthreads();
    const int ne = overlap ? 2 * ratio : ratio;
    if (c < d) {
        float mx = -INFINITY;
        for (int e = 0; e < ne; e++) {
            float p = (overlap && e >= ratio) ? scs[(size_t)e * cd + d + c] : scs[(size_t)e * cd + c];
            mx = fmaxf(mx, p);
        }
        float sum = 0.f;
        for (int e = 0; e < ne; e++) {
            float p = (overlap && e >= ratio) ? scs[(size_t)e * cd + d + c] : scs[(size_t)e * cd + c];
            sum = __fadd_rn(sum, exp_rn(__fsub_rn(p, mx)));
        }
        float acc = 0.f;
        for (int e = 0; e < ne; e++) {
            const size_t off = (overlap && e >= ratio) ? (size_t)e * cd + d + c : (size_t)e * cd + c;
            float p = exp_rn(__fsub_rn(scs[off], mx));
            acc = __fadd_rn(acc, __fmul_rn(kvs[off], __fdiv_rn(p, sum)));
        }
        pooled[(size_t)seq * pooled_stride + c] = acc;
    }
    if (overlap) {
        __syncthreads();
        if (c < cd)
            for (int e = 0; e < ratio; e++) {
                kvs[(size_t)e * cd + c] = kvs[(size_t)(ratio + e) * cd + c];
                scs[(size_t)e * cd + c] = scs[(size_t)(ratio + e) * cd + c];
            }
    }
}

int comp_step(float *kv_state, float *sc_state, long long state_stride, const float *kv_new,
              const float *sc_new, int new_stride, const float *ape, int ratio, int overlap, int d,
              int slot, int should, float *pooled, int pooled_stride, int n_seq, cudaStream_t st,
              const long long *dyn_pos) {
    const int cd = (1 + overlap) * d;
    APUS_REQUIRE(cd <= 1024, "compressor: state width %d exceeds 1024", cd);
    if (n_seq <= 0) return 0;
    launch_k(comp_step_kernel, n_seq, ((cd + 31) / 32) * 32, 0, st, kv_state, sc_state, state_stride, kv_new,
                                                              sc_new, new_stride, ape, ratio, overlap, d,
                                                              slot, should, pooled, pooled_stride, dyn_pos);
    APUS_LAUNCHED();
    return 0;
}

// ---- indexer scores (reference c/attn.h:1049-1067) ---------------------------------------------
// score[b] = bf16( sum_h bf16( relu(bf16(q_h . k_b)) * w_h ) ), heads summed in order.
// CTA = ih threads x IDX_B cache entries; each thread computes one (head, entry)
// dot sequentially in k order with separately rounded multiply and add, then one
// thread per entry adds the per-head terms in head order.
#define IDX_B 4
__global__ void __launch_bounds__(64 * IDX_B)
idx_score_kernel(const float *__restrict__ q, const float *__restrict__ wt_raw, float wscale,
                 const float *__restrict__ cache, long long cache_stride, long long nb, int ih, int idm,
                 float *__restrict__ sc, const long long *__restrict__ dyn_pos, int ratio, long long chunk_pos0,
                 int chunk_seqs) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ float sm[];             // q [ih*idm], k [IDX_B*idm], terms [IDX_B*ih]
    q += (size_t)blockIdx.y * ih * idm;
    wt_raw += (size_t)blockIdx.y * ih;
    // rows of a chunk are time-major: row = t * chunk_seqs + sequence, at position chunk_pos0 + t
    cache += (size_t)(chunk_seqs > 0 ? blockIdx.y % chunk_seqs : blockIdx.y) * cache_stride;
    sc += (size_t)blockIdx.y * nb;             // row stride: the capacity when the count is derived on the device
    if (dyn_pos || chunk_seqs > 0) {
        nb = ((dyn_pos ? *dyn_pos : chunk_pos0 + blockIdx.y / chunk_seqs) + 1) / ratio;
        if ((long long)blockIdx.x * IDX_B >= nb) return;
    }
    // q rows are padded by one word: the lanes of a warp walk different heads at the same k, and a
    // pitch of idm (a multiple of 32) would put all of them on one bank
    const int qp = idm + 1;
    float *s_q = sm, *s_k = sm + ih * qp, *s_t = s_k + IDX_B * idm;
    const int hh = threadIdx.x % ih, bl = threadIdx.x / ih;
    const long long b = (long long)blockIdx.x * IDX_B + bl;
    for (int i = threadIdx.x; i < ih * idm; i += blockDim.x) s_q[(i / idm) * qp + i % idm] = q[i];
    for (int i = threadIdx.x; i < IDX_B * idm; i += blockDim.x) {
        long long bb = (long long)blockIdx.x * IDX_B + i / idm;
        s_k[i] = bb < nb ? cache[bb * idm + i % idm] : 0.f;
    }
    __syncthreads();
    const float *qv = s_q + hh * qp, *kv = s_k + bl * idm;
    float dot = 0.f;
    for (int i = 0; i < idm; i++) dot = __fadd_rn(dot, __fmul_rn(qv[i], kv[i]));
    dot = bf16_round(dot);
    // head weight: bf16(bf16_linear(x) * idm^-0.5 * ih^-0.5) (reference c/attn.h:1133-1135)
    const float w = bf16_round(__fmul_rn(wt_raw[hh], wscale));
    float v = dot > 0.f ? __fmul_rn(dot, w) : 0.f;
    s_t[bl * ih + hh] = bf16_round(v);
    __syncthreads();
    if (hh == 0 && b < nb) {
        float acc = 0.f;
        for (int h2 = 0; h2 < ih; h2++) acc = __fadd_rn(acc, s_t[bl * ih + h2]);
        sc[b] = bf16_round(acc);
    }
}

int idx_scores(const float *q, const float *wt_raw, float wscale, const float *cache, long long cache_stride,
               long long nb, int ih, int idm, float *sc, int n_seq, cudaStream_t st, const long long *dyn_pos,
               int ratio, long long chunk_pos0, int chunk_seqs) {
    APUS_REQUIRE(ih <= 64 && ih >= 1, "indexer: %d heads unsupported", ih);
    if (nb <= 0 || n_seq <= 0) return 0;
    size_t smem = ((size_t)ih * (idm + 1) + IDX_B * idm + IDX_B * ih) * sizeof(float);
    if (ensure_dyn_smem((const void *)idx_score_kernel, smem)) return 1;
    dim3 grid((unsigned)((nb + IDX_B - 1) / IDX_B), (unsigned)n_seq);
    launch_k(idx_score_kernel, grid, ih * IDX_B, smem, st, q, wt_raw, wscale, cache, cache_stride, nb, ih, idm, sc,
                                                     dyn_pos, ratio, chunk_pos0, chunk_seqs);
    APUS_LAUNCHED();
    return 0;
}

// ---- index set of one decode step (reference c/attn.h:692-737) -------------------------------------
// row = [window ids in ring order] ++ [compressed ids + win]; comp ids either the
// indexer's top-k (sel != NULL) or the dense list 0..compw-1.
__global__ void build_idx_kernel(int32_t *__restrict__ out, int win, long long pos,
                                 const int32_t *__restrict__ sel, int compw,
                                 const long long *__restrict__ dyn_pos, int ratio) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    out += (size_t)blockIdx.y * (win + compw);
    if (sel) sel += (size_t)blockIdx.y * compw;
    if (dyn_pos) {                             // compw so far = capacity; the rest of the row is padding
        const int cap = compw;
        pos = *dyn_pos;
        const long long nbs = ratio ? (pos + 1) / ratio : 0;
        compw = (int)(nbs < cap ? nbs : cap);
        if (j >= win + compw && j < win + cap) { out[j] = -1; return; }
    }
    if (j < win) {
        int v;
        if (pos >= win - 1) {
            int sp = (int)(pos % win);
            v = j < win - 1 - sp ? sp + 1 + j : j - (win - 1 - sp);
        } else {
            v = j <= pos ? j : -1;
        }
        out[j] = v;
    } else if (j < win + compw) {
        out[j] = (sel ? sel[j - win] : j - win) + win;
    }
}

int build_idx(int32_t *out, int win, long long pos, const int32_t *sel, int compw, int n_seq, cudaStream_t st,
              const long long *dyn_pos, int ratio) {
    if (n_seq <= 0) return 0;
    launch_k(build_idx_kernel, dim3(ceil_div(win + compw, 256), n_seq), 256, 0, st, out, win, pos, sel, compw, dyn_pos,
                                                                              ratio);
    APUS_LAUNCHED();
    return 0;
}

__global__ void scatter_rows_kernel(float *__restrict__ dst, long long dst_stride,
                                    const float *__restrict__ src, int n,
                                    const long long *__restrict__ dyn_pos, int win) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    if (dyn_pos) dst += (size_t)(*dyn_pos % win) * n;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[(size_t)blockIdx.y * dst_stride + i] = src[(size_t)blockIdx.y * n + i];
}

int scatter_rows(float *dst, long long dst_stride, const float *src, int n, int rows, cudaStream_t st,
                 const long long *dyn_pos, int win) {
    if (rows <= 0) return 0;
    launch_k(scatter_rows_kernel, dim3(ceil_div(n, 256), rows), 256, 0, st, dst, dst_stride, src, n, dyn_pos, win);
    APUS_LAUNCHED();
    return 0;
}

// ---- a chunk of consecutive positions (batched prefill, reference c/attn.h:1621-1680) ----------
// Rows of a chunk are time-major: row = t * n_seq + sequence, at position pos0 + t.  The window
// candidates of a chunk live in a position-ordered buffer per sequence,
//   ext[seq][j] = KV row of position pos0 - win + j,   j in [0, win + s),
// the first `win` rows copied from the ring, the rest the chunk's own rows; the index row of a
// token lists its window oldest first (the order of c/attn.h:692-720 once the -1 entries are
// dropped) and then its compressed ids, offset by win + s.
__global__ void win_ext_kernel(float *__restrict__ ext, const float *__restrict__ ring, const float *__restrict__ kv,
                               int win, int s, int d, int n_seq, long long pos0) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int j = blockIdx.y, seq = blockIdx.z;
    float *dst = ext + ((size_t)seq * (win + s) + j) * d;
    const float *src = nullptr;
    if (j >= win) src = kv + ((size_t)(j - win) * n_seq + seq) * d;
    else {
        const long long q = pos0 - win + j;
        if (q >= 0) src = ring + ((size_t)seq * win + (size_t)(q % win)) * d;
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < d; i += gridDim.x * blockDim.x) dst[i] = src ? src[i] : 0.f;
}
// the ring after the chunk: the last min(s, win) rows at their slots (c/attn.h:1642-1658)
__global__ void ring_update_kernel(float *__restrict__ ring, const float *__restrict__ kv, int win, int s, int d,
                                   int n_seq, long long pos0, int t0) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int t = t0 + blockIdx.y, seq = blockIdx.z;
    float *dst = ring + ((size_t)seq * win + (size_t)((pos0 + t) % win)) * d;
    const float *src = kv + ((size_t)t * n_seq + seq) * d;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < d; i += gridDim.x * blockDim.x) dst[i] = src[i];
}
int win_ext(float *ext, const float *ring, const float *kv, int win, int s, int d, int n_seq, long long pos0,
            cudaStream_t st) {
    if (s <= 0 || n_seq <= 0) return 0;
    launch_k(win_ext_kernel, dim3(ceil_div(d, 256), win + s, n_seq), 256, 0, st, ext, ring, kv, win, s, d, n_seq, pos0);
    APUS_LAUNCHED();
    return 0;
}
int ring_update(float *ring, const float *kv, int win, int s, int d, int n_seq, long long pos0, cudaStream_t st) {
    if (s <= 0 || n_seq <= 0) return 0;
    const int t0 = s > win ? s - win : 0;
    launch_k(ring_update_kernel, dim3(ceil_div(d, 256), s - t0, n_seq), 256, 0, st, ring, kv, win, s, d, n_seq, pos0, t0);
    APUS_LAUNCHED();
    return 0;
}

__global__ void build_idx_chunk_kernel(int32_t *__restrict__ out, int win, int s, long long pos0, int n_seq,
                                       const int32_t *__restrict__ sel, int compcap, int ratio) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int j = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
    if (j >= win + compcap) return;
    const int t = row / n_seq;
    const long long p = pos0 + t;
    int v = -1;
    if (j < win) {
        if (p - win + 1 + j >= 0) v = t + 1 + j;                 // position p - win + 1 + j in ext coordinates
    } else {
        const long long nbs = ratio ? (p + 1) / ratio : 0;
        const int jj = j - win;
        if (jj < nbs) v = (sel ? sel[(size_t)row * compcap + jj] : jj) + win + s;
    }
    out[(size_t)row * (win + compcap) + j] = v;
}
int build_idx_chunk(int32_t *out, int win, int s, long long pos0, int n_seq, const int32_t *sel, int compcap, int ratio,
                    cudaStream_t st) {
    if (s <= 0 || n_seq <= 0) return 0;
    launch_k(build_idx_chunk_kernel, dim3(ceil_div(win + compcap, 256), s * n_seq), 256, 0, st, out, win, s, pos0, n_seq, sel,
                                                                                          compcap, ratio);
    APUS_LAUNCHED();
    return 0;
}

// First index of the maximum: strict greater-than scan order (reference c/sample.h:76-81).
__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const float *__restrict__ x, int n, int32_t *__restrict__ out) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    const float *r = x + (size_t)blockIdx.x * n;
    float v = -INFINITY;
    int vi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float t = r[i];
        if (t > v || (t == v && i < vi)) { v = t; vi = i; }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, vi, o);
        if (ov > v || (ov == v && oi < vi)) { v = ov; vi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = v; s_i[threadIdx.x >> 5] = vi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        v = threadIdx.x < (blockDim.x >> 5) ? s_v[threadIdx.x] : -INFINITY;
        vi = threadIdx.x < (blockDim.x >> 5) ? s_i[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, v, o);
            int oi = __shfl_xor_sync(0xffffffffu, vi, o);
            if (ov > v || (ov == v && oi < vi)) { v = ov; vi = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = vi == 0x7fffffff ? 0 : vi;
    }
}

// The same for long rows (a vocabulary of 129,280 logits is 517 KB): a cluster of eight CTAs
// per row, 16-byte loads, the eight candidates combined through distributed shared memory
// with the same rule (larger value, lower index on ties), so the pick is the scan order's.
#define AMAX_CL 8
__device__ __forceinline__ void amax_take(float &v, int &vi, float ov, int oi) {
    if (ov > v || (ov == v && oi < vi)) { v = ov; vi = oi; }
}
__global__ void __cluster_dims__(AMAX_CL, 1, 1) __launch_bounds__(512)
argmax_rows_cl_kernel(const float *__restrict__ x, int n, int32_t *__restrict__ out) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    __shared__ float s_bv;
    __shared__ int s_bi;
    const int row = blockIdx.x / AMAX_CL, rank = (int)cluster.block_rank();
    const float *r = x + (size_t)row * n;
    const int n4 = n >> 2;
    const int per = (n4 + AMAX_CL - 1) / AMAX_CL, q0 = min(n4, rank * per), q1 = min(n4, q0 + per);
    float v = -INFINITY;
    int vi = 0x7fffffff;
    for (int q = q0 + threadIdx.x; q < q1; q += blockDim.x) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(r) + q);
        amax_take(v, vi, t.x, 4 * q); amax_take(v, vi, t.y, 4 * q + 1);
        amax_take(v, vi, t.z, 4 * q + 2); amax_take(v, vi, t.w, 4 * q + 3);
    }
    if (rank == AMAX_CL - 1)                               // the tail when n is not a multiple of 4
        for (int i = 4 * n4 + threadIdx.x; i < n; i += blockDim.x) amax_take(v, vi, r[i], i);
#pragma unroll
    for (int o = 16; o; o >>= 1)
        amax_take(v, vi, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, vi, o));
    if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = v; s_i[threadIdx.x >> 5] = vi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        v = threadIdx.x < (blockDim.x >> 5) ? s_v[threadIdx.x] : -INFINITY;
        vi = threadIdx.x < (blockDim.x >> 5) ? s_i[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o; o >>= 1)
            amax_take(v, vi, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, vi, o));
        if (threadIdx.x == 0) { s_bv = v; s_bi = vi; }
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        v = -INFINITY; vi = 0x7fffffff;
        for (int q = 0; q < AMAX_CL; q++) amax_take(v, vi, *cluster.map_shared_rank(&s_bv, q), *cluster.map_shared_rank(&s_bi, q));
        out[row] = vi == 0x7fffffff ? 0 : vi;
    }
    cluster.sync();                                        // nobody leaves while its candidate may still be read
}

int argmax_rows(const float *x, int n, int rows, int32_t *out, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (n >= 16384 && n % 4 == 0 && ((uintptr_t)x & 15) == 0)
        argmax_rows_cl_kernel<<<rows * AMAX_CL, 512, 0, st>>>(x, n, out);
    else
        launch_k(argmax_rows_kernel, rows, 1024, 0, st, x, n, out);
    APUS_LAUNCHED();
    return 0;
}

__global__ void embed_rows_kernel(const void *__restrict__ table, int bf16, const int64_t *__restrict__ ids,
                                  int hc, int dim, float *__restrict__ out) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int r = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dim) return;
    const int64_t id = ids[r];
    float v = bf16 ? __uint_as_float((uint32_t)reinterpret_cast<const uint16_t *>(table)[id * dim + i] << 16)
                   : reinterpret_cast<const float *>(table)[id * dim + i];
    for (int j = 0; j < hc; j++) out[((size_t)r * hc + j) * dim + i] = v;
}

int embed_rows(const void *table, int bf16, const int64_t *ids, int rows, int hc, int dim, float *out,
               cudaStream_t st) {
    if (rows <= 0) return 0;
    launch_k(embed_rows_kernel, dim3(ceil_div(dim, 256), rows), 256, 0, st, table, bf16, ids, hc, dim, out);
    APUS_LAUNCHED();
    return 0;
}

}  // namespace apus
