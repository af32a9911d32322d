// Stable top-k selection and index-gathered sparse attention.
#include <map>
#include <cooperative_groups.h>
#include "common.cuh"
#include "kernels.cuh"

namespace apus {

// ---- stable top-k --------------------------------------------------------------
//
// Reference c/attn.h:668-687: k passes of strict-greater argmax over unused
// entries, i.e. the k largest scores, equal scores ordered by ascending index,
// emitted in that order.  Restated as a selection on the composite key
// (score, -index): an 8-bit radix select on the order-preserving integer image
// of the score finds the k-th largest score value T and how many scores are
// strictly greater; a second, index-ordered sweep takes every score > T and
// the lowest-index scores == T until k are chosen; a bitonic sort of the k
// (key, index) pairs gives the output order.  One CTA per row.
// Bytes per row: 5 sweeps over n*4 (L2-resident for n <= a few million).
__device__ __forceinline__ uint32_t order_key(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u << 1) == 0) u = 0;                 // -0.0 and +0.0 compare equal
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

#define TOPK_THREADS 1024
#define TOPK_MAX_K 2048

__global__ void __launch_bounds__(TOPK_THREADS)
topk_stable_kernel(const float *__restrict__ scores, int n, int k, int32_t *__restrict__ idx_out,
                   const long long *__restrict__ dyn_pos, int ratio, long long chunk_pos0, int rows_per_pos) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    __shared__ unsigned hist[256];
    __shared__ unsigned s_prefix, s_need, s_greater, s_taken, s_base;
    __shared__ unsigned long long sel[TOPK_MAX_K];
    const float *row = scores + (size_t)blockIdx.x * n;     // n, k as given are the row strides
    int32_t *out = idx_out + (size_t)blockIdx.x * k;
    if (dyn_pos || rows_per_pos > 0) {                      // live sizes from the position (of the row, in a chunk)
        const long long nbs = ((dyn_pos ? *dyn_pos : chunk_pos0 + blockIdx.x / rows_per_pos) + 1) / ratio;
        n = (int)(nbs < n ? nbs : n);
        k = k < n ? k : n;
        if (k <= 0) return;
    }
    const int tid = threadIdx.x;

    const int lane = tid & 31, warp = tid >> 5;
    if (k >= n) {
        // every score is selected (a row shorter than k: the first 4 k positions of a sequence): only the order is left
        for (int i = tid; i < n; i += TOPK_THREADS)
            sel[i] = ((unsigned long long)order_key(row[i]) << 32) | (0xffffffffu - (unsigned)i);
        k = n;
        __syncthreads();
    } else {
    // radix select: after the loop `prefix` is the key of the k-th largest score
    if (tid == 0) { s_prefix = 0; s_need = (unsigned)k; s_greater = 0; }
    for (int pass = 0; pass < 4; pass++) {
        const int shift = 24 - 8 * pass;
        for (int i = tid; i < 256; i += TOPK_THREADS) hist[i] = 0;
        __syncthreads();
        const unsigned prefix = s_prefix;
        const unsigned himask = pass ? (0xffffffffu << (shift + 8)) : 0u;
        for (int i = tid; i < n; i += TOPK_THREADS) {
            unsigned key = order_key(row[i]);
            if ((key & himask) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
        }
        __syncthreads();
        if (warp == 0) {
            // the bin where the count from the top reaches `need` (bin 0 if it never does before it):
            // lane L sums bins 255 - 8L .. 248 - 8L, a warp scan finds the lane, the lane walks its 8 bins
            const unsigned need = s_need;
            unsigned c[8], tot = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) { c[j] = hist[255 - 8 * lane - j]; tot += c[j]; }
            unsigned inc = tot;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const unsigned v = __shfl_up_sync(0xffffffffu, inc, off);
                if (lane >= off) inc += v;
            }
            const unsigned exc = inc - tot;
            const unsigned hit = __ballot_sync(0xffffffffu, exc < need && inc >= need);
            const int owner = hit ? __ffs(hit) - 1 : 31;
            if (lane == owner) {
                unsigned acc = exc;
                int b = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int bin = 255 - 8 * lane - j;
                    if (bin == 0) break;                          // bin 0 takes whatever is left
                    if (acc + c[j] >= need) { b = bin; break; }
                    acc += c[j];
                }
                s_greater += acc;
                s_need = need - acc;
                s_prefix = prefix | ((unsigned)b << shift);
            }
        }
        __syncthreads();
    }
    const unsigned T = s_prefix;
    const unsigned n_greater = s_greater;          // scores with key > T
    const unsigned n_ties = (unsigned)k - n_greater;   // lowest-index scores == T to take
    if (tid == 0) { s_taken = 0; s_base = 0; }
    __syncthreads();

    // index-ordered sweep: greater keys go to slots [0, n_greater) in any order
    // (sorted below); ties are appended in ascending index order.
    __shared__ unsigned w_tie[TOPK_THREADS / 32];
    for (int base = 0; base < n; base += TOPK_THREADS) {
        int i = base + tid;
        unsigned key = i < n ? order_key(row[i]) : 0u;
        bool gt = i < n && key > T;
        bool eq = i < n && key == T;
        if (gt) {
            unsigned slot = atomicAdd(&s_taken, 1u);
            sel[slot] = ((unsigned long long)key << 32) | (0xffffffffu - (unsigned)i);
        }
        unsigned m = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) w_tie[warp] = __popc(m);
        __syncthreads();
        unsigned before = 0;
        for (int w = 0; w < warp; w++) before += w_tie[w];
        unsigned total = 0;
        for (int w = 0; w < TOPK_THREADS / 32; w++) total += w_tie[w];
        unsigned rank = s_base + before + __popc(m & ((1u << lane) - 1u));
        if (eq && rank < n_ties)
            sel[n_greater + rank] = ((unsigned long long)key << 32) | (0xffffffffu - (unsigned)i);
        __syncthreads();
        if (tid == 0) s_base += total;
        __syncthreads();
    }
    }

    // bitonic sort, descending, on the composite (key, -index)
    int kp = 1;
    while (kp < k) kp <<= 1;
    for (int i = k + tid; i < kp; i += TOPK_THREADS) sel[i] = 0ull;
    __syncthreads();
    for (int size = 2; size <= kp; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < kp; i += TOPK_THREADS) {
                int j = i ^ stride;
                if (j > i) {
                    unsigned long long a = sel[i], b = sel[j];
                    bool desc = ((i & size) == 0);
                    if (desc ? (a < b) : (a > b)) { sel[i] = b; sel[j] = a; }
                }
            }
            __syncthreads();
        }
    for (int i = tid; i < k; i += TOPK_THREADS)
        out[i] = (int32_t)(0xffffffffu - (unsigned)(sel[i] & 0xffffffffu));
}

// The same selection for long rows, a row spread over a cluster of TOPK_CL CTAs (one CTA sweeping 262,144
// scores five times takes ~350 us): every CTA histograms its slice, all of them add the eight histograms
// through distributed shared memory and derive the same digit, so no result has to be sent around; the
// chosen entries are stored into rank 0's shared memory (greater keys at slots counted per slice, ties in
// index order behind them), where rank 0 sorts and writes them out.  Nobody touches another CTA's shared
// memory before a first cluster barrier (a CTA of the cluster may not have started yet), and nobody leaves
// before the last reader is done.
#define TOPK_CL 8
__global__ void __cluster_dims__(TOPK_CL, 1, 1) __launch_bounds__(TOPK_THREADS)
topk_stable_cl_kernel(const float *__restrict__ scores, int n, int k, int32_t *__restrict__ idx_out,
                      const long long *__restrict__ dyn_pos, int ratio, long long chunk_pos0, int rows_per_pos) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ unsigned hist[256];
    __shared__ unsigned ghist[2][256];                 // rank 0's copies: the eight slices' histograms added up
    __shared__ unsigned s_digit[2];
    __shared__ unsigned s_cnt[2];                      // this slice's keys > T and keys == T
    __shared__ unsigned s_taken, s_base;
    __shared__ unsigned w_tie[TOPK_THREADS / 32];
    __shared__ unsigned long long sel[TOPK_MAX_K];     // rank 0's copy collects the choice
    const int rowi = blockIdx.x / TOPK_CL, rank = (int)cluster.block_rank();
    const float *row = scores + (size_t)rowi * n;       // n, k as given are the row strides
    int32_t *out = idx_out + (size_t)rowi * k;
    if (dyn_pos || rows_per_pos > 0) {
        const long long nbs = ((dyn_pos ? *dyn_pos : chunk_pos0 + rowi / rows_per_pos) + 1) / ratio;
        n = (int)(nbs < n ? nbs : n);
        k = k < n ? k : n;
    }
    cluster.sync();                                    // every CTA of the cluster runs from here on
    if (k <= 0) return;                                // the same decision in all eight
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = (n + TOPK_CL - 1) / TOPK_CL, i0 = min(n, rank * per), i1 = min(n, i0 + per);
    unsigned prefix = 0, need = (unsigned)(k < n ? k : n), n_greater = 0;
    const bool all = k >= n;                           // every score is taken: only the order is left
    if (all) k = n;
    unsigned *g0 = cluster.map_shared_rank(&ghist[0][0], 0);     // rank 0 holds the summed histograms (two, alternating)
    for (int pass = 0; pass < 4 && !all; pass++) {
        const int shift = 24 - 8 * pass;
        unsigned *gh = g0 + (pass & 1) * 256;
        for (int i = tid; i < 256; i += TOPK_THREADS) {
            hist[i] = 0;
            if (rank == 0) ghist[pass & 1][i] = 0;             // last read two barriers ago
        }
        cluster.sync();
        const unsigned himask = pass ? (0xffffffffu << (shift + 8)) : 0u;
        for (int i = i0 + tid; i < i1; i += TOPK_THREADS) {
            const unsigned key = order_key(row[i]);
            if ((key & himask) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
        }
        __syncthreads();
        if (tid < 256 && hist[tid]) atomicAdd(gh + tid, hist[tid]);   // one remote add per bin and CTA
        cluster.sync();                                // the sum is complete
        if (warp == 0) {
            // the digit from the summed histogram (lane L: bins 255-8L .. 248-8L), the same in every CTA
            unsigned c[8], tot = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) { c[j] = gh[255 - 8 * lane - j]; tot += c[j]; }
            unsigned inc = tot;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const unsigned v = __shfl_up_sync(0xffffffffu, inc, off);
                if (lane >= off) inc += v;
            }
            const unsigned exc = inc - tot;
            const unsigned hit = __ballot_sync(0xffffffffu, exc < need && inc >= need);
            const int owner = hit ? __ffs(hit) - 1 : 31;
            if (lane == owner) {
                unsigned acc = exc;
                int b = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int bin = 255 - 8 * lane - j;
                    if (bin == 0) break;                    // bin 0 takes whatever is left
                    if (acc + c[j] >= need) { b = bin; break; }
                    acc += c[j];
                }
                s_digit[0] = acc; s_digit[1] = (unsigned)b;
            }
        }
        __syncthreads();
        n_greater += s_digit[0];
        need -= s_digit[0];
        prefix |= s_digit[1] << shift;
        __syncthreads();                               // s_digit is rewritten in the next pass
    }
    const unsigned T = all ? 0u : prefix;
    const unsigned n_ties = all ? 0u : (unsigned)k - n_greater;
    // this slice's counts, then where its entries go: greater keys after those of lower slices, ties (in
    // index order) after the ties of lower slices
    if (tid == 0) { s_cnt[0] = 0; s_cnt[1] = 0; s_taken = 0; s_base = 0; }
    __syncthreads();
    {
        unsigned g = 0, e = 0;
        for (int i = i0 + tid; i < i1; i += TOPK_THREADS) {
            const unsigned key = order_key(row[i]);
            g += all || key > T;
            e += !all && key == T;
        }
        g = __reduce_add_sync(0xffffffffu, g);
        e = __reduce_add_sync(0xffffffffu, e);
        if (lane == 0) { atomicAdd(&s_cnt[0], g); atomicAdd(&s_cnt[1], e); }
    }
    cluster.sync();
    unsigned g_base = 0, e_base = 0;
    for (int q = 0; q < rank; q++) {
        const unsigned *cq = cluster.map_shared_rank(s_cnt, q);
        g_base += cq[0]; e_base += cq[1];
    }
    unsigned long long *sel0 = cluster.map_shared_rank(sel, 0);
    for (int base = i0; base < i1; base += TOPK_THREADS) {
        const int i = base + tid;
        const unsigned key = i < i1 ? order_key(row[i]) : 0u;
        const bool gt = i < i1 && (all || key > T);
        const bool eq = i < i1 && !all && key == T;
        if (gt) {
            const unsigned slot = g_base + atomicAdd(&s_taken, 1u);
            sel0[slot] = ((unsigned long long)key << 32) | (0xffffffffu - (unsigned)i);
        }
        const unsigned m = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) w_tie[warp] = __popc(m);
        __syncthreads();
        unsigned before = 0, total = 0;
        for (int w = 0; w < TOPK_THREADS / 32; w++) {
            if (w < warp) before += w_tie[w];
            total += w_tie[w];
        }
        const unsigned trank = e_base + s_base + before + __popc(m & ((1u << lane) - 1u));
        if (eq && trank < n_ties)
            sel0[n_greater + trank] = ((unsigned long long)key << 32) | (0xffffffffu - (unsigned)i);
        __syncthreads();
        if (tid == 0) s_base += total;
        __syncthreads();
    }
    cluster.sync();                                    // the whole choice sits in rank 0
    if (rank != 0) return;
    int kp = 1;
    while (kp < k) kp <<= 1;
    for (int i = k + tid; i < kp; i += TOPK_THREADS) sel[i] = 0ull;
    __syncthreads();
    for (int size = 2; size <= kp; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < kp; i += TOPK_THREADS) {
                const int j = i ^ stride;
                if (j > i) {
                    const unsigned long long a = sel[i], b = sel[j];
                    const bool desc = ((i & size) == 0);
                    if (desc ? (a < b) : (a > b)) { sel[i] = b; sel[j] = a; }
                }
            }
            __syncthreads();
        }
    for (int i = tid; i < k; i += TOPK_THREADS)
        out[i] = (int32_t)(0xffffffffu - (unsigned)(sel[i] & 0xffffffffu));
}

int topk_stable(const float *scores, int n, int k, int32_t *idx, int rows,
                cudaStream_t st, const long long *dyn_pos, int ratio, long long chunk_pos0, int rows_per_pos) {
    APUS_REQUIRE(k >= 1 && (k <= n || dyn_pos || rows_per_pos > 0) && k <= TOPK_MAX_K, "topk: n=%d k=%d unsupported", n, k);
    if (rows <= 0) return 0;
    static const int cl_min = [] { const char *e = getenv("APUS_TOPK_CLUSTER_MIN"); return e && e[0] ? atoi(e) : 16384; }();
    if (n >= cl_min) {                                  // long rows: a cluster of CTAs per row
        topk_stable_cl_kernel<<<rows * TOPK_CL, TOPK_THREADS, 0, st>>>(scores, n, k, idx, dyn_pos, ratio, chunk_pos0, rows_per_pos);
        APUS_LAUNCHED();
        return 0;
    }
    launch_k(topk_stable_kernel, rows, TOPK_THREADS, 0, st, scores, n, k, idx, dyn_pos, ratio, chunk_pos0, rows_per_pos);
    APUS_LAUNCHED();
    return 0;
}

// ---- sparse attention --------------------------------------------------------------
//
// Reference c/attn.h:1193-1326.  Per (token t, head h): ids < 0 are dropped
// (order kept); s_j = (q . kv_j) * scale; p_j = bf16(exp(s_j - max_j s));
// o = sum_j p_j * kv_j accumulated in j order; o = bf16(o / (sum_j p_j +
// exp(sink_h - max))); no ids -> zeros.  K and V are the same vector; ids
// below `na` index kv_a, the rest kv_b (offset by na).
//
// Kernel 1 (scores): one thread per (head, id) computes the full d-long dot in
// the reference's k order with separate rounded multiply and add, from a
// shared-memory tile of 32 gathered KV rows shared by 16 heads.
// Kernel 2 (softmax + PV): one CTA per (token, head); p_j in shared memory,
// each thread owns two adjacent output channels and walks j in order.
template <bool BF16>
__device__ __forceinline__ float2 kv_pair(const void *base, size_t row, int d, int k2) {
    if (BF16) {
        uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(
            reinterpret_cast<const uint16_t *>(base) + row * d) + k2);
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
    return __ldg(reinterpret_cast<const float2 *>(reinterpret_cast<const float *>(base) + row * d) + k2);
}

#define SA_IDS 32
#define SA_HEADS 16

template <bool BF16>
__global__ void __launch_bounds__(SA_IDS * SA_HEADS)
sparse_scores_kernel(const float *__restrict__ q, int h, int d, const int32_t *__restrict__ ids,
                     const int *__restrict__ ns, int idxw, float scale, const void *kv_a,
                     int64_t na, const void *kv_b, float *__restrict__ sc, size_t a_stride,
                     size_t b_stride, int seq_mod) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ float sm[];
    const int t = blockIdx.z, hb = blockIdx.y, tile = blockIdx.x;
    const int own = seq_mod > 0 ? t % seq_mod : t;         // whose caches: rows of a chunk are time-major
    kv_a = reinterpret_cast<const char *>(kv_a) + (size_t)own * a_stride;
    kv_b = reinterpret_cast<const char *>(kv_b) + (size_t)own * b_stride;
    const int n = ns[t];
    if (tile * SA_IDS >= n) return;
    const int pitch = d + 1;
    float *s_kv = sm;                          // [SA_IDS][d+1]
    float *s_q = sm + SA_IDS * pitch;          // [SA_HEADS][d]
    const int tid = threadIdx.x;
    const int32_t *idr = ids + (size_t)t * idxw + tile * SA_IDS;
    const int cnt = min(SA_IDS, n - tile * SA_IDS);
    for (int i = tid; i < SA_IDS * (d / 2); i += blockDim.x) {
        int r = i / (d / 2), k2 = i - r * (d / 2);
        float2 v = make_float2(0.f, 0.f);
        if (r < cnt) {
            int32_t id = idr[r];
            v = id < na ? kv_pair<BF16>(kv_a, (size_t)id, d, k2)
                        : kv_pair<BF16>(kv_b, (size_t)(id - na), d, k2);
        }
        s_kv[r * pitch + 2 * k2] = v.x;
        s_kv[r * pitch + 2 * k2 + 1] = v.y;
    }
    for (int i = tid; i < SA_HEADS * d; i += blockDim.x) {
        int hh = i / d, k = i - hh * d;
        int head = hb * SA_HEADS + hh;
        s_q[i] = head < h ? q[((size_t)t * h + head) * d + k] : 0.f;
    }
    __syncthreads();
    const int j = tid & 31, hh = tid >> 5;
    const int head = hb * SA_HEADS + hh;
    if (j >= cnt || head >= h) return;
    const float *kvr = s_kv + j * pitch, *qr = s_q + hh * d;
    float dot = 0.f;
#pragma unroll 8
    for (int k = 0; k < d; k++) dot = __fadd_rn(dot, __fmul_rn(qr[k], kvr[k]));
    sc[((size_t)t * h + head) * idxw + tile * SA_IDS + j] = __fmul_rn(dot, scale);
}

template <bool BF16>
__global__ void __launch_bounds__(256)
sparse_pv_kernel(const float *__restrict__ sc, const float *__restrict__ sink, int h, int d,
                 const int32_t *__restrict__ ids, const int *__restrict__ ns, int idxw,
                 const void *kv_a, int64_t na, const void *kv_b, float *__restrict__ o, size_t a_stride,
                 size_t b_stride, int seq_mod) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ float s_p[];             // [idxw]
    __shared__ float red[32];
    __shared__ float s_mx, s_sum;
    const int t = blockIdx.y, head = blockIdx.x, tid = threadIdx.x;
    const int own = seq_mod > 0 ? t % seq_mod : t;
    kv_a = reinterpret_cast<const char *>(kv_a) + (size_t)own * a_stride;
    kv_b = reinterpret_cast<const char *>(kv_b) + (size_t)own * b_stride;
    const int n = ns[t];
    float *ov = o + ((size_t)t * h + head) * d;
    if (n == 0) {
        for (int k = tid; k < d; k += blockDim.x) ov[k] = 0.f;
        return;
    }
    const float *sr = sc + ((size_t)t * h + head) * idxw;
    float mx = -INFINITY;
    for (int j = tid; j < n; j += blockDim.x) mx = fmaxf(mx, sr[j]);
    mx = warp_max(mx);
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) {
        float v = tid < (blockDim.x >> 5) ? red[tid] : -INFINITY;
        v = warp_max(v);
        if (tid == 0) s_mx = v;
    }
    __syncthreads();
    mx = s_mx;
    for (int j = tid; j < n; j += blockDim.x) s_p[j] = bf16_round(exp_rn(__fsub_rn(sr[j], mx)));
    __syncthreads();
    if (tid == 0) {
        float sum = 0.f;
        if (n <= 1024) { for (int j = 0; j < n; j++) sum = __fadd_rn(sum, s_p[j]); s_sum = sum; }
    }
    if (n > 1024) {                            // long HCA rows: tree sum
        float part = 0.f;
        for (int j = tid; j < n; j += blockDim.x) part += s_p[j];
        part = warp_sum(part);
        __syncthreads();
        if ((tid & 31) == 0) red[tid >> 5] = part;
        __syncthreads();
        if (tid == 0) {
            float sum = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); w++) sum += red[w];
            s_sum = sum;
        }
    }
    __syncthreads();
    const float den = __fadd_rn(s_sum, exp_rn(__fsub_rn(sink[head], mx)));
    const int32_t *idr = ids + (size_t)t * idxw;
    for (int k2 = tid; k2 < d / 2; k2 += blockDim.x) {
        float a0 = 0.f, a1 = 0.f;
        for (int j = 0; j < n; j++) {
            int32_t id = idr[j];
            float2 v = id < na ? kv_pair<BF16>(kv_a, (size_t)id, d, k2)
                               : kv_pair<BF16>(kv_b, (size_t)(id - na), d, k2);
            float p = s_p[j];
            a0 = __fadd_rn(a0, __fmul_rn(p, v.x));
            a1 = __fadd_rn(a1, __fmul_rn(p, v.y));
        }
        ov[2 * k2] = bf16_round(__fdiv_rn(a0, den));
        ov[2 * k2 + 1] = bf16_round(__fdiv_rn(a1, den));
    }
}

// ---- the same two steps, register-tiled ---------------------------------------------------------
// Same arithmetic, same order, same bits as the two kernels above; what changes is how often a
// number is fetched per flop.
//
// Scores: a warp owns a tile of 16 heads x 32 candidates and walks k in chunks of 64 staged in shared
// memory TRANSPOSED (q chunk [k][16 heads], KV chunk [k][32 ids], pitch 36 words so the 16-byte
// stores of four gathered rows at one k do not collide); a lane owns 4 heads x 4 candidates, so one
// k costs it two 16-byte shared loads for 16 multiply-add pairs -- the kernel is bound by the FP32
// pipes (its floor: every (head, candidate) dot is 512 dependent multiply/add pairs), where the
// kernel above is bound by shared-memory loads at one 4-byte load per flop.
// softmax: max, p_j = bf16(exp(s_j - max)) written over the scores, denominator per (row, head).
// P.V: a CTA owns HG heads of a row; a thread owns one channel pair for all HG heads (accumulators
// in registers), so a gathered KV row is fetched once per HG heads instead of once per head; the
// probabilities of a chunk of candidates sit transposed in shared memory ([j][HG], one 16-byte
// broadcast load per 4 heads).
#define SS_ROWB 128                       // bytes of a KV row staged per chunk: 64 BF16 or 32 f32 values of k
#define SS_PITCHW 36                      // row pitch of the staged tile in 32-bit words (128 B + 16 B pad)

__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int sz = valid ? 16 : 0;        // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(sz) : "memory");
}

// Scores.  A warp owns 16 heads x 8 NB candidates; lane = (hg, jg) owns heads 4hg..4hg+3 and candidates
// jg, jg+8, ... (NB of them: 4 where the launch fills the GPU anyway; 1 for the few rows of a small step,
// whose duration is one warp's instruction stream -- a quarter of it per warp and four times the warps).  The warp's 32 gathered rows are staged 128 bytes of k at a time in their
// natural layout by 16-byte cp.async (two buffers: the next chunk is in flight while this one is
// consumed); with a pitch of 36 words the eight rows the lanes of a load touch fall into different
// banks.  The q chunk is shared by the CTA's warps, transposed ([k][16 heads]: one 16-byte load gives
// a lane its four heads).  Per k a lane issues 5 shared loads for 16 multiply/add pairs.
template <bool BF16, int W, int NB>
__global__ void __launch_bounds__(32 * W)
sparse_scores_tile_kernel(const float *__restrict__ q, int h, int d, const int32_t *__restrict__ ids,
                          const int *__restrict__ ns, int idxw, float scale, const void *kv_a, int64_t na,
                          const void *kv_b, float *__restrict__ sc, size_t a_stride, size_t b_stride, int seq_mod) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    constexpr int KC = BF16 ? 64 : 32;                         // k values per chunk
    extern __shared__ __align__(16) unsigned char ss_raw[];
    float (*s_q)[KC][16] = reinterpret_cast<float (*)[KC][16]>(ss_raw);                       // [2][KC][16]
    constexpr int TJ = 8 * NB;                                  // candidates of a warp's tile
    uint32_t (*s_kv)[2][TJ][SS_PITCHW] =
        reinterpret_cast<uint32_t (*)[2][TJ][SS_PITCHW]>(ss_raw + 2 * KC * 16 * 4);           // [W][2][TJ][pitch]
    const int t = blockIdx.z, hb = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n = ns[t];
    const int j0 = ((int)blockIdx.x * W + warp) * TJ;          // first candidate of this warp's tile
    if ((int)blockIdx.x * W * TJ >= n) return;                  // whole CTA past the row
    const int own = seq_mod > 0 ? t % seq_mod : t;
    const size_t esz = BF16 ? 2 : 4;
    // lane u-th copy of a chunk: row (lane + 32u) / 8, 16-byte segment (lane + 32u) % 8; the four rows a
    // lane copies from are fixed, so their base pointers stay in registers
    const char *rowp[2 * NB];
    const char *dummy = reinterpret_cast<const char *>(kv_a ? kv_a : kv_b);
#pragma unroll
    for (int u = 0; u < 2 * NB; u++) {
        const int r = (lane + 32 * u) >> 3, j = j0 + r;
        const char *ptr = nullptr;
        if (j < n) {
            const int32_t id = ids[(size_t)t * idxw + j];
            ptr = id < na ? reinterpret_cast<const char *>(kv_a) + (size_t)own * a_stride + (size_t)id * d * esz
                          : reinterpret_cast<const char *>(kv_b) + (size_t)own * b_stride + (size_t)(id - na) * d * esz;
        }
        rowp[u] = ptr;
    }
    const bool live = j0 < n;                                   // warps past the row still help with the q chunk
    const int hg = lane & 3, jg = lane >> 2;
    const int nchunk = d / KC;
    // the q chunk of the NEXT step travels through registers: loaded before this step's arithmetic,
    // stored (transposed) after it, so its latency hides behind the multiply/adds
    constexpr int QN = (KC * 16 + 32 * W - 1) / (32 * W);
    float qreg[QN];
    auto q_load = [&](int c) {
#pragma unroll
        for (int u = 0; u < QN; u++) {
            const int i = tid + 32 * W * u, hh = i / KC, kk = i - hh * KC, head = hb * 16 + hh;
            qreg[u] = (i < KC * 16 && head < h) ? q[((size_t)t * h + head) * d + c * KC + kk] : 0.f;
        }
    };
    auto q_store = [&](int buf) {
#pragma unroll
        for (int u = 0; u < QN; u++) {
            const int i = tid + 32 * W * u, hh = i / KC, kk = i - hh * KC;
            if (i < KC * 16) s_q[buf][kk][hh] = qreg[u];
        }
    };
    auto kv_stage = [&](int c, int buf) {
        if (live) {
#pragma unroll
            for (int u = 0; u < 2 * NB; u++) {
                const int i = lane + 32 * u, r = i >> 3, seg = i & 7;
                cp_async16(&s_kv[warp][buf][r][seg * 4], rowp[u] ? rowp[u] + (size_t)c * SS_ROWB + seg * 16 : dummy, rowp[u] != nullptr);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc[4][NB];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < NB; b++) acc[a][b] = 0.f;
    kv_stage(0, 0);
    if (nchunk > 1) kv_stage(1, 1);
    q_load(0);
    q_store(0);
    for (int c = 0; c < nchunk; c++) {
        const int buf = c & 1;
        if (c + 1 < nchunk) {
            q_load(c + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                                        // chunk c (q and the warp's rows) is visible
        if (live) {
            if (BF16) {
#pragma unroll 4
                for (int k2 = 0; k2 < KC / 2; k2++) {           // one 32-bit word holds k = 2 k2 and 2 k2 + 1
                    const float4 qa = *reinterpret_cast<const float4 *>(&s_q[buf][2 * k2][4 * hg]);
                    const float4 qb = *reinterpret_cast<const float4 *>(&s_q[buf][2 * k2 + 1][4 * hg]);
                    const float q0[4] = {qa.x, qa.y, qa.z, qa.w}, q1[4] = {qb.x, qb.y, qb.z, qb.w};
                    float k0v[NB], k1v[NB];
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const uint32_t w = s_kv[warp][buf][jg + 8 * b][k2];
                        k0v[b] = __uint_as_float(w << 16);
                        k1v[b] = __uint_as_float(w & 0xffff0000u);
                    }
#pragma unroll
                    for (int a = 0; a < 4; a++)
#pragma unroll
                        for (int b = 0; b < NB; b++) acc[a][b] = __fadd_rn(acc[a][b], __fmul_rn(q0[a], k0v[b]));
#pragma unroll
                    for (int a = 0; a < 4; a++)
#pragma unroll
                        for (int b = 0; b < NB; b++) acc[a][b] = __fadd_rn(acc[a][b], __fmul_rn(q1[a], k1v[b]));
                }
            } else {
#pragma unroll 8
                for (int kk = 0; kk < KC; kk++) {
                    const float4 q4 = *reinterpret_cast<const float4 *>(&s_q[buf][kk][4 * hg]);
                    const float qa[4] = {q4.x, q4.y, q4.z, q4.w};
                    float kb[NB];
#pragma unroll
                    for (int b = 0; b < NB; b++) kb[b] = __uint_as_float(s_kv[warp][buf][jg + 8 * b][kk]);
#pragma unroll
                    for (int a = 0; a < 4; a++)
#pragma unroll
                        for (int b = 0; b < NB; b++) acc[a][b] = __fadd_rn(acc[a][b], __fmul_rn(qa[a], kb[b]));
                }
            }
        }
        if (c + 1 < nchunk) q_store(buf ^ 1);                   // read last at step c - 1, behind that step's barrier
        __syncthreads();                                        // this step's buffers are free again
        if (c + 2 < nchunk) kv_stage(c + 2, buf);
    }
    if (!live) return;
#pragma unroll
    for (int a = 0; a < 4; a++) {
        const int head = hb * 16 + 4 * hg + a;
        if (head >= h) continue;
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int j = j0 + jg + 8 * b;
            if (j < n) sc[((size_t)t * h + head) * idxw + j] = __fmul_rn(acc[a][b], scale);
        }
    }
}

// max, p over the scores, the denominator sum_j p_j + exp(sink - max): the sums in the order of
// sparse_pv_kernel (one accumulator for n <= 1024, the strided tree above it)
__global__ void __launch_bounds__(256)
sparse_softmax_kernel(float *__restrict__ sc, const float *__restrict__ sink, int h, const int *__restrict__ ns, int idxw,
                      float *__restrict__ den) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    extern __shared__ float s_p[];             // [idxw]
    __shared__ float red[32];
    __shared__ float s_mx, s_sum;
    const int t = blockIdx.y, head = blockIdx.x, tid = threadIdx.x;
    const int n = ns[t];
    if (n == 0) return;
    float *sr = sc + ((size_t)t * h + head) * idxw;
    float mx = -INFINITY;
    for (int j = tid; j < n; j += blockDim.x) mx = fmaxf(mx, sr[j]);
    mx = warp_max(mx);
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) {
        float v = tid < (blockDim.x >> 5) ? red[tid] : -INFINITY;
        v = warp_max(v);
        if (tid == 0) s_mx = v;
    }
    __syncthreads();
    mx = s_mx;
    for (int j = tid; j < n; j += blockDim.x) {
        const float p = bf16_round(exp_rn(__fsub_rn(sr[j], mx)));
        s_p[j] = p;
        sr[j] = p;
    }
    __syncthreads();
    if (tid == 0 && n <= 1024) {
        float sum = 0.f;
        for (int j = 0; j < n; j++) sum = __fadd_rn(sum, s_p[j]);
        s_sum = sum;
    }
    if (n > 1024) {                            // long rows: tree sum
        float part = 0.f;
        for (int j = tid; j < n; j += blockDim.x) part += s_p[j];
        part = warp_sum(part);
        __syncthreads();
        if ((tid & 31) == 0) red[tid >> 5] = part;
        __syncthreads();
        if (tid == 0) {
            float sum = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); w++) sum += red[w];
            s_sum = sum;
        }
    }
    __syncthreads();
    if (tid == 0) den[(size_t)t * h + head] = __fadd_rn(s_sum, exp_rn(__fsub_rn(sink[head], mx)));
}

#define PV_JC 128
template <bool BF16, int HG>
__global__ void __launch_bounds__(256)
sparse_pv_tile_kernel(const float *__restrict__ p, const float *__restrict__ den, int h, int d,
                      const int32_t *__restrict__ ids, const int *__restrict__ ns, int idxw, const void *kv_a, int64_t na,
                      const void *kv_b, float *__restrict__ o, size_t a_stride, size_t b_stride, int seq_mod, const SaRope rope) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    __shared__ __align__(16) float s_p[PV_JC][HG];
    __shared__ int32_t s_id[PV_JC];
    const int t = blockIdx.y, h0 = (int)blockIdx.x * HG, tid = threadIdx.x;
    const int own = seq_mod > 0 ? t % seq_mod : t;
    kv_a = reinterpret_cast<const char *>(kv_a) + (size_t)own * a_stride;
    kv_b = reinterpret_cast<const char *>(kv_b) + (size_t)own * b_stride;
    const int n = ns[t];
    const int32_t *idr = ids + (size_t)t * idxw;
    for (int c0 = 0; c0 < d / 2; c0 += 256) {
        const int k2 = c0 + tid;
        const bool on = k2 < d / 2;
        float a0[HG], a1[HG];
#pragma unroll
        for (int a = 0; a < HG; a++) a0[a] = a1[a] = 0.f;
        for (int j0 = 0; j0 < n; j0 += PV_JC) {
            const int cnt = min(PV_JC, n - j0);
            __syncthreads();
            for (int i = tid; i < PV_JC * HG; i += 256) {
                const int a = i / PV_JC, jj = i - a * PV_JC;
                s_p[jj][a] = (jj < cnt && h0 + a < h) ? p[((size_t)t * h + h0 + a) * idxw + j0 + jj] : 0.f;
            }
            for (int i = tid; i < cnt; i += 256) s_id[i] = idr[j0 + i];
            __syncthreads();
            if (on) {
                // LB gathered rows in flight per thread: the rows come from L2 / HBM with nothing else to
                // hide their latency behind (few heads per CTA: little arithmetic per row, so more rows)
                constexpr int LB = HG >= 16 ? 16 : 32;
                for (int jb = 0; jb < cnt; jb += LB) {
                    float2 v[LB];
#pragma unroll
                    for (int u = 0; u < LB; u++) {
                        const int jj = jb + u < cnt ? jb + u : cnt - 1;
                        const int32_t id = s_id[jj];
                        v[u] = id < na ? kv_pair<BF16>(kv_a, (size_t)id, d, k2) : kv_pair<BF16>(kv_b, (size_t)(id - na), d, k2);
                    }
#pragma unroll
                    for (int u = 0; u < LB; u++) {
                        if (jb + u >= cnt) break;
#pragma unroll
                        for (int m = 0; m < HG / 4; m++) {
                            const float4 p4 = *reinterpret_cast<const float4 *>(&s_p[jb + u][4 * m]);
                            const float pa[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                a0[4 * m + e] = __fadd_rn(a0[4 * m + e], __fmul_rn(pa[e], v[u].x));
                                a1[4 * m + e] = __fadd_rn(a1[4 * m + e], __fmul_rn(pa[e], v[u].y));
                            }
                        }
                    }
                }
            }
        }
        if (on) {
            // a thread holds one (even, odd) pair of every head row: the pairs of the rotated tail are
            // turned back here (the operations of the row kernel, c/attn.h:290-299 with -sin)
            const int ri = rope.cs ? k2 - (d - rope.rd) / 2 : -1;
            float co = 1.f, si = 0.f;
            if (ri >= 0) {
                const float *c = rope.cs + (rope.pos ? (size_t)*rope.pos * rope.rd : 0);
                co = c[ri]; si = -c[rope.rd / 2 + ri];
            }
#pragma unroll
            for (int a = 0; a < HG; a++) {
                if (h0 + a >= h) continue;
                float *ov = o + ((size_t)t * h + h0 + a) * d;
                if (n == 0) { ov[2 * k2] = 0.f; ov[2 * k2 + 1] = 0.f; continue; }
                const float dn = den[(size_t)t * h + h0 + a];
                float x1 = bf16_round(__fdiv_rn(a0[a], dn)), x2 = bf16_round(__fdiv_rn(a1[a], dn));
                if (ri >= 0) {
                    const float y1 = bf16_round(__fsub_rn(__fmul_rn(x1, co), __fmul_rn(x2, si)));
                    const float y2 = bf16_round(__fadd_rn(__fmul_rn(x1, si), __fmul_rn(x2, co)));
                    x1 = y1; x2 = y2;
                }
                ov[2 * k2] = x1;
                ov[2 * k2 + 1] = x2;
            }
        }
    }
}

// P.V for the few (row, head group)s of a small step.  There the kernel above is a chain of load latencies:
// a thread fetches a batch of gathered rows into registers, waits, accumulates, fetches the next -- and one
// or two warps per SM keep too few bytes in flight to pull the rows out of L2 any faster.  Here a CTA owns
// 4 heads x PVS_NP channel pairs of a row and stages the row segments of PVS_T candidates at a time in
// shared memory with 16-byte asynchronous copies, two tiles in flight while a third is consumed (the
// probabilities travel the same way, 4 bytes each), so the copies of the whole row are issued back to
// back and the accumulation reads shared memory.  Same products, same order of adds, same bits.
#define PVS_NS 3
// HG heads x NP channel pairs per CTA (NP threads), T candidates per staged tile
template <bool BF16, int HG, int NP, int T>
__global__ void __launch_bounds__(NP)
sparse_pv_stage_kernel(const float *__restrict__ p, const float *__restrict__ den, int h, int d,
                       const int32_t *__restrict__ ids, const int *__restrict__ ns, int idxw, const void *kv_a, int64_t na,
                       const void *kv_b, float *__restrict__ o, size_t a_stride, size_t b_stride, int seq_mod, const SaRope rope) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    constexpr int ROWB = NP * (BF16 ? 4 : 8);              // bytes of a row's segment
    constexpr int CPR = ROWB / 16;                             // 16-byte copies per row
    constexpr int STAGE = T * ROWB + T * HG * 4;       // rows, then the tile's probabilities [T][HG]
    extern __shared__ __align__(16) unsigned char pvs[];
    const int t = blockIdx.y, h0 = (int)blockIdx.x * HG, tid = threadIdx.x;
    const int k2 = (int)blockIdx.z * NP + tid;             // this thread's channel pair
    const int own = seq_mod > 0 ? t % seq_mod : t;
    const size_t esz = BF16 ? 2 : 4;
    const char *base_a = reinterpret_cast<const char *>(kv_a) + (size_t)own * a_stride + (size_t)blockIdx.z * ROWB;
    const char *base_b = reinterpret_cast<const char *>(kv_b) + (size_t)own * b_stride + (size_t)blockIdx.z * ROWB;
    const int n = ns[t];
    const int32_t *idr = ids + (size_t)t * idxw;
    const int ntile = (n + T - 1) / T;
    auto stage = [&](int c) {
        if (c < ntile) {
            unsigned char *st = pvs + (size_t)(c % PVS_NS) * STAGE;
            const int j0 = c * T, cnt = min(T, n - j0);
#pragma unroll 4
            for (int i = tid; i < T * CPR; i += NP) {
                const int r = i / CPR, seg = i - r * CPR;
                if (r < cnt) {
                    const int32_t id = idr[j0 + r];
                    const char *src = id < na ? base_a + (size_t)id * d * esz : base_b + (size_t)(id - na) * d * esz;
                    cp_async16(st + (size_t)r * ROWB + seg * 16, src + seg * 16, true);
                }
            }
            for (int i = tid; i < T * HG; i += NP) {
                const int r = i / HG, a = i - r * HG;
                if (r < cnt && h0 + a < h) {
                    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(st + T * ROWB + i * 4);
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(p + ((size_t)t * h + h0 + a) * idxw + j0 + r) : "memory");
                } else {
                    *reinterpret_cast<float *>(st + T * ROWB + i * 4) = 0.f;
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float a0[HG], a1[HG];
#pragma unroll
    for (int a = 0; a < HG; a++) a0[a] = a1[a] = 0.f;
    stage(0);
    stage(1);
    for (int c = 0; c < ntile; c++) {
        stage(c + 2);                                          // its buffer was consumed at step c - 1, behind that step's barrier
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        __syncthreads();                                       // tile c of every thread has landed
        const unsigned char *st = pvs + (size_t)(c % PVS_NS) * STAGE;
        const float4 *sp = reinterpret_cast<const float4 *>(st + T * ROWB);
        const int cnt = min(T, n - c * T);
#pragma unroll 4
        for (int j = 0; j < cnt; j++) {
            float2 v;
            if (BF16) {
                const uint32_t w = *reinterpret_cast<const uint32_t *>(st + (size_t)j * ROWB + tid * 4);
                v = make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
            } else {
                v = *reinterpret_cast<const float2 *>(st + (size_t)j * ROWB + tid * 8);
            }
#pragma unroll
            for (int m = 0; m < HG / 4; m++) {
                const float4 p4 = sp[j * (HG / 4) + m];
                const float pa[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    a0[4 * m + e] = __fadd_rn(a0[4 * m + e], __fmul_rn(pa[e], v.x));
                    a1[4 * m + e] = __fadd_rn(a1[4 * m + e], __fmul_rn(pa[e], v.y));
                }
            }
        }
        __syncthreads();                                       // this tile's buffer is free again
    }
    const int ri = rope.cs ? k2 - (d - rope.rd) / 2 : -1;
    float co = 1.f, si = 0.f;
    if (ri >= 0) {
        const float *c = rope.cs + (rope.pos ? (size_t)*rope.pos * rope.rd : 0);
        co = c[ri]; si = -c[rope.rd / 2 + ri];
    }
#pragma unroll
    for (int a = 0; a < HG; a++) {
        if (h0 + a >= h) continue;
        float *ov = o + ((size_t)t * h + h0 + a) * d;
        if (n == 0) { ov[2 * k2] = 0.f; ov[2 * k2 + 1] = 0.f; continue; }
        const float dn = den[(size_t)t * h + h0 + a];
        float x1 = bf16_round(__fdiv_rn(a0[a], dn)), x2 = bf16_round(__fdiv_rn(a1[a], dn));
        if (ri >= 0) {
            const float y1 = bf16_round(__fsub_rn(__fmul_rn(x1, co), __fmul_rn(x2, si)));
            const float y2 = bf16_round(__fadd_rn(__fmul_rn(x1, si), __fmul_rn(x2, co)));
            x1 = y1; x2 = y2;
        }
        ov[2 * k2] = x1;
        ov[2 * k2 + 1] = x2;
    }
}

// Drops negative ids keeping order (reference c/attn.h:1314-1321).
__global__ void compact_ids_kernel(const int32_t *__restrict__ idxs, int idxw,
                                   int32_t *__restrict__ out, int *__restrict__ ns) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    __shared__ int s_base;
    __shared__ int w_cnt[32];
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_base = 0;
    __syncthreads();
    for (int base = 0; base < idxw; base += blockDim.x) {
        int i = base + tid;
        int32_t v = i < idxw ? idxs[(size_t)t * idxw + i] : -1;
        bool keep = v >= 0;
        unsigned m = __ballot_sync(0xffffffffu, keep);
        if (lane == 0) w_cnt[warp] = __popc(m);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) {
            if (w < warp) before += w_cnt[w];
            total += w_cnt[w];
        }
        if (keep) out[(size_t)t * idxw + s_base + before + __popc(m & ((1u << lane) - 1u))] = v;
        __syncthreads();
        if (tid == 0) s_base += total;
        __syncthreads();
    }
    if (tid == 0) ns[t] = s_base;
}

// Scores / compacted ids between the kernels of a call: the caller's scratch (a model
// object keeps its own), else one buffer of the library, which only grows.
static void *g_scratch = nullptr;
static size_t g_scratch_cap = 0;
static void *ensure_scratch(size_t bytes) {
    if (bytes <= g_scratch_cap) return g_scratch;
    if (g_scratch) { cudaDeviceSynchronize(); cudaFree(g_scratch); }
    g_scratch = nullptr; g_scratch_cap = 0;
    if (cudaMalloc(&g_scratch, bytes) != cudaSuccess) {
        set_error("sparse_attn: scratch of %zu bytes", bytes);
        g_scratch = nullptr;
        return nullptr;
    }
    g_scratch_cap = bytes;
    return g_scratch;
}
size_t sparse_attn_scratch(int h, int idxw, int s) {
    const size_t sc_bytes = (size_t)s * h * idxw * sizeof(float), ids_bytes = (size_t)s * idxw * sizeof(int32_t);
    const size_t ns_off = (sc_bytes + ids_bytes + 255) & ~(size_t)255;
    return ((ns_off + (size_t)s * sizeof(int) + 255) & ~(size_t)255) + (size_t)s * h * sizeof(float);
}

int sparse_attn(const float *q, const float *sink, int h, int d,
                const int32_t *idxs, int idxw, int s, float scale,
                const void *kv_a, int64_t na, const void *kv_b, int64_t nb,
                int kv_bf16, float *o, cudaStream_t st, long long kv_a_stride, long long kv_b_stride,
                void *callers, size_t callers_cap, int seq_mod, bool ids_ready, const SaRope *rope) {
    (void)nb;
    const size_t esz = kv_bf16 ? 2 : 4;
    const size_t sa = (size_t)kv_a_stride * esz, sb = (size_t)kv_b_stride * esz;
    APUS_REQUIRE(d % 2 == 0 && d <= 1024, "sparse_attn: d=%d unsupported", d);
    APUS_REQUIRE((size_t)idxw * sizeof(float) <= 160 * 1024, "sparse_attn: idxw=%d too wide", idxw);
    if (s <= 0 || idxw <= 0) return 0;
    size_t sc_bytes = (size_t)s * h * idxw * sizeof(float);
    size_t ids_bytes = (size_t)s * idxw * sizeof(int32_t);
    size_t ns_off = (sc_bytes + ids_bytes + 255) & ~(size_t)255;
    const size_t den_off = (ns_off + (size_t)s * sizeof(int) + 255) & ~(size_t)255;
    const size_t need = den_off + (size_t)s * h * sizeof(float);
    APUS_REQUIRE(!callers || need <= callers_cap, "sparse_attn: scratch of %zu bytes given, %zu needed", callers_cap, need);
    void *scratch = callers ? callers : ensure_scratch(need);
    if (!scratch) return 1;
    float *sc = (float *)scratch;
    int32_t *ids = (int32_t *)((char *)scratch + sc_bytes);
    int *ns = (int *)((char *)scratch + ns_off);
    float *den = (float *)((char *)scratch + den_off);
    APUS_REQUIRE(!ids_ready || callers, "sparse_attn: compacted ids need the caller's scratch");
    if (!ids_ready) {
        launch_k(compact_ids_kernel, s, 256, 0, st, idxs, idxw, ids, ns);
        APUS_LAUNCHED();
    }
    const SaRope no_rope = {nullptr, nullptr, 0};
    static const int tiled = [] { const char *e = getenv("APUS_ATTN_TILED"); return !(e && e[0] == '0'); }();
    if (tiled && d % 64 == 0) {
        // register-tiled kernels: enough CTAs to cover the SMs decide the tile sizes
        const long long wide = (long long)ceil_div(idxw, 256) * ceil_div(h, 16) * s;
        const size_t sm2 = (size_t)idxw * sizeof(float);
        if (ensure_dyn_smem((const void *)sparse_softmax_kernel, sm2)) return 1;
        const int hgs = h >= 16 && (long long)s * ceil_div(h, 16) >= 96 ? 16 : 4;
        const size_t kc = kv_bf16 ? 64 : 32;
        const size_t ss8 = 2 * kc * 16 * 4 + 8 * (2 * 32 * SS_PITCHW * 4), ss2 = 2 * kc * 16 * 4 + 2 * (2 * 32 * SS_PITCHW * 4);
        const size_t ss1 = 2 * kc * 16 * 4 + 2 * (2 * 8 * SS_PITCHW * 4);
        // a small step (few rows, few candidates): 8-candidate tiles, so that no warp walks more than a quarter
        static const bool small_on = [] { const char *e = getenv("APUS_ATTN_SMALL"); return !(e && e[0] == '0'); }();
        const bool narrow = small_on && (long long)ceil_div(idxw, 32) * ceil_div(h, 16) * s <= 296;
        // P.V from staged rows where the row splits into whole CTAs' worth of channel pairs: 16 heads x 128 pairs
        // per CTA when there are (row, 16 heads) groups enough to fill the GPU, else 4 heads x 64 pairs
        static const bool stage_on = [] { const char *e = getenv("APUS_ATTN_STAGE"); return !(e && e[0] == '0'); }();
        const bool pv_stage = stage_on && d % 256 == 0;
        const size_t rowb = kv_bf16 ? 4 : 8;
        const size_t pvs4 = (size_t)PVS_NS * (64 * 64 * rowb + 64 * 4 * 4);
        const size_t pvs16 = (size_t)PVS_NS * ((kv_bf16 ? 64 : 32) * 128 * rowb + (kv_bf16 ? 64 : 32) * 16 * 4);
        if (pv_stage && (ensure_dyn_smem(kv_bf16 ? (const void *)sparse_pv_stage_kernel<true, 4, 64, 64>
                                                 : (const void *)sparse_pv_stage_kernel<false, 4, 64, 64>, pvs4) ||
                         ensure_dyn_smem(kv_bf16 ? (const void *)sparse_pv_stage_kernel<true, 16, 128, 64>
                                                 : (const void *)sparse_pv_stage_kernel<false, 16, 128, 32>, pvs16)))
            return 1;
        if (ensure_dyn_smem(kv_bf16 ? (const void *)sparse_scores_tile_kernel<true, 8, 4> : (const void *)sparse_scores_tile_kernel<false, 8, 4>, ss8))
            return 1;
#define APUS_SA_LAUNCH(BF)                                                                                              \
        do {                                                                                                            \
            if (wide >= 148) {                                                                                          \
                dim3 g((unsigned)ceil_div(idxw, 256), (unsigned)ceil_div(h, 16), (unsigned)s);                          \
                launch_k(sparse_scores_tile_kernel<BF, 8, 4>, g, 256, ss8, st, q, h, d, ids, ns, idxw, scale, kv_a, na, kv_b, sc,  \
                                                                   sa, sb, seq_mod);                                    \
            } else if (narrow) {                                                                                        \
                dim3 g((unsigned)ceil_div(idxw, 16), (unsigned)ceil_div(h, 16), (unsigned)s);                           \
                launch_k(sparse_scores_tile_kernel<BF, 2, 1>, g, 64, ss1, st, q, h, d, ids, ns, idxw, scale, kv_a, na, kv_b, sc,   \
                                                                  sa, sb, seq_mod);                                     \
            } else {                                                                                                    \
                dim3 g((unsigned)ceil_div(idxw, 64), (unsigned)ceil_div(h, 16), (unsigned)s);                           \
                launch_k(sparse_scores_tile_kernel<BF, 2, 4>, g, 64, ss2, st, q, h, d, ids, ns, idxw, scale, kv_a, na, kv_b, sc,   \
                                                                  sa, sb, seq_mod);                                     \
            }                                                                                                           \
            APUS_LAUNCHED();                                                                                            \
            launch_k(sparse_softmax_kernel, dim3((unsigned)h, (unsigned)s), 256, sm2, st, sc, sink, h, ns, idxw, den);       \
            APUS_LAUNCHED();                                                                                            \
            if (pv_stage && hgs == 16)                                                                                  \
                launch_k(sparse_pv_stage_kernel<BF, 16, 128, (BF ? 64 : 32)>,                                           \
                    dim3((unsigned)ceil_div(h, 16), (unsigned)s, (unsigned)(d / 2 / 128)), 128, pvs16, st,              \
                    sc, den, h, d, ids, ns, idxw, kv_a, na, kv_b, o, sa, sb, seq_mod, rope ? *rope : no_rope);          \
            else if (pv_stage)                                                                                          \
                launch_k(sparse_pv_stage_kernel<BF, 4, 64, 64>,                                                         \
                    dim3((unsigned)ceil_div(h, 4), (unsigned)s, (unsigned)(d / 2 / 64)), 64, pvs4, st,                  \
                    sc, den, h, d, ids, ns, idxw, kv_a, na, kv_b, o, sa, sb, seq_mod, rope ? *rope : no_rope);          \
            else if (hgs == 16)                                                                                         \
                launch_k(sparse_pv_tile_kernel<BF, 16>, dim3((unsigned)ceil_div(h, 16), (unsigned)s), 256, 0, st,             \
                    sc, den, h, d, ids, ns, idxw, kv_a, na, kv_b, o, sa, sb, seq_mod, rope ? *rope : no_rope);          \
            else                                                                                                        \
                launch_k(sparse_pv_tile_kernel<BF, 4>, dim3((unsigned)ceil_div(h, 4), (unsigned)s), 256, 0, st,               \
                    sc, den, h, d, ids, ns, idxw, kv_a, na, kv_b, o, sa, sb, seq_mod, rope ? *rope : no_rope);          \
            APUS_LAUNCHED();                                                                                            \
        } while (0)
        if (kv_bf16) APUS_SA_LAUNCH(true); else APUS_SA_LAUNCH(false);
#undef APUS_SA_LAUNCH
        return 0;
    }
    size_t sm1 = ((size_t)SA_IDS * (d + 1) + (size_t)SA_HEADS * d) * sizeof(float);
    dim3 g1((unsigned)ceil_div(idxw, SA_IDS), (unsigned)ceil_div(h, SA_HEADS), (unsigned)s);
    size_t sm2 = (size_t)idxw * sizeof(float);
    dim3 g2((unsigned)h, (unsigned)s);
    // each kernel's limit only ever grows (per device): a later call with a smaller size keeps the larger one
    if (ensure_dyn_smem(kv_bf16 ? (const void *)sparse_scores_kernel<true> : (const void *)sparse_scores_kernel<false>, sm1) ||
        ensure_dyn_smem(kv_bf16 ? (const void *)sparse_pv_kernel<true> : (const void *)sparse_pv_kernel<false>, sm2))
        return 1;
    if (kv_bf16) {
        launch_k(sparse_scores_kernel<true>, g1, SA_IDS * SA_HEADS, sm1, st, q, h, d, ids, ns, idxw, scale,
                                                                       kv_a, na, kv_b, sc, sa, sb, seq_mod);
        APUS_LAUNCHED();
        launch_k(sparse_pv_kernel<true>, g2, 256, sm2, st, sc, sink, h, d, ids, ns, idxw, kv_a, na, kv_b, o, sa, sb, seq_mod);
        APUS_LAUNCHED();
    } else {
        launch_k(sparse_scores_kernel<false>, g1, SA_IDS * SA_HEADS, sm1, st, q, h, d, ids, ns, idxw, scale,
                                                                        kv_a, na, kv_b, sc, sa, sb, seq_mod);
        APUS_LAUNCHED();
        launch_k(sparse_pv_kernel<false>, g2, 256, sm2, st, sc, sink, h, d, ids, ns, idxw, kv_a, na, kv_b, o, sa, sb, seq_mod);
        APUS_LAUNCHED();
    }
    if (rope && rope->cs) {                           // these kernels do not rotate: the row kernel does
        const RowDyn dyn = {rope->pos, 0, 0, 0};
        return row_ops(o, d, o, d, s * h, d, ROW_ROPE_INV, nullptr, 0.f, rope->rd, rope->cs, s * h, 0, st, rope->pos ? &dyn : nullptr);
    }
    return 0;
}

int sparse_attn_compact(const int32_t *idxs, int h, int idxw, int s, void *scratch, size_t scratch_cap, cudaStream_t st) {
    if (s <= 0 || idxw <= 0) return 0;
    APUS_REQUIRE(scratch && sparse_attn_scratch(h, idxw, s) <= scratch_cap, "sparse_attn_compact: scratch of %zu bytes given, %zu needed",
                 scratch_cap, sparse_attn_scratch(h, idxw, s));
    const size_t sc_bytes = (size_t)s * h * idxw * sizeof(float), ids_bytes = (size_t)s * idxw * sizeof(int32_t);
    const size_t ns_off = (sc_bytes + ids_bytes + 255) & ~(size_t)255;
    launch_k(compact_ids_kernel, s, 256, 0, st, idxs, idxw, (int32_t *)((char *)scratch + sc_bytes), (int *)((char *)scratch + ns_off));
    APUS_LAUNCHED();
    return 0;
}

}  // namespace apus
