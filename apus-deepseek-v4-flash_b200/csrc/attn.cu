// Stable top-k selection and index-gathered sparse attention.
#include <map>
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
        if (tid == 0) {
            unsigned need = s_need, acc = 0;
            int b = 255;
            for (; b > 0; b--) {
                if (acc + hist[b] >= need) break;
                acc += hist[b];
            }
            s_greater += acc;
            s_need = need - acc;
            s_prefix = prefix | ((unsigned)b << shift);
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
    const int lane = tid & 31, warp = tid >> 5;
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

int topk_stable(const float *scores, int n, int k, int32_t *idx, int rows,
                cudaStream_t st, const long long *dyn_pos, int ratio, long long chunk_pos0, int rows_per_pos) {
    APUS_REQUIRE(k >= 1 && (k <= n || dyn_pos || rows_per_pos > 0) && k <= TOPK_MAX_K, "topk: n=%d k=%d unsupported", n, k);
    if (rows <= 0) return 0;
    topk_stable_kernel<<<rows, TOPK_THREADS, 0, st>>>(scores, n, k, idx, dyn_pos, ratio, chunk_pos0, rows_per_pos);
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

// Drops negative ids keeping order (reference c/attn.h:1314-1321).
__global__ void compact_ids_kernel(const int32_t *__restrict__ idxs, int idxw,
                                   int32_t *__restrict__ out, int *__restrict__ ns) {
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
    return ((sc_bytes + ids_bytes + 255) & ~(size_t)255) + (size_t)s * sizeof(int);
}

int sparse_attn(const float *q, const float *sink, int h, int d,
                const int32_t *idxs, int idxw, int s, float scale,
                const void *kv_a, int64_t na, const void *kv_b, int64_t nb,
                int kv_bf16, float *o, cudaStream_t st, long long kv_a_stride, long long kv_b_stride,
                void *callers, size_t callers_cap, int seq_mod) {
    (void)nb;
    const size_t esz = kv_bf16 ? 2 : 4;
    const size_t sa = (size_t)kv_a_stride * esz, sb = (size_t)kv_b_stride * esz;
    APUS_REQUIRE(d % 2 == 0 && d <= 1024, "sparse_attn: d=%d unsupported", d);
    APUS_REQUIRE((size_t)idxw * sizeof(float) <= 160 * 1024, "sparse_attn: idxw=%d too wide", idxw);
    if (s <= 0 || idxw <= 0) return 0;
    size_t sc_bytes = (size_t)s * h * idxw * sizeof(float);
    size_t ids_bytes = (size_t)s * idxw * sizeof(int32_t);
    size_t ns_off = (sc_bytes + ids_bytes + 255) & ~(size_t)255;
    const size_t need = ns_off + (size_t)s * sizeof(int);
    APUS_REQUIRE(!callers || need <= callers_cap, "sparse_attn: scratch of %zu bytes given, %zu needed", callers_cap, need);
    void *scratch = callers ? callers : ensure_scratch(need);
    if (!scratch) return 1;
    float *sc = (float *)scratch;
    int32_t *ids = (int32_t *)((char *)scratch + sc_bytes);
    int *ns = (int *)((char *)scratch + ns_off);
    compact_ids_kernel<<<s, 256, 0, st>>>(idxs, idxw, ids, ns);
    APUS_LAUNCHED();
    size_t sm1 = ((size_t)SA_IDS * (d + 1) + (size_t)SA_HEADS * d) * sizeof(float);
    dim3 g1((unsigned)ceil_div(idxw, SA_IDS), (unsigned)ceil_div(h, SA_HEADS), (unsigned)s);
    size_t sm2 = (size_t)idxw * sizeof(float);
    dim3 g2((unsigned)h, (unsigned)s);
    // each kernel's limit only ever grows (per device): a later call with a smaller size keeps the larger one
    if (ensure_dyn_smem(kv_bf16 ? (const void *)sparse_scores_kernel<true> : (const void *)sparse_scores_kernel<false>, sm1) ||
        ensure_dyn_smem(kv_bf16 ? (const void *)sparse_pv_kernel<true> : (const void *)sparse_pv_kernel<false>, sm2))
        return 1;
    if (kv_bf16) {
        sparse_scores_kernel<true><<<g1, SA_IDS * SA_HEADS, sm1, st>>>(q, h, d, ids, ns, idxw, scale,
                                                                       kv_a, na, kv_b, sc, sa, sb, seq_mod);
        APUS_LAUNCHED();
        sparse_pv_kernel<true><<<g2, 256, sm2, st>>>(sc, sink, h, d, ids, ns, idxw, kv_a, na, kv_b, o, sa, sb, seq_mod);
        APUS_LAUNCHED();
    } else {
        sparse_scores_kernel<false><<<g1, SA_IDS * SA_HEADS, sm1, st>>>(q, h, d, ids, ns, idxw, scale,
                                                                        kv_a, na, kv_b, sc, sa, sb, seq_mod);
        APUS_LAUNCHED();
        sparse_pv_kernel<false><<<g2, 256, sm2, st>>>(sc, sink, h, d, ids, ns, idxw, kv_a, na, kv_b, o, sa, sb, seq_mod);
        APUS_LAUNCHED();
    }
    return 0;
}

}  // namespace apus
