// Temperature + nucleus (top-p) sampling and the splitmix64 stream on the device
// (reference c/sample.h:91-180): per row
//   p_i = (float)(expf((l_i - max) / temp) / sum)            (sum in double)
//   order the tokens by (p descending, index ascending)
//   keep token i of that order iff the mass before it is <= top_p
//   draw: first kept token whose renormalised inclusive mass exceeds u.
//
// The reference sorts all n probabilities.  Both walks over the sorted list
// ask the same question -- "which is the first token, in (p desc, index asc)
// order, whose inclusive prefix mass exceeds M?" -- and that is a WEIGHTED
// SELECTION, answered here without sorting: four radix passes over the
// order-preserving integer image of p, each building a 256-bin histogram of
// probability MASS under the prefix found so far, locate the value p* at which
// the running mass crosses M; the ties at p* are then counted in index order.
// Mass is accumulated as 2^-60 fixed point in 64-bit integers, so the sums are
// exact, associative and therefore deterministic whatever the order of the
// atomic adds (the reference's double sums differ from exact sums by ~1e-16,
// which can only matter for a u within that distance of a boundary).
// One CTA per row; ~9 sweeps over the row's probabilities (L2 resident).
#include "common.cuh"
#include "kernels.cuh"

namespace apus {

namespace {

constexpr int SMP_THREADS = 1024;
constexpr double SMP_ONE = 1152921504606846976.0;        // 2^60

__device__ __forceinline__ unsigned long long mass_of(float p) {
    return (unsigned long long)((double)p * SMP_ONE);     // exact: p has 24 significant bits, p <= 1
}

struct Sel {                 // answer of first_exceed
    int found;               // 0: the total mass does not exceed M
    unsigned key;            // integer image of p*
    unsigned long long above;// mass of the tokens with p > p*
    unsigned long long k;    // the k-th tie at p* (1-based, index order) is the token
    int token;
};

// First token, in (p desc, index asc) order, whose inclusive prefix mass exceeds M.
// All threads of the CTA call it; the result is valid in every thread.
__device__ Sel first_exceed(const float *p, int n, unsigned long long M,
                            unsigned long long *s_hist, unsigned *s_misc, int *s_cnt) {
    const int tid = threadIdx.x;
    unsigned prefix = 0;
    unsigned long long above = 0;
    Sel r;
    r.found = 1;
    for (int pass = 0; pass < 4; pass++) {
        const int shift = 24 - 8 * pass;
        const unsigned himask = pass ? (0xffffffffu << (shift + 8)) : 0u;
        for (int i = tid; i < 256; i += SMP_THREADS) s_hist[i] = 0ull;
        __syncthreads();
        for (int i = tid; i < n; i += SMP_THREADS) {
            const float v = p[i];
            const unsigned key = __float_as_uint(v);      // p >= 0: the bit pattern orders like the value
            if ((key & himask) == prefix) atomicAdd(&s_hist[(key >> shift) & 0xffu], mass_of(v));
        }
        __syncthreads();
        if (tid == 0) {
            unsigned long long acc = above;
            int b = 255;
            for (; b >= 0; b--) {
                if (acc + s_hist[b] > M) break;
                acc += s_hist[b];
            }
            s_misc[0] = (unsigned)(b < 0 ? 0xffffffffu : (unsigned)b);
            reinterpret_cast<unsigned long long *>(s_misc + 2)[0] = acc;
        }
        __syncthreads();
        const unsigned b = s_misc[0];
        if (b == 0xffffffffu) { r.found = 0; r.key = 0; r.above = 0; r.k = 0; r.token = -1; __syncthreads(); return r; }
        above = reinterpret_cast<unsigned long long *>(s_misc + 2)[0];
        prefix |= b << shift;
        __syncthreads();
    }
    // ties at p*: the k-th of them in index order crosses M
    const float pstar = __uint_as_float(prefix);
    const unsigned long long pm = mass_of(pstar);
    unsigned long long k = pm ? (M - above) / pm + 1 : 1;
    r.key = prefix; r.above = above; r.k = k;
    // thread t owns the contiguous index range [t*chunk, (t+1)*chunk)
    const int chunk = (n + SMP_THREADS - 1) / SMP_THREADS;
    const int lo = tid * chunk, hi = min(n, lo + chunk);
    int cnt = 0;
    for (int i = lo; i < hi; i++) cnt += __float_as_uint(p[i]) == prefix;
    s_cnt[tid] = cnt;
    __syncthreads();
    if (tid == 0) {                                        // exclusive scan; 1024 adds
        int run = 0;
        for (int t = 0; t < SMP_THREADS; t++) { int c = s_cnt[t]; s_cnt[t] = run; run += c; }
        s_misc[1] = (unsigned)run;
    }
    __syncthreads();
    const unsigned total_ties = s_misc[1];
    if (k > total_ties) k = total_ties;                    // cannot happen for an exact crossing; keeps the walk in range
    r.k = k;
    const int before = s_cnt[tid];
    if ((unsigned long long)before < k && k <= (unsigned long long)(before + cnt)) {
        int seen = before;
        for (int i = lo; i < hi; i++)
            if (__float_as_uint(p[i]) == prefix && (unsigned long long)(++seen) == k) { s_misc[4] = (unsigned)i; break; }
    }
    __syncthreads();
    r.token = (int)s_misc[4];
    __syncthreads();
    return r;
}

__device__ __forceinline__ double block_sum_d(double v, double *s_red) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        double t = threadIdx.x < (SMP_THREADS >> 5) ? s_red[threadIdx.x] : 0.0;
#pragma unroll
        for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) s_red[0] = t;
    }
    __syncthreads();
    return s_red[0];
}

// u == NULL: the row's uniform comes from its splitmix64 state (advanced here).
__global__ void __launch_bounds__(SMP_THREADS)
sample_rows_kernel(const float *__restrict__ logits, int n, float temp, float top_p,
                   const double *__restrict__ u_in, unsigned long long *__restrict__ rng,
                   float *probs, int32_t *__restrict__ out) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    __shared__ unsigned long long s_hist[256];
    __shared__ __align__(8) unsigned s_misc[8];
    __shared__ int s_cnt[SMP_THREADS];
    __shared__ double s_red[32];
    __shared__ float s_f[32];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float *l = logits + (size_t)row * n;
    float *p = probs + (size_t)row * n;
    // max
    float mx = -INFINITY;
    for (int i = tid; i < n; i += SMP_THREADS) mx = fmaxf(mx, l[i]);
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((tid & 31) == 0) s_f[tid >> 5] = mx;
    __syncthreads();
    mx = s_f[0];
    for (int w = 1; w < SMP_THREADS / 32; w++) mx = fmaxf(mx, s_f[w]);
    // softmax: f32 exponent argument, double sum (a tree here), one rounding back to f32
    double part = 0.0;
    for (int i = tid; i < n; i += SMP_THREADS) {
        const float e = exp_rn(__fdiv_rn(__fsub_rn(l[i], mx), temp));
        p[i] = e;
        part += (double)e;
    }
    const double sum = block_sum_d(part, s_red);
    unsigned long long tot = 0;
    for (int i = tid; i < n; i += SMP_THREADS) {
        const float q = (float)((double)p[i] / sum);
        p[i] = q;
        tot += mass_of(q);
    }
    // total mass (exact integer sum)
    if (tid == 0) reinterpret_cast<unsigned long long *>(s_misc + 6)[0] = 0ull;
    __syncthreads();
    atomicAdd(reinterpret_cast<unsigned long long *>(s_misc + 6), tot);
    __syncthreads();
    const unsigned long long total = reinterpret_cast<unsigned long long *>(s_misc + 6)[0];
    __syncthreads();
    // the row's uniform
    double u;
    if (u_in) u = u_in[row];
    else {
        unsigned long long s = rng[row] + 0x9E3779B97F4A7C15ull, z = s;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        u = (double)(z >> 11) * 0x1.0p-53;
        __syncthreads();
        if (tid == 0) rng[row] = s;
    }
    // nucleus: tokens are kept up to and including the first whose inclusive mass exceeds top_p
    const double tp = (double)top_p;
    unsigned long long kept = total;
    Sel cut;
    cut.found = 0; cut.token = -1;
    if (tp < 1.5) {                                          // top_p >= 1.5 can never be exceeded by probabilities
        const unsigned long long Mp = tp <= 0.0 ? 0ull : (unsigned long long)(tp * SMP_ONE);
        cut = first_exceed(p, n, Mp, s_hist, s_misc, s_cnt);
        if (cut.found) kept = cut.above + cut.k * mass_of(__uint_as_float(cut.key));
    }
    // draw inside the kept mass
    const unsigned long long Mu = (unsigned long long)(u * (double)kept);
    Sel d = first_exceed(p, n, Mu < kept ? Mu : kept - 1, s_hist, s_misc, s_cnt);
    int token = d.found ? d.token : cut.token;
    if (token < 0) token = 0;
    if (tid == 0) out[row] = token;
}

}  // namespace

// logits [rows, n] -> tokens [rows]; temp <= 0: greedy.  probs: scratch [rows, n] floats.
// u (device, [rows], nullable) are explicit uniforms in [0, 1); otherwise rng [rows]
// holds the rows' splitmix64 states and is advanced by one draw.
int sample_rows(const float *logits, int n, int rows, float temp, float top_p, const double *u,
                unsigned long long *rng, float *probs, int32_t *out, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (temp <= 0.f) return argmax_rows(logits, n, rows, out, st);
    APUS_REQUIRE(u || rng, "sample: neither uniforms nor generator states given");
    launch_k(sample_rows_kernel, rows, SMP_THREADS, 0, st, logits, n, temp, top_p, u, rng, probs, out);
    APUS_LAUNCHED();
    return 0;
}

}  // namespace apus
