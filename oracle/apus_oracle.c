/*
 * oracle/apus_oracle.c — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Plain-C, single-threaded restatement of the reference's arithmetic for the
 * decode/prefill hot path (format conversions, activation quantisation,
 * MXFP4 / FP8 block-scaled products, the SwiGLU expert, the router, the MoE
 * sublayer, RMSNorm, index-gathered sparse attention, mHC maps).  It exists so
 * the CUDA kernels can be checked on a machine that does not have the
 * reference checkout.  Nothing in the product library links or calls it.
 *
 * PARITY PIN: every function here is compared bit-for-bit against the
 * unmodified reference (oracle/_ref/libapus_ref.so, built from the reference's
 * own headers) in tests/test_oracle_pin.py, and against the committed golden
 * vectors under tests/golden/ (produced by tests/golden/make_golden.py from the
 * reference itself and from the reference's own generator scripts).
 *
 * All arithmetic is IEEE f32 with no contraction (build with
 * -ffp-contract=off): each `a*b + c` below is two roundings, as in the
 * reference's x86 build (reference Makefile:22-27).
 *
 * Citations are `file:line` relative to the reference project root.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- bit helpers ----------------------------------------------------------- */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* c/fp4.h:262-270 — round-to-nearest-even to BF16, NaN passes through. */
float ora_bf16_round(float x) {
    uint32_t u = f2u(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x;
    uint32_t lsb = (u >> 16) & 1u;
    return u2f((u + 0x7fffu + lsb) & 0xffff0000u);
}

/* c/fp4.h:209-217 — UE8M0 byte to f32: 0 -> 2^-127 (subnormal), 255 -> +inf. */
float ora_ue8m0(uint8_t b) {
    return u2f(b ? (uint32_t)b << 23 : 0x00400000u);
}

/* c/fp4.h:204-207 — E2M1 value table, bit 3 is the sign. */
static const float E2M1[16] = { 0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f };

/* c/fp4.h:255-260 — E4M3 code to f32 (codes 0x7f/0xff give +-480). */
float ora_e4m3_to_f32(uint8_t c) {
    int e = (c >> 3) & 15, m = c & 7;
    float mag = e ? ldexpf((float)(8 + m), e - 10) : ldexpf((float)m, -9);
    return (c & 0x80) ? -mag : mag;
}

/* c/fp4.h:229-253 — f32 to E4M3, clamp to +-448, round to nearest even.
 * Restated as "find the nearest code on the E4M3 grid": the grid spacing in
 * binade e (e >= -6) is 2^(e-3); below 2^-6 it is the fixed 2^-9. */
uint8_t ora_e4m3_from_f32(float x) {
    uint8_t sign = (f2u(x) >> 31) ? 0x80 : 0;
    float a = fabsf(x);
    if (a > 448.0f) a = 448.0f;
    if (a == 0.0f) return sign;
    int ex;
    (void)frexpf(a, &ex);                  /* a = f * 2^ex, f in [0.5,1) */
    int e = ex - 1;                        /* binade: 2^e <= a < 2^(e+1) */
    if (e < -6) e = -6;                    /* subnormal grid shares 2^-9 */
    float q = ldexpf(a, 3 - e);            /* a in units of the spacing (exact) */
    float r = nearbyintf(q);               /* default rounding mode: RNE */
    int steps = (int)r;                    /* 0..16 */
    int code;
    if (e == -6 && steps < 8) code = steps;            /* subnormal codes 0..7 */
    else {
        if (steps == 16) { steps = 8; e++; }           /* carried into next binade */
        code = ((e + 7) << 3) | (steps - 8);
        if (code > 0x7e) code = 0x7e;
    }
    return (uint8_t)(sign | code);
}

/* c/attn.h:314-323 — 2^ceil(log2(p)) for positive normal p by the exponent
 * field plus one when any mantissa bit is set. */
static float ceil_pow2(float p) {
    uint32_t b = f2u(p);
    uint32_t e = ((b >> 23) & 0xff) + ((b & 0x7fffffu) ? 1u : 0u);
    return u2f(e << 23);
}

/* c/fp4.h:293-321 — per-128 activation quantisation of one row of K floats
 * (K % 32 == 0; a trailing partial group takes the amax of what is left). */
void ora_act_quant_row(const float *x, size_t K, uint8_t *codes, float *scales) {
    for (size_t g0 = 0, b = 0; g0 < K; g0 += 128, b++) {
        size_t g1 = g0 + 128 < K ? g0 + 128 : K;
        float amax = 0.0f;
        for (size_t i = g0; i < g1; i++) if (fabsf(x[i]) > amax) amax = fabsf(x[i]);
        if (amax < 1e-4f) amax = 1e-4f;
        float s = ceil_pow2(amax * (1.0f / 448.0f));
        scales[b] = s;
        for (size_t i = g0; i < g1; i++) codes[i] = ora_e4m3_from_f32(x[i] / s);
    }
}

/* c/attn.h:393-402 — the linears' front end: BF16-round each row, then
 * quantise it. xb (optional) receives the rounded rows. */
void ora_act_quant(const float *x, int M, int K, float *xb, uint8_t *codes,
                   float *scales) {
    size_t nab = ((size_t)K + 127) / 128;
    float *tmp = xb ? NULL : malloc((size_t)K * sizeof(float));
    for (int m = 0; m < M; m++) {
        float *row = xb ? xb + (size_t)m * K : tmp;
        for (int i = 0; i < K; i++) row[i] = ora_bf16_round(x[(size_t)m * K + i]);
        ora_act_quant_row(row, (size_t)K, codes + (size_t)m * K, scales + (size_t)m * nab);
    }
    free(tmp);
}

/* ---- block-scaled products -------------------------------------------------- */

/* c/fp4.h:367-395 — MXFP4 GEMM on pre-quantised activations.
 * out[m,o] = sum over 32-blocks kb of (dot_kb * as[m,kb/4]) * 2^(ws[o,kb]-127),
 * dot_kb summed in k order, blocks folded in kb order. */
void ora_fp4_gemm(const uint8_t *w, const uint8_t *ws, const uint8_t *acodes,
                  const float *as, float *out, size_t M, size_t O, size_t K) {
    size_t nb = K / 32, nab = (K + 127) / 128;
    float *a = malloc(K * sizeof(float));
    for (size_t m = 0; m < M; m++) {
        for (size_t k = 0; k < K; k++) a[k] = ora_e4m3_to_f32(acodes[m * K + k]);
        for (size_t o = 0; o < O; o++) {
            const uint8_t *row = w + o * (K / 2);
            float total = 0.0f;
            for (size_t kb = 0; kb < nb; kb++) {
                float dot = 0.0f;
                for (size_t k = kb * 32; k < kb * 32 + 32; k++) {
                    uint8_t byte = row[k >> 1];
                    uint8_t nib = (k & 1) ? (byte >> 4) : (byte & 15);
                    float prod = a[k] * E2M1[nib];
                    dot = dot + prod;
                }
                float t = dot * as[m * nab + kb / 4];
                t = t * ora_ue8m0(ws[o * nb + kb]);
                total = total + t;
            }
            out[m * O + o] = total;
        }
    }
    free(a);
}

/* c/fp8.h:191-218 — FP8 GEMM on pre-quantised activations.
 * out[m,o] = sum over 128-blocks kb of dot_kb * (as[m,kb] * 2^(ws[o/128,kb]-127)):
 * the two scales are multiplied FIRST (unlike the MXFP4 product). */
void ora_fp8_gemm(const uint8_t *w, const uint8_t *ws, const uint8_t *acodes,
                  const float *as, float *out, size_t M, size_t O, size_t K) {
    size_t nb = (K + 127) / 128;
    float *a = malloc(K * sizeof(float));
    float lut[256];
    for (int c = 0; c < 256; c++) lut[c] = ora_e4m3_to_f32((uint8_t)c);
    for (size_t m = 0; m < M; m++) {
        for (size_t k = 0; k < K; k++) a[k] = lut[acodes[m * K + k]];
        for (size_t o = 0; o < O; o++) {
            const uint8_t *row = w + o * K;
            float total = 0.0f;
            for (size_t kb = 0; kb < nb; kb++) {
                size_t k1 = kb * 128 + 128 < K ? kb * 128 + 128 : K;
                float dot = 0.0f;
                for (size_t k = kb * 128; k < k1; k++) {
                    float prod = a[k] * lut[row[k]];
                    dot = dot + prod;
                }
                float sc = as[m * nb + kb] * ora_ue8m0(ws[(o / 128) * nb + kb]);
                float t = dot * sc;
                total = total + t;
            }
            out[m * O + o] = total;
        }
    }
    free(a);
}

/* c/attn.h:408-449 — quantised linears: round+quantise x, block-scaled
 * product, BF16-round every output. kind 0 = MXFP4, 1 = FP8. */
void ora_qlinear(int kind, const uint8_t *w, const uint8_t *ws, const float *x,
                 float *out, int M, int K, int O) {
    size_t nab = ((size_t)K + 127) / 128;
    uint8_t *codes = malloc((size_t)M * K);
    float *as = malloc((size_t)M * nab * sizeof(float));
    ora_act_quant(x, M, K, NULL, codes, as);
    if (kind == 0) ora_fp4_gemm(w, ws, codes, as, out, (size_t)M, (size_t)O, (size_t)K);
    else           ora_fp8_gemm(w, ws, codes, as, out, (size_t)M, (size_t)O, (size_t)K);
    for (size_t i = 0; i < (size_t)M * O; i++) out[i] = ora_bf16_round(out[i]);
    free(codes); free(as);
}

/* c/attn.h:460-465, 621-666 — sequential-k f32 matmul. flags bit0: BF16-round
 * the inputs, bit1: BF16-round the outputs, bit2: w is BF16 bits (u16). */
void ora_f32_linear(const void *w, const float *x, float *out, int M, int K,
                    int O, int flags) {
    const float *wf = w;
    const uint16_t *wh = w;
    for (int m = 0; m < M; m++)
        for (int o = 0; o < O; o++) {
            float dot = 0.0f;
            for (int k = 0; k < K; k++) {
                float xv = x[(size_t)m * K + k];
                if (flags & 1) xv = ora_bf16_round(xv);
                float wv = (flags & 4) ? u2f((uint32_t)wh[(size_t)o * K + k] << 16)
                                       : wf[(size_t)o * K + k];
                float prod = xv * wv;
                dot = dot + prod;
            }
            out[(size_t)m * O + o] = (flags & 2) ? ora_bf16_round(dot) : dot;
        }
}

/* c/model.h:528-647 — LM-head GEMV: BF16 weights widened exactly, product
 * written weight-first (w*x), sequential k, unrounded f32 out. */
void ora_head_gemv_bf16(const uint16_t *w, const float *x, float *out,
                        int64_t O, int64_t K) {
    for (int64_t o = 0; o < O; o++) {
        float acc = 0.0f;
        for (int64_t k = 0; k < K; k++) {
            float prod = u2f((uint32_t)w[o * K + k] << 16) * x[k];
            acc = acc + prod;
        }
        out[o] = acc;
    }
}

/* c/attn.h:371-378 — RMSNorm with BF16-rounded output. */
void ora_rms_norm(const float *x, const float *w, float eps, float *y, size_t n) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; i++) { float sq = x[i] * x[i]; ss = ss + sq; }
    float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (size_t i = 0; i < n; i++) {
        float xn = x[i] * inv;
        y[i] = ora_bf16_round(w[i] * xn);
    }
}

/* ---- expert / router / MoE --------------------------------------------------- */

/* c/moe.h:113-126 — clamp, silu(gate)*up, BF16 round. */
void ora_swiglu(const float *g, const float *u, float *h, size_t n, float limit) {
    for (size_t i = 0; i < n; i++) {
        float gv = g[i], uv = u[i];
        if (limit > 0.0f) {
            uv = uv > limit ? limit : (uv < -limit ? -limit : uv);
            gv = gv > limit ? limit : gv;
        }
        float sig = 1.0f / (1.0f + expf(-gv));
        float act = gv * sig;
        h[i] = ora_bf16_round(act * uv);
    }
}

typedef struct { const uint8_t *codes, *scales; int64_t O, K; } OraQW;

/* c/moe.h:333-350 — one SwiGLU expert for `rows` tokens (the reference calls
 * it per token; rows are independent). kind 0 = MXFP4, 1 = FP8. */
void ora_expert(const OraQW *w1, const OraQW *w2, const OraQW *w3, int kind,
                float limit, const float *x, int rows, int dim, int inter,
                float *out) {
    float *g = malloc((size_t)rows * inter * sizeof(float));
    float *u = malloc((size_t)rows * inter * sizeof(float));
    float *h = malloc((size_t)rows * inter * sizeof(float));
    ora_qlinear(kind, w1->codes, w1->scales, x, g, rows, dim, inter);
    ora_qlinear(kind, w3->codes, w3->scales, x, u, rows, dim, inter);
    ora_swiglu(g, u, h, (size_t)rows * inter, limit);
    ora_qlinear(kind, w2->codes, w2->scales, h, out, rows, inter, dim);
    free(g); free(u); free(h);
}

/* c/attn.h:668-687 — k passes of strict-greater argmax over unused entries;
 * the lowest index wins a tie; output is in descending score order. */
void ora_topk_stable(const float *row, int n, int k, int32_t *idx) {
    uint8_t *taken = calloc((size_t)n, 1);
    for (int j = 0; j < k; j++) {
        int best = -1;
        for (int i = 0; i < n; i++) {
            if (taken[i]) continue;
            if (best < 0 || row[i] > row[best]) best = i;
        }
        idx[j] = best;
        taken[best] = 1;
    }
    free(taken);
}

/* c/moe.h:96-100, 352-367 — sp = sqrt(softplus(x . gate_w^T)) (softplus is the
 * identity above 20), biased = sp + bias. The gate product is the sequential
 * f32 matmul, unrounded. */
void ora_router_score(const float *gate_w, const float *gate_bias, int E,
                      int dim, const float *x, int s, float *sp, float *biased) {
    ora_f32_linear(gate_w, x, sp, s, dim, E, 0);
    for (int i = 0; i < s * E; i++) {
        float z = sp[i];
        float soft = z > 20.0f ? z : log1pf(expf(z));
        sp[i] = sqrtf(soft);
        if (biased) biased[i] = sp[i] + gate_bias[i % E];
    }
}

/* c/moe.h:369-595 — the MoE sublayer, stated token by token (the reference's
 * batched path is bitwise equal to this by its tests/m9e gate): route, run
 * the top-k experts in slot order accumulating y += w_j * eo_j in f32, add the
 * FP8 shared expert, BF16-round.  w1/w2/w3 are arrays of E expert views. */
void ora_moe_forward(int E, int topk, int inter, int dim, int hash,
                     float route_scale, float limit, const float *gate_w,
                     const float *gate_bias, const int64_t *tid2eid,
                     const OraQW *w1, const OraQW *w2, const OraQW *w3,
                     const OraQW *sw1, const OraQW *sw2, const OraQW *sw3,
                     const float *x, const int64_t *ids, int s, float *out,
                     int32_t *idx_out, float *wgt_out, float *routed_out,
                     float *shared_out) {
    float *sp = malloc((size_t)s * E * sizeof(float));
    float *biased = hash ? NULL : malloc((size_t)s * E * sizeof(float));
    float *eo = malloc((size_t)dim * sizeof(float));
    float *sh = malloc((size_t)dim * sizeof(float));
    float *y = malloc((size_t)dim * sizeof(float));
    int32_t *idx = malloc((size_t)topk * sizeof(int32_t));
    float *wgt = malloc((size_t)topk * sizeof(float));
    ora_router_score(gate_w, gate_bias, E, dim, x, s, sp, biased);
    for (int t = 0; t < s; t++) {
        const float *xt = x + (size_t)t * dim;
        if (hash) for (int j = 0; j < topk; j++) idx[j] = (int32_t)tid2eid[ids[t] * topk + j];
        else ora_topk_stable(biased + (size_t)t * E, E, topk, idx);
        float sum = 0.0f;
        for (int j = 0; j < topk; j++) { wgt[j] = sp[(size_t)t * E + idx[j]]; sum = sum + wgt[j]; }
        for (int j = 0; j < topk; j++) wgt[j] = wgt[j] / sum * route_scale;
        memset(y, 0, (size_t)dim * sizeof(float));
        for (int j = 0; j < topk; j++) {
            int e = idx[j];
            ora_expert(&w1[e], &w2[e], &w3[e], 0, limit, xt, 1, dim, inter, eo);
            for (int i = 0; i < dim; i++) { float p = wgt[j] * eo[i]; y[i] = y[i] + p; }
        }
        ora_expert(sw1, sw2, sw3, 1, limit, xt, 1, dim, inter, sh);
        for (int i = 0; i < dim; i++) out[(size_t)t * dim + i] = ora_bf16_round(y[i] + sh[i]);
        if (idx_out) memcpy(idx_out + (size_t)t * topk, idx, (size_t)topk * sizeof(int32_t));
        if (wgt_out) memcpy(wgt_out + (size_t)t * topk, wgt, (size_t)topk * sizeof(float));
        if (routed_out) memcpy(routed_out + (size_t)t * dim, y, (size_t)dim * sizeof(float));
        if (shared_out) memcpy(shared_out + (size_t)t * dim, sh, (size_t)dim * sizeof(float));
    }
    free(sp); free(biased); free(eo); free(sh); free(y); free(idx); free(wgt);
}

/* ---- sparse attention ---------------------------------------------------------- */

/* c/attn.h:1193-1326 — per (token, head): drop negative ids, s_j = (q.kv_j) *
 * scale with a sequential-k dot, p_j = bf16(exp(s_j - max)), o = sum_j p_j *
 * kv_j in j order (mul then add), divided by (sum p + exp(sink - max)),
 * BF16-rounded; no ids -> zeros. Rows below `na` come from kv_a, the rest
 * from kv_b (K and V are the same vector). */
void ora_sparse_attn(const float *q, const float *sink, int h, int d,
                     const int32_t *idxs, int idxw, int s, float scale,
                     const float *kv_a, int64_t na, const float *kv_b,
                     float *o) {
    float *sc = malloc((size_t)idxw * sizeof(float));
    float *p = malloc((size_t)idxw * sizeof(float));
    int32_t *ids = malloc((size_t)idxw * sizeof(int32_t));
    for (int t = 0; t < s; t++) {
        int n = 0;
        for (int j = 0; j < idxw; j++)
            if (idxs[(size_t)t * idxw + j] >= 0) ids[n++] = idxs[(size_t)t * idxw + j];
        for (int hh = 0; hh < h; hh++) {
            const float *qv = q + ((size_t)t * h + hh) * d;
            float *ov = o + ((size_t)t * h + hh) * d;
            memset(ov, 0, (size_t)d * sizeof(float));
            if (!n) continue;
            float mx = -INFINITY;
            for (int j = 0; j < n; j++) {
                const float *kv = ids[j] < na ? kv_a + (size_t)ids[j] * d
                                              : kv_b + (size_t)(ids[j] - na) * d;
                float dot = 0.0f;
                for (int k = 0; k < d; k++) { float pr = qv[k] * kv[k]; dot = dot + pr; }
                sc[j] = dot * scale;
                if (sc[j] > mx) mx = sc[j];
            }
            float sum = 0.0f;
            for (int j = 0; j < n; j++) { p[j] = ora_bf16_round(expf(sc[j] - mx)); sum = sum + p[j]; }
            for (int j = 0; j < n; j++) {
                const float *kv = ids[j] < na ? kv_a + (size_t)ids[j] * d
                                              : kv_b + (size_t)(ids[j] - na) * d;
                for (int k = 0; k < d; k++) { float pr = p[j] * kv[k]; ov[k] = ov[k] + pr; }
            }
            float den = sum + expf(sink[hh] - mx);
            for (int k = 0; k < d; k++) ov[k] = ora_bf16_round(ov[k] / den);
        }
    }
    free(sc); free(p); free(ids);
}

/* ---- mHC ------------------------------------------------------------------------ */

static float sigm(float x) { return 1.0f / (1.0f + expf(-x)); }

/* c/mhc.h:181-218 — Sinkhorn on an n x n matrix: row softmax (+eps on every
 * element), column normalise, then (iters-1) x (row normalise, column
 * normalise), the eps of the normalisations inside the denominator. */
void ora_sinkhorn(float *c, int n, int iters, float eps) {
    for (int j = 0; j < n; j++) {
        float *r = c + j * n, mx = r[0], sum = 0.0f;
        for (int k = 1; k < n; k++) if (r[k] > mx) mx = r[k];
        for (int k = 0; k < n; k++) { r[k] = expf(r[k] - mx); sum = sum + r[k]; }
        for (int k = 0; k < n; k++) r[k] = r[k] / sum + eps;
    }
    for (int it = 0; it < iters; it++) {
        if (it) for (int j = 0; j < n; j++) {
            float sum = 0.0f;
            for (int k = 0; k < n; k++) sum = sum + c[j * n + k];
            float den = sum + eps;
            for (int k = 0; k < n; k++) c[j * n + k] = c[j * n + k] / den;
        }
        for (int k = 0; k < n; k++) {
            float sum = 0.0f;
            for (int j = 0; j < n; j++) sum = sum + c[j * n + k];
            float den = sum + eps;
            for (int j = 0; j < n; j++) c[j * n + k] = c[j * n + k] / den;
        }
    }
}

/* c/mhc.h:159-175 — r = 1/sqrt(mean(x^2)+eps); mixes[j] = (fn_j . x) * r with
 * r applied after the sequential dot. */
static void mhc_mixes(const float *x, size_t nx, const float *fn, float norm_eps,
                      float *mixes, size_t nmix) {
    float ss = 0.0f;
    for (size_t i = 0; i < nx; i++) { float sq = x[i] * x[i]; ss = ss + sq; }
    float r = 1.0f / sqrtf(ss / (float)nx + norm_eps);
    for (size_t j = 0; j < nmix; j++) {
        float dot = 0.0f;
        for (size_t i = 0; i < nx; i++) { float p = fn[j * nx + i] * x[i]; dot = dot + p; }
        mixes[j] = dot * r;
    }
}

/* c/mhc.h:221-248 — pre/post gates and the Sinkhorn-normalised comb matrix for
 * one token. mixes_out (optional) receives the (2+n)*n raw mixes. */
void ora_mhc_prepost(const float *x4, size_t d, size_t n, const float *fn,
                     const float *scale, const float *base, float norm_eps,
                     float hc_eps, int iters, float *pre, float *post,
                     float *comb, float *mixes_out) {
    size_t nmix = (2 + n) * n;
    float *mixes = malloc(nmix * sizeof(float));
    mhc_mixes(x4, n * d, fn, norm_eps, mixes, nmix);
    for (size_t j = 0; j < n; j++) {
        pre[j] = sigm(mixes[j] * scale[0] + base[j]) + hc_eps;
        post[j] = 2.0f * sigm(mixes[n + j] * scale[1] + base[n + j]);
    }
    for (size_t i = 0; i < n * n; i++) comb[i] = mixes[2 * n + i] * scale[2] + base[2 * n + i];
    ora_sinkhorn(comb, (int)n, iters, hc_eps);
    if (mixes_out) memcpy(mixes_out, mixes, nmix * sizeof(float));
    free(mixes);
}

/* c/mhc.h:250-257 — y[i] = sum_j pre[j] * X[j,i], j ascending. */
void ora_mhc_collapse(const float *x4, const float *pre, float *y, size_t d, size_t n) {
    for (size_t i = 0; i < d; i++) {
        float acc = 0.0f;
        for (size_t j = 0; j < n; j++) { float p = pre[j] * x4[j * d + i]; acc = acc + p; }
        y[i] = acc;
    }
}

/* c/mhc.h:259-270 — Y[j,i] = post[j]*f[i] + sum_k comb[k,j]*R[k,i]. */
void ora_mhc_apply(const float *f, const float *res, const float *post,
                   const float *comb, float *y4, size_t d, size_t n) {
    for (size_t j = 0; j < n; j++)
        for (size_t i = 0; i < d; i++) {
            float acc = post[j] * f[i];
            for (size_t k = 0; k < n; k++) { float p = comb[k * n + j] * res[k * d + i]; acc = acc + p; }
            y4[j * d + i] = acc;
        }
}

/* c/mhc.h:272-285 — hc_head: sigmoid-gated collapse, no Sinkhorn. */
void ora_mhc_head(const float *x4, size_t d, size_t n, const float *fn,
                  float scale, const float *base, float norm_eps, float hc_eps,
                  float *y) {
    float *pre = malloc(n * sizeof(float));
    mhc_mixes(x4, n * d, fn, norm_eps, pre, n);
    for (size_t j = 0; j < n; j++) pre[j] = sigm(pre[j] * scale + base[j]) + hc_eps;
    ora_mhc_collapse(x4, pre, y, d, n);
    free(pre);
}

/* ---- attention row helpers ------------------------------------------------------- */

/* c/attn.h:290-299 — interleaved-pair rotation of rd floats, each output BF16-
 * rounded; inverse = conjugate. Products and the sum are rounded separately. */
void ora_apply_rope(float *x, const float *cos, const float *sin, int rd, int inverse) {
    for (int j = 0; j < rd / 2; j++) {
        float a = x[2 * j], b = x[2 * j + 1], c = cos[j], s = inverse ? -sin[j] : sin[j];
        float ac = a * c, bs = b * s, as = a * s, bc = b * c;
        x[2 * j] = ora_bf16_round(ac - bs);
        x[2 * j + 1] = ora_bf16_round(as + bc);
    }
}

/* c/attn.h:301-311 — Sylvester butterflies, then * n^-1/2 and BF16 round. */
void ora_hadamard(float *x, int n) {
    for (int len = 1; len < n; len *= 2)
        for (int i = 0; i < n; i++)
            if (!(i & len)) {
                float a = x[i], b = x[i + len];
                x[i] = a + b;
                x[i + len] = a - b;
            }
    float inv = (float)pow((double)n, -0.5);
    for (int i = 0; i < n; i++) x[i] = ora_bf16_round(x[i] * inv);
}

/* c/attn.h:325-339 — E4M3 quantise-dequantise per `group` with a power-of-two
 * scale (amax floored at 1e-4). */
void ora_fp8_qat_sim(float *x, size_t K, size_t group) {
    for (size_t g0 = 0; g0 < K; g0 += group) {
        size_t g1 = g0 + group < K ? g0 + group : K;
        float amax = 0.0f;
        for (size_t i = g0; i < g1; i++) if (fabsf(x[i]) > amax) amax = fabsf(x[i]);
        if (amax < 1e-4f) amax = 1e-4f;
        float s = ceil_pow2(amax * (1.0f / 448.0f));
        for (size_t i = g0; i < g1; i++) x[i] = ora_e4m3_to_f32(ora_e4m3_from_f32(x[i] / s)) * s;
    }
}

/* c/attn.h:342-369 — E2M1 quantise-dequantise per 32 (amax floor 6*2^-126,
 * clamp +-6, ties to the even code). */
void ora_fp4_qat_sim(float *x, size_t K) {
    static const float cut[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
    for (size_t g0 = 0; g0 < K; g0 += 32) {
        float amax = 0.0f;
        for (size_t i = g0; i < g0 + 32; i++) if (fabsf(x[i]) > amax) amax = fabsf(x[i]);
        if (amax < 7.05484372e-38f) amax = 7.05484372e-38f;
        float s = ceil_pow2(amax * (1.0f / 6.0f));
        for (size_t i = g0; i < g0 + 32; i++) {
            float y = x[i] / s;
            y = y > 6.0f ? 6.0f : (y < -6.0f ? -6.0f : y);
            float a = fabsf(y);
            int mag = 0;
            for (int j = 0; j < 7; j++) mag += (a > cut[j]) || (a == cut[j] && (j & 1));
            x[i] = E2M1[signbit(y) ? (mag | 8) : mag] * s;
        }
    }
}

/* ---- sampling (c/sample.h:76-180) ------------------------------------------------- */
/* greedy: strict >, lowest index on ties (c/sample.h:76-81) */
int ora_sample_argmax(const float *logits, size_t n) {
    size_t best = 0;
    for (size_t i = 1; i < n; i++) if (logits[i] > logits[best]) best = i;
    return (int)best;
}

/* splitmix64 and the 53-bit uniform (c/sample.h:160-171) */
uint64_t ora_rng_next(uint64_t *state) {
    uint64_t z = (*state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
double ora_rng_uniform(uint64_t *state) { return (double)(ora_rng_next(state) >> 11) * 0x1.0p-53; }

/* temperature softmax + nucleus draw with an explicit uniform (c/sample.h:91-158).
 * The reference sorts the probabilities (descending, lower index first on ties)
 * and walks the sorted list twice; this restatement does the same with an
 * insertion-free O(n log n) merge sort on (prob desc, index asc), which yields
 * the identical order.  ord: scratch of n int32, p: scratch of n floats. */
static void ora_merge_sort(int32_t *ord, int32_t *tmp, const float *p, size_t n) {
    for (size_t w = 1; w < n; w *= 2) {
        for (size_t lo = 0; lo < n; lo += 2 * w) {
            size_t mid = lo + w < n ? lo + w : n, hi = lo + 2 * w < n ? lo + 2 * w : n;
            size_t a = lo, b = mid, o = lo;
            while (a < mid && b < hi) {
                int32_t x = ord[a], y = ord[b];
                /* take from the left run unless the right element sorts strictly before it */
                int right_first = p[y] > p[x] || (p[y] == p[x] && y < x);
                tmp[o++] = right_first ? ord[b++] : ord[a++];
            }
            while (a < mid) tmp[o++] = ord[a++];
            while (b < hi) tmp[o++] = ord[b++];
        }
        for (size_t i = 0; i < n; i++) ord[i] = tmp[i];
    }
}

int ora_sample_logits_u(const float *logits, size_t n, float temp, float top_p, double u,
                        float *p, int32_t *ord, int32_t *tmp) {
    if (temp <= 0.0f) return ora_sample_argmax(logits, n);
    float mx = logits[0];
    for (size_t i = 1; i < n; i++) if (logits[i] > mx) mx = logits[i];
    double sum = 0.0;
    for (size_t i = 0; i < n; i++) { p[i] = expf((logits[i] - mx) / temp); sum += p[i]; }
    for (size_t i = 0; i < n; i++) p[i] = (float)(p[i] / sum);
    for (size_t i = 0; i < n; i++) ord[i] = (int32_t)i;
    ora_merge_sort(ord, tmp, p, n);
    /* nucleus: keep token i iff the mass before it is <= top_p; always the top token */
    double cum = 0.0, kept = 0.0;
    size_t nk = 0;
    for (size_t i = 0; i < n; i++) {
        if (cum <= (double)top_p) { cum += p[ord[i]]; kept = cum; nk = i + 1; }
        else break;
    }
    if (nk == 0) { nk = 1; kept = p[ord[0]]; }
    double c = 0.0;
    for (size_t i = 0; i < nk; i++) {
        c += (double)p[ord[i]] / kept;
        if (u < c) return ord[i];
    }
    return ord[nk - 1];
}
