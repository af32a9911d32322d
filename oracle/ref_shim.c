/*
 * oracle/ref_shim.c — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Single translation unit that instantiates the reference's own header-only
 * C implementation (included read-only from the reference checkout; nothing
 * is copied into this repository) and exports thin wrappers around the
 * functions that are `static` there, so that tests and the CPU-baseline leg
 * of the benchmark can call the unmodified reference through ctypes.
 *
 * The non-static reference functions (apus_fp4_linear, apus_fp8_linear,
 * apus_moe_forward, apus_router_score, apus_topk_stable, apus_rms_norm,
 * apus_mhc_*, apus_fp4_gemm_mt, apus_fp8_gemm_mt, ...) are exported from the
 * resulting shared object under their own names.
 *
 * Built by oracle/Makefile into oracle/_ref/libapus_ref.so with the
 * reference's flags (reference Makefile:21-49).  Only tests/, the smoke
 * check and the benchmark's cpu_baseline / reference arm may load it.
 */
#define APUS_JSON_IMPLEMENTATION
#define APUS_FP4_IMPLEMENTATION
#define APUS_FP8_IMPLEMENTATION
#define APUS_MHC_IMPLEMENTATION
#define APUS_ST_IMPLEMENTATION
#define APUS_ATTN_IMPLEMENTATION
#define APUS_MOE_IMPLEMENTATION

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "moe.h"
#include "mhc.h"

/* c/moe.h:333 (static apus_expert). kind 0 = MXFP4, 1 = FP8. */
void ref_expert(const void *w1, const void *w2, const void *w3, int kind,
                float limit, const float *x, int dim, int inter, float *out) {
    apus_expert(w1, w2, w3, kind, limit, x, dim, inter, out);
}

/* c/moe.h:113 (static SwiGLU range worker). */
void ref_expert_swiglu(const float *g, const float *u, float *h, size_t n,
                       float limit) {
    apus_expert_swiglu(g, u, h, n, limit);
}

/* c/attn.h:393 (static row worker): BF16 round + per-128 act quant. */
void ref_act_quant_rows(const float *x, float *xb, uint8_t *codes, float *as,
                        int M, int K) {
    ApusActQuantJob aq = { x, xb, codes, as, K,
                           apus_fp4_act_blocks((size_t)K) };
    apus_act_quant_rows(&aq, 0, (size_t)M);
}

/* c/attn.h:1308 (static apus_sparse_attn). */
void ref_sparse_attn(const float *q, const float *sink, int h, int d,
                     const int32_t *idxs, int idxw, int s, float scale,
                     const float *kv_a, int64_t na, const float *kv_b,
                     float *o) {
    apus_sparse_attn(q, sink, h, d, idxs, idxw, s, scale, kv_a, na, kv_b, o);
}

/* c/attn.h:692 / 722 (static index-set builders). Return the row width. */
int ref_window_idxs(int32_t *out, int s, int64_t start_pos, int win) {
    return apus_window_idxs(out, s, start_pos, win);
}
int ref_compress_idxs(int32_t *out, int ratio, int s, int64_t start_pos,
                      int offset) {
    return apus_compress_idxs(out, ratio, s, start_pos, offset);
}

/* c/x86.h:79 — how many dispatches took the AVX2 row kernels. */
uint64_t ref_avx2_hits(void) { return apus_x86_avx2_hits(); }

/* c/pool.h — lanes the pool was configured with (APUS_THREADS or nproc). */
int ref_pool_threads(void) { return apus_pool_threads(); }
