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
#define APUS_LAYER_IMPLEMENTATION
#define APUS_MODEL_IMPLEMENTATION
#define APUS_SAMPLE_IMPLEMENTATION
#define APUS_MTP_IMPLEMENTATION
#define APUS_DSPARK_IMPLEMENTATION

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "moe.h"
#include "mhc.h"
#include "model.h"
#include "sample.h"
#include "mtp.h"
#include "dspark.h"
/* after the reference headers: their include guards make this header skip its
 * layout-identical copies of the reference types and only add the plain
 * descriptors ApusCudaLayerDesc / ApusCudaModelDesc used below */
#include "../include/apus_b200.h"

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

/* c/layer.h:495 apus_block_forward on an ApusLayer assembled from a descriptor. */
static void shim_fill_layer(ApusLayer *L, ApusRopeTab *tab, const ApusCudaLayerDesc *d,
                            int hc, int iters, float hc_eps, float norm_eps) {
    memset(L, 0, sizeof *L);
    L->cfg.dim = d->acfg.dim;
    L->cfg.hc_mult = hc;
    L->cfg.hc_sinkhorn_iters = iters;
    L->cfg.hc_eps = hc_eps;
    L->cfg.norm_eps = norm_eps;
    L->cfg.n_activated_experts = d->mw.topk;
    L->ratio = d->acfg.ratio;
    L->hash = d->mw.hash;
    L->attn_norm_w = (float *)d->attn_norm_w;
    L->ffn_norm_w = (float *)d->ffn_norm_w;
    L->hc_attn_fn = (float *)d->hc_attn_fn; L->hc_attn_base = (float *)d->hc_attn_base;
    L->hc_attn_scale = (float *)d->hc_attn_scale;
    L->hc_ffn_fn = (float *)d->hc_ffn_fn; L->hc_ffn_base = (float *)d->hc_ffn_base;
    L->hc_ffn_scale = (float *)d->hc_ffn_scale;
    L->acfg = d->acfg; L->aw = d->aw; L->mw = d->mw;
    memset(tab, 0, sizeof *tab);
    tab->rd = d->acfg.rope_dim;
    tab->cap = d->rope_rows;              /* fully built: apus_rope_tab_ensure never grows it */
    tab->cos = (float *)d->cos; tab->sin = (float *)d->sin;
    L->rope = tab;
}

/* `interm` (nullable) is the reference's ApusInterm (c/layer.h:88-104). */
void ref_block_forward_interm(const ApusCudaLayerDesc *d, int hc, int iters, float hc_eps, float norm_eps,
                              ApusAttnS *st, float *h, const int64_t *ids, int s, int64_t start_pos,
                              void *interm) {
    ApusLayer L;
    ApusRopeTab tab;
    ApusLayerState ls;
    shim_fill_layer(&L, &tab, d, hc, iters, hc_eps, norm_eps);
    ls.attn = *st;
    apus_block_forward(&L, &ls, h, ids, s, start_pos, (ApusInterm *)interm);
    *st = ls.attn;
}

void ref_block_forward(const ApusCudaLayerDesc *d, int hc, int iters, float hc_eps, float norm_eps,
                       ApusAttnS *st, float *h, const int64_t *ids, int s, int64_t start_pos) {
    ref_block_forward_interm(d, hc, iters, hc_eps, norm_eps, st, h, ids, s, start_pos, NULL);
}

/* c/model.h:722 apus_model_forward on an ApusModel assembled from a descriptor.
 * states[i] is layer i's attention state; *pos is advanced by s. */
typedef struct {
    ApusModel m;
    ApusModelState st;
    ApusLayer *Ls;
    ApusRopeTab *tabs;
    ApusLayerState *lst;
    ApusStTensor te, th;
} ShimModel;

static void shim_model_open(ShimModel *S, const ApusCudaModelDesc *d, ApusAttnS *states, int64_t pos) {
    memset(S, 0, sizeof *S);
    ApusModel *m = &S->m;
    m->n_layers = d->n_layers;
    m->cfg.dim = d->dim; m->cfg.hc_mult = d->hc_mult; m->cfg.vocab_size = d->vocab;
    m->cfg.hc_eps = d->hc_eps; m->cfg.norm_eps = d->norm_eps; m->cfg.hc_sinkhorn_iters = d->hc_sinkhorn_iters;
    m->cfg.n_activated_experts = d->layers[0].mw.topk;
    m->cfg.max_pos = d->layers[0].acfg.max_pos;
    S->Ls = calloc((size_t)d->n_layers, sizeof *S->Ls);
    S->tabs = calloc((size_t)d->n_layers, sizeof *S->tabs);
    S->lst = calloc((size_t)d->n_layers, sizeof *S->lst);
    for (int i = 0; i < d->n_layers; i++) {
        shim_fill_layer(&S->Ls[i], &S->tabs[i], &d->layers[i], d->hc_mult, d->hc_sinkhorn_iters, d->hc_eps, d->norm_eps);
        S->Ls[i].cfg.vocab_size = d->vocab;
        S->lst[i].attn = states[i];
    }
    m->layers = S->Ls;
    S->te.dtype = d->embed_bf16 ? APUS_ST_BF16 : APUS_ST_F32; S->te.data = d->embed;
    S->th.dtype = d->head_bf16 ? APUS_ST_BF16 : APUS_ST_F32; S->th.data = d->head;
    m->embed = &S->te; m->head = &S->th;
    m->norm_w = (float *)d->norm_w;
    m->hc_head_fn = (float *)d->hc_head_fn; m->hc_head_base = (float *)d->hc_head_base;
    m->hc_head_scale = d->hc_head_scale;
    S->st.layers = S->lst; S->st.pos = pos;
}
static void shim_model_close(ShimModel *S, ApusAttnS *states, int64_t *pos) {
    *pos = S->st.pos;
    for (int i = 0; i < S->m.n_layers; i++) states[i] = S->lst[i].attn;
    free(S->Ls); free(S->tabs); free(S->lst);
}

/* c/model.h:722 apus_model_forward on an ApusModel assembled from a descriptor.
 * states[i] is layer i's attention state; *pos is advanced by s. */
void ref_model_forward(const ApusCudaModelDesc *d, ApusAttnS *states, int64_t *pos,
                       const int64_t *ids, int s, float *logits, int logits_all) {
    ShimModel S;
    shim_model_open(&S, d, states, *pos);
    apus_model_forward(&S.m, &S.st, ids, s, logits, logits_all);
    shim_model_close(&S, states, pos);
}

/* c/model.h:731-743 apus_model_forward_h / _mh: h_out [s, hc*dim] or, with the target layers
 * given, mh_out [s, n_targets*dim] (both nullable). */
void ref_model_forward_hm(const ApusCudaModelDesc *d, ApusAttnS *states, int64_t *pos, const int64_t *ids, int s,
                          float *logits, int logits_all, float *h_out, const int *targets, int n_targets,
                          float *mh_out) {
    ShimModel S;
    shim_model_open(&S, d, states, *pos);
    if (mh_out) {
        S.m.dspark = 1;
        S.m.dsc.n_targets = n_targets;
        for (int i = 0; i < n_targets; i++) S.m.dsc.targets[i] = targets[i];
        apus_model_forward_mh(&S.m, &S.st, ids, s, logits, logits_all, mh_out);
    } else {
        apus_model_forward_h(&S.m, &S.st, ids, s, logits, logits_all, h_out);
    }
    shim_model_close(&S, states, pos);
}

static void shim_fill_mtp(ApusMtp *mt, ApusRopeTab *tab, const ApusModel *m, const ApusCudaMtpDesc *md,
                          const ApusCudaModelDesc *d) {
    memset(mt, 0, sizeof *mt);
    mt->m = m;
    shim_fill_layer(&mt->block, tab, &md->block, d->hc_mult, d->hc_sinkhorn_iters, d->hc_eps, d->norm_eps);
    mt->block.cfg.vocab_size = d->vocab;
    mt->e_proj = md->e_proj; mt->h_proj = md->h_proj;
    mt->enorm_w = (float *)md->enorm_w; mt->hnorm_w = (float *)md->hnorm_w; mt->norm_w = (float *)md->norm_w;
    mt->hc_head_fn = (float *)md->hc_head_fn; mt->hc_head_base = (float *)md->hc_head_base;
    mt->hc_head_scale = md->hc_head_scale;
}

/* c/mtp.h:303 apus_mtp_forward on an ApusMtp assembled from descriptors (the parent model only
 * lends its embedding, head and sizes). */
void ref_mtp_forward(const ApusCudaModelDesc *d, const ApusCudaMtpDesc *md, ApusAttnS *mtp_state, const float *h_in,
                     const int64_t *ids, int s, int64_t start_pos, float *logits, float *h_last) {
    ShimModel S;
    ApusAttnS none[64];
    memset(none, 0, sizeof none);
    int64_t pos = 0;
    shim_model_open(&S, d, none, 0);
    ApusMtp mt;
    ApusRopeTab tab;
    ApusMtpState mst;
    shim_fill_mtp(&mt, &tab, &S.m, md, d);
    mst.block.attn = *mtp_state;
    apus_mtp_forward(&mt, &mst, h_in, ids, s, start_pos, logits, h_last);
    *mtp_state = mst.block.attn;
    shim_model_close(&S, none, &pos);
}

/* c/mtp.h:472-616 apus_spec_prefill + apus_spec_step until n_gen tokens are out, with the MTP head
 * as the proposer (greedy).  out_tokens [n_gen]; stats [8] = emitted, batches, batch_tokens,
 * refeed_tokens, offered, accepted, d1_offered, d1_hits; first_drafts [depth] = the chain after
 * the prompt. */
int ref_spec_generate_mtp(const ApusCudaModelDesc *d, const ApusCudaMtpDesc *md, ApusAttnS *states,
                          ApusAttnS *mtp_state, const int64_t *prompt, int n_prompt, int n_gen, int depth,
                          int32_t *out_tokens, uint64_t *stats, int64_t *first_drafts) {
    ShimModel S;
    int64_t pos = 0;
    shim_model_open(&S, d, states, 0);
    ApusMtp mt;
    ApusRopeTab tab;
    ApusMtpState mst;
    shim_fill_mtp(&mt, &tab, &S.m, md, d);
    mst.block.attn = *mtp_state;
    ApusSpec sp;
    ApusRng rng;
    apus_rng_seed(&rng, 0);
    apus_spec_init(&sp, &S.m, &S.st, &mt, &mst, depth, 0.0f, 1.0f, &rng, NULL);
    apus_spec_prefill(&sp, prompt, n_prompt);
    for (int i = 0; i < depth; i++) first_drafts[i] = sp.drafts[i];
    int n = 0, buf[80];
    while (n < n_gen) {
        int ne = apus_spec_step(&sp, buf, 80);
        if (ne <= 0) break;
        for (int i = 0; i < ne && n < n_gen; i++) out_tokens[n++] = buf[i];
    }
    uint64_t st8[8] = {sp.emitted, sp.batches, sp.batch_tokens, sp.refeed_tokens, sp.offered, sp.accepted,
                       sp.d1_offered, sp.d1_hits};
    memcpy(stats, st8, sizeof st8);
    apus_spec_free(&sp);
    *mtp_state = mst.block.attn;
    shim_model_close(&S, states, &pos);
    return n;
}

/* An ApusDspark assembled from descriptors (c/dspark.h:88-107); tabs [n_stages]. */
static void shim_fill_dspark(ApusDspark *ds, ApusRopeTab *tabs, ApusModel *m, const ApusCudaDsparkDesc *dd,
                             const ApusCudaModelDesc *d) {
    memset(ds, 0, sizeof *ds);
    m->dspark = 1;
    m->dsc.block_size = dd->block_size; m->dsc.noise_id = dd->noise_id; m->dsc.markov_rank = dd->markov_rank;
    m->dsc.n_stages = dd->n_stages; m->dsc.n_targets = dd->n_targets;
    for (int i = 0; i < dd->n_targets; i++) m->dsc.targets[i] = dd->targets[i];
    ds->m = m;
    ds->cfg = m->dsc;
    ds->n_stages = dd->n_stages;
    for (int k = 0; k < dd->n_stages; k++) {
        shim_fill_layer(&ds->stages[k], &tabs[k], &dd->stages[k], d->hc_mult, d->hc_sinkhorn_iters, d->hc_eps, d->norm_eps);
        ds->stages[k].cfg.vocab_size = d->vocab;
    }
    ds->main_proj = dd->main_proj;
    ds->main_norm_w = (float *)dd->main_norm_w; ds->norm_w = (float *)dd->norm_w;
    ds->hc_head_fn = (float *)dd->hc_head_fn; ds->hc_head_base = (float *)dd->hc_head_base;
    ds->hc_head_scale = dd->hc_head_scale;
    ds->markov_w1 = (float *)dd->markov_w1; ds->markov_w2 = (float *)dd->markov_w2; ds->conf_proj = (float *)dd->conf_proj;
}

/* c/dspark.h:365-455, 611: stage-0 projection + ring prefill over the n main-hidden rows mh_all, then one
 * draft round at start_pos = n - 1 from the last row (greedy); stage_states [n_stages] in/out. */
void ref_dspark_prefill_round_t(const ApusCudaModelDesc *d, const ApusCudaDsparkDesc *dd, ApusAttnS *stage_states,
                                const float *mh_all, int n, int64_t anchor, float temp, uint64_t draft_seed,
                                int64_t *drafts, float *confidence, float *logits_final, float *stage_h);
void ref_dspark_prefill_round(const ApusCudaModelDesc *d, const ApusCudaDsparkDesc *dd, ApusAttnS *stage_states,
                              const float *mh_all, int n, int64_t anchor, int64_t *drafts, float *confidence,
                              float *logits_final, float *stage_h) {
    ref_dspark_prefill_round_t(d, dd, stage_states, mh_all, n, anchor, 0.0f, 1, drafts, confidence, logits_final, stage_h);
}
/* the same with the draft picks drawn at `temp` from a stream seeded with draft_seed (c/dspark.h:666-676) */
void ref_dspark_prefill_round_t(const ApusCudaModelDesc *d, const ApusCudaDsparkDesc *dd, ApusAttnS *stage_states,
                                const float *mh_all, int n, int64_t anchor, float temp, uint64_t draft_seed,
                                int64_t *drafts, float *confidence, float *logits_final, float *stage_h) {
    ShimModel S;
    ApusAttnS none[64];
    memset(none, 0, sizeof none);
    int64_t pos = 0;
    shim_model_open(&S, d, none, 0);
    ApusDspark ds;
    ApusRopeTab tabs[APUS_DSPARK_MAX_STAGES];
    ApusDsparkState dst;
    shim_fill_dspark(&ds, tabs, &S.m, dd, d);
    for (int k = 0; k < ds.n_stages; k++) dst.stages[k].attn = stage_states[k];
    int dim = d->dim, hcd = d->hc_mult * d->dim, B = dd->block_size;
    float *mx = malloc((size_t)n * dim * sizeof(float));
    apus_dspark_stage0_project(&ds, mh_all, n, mx);
    apus_dspark_prefill(&ds, &dst, mx, n);
    ApusDsparkDbg dbg;
    memset(&dbg, 0, sizeof dbg);
    dbg.confidence = confidence; dbg.logits_final = logits_final;
    for (int k = 0; k < ds.n_stages && stage_h; k++) dbg.stage_h[k] = stage_h + (size_t)k * B * hcd;
    ApusRng drng;
    apus_rng_seed(&drng, draft_seed);
    apus_dspark_draft_round(&ds, &dst, anchor, mx + (size_t)(n - 1) * dim, n - 1, temp, &drng, NULL, drafts, &dbg);
    free(mx);
    for (int k = 0; k < ds.n_stages; k++) stage_states[k] = dst.stages[k].attn;
    shim_model_close(&S, none, &pos);
}

/* c/dspark.h:747-862 apus_dspec_prefill + apus_dspec_step until n_gen tokens are out (greedy).  stats [7] =
 * emitted, batches, batch_tokens, refeed_tokens, offered, accepted, bonus_rounds. */
int ref_spec_generate_dspark_t(const ApusCudaModelDesc *d, const ApusCudaDsparkDesc *dd, ApusAttnS *states,
                               ApusAttnS *stage_states, const int64_t *prompt, int n_prompt, int n_gen, float temp,
                               float top_p, uint64_t rng_seed, uint64_t draft_seed, int32_t *out_tokens, uint64_t *stats);
int ref_spec_generate_dspark(const ApusCudaModelDesc *d, const ApusCudaDsparkDesc *dd, ApusAttnS *states,
                             ApusAttnS *stage_states, const int64_t *prompt, int n_prompt, int n_gen,
                             int32_t *out_tokens, uint64_t *stats) {
    return ref_spec_generate_dspark_t(d, dd, states, stage_states, prompt, n_prompt, n_gen, 0.0f, 1.0f, 0, 7, out_tokens, stats);
}
/* the same with a sampled main stream (temp, top_p, stream seeded with rng_seed) and drafts drawn at temp from a
 * stream of their own (draft_seed), as apus_dspec_init sets them up */
int ref_spec_generate_dspark_t(const ApusCudaModelDesc *d, const ApusCudaDsparkDesc *dd, ApusAttnS *states,
                               ApusAttnS *stage_states, const int64_t *prompt, int n_prompt, int n_gen, float temp,
                               float top_p, uint64_t rng_seed, uint64_t draft_seed, int32_t *out_tokens, uint64_t *stats) {
    ShimModel S;
    int64_t pos = 0;
    shim_model_open(&S, d, states, 0);
    ApusDspark ds;
    ApusRopeTab tabs[APUS_DSPARK_MAX_STAGES];
    ApusDsparkState dst;
    shim_fill_dspark(&ds, tabs, &S.m, dd, d);
    for (int k = 0; k < ds.n_stages; k++) dst.stages[k].attn = stage_states[k];
    ApusDspec sp;
    ApusRng rng;
    apus_rng_seed(&rng, rng_seed);
    apus_dspec_init(&sp, &S.m, &S.st, &ds, &dst, temp, top_p, &rng, draft_seed, NULL);
    apus_dspec_prefill(&sp, prompt, n_prompt);
    int n = 0, buf[80];
    while (n < n_gen) {
        int ne = apus_dspec_step(&sp, buf, 80);
        if (ne <= 0) break;
        for (int i = 0; i < ne && n < n_gen; i++) out_tokens[n++] = buf[i];
    }
    uint64_t s7[7] = {sp.emitted, sp.batches, sp.batch_tokens, sp.refeed_tokens, sp.offered, sp.accepted, sp.bonus_rounds};
    memcpy(stats, s7, sizeof s7);
    apus_dspec_free(&sp);
    for (int k = 0; k < ds.n_stages; k++) stage_states[k] = dst.stages[k].attn;
    shim_model_close(&S, states, &pos);
    return n;
}

/* c/model.h:638-647 (static apus_head_gemv) on a BF16 [O, K] matrix. */
void ref_head_gemv(const void *w_bf16, const float *x, float *out, int64_t O, int64_t K) {
    ApusStTensor t;
    memset(&t, 0, sizeof t);
    t.dtype = APUS_ST_BF16;
    t.data = w_bf16;
    apus_head_gemv(&t, x, out, O, K);
}

/* c/model.h:392 apus_model_load on a checkpoint directory, then the greedy loop
 * of c/apus.c:895-944 on the loaded model: what the reference's own loader makes
 * of the files.  cfg_out receives the parsed ApusCfg followed by n_layers, bos,
 * eos, n_mtp, mtp_ratio, mtp_hash, dspark (the layout of ApusCudaCkptCfg);
 * ratios/hash [n_layers]; wo_a0 = layer 0's BF16 wo_a; rope rows [0, rope_rows)
 * of the two table classes.  Returns 0, or -1 with err filled. */
int ref_ckpt_run(const char *dir, const int64_t *prompt, int n_prompt, int n_gen,
                 int32_t *tokens, float *logits, void *cfg_out, int *ratios, int *hash,
                 uint16_t *wo_a0, size_t n_wo, int rope_rows, float *cos_plain,
                 float *sin_plain, float *cos_yarn, float *sin_yarn, char *err, size_t errcap) {
    ApusModel m;
    if (apus_model_load(&m, dir, err, errcap)) return -1;
    if (cfg_out) {
        ApusCudaCkptCfg *o = cfg_out;
        memcpy(o, &m.cfg, sizeof m.cfg);
        o->n_layers = m.n_layers; o->bos_id = m.bos_id; o->eos_id = m.eos_id;
        o->n_mtp = m.n_mtp; o->mtp_ratio = m.mtp_ratio; o->mtp_hash = m.mtp_hash; o->dspark = m.dspark;
    }
    for (int i = 0; i < m.n_layers; i++) {
        if (ratios) ratios[i] = m.layers[i].ratio;
        if (hash) hash[i] = m.layers[i].hash;
    }
    if (wo_a0) memcpy(wo_a0, m.layers[0].wo_a, n_wo * sizeof(uint16_t));
    int half = m.cfg.rope_head_dim / 2;
    for (int cls = 0; cls < 2 && rope_rows > 0; cls++) {
        ApusRopeTab *t = apus_rope_tab_get(&m.cfg, cls ? 4 : 0);
        apus_rope_tab_ensure(t, rope_rows);
        memcpy(cls ? cos_yarn : cos_plain, t->cos, (size_t)rope_rows * half * sizeof(float));
        memcpy(cls ? sin_yarn : sin_plain, t->sin, (size_t)rope_rows * half * sizeof(float));
    }
    if (n_gen > 0) {
        int V = m.cfg.vocab_size;
        ApusModelState st;
        apus_model_state_init(&st, &m);
        float *lg = malloc((size_t)V * sizeof(float));
        apus_model_forward(&m, &st, prompt, n_prompt, lg, 0);
        for (int g = 0; g < n_gen; g++) {
            int tok = apus_sample_argmax(lg, (size_t)V);
            tokens[g] = tok;
            if (logits) memcpy(logits + (size_t)g * V, lg, (size_t)V * sizeof(float));
            if (g + 1 < n_gen) {
                int64_t id = tok;
                apus_model_forward(&m, &st, &id, 1, lg, 0);
            }
        }
        free(lg);
        apus_model_state_free(&st, &m);
    }
    apus_model_free(&m);
    return 0;
}

/* c/model.h:195 (static apus_model_parse_config) alone: cfg_out as in ref_ckpt_run,
 * ratios/hash up to cap entries.  Returns 0, or -1 with err filled. */
int ref_parse_config(const char *path, void *cfg_out, int *ratios, int *hash, int cap,
                     char *err, size_t errcap) {
    ApusCfg c;
    ApusDsparkCfg dsc;
    int n_layers = 0, *r = NULL, *h = NULL, bos, eos, n_mtp, mtp_ratio, mtp_hash, dspark;
    if (apus_model_parse_config(&c, &n_layers, &r, &h, &bos, &eos, &n_mtp, &mtp_ratio,
                                &mtp_hash, &dspark, &dsc, path, err, errcap))
        return -1;
    ApusCudaCkptCfg *o = cfg_out;
    memset(o, 0, sizeof *o);
    memcpy(o, &c, sizeof c);
    o->n_layers = n_layers; o->bos_id = bos; o->eos_id = eos;
    o->n_mtp = n_mtp; o->mtp_ratio = mtp_ratio; o->mtp_hash = mtp_hash; o->dspark = dspark;
    for (int i = 0; i < n_layers && i < cap; i++) { ratios[i] = r[i]; hash[i] = h[i]; }
    free(r); free(h);
    return 0;
}
