/*
 * apus_b200.h — C ABI of libapus_b200.so: the B200 (sm_100a) backend for the
 * decode/prefill arithmetic of the apus DeepSeek-V4-Flash engine.
 *
 * Two tiers, both plain C (pointers + sizes, no C++/torch types):
 *
 *  1. HOST-POINTER tier — drop-in twins of the reference's backend plugin table
 *     and of the kernel/sublayer functions it calls.  Every buffer is
 *     caller-owned host memory, results are in the host `out` buffer on return
 *     (synchronous), weights are uploaded once and cached by host address.
 *     Same names (apus_cuda_* for apus_metal_* / apus_*), argument meaning and
 *     error convention as the reference: 0 = result produced, nonzero =
 *     failed (message in apus_cuda_last_error()).  There is NO CPU fallback
 *     inside this library: without a usable CUDA device every call fails.
 *
 *  2. DEVICE-RESIDENT tier (`*_dev`) — the same operators on device pointers and
 *     a caller-supplied CUDA stream (passed as void*), asynchronous, no
 *     host<->device copies.  This is what a fused token loop and the
 *     expert-parallel multi-GPU path are built from.
 *
 * Each declaration cites the reference interface it replaces as
 * `file:line` relative to the reference project root.
 *
 * Data formats (reference c/st.h:88-89, c/fp4.h:8-11, c/fp8.h:11-14):
 *   MXFP4 weight  packed u8 [O, K/2] row-major, low nibble = even K; E2M1 codes
 *                 scales u8 [O, K/32] UE8M0 (value 2^(b-127))
 *   FP8 weight    codes  u8 [O, K] E4M3; scales u8 [ceil(O/128), ceil(K/128)] UE8M0
 *   activations   f32 carrying BF16 values; quantised per token per 128 along K
 *                 to E4M3 codes with a power-of-two f32 scale
 */
#ifndef APUS_B200_H
#define APUS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- types shared with the reference (layout-identical) ------------------ */

#ifndef APUS_ST_H
/* c/st.h:88 */
typedef struct { const uint8_t *codes, *scales; int64_t O, K; } ApusFp8W;
/* c/st.h:89 */
typedef struct { const uint8_t *packed, *scales; int64_t O, K; } ApusFp4W;
#endif

#ifndef APUS_MOE_H
/* c/moe.h:37-63 */
typedef struct {
    int E, topk, inter, dim, hash;
    float route_scale, limit;
    const float *gate_w;      /* [E, dim] BF16-valued f32 */
    const float *gate_bias;   /* [E] f32, NULL when hash */
    const int64_t *tid2eid;   /* [vocab, topk], NULL unless hash */
    ApusFp4W *w1, *w2, *w3;   /* [E] routed experts (MXFP4) */
    ApusFp8W sw1, sw2, sw3;   /* shared expert (FP8) */
    void *hook_ctx;
    int  (*hook_resolve)(void *ctx, int layer, int eid,
                         ApusFp4W *w1, ApusFp4W *w2, ApusFp4W *w3);
    void (*hook_hint)(void *ctx, int layer, int eid);
    void (*hook_layer_end)(void *ctx, int layer);
    void *hook_hint_ctx;
    void *hook_layer_end_ctx;
    int layer_id;
} ApusMoeW;

/* c/moe.h:67-71 — optional named intermediates (NULL members are skipped). */
typedef struct {
    float *router_scores, *router_scores_biased, *router_w;
    int32_t *router_idx;
    float *moe_routed, *moe_shared;
} ApusMoeInterm;
#endif

#ifndef APUS_ATTN_H
/* c/attn.h:114-122 */
typedef struct {
    int dim, n_heads, head_dim, rope_dim, q_lora, o_groups, o_lora;
    int window, ratio;              /* ratio == 0 => sliding window only */
    int has_indexer;                /* ratio == 4 */
    int idx_heads, idx_dim, idx_topk;
    float eps;
    int max_pos;
} ApusAttnCfg;
/* c/attn.h:126-130 — compressor weights: wkv/wgate [coff*d, dim] f32, ape
 * [ratio, coff*d], norm [d]; coff = 1 + overlap. */
typedef struct {
    const float *wkv, *wgate, *ape, *norm;
    int ratio, overlap, d, rd, rotate;
    float eps;
} ApusCompW;
/* c/attn.h:132-143 */
typedef struct {
    ApusFp8W wq_a, wq_b, wkv, wo_b;
    const uint16_t *wo_a;   /* [G*o_lora, h*d/G] BF16 bits */
    const float *q_norm, *kv_norm, *sink;
    ApusCompW comp, idx_comp;
    ApusFp8W idx_wq_b;
    const float *idx_wproj; /* [idx_heads, dim] */
} ApusAttnW;
/* c/attn.h:147-153 — compressor state: carries kv/sc [rows, cols] (sc starts at
 * -inf), cache [cap, d] of finished entries, nb entries valid. */
typedef struct {
    int rows, cols;
    float *kv, *sc;
    float *cache;
    int nb, max_nb, d;
    int cap;
} ApusCompS;
/* c/attn.h:155-160 */
typedef struct {
    int64_t pos;
    float *win;             /* [window, head_dim] ring */
    ApusCompS comp, idx_comp;
} ApusAttnS;
/* c/attn.h:168-173 — optional named intermediates. */
typedef struct {
    float *q, *win_kv, *comp_kv, *idx_comp_kv, *idx_scores;
    int32_t *idx_topk;
    float *attn_out, *o_out;
    int comp_nb, idx_nb, idx_k;
} ApusAttnInterm;
#endif

#ifndef APUS_FP4_H
/* c/fp4.h:184-188 — one entry of a grouped MXFP4 GEMM. */
typedef struct {
    const uint8_t *w, *ws;   /* [O, K/2] / [O, K/32] */
    float *out;              /* [M, O] row-major */
    size_t m0, M;            /* rows [m0, m0+M) of the shared activation space */
} ApusFp4GemmEnt;
#endif

/* c/backend_metal.h:57-61 — f32_linear flags. */
#define APUS_CUDA_R_IN   1   /* BF16-round the input elements */
#define APUS_CUDA_R_OUT  2   /* BF16-round the outputs */
#define APUS_CUDA_W_BF16 4   /* w points at BF16 bits (u16), not f32 */

/* c/backend_metal.h:73-80 — the plugin table.  head_gemv's first argument is
 * the reference's ApusStTensor*; only its dtype/data members are read (see
 * apus_cuda_fill_hooks). */
typedef struct {
    int (*fp8_linear)(const ApusFp8W *w, const float *x, float *out,
                      int M, int K, int O);
    int (*f32_linear)(const float *w, const float *x, float *out,
                      int M, int K, int O, int flags);
    int (*head_gemv)(const void *head_sttensor, const float *x, float *out,
                     int64_t O, int64_t K);
} ApusCudaHooks;

/* ---- lifecycle (c/backend_metal.h:88-97) ---------------------------------- */

/* c/backend_metal.h:88 apus_metal_enable. Selects the current CUDA device,
 * creates the backend stream and workspace. Idempotent. */
int  apus_cuda_enable(char *err, size_t errcap);
/* c/backend_metal.h:90 apus_metal_disable. Drops the weight cache and frees
 * all device memory held by the host-pointer tier. */
void apus_cuda_disable(void);
/* c/backend_metal.h:91 */
int  apus_cuda_is_enabled(void);
/* c/backend_metal.h:96 — weight bytes uploaded into the device cache. */
uint64_t apus_cuda_bytes_uploaded(void);
/* c/backend_metal.h:97 — kernels launched by this library since load. */
uint64_t apus_cuda_dispatches(void);
/* Fills the three hook slots (c/backend_metal.h:73-80; the assignment done by
 * apus_metal_enable at c/backend_metal.mm:738). `struct_dtype_off` and
 * `struct_data_off` are offsetof(ApusStTensor, dtype) / offsetof(.., data) in
 * the caller's build, so this library need not know that struct. */
int  apus_cuda_fill_hooks(ApusCudaHooks *hooks, size_t struct_dtype_off,
                          size_t struct_data_off);
/* Message of the most recent failure on the calling thread ("" if none). */
const char *apus_cuda_last_error(void);
/* Device-side waits (mbarriers of the TMA/tcgen05 pipeline) are bounded: when one
 * expires the kernel records a code, frees its tensor memory and returns
 * instead of hanging.  Returns the first code recorded since the last reset
 * (0 = none); synchronises the device. */
int apus_cuda_kernel_status(int reset);
/* Order of the long f32 sums whose result the reference defines by its loop
 * order: the mHC map dots and sum of squares (c/mhc.h:159-176), the RMSNorm
 * sum of squares (c/attn.h:371-378), the dense f32/BF16 linears (c/attn.h:460-465).
 *   APUS_CUDA_SUM_REFERENCE: one accumulator, index ascending, products rounded
 *     before each add -- the bits of the CPU path; the sums become chains of
 *     dependent adds (about 35 us per mHC map at hc_mult 4 x dim 4096).
 *   APUS_CUDA_SUM_TREE: pairwise tree / tensor-core sums with FMA; faster and
 *     closer to the exact sum, but off the reference by ~1e-6..1e-5 relative, which
 *     can flip a BF16 step downstream (the reference's own NEON and BLAS variants
 *     differ from its scalar code by as much, c/mhc.h:296-330, c/blas.h:25-40).
 * The choice is per operator class (apus_cuda_set_tree_ops, a bit mask of the
 * classes summed in tree order; mask == -1 only queries and returns the mask in
 * force; mask == -2 returns APUS_CUDA_TREE_DEFAULT and changes nothing).
 * apus_cuda_set_sum_order(REFERENCE / TREE) clears / sets every class; order < 0
 * only queries; it returns TREE only when every class is in tree order.
 * Environment at load time: APUS_TREE_OPS=<mask>, or APUS_SUM_ORDER=1 for all. */
#define APUS_CUDA_SUM_REFERENCE 0
#define APUS_CUDA_SUM_TREE 1
#define APUS_CUDA_TREE_MHC_MAPS   1    /* mHC map dots + sum of squares over hc_mult*dim */
#define APUS_CUDA_TREE_NORMS      2    /* RMSNorm sums of squares (norm, q/kv norm rows, mHC collapse + norm) */
#define APUS_CUDA_TREE_HEAD       4    /* vocabulary head: logits are unrounded and feed only the pick */
#define APUS_CUDA_TREE_WO_A       8    /* grouped low-rank o-projection (c/attn.h:1692-1737) */
#define APUS_CUDA_TREE_ROUTER    16    /* router gate matmul (c/moe.h:352-367) */
#define APUS_CUDA_TREE_COMPRESSOR 32   /* compressor wkv / wgate projections (c/attn.h:892-1011) */
#define APUS_CUDA_TREE_IDX_WPROJ 64    /* indexer weights projection (c/attn.h:1105-1168) */
#define APUS_CUDA_TREE_LINEAR   128    /* apus_cuda_f32_linear / the f32_linear hook */
#define APUS_CUDA_TREE_FP8_SPLITK 256  /* reserved (the FP8 K split adds the per-block terms in block order: the
                                          bits of the single fold, c/fp8.h:166-218, so it needs no setting) */
#define APUS_CUDA_TREE_ALL      511
/* The classes in tree order when nothing else is asked for: those the reference's own
 * ARM build sums in another order than its scalar code (the mHC map dots and sum of
 * squares, c/mhc.h:288-316; the o-projection, c/attn.h:1457-1466, "accepted SIMD
 * tolerance class") and the head, whose unrounded logits only feed the pick.  The
 * norms, the router gate, the compressor and indexer projections (c/attn.h:450-458:
 * "leave no room for reorder noise") and the FP8 fold keep the reference's order. */
#define APUS_CUDA_TREE_DEFAULT  (1 + 4 + 8)
int apus_cuda_set_tree_ops(int mask);
int apus_cuda_set_sum_order(int order);
/* Calls that carry s > 1 positions (apus_cuda_attention, apus_cuda_block_forward,
 * apus_cuda_model_forward / _generate on the prompt) run them as chunks of positions: every
 * weight is read once per chunk, rows are (position, sequence) pairs, and only the
 * attention state is walked in position order -- the batched forms of the reference
 * (c/attn.h:1621-1680 prefill, 1576-1620 mid-stream batch, c/moe.h:217-330 expert
 * grouping, c/model.h:651-720).  Each row goes through the operations of a single step in
 * the same order, so a chunk leaves the outputs and the state of s consecutive steps bit
 * for bit, whatever the chunk size (the reference's chunk invariance, tests/m4c).
 * `rows` = the most rows (positions x sequences) one chunk may hold; 0 = one step per
 * position; negative only queries.  Returns the previous value (default 2048;
 * environment at load time: APUS_PREFILL=<rows>). */
int apus_cuda_set_prefill_chunk(int rows);
/* Run the entry points that take no stream argument (host-pointer tier, model
 * loop) on the caller's stream instead of the library's own, e.g. to order them
 * with the caller's collectives without events; use_own != 0 switches back.
 * The previous stream is synchronised first. */
int apus_cuda_use_stream(void *stream, int use_own);
/* Forget the cached device copy of a weight buffer (the reference frees and
 * reuses host addresses between tests, tests/m7b/README.md:90-94). */
void apus_cuda_forget(const void *host_ptr);

/* ---- host-pointer tier: kernel-level entry points ------------------------- */

/* c/sample.h:66-67 apus_sample_logits_u for `rows` rows: logits [rows, n], one
 * explicit uniform u[row] in [0, 1) per row (unused when temp <= 0: greedy),
 * tokens [rows].  The nucleus walk over the sorted probabilities is a weighted
 * selection on the device (no sort); see csrc/sample.cu. */
int apus_cuda_sample_logits_u(const float *logits, size_t n, float temp, float top_p,
                              const double *u, int32_t *tokens, int rows);

/* c/backend_metal.h:102 apus_metal_fp8_linear == c/attn.h:408 apus_fp8_linear:
 * BF16-round x, per-128 act quant, block-scaled FP8 GEMM, BF16-rounded out. */
int apus_cuda_fp8_linear(const ApusFp8W *w, const float *x, float *out,
                         int M, int K, int O);
/* c/attn.h:432 apus_fp4_linear (no reference hook exists for it). */
int apus_cuda_fp4_linear(const ApusFp4W *w, const float *x, float *out,
                         int M, int K, int O);
/* c/backend_metal.h:104 apus_metal_f32_linear == c/attn.h:621/652
 * apus_bf16_linear / apus_f32_linear and the wo_a groups (c/attn.h:1698). */
int apus_cuda_f32_linear(const float *w, const float *x, float *out,
                         int M, int K, int O, int flags);
/* c/backend_metal.h:106 apus_metal_head_gemv_bf16 == c/model.h:638. */
int apus_cuda_head_gemv_bf16(const void *w_bf16, const float *x, float *out,
                             int64_t O, int64_t K);
/* c/backend_metal.h:110 apus_metal_fp8_gemm == c/fp8.h:136 apus_fp8_gemm_mt:
 * pre-quantised activations, unrounded f32 out. */
int apus_cuda_fp8_gemm(const uint8_t *w, const uint8_t *ws,
                       const uint8_t *acodes, const float *as, float *out,
                       int M, int O, int K);
/* c/fp4.h:166 apus_fp4_gemm_mt: pre-quantised activations, unrounded out. */
int apus_cuda_fp4_gemm(const uint8_t *w, const uint8_t *ws,
                       const uint8_t *acodes, const float *as, float *out,
                       int M, int O, int K);
/* c/fp4.h:166 apus_fp4_gemm_mt again, on the tcgen05 block-scaled tensor-core
 * path: the weights stay in the reference storage ([O,K/2] nibbles, [O,K/32]
 * scales) and are unpacked by TMA.  O and K multiples of 128. */
int apus_cuda_fp4_gemm_tc(const uint8_t *w, const uint8_t *ws,
                          const uint8_t *acodes, const float *as, float *out,
                          int M, int O, int K);
/* c/fp4.h:190 apus_fp4_gemm_mt_grouped: several same-(O,K) GEMMs sharing one
 * activation row space of `rows` rows (rows = max(m0+M) over the entries). */
int apus_cuda_fp4_gemm_grouped(const ApusFp4GemmEnt *ents, size_t n_ent,
                               const uint8_t *acodes, const float *as,
                               size_t rows, size_t O, size_t K);
/* c/backend_metal.h:115 apus_metal_fp8_act_quant == c/attn.h:393 row worker:
 * BF16 round + per-128 E4M3 quant. codes [M,K], scales [M, ceil(K/128)]. */
int apus_cuda_fp8_act_quant(const float *x, int M, int K,
                            uint8_t *codes, float *scales);
/* c/backend_metal.h:118 apus_metal_rmsnorm == c/attn.h:371 apus_rms_norm,
 * extended to `rows` independent rows of n (rows = 1 is the reference call). */
int apus_cuda_rmsnorm(const float *x, const float *w, float eps, float *y,
                      int64_t n, int64_t rows);
/* c/moe.h:333 apus_expert (static there) for `rows` tokens: SwiGLU FFN with
 * the limit clamps; kind 0 = MXFP4 (ApusFp4W*), 1 = FP8 (ApusFp8W*). */
int apus_cuda_expert(const void *w1, const void *w2, const void *w3, int kind,
                     float limit, const float *x, int rows, int dim, int inter,
                     float *out);
/* c/attn.h:668 apus_topk_stable for `rows` independent rows of n: strict
 * greater-than selection, lowest index wins ties, descending order out. */
int apus_cuda_topk_stable(const float *row, int n, int k, int32_t *idx,
                          int rows);

/* ---- host-pointer tier: sublayer entry points ------------------------------ */

/* c/moe.h:77 apus_router_score. */
int apus_cuda_router_score(const ApusMoeW *w, const float *x, int s,
                           float *sp, float *biased);
/* c/moe.h:82 apus_moe_forward. Expert weights are taken from w->w1/w2/w3 or,
 * when w->hook_resolve is set, resolved through it once per expert and
 * cached (the resolve/hint/layer_end hooks are storage tiering in the
 * reference; here every resolved expert stays resident in HBM). */
int apus_cuda_moe_forward(const ApusMoeW *w, const float *x,
                          const int64_t *ids, int s, float *out,
                          ApusMoeInterm *interm);
/* c/attn.h:1308 apus_sparse_attn (static there): index-gathered attention with
 * BF16 softmax numerator and the per-head sink in the denominator. */
int apus_cuda_sparse_attn(const float *q, const float *sink, int h, int d,
                          const int32_t *idxs, int idxw, int s, float scale,
                          const float *kv_a, int64_t na, const float *kv_b,
                          int64_t nb, float *o);
/* c/attn.h:178 apus_attention: the attention sublayer for s tokens of ONE
 * sequence starting at start_pos; x [s,dim], out [s,dim]; cos/sin are the
 * layer's rope tables [>= start_pos+s, rope_dim/2]; `st` is the caller's host
 * state, read at entry and updated at exit exactly as the reference mutates it
 * (ring row(s), compressor carries, appended cache entries, nb; the caches
 * must have room: cap >= nb + new entries).  Tokens are processed as
 * consecutive decode steps, which the reference defines to be equal to its
 * batched prefill (tests/m4c chunk invariance).  interm: q, win_kv, attn_out,
 * o_out, comp_nb, idx_nb and (decode form: offsets relative to the ring)
 * idx_topk / idx_k are filled when non-NULL; the other members are ignored. */
int apus_cuda_attention(const ApusAttnCfg *cfg, const ApusAttnW *w,
                        ApusAttnS *st, const float *x, int s,
                        int64_t start_pos, const float *cos, const float *sin,
                        float *out, ApusAttnInterm *interm);
/* c/attn.h:76-90 row helpers on `rows` rows of n (stride n): apus_apply_rope
 * on the last rd elements with one cos/sin row [rd/2] each, apus_hadamard,
 * apus_fp8_qat_sim (per `group` = 64 on the first K elements), apus_fp4_qat_sim. */
int apus_cuda_apply_rope(float *x, const float *cos, const float *sin, int n,
                         int rd, int inverse, int rows);
int apus_cuda_hadamard(float *x, int n, int rows);
int apus_cuda_fp8_qat_sim(float *x, int n, int K, int rows);
int apus_cuda_fp4_qat_sim(float *x, int n, int rows);
/* c/mhc.h:103 apus_mhc_prepost_scalar for `rows` tokens (x4 [rows, n*d]). */
int apus_cuda_mhc_prepost(const float *x4, size_t d, size_t n,
                          const float *fn, const float *scale,
                          const float *base, float norm_eps, float hc_eps,
                          int iters, float *pre, float *post, float *comb,
                          int rows);
/* c/layer.h:401 apus_hc_pre_rows: mHC pre maps + collapse (c/mhc.h:110) + BF16
 * round, optionally followed by RMSNorm (c/attn.h:371) in the same kernel
 * when norm_w != NULL.  y [rows, d]; post [rows,n], comb [rows,n,n] out. */
int apus_cuda_hc_pre(const float *x4, size_t d, size_t n, const float *fn,
                     const float *scale, const float *base, float norm_eps,
                     float hc_eps, int iters, const float *norm_w,
                     float rms_eps, float *y, float *y_normed, float *post,
                     float *comb, int rows);
/* c/layer.h:445 apus_hc_post_rows: c/mhc.h:116 apply + BF16 round. */
int apus_cuda_hc_post(const float *f, const float *res4, const float *post,
                      const float *comb, float *y4, size_t d, size_t n,
                      int rows);
/* c/mhc.h:123 apus_mhc_head_scalar (+ BF16 round as c/model.h:711). */
int apus_cuda_hc_head(const float *x4, size_t d, size_t n, const float *fn,
                      float scale, const float *base, float norm_eps,
                      float hc_eps, float *y, int rows);

/* ---- device-resident tier --------------------------------------------------- */

/* Quantised-weight handles living in HBM. */
typedef struct ApusCudaFp4 ApusCudaFp4;   /* one MXFP4 matrix */
typedef struct ApusCudaFp8 ApusCudaFp8;   /* one FP8 matrix */
typedef struct ApusCudaMoe ApusCudaMoe;   /* one MoE sublayer (local experts) */

/* Upload the experts [e_lo, e_hi) of a MoE sublayer plus its gate and shared
 * expert (c/moe.h:37-63 describes the fields) into HBM.  e_lo/e_hi implement
 * the contiguous expert-parallel partition (expert e lives on rank
 * e / (E / world)).  Returns NULL on failure. */
ApusCudaMoe *apus_cuda_moe_create(const ApusMoeW *w, int e_lo, int e_hi);
void apus_cuda_moe_destroy(ApusCudaMoe *m);
/* Bytes of expert + dense weights resident for this sublayer. */
uint64_t apus_cuda_moe_bytes(const ApusCudaMoe *m);
/* The backend-owned handle that apus_cuda_moe_forward uses for `w` (all experts
 * local), created on first use and keyed by w->gate_w; freed by
 * apus_cuda_disable / apus_cuda_forget(w->gate_w).  Lets a caller mix the
 * host-pointer call with the *_dev calls on one resident copy of the weights. */
ApusCudaMoe *apus_cuda_moe_get(const ApusMoeW *w);
/* Selects the routed-expert kernel of this sublayer: 1 = tcgen05 block-scaled
 * MMA with TMA-unpacked weights in the reference storage (default when the
 * shapes are multiples of 128; APUS_MOE_TC=0 in the environment disables it at
 * creation), 0 = the mma.sync kernel on the re-tiled copy; a negative value
 * only queries.  Returns the setting in force.  Both compute c/moe.h:333-350. */
int apus_cuda_moe_use_tc(ApusCudaMoe *m, int enable);
/* Per-kernel timing of the two expert GEMM launches (gate/up pair, down) with
 * CUDA events on the launching stream — the counterpart of the reference's
 * dispatch counters (c/backend_metal.h:93-97) for roofline reporting.
 * _timing_read sums the elapsed milliseconds recorded since the last read. */
void apus_cuda_moe_timing(ApusCudaMoe *m, int enable);
int apus_cuda_moe_timing_enabled(const ApusCudaMoe *m);
int apus_cuda_moe_timing_read(ApusCudaMoe *m, double *ms_gate_up,
                              double *ms_down, int *launches);
/* Work items (one expert x up to 32 rows each) the expert kernels were launched
 * for since the last reset; at decode sizes that is the number of distinct
 * experts whose weights were streamed.  Synchronises the library stream. */
long long apus_cuda_moe_work_items(ApusCudaMoe *m, int reset);
/* Hash-routed layers (c/moe.h:42, 391-394): place the tid2eid table
 * [vocab, topk] in HBM so that apus_cuda_moe_route_dev / _forward_dev can look
 * token ids up on device.  (The host-pointer apus_cuda_moe_forward does not
 * need it: it reads w->tid2eid on the host.) */
int apus_cuda_moe_set_hash_table(ApusCudaMoe *m, const int64_t *tid2eid,
                                 int64_t vocab);

/* c/moe.h:352-412 on device: gate matmul, sqrtsoftplus, bias, stable top-k or
 * hash lookup, normalised weights.  x [s,dim] f32; ids [s] i64 (hash layers,
 * else may be NULL); idx [s,topk] i32 and wgt [s,topk] f32 out; sp/biased
 * [s,E] optional (NULL to skip). */
int apus_cuda_moe_route_dev(const ApusCudaMoe *m, const float *x,
                            const int64_t *ids, int s, int32_t *idx,
                            float *wgt, float *sp, float *biased,
                            void *stream);
/* c/moe.h:435-563 on device for routings whose expert is local: `n_rout`
 * (token row, expert) pairs; xrows [n_rows, dim] f32 are the distinct token
 * rows, rout_row[i] indexes into them, rout_eid[i] is the GLOBAL expert id
 * (must lie in [e_lo, e_hi)).  eo [n_rout, dim] receives each routing's
 * BF16-rounded expert output (c/attn.h:447).  Routings may come in any
 * order; the library groups them by expert internally. */
int apus_cuda_moe_experts_dev(ApusCudaMoe *m, const float *xrows, int n_rows,
                              const int32_t *rout_row,
                              const int32_t *rout_eid, int n_rout, float *eo,
                              void *stream);
/* c/moe.h:148-158 + 570-585 on device: y[t] = sum_j wgt[t,j]*eo[t,j] strictly
 * in j order, shared expert added, BF16 round.  eo [s*topk, dim] in (t,j)
 * order; `shared` [s,dim] from apus_cuda_moe_shared_dev. */
int apus_cuda_moe_combine_dev(const ApusCudaMoe *m, const float *eo,
                              const float *wgt, const float *shared, int s,
                              float *out, float *routed, void *stream);
/* The fixed-shape exchange of an expert-parallel sublayer (no counterpart in the
 * reference): every (source, destination) pair of ranks carries `slots` row slots.
 * plan: routing p = t*topk + j (idx [n_rout], global expert ids) goes to rank
 * idx[p] / (n_experts / world), into the next free slot of that rank's block in
 * the order of p; slot_of [n_rout] receives destination * slots + position,
 * send_eids [world * slots] the expert ids by slot with -1 in unused slots (the
 * expert kernels skip those).  rows: gather == 0 copies token row p / topk of src
 * [s, dim] to dst[slot_of[p]]; gather == 1 copies src[slot_of[p]] (expert outputs
 * as they came back) to dst[p], i.e. back to (t, j) order. */
int apus_cuda_moe_ep_plan_dev(const int32_t *idx, int n_rout, int n_experts,
                              int world, int slots, int32_t *send_eids,
                              int32_t *slot_of, void *stream);
int apus_cuda_moe_ep_rows_dev(const float *src, int dim, const int32_t *slot_of,
                              int n_rout, int topk, int gather, float *dst,
                              void *stream);
/* The same exchange with the compact payload (what crosses the links is what the arithmetic
 * needs): a token row travels as its E4M3 codes + per-128 scales, quantised ONCE on the token's
 * home rank (the quantisation is per token, c/moe.h:246-254, so the owner of the expert would
 * compute the same codes), apus_cuda_moe_ep_row_bytes() = dim + dim/128*4 bytes per row slot;
 * expert outputs are BF16 values (c/attn.h:447) and travel back as their 16 bits.
 * pack: quantise x [s, dim] and copy the row of routing p = t*topk + j into slot slot_of[p] of
 * `send` [world * slots rows].  experts_q: routing i = received row i with global expert id
 * rout_eid[i] (-1: empty slot, skipped), outputs as BF16 bits [n_rows, dim].  unpack: eo[p] =
 * widen(back[slot_of[p]]), back to (t, j) order for apus_cuda_moe_combine_dev.  Needs the
 * tcgen05 expert path. */
size_t apus_cuda_moe_ep_row_bytes(const ApusCudaMoe *m);
int apus_cuda_moe_ep_pack_dev(ApusCudaMoe *m, const float *x, int s, const int32_t *slot_of,
                              int n_rout, uint8_t *send, void *stream);
int apus_cuda_moe_experts_q_dev(ApusCudaMoe *m, const uint8_t *qrows, int n_rows,
                                const int32_t *rout_eid, uint16_t *eo_bf16, void *stream);
int apus_cuda_moe_ep_unpack_dev(const uint16_t *back, int dim, const int32_t *slot_of,
                                int n_rout, float *eo, void *stream);
/* c/moe.h:570-581 on device: the FP8 shared expert for s tokens. */
int apus_cuda_moe_shared_dev(ApusCudaMoe *m, const float *x, int s,
                             float *shared, void *stream);
/* The whole sublayer on one GPU (all experts local): route + experts +
 * shared + combine, c/moe.h:369-595.  x/out device f32 [s,dim]. */
int apus_cuda_moe_forward_dev(ApusCudaMoe *m, const float *x,
                              const int64_t *ids, int s, float *out,
                              void *stream);
/* Copy back the router decisions of the last *_forward_dev / route call
 * (device-to-host, synchronises the stream): idx [s,topk], wgt [s,topk]. */
int apus_cuda_moe_last_routing(ApusCudaMoe *m, int s, int32_t *idx,
                               float *wgt, void *stream);

/* Single matrices on device (c/attn.h:408-449 semantics). */
ApusCudaFp4 *apus_cuda_fp4_upload(const ApusFp4W *w);
ApusCudaFp8 *apus_cuda_fp8_upload(const ApusFp8W *w);
void apus_cuda_fp4_free(ApusCudaFp4 *w);
void apus_cuda_fp8_free(ApusCudaFp8 *w);
int apus_cuda_fp4_linear_dev(const ApusCudaFp4 *w, const float *x, float *out,
                             int M, void *stream);
int apus_cuda_fp8_linear_dev(const ApusCudaFp8 *w, const float *x, float *out,
                             int M, void *stream);
/* c/moe.h:333 on device, MXFP4 kind: out = w2(swiglu(w1 x, w3 x)). */
int apus_cuda_expert_fp4_dev(const ApusCudaFp4 *w1, const ApusCudaFp4 *w2,
                             const ApusCudaFp4 *w3, float limit,
                             const float *x, int rows, float *out,
                             void *stream);
/* c/attn.h:668 on device, `rows` rows of n scores -> idx [rows,k]. */
int apus_cuda_topk_stable_dev(const float *scores, int n, int k, int32_t *idx,
                              int rows, void *stream);
/* c/attn.h:1308 on device. kv_a [na,d] and kv_b [nb,d] are BF16 (u16 bits,
 * value-identical to the reference's f32-carrying-BF16 caches). */
int apus_cuda_sparse_attn_dev(const float *q, const float *sink, int h, int d,
                              const int32_t *idxs, int idxw, int s,
                              float scale, const uint16_t *kv_a, int64_t na,
                              const uint16_t *kv_b, int64_t nb, float *o,
                              void *stream);

/* The decode form of c/attn.h:1308 for `s` sequences that each attend their OWN caches
 * (row t of q / idxs belongs to sequence t): kv_a [s, >= na, d] and kv_b [s, >= nb, d]
 * BF16, kv_a_stride / kv_b_stride = rows between consecutive sequences' caches (0: one
 * cache shared by all rows, as apus_cuda_sparse_attn_dev). */
int apus_cuda_sparse_attn_batch_dev(const float *q, const float *sink, int h, int d,
                                    const int32_t *idxs, int idxw, int s, float scale,
                                    const uint16_t *kv_a, int64_t na, int64_t kv_a_stride,
                                    const uint16_t *kv_b, int64_t nb, int64_t kv_b_stride,
                                    float *o, void *stream);

/* ---- block and model (c/layer.h, c/model.h) --------------------------------- */

/* The fields of the reference's ApusLayer (c/layer.h:45-71) that
 * apus_block_forward reads, gathered in one plain descriptor (the integrator
 * fills it from its ApusLayer, field by field).  cos/sin are the rope
 * tables of this layer's theta class, [rope_rows, rope_dim/2]. */
typedef struct {
    ApusAttnCfg acfg;
    ApusAttnW aw;
    ApusMoeW mw;
    const float *attn_norm_w, *ffn_norm_w;                        /* [dim] */
    const float *hc_attn_fn, *hc_attn_base, *hc_attn_scale;       /* [(2+hc)*hc, hc*dim], [(2+hc)*hc], [3] */
    const float *hc_ffn_fn, *hc_ffn_base, *hc_ffn_scale;
    const float *cos, *sin;
    int rope_rows;
} ApusCudaLayerDesc;

/* The top-level tensors and sizes of the reference's ApusModel / ApusCfg
 * (c/model.h:58-84, c/layer.h:32-43). embed/head are [vocab, dim], BF16 bits or f32. */
typedef struct {
    int n_layers, dim, hc_mult, hc_sinkhorn_iters, vocab;
    float hc_eps, norm_eps;
    const ApusCudaLayerDesc *layers;
    const void *embed; int embed_bf16;
    const void *head;  int head_bf16;
    const float *norm_w, *hc_head_fn, *hc_head_base;
    float hc_head_scale;
} ApusCudaModelDesc;

typedef struct ApusCudaModel ApusCudaModel;

/* c/layer.h:110 apus_block_forward: one block for s tokens of one sequence,
 * h [s, hc_mult, dim] in/out, host state `st` read and updated like
 * apus_cuda_attention does. */
int apus_cuda_block_forward(const ApusCudaLayerDesc *L, int hc_mult,
                            int hc_sinkhorn_iters, float hc_eps,
                            float norm_eps, ApusAttnS *st, float *h,
                            const int64_t *ids, int s, int64_t start_pos);
/* The same for hash-routed layers too (c/moe.h:391-394 looks the experts up in
 * tid2eid [vocab, topk] by token id; the reference's ApusLayer carries the
 * vocabulary size in its cfg, c/layer.h:32-43): `vocab` rows of L->mw.tid2eid. */
int apus_cuda_block_forward_v(const ApusCudaLayerDesc *L, int hc_mult,
                              int hc_sinkhorn_iters, float hc_eps,
                              float norm_eps, ApusAttnS *st, float *h,
                              const int64_t *ids, int s, int64_t start_pos,
                              int64_t vocab);
/* c/model.h:396 + 485 apus_model_load / apus_model_state_init replaced by HBM
 * residency: uploads every weight, allocates the state of `batch` sequences
 * (1..32, advancing in lockstep) for positions < max_pos. */
ApusCudaModel *apus_cuda_model_create(const ApusCudaModelDesc *d, int batch,
                                      int max_pos);
/* The same with only the routed experts [e_lo, e_hi) of every layer resident
 * (expert parallelism: rank r of N holds [r*E/N, (r+1)*E/N); descriptors of the
 * other experts are not read).  Such a model is driven layer by layer, below. */
ApusCudaModel *apus_cuda_model_create_ep(const ApusCudaModelDesc *d, int batch,
                                         int max_pos, int e_lo, int e_hi);
void apus_cuda_model_destroy(ApusCudaModel *m);
/* c/model.h:485: back to position 0 with empty caches. */
int apus_cuda_model_reset(ApusCudaModel *m);
int64_t apus_cuda_model_pos(const ApusCudaModel *m);
/* c/sample.h:44-71 for the loop above: temp <= 0 keeps the greedy pick; otherwise
 * every step draws with temperature and nucleus (top-p) sampling, one uniform
 * per sequence and step from a splitmix64 stream kept on the device; sequence b
 * uses the stream seeded with seed + b (sequence 0 = the reference CLI's --seed). */
int apus_cuda_model_set_sampling(ApusCudaModel *m, float temp, float top_p, uint64_t seed);
/* A decode step is the same sequence of launches at every position (the kernels
 * read the position on the device), so apus_cuda_model_forward / _generate
 * replay it from a CUDA graph after the first step (default on; it is bypassed
 * while apus_cuda_moe_timing is enabled on a layer).  enable < 0 only queries.
 * Returns the setting in force. */
int apus_cuda_model_use_graph(ApusCudaModel *m, int enable);
/* The MoE sublayer object of one layer (owned by the model), e.g. for
 * apus_cuda_moe_timing / apus_cuda_moe_use_tc. */
ApusCudaMoe *apus_cuda_model_moe(ApusCudaModel *m, int layer);
/* c/model.h:722 apus_model_forward for every sequence: ids [batch, s] host,
 * consumes s positions; logits [batch, vocab] of the last position and/or the
 * greedy next token [batch] (c/sample.h:76-81, lowest index on ties) are
 * copied back when non-NULL. */
int apus_cuda_model_forward(ApusCudaModel *m, const int64_t *ids, int s,
                            float *logits, int32_t *next);
/* The same with the reference's logits_all: logits_all [batch, s, vocab] and
 * next_all [batch, s] (both nullable) receive every position's row and greedy
 * (or sampled) pick -- the verify batch of speculative decoding (c/mtp.h). */
int apus_cuda_model_forward_all(ApusCudaModel *m, const int64_t *ids, int s,
                                float *logits_all, int32_t *next_all);
/* c/apus.c:895-944, greedy: prompt [batch, n_prompt] then n_gen tokens per
 * sequence, the sampled token fed back on the device; out_tokens [batch,
 * n_gen].  ms_prefill / ms_decode (nullable) receive the CUDA-event times of
 * the prompt steps and of the n_gen - 1 decode steps. */
int apus_cuda_model_generate(ApusCudaModel *m, const int64_t *prompt,
                             int n_prompt, int n_gen, int32_t *out_tokens,
                             float *ms_prefill, float *ms_decode);

/* Models that step side by side.  A decode step at batch 32 is mostly a chain of
 * short kernels that leave the GPU idle between them; sequences are independent,
 * so a batch can be split over several model objects (created from the same
 * descriptor with device-resident weights they share without copying them),
 * each enqueuing on a stream of its own, and their steps overlap on the GPU.
 * Every sequence computes exactly what it computes alone.
 * set_stream: `create` != 0 gives the model a stream made by the library,
 * otherwise `stream` (a cudaStream_t; NULL = back to the library stream); the next
 * step runs eagerly on the new stream before steps are recorded again.
 * forward_group / generate_group are apus_cuda_model_forward / _generate for n
 * models at once (arrays of n prompts / outputs, batch of model i rows each);
 * the models must be on different streams; the times cover the whole group. */
int apus_cuda_model_set_stream(ApusCudaModel *m, void *stream, int create);
int apus_cuda_model_forward_group(ApusCudaModel *const *ms, int n,
                                  const int64_t *const *ids, int s,
                                  float *const *logits, int32_t *const *next);
int apus_cuda_model_generate_group(ApusCudaModel *const *ms, int n,
                                   const int64_t *const *prompts, int n_prompt,
                                   int n_gen, int32_t *const *out_tokens,
                                   float *ms_prefill, float *ms_decode);

/* c/model.h:115-129, 731-743 apus_model_forward_h / apus_model_forward_mh for every sequence: the
 * forward with, besides the logits, the hidden state after the last block of every position
 * (h_out [batch, s, hc_mult * dim], BF16-valued f32, the MTP head's input) or, after each layer
 * listed in `targets`, the mean over the hc streams of every position (mh_out
 * [batch, s, n_targets * dim], f32 accumulate in stream order, BF16 result: the DSpark
 * drafter's main_hidden; the reference reads the target list from the checkpoint's dspark
 * config, here the caller passes it).  ids [batch, s]; logits [batch, vocab] of the last
 * position, or [batch, s, vocab] when logits_all; next [batch] or [batch, s] the picks
 * (greedy, or sampled under apus_cuda_model_set_sampling); all outputs nullable. */
int apus_cuda_model_forward_h(ApusCudaModel *m, const int64_t *ids, int s, float *logits,
                              int logits_all, int32_t *next, float *h_out);
int apus_cuda_model_forward_mh(ApusCudaModel *m, const int64_t *ids, int s, float *logits,
                               int logits_all, int32_t *next, const int *targets,
                               int n_targets, float *mh_out);

/* c/mtp.h:66-110 ApusMtp: the MTP draft head of a model -- e = enorm(embed(id)) -> e_proj,
 * x_j = hnorm(h_j) -> h_proj per hc stream, bf16(e + x_j) -> one full block (sliding-window
 * attention with its own state, the full MoE) -> its own hc_head collapse and norm -> the
 * parent's LM head.  The head shares the parent's embedding, head, sizes, batch and stream;
 * its weights are copied to HBM at creation (the host copies may go afterwards). */
typedef struct {
    ApusCudaLayerDesc block;              /* "mtp.<idx>.*" block (c/mtp.h:223-226) */
    ApusFp8W e_proj, h_proj;              /* FP8 [dim, dim] */
    const float *enorm_w, *hnorm_w, *norm_w;      /* [dim] */
    const float *hc_head_fn, *hc_head_base;       /* [hc, hc*dim], [hc] */
    float hc_head_scale;
} ApusCudaMtpDesc;
typedef struct ApusCudaMtp ApusCudaMtp;
ApusCudaMtp *apus_cuda_mtp_create(ApusCudaModel *parent, const ApusCudaMtpDesc *d);
/* c/mtp.h:213-281 apus_mtp_load: MTP block `idx` ("mtp.<idx>.*") read from the checkpoint directory
 * `parent` was loaded from (same files, names and conversions as the reference's loader). */
ApusCudaMtp *apus_cuda_mtp_load(ApusCudaModel *parent, const char *dir, int idx);
void apus_cuda_mtp_destroy(ApusCudaMtp *mt);
/* c/mtp.h:293-299: a fresh attention state. */
int apus_cuda_mtp_reset(ApusCudaMtp *mt);
/* c/mtp.h:303-357 apus_mtp_forward for every sequence: h_in [batch, s, hc_mult * dim] (the
 * main model's hidden after its last block, or the head's own when chaining), ids [batch, s]
 * at positions start_pos .. start_pos + s - 1; advances the head's attention state.  Of the
 * LAST position: logits [batch, vocab], the greedy pick next [batch], and the head's own
 * post-block hidden h_last [batch, hc_mult * dim] (all nullable). */
int apus_cuda_mtp_forward(ApusCudaMtp *mt, const float *h_in, const int64_t *ids, int s,
                          int64_t start_pos, float *logits, int32_t *next, float *h_last);

/* c/dspark.h:88-118 ApusDspark: the DSpark draft module -- n_stages full sliding-window blocks (scored
 * routing) whose rings hold, for every true position, the KV row made from
 * main_x = main_norm(main_proj(main_hidden)) (apus_cuda_model_forward_mh rows), the last stage's own
 * hc_head and norm, the parent's LM head, the bigram ("markov") bias and the confidence head.  One
 * sequence per model.  Weights are copied to HBM at creation. */
typedef struct {
    int n_stages, block_size, noise_id, markov_rank, n_targets;   /* ApusDsparkCfg (c/model.h:48-56) */
    int targets[8];                         /* layers whose mean hidden feeds main_proj */
    const ApusCudaLayerDesc *stages;        /* [n_stages] "mtp.<k>.*" blocks, ratio 0 */
    ApusFp8W main_proj;                     /* FP8 [dim, n_targets * dim] */
    const float *main_norm_w, *norm_w;      /* [dim] */
    const float *hc_head_fn, *hc_head_base; /* [hc, hc*dim], [hc] */
    float hc_head_scale;
    const float *markov_w1, *markov_w2;     /* [vocab, markov_rank] f32 */
    const float *conf_proj;                 /* [dim + markov_rank] */
} ApusCudaDsparkDesc;
typedef struct ApusCudaDspark ApusCudaDspark;
ApusCudaDspark *apus_cuda_dspark_create(ApusCudaModel *parent, const ApusCudaDsparkDesc *d);
/* c/dspark.h:272-341 apus_dspark_load: the stages "mtp.0 .. mtp.<n-1>" and their glue from the checkpoint
 * directory, sizes from its DSpark config section (c/model.h:336-373). */
ApusCudaDspark *apus_cuda_dspark_load(ApusCudaModel *parent, const char *dir);
void apus_cuda_dspark_destroy(ApusCudaDspark *ds);
/* c/dspark.h:353-356: empty stage rings. */
int apus_cuda_dspark_reset(ApusCudaDspark *ds);
/* c/dspark.h:365-376 + 397-455 apus_dspark_stage0_project followed by apus_dspark_prefill (pos0 = 0,
 * the whole prompt) or apus_dspark_catchup: the stage rings' rows of the n true positions
 * pos0 .. pos0 + n - 1 from their main hiddens mh [n, n_targets * dim]. */
int apus_cuda_dspark_feed(ApusCudaDspark *ds, const float *mh, int64_t pos0, int n);
/* c/dspark.h:702-711 apus_dspec_init's temp and draft_seed: temp > 0 makes every draft pick one draw at
 * that temperature (top_p 1) from the module's own splitmix64 stream, seeded here, one uniform per draft
 * row, never rolled back (c/dspark.h:666-676); temp <= 0 (the state after create / load) = greedy drafts.
 * The reference drafts at the temperature of the main stream: pass the model's. */
int apus_cuda_dspark_set_sampling(ApusCudaDspark *ds, float temp, uint64_t draft_seed);
/* c/dspark.h:611-697 apus_dspark_draft_round: anchor = the held token, mh_row
 * [n_targets * dim] = main hidden of position start_pos (its ring slot is rewritten, idempotent
 * with apus_cuda_dspark_feed); drafts [block_size] = candidates for start_pos + 2 ..; nullable
 * outputs as in ApusDsparkDbg: confidence [block_size], logits_final [block_size, vocab], stage_h
 * [n_stages, block_size, hc_mult * dim]. */
int apus_cuda_dspark_draft_round(ApusCudaDspark *ds, int64_t anchor, const float *mh_row,
                                 int64_t start_pos, int64_t *drafts, float *confidence,
                                 float *logits_final, float *stage_h);
/* c/dspark.h:747-862 apus_dspec_prefill + apus_dspec_step until n_gen tokens are out: draft a block,
 * verify [held, d1 .. dB] in one pass, accept while the drafts equal the model's own picks, roll back
 * and re-feed the true prefix otherwise; the stage rings are caught up from the verify pass's
 * hiddens.  The emitted stream is the plain stream of apus_cuda_model_generate, bit for bit.
 * stats (nullable) [7]: emitted, batches, batch_tokens, refeed_tokens, offered, accepted,
 * bonus_rounds (ApusDspec). */
int apus_cuda_model_spec_generate_dspark(ApusCudaModel *m, ApusCudaDspark *ds, const int64_t *prompt,
                                         int n_prompt, int n_gen, int32_t *out_tokens,
                                         uint64_t *stats);

/* c/mtp.h:113-138, 398-439 apus_snap_take / apus_snap_restore on the device (the
 * rollback of speculative decoding: draft and verify a few positions, keep the
 * accepted prefix).  A snapshot holds, per layer, the sliding-window ring, the
 * compressor carries and the entry counts -- cache entries past a restored
 * count are dead capacity, so rollback is a copy plus truncation -- and the
 * position, the token fed back for the next step and the sampler streams.
 * Copies are device-to-device on the model's stream, nothing waits on the host.
 * snapshot: `reuse` (nullable) is an earlier snapshot of the same model to
 * overwrite instead of allocating. */
typedef struct ApusCudaSnap ApusCudaSnap;
ApusCudaSnap *apus_cuda_model_snapshot(ApusCudaModel *m, ApusCudaSnap *reuse);
int apus_cuda_model_restore(ApusCudaModel *m, const ApusCudaSnap *snap);
void apus_cuda_snap_free(ApusCudaSnap *snap);

/* c/mtp.h:142-190, 531-616: the draft/verify engine with a caller-supplied proposer
 * (the reference's draft_override hook: fill drafts[0..n-1], candidates for
 * positions q..q+n-1; drafts[0] is only compared with the held token for the
 * statistics).  One sequence per model.  Emits n_gen tokens after the prompt
 * that are bit for bit those of apus_cuda_model_generate (greedy or sampled
 * with the same seed): a draft is accepted iff it equals the model's own pick.
 * stats (nullable, 8 counters as in ApusSpec): emitted, batches, batch_tokens,
 * refeed_tokens, offered, accepted, d1_offered, d1_hits.  The verify batch is one pass
 * over its positions (a chunk), each row bit for bit the single step's.
 * apus_cuda_model_spec_generate_mtp: the same loop with the MTP head as the proposer
 * (c/mtp.h:441-528, 600-612): the head replays the true (hidden, token) pairs, chains
 * `depth` drafts from its own hidden, and is rolled back to the true pairs after every
 * verify batch.  Hiddens and drafts stay on the device except the draft ids. */
typedef void (*ApusCudaDraftFn)(void *ctx, int64_t q, int64_t *drafts, int n);
int apus_cuda_model_spec_generate_mtp(ApusCudaModel *m, ApusCudaMtp *mt, const int64_t *prompt,
                                      int n_prompt, int n_gen, int depth, int32_t *out_tokens,
                                      uint64_t *stats);
int apus_cuda_model_spec_generate(ApusCudaModel *m, const int64_t *prompt,
                                  int n_prompt, int n_gen, int depth,
                                  ApusCudaDraftFn draft, void *draft_ctx,
                                  int32_t *out_tokens, uint64_t *stats);

/* One decode step of all sequences in pieces, on the library stream, for callers
 * that run the MoE sublayer themselves (expert parallelism: route, exchange
 * rows with the expert owners, apus_cuda_moe_experts_dev, exchange back,
 * combine -- apus_b200/ep_model.py).  Per step: set_ids (host or device
 * pointer, [batch]) or the fed-back token; begin_step (embedding); per layer
 * attn_half, then ffn_input returns the device pointer of the normed sublayer
 * input [batch, dim] and ffn_output takes the sublayer result [batch, dim];
 * end_step advances the position and, if asked, computes logits, the greedy
 * token and feeds it back as the next step's ids.  read copies logits / tokens
 * to the host and synchronises. */
int apus_cuda_model_set_ids(ApusCudaModel *m, const int64_t *ids);
int apus_cuda_model_begin_step(ApusCudaModel *m);
int apus_cuda_model_attn_half(ApusCudaModel *m, int layer);
const float *apus_cuda_model_ffn_input(ApusCudaModel *m, int layer);
int apus_cuda_model_ffn_output(ApusCudaModel *m, int layer, const float *sub);
int apus_cuda_model_end_step(ApusCudaModel *m, int want_logits, int feed_back);
/* The pieces read the position on the device, so a caller may record one whole
 * step (its own collectives included) into a CUDA graph by stream capture on the
 * stream given to apus_cuda_use_stream: capturing(1) before the recording,
 * capturing(0) after it (the recorded calls must not move the host-side
 * position), and note_step() after every replay, which moves the host-side
 * position and entry counts like the replayed step did on the device. */
int apus_cuda_model_capturing(ApusCudaModel *m, int on);
int apus_cuda_model_note_step(ApusCudaModel *m);
const int64_t *apus_cuda_model_ids(ApusCudaModel *m);
int apus_cuda_model_read(ApusCudaModel *m, float *logits, int32_t *next);

/* ---- checkpoint directory -> HBM (c/st.h, c/model.h:195-470, c/layer.h:193-330) ----
 * The reference loads <dir>/config.json and the safetensors shards named by
 * <dir>/model.safetensors.index.json (else <dir>/weights/...), c/model.h:396-423.
 * The reader below is host code (no GPU needed): it parses the same two config
 * schemas, resolves tensors by the same names and dtypes and fails with the same
 * messages; apus_cuda_model_load streams layer after layer into HBM, so host
 * memory holds one layer at a time.  A shard is 8 bytes of little-endian header
 * length, a JSON header {name: {dtype, shape, data_offsets}}, then the payloads
 * (c/st.h:5-9). */
typedef enum {                       /* c/st.h:42-46 */
    APUS_CUDA_ST_I8, APUS_CUDA_ST_U8, APUS_CUDA_ST_F8_E8M0, APUS_CUDA_ST_F8_E4M3,
    APUS_CUDA_ST_BF16, APUS_CUDA_ST_F16, APUS_CUDA_ST_F32, APUS_CUDA_ST_I32,
    APUS_CUDA_ST_I64, APUS_CUDA_ST_OTHER
} ApusCudaStDtype;
/* The reference's ApusCfg (c/layer.h:32-41) followed by what
 * apus_model_parse_config returns beside it (c/model.h:195-376). */
typedef struct {
    int dim, n_heads, head_dim, rope_head_dim, q_lora_rank;
    int o_groups, o_lora_rank, window_size;
    int moe_inter_dim, n_routed_experts, n_activated_experts;
    int index_n_heads, index_head_dim, index_topk;
    int hc_mult, hc_sinkhorn_iters;
    int original_seq_len, beta_fast, beta_slow, vocab_size, max_pos;
    float route_scale, swiglu_limit, hc_eps, norm_eps;
    double rope_theta, compress_rope_theta, rope_factor;
    int n_layers, bos_id, eos_id, n_mtp, mtp_ratio, mtp_hash, dspark;
} ApusCudaCkptCfg;
typedef struct ApusCudaCkpt ApusCudaCkpt;

/* c/model.h:396-423: config + shard index; shard headers are parsed when a
 * tensor of theirs is first asked for.  NULL + err on failure. */
ApusCudaCkpt *apus_cuda_ckpt_open(const char *dir, char *err, size_t errcap);
void apus_cuda_ckpt_close(ApusCudaCkpt *c);
const ApusCudaCkptCfg *apus_cuda_ckpt_cfg(const ApusCudaCkpt *c);
/* compress ratio (0 sliding window, 4 compressed sparse, 128 heavily compressed)
 * and hash routing of a layer. */
int apus_cuda_ckpt_layer_kind(const ApusCudaCkpt *c, int layer, int *ratio, int *hash);
/* c/st.h:85 apus_st_set_get: 0 and the tensor's dtype / shape [8] / size, or 1. */
int apus_cuda_ckpt_tensor(ApusCudaCkpt *c, const char *name, int *dtype, int *ndim,
                          int64_t *shape, uint64_t *nbytes);
/* The raw payload (nbytes must match). */
int apus_cuda_ckpt_read(ApusCudaCkpt *c, const char *name, void *dst, uint64_t nbytes);
/* c/st.h:73 apus_st_f32: F32 or BF16 (widened exactly) -> f32 [n]. */
int apus_cuda_ckpt_read_f32(ApusCudaCkpt *c, const char *name, float *out, uint64_t n);
/* c/layer.h:226-247: layers.<i>.attn.wo_a, FP8 on disk, as the BF16 bits the
 * attention uses (dequantise, round to BF16); out [G*o_lora, n_heads*head_dim/G]. */
int apus_cuda_ckpt_wo_a(ApusCudaCkpt *c, int layer, uint16_t *out, uint64_t n);
/* c/layer.h:145-178 + c/attn.h:247-281: rows [0, rows) of the rope table of the
 * layer class (ratio == 0: plain theta; else the compress theta with YaRN),
 * cos/sin [rows, rope_head_dim/2], computed with the host's cosf/sinf like the
 * reference does. */
int apus_cuda_ckpt_rope(const ApusCudaCkpt *c, int ratio, int64_t rows, float *cos, float *sin);
/* The six tensors of one routed expert (w1/w2/w3 weight + scale) into `slab`
 * (cap >= the sum of their sizes) and views into it.  When the container keeps
 * them adjacent (tools/convert.py's coalesced layout, c/cache.h:8-15) this is ONE
 * positional read, otherwise six. */
int apus_cuda_ckpt_expert(ApusCudaCkpt *c, int layer, int expert, void *slab, uint64_t cap,
                          ApusFp4W *w1, ApusFp4W *w2, ApusFp4W *w3);
/* Loads one layer into host memory exactly as apus_cuda_model_load does (all
 * conversions, experts [e_lo, e_hi) read by the I/O threads), and returns an
 * FNV-1a digest of every tensor in descriptor order plus the byte count: a
 * check of a container (or of the reader) that needs no GPU. */
int apus_cuda_ckpt_layer_digest(ApusCudaCkpt *c, int layer, int e_lo, int e_hi,
                                uint64_t *digest, uint64_t *bytes);
/* c/st.h:143-144: positional reads issued so far and the bytes they returned. */
uint64_t apus_cuda_ckpt_read_count(const ApusCudaCkpt *c);
uint64_t apus_cuda_ckpt_read_bytes(const ApusCudaCkpt *c);
/* c/model.h:392 apus_model_load + c/model.h:485 apus_model_state_init for HBM
 * residency: every layer read, converted like the reference's loader does and
 * uploaded, rope tables built for positions < max_pos (clamped to the config's
 * max_pos), routed experts [e_lo, e_hi) only (e_hi < 0: all).  NULL on failure,
 * message in apus_cuda_last_error(). */
ApusCudaModel *apus_cuda_model_load(const char *dir, int batch, int max_pos, int e_lo, int e_hi);

/* Sizes of a model object (any pointer may be NULL). */
int apus_cuda_model_info(const ApusCudaModel *m, int *batch, int *max_pos, int *vocab, int *n_layers);

/* c/apus.c:451-662 `apus serve`: the newline-delimited JSON loop on file descriptors, until end of
 * input.  Requests {"id", "cmd":"generate", "ids":[...], "max_tokens", "temperature", "top_p",
 * "seed"}; responses {"id","type":"prompt"|"token"|"done"|"error", ...} with the reference's
 * fields, defaults (32 tokens, temperature 1, top_p 1, seed 0), clamps and messages.  eos_id ends a
 * completion ("finish_reason":"stop").  Text prompts, chat messages and "encode" need the
 * tokenizer, which is outside this library: they get the reference's "no tokenizer in model dir"
 * error, and tokens carry no text.  The model must hold one sequence. */
int apus_cuda_serve(ApusCudaModel *m, int in_fd, int out_fd, int eos_id);

/* No counterpart in the reference.  apus_cuda_hc_pre on device pointers for
 * callers that must not allocate device memory while they run (an engine whose
 * own arena already owns the HBM, a region where allocation is forbidden, a loop
 * that must stay off the allocator's lock): the scratch between its two kernels
 * is a fixed array inside the library, 82,944 bytes on every GPU that loads it,
 * enough for rows <= 256; more rows are rejected with an error.  It calls no
 * cudaMalloc/cudaFree.  The first call on a device resolves the array's device
 * address: make it before any stream capture.  All calls on a device share the
 * array; calls that may overlap on the GPU race on it. */
int apus_cuda_hc_pre_noalloc_dev(const float *x4, size_t d, size_t n,
                                 const float *fn, const float *scale,
                                 const float *base, float norm_eps,
                                 float hc_eps, int iters, const float *norm_w,
                                 float rms_eps, float *y, float *y_normed,
                                 float *post, float *comb, int rows,
                                 void *stream);

#ifdef __cplusplus
}
#endif
#endif /* APUS_B200_H */
