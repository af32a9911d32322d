// Host-callable launchers of the device kernels (one group per .cu file).
// Every launcher is asynchronous on `st`, returns 0 on success and nonzero
// after recording a message with apus::set_error().
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace apus {

// ---- fragment-tiled weight layouts (repack.cu) --------------------------------
//
// Weights are re-tiled once, at upload, into the order in which the tensor-core
// fragments of the streaming kernels consume them (same number of bytes as the
// reference storage; see repack.cu for the exact bit layout).
int repack_fp4(const uint8_t *packed, const uint8_t *scales, int O, int K,
               uint8_t *out_codes, uint8_t *out_scales, int *zero_scale_flag,
               cudaStream_t st);
int repack_fp8(const uint8_t *codes, int O, int K, uint8_t *out_codes,
               cudaStream_t st);

// ---- quantisation / norms (quant.cu) ----------------------------------------------
// BF16 round + per-128 E4M3 quant of M rows (reference c/attn.h:393-402).
// arow (nullable) gathers input rows: row m is read from x[arow[m]].
int act_quant(const float *x, const int *arow, int M, int K, uint8_t *codes,
              float *scales, const int *m_dev, cudaStream_t st);
// RMSNorm rows (reference c/attn.h:371-378).
int rms_norm(const float *x, const float *w, float eps, float *y, int64_t n,
             int64_t rows, cudaStream_t st);

// ---- small-M block-scaled GEMM (gemm_small.cu) ---------------------------------------
//
// One work item = one weight matrix (or a gate/up pair) times a contiguous run
// of activation rows.  Used for decode GEMVs, expert groups and the prefill of
// short prompts.
struct GemmGroup {
    const uint8_t *wa, *sa;   // matrix A: tiled codes / scales
    const uint8_t *wb, *sb;   // matrix B (gate/up pair mode), else unused
    int row0, nrows;          // activation rows [row0, row0+nrows), nrows <= 32
};

struct GemmSmallArgs {
    int fmt;                  // 4 = MXFP4, 8 = FP8
    int pair;                 // 1: out = swiglu(A x, B x) (reference c/moe.h:113-126)
    int round_out;            // BF16-round outputs (ignored in pair mode: always)
    float limit;              // SwiGLU clamp (pair mode)
    int O, K;
    const GemmGroup *groups;  // device array
    const int *n_groups_dev;  // device scalar, or NULL to use n_groups
    int n_groups;             // launch bound (grid.y)
    int max_rows;             // largest nrows of any group (<= 32), picks the tile count
    const uint8_t *acodes;    // [*, K]
    const float *ascales;     // [*, K/128]
    const int *arow;          // nullable: activation row of sorted position p
    const int *orow;          // nullable: output row of sorted position p
    float *out;               // [*, O]
    int zero_scale;           // MXFP4: some weight scale byte is 0 (slow exact path)
};
int gemm_small(const GemmSmallArgs &a, cudaStream_t st);

// ---- tcgen05 MXFP4 GEMM on the reference weight storage (gemm_tc.cu) ---------------------
struct TcGroup {
    int a_row;                // first row of this work item's matrix in the weight slab
    int row0, nrows;          // activation rows [row0, row0+nrows) in sorted order, nrows <= 32
    int pad;
};
struct TcArgs {
    const void *map_a, *map_b, *map_x;   // host pointers to CUtensorMap objects (weights A/B, act codes)
    const uint8_t *scales_a, *scales_b;  // weight scale slabs, reference layout [rows, K/32]
    const float *ascales;                // activation scales [*, K/128], rows in sorted order
    const TcGroup *groups;
    const int *n_groups_dev;
    int n_groups;
    int O, K, pair, round_out;
    float limit;
    const int *orow;                     // nullable: output row of sorted position p
    float *out;
    int tx_bytes;                        // 0 = default transaction bytes per stage
    uint8_t *q_out;                      // pair mode, optional: write the outputs quantised for the next GEMM
    float *qs_out;                       //   (E4M3 codes [rows, O] + scales [rows, O/128], sorted order) instead of `out`
    int total_rows;                      // activation rows over all work items (0: unknown, K is never split)
    int ksplit;                          // set by gemm_tc: K chunks (grid.z); > 1 uses part + counters
    float *part;                         // [(pair ? 2 : 1) * ksplit, total_rows, O] chunk sums
    int *counters;                       // zeroed, one per (output tile, work item); left zeroed
};
int gemm_tc(const TcArgs &a, cudaStream_t st);
int gemm_tc_status(int reset);
int tc_make_weight_map(void *out_map, const void *codes, long long rows, int K);
int tc_make_act_map(void *out_map, const void *codes, long long rows, int K);

// ---- tcgen05 FP8 GEMM on the reference weight storage (gemm_tc8.cu) -----------------------
struct Tc8Args {
    const void *map_a, *map_b, *map_x;   // host pointers to CUtensorMap objects (weights A/B, act codes)
    const uint8_t *scales_a, *scales_b;  // weight tile scales [O/128, K/128]
    const float *ascales;                // activation scales [M, K/128]
    int M, O, K, pair, round_out;        // activation rows 32*y .. of CTA row y
    float limit;
    float *out;                          // [M, O]
    int ksplit;                          // set by gemm_tc8: K chunks (grid.z); > 1 uses part + counters
    float *part;                         // [(pair ? 2 : 1) * K/128, M, O] per-block terms
    int *counters;                       // zeroed, one per (output tile, row group); left zeroed
};
int gemm_tc8(const Tc8Args &a, cudaStream_t st);
int gemm_tc8_wide(const Tc8Args &a, cudaStream_t st);      // 128 activation rows per CTA; map_x from tc8_make_act_map_wide
int tc8_make_act_map_wide(void *out_map, const void *codes, long long rows, int K);
int gemm_tc8_status(int reset);
int tc8_make_weight_map(void *out_map, const void *codes, long long rows, int K);

// ---- tcgen05 BF16 GEMM on row-major BF16 weights (gemm_tcbf.cu) ---------------------------
// out[m, g*O + o] = sum_k x[m, g*x_koff + k] * w[g*O + o, k] for g < batch (tree-order class).
struct TcbfArgs {
    const void *map_w, *map_x;           // host pointers to CUtensorMap objects (tcbf_make_*_map)
    int M, O, K, batch;
    int x_koff;                          // activation column offset between problems (elements)
    int out_ld, round_out;
    float *out;                          // [M, out_ld]
    int ksplit;                          // K chunks (tcbf_ksplit); > 1 needs part + counters
    float *part;                         // [ksplit, M, batch*O] scratch
    int *counters;                       // zeroed, one per (output tile, row group); left zeroed
    uint8_t *q_out;                      // ksplit > 1, out_ld % 128 == 0: also the E4M3 activation codes [M, out_ld] ...
    float *qs_out;                       // ... and per-128 scales [M, out_ld / 128] of the finished rows (act_quant's)
};
int gemm_tcbf(const TcbfArgs &a, cudaStream_t st);
int gemm_tcbf_status(int reset);
int tcbf_ksplit(int O, int K, int batch, int M);
int tcbf_make_weight_map(void *out_map, const void *w_bf16, long long rows, int K);
int tcbf_make_act_map(void *out_map, const void *x_bf16, long long rows, long long cols);
int f32_to_bf16(const float *x, uint16_t *y, long long n, cudaStream_t st);
// Scratch memory that belongs to a stream (launches on one stream run one after another, so
// they may share it): `bytes` of workspace and, separately, `n_counters` ints that are zero
// whenever no kernel is using them.  Grows on demand (not while the stream is being captured).
int stream_scratch(cudaStream_t st, size_t bytes, void **ws, size_t n_counters, int **counters);

// ---- temperature / top-p sampling (sample.cu; reference c/sample.h) ------------------------
int sample_rows(const float *logits, int n, int rows, float temp, float top_p, const double *u,
                unsigned long long *rng, float *probs, int32_t *out, cudaStream_t st);

// ---- dense f32 / bf16 linears (linear.cu) ------------------------------------------------
// out[m,o] = sum_k x[m,k]*w[o,k]; flags as APUS_CUDA_R_IN/R_OUT/W_BF16.
int f32_linear(const void *w, const float *x, float *out, int M, int K, int O,
               int flags, cudaStream_t st);
// `batch` independent problems: problem b uses w + b*w_stride (elements of w's
// type), x + b*x_stride with rows x_ld apart, out + b*out_stride with rows out_ld apart.
// codes != NULL: a kernel that can also writes the activation codes and per-128 scales of the output rows
// ([M, out_ld] seen as one row per token, what act_quant would make of them) and sets codes->written.
struct LinCodes {
    uint8_t *q;
    float *s;
    int written;
};
int f32_linear_batched(const void *w, long long w_stride, const float *x, long long x_stride, int x_ld,
                       float *out, long long out_stride, int out_ld, int batch, int M, int K, int O,
                       int flags, cudaStream_t st, LinCodes *codes = nullptr);

// ---- MoE glue (moe.cu) ---------------------------------------------------------------------
// sqrtsoftplus of gate logits, bias, stable top-k or hash lookup, weights.
int router_finish(const float *logits, const float *bias, const int64_t *tid2eid,
                  const int64_t *ids, int s, int E, int topk, float route_scale,
                  float *sp, float *biased, int32_t *idx, float *wgt,
                  cudaStream_t st);
// Stable counting sort of routings by expert + work-item table.
struct MoeSlab {            // where expert e's tiled tensors live
    const uint8_t *w1, *s1, *w3, *s3, *w2, *s2;
    size_t code_stride13, scale_stride13, code_stride2, scale_stride2;
    int e_lo, e_hi;
};
// rout_row == NULL: routing i belongs to row i / row_div (the (t, j) order).
int moe_group(const int32_t *rout_eid, const int32_t *rout_row, int row_div, int n_rout,
              const MoeSlab &slab, int chunk, int *sorted_pos, int *sorted_row,
              GemmGroup *g13, GemmGroup *g2, int *n_groups, int max_groups,
              cudaStream_t st, TcGroup *t13 = nullptr, TcGroup *t2 = nullptr, int o13 = 0, int o2 = 0);
// quantised rows for the expert-parallel exchange (dim codes + dim/128 f32 scales per row)
int ep_pack_q(const uint8_t *codes, const float *scales, int dim, const int32_t *slot_of, int n_rout, int topk,
              uint8_t *packed, cudaStream_t st);
int ep_gather_q(const uint8_t *packed, int dim, const int *sorted_row, const int *n_dev, int n_max, uint8_t *codes,
                float *scales, cudaStream_t st);
int ep_unpack_bf16(const uint16_t *src, int dim, const int32_t *slot_of, int n_rout, float *dst, cudaStream_t st);
// y[t] = sum_j wgt[t,j]*eo[t*topk+j] (j order) ; out = bf16(y + shared).
int moe_combine(const float *eo, const float *wgt, const float *shared, int s,
                int topk, int dim, float *out, float *routed, cudaStream_t st);

// ---- selection + attention (attn.cu) ----------------------------------------------------------
int topk_stable(const float *scores, int n, int k, int32_t *idx, int rows,
                cudaStream_t st, const long long *dyn_pos = nullptr, int ratio = 0, long long chunk_pos0 = 0,
                int rows_per_pos = 0);
// dyn_pos: n and k are capacities (row strides); live n = (*dyn_pos + 1) / ratio, live k = min(k, n).
// rows_per_pos > 0 (a chunk of positions, time-major rows): the same with the row's own position
// chunk_pos0 + row / rows_per_pos.
int sparse_attn(const float *q, const float *sink, int h, int d,
                const int32_t *idxs, int idxw, int s, float scale,
                const void *kv_a, int64_t na, const void *kv_b, int64_t nb,
                int kv_bf16, float *o, cudaStream_t st, long long kv_a_stride = 0,
                long long kv_b_stride = 0,    // strides (elements) between the tokens' own caches; 0 = shared
                void *scratch = nullptr, size_t scratch_cap = 0,    // caller's scratch (sparse_attn_scratch bytes) or the shared one
                int seq_mod = 0,     // > 0: token t reads the caches of sequence t % seq_mod (time-major rows of a chunk)
                bool ids_ready = false,              // sparse_attn_compact has run on this scratch with these index rows
                const struct SaRope *rope = nullptr);   // rotate the output rows back before they are written
size_t sparse_attn_scratch(int h, int idxw, int s);
// The first launch of sparse_attn (negative ids dropped, order kept) on its own: a caller that has the
// index rows before the queries (a side chain) runs it there, into the scratch it then hands to sparse_attn.
int sparse_attn_compact(const int32_t *idxs, int h, int idxw, int s, void *scratch, size_t scratch_cap, cudaStream_t st);
// Inverse RoPE of the output rows (reference c/attn.h:1384-1388), applied by the kernel that writes them:
// the last rd elements of every head row, cos/sin row `cs` (or, pos != NULL, row *pos of the table `cs`).
struct SaRope {
    const float *cs;
    const long long *pos;
    int rd;
};

// ---- attention row helpers, compressor and indexer steps (attn_ops.cu) -----------------------
enum {
    ROW_BF16_IN = 1,      // BF16-round the input
    ROW_RMS_W = 2,        // y = bf16(w * (x * rsqrt(mean x^2 + eps)))
    ROW_RMS_PLAIN = 4,    // y = bf16(x * rsqrt(mean x^2 + eps))
    ROW_ROPE = 8,         // interleaved-pair rotation of the last rd elements, BF16 out
    ROW_ROPE_INV = 16,    // the conjugate rotation
    ROW_HADAMARD = 32,    // Sylvester butterflies * n^-1/2, BF16 out
    ROW_FP8QAT = 64,      // E4M3 quant-dequant per 64 on the first n - rd elements
    ROW_FP4QAT = 128,     // E2M1 quant-dequant per 32
    ROW_BF16_OUT = 256,
    ROW_SEQ_SUM = 512     // set by the launcher: sums of squares in the reference's loop order
};
// cs: per position [cos(half) | sin(half)]; row r uses cs + (r / rows_per_cs) * cs_stride.
// Position-dependent arguments read on the device, so that the launch sequence
// of a decode step is the same at every position (a step can then be replayed
// from a CUDA graph).  pos == NULL: the host arguments are used as given.
struct RowDyn {
    const long long *pos;     // device scalar: position of the step
    int cs_bias;              // `cs` is the table base; the row of position pos + cs_bias (>= 0) is used
    int gate_ratio;           // > 0: run only when (pos + 1) % gate_ratio == 0 ...
    long long y_step;         // ... and write to y + ((pos + 1) / gate_ratio - 1) * y_step
};
int row_ops(const float *x, int x_stride, float *y, int y_stride, int rows, int n, int flags,
            const float *norm_w, float eps, int rd, const float *cs, int rows_per_cs, int cs_stride,
            cudaStream_t st, const RowDyn *dyn = nullptr, uint8_t *q_codes = nullptr, float *q_scales = nullptr);
// q_codes != NULL (n % 128 == 0): the finished rows are also written as the E4M3 codes [rows, n] and the
// per-128 scales [rows, n / 128] that act_quant would make of y -- the same arithmetic, one launch less.
int comp_step(float *kv_state, float *sc_state, long long state_stride, const float *kv_new,
              const float *sc_new, int new_stride, const float *ape, int ratio, int overlap, int d,
              int slot, int should, float *pooled, int pooled_stride, int n_seq, cudaStream_t st,
              const long long *dyn_pos = nullptr);    // dyn_pos: slot and should derived from *dyn_pos
// n_seq sequences in lockstep: q [n_seq, ih*idm], wt_raw [n_seq, ih], caches cache_stride floats
// apart, sc [n_seq, nb].
int idx_scores(const float *q, const float *wt_raw, float wscale, const float *cache, long long cache_stride,
               long long nb, int ih, int idm, float *sc, int n_seq, cudaStream_t st,
               const long long *dyn_pos = nullptr, int ratio = 0, long long chunk_pos0 = 0, int chunk_seqs = 0);
// dyn_pos: nb is the capacity (grid size and row stride of sc); the live count is (*dyn_pos + 1) / ratio.
// chunk_seqs > 0: n_seq counts the time-major rows of a chunk of positions; row r scores the cache of
// sequence r % chunk_seqs up to its own position chunk_pos0 + r / chunk_seqs.
// out [n_seq, win + compw]; sel [n_seq, compw] or NULL for the dense list.
int build_idx(int32_t *out, int win, long long pos, const int32_t *sel, int compw, int n_seq, cudaStream_t st,
              const long long *dyn_pos = nullptr, int ratio = 0);
// dyn_pos: compw is the row capacity (row stride win + compw, unused tail -1, sel stride compw); the live
// width is min(compw, (*dyn_pos + 1) / ratio)
// dst[b * dst_stride + i] = src[b * n + i] for b < rows (ring / cache row scatter).
int scatter_rows(float *dst, long long dst_stride, const float *src, int n, int rows, cudaStream_t st,
                 const long long *dyn_pos = nullptr, int win = 0);   // dyn_pos: dst += (*dyn_pos % win) * n
// A chunk of s consecutive positions of n_seq sequences (time-major rows): the position-ordered window
// buffer ext [n_seq][win + s][d] from the ring and the chunk's rows, the ring after the chunk, and the
// index rows [s * n_seq][win + compcap] (window ids into ext, compressed ids + win + s, -1 padding).
int win_ext(float *ext, const float *ring, const float *kv, int win, int s, int d, int n_seq, long long pos0,
            cudaStream_t st);
int ring_update(float *ring, const float *kv, int win, int s, int d, int n_seq, long long pos0, cudaStream_t st);
int build_idx_chunk(int32_t *out, int win, int s, long long pos0, int n_seq, const int32_t *sel, int compcap, int ratio,
                    cudaStream_t st);
// First index of the row maximum (reference c/sample.h:76-81), rows of n.
int argmax_rows(const float *x, int n, int rows, int32_t *out, cudaStream_t st);
// Embedding rows replicated hc times (reference c/model.h:512-517): out [rows, hc, dim].
int embed_rows(const void *table, int bf16, const int64_t *ids, int rows, int hc, int dim, float *out,
               cudaStream_t st);

// expert-parallel exchange helpers (moe.cu)
int ep_plan(const int32_t *idx, int n_rout, int per_rank, int world, int slots, int32_t *send_eids,
            int32_t *slot_of, cudaStream_t st);
int ep_rows(const float *src, int dim, const int32_t *slot_of, int n_rout, int topk, int gather, float *dst,
            cudaStream_t st);

// ---- mHC (mhc.cu) -----------------------------------------------------------------------------------
int mhc_pre(const float *x4, int d, int n, const float *fn, const float *scale,
            const float *base, float norm_eps, float hc_eps, int iters,
            const float *norm_w, float rms_eps, float *pre, float *post,
            float *comb, float *y, float *y_normed, int rows, cudaStream_t st,
            float *raw = nullptr,             // caller's scratch of rows * ((2+n)*n + 1) floats, or the shared one
            uint8_t *xq = nullptr, float *xs = nullptr, int *codes_written = nullptr);
// xq != NULL: where the row layout allows it, the kernel that writes y_normed also writes its activation
// codes [rows, d] and per-128 scales [rows, d / 128] (what act_quant makes of y_normed) and
// *codes_written is set to 1; otherwise it is set to 0 and the caller quantises.
int mhc_post(const float *f, const float *res4, const float *post,
             const float *comb, float *y4, int d, int n, int rows,
             cudaStream_t st);
int mhc_head(const float *x4, int d, int n, const float *fn, float scale,
             const float *base, float norm_eps, float hc_eps, float *y,
             int rows, cudaStream_t st, float *raw = nullptr);

}  // namespace apus
