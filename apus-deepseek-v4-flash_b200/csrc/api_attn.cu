// C ABI, part 3: the attention sublayer (include/apus_b200.h; reference
// c/attn.h:1515-1740) and its row helpers.
//
// A token is one fixed sequence of kernels on the backend stream — low-rank q
// path, window KV, (CSA) indexer with its own compressor and stable top-k,
// ring write, attention compressor, index-gathered attention with sink,
// inverse RoPE, grouped o-projection — in the reference's call order, because
// the indexer and the two compressors mutate the sequence state.  The host
// knows the position, so every data-independent decision (does this token
// complete a compressed block, how many entries exist) is taken on the host
// and no kernel result is read back inside a step.
#include <math.h>
#include <vector>

#include "attn_engine.cuh"

using namespace apus;

namespace apus {

void WeightOwner::release() {
    for (DevQW *q : qws) { q->release(); delete q; }
    for (DevBuf *b : bufs) { b->release(); delete b; }
    qws.clear(); bufs.clear();
}

// Weights of the global cache (own == NULL: the host-pointer tier, keyed by
// host address) or owned by `own` (a model: freed with it).
DevQW *get_qw(WeightOwner *own, int fmt, const uint8_t *codes, const uint8_t *scales, int O, int K) {
    if (!own) return cached_qw(fmt, codes, scales, O, K);
    DevQW *q = new_qw(fmt, codes, scales, O, K);
    if (q) own->qws.push_back(q);
    return q;
}
const void *get_dense(WeightOwner *own, const void *src, size_t bytes) {
    if (!own) return cached_dense(src, bytes);
    if (is_device_ptr(src)) return src;           // used in place; the caller keeps it alive
    DevBuf *b = new DevBuf();
    if (b->get(bytes, nullptr) || cudaMemcpy(b->p, src, bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
        set_error("upload of %zu dense weight bytes failed", bytes);
        b->release(); delete b;
        return nullptr;
    }
    ctx().bytes_uploaded += bytes;
    own->bufs.push_back(b);
    return b->p;
}

static int comp_weights(const ApusCompW &h, int dim, CompDev *d, WeightOwner *own) {
    const int cd = (1 + h.overlap) * h.d;
    d->ratio = h.ratio; d->overlap = h.overlap; d->d = h.d; d->rd = h.rd; d->rotate = h.rotate; d->eps = h.eps;
    d->wkv = (const float *)get_dense(own, h.wkv, (size_t)cd * dim * 4);
    d->wgate = (const float *)get_dense(own, h.wgate, (size_t)cd * dim * 4);
    d->ape = (const float *)get_dense(own, h.ape, (size_t)h.ratio * cd * 4);
    d->norm = (const float *)get_dense(own, h.norm, (size_t)h.d * 4);
    return (d->wkv && d->wgate && d->ape && d->norm) ? 0 : 1;
}

int attn_weights(const ApusAttnCfg *cfg, const ApusAttnW *w, AttnDev *A, WeightOwner *own) {
    const int hd = cfg->n_heads * cfg->head_dim, G = cfg->o_groups;
    A->cfg = *cfg;
    A->wq_a = get_qw(own, 8, w->wq_a.codes, w->wq_a.scales, cfg->q_lora, cfg->dim);
    A->wq_b = get_qw(own, 8, w->wq_b.codes, w->wq_b.scales, hd, cfg->q_lora);
    A->wkv = get_qw(own, 8, w->wkv.codes, w->wkv.scales, cfg->head_dim, cfg->dim);
    A->wo_b = get_qw(own, 8, w->wo_b.codes, w->wo_b.scales, cfg->dim, G * cfg->o_lora);
    if (!A->wq_a || !A->wq_b || !A->wkv || !A->wo_b) return 1;
    A->wo_a = (const uint16_t *)get_dense(own, w->wo_a, (size_t)G * cfg->o_lora * (hd / G) * 2);
    A->q_norm = (const float *)get_dense(own, w->q_norm, (size_t)cfg->q_lora * 4);
    A->kv_norm = (const float *)get_dense(own, w->kv_norm, (size_t)cfg->head_dim * 4);
    A->sink = (const float *)get_dense(own, w->sink, (size_t)cfg->n_heads * 4);
    if (!A->wo_a || !A->q_norm || !A->kv_norm || !A->sink) return 1;
    A->idx_wq_b = nullptr; A->idx_wproj = nullptr;
    if (cfg->ratio && comp_weights(w->comp, cfg->dim, &A->comp, own)) return 1;
    if (cfg->ratio && cfg->has_indexer) {
        if (comp_weights(w->idx_comp, cfg->dim, &A->idx_comp, own)) return 1;
        A->idx_wq_b = get_qw(own, 8, w->idx_wq_b.codes, w->idx_wq_b.scales, cfg->idx_heads * cfg->idx_dim,
                                cfg->q_lora);
        A->idx_wproj = (const float *)get_dense(own, w->idx_wproj, (size_t)cfg->idx_heads * cfg->dim * 4);
        if (!A->idx_wq_b || !A->idx_wproj) return 1;
    }
    return 0;
}

void StateDev::release() {
    win.release();
    comp.kv.release(); comp.sc.release(); comp.cache.release();
    idx.kv.release(); idx.sc.release(); idx.cache.release();
}

__global__ void fill_kernel(float *p, size_t n, float v) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

static int comp_state_alloc(CompStateDev &S, int B, int ratio, int overlap, int d, int cap) {
    const int coff = 1 + overlap;
    S.carry = (size_t)coff * ratio * coff * d;
    S.cap = cap; S.nb = 0;
    if (S.kv.get(S.carry * B * 4, nullptr) || S.sc.get(S.carry * B * 4, nullptr) ||
        S.cache.get((size_t)B * cap * d * 4 + 16, nullptr))
        return 1;
    return 0;
}

int attn_state_init(const ApusAttnCfg &c, StateDev &S, int B, int cap) {
    Ctx &cx = ctx();
    S.B = B;
    if (S.win.get((size_t)B * c.window * c.head_dim * 4, nullptr)) return 1;
    APUS_CUDA_OK(cudaMemsetAsync(S.win.p, 0, (size_t)B * c.window * c.head_dim * 4, cx.stream));
    if (c.ratio) {
        if (comp_state_alloc(S.comp, B, c.ratio, c.ratio == 4, c.head_dim, cap)) return 1;
        APUS_CUDA_OK(cudaMemsetAsync(S.comp.kv.p, 0, S.comp.carry * B * 4, cx.stream));
        fill_kernel<<<ceil_div(S.comp.carry * B, 256), 256, 0, cx.stream>>>(S.comp.sc.as<float>(), S.comp.carry * B, -INFINITY);
        if (c.has_indexer) {
            if (comp_state_alloc(S.idx, B, c.ratio, 1, c.idx_dim, cap)) return 1;
            APUS_CUDA_OK(cudaMemsetAsync(S.idx.kv.p, 0, S.idx.carry * B * 4, cx.stream));
            fill_kernel<<<ceil_div(S.idx.carry * B, 256), 256, 0, cx.stream>>>(S.idx.sc.as<float>(), S.idx.carry * B, -INFINITY);
        }
    }
    return 0;
}

int attn_step_bufs(const ApusAttnCfg &c, long long max_nb, int B, DevBuf *ws, StepBufs *b) {
    const int hd = c.n_heads * c.head_dim;
    int kmax = c.dim;
    if (c.q_lora > kmax) kmax = c.q_lora;
    if (c.o_groups * c.o_lora > kmax) kmax = c.o_groups * c.o_lora;
    const size_t cdmax = 2 * (size_t)(c.head_dim > c.idx_dim ? c.head_dim : c.idx_dim);
    const size_t idxw = (size_t)c.window + (size_t)(c.has_indexer ? c.idx_topk : max_nb) + 8;
    void *p[22];
    size_t sz[22] = {(size_t)c.q_lora * 4, (size_t)c.q_lora * 4, (size_t)hd * 4, (size_t)c.head_dim * 4,
                     (size_t)c.head_dim * 4, (size_t)(c.idx_heads * c.idx_dim + 4) * 4, cdmax * 4, cdmax * 4,
                     cdmax * 4, (size_t)(c.idx_heads + 4) * 4, (size_t)(max_nb + 8) * 4, (size_t)hd * 4,
                     (size_t)c.o_groups * c.o_lora * 4, (size_t)kmax, (size_t)(kmax / 128 + 1) * 4,
                     (size_t)(c.idx_topk + 8) * 4, idxw * 4,
                     (size_t)kmax, (size_t)(kmax / 128 + 1) * 4, cdmax * 4, cdmax * 4, cdmax * 4};
    for (int i = 0; i < 22; i++)
        if (ws[i].get(sz[i] * B, &p[i])) return 1;
    b->xq2 = (uint8_t *)p[17]; b->xs2 = (float *)p[18]; b->ckv2 = (float *)p[19]; b->csc2 = (float *)p[20];
    b->pooled2 = (float *)p[21];
    b->qa = (float *)p[0]; b->qr = (float *)p[1]; b->q = (float *)p[2]; b->kva = (float *)p[3];
    b->kv = (float *)p[4]; b->iq = (float *)p[5]; b->ckv = (float *)p[6]; b->csc = (float *)p[7];
    b->pooled = (float *)p[8]; b->wt = (float *)p[9]; b->scores = (float *)p[10]; b->o = (float *)p[11];
    b->y = (float *)p[12]; b->xq = (uint8_t *)p[13]; b->xs = (float *)p[14]; b->sel = (int32_t *)p[15];
    b->idxs = (int32_t *)p[16];
    return 0;
}

// The two projections of a compressor (kv rows and gate scores, c/attn.h:960-975) read the same rows:
// one launch over two problems when the two weights and the two outputs are a whole number of 16-byte
// steps apart (device allocations are), else one launch each.  Same kernels, same sums either way.
static int comp_project(const CompDev &W, const float *x, float *ckv, float *csc, int rows, int dim, int cd, cudaStream_t st) {
    // distances in the flat device address space, in floats (the two tensors are separate allocations)
    const long long bw = (long long)((uintptr_t)W.wgate - (uintptr_t)W.wkv), bo = (long long)((uintptr_t)csc - (uintptr_t)ckv);
    const long long dw = bw / 4, dout = bo / 4;
    if (bw > 0 && bo > 0 && bw % 16 == 0 && bo % 16 == 0)
        return f32_linear_batched(W.wkv, (long long)dw, x, 0, dim, ckv, (long long)dout, cd, 2, rows, dim, cd,
                                  APUS_LIN_CLASS(APUS_CUDA_TREE_COMPRESSOR), st);
    return f32_linear(W.wkv, x, ckv, rows, dim, cd, APUS_LIN_CLASS(APUS_CUDA_TREE_COMPRESSOR), st) ||
           f32_linear(W.wgate, x, csc, rows, dim, cd, APUS_LIN_CLASS(APUS_CUDA_TREE_COMPRESSOR), st);
}

// One compressor decode step of B sequences; appends a finished entry to every
// cache when the block completes (reference c/attn.h:960-1008 + 797-819).
static int compressor_step(const CompDev &W, CompStateDev &S, const float *x, int B, int dim, long long pos,
                           const float *cs_rp, const StepBufs &b0, cudaStream_t st, const long long *pos_dev,
                           const float *cs_table, bool second_set = false) {
    StepBufs b = b0;
    if (second_set) { b.ckv = b0.ckv2; b.csc = b0.csc2; b.pooled = b0.pooled2; }
    const int cd = (1 + W.overlap) * W.d;
    if (comp_project(W, x, b.ckv, b.csc, B, dim, cd, st)) return 1;
    const int slot = (int)(pos % W.ratio);
    const int should = (pos + 1) % W.ratio == 0;
    if (comp_step(S.kv.as<float>(), S.sc.as<float>(), (long long)S.carry, b.ckv, b.csc, cd, W.ape, W.ratio,
                  W.overlap, W.d, slot, should, b.pooled, W.d, B, st, pos_dev))
        return 1;
    if (pos_dev) {
        // position on the device: the append is always launched and gates itself; the
        // entry index and the rope row follow from the position; the caller keeps S.nb
        int flags = ROW_BF16_IN | ROW_RMS_W | ROW_ROPE | ROW_BF16_OUT |
                    (W.rotate ? (ROW_HADAMARD | ROW_FP4QAT) : ROW_FP8QAT);
        const RowDyn dyn = {pos_dev, 1 - W.ratio, W.ratio, (long long)W.d};
        return row_ops(b.pooled, W.d, S.cache.as<float>(), S.cap * W.d, B, W.d, flags, W.norm, W.eps, W.rd, cs_table,
                       B, 0, st, &dyn);
    }
    if (should) {
        APUS_REQUIRE(S.nb < S.cap, "compressed cache is full (%d entries)", S.cap);
        int flags = ROW_BF16_IN | ROW_RMS_W | ROW_ROPE | ROW_BF16_OUT |
                    (W.rotate ? (ROW_HADAMARD | ROW_FP4QAT) : ROW_FP8QAT);
        if (row_ops(b.pooled, W.d, S.cache.as<float>() + (size_t)S.nb * W.d, S.cap * W.d, B, W.d, flags, W.norm,
                    W.eps, W.rd, cs_rp, B, 0, st))
            return 1;
        S.nb++;
    }
    return 0;
}

int attn_step(const AttnDev &A, StateDev &S, const float *x, long long pos, const float *cs_pos,
              const float *cs_rp, float *out, const StepBufs &b, int *idx_k_out, cudaStream_t st,
              const long long *pos_dev, const float *cs_table, bool x_codes) {
    const ApusAttnCfg &c = A.cfg;
    const int B = S.B;
    // pos_dev != NULL: every position-dependent value is read on the device from
    // *pos_dev (rope rows from cs_table), so the launches are the same at every position
    const RowDyn dyn_pos = {pos_dev, 0, 0, 0};
    const RowDyn *dp = pos_dev ? &dyn_pos : nullptr;
    if (pos_dev) cs_pos = cs_table;
    const int h = c.n_heads, d = c.head_dim, rd = c.rope_dim, win = c.window, ratio = c.ratio;
    const int hd = h * d;
    // Independent chains of the step run on side streams and are joined before the
    // gathered attention: (a) window KV, (b) the attention compressor, (c) the
    // indexer with its own compressor; the q path stays on `st`.  Each chain has
    // its own scratch.  The reference's order (indexer, ring write, compressor,
    // attention; c/attn.h:1572-1665) only matters through the data each step
    // reads, which the joins preserve.
    if (!x_codes && act_quant(x, nullptr, B, c.dim, b.xq, b.xs, nullptr, st)) return 1;   // x codes: wq_a and wkv
    cudaStream_t sa = branch_begin(st, 0);
    if (qgemm_dev(A.wkv, nullptr, b.xq, b.xs, B, b.kva, true, 0.f, sa)) return 1;       // (a) c/attn.h:1552-1569
    if (row_ops(b.kva, d, b.kv, d, B, d, ROW_RMS_W | ROW_ROPE | ROW_FP8QAT | ROW_BF16_OUT, A.kv_norm, c.eps, rd,
                cs_pos, B, 0, sa, dp))
        return 1;
    // ring write (c/attn.h:1642-1658): nothing reads the ring before the gathered attention, so it stays on (a)
    if (scatter_rows(S.win.as<float>() + (pos_dev ? 0 : (size_t)(pos % win) * d), (long long)win * d, b.kv, d, B, sa,
                     pos_dev, win))
        return 1;
    cudaStream_t sb = st;
    if (ratio) {                                                                         // (b) c/attn.h:1660-1665
        sb = branch_begin(st, 1);
        if (compressor_step(A.comp, S.comp, x, B, c.dim, pos, cs_rp, b, sb, pos_dev, cs_table)) return 1;
    }
    // the indexer's own compressor and its head weights read only x: they start with the step on a chain
    // of their own (d) and meet the q-dependent part of the indexer (c) before the scores
    cudaStream_t sd = st, se = st;
    if (ratio && c.has_indexer) {
        sd = branch_begin(st, 3);
        if (compressor_step(A.idx_comp, S.idx, x, B, c.dim, pos, cs_rp, b, sd, pos_dev, cs_table, true)) return 1;
        se = branch_begin(st, 4);                                  // (e) the head weights, beside (d)
        if (f32_linear(A.idx_wproj, x, b.wt, B, c.dim, c.idx_heads,
                       APUS_CUDA_R_IN | APUS_CUDA_R_OUT | APUS_LIN_CLASS(APUS_CUDA_TREE_IDX_WPROJ), se))
            return 1;
    }
    // q path (c/attn.h:1525-1548)
    if (qgemm_dev(A.wq_a, nullptr, b.xq, b.xs, B, b.qa, true, 0.f, st)) return 1;
    if (row_ops(b.qa, c.q_lora, b.qr, c.q_lora, B, c.q_lora, ROW_RMS_W, A.q_norm, c.eps, 0, nullptr, 1, 0, st, nullptr,
                b.xq2, b.xs2))                                                           // + qr codes: wq_b and idx_wq_b
        return 1;
    // compressed ids (c): the indexer
    int compw = 0;
    const int32_t *sel = nullptr;
    cudaStream_t sc = st;
    if (ratio) {
        const long long nbs = (pos + 1) / ratio;
        if (c.has_indexer) {
            const int ih = c.idx_heads, idm = c.idx_dim;
            sc = branch_begin(st, 2);
            if (qgemm_dev(A.idx_wq_b, nullptr, b.xq2, b.xs2, B, b.iq, true, 0.f, sc)) return 1;
            if (row_ops(b.iq, idm, b.iq, idm, B * ih, idm, ROW_ROPE | ROW_HADAMARD | ROW_FP4QAT | ROW_BF16_OUT, nullptr,
                        0.f, rd, cs_pos, B * ih, 0, sc, dp))
                return 1;
            if (sd != st && branch_end(3, sc)) return 1;          // (d), (e) -> (c): cache entry and head weights are ready
            if (se != st && branch_end(4, sc)) return 1;
            const float wscale = (float)(pow((double)idm, -0.5) * pow((double)ih, -0.5));
            compw = (int)(c.idx_topk < nbs ? c.idx_topk : nbs);
            if (pos_dev) {                         // capacities; the live counts are derived on the device
                compw = c.idx_topk < S.idx.cap ? c.idx_topk : S.idx.cap;
                if (idx_scores(b.iq, b.wt, wscale, S.idx.cache.as<float>(), (long long)S.idx.cap * idm, S.idx.cap, ih,
                               idm, b.scores, B, sc, pos_dev, ratio))
                    return 1;
                if (topk_stable(b.scores, S.idx.cap, compw, b.sel, B, sc, pos_dev, ratio)) return 1;
                sel = b.sel;
            } else if (compw > 0) {
                if (idx_scores(b.iq, b.wt, wscale, S.idx.cache.as<float>(), (long long)S.idx.cap * idm, nbs, ih, idm,
                               b.scores, B, sc))
                    return 1;
                if (topk_stable(b.scores, (int)nbs, compw, b.sel, B, sc)) return 1;
                sel = b.sel;
            }
        } else {
            compw = pos_dev ? S.comp.cap : (int)nbs;
        }
    }
    // the index row of the step (c/attn.h:692-737) reads the indexer's picks, or only the position: it is
    // written on the chain that has its last input, off the q path
    if (build_idx(b.idxs, win, pos, sel, compw, B, sel ? sc : sa, pos_dev, ratio)) return 1;
    // ... and compacted there, when the step has a scratch of its own to compact into
    if (b.sa && sparse_attn_compact(b.idxs, h, win + compw, B, b.sa, b.sa_cap, sel ? sc : sa)) return 1;
    if (qgemm_dev(A.wq_b, nullptr, b.xq2, b.xs2, B, b.q, true, 0.f, st)) return 1;
    if (row_ops(b.q, d, b.q, d, B * h, d, ROW_RMS_PLAIN | ROW_ROPE, nullptr, c.eps, rd, cs_pos, B * h, 0, st, dp)) return 1;
    // join the side chains: everything below reads what they produced
    if (sa != st && branch_end(0, st)) return 1;
    if (sb != st && branch_end(1, st)) return 1;
    if (sc != st && branch_end(2, st)) return 1;
    if (idx_k_out) *idx_k_out = compw;
    // gathered attention over ring ++ compressed cache, inverse RoPE
    const float scale = (float)pow((double)d, -0.5);
    const SaRope back = {cs_pos, pos_dev, rd};        // the rows leave the attention rotated back (c/attn.h:1384-1388)
    if (sparse_attn(b.q, A.sink, h, d, b.idxs, win + compw, B, scale, S.win.p, win,
                    ratio ? S.comp.cache.p : nullptr, ratio ? S.comp.nb : 0, 0, b.o, st, (long long)win * d,
                    ratio ? (long long)S.comp.cap * d : 0, b.sa, b.sa_cap, 0, b.sa != nullptr, &back))
        return 1;
    // grouped low-rank o-projection (c/attn.h:1692-1737)
    const int G = c.o_groups, ol = c.o_lora, sub = hd / G;
    LinCodes yq = {b.xq, b.xs, 0};                    // the codes of y for wo_b, from the kernel that finishes y when it can
    if (f32_linear_batched(A.wo_a, (long long)ol * sub, b.o, sub, hd, b.y, ol, G * ol, G, B, sub, ol,
                           APUS_CUDA_W_BF16 | APUS_CUDA_R_OUT | APUS_LIN_CLASS(APUS_CUDA_TREE_WO_A), st, &yq))
        return 1;
    if (yq.written) return qgemm_dev(A.wo_b, nullptr, b.xq, b.xs, B, out, true, 0.f, st);
    return qlinear_dev(A.wo_b, b.y, out, B, b.xq, b.xs, true, st);
}

// The compressor over a chunk: the two projections of every row at once, then the state machine
// position by position (it is sequential in t by definition, c/attn.h:960-1008; a launch per
// position on B CTAs) with the entries it completes appended as it goes.
static int compressor_chunk(const CompDev &W, CompStateDev &S, const float *x, int B, int s, int dim, long long pos0,
                            const float *cs_table, const StepBufs &b0, cudaStream_t st, bool second_set = false) {
    StepBufs b = b0;
    if (second_set) { b.ckv = b0.ckv2; b.csc = b0.csc2; b.pooled = b0.pooled2; }
    const int cd = (1 + W.overlap) * W.d, T = B * s;
    if (comp_project(W, x, b.ckv, b.csc, T, dim, cd, st)) return 1;
    const int flags = ROW_BF16_IN | ROW_RMS_W | ROW_ROPE | ROW_BF16_OUT | (W.rotate ? (ROW_HADAMARD | ROW_FP4QAT) : ROW_FP8QAT);
    for (int t = 0; t < s; t++) {
        const long long pos = pos0 + t;
        const int slot = (int)(pos % W.ratio), should = (pos + 1) % W.ratio == 0;
        float *pooled = b.pooled + (size_t)t * B * W.d;
        if (comp_step(S.kv.as<float>(), S.sc.as<float>(), (long long)S.carry, b.ckv + (size_t)t * B * cd,
                      b.csc + (size_t)t * B * cd, cd, W.ape, W.ratio, W.overlap, W.d, slot, should, pooled, W.d, B, st))
            return 1;
        if (!should) continue;
        APUS_REQUIRE(S.nb < S.cap, "compressed cache is full (%d entries)", S.cap);
        if (row_ops(pooled, W.d, S.cache.as<float>() + (size_t)S.nb * W.d, S.cap * W.d, B, W.d, flags, W.norm, W.eps,
                    W.rd, cs_table + (size_t)(pos + 1 - W.ratio) * W.rd, B, 0, st))
            return 1;
        S.nb++;
    }
    return 0;
}

int attn_chunk(const AttnDev &A, StateDev &S, const float *x, long long pos0, int s, const float *cs_table,
               float *out, const StepBufs &b, cudaStream_t st) {
    const ApusAttnCfg &c = A.cfg;
    const int B = S.B, T = B * s;
    const int h = c.n_heads, d = c.head_dim, rd = c.rope_dim, win = c.window, ratio = c.ratio;
    const int hd = h * d;
    const float *cs0 = cs_table + (size_t)pos0 * rd;       // row t of the chunk rotates by table row pos0 + t
    APUS_REQUIRE(b.ext != nullptr, "attn_chunk: no window buffer");
    if (act_quant(x, nullptr, T, c.dim, b.xq, b.xs, nullptr, st)) return 1;
    // window KV rows (c/attn.h:1552-1569)
    if (qgemm_dev(A.wkv, nullptr, b.xq, b.xs, T, b.kva, true, 0.f, st)) return 1;
    if (row_ops(b.kva, d, b.kv, d, T, d, ROW_RMS_W | ROW_ROPE | ROW_FP8QAT | ROW_BF16_OUT, A.kv_norm, c.eps, rd, cs0, B, rd, st))
        return 1;
    // q path (c/attn.h:1525-1548)
    if (qgemm_dev(A.wq_a, nullptr, b.xq, b.xs, T, b.qa, true, 0.f, st)) return 1;
    if (row_ops(b.qa, c.q_lora, b.qr, c.q_lora, T, c.q_lora, ROW_RMS_W, A.q_norm, c.eps, 0, nullptr, 1, 0, st, nullptr, b.xq2,
                b.xs2))
        return 1;
    if (qgemm_dev(A.wq_b, nullptr, b.xq2, b.xs2, T, b.q, true, 0.f, st)) return 1;
    if (row_ops(b.q, d, b.q, d, T * h, d, ROW_RMS_PLAIN | ROW_ROPE, nullptr, c.eps, rd, cs0, B * h, rd, st)) return 1;
    // compressed entries and the ids each row may attend to (c/attn.h:1105-1168, 1660-1665): an entry is
    // final once appended, and row t reads only the (pos0 + t + 1) / ratio entries complete at its position
    int compcap = 0;
    const int32_t *sel = nullptr;
    if (ratio) {
        if (compressor_chunk(A.comp, S.comp, x, B, s, c.dim, pos0, cs_table, b, st)) return 1;
        const long long nb_end = (pos0 + s) / ratio;
        if (c.has_indexer) {
            const int ih = c.idx_heads, idm = c.idx_dim;
            if (qgemm_dev(A.idx_wq_b, nullptr, b.xq2, b.xs2, T, b.iq, true, 0.f, st)) return 1;
            if (row_ops(b.iq, idm, b.iq, idm, T * ih, idm, ROW_ROPE | ROW_HADAMARD | ROW_FP4QAT | ROW_BF16_OUT, nullptr, 0.f,
                        rd, cs0, B * ih, rd, st))
                return 1;
            if (compressor_chunk(A.idx_comp, S.idx, x, B, s, c.dim, pos0, cs_table, b, st, true)) return 1;
            if (f32_linear(A.idx_wproj, x, b.wt, T, c.dim, ih,
                           APUS_CUDA_R_IN | APUS_CUDA_R_OUT | APUS_LIN_CLASS(APUS_CUDA_TREE_IDX_WPROJ), st))
                return 1;
            const float wscale = (float)(pow((double)idm, -0.5) * pow((double)ih, -0.5));
            compcap = (int)(c.idx_topk < nb_end ? c.idx_topk : nb_end);
            if (compcap > 0) {
                if (idx_scores(b.iq, b.wt, wscale, S.idx.cache.as<float>(), (long long)S.idx.cap * idm, nb_end, ih, idm,
                               b.scores, T, st, nullptr, ratio, pos0, B))
                    return 1;
                if (topk_stable(b.scores, (int)nb_end, compcap, b.sel, T, st, nullptr, ratio, pos0, B)) return 1;
                sel = b.sel;
            }
        } else {
            compcap = (int)nb_end;
        }
    }
    // window candidates in position order, index rows, gathered attention, inverse RoPE
    if (win_ext(b.ext, S.win.as<float>(), b.kv, win, s, d, B, pos0, st)) return 1;
    if (build_idx_chunk(b.idxs, win, s, pos0, B, sel, compcap, ratio, st)) return 1;
    const float scale = (float)pow((double)d, -0.5);
    if (sparse_attn(b.q, A.sink, h, d, b.idxs, win + compcap, T, scale, b.ext, win + s, ratio ? S.comp.cache.p : nullptr,
                    ratio ? S.comp.nb : 0, 0, b.o, st, (long long)(win + s) * d, ratio ? (long long)S.comp.cap * d : 0, b.sa,
                    b.sa_cap, B))
        return 1;
    if (ring_update(S.win.as<float>(), b.kv, win, s, d, B, pos0, st)) return 1;
    if (row_ops(b.o, d, b.o, d, T * h, d, ROW_ROPE_INV, nullptr, 0.f, rd, cs0, B * h, rd, st)) return 1;
    // grouped low-rank o-projection (c/attn.h:1692-1737)
    const int G = c.o_groups, ol = c.o_lora, sub = hd / G;
    if (f32_linear_batched(A.wo_a, (long long)ol * sub, b.o, sub, hd, b.y, ol, G * ol, G, T, sub, ol,
                           APUS_CUDA_W_BF16 | APUS_CUDA_R_OUT | APUS_LIN_CLASS(APUS_CUDA_TREE_WO_A), st))
        return 1;
    return qlinear_dev(A.wo_b, b.y, out, T, b.xq, b.xs, true, st);
}

static int upload_comp(const ApusCompS &h, CompStateDev &d, int extra, cudaStream_t st) {
    const size_t sb = (size_t)h.rows * h.cols * 4;
    d.carry = (size_t)h.rows * h.cols;
    d.cap = h.nb + extra + 1;
    if (d.kv.get(sb, nullptr) || d.sc.get(sb, nullptr) || d.cache.get((size_t)d.cap * h.d * 4, nullptr))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(d.kv.p, h.kv, sb, cudaMemcpyHostToDevice, st));
    APUS_CUDA_OK(cudaMemcpyAsync(d.sc.p, h.sc, sb, cudaMemcpyHostToDevice, st));
    if (h.nb) APUS_CUDA_OK(cudaMemcpyAsync(d.cache.p, h.cache, (size_t)h.nb * h.d * 4, cudaMemcpyHostToDevice, st));
    d.nb = h.nb;
    return 0;
}

static int download_comp(ApusCompS &h, const CompStateDev &d, cudaStream_t st) {
    const size_t sb = (size_t)h.rows * h.cols * 4;
    APUS_REQUIRE(d.nb <= h.cap, "attention: the host compressed cache holds %d entries but %d are needed", h.cap, d.nb);
    APUS_CUDA_OK(cudaMemcpyAsync(h.kv, d.kv.p, sb, cudaMemcpyDeviceToHost, st));
    APUS_CUDA_OK(cudaMemcpyAsync(h.sc, d.sc.p, sb, cudaMemcpyDeviceToHost, st));
    if (d.nb > h.nb)
        APUS_CUDA_OK(cudaMemcpyAsync(h.cache + (size_t)h.nb * h.d, (const float *)d.cache.p + (size_t)h.nb * h.d,
                                     (size_t)(d.nb - h.nb) * h.d * 4, cudaMemcpyDeviceToHost, st));
    return 0;
}


int attn_state_upload(const ApusAttnCfg &c, const ApusAttnS *st, StateDev &S, int extra, cudaStream_t sm) {
    S.B = 1;
    if (S.win.get((size_t)c.window * c.head_dim * 4, nullptr)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(S.win.p, st->win, (size_t)c.window * c.head_dim * 4, cudaMemcpyHostToDevice, sm));
    if (c.ratio && upload_comp(st->comp, S.comp, extra, sm)) return 1;
    if (c.ratio && c.has_indexer && upload_comp(st->idx_comp, S.idx, extra, sm)) return 1;
    return 0;
}

// Copies ring, carries and the appended cache entries back; the caller updates
// the host entry counts with attn_state_commit after synchronising.
int attn_state_download(const ApusAttnCfg &c, ApusAttnS *st, const StateDev &S, cudaStream_t sm) {
    APUS_CUDA_OK(cudaMemcpyAsync(st->win, S.win.p, (size_t)c.window * c.head_dim * 4, cudaMemcpyDeviceToHost, sm));
    if (c.ratio) {
        if (download_comp(st->comp, S.comp, sm)) return 1;
        if (c.has_indexer && download_comp(st->idx_comp, S.idx, sm)) return 1;
    }
    return 0;
}

void attn_state_commit(const ApusAttnCfg &c, ApusAttnS *st, const StateDev &S) {
    if (c.ratio) {
        st->comp.nb = S.comp.nb;
        if (c.has_indexer) st->idx_comp.nb = S.idx.nb;
    }
}

}  // namespace apus

namespace {

StateDev g_state;
DevBuf g_ws[30];

void attn_release_all() {
    g_state.release();
    for (auto &b : g_ws) b.release();
}
struct AttnReg { AttnReg() { apus::on_disable(attn_release_all, nullptr); } } g_attn_reg;

}  // namespace

extern "C" {

int apus_cuda_attention(const ApusAttnCfg *cfg, const ApusAttnW *w, ApusAttnS *st, const float *x, int s,
                        int64_t start_pos, const float *cos, const float *sin, float *out,
                        ApusAttnInterm *interm) {
    if (ensure_enabled()) return 1;
    if (s <= 0) return 0;
    APUS_REQUIRE(cfg->head_dim <= 1024 && cfg->q_lora <= 1024 && cfg->head_dim % 32 == 0 && cfg->q_lora % 128 == 0 &&
                 cfg->dim % 128 == 0 && (cfg->o_groups * cfg->o_lora) % 128 == 0 && cfg->rope_dim % 2 == 0,
                 "attention: unsupported dimensions");
    Ctx &c = ctx();
    cudaStream_t sm = c.stream;
    AttnDev A;
    if (attn_weights(cfg, w, &A)) return 1;
    const int d = cfg->head_dim, win = cfg->window, ratio = cfg->ratio, half = cfg->rope_dim / 2;
    const int hd = cfg->n_heads * d;
    const long long max_nb = ratio ? (start_pos + s) / ratio + 2 : 0;
    StepBufs b;
    if (attn_step_bufs(*cfg, max_nb, 1, g_ws, &b)) return 1;
    g_state.B = 1;
    // state in
    const int extra = ratio ? s / ratio + 2 : 0;
    if (attn_state_upload(*cfg, st, g_state, extra, sm)) return 1;
    if (s > 1 && chunks_enabled()) {
        // one pass over the s positions; rope rows [p_lo, start_pos + s) staged as a table indexed by position
        const long long p_lo = ratio && start_pos + 1 - ratio < 0 ? 0 : (ratio ? start_pos + 1 - ratio : start_pos);
        const size_t n_cs = (size_t)(start_pos + s - p_lo);
        std::vector<float> cs(n_cs * 2 * half);
        for (size_t i = 0; i < n_cs; i++) {
            memcpy(&cs[i * 2 * half], cos + (p_lo + (long long)i) * half, half * 4);
            memcpy(&cs[i * 2 * half + half], sin + (p_lo + (long long)i) * half, half * 4);
        }
        StepBufs bc;
        if (attn_step_bufs(*cfg, max_nb, s, g_ws, &bc)) return 1;
        void *dcs, *dx, *dout, *dext;
        if (g_ws[22].get(cs.size() * 4, &dcs) || g_ws[23].get((size_t)s * cfg->dim * 4, &dx) ||
            g_ws[24].get((size_t)s * cfg->dim * 4, &dout) || g_ws[25].get((size_t)(win + s) * d * 4, &dext))
            return 1;
        bc.ext = (float *)dext;
        APUS_CUDA_OK(cudaMemcpyAsync(dcs, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, sm));
        APUS_CUDA_OK(cudaMemcpyAsync(dx, x, (size_t)s * cfg->dim * 4, cudaMemcpyHostToDevice, sm));
        const int nb0 = ratio ? st->comp.nb : 0, inb0 = (ratio && cfg->has_indexer) ? st->idx_comp.nb : 0;
        // the table pointer is only ever dereferenced at rows >= p_lo
        const float *table = (const float *)dcs - (ptrdiff_t)p_lo * 2 * half;
        if (attn_chunk(A, g_state, (const float *)dx, start_pos, s, table, (float *)dout, bc, sm)) return 1;
        if (interm) {
            if (interm->q) APUS_CUDA_OK(cudaMemcpyAsync(interm->q, bc.q, (size_t)s * hd * 4, cudaMemcpyDeviceToHost, sm));
            if (interm->win_kv) APUS_CUDA_OK(cudaMemcpyAsync(interm->win_kv, bc.kv, (size_t)s * d * 4, cudaMemcpyDeviceToHost, sm));
            if (interm->attn_out) APUS_CUDA_OK(cudaMemcpyAsync(interm->attn_out, bc.o, (size_t)s * hd * 4, cudaMemcpyDeviceToHost, sm));
            const long long nb_end = ratio ? (start_pos + s) / ratio : 0;
            const int compcap = (int)(cfg->idx_topk < nb_end ? cfg->idx_topk : nb_end);
            if (cfg->has_indexer && ratio) {
                std::vector<int32_t> hsel((size_t)s * (compcap > 0 ? compcap : 1));
                if (compcap > 0 && interm->idx_topk) {
                    APUS_CUDA_OK(cudaMemcpyAsync(hsel.data(), bc.sel, (size_t)s * compcap * 4, cudaMemcpyDeviceToHost, sm));
                    APUS_CUDA_OK(cudaStreamSynchronize(sm));
                }
                int idx_k = 0;
                for (int t = 0; t < s; t++) {
                    const long long nbs = (start_pos + t + 1) / ratio;
                    idx_k = (int)(cfg->idx_topk < nbs ? cfg->idx_topk : nbs);
                    if (interm->idx_topk)                 // ids as the attention sees them in a step: entry + window
                        for (int j = 0; j < idx_k; j++) interm->idx_topk[(size_t)t * cfg->idx_topk + j] = hsel[(size_t)t * compcap + j] + win;
                }
                interm->idx_k = idx_k;
            }
        }
        APUS_CUDA_OK(cudaMemcpyAsync(out, dout, (size_t)s * cfg->dim * 4, cudaMemcpyDeviceToHost, sm));
        if (interm && interm->o_out)
            APUS_CUDA_OK(cudaMemcpyAsync(interm->o_out, dout, (size_t)s * cfg->dim * 4, cudaMemcpyDeviceToHost, sm));
        if (attn_state_download(*cfg, st, g_state, sm)) return 1;
        APUS_CUDA_OK(cudaStreamSynchronize(sm));
        attn_state_commit(*cfg, st, g_state);
        if (ratio && interm) { interm->comp_nb = st->comp.nb - nb0; interm->idx_nb = cfg->has_indexer ? st->idx_comp.nb - inb0 : 0; }
        int stt = gemm_tc_status(1);
        APUS_REQUIRE(stt == 0, "attention: a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
        return 0;
    }
    // rope rows: per token [cos | sin] at its position and at the first position of the block it completes
    std::vector<float> cs((size_t)s * 4 * half, 0.f);
    for (int t = 0; t < s; t++) {
        const int64_t pos = start_pos + t, rp = ratio ? pos + 1 - ratio : -1;
        memcpy(&cs[(size_t)t * 4 * half], cos + pos * half, half * 4);
        memcpy(&cs[(size_t)t * 4 * half + half], sin + pos * half, half * 4);
        if (rp >= 0) {
            memcpy(&cs[(size_t)t * 4 * half + 2 * half], cos + rp * half, half * 4);
            memcpy(&cs[(size_t)t * 4 * half + 3 * half], sin + rp * half, half * 4);
        }
    }
    void *dcs, *dx, *dout;
    if (g_ws[22].get(cs.size() * 4, &dcs) || g_ws[23].get((size_t)s * cfg->dim * 4, &dx) ||
        g_ws[24].get((size_t)s * cfg->dim * 4, &dout))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dcs, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, sm));
    APUS_CUDA_OK(cudaMemcpyAsync(dx, x, (size_t)s * cfg->dim * 4, cudaMemcpyHostToDevice, sm));
    const int nb0 = ratio ? st->comp.nb : 0, inb0 = (ratio && cfg->has_indexer) ? st->idx_comp.nb : 0;
    for (int t = 0; t < s; t++) {
        const float *cs_pos = (const float *)dcs + (size_t)t * 4 * half;
        int idx_k = 0;
        if (attn_step(A, g_state, (const float *)dx + (size_t)t * cfg->dim, start_pos + t, cs_pos, cs_pos + 2 * half,
                      (float *)dout + (size_t)t * cfg->dim, b, &idx_k, sm))
            return 1;
        if (interm) {
            if (interm->q) APUS_CUDA_OK(cudaMemcpyAsync(interm->q + (size_t)t * hd, b.q, (size_t)hd * 4, cudaMemcpyDeviceToHost, sm));
            if (interm->win_kv) APUS_CUDA_OK(cudaMemcpyAsync(interm->win_kv + (size_t)t * d, b.kv, (size_t)d * 4, cudaMemcpyDeviceToHost, sm));
            if (interm->attn_out) APUS_CUDA_OK(cudaMemcpyAsync(interm->attn_out + (size_t)t * hd, b.o, (size_t)hd * 4, cudaMemcpyDeviceToHost, sm));
            if (interm->idx_topk && idx_k && cfg->has_indexer)
                APUS_CUDA_OK(cudaMemcpyAsync(interm->idx_topk + (size_t)t * cfg->idx_topk, b.idxs + win, (size_t)idx_k * 4,
                                             cudaMemcpyDeviceToHost, sm));
            interm->idx_k = idx_k;
            // the step buffers are reused by the next token
            if (interm->q || interm->win_kv || interm->attn_out || interm->idx_topk) APUS_CUDA_OK(cudaStreamSynchronize(sm));
        }
    }
    APUS_CUDA_OK(cudaMemcpyAsync(out, dout, (size_t)s * cfg->dim * 4, cudaMemcpyDeviceToHost, sm));
    if (interm && interm->o_out)
        APUS_CUDA_OK(cudaMemcpyAsync(interm->o_out, dout, (size_t)s * cfg->dim * 4, cudaMemcpyDeviceToHost, sm));
    // state out
    if (attn_state_download(*cfg, st, g_state, sm)) return 1;
    APUS_CUDA_OK(cudaStreamSynchronize(sm));
    attn_state_commit(*cfg, st, g_state);
    if (ratio) {
        if (interm) { interm->comp_nb = st->comp.nb - nb0; interm->idx_nb = cfg->has_indexer ? st->idx_comp.nb - inb0 : 0; }
    }
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "attention: a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
    return 0;
}

// ---- row helpers (c/attn.h:76-90) -------------------------------------------------------------
static int rows_host(float *x, int n, int rows, int flags, int rd, const float *cos, const float *sin) {
    if (ensure_enabled()) return 1;
    if (rows <= 0) return 0;
    Ctx &c = ctx();
    void *dx, *dcs = nullptr;
    if (g_ws[25].get((size_t)rows * n * 4, &dx)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dx, x, (size_t)rows * n * 4, cudaMemcpyHostToDevice, c.stream));
    if (cos) {
        const int half = rd / 2;
        std::vector<float> cs((size_t)rd);
        memcpy(cs.data(), cos, half * 4);
        memcpy(cs.data() + half, sin, half * 4);
        if (g_ws[26].get((size_t)rd * 4, &dcs)) return 1;
        APUS_CUDA_OK(cudaMemcpyAsync(dcs, cs.data(), (size_t)rd * 4, cudaMemcpyHostToDevice, c.stream));
        APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    }
    if (row_ops((float *)dx, n, (float *)dx, n, rows, n, flags, nullptr, 0.f, rd, (const float *)dcs, rows, 0, c.stream))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(x, dx, (size_t)rows * n * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

int apus_cuda_apply_rope(float *x, const float *cos, const float *sin, int n, int rd, int inverse, int rows) {
    return rows_host(x, n, rows, inverse ? ROW_ROPE_INV : ROW_ROPE, rd, cos, sin);
}
int apus_cuda_hadamard(float *x, int n, int rows) { return rows_host(x, n, rows, ROW_HADAMARD, 0, nullptr, nullptr); }
int apus_cuda_fp8_qat_sim(float *x, int n, int K, int rows) {
    return rows_host(x, n, rows, ROW_FP8QAT, n - K, nullptr, nullptr);
}
int apus_cuda_fp4_qat_sim(float *x, int n, int rows) { return rows_host(x, n, rows, ROW_FP4QAT, 0, nullptr, nullptr); }

}  // extern "C"
