// C ABI, part 2: the MoE sublayer (include/apus_b200.h; reference c/moe.h).
//
// An ApusCudaMoe holds, in HBM, the tiled weights of the local experts
// [e_lo, e_hi) as three slabs (w1, w3, w2 — expert-major), the f32 gate, the
// selection bias and the FP8 shared expert, plus the per-call workspaces
// (grown on demand, never shrunk).  A forward is a fixed sequence of kernels
// on the caller's stream, with no host synchronisation and no host-side
// decisions that depend on device data:
//   gate matmul -> router finish -> act quant(x) -> group routings by expert
//   -> gate/up GEMM + SwiGLU -> act quant(h) -> down GEMM (scatter to (t,j))
//   -> shared expert (3 FP8 GEMMs) -> ordered combine.
#include <stdlib.h>
#include <vector>

#include "runtime.cuh"

using namespace apus;

struct ApusCudaMoe {
    int E = 0, topk = 0, inter = 0, dim = 0, hash = 0, e_lo = 0, e_hi = 0;
    float route_scale = 0.f, limit = 0.f;
    const void *host_key = nullptr;
    float *gate_w = nullptr, *gate_bias = nullptr;
    int64_t *tid2eid = nullptr;           // device [vocab, topk] (hash layers)
    int64_t vocab = 0;
    uint8_t *slab = nullptr;              // all local expert tensors
    MoeSlab sl = {};
    int zero_scale = 0;
    DevQW sw1, sw2, sw3;                  // shared expert
    uint64_t weight_bytes = 0;
    // tcgen05 path: the same experts in the reference storage + TMA tensor maps
    bool use_tc = false, can_tc = false;
    uint8_t *raw = nullptr;               // owned copy of the reference storage (NULL when adopted)
    const uint8_t *rw1 = nullptr, *rw3 = nullptr, *rw2 = nullptr, *rs1 = nullptr, *rs3 = nullptr, *rs2 = nullptr;
    alignas(64) unsigned char map_w1[128], map_w3[128], map_w2[128], map_xq[128], map_hq[128];
    DevBuf b_t13, b_t2;
    // workspaces
    int cap_s = 0, cap_r = 0;
    DevBuf b_logits, b_sp, b_biased, b_idx, b_wgt, b_xq, b_xs, b_routrow, b_spos, b_srow,
        b_g13, b_g2, b_ng, b_h, b_hq, b_hs, b_eo, b_shared, b_sh_h, b_sh_hq, b_sh_hs, b_ids,
        b_tab, b_sh_xq, b_sh_xs;
    // optional per-kernel timing of the two expert GEMM launches
    bool timing = false;
    std::vector<cudaEvent_t> ev;
    size_t ev_used = 0;
    int ensure(int s, int n_rout);
    int mark(cudaStream_t st);
};

int ApusCudaMoe::mark(cudaStream_t st) {
    if (!timing) return 0;
    if (ev_used == ev.size()) {
        cudaEvent_t e;
        APUS_CUDA_OK(cudaEventCreate(&e));
        ev.push_back(e);
    }
    APUS_CUDA_OK(cudaEventRecord(ev[ev_used++], st));
    return 0;
}

int ApusCudaMoe::ensure(int s, int n_rout) {
    const size_t S = (size_t)(s > 0 ? s : 1), R = (size_t)(n_rout > 0 ? n_rout : 1);
    if (s > cap_s) {
        if (b_logits.get(S * E * 4, nullptr) || b_sp.get(S * E * 4, nullptr) ||
            b_biased.get(S * E * 4, nullptr) || b_idx.get(S * topk * 4, nullptr) ||
            b_wgt.get(S * topk * 4, nullptr) || b_shared.get(S * dim * 4, nullptr) ||
            b_sh_h.get(S * inter * 4, nullptr) || b_sh_hq.get(S * inter, nullptr) ||
            b_sh_hs.get(S * (inter / 128) * 4, nullptr) || b_ids.get(S * 8, nullptr) ||
            b_sh_xq.get(S * dim, nullptr) || b_sh_xs.get(S * (dim / 128) * 4, nullptr) ||
            b_tab.get(S * topk * 8, nullptr))
            return 1;
        cap_s = s;
    }
    // the activation-quant buffers serve both the token rows (route/forward)
    // and explicit xrows (experts_dev): size them by the larger of the two
    const size_t XR = S > R ? S : R;
    if ((int)XR > cap_r || n_rout > cap_r) {
        const size_t max_groups = R + (size_t)(e_hi - e_lo);
        if (b_xq.get(XR * dim, nullptr) || b_xs.get(XR * (dim / 128) * 4, nullptr) ||
            b_routrow.get(R * 4, nullptr) || b_spos.get(R * 4, nullptr) || b_srow.get(R * 4, nullptr) ||
            b_g13.get(max_groups * sizeof(GemmGroup), nullptr) ||
            b_g2.get(max_groups * sizeof(GemmGroup), nullptr) || b_ng.get(256, nullptr) ||
            b_h.get(R * inter * 4, nullptr) || b_hq.get(R * inter, nullptr) ||
            b_hs.get(R * (inter / 128) * 4, nullptr) || b_eo.get(R * dim * 4, nullptr) ||
            b_t13.get(max_groups * sizeof(TcGroup), nullptr) || b_t2.get(max_groups * sizeof(TcGroup), nullptr))
            return 1;
        APUS_CUDA_OK(cudaMemset(b_ng.p, 0, 256));
        if (use_tc && (tc_make_act_map(map_xq, b_xq.p, (long long)(b_xq.cap / dim), dim) ||
                       tc_make_act_map(map_hq, b_hq.p, (long long)(b_hq.cap / inter), inter)))
            return 1;
        cap_r = (int)XR;
    }
    return 0;
}

static int pick_chunk(int n_rout, int n_local) {
    // rows per work item: small batches keep one 8-column MMA tile
    long long avg = n_local > 0 ? ((long long)n_rout + n_local - 1) / n_local : n_rout;
    if (avg <= 4) return 8;
    if (avg <= 12) return 16;
    return 32;
}

// Routed experts on the tcgen05 path: group first, quantise the token rows
// straight into sorted order, then two block-scaled tensor-core GEMMs.
// qrows != NULL: the token rows arrive quantised (EP exchange: dim codes + dim/128 scales per row,
// quantised once on the token's home rank -- the quantisation is per token, so the codes are the
// ones this rank would compute); they are gathered into sorted order instead of being quantised here.
static int experts_run_tc(ApusCudaMoe *m, const float *xrows, const int32_t *rout_row,
                          const int32_t *rout_eid, int n_rout, float *eo, cudaStream_t st,
                          const uint8_t *qrows = nullptr) {
    const int dim = m->dim, inter = m->inter;
    const int n_local = m->e_hi - m->e_lo;
    const int chunk = 32;
    const int max_groups = n_rout < n_local + n_rout / chunk + 1 ? n_rout : n_local + n_rout / chunk + 1;
    int *ng = m->b_ng.as<int>();
    if (moe_group(rout_eid, rout_row, qrows ? 1 : m->topk, n_rout, m->sl, chunk, m->b_spos.as<int>(), m->b_srow.as<int>(),
                  m->b_g13.as<GemmGroup>(), m->b_g2.as<GemmGroup>(), ng, max_groups, st,
                  m->b_t13.as<TcGroup>(), m->b_t2.as<TcGroup>(), inter, dim))
        return 1;
    if (qrows ? ep_gather_q(qrows, dim, m->b_srow.as<int>(), ng + 1, n_rout, m->b_xq.as<uint8_t>(), m->b_xs.as<float>(), st)
              : act_quant(xrows, m->b_srow.as<int>(), n_rout, dim, m->b_xq.as<uint8_t>(), m->b_xs.as<float>(), ng + 1, st))
        return 1;
    TcArgs a = {};
    a.map_a = m->map_w1; a.map_b = m->map_w3; a.map_x = m->map_xq;
    a.scales_a = m->rs1; a.scales_b = m->rs3; a.ascales = m->b_xs.as<float>();
    a.groups = m->b_t13.as<TcGroup>(); a.n_groups_dev = ng; a.n_groups = max_groups;
    a.O = inter; a.K = dim; a.pair = 1; a.limit = m->limit; a.out = m->b_h.as<float>();
    a.total_rows = n_rout;
    // the gate/up kernel quantises its SwiGLU outputs for the down projection in its epilogue
    // (unless K is split, when the outputs only exist after the chunks are added)
    static const bool fuse_hq = !(getenv("APUS_FUSE_HQ") && getenv("APUS_FUSE_HQ")[0] == '0');
    const bool split = getenv("APUS_TC_KSPLIT") && atoi(getenv("APUS_TC_KSPLIT")) > 1;
    if (fuse_hq && !split) { a.q_out = m->b_hq.as<uint8_t>(); a.qs_out = m->b_hs.as<float>(); }
    if (m->mark(st) || gemm_tc(a, st) || m->mark(st)) return 1;
    if (!a.q_out && act_quant(m->b_h.as<float>(), nullptr, n_rout, inter, m->b_hq.as<uint8_t>(), m->b_hs.as<float>(),
                              ng + 1, st))
        return 1;
    TcArgs b = {};
    b.map_a = m->map_w2; b.map_b = m->map_w2; b.map_x = m->map_hq;
    b.scales_a = m->rs2; b.ascales = m->b_hs.as<float>();
    b.groups = m->b_t2.as<TcGroup>(); b.n_groups_dev = ng; b.n_groups = max_groups;
    b.O = dim; b.K = inter; b.pair = 0; b.round_out = 1; b.orow = m->b_spos.as<int>(); b.out = eo;
    b.total_rows = n_rout;
    if (m->mark(st) || gemm_tc(b, st) || m->mark(st)) return 1;
    return 0;
}

// Routed experts for arbitrary local routings (device pointers).
static int experts_run(ApusCudaMoe *m, const float *xrows, int n_rows, const int32_t *rout_row,
                       const int32_t *rout_eid, int n_rout, float *eo, cudaStream_t st) {
    if (n_rout <= 0) return 0;
    if (m->use_tc) return experts_run_tc(m, xrows, rout_row, rout_eid, n_rout, eo, st);
    const int dim = m->dim, inter = m->inter;
    const int n_local = m->e_hi - m->e_lo;
    const int chunk = pick_chunk(n_rout, n_local);
    const int max_groups = n_rout < n_local + n_rout / chunk + 1 ? n_rout : n_local + n_rout / chunk + 1;
    if (act_quant(xrows, nullptr, n_rows, dim, m->b_xq.as<uint8_t>(), m->b_xs.as<float>(), nullptr, st))
        return 1;
    if (moe_group(rout_eid, rout_row, m->topk, n_rout, m->sl, chunk, m->b_spos.as<int>(), m->b_srow.as<int>(),
                  m->b_g13.as<GemmGroup>(), m->b_g2.as<GemmGroup>(), m->b_ng.as<int>(), max_groups, st))
        return 1;
    GemmSmallArgs a = {};
    a.fmt = 4; a.pair = 1; a.limit = m->limit; a.O = inter; a.K = dim;
    a.groups = m->b_g13.as<GemmGroup>(); a.n_groups_dev = m->b_ng.as<int>(); a.n_groups = max_groups;
    a.max_rows = chunk;
    a.acodes = m->b_xq.as<uint8_t>(); a.ascales = m->b_xs.as<float>();
    a.arow = m->b_srow.as<int>(); a.orow = nullptr; a.out = m->b_h.as<float>();
    a.zero_scale = m->zero_scale;
    if (m->mark(st) || gemm_small(a, st) || m->mark(st)) return 1;
    // h rows are in sorted order; rows past the local routings are never read
    if (act_quant(m->b_h.as<float>(), nullptr, n_rout, inter, m->b_hq.as<uint8_t>(),
                  m->b_hs.as<float>(), nullptr, st))
        return 1;
    GemmSmallArgs b = {};
    b.fmt = 4; b.pair = 0; b.round_out = 1; b.O = dim; b.K = inter;
    b.groups = m->b_g2.as<GemmGroup>(); b.n_groups_dev = m->b_ng.as<int>(); b.n_groups = max_groups;
    b.max_rows = chunk;
    b.acodes = m->b_hq.as<uint8_t>(); b.ascales = m->b_hs.as<float>();
    b.arow = nullptr; b.orow = m->b_spos.as<int>(); b.out = eo;
    b.zero_scale = m->zero_scale;
    if (m->mark(st) || gemm_small(b, st) || m->mark(st)) return 1;
    return 0;
}

static int shared_run(ApusCudaMoe *m, const float *x, int s, float *shared, cudaStream_t st) {
    // own activation-code buffers: the shared expert may run beside the routed experts
    ExpertWs ws = {m->b_sh_h.as<float>(), m->b_sh_xq.as<uint8_t>(), m->b_sh_hq.as<uint8_t>(),
                   m->b_sh_xs.as<float>(), m->b_sh_hs.as<float>()};
    return expert_dev(&m->sw1, &m->sw2, &m->sw3, m->limit, x, s, shared, ws, st);
}

static int route_run(ApusCudaMoe *m, const float *x, const int64_t *ids, const int64_t *table,
                     int s, int32_t *idx, float *wgt, float *sp, float *biased, cudaStream_t st) {
    if (f32_linear(m->gate_w, x, m->b_logits.as<float>(), s, m->dim, m->E, APUS_LIN_CLASS(APUS_CUDA_TREE_ROUTER), st)) return 1;
    if (!sp) sp = m->b_sp.as<float>();
    if (m->hash) {
        APUS_REQUIRE(table && ids, "hash-routed layer: no tid2eid table / ids on device");
        return router_finish(m->b_logits.as<float>(), nullptr, table, ids, s, m->E, m->topk,
                             m->route_scale, sp, nullptr, idx, wgt, st);
    }
    if (!biased) biased = m->b_biased.as<float>();
    return router_finish(m->b_logits.as<float>(), m->gate_bias, nullptr, nullptr, s, m->E, m->topk,
                         m->route_scale, sp, biased, idx, wgt, st);
}

static int forward_run(ApusCudaMoe *m, const float *x, const int64_t *ids, const int64_t *table,
                       int s, float *out, float *routed, cudaStream_t st) {
    const int R = s * m->topk;
    if (m->ensure(s, R)) return 1;
    APUS_REQUIRE(m->e_lo == 0 && m->e_hi == m->E,
                 "moe_forward_dev needs all experts local (this handle holds [%d,%d) of %d)",
                 m->e_lo, m->e_hi, m->E);
    // the shared expert depends only on x: it runs on a side stream beside the
    // router and the routed experts and is joined before the combine
    cudaStream_t ss = branch_begin(st, 0);
    if (shared_run(m, x, s, m->b_shared.as<float>(), ss)) return 1;
    if (route_run(m, x, ids, table, s, m->b_idx.as<int32_t>(), m->b_wgt.as<float>(), nullptr, nullptr, st))
        return 1;
    if (experts_run(m, x, s, nullptr, m->b_idx.as<int32_t>(), R,
                    m->b_eo.as<float>(), st))
        return 1;
    if (ss != st && branch_end(0, st)) return 1;
    return moe_combine(m->b_eo.as<float>(), m->b_wgt.as<float>(), m->b_shared.as<float>(), s,
                       m->topk, m->dim, out, routed, st);
}

// One expert's three matrices as the descriptor gives them (directly or through
// the resolve hook, reference c/moe.h:57-62).
static int resolve_expert(const ApusMoeW *w, int e, ApusFp4W *r1, ApusFp4W *r2, ApusFp4W *r3) {
    if (w->hook_resolve) {
        if (w->hook_resolve(w->hook_ctx, w->layer_id, e, r1, r2, r3)) {
            set_error("moe_create: hook_resolve failed for expert %d", e);
            return 1;
        }
    } else { *r1 = w->w1[e]; *r2 = w->w2[e]; *r3 = w->w3[e]; }
    if (r1->O != w->inter || r1->K != w->dim || r3->O != w->inter || r3->K != w->dim ||
        r2->O != w->dim || r2->K != w->inter) {
        set_error("moe_create: expert %d has unexpected shapes", e);
        return 1;
    }
    return 0;
}

// The re-tiled copy of the local experts for the mma.sync kernel, built from
// the reference-storage copy already in HBM.
static int build_tiled(ApusCudaMoe *m) {
    if (m->slab) return 0;
    const int nl = m->e_hi - m->e_lo;
    const size_t c13 = (size_t)m->inter * m->dim / 2, s13 = (size_t)m->inter * m->dim / 32;
    const size_t c2 = c13, s2 = s13;
    const size_t total = (size_t)nl * (2 * (c13 + s13) + c2 + s2);
    if (!total) return 0;
    APUS_REQUIRE(m->rw1 != nullptr, "moe: no expert storage to re-tile from");
    if (cudaMalloc(&m->slab, total) != cudaSuccess) {
        set_error("moe: device allocation of %zu bytes (re-tiled experts) failed", total);
        m->slab = nullptr;
        return 1;
    }
    uint8_t *p = m->slab;
    m->sl.w1 = p; p += (size_t)nl * c13;
    m->sl.w3 = p; p += (size_t)nl * c13;
    m->sl.w2 = p; p += (size_t)nl * c2;
    m->sl.s1 = p; p += (size_t)nl * s13;
    m->sl.s3 = p; p += (size_t)nl * s13;
    m->sl.s2 = p;
    for (int le = 0; le < nl; le++) {
        int z1 = 0, z2 = 0, z3 = 0;
        if (upload_qw(4, m->rw1 + le * c13, m->rs1 + le * s13, m->inter, m->dim, (uint8_t *)m->sl.w1 + le * c13,
                      (uint8_t *)m->sl.s1 + le * s13, &z1) ||
            upload_qw(4, m->rw3 + le * c13, m->rs3 + le * s13, m->inter, m->dim, (uint8_t *)m->sl.w3 + le * c13,
                      (uint8_t *)m->sl.s3 + le * s13, &z3) ||
            upload_qw(4, m->rw2 + le * c2, m->rs2 + le * s2, m->dim, m->inter, (uint8_t *)m->sl.w2 + le * c2,
                      (uint8_t *)m->sl.s2 + le * s2, &z2))
            return 1;
        m->zero_scale |= z1 | z2 | z3;
    }
    return 0;
}

extern "C" {

ApusCudaMoe *apus_cuda_moe_create(const ApusMoeW *w, int e_lo, int e_hi) {
    if (ensure_enabled()) return nullptr;
    if (!w || e_lo < 0 || e_hi > w->E || e_lo > e_hi) { set_error("moe_create: bad expert range [%d,%d)", e_lo, e_hi); return nullptr; }
    if (w->dim % 128 || w->inter % 128) { set_error("moe_create: dim=%d inter=%d must be multiples of 128", w->dim, w->inter); return nullptr; }
    Ctx &c = ctx();
    ApusCudaMoe *m = new ApusCudaMoe();
    m->E = w->E; m->topk = w->topk; m->inter = w->inter; m->dim = w->dim; m->hash = w->hash;
    m->route_scale = w->route_scale; m->limit = w->limit; m->e_lo = e_lo; m->e_hi = e_hi;
    m->host_key = w->gate_w;
    const int nl = e_hi - e_lo;
    const size_t c13 = (size_t)w->inter * w->dim / 2, s13 = (size_t)w->inter * w->dim / 32;
    const size_t c2 = (size_t)w->dim * w->inter / 2, s2 = (size_t)w->dim * w->inter / 32;
    const size_t total = (size_t)nl * (2 * (c13 + s13) + c2 + s2);
    bool ok = true;
    ok = ok && cudaMalloc(&m->gate_w, (size_t)w->E * w->dim * 4) == cudaSuccess;
    ok = ok && cudaMemcpy(m->gate_w, w->gate_w, (size_t)w->E * w->dim * 4, cudaMemcpyDefault) == cudaSuccess;
    if (ok && !w->hash) {
        ok = ok && cudaMalloc(&m->gate_bias, (size_t)w->E * 4) == cudaSuccess;
        ok = ok && cudaMemcpy(m->gate_bias, w->gate_bias, (size_t)w->E * 4, cudaMemcpyDefault) == cudaSuccess;
    }
    if (!ok) { set_error("moe_create: upload of the gate failed"); apus_cuda_moe_destroy(m); return nullptr; }
    m->sl.code_stride13 = c13; m->sl.scale_stride13 = s13;
    m->sl.code_stride2 = c2; m->sl.scale_stride2 = s2;
    m->sl.e_lo = e_lo; m->sl.e_hi = e_hi;
    // The local experts in the reference storage (packed nibbles [O, K/2], scale
    // bytes [O, K/32]) as six expert-major slabs.  Device pointers that already
    // form such slabs are used in place (the caller keeps them alive, like the
    // stable host pointers of the reference's views); anything else is copied.
    std::vector<ApusFp4W> r1(nl), r2(nl), r3(nl);
    for (int le = 0; le < nl; le++)
        if (resolve_expert(w, e_lo + le, &r1[le], &r2[le], &r3[le])) { apus_cuda_moe_destroy(m); return nullptr; }
    bool adopt = nl > 0;
    for (int le = 0; le < nl && adopt; le++)
        adopt = r1[le].packed == r1[0].packed + le * c13 && r3[le].packed == r3[0].packed + le * c13 &&
                r2[le].packed == r2[0].packed + le * c2 && r1[le].scales == r1[0].scales + le * s13 &&
                r3[le].scales == r3[0].scales + le * s13 && r2[le].scales == r2[0].scales + le * s2;
    if (adopt)
        adopt = is_device_ptr(r1[0].packed) && is_device_ptr(r3[0].packed) && is_device_ptr(r2[0].packed) &&
                is_device_ptr(r1[0].scales) && is_device_ptr(r3[0].scales) && is_device_ptr(r2[0].scales) &&
                ((uintptr_t)r1[0].packed % 128 == 0) && ((uintptr_t)r3[0].packed % 128 == 0) &&
                ((uintptr_t)r2[0].packed % 128 == 0) && ((uintptr_t)r1[0].scales % 16 == 0) &&
                ((uintptr_t)r3[0].scales % 16 == 0) && ((uintptr_t)r2[0].scales % 16 == 0);
    if (adopt) {
        m->rw1 = r1[0].packed; m->rw3 = r3[0].packed; m->rw2 = r2[0].packed;
        m->rs1 = r1[0].scales; m->rs3 = r3[0].scales; m->rs2 = r2[0].scales;
    } else if (nl > 0) {
        if (cudaMalloc(&m->raw, total) != cudaSuccess) {
            set_error("moe_create: device allocation of %zu bytes failed", total);
            m->raw = nullptr;
            apus_cuda_moe_destroy(m); return nullptr;
        }
        uint8_t *q = m->raw;
        uint8_t *d1 = q; q += (size_t)nl * c13;
        uint8_t *d3 = q; q += (size_t)nl * c13;
        uint8_t *d2 = q; q += (size_t)nl * c2;
        uint8_t *e1 = q; q += (size_t)nl * s13;
        uint8_t *e3 = q; q += (size_t)nl * s13;
        uint8_t *e2 = q;
        m->rw1 = d1; m->rw3 = d3; m->rw2 = d2; m->rs1 = e1; m->rs3 = e3; m->rs2 = e2;
        for (int le = 0; le < nl; le++) {
            bool ok2 = cudaMemcpy(d1 + le * c13, r1[le].packed, c13, cudaMemcpyDefault) == cudaSuccess &&
                       cudaMemcpy(d3 + le * c13, r3[le].packed, c13, cudaMemcpyDefault) == cudaSuccess &&
                       cudaMemcpy(d2 + le * c2, r2[le].packed, c2, cudaMemcpyDefault) == cudaSuccess &&
                       cudaMemcpy(e1 + le * s13, r1[le].scales, s13, cudaMemcpyDefault) == cudaSuccess &&
                       cudaMemcpy(e3 + le * s13, r3[le].scales, s13, cudaMemcpyDefault) == cudaSuccess &&
                       cudaMemcpy(e2 + le * s2, r2[le].scales, s2, cudaMemcpyDefault) == cudaSuccess;
            if (!ok2) { set_error("moe_create: upload of expert %d failed", e_lo + le); apus_cuda_moe_destroy(m); return nullptr; }
        }
        c.bytes_uploaded += total;
    }
    // tcgen05 kernel on that storage when the shapes allow; otherwise (or on
    // request, apus_cuda_moe_use_tc) the mma.sync kernel on a re-tiled copy
    {
        const char *env = getenv("APUS_MOE_TC");
        m->use_tc = !(env && env[0] == '0') && w->inter % 512 == 0 && w->dim % 512 == 0 && nl > 0;
    }
    if (m->use_tc) {
        if (tc_make_weight_map(m->map_w1, m->rw1, (long long)nl * w->inter, w->dim) ||
            tc_make_weight_map(m->map_w3, m->rw3, (long long)nl * w->inter, w->dim) ||
            tc_make_weight_map(m->map_w2, m->rw2, (long long)nl * w->dim, w->inter)) {
            apus_cuda_moe_destroy(m); return nullptr;
        }
        m->can_tc = true;
    } else if (build_tiled(m)) {
        apus_cuda_moe_destroy(m); return nullptr;
    }
    // shared expert
    struct { DevQW *d; const ApusFp8W *h; int O, K; } sh[3] = {
        {&m->sw1, &w->sw1, w->inter, w->dim}, {&m->sw3, &w->sw3, w->inter, w->dim},
        {&m->sw2, &w->sw2, w->dim, w->inter}};
    for (auto &q : sh) {
        DevQW *d = new_qw(8, q.h->codes, q.h->scales, q.O, q.K);
        if (!d) { apus_cuda_moe_destroy(m); return nullptr; }
        *q.d = *d;
        delete d;                               // storage now owned by the member copy
    }
    m->weight_bytes = total + m->sw1.bytes() + m->sw2.bytes() + m->sw3.bytes() +
                      (size_t)w->E * w->dim * 4 + (w->hash ? 0 : (size_t)w->E * 4);
    return m;
}

void apus_cuda_moe_destroy(ApusCudaMoe *m) {
    if (!m) return;
    cudaDeviceSynchronize();
    if (m->gate_w) cudaFree(m->gate_w);
    if (m->gate_bias) cudaFree(m->gate_bias);
    if (m->tid2eid) cudaFree(m->tid2eid);
    if (m->slab) cudaFree(m->slab);
    if (m->raw) cudaFree(m->raw);
    m->sw1.release(); m->sw2.release(); m->sw3.release();
    DevBuf *bufs[] = {&m->b_logits, &m->b_sp, &m->b_biased, &m->b_idx, &m->b_wgt, &m->b_xq, &m->b_xs,
                      &m->b_routrow, &m->b_spos, &m->b_srow, &m->b_g13, &m->b_g2, &m->b_ng, &m->b_h,
                      &m->b_hq, &m->b_hs, &m->b_eo, &m->b_shared, &m->b_sh_h, &m->b_sh_hq,
                      &m->b_sh_hs, &m->b_ids, &m->b_tab, &m->b_t13, &m->b_t2, &m->b_sh_xq, &m->b_sh_xs};
    for (DevBuf *b : bufs) b->release();
    for (cudaEvent_t e : m->ev) cudaEventDestroy(e);
    delete m;
}

uint64_t apus_cuda_moe_bytes(const ApusCudaMoe *m) { return m ? m->weight_bytes : 0; }

ApusCudaMoe *apus_cuda_moe_get(const ApusMoeW *w) {
    if (ensure_enabled()) return nullptr;
    Ctx &c = ctx();
    auto it = c.moes.find(w->gate_w);
    if (it != c.moes.end()) return it->second;
    ApusCudaMoe *m = apus_cuda_moe_create(w, 0, w->E);
    if (m) c.moes[w->gate_w] = m;
    return m;
}

/* 1 = tcgen05 block-scaled kernel on the reference weight storage, 0 = the
 * mma.sync kernel on the re-tiled copy.  Returns the setting now in force. */
int apus_cuda_moe_use_tc(ApusCudaMoe *m, int enable) {
    if (!m) return -1;
    if (enable >= 0 && m->can_tc) {
        bool on = enable != 0;
        if (!on && build_tiled(m)) return -1;
        if (on != m->use_tc) { m->use_tc = on; m->cap_r = 0; }    // act maps are rebuilt by ensure()
    }
    return m->use_tc ? 1 : 0;
}

int apus_cuda_moe_timing_enabled(const ApusCudaMoe *m) { return m && m->timing ? 1 : 0; }

void apus_cuda_moe_timing(ApusCudaMoe *m, int enable) {
    if (!m) return;
    m->timing = enable != 0;
    m->ev_used = 0;
}

int apus_cuda_moe_timing_read(ApusCudaMoe *m, double *ms_gate_up, double *ms_down, int *launches) {
    if (!m) { set_error("NULL moe handle"); return 1; }
    double a = 0, b = 0;
    int n = 0;
    for (size_t i = 0; i + 3 < m->ev_used; i += 4) {
        float t;
        APUS_CUDA_OK(cudaEventSynchronize(m->ev[i + 3]));
        APUS_CUDA_OK(cudaEventElapsedTime(&t, m->ev[i], m->ev[i + 1]));
        a += t;
        APUS_CUDA_OK(cudaEventElapsedTime(&t, m->ev[i + 2], m->ev[i + 3]));
        b += t;
        n++;
    }
    if (ms_gate_up) *ms_gate_up = a;
    if (ms_down) *ms_down = b;
    if (launches) *launches = n;
    m->ev_used = 0;
    return 0;
}

/* Work items (expert x up to 32 rows) launched since the last reset: at decode
 * sizes one per distinct expert touched, i.e. the number of expert weight sets
 * the GEMV kernels streamed. */
long long apus_cuda_moe_work_items(ApusCudaMoe *m, int reset) {
    if (!m || !m->b_ng.p) return 0;
    int v[4] = {0, 0, 0, 0};
    cudaStream_t st = ctx().stream;
    if (cudaMemcpyAsync(v, m->b_ng.p, sizeof v, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess)
        return -1;
    if (reset) { cudaMemsetAsync(m->b_ng.as<int>() + 2, 0, sizeof(int), st); cudaStreamSynchronize(st); }
    return v[2];
}

int apus_cuda_moe_set_hash_table(ApusCudaMoe *m, const int64_t *tid2eid, int64_t vocab) {
    if (!m || !m->hash) { set_error("set_hash_table: not a hash-routed layer"); return 1; }
    if (m->tid2eid) { cudaDeviceSynchronize(); cudaFree(m->tid2eid); m->tid2eid = nullptr; }
    size_t bytes = (size_t)vocab * m->topk * 8;
    APUS_CUDA_OK(cudaMalloc(&m->tid2eid, bytes));
    APUS_CUDA_OK(cudaMemcpy(m->tid2eid, tid2eid, bytes, cudaMemcpyDefault));
    m->vocab = vocab;
    return 0;
}

int apus_cuda_moe_route_dev(const ApusCudaMoe *mc, const float *x, const int64_t *ids, int s,
                            int32_t *idx, float *wgt, float *sp, float *biased, void *stream) {
    ApusCudaMoe *m = const_cast<ApusCudaMoe *>(mc);
    if (!m) { set_error("NULL moe handle"); return 1; }
    if (s <= 0) return 0;
    if (m->ensure(s, s * m->topk)) return 1;
    return route_run(m, x, ids, m->tid2eid, s, idx, wgt, sp, biased, (cudaStream_t)stream);
}

int apus_cuda_moe_experts_dev(ApusCudaMoe *m, const float *xrows, int n_rows, const int32_t *rout_row,
                              const int32_t *rout_eid, int n_rout, float *eo, void *stream) {
    if (!m) { set_error("NULL moe handle"); return 1; }
    if (n_rout <= 0) return 0;
    if (m->ensure(n_rows, n_rout)) return 1;
    return experts_run(m, xrows, n_rows, rout_row, rout_eid, n_rout, eo, (cudaStream_t)stream);
}

// ---- expert parallelism with the compact payload -------------------------------------------
size_t apus_cuda_moe_ep_row_bytes(const ApusCudaMoe *m) { return m ? (size_t)m->dim + (size_t)(m->dim / 128) * 4 : 0; }

int apus_cuda_moe_ep_pack_dev(ApusCudaMoe *m, const float *x, int s, const int32_t *slot_of, int n_rout,
                              uint8_t *send, void *stream) {
    if (!m) { set_error("NULL moe handle"); return 1; }
    if (s <= 0 || n_rout <= 0) return 0;
    APUS_REQUIRE(m->dim % 128 == 0, "moe_ep_pack: dim=%d must be a multiple of 128", m->dim);
    if (m->ensure(s, n_rout)) return 1;
    cudaStream_t st = (cudaStream_t)stream;
    // one quantisation per token (c/moe.h:246-254), then every routing's copy goes into its slot
    if (act_quant(x, nullptr, s, m->dim, m->b_xq.as<uint8_t>(), m->b_xs.as<float>(), nullptr, st)) return 1;
    return ep_pack_q(m->b_xq.as<uint8_t>(), m->b_xs.as<float>(), m->dim, slot_of, n_rout, m->topk, send, st);
}

int apus_cuda_moe_experts_q_dev(ApusCudaMoe *m, const uint8_t *qrows, int n_rows, const int32_t *rout_eid,
                                uint16_t *eo_bf16, void *stream) {
    if (!m) { set_error("NULL moe handle"); return 1; }
    if (n_rows <= 0) return 0;
    APUS_REQUIRE(m->use_tc, "moe_experts_q: needs the tcgen05 expert path (shapes that are multiples of 512)");
    if (m->ensure(n_rows, n_rows)) return 1;
    cudaStream_t st = (cudaStream_t)stream;
    // routing i is row i; the rows' expert outputs are BF16 values (c/attn.h:447): their bits travel back
    if (experts_run_tc(m, nullptr, nullptr, rout_eid, n_rows, m->b_eo.as<float>(), st, qrows)) return 1;
    return f32_to_bf16(m->b_eo.as<float>(), eo_bf16, (long long)n_rows * m->dim, st);
}

int apus_cuda_moe_ep_unpack_dev(const uint16_t *back, int dim, const int32_t *slot_of, int n_rout, float *eo,
                                void *stream) {
    return ep_unpack_bf16(back, dim, slot_of, n_rout, eo, (cudaStream_t)stream);
}

int apus_cuda_moe_shared_dev(ApusCudaMoe *m, const float *x, int s, float *shared, void *stream) {
    if (!m) { set_error("NULL moe handle"); return 1; }
    if (s <= 0) return 0;
    if (m->ensure(s, s * m->topk)) return 1;
    return shared_run(m, x, s, shared, (cudaStream_t)stream);
}

int apus_cuda_moe_combine_dev(const ApusCudaMoe *m, const float *eo, const float *wgt,
                              const float *shared, int s, float *out, float *routed, void *stream) {
    if (!m) { set_error("NULL moe handle"); return 1; }
    return moe_combine(eo, wgt, shared, s, m->topk, m->dim, out, routed, (cudaStream_t)stream);
}

int apus_cuda_moe_ep_plan_dev(const int32_t *idx, int n_rout, int n_experts, int world, int slots,
                              int32_t *send_eids, int32_t *slot_of, void *stream) {
    if (n_rout <= 0) return 0;
    APUS_REQUIRE(world >= 1 && n_experts % world == 0 && slots >= n_rout && n_rout <= 8192,
                 "moe_ep_plan: %d routings, %d experts over %d ranks, %d slots per rank", n_rout, n_experts, world, slots);
    return ep_plan(idx, n_rout, n_experts / world, world, slots, send_eids, slot_of, (cudaStream_t)stream);
}
int apus_cuda_moe_ep_rows_dev(const float *src, int dim, const int32_t *slot_of, int n_rout, int topk, int gather,
                              float *dst, void *stream) {
    if (n_rout <= 0) return 0;
    APUS_REQUIRE(dim % 4 == 0 && topk >= 1, "moe_ep_rows: dim %d, topk %d", dim, topk);
    return ep_rows(src, dim, slot_of, n_rout, topk, gather, dst, (cudaStream_t)stream);
}

int apus_cuda_moe_forward_dev(ApusCudaMoe *m, const float *x, const int64_t *ids, int s, float *out,
                              void *stream) {
    if (!m) { set_error("NULL moe handle"); return 1; }
    if (s <= 0) return 0;
    return forward_run(m, x, ids, m->tid2eid, s, out, nullptr, (cudaStream_t)stream);
}

int apus_cuda_moe_last_routing(ApusCudaMoe *m, int s, int32_t *idx, float *wgt, void *stream) {
    if (!m || s > m->cap_s) { set_error("last_routing: no routing of %d tokens recorded", s); return 1; }
    cudaStream_t st = (cudaStream_t)stream;
    APUS_CUDA_OK(cudaMemcpyAsync(idx, m->b_idx.p, (size_t)s * m->topk * 4, cudaMemcpyDeviceToHost, st));
    APUS_CUDA_OK(cudaMemcpyAsync(wgt, m->b_wgt.p, (size_t)s * m->topk * 4, cudaMemcpyDeviceToHost, st));
    APUS_CUDA_OK(cudaStreamSynchronize(st));
    return 0;
}

// ---- host-pointer tier ----------------------------------------------------------------------------
static ApusCudaMoe *moe_for(const ApusMoeW *w) { return apus_cuda_moe_get(w); }

int apus_cuda_router_score(const ApusMoeW *w, const float *x, int s, float *sp, float *biased) {
    if (ensure_enabled()) return 1;
    if (s <= 0) return 0;
    Ctx &c = ctx();
    const float *gw = (const float *)cached_dense(w->gate_w, (size_t)w->E * w->dim * 4);
    if (!gw) return 1;
    void *dx, *dl, *dsp, *db, *dbias, *didx, *dwgt;
    const size_t se = (size_t)s * w->E * 4;
    if (c.ws[0].get((size_t)s * w->dim * 4, &dx) || c.ws[1].get(se, &dl) || c.ws[2].get(se, &dsp) ||
        c.ws[3].get(se, &db) || c.ws[4].get((size_t)w->E * 4, &dbias) ||
        c.ws[5].get((size_t)s * w->topk * 4, &didx) || c.ws[6].get((size_t)s * w->topk * 4, &dwgt))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dx, x, (size_t)s * w->dim * 4, cudaMemcpyHostToDevice, c.stream));
    if (f32_linear(gw, (float *)dx, (float *)dl, s, w->dim, w->E, APUS_LIN_CLASS(APUS_CUDA_TREE_ROUTER), c.stream)) return 1;
    // scores only: run the finish kernel with a zero bias when none is wanted
    if (biased && w->gate_bias)
        APUS_CUDA_OK(cudaMemcpyAsync(dbias, w->gate_bias, (size_t)w->E * 4, cudaMemcpyHostToDevice, c.stream));
    else
        APUS_CUDA_OK(cudaMemsetAsync(dbias, 0, (size_t)w->E * 4, c.stream));
    if (router_finish((float *)dl, (float *)dbias, nullptr, nullptr, s, w->E, w->topk, w->route_scale,
                      (float *)dsp, (float *)db, (int32_t *)didx, (float *)dwgt, c.stream))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(sp, dsp, se, cudaMemcpyDeviceToHost, c.stream));
    if (biased) APUS_CUDA_OK(cudaMemcpyAsync(biased, db, se, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

int apus_cuda_moe_forward(const ApusMoeW *w, const float *x, const int64_t *ids, int s, float *out,
                          ApusMoeInterm *interm) {
    if (ensure_enabled()) return 1;
    if (s <= 0) return 0;
    Ctx &c = ctx();
    ApusCudaMoe *m = moe_for(w);
    if (!m) return 1;
    const int R = s * m->topk;
    if (m->ensure(s, R)) return 1;
    void *dx, *dout, *drouted;
    if (c.ws[0].get((size_t)s * m->dim * 4, &dx) || c.ws[3].get((size_t)s * m->dim * 4, &dout) ||
        c.ws[4].get((size_t)s * m->dim * 4, &drouted))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dx, x, (size_t)s * m->dim * 4, cudaMemcpyHostToDevice, c.stream));
    const int64_t *d_ids = nullptr, *d_tab = nullptr;
    if (m->hash) {
        // compact lookup table: row t holds tid2eid[ids[t]] (c/moe.h:391-394)
        APUS_REQUIRE(w->tid2eid && ids, "hash-routed layer needs tid2eid and ids");
        std::vector<int64_t> tab((size_t)R), iota((size_t)s);
        for (int t = 0; t < s; t++) {
            iota[t] = t;
            for (int j = 0; j < m->topk; j++) tab[(size_t)t * m->topk + j] = w->tid2eid[ids[t] * m->topk + j];
        }
        APUS_CUDA_OK(cudaMemcpyAsync(m->b_ids.p, iota.data(), (size_t)s * 8, cudaMemcpyHostToDevice, c.stream));
        APUS_CUDA_OK(cudaMemcpyAsync(m->b_tab.p, tab.data(), (size_t)R * 8, cudaMemcpyHostToDevice, c.stream));
        APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
        d_ids = m->b_ids.as<int64_t>(); d_tab = m->b_tab.as<int64_t>();
    }
    if (forward_run(m, (float *)dx, d_ids, d_tab, s, (float *)dout, (float *)drouted, c.stream)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(out, dout, (size_t)s * m->dim * 4, cudaMemcpyDeviceToHost, c.stream));
    if (interm) {
        const size_t se = (size_t)s * m->E * 4, sd = (size_t)s * m->dim * 4, sk = (size_t)s * m->topk * 4;
        if (interm->router_scores) APUS_CUDA_OK(cudaMemcpyAsync(interm->router_scores, m->b_sp.p, se, cudaMemcpyDeviceToHost, c.stream));
        if (interm->router_scores_biased && !m->hash) APUS_CUDA_OK(cudaMemcpyAsync(interm->router_scores_biased, m->b_biased.p, se, cudaMemcpyDeviceToHost, c.stream));
        if (interm->router_w) APUS_CUDA_OK(cudaMemcpyAsync(interm->router_w, m->b_wgt.p, sk, cudaMemcpyDeviceToHost, c.stream));
        if (interm->router_idx) APUS_CUDA_OK(cudaMemcpyAsync(interm->router_idx, m->b_idx.p, sk, cudaMemcpyDeviceToHost, c.stream));
        if (interm->moe_routed) APUS_CUDA_OK(cudaMemcpyAsync(interm->moe_routed, drouted, sd, cudaMemcpyDeviceToHost, c.stream));
        if (interm->moe_shared) APUS_CUDA_OK(cudaMemcpyAsync(interm->moe_shared, m->b_shared.p, sd, cudaMemcpyDeviceToHost, c.stream));
    }
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    if (m->use_tc) {
        int stt = gemm_tc_status(1);
        APUS_REQUIRE(stt == 0, "moe_forward: a bounded wait expired inside the tcgen05 kernel (code %d)", stt);
    }
    return 0;
}

int apus_cuda_kernel_status(int reset) { return gemm_tc_status(reset); }

}  // extern "C"
