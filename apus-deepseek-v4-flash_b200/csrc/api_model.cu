// C ABI, part 4: block wiring and the device-resident token loop
// (include/apus_b200.h; reference c/layer.h:495-545, c/model.h:651-720,
// c/apus.c:895-944).
//
// ApusCudaModel keeps every weight and the state of `batch` sequences in HBM.
// One decode step of all sequences (they advance in lockstep) is a fixed
// sequence of kernel launches: embed x hc -> per layer [mHC pre + RMSNorm,
// attention, mHC post, mHC pre + RMSNorm, MoE, mHC post] -> mHC head ->
// RMSNorm -> LM-head GEMV -> greedy argmax, whose token feeds the next step on
// the device.  Nothing is read back until the caller asks for logits or
// tokens.  A prompt is consumed as consecutive steps; the reference defines
// its batched prefill to be equal to that (tests/m4c chunk invariance).
#include <math.h>
#include <string>
#include <vector>

#include "attn_engine.cuh"
#include "ckpt.cuh"

using namespace apus;

namespace {

struct LayerDev {
    AttnDev attn;
    ApusCudaMoe *moe = nullptr;
    const float *attn_norm_w, *ffn_norm_w;
    const float *hc_attn_fn, *hc_attn_base, *hc_attn_scale, *hc_ffn_fn, *hc_ffn_base, *hc_ffn_scale;
    const float *cs = nullptr;        // device rope rows [rope_rows][cos(half) | sin(half)]
    int rope_rows = 0;
};

struct BlockBufs {
    float *x, *y, *sub, *post, *comb, *raw;   // raw: mHC scratch of the owner (NULL: the library's)
};

// One token of B sequences through one block (reference c/layer.h:495-545), in
// three pieces so that an expert-parallel caller can run the MoE sublayer
// itself between the second and the third.
int block_attn_half(const LayerDev &L, StateDev &S, float **h, float **hn, int B, long long pos, int hc,
                    int iters, float hc_eps, float norm_eps, const BlockBufs &bb, const StepBufs &sb,
                    cudaStream_t st, const long long *pos_dev = nullptr) {
    const int dim = L.attn.cfg.dim, half2 = L.attn.cfg.rope_dim, ratio = L.attn.cfg.ratio;
    APUS_REQUIRE(pos < L.rope_rows, "position %lld is beyond the rope table (%d rows)", pos, L.rope_rows);
    const float *cs_pos = L.cs + (size_t)pos * half2;
    const long long rp = ratio ? pos + 1 - ratio : -1;
    const float *cs_rp = rp >= 0 ? L.cs + (size_t)rp * half2 : cs_pos;
    int x_codes = 0;                            // the mHC step leaves the codes of the sublayer input where it can
    if (mhc_pre(*h, dim, hc, L.hc_attn_fn, L.hc_attn_scale, L.hc_attn_base, norm_eps, hc_eps, iters,
                L.attn_norm_w, norm_eps, nullptr, bb.post, bb.comb, bb.y, bb.x, B, st, bb.raw, sb.xq, sb.xs, &x_codes))
        return 1;
    if (attn_step(L.attn, S, bb.x, pos, cs_pos, cs_rp, bb.sub, sb, nullptr, st, pos_dev, L.cs, x_codes != 0)) return 1;
    if (mhc_post(bb.sub, *h, bb.post, bb.comb, *hn, dim, hc, B, st)) return 1;
    { float *t = *h; *h = *hn; *hn = t; }
    return 0;
}
// mHC pre + RMSNorm of the ffn half: leaves the sublayer input in bb.x
int block_ffn_pre(const LayerDev &L, float *h, int B, int hc, int iters, float hc_eps, float norm_eps,
                  const BlockBufs &bb, cudaStream_t st) {
    return mhc_pre(h, L.attn.cfg.dim, hc, L.hc_ffn_fn, L.hc_ffn_scale, L.hc_ffn_base, norm_eps, hc_eps, iters,
                   L.ffn_norm_w, norm_eps, nullptr, bb.post, bb.comb, bb.y, bb.x, B, st, bb.raw);
}
int block_ffn_post(const LayerDev &L, const float *sub, float **h, float **hn, int B, int hc, const BlockBufs &bb,
                   cudaStream_t st) {
    if (mhc_post(sub, *h, bb.post, bb.comb, *hn, L.attn.cfg.dim, hc, B, st)) return 1;
    { float *t = *h; *h = *hn; *hn = t; }
    return 0;
}
int block_step(const LayerDev &L, StateDev &S, float **h, float **hn, const int64_t *ids, int B, long long pos,
               int hc, int iters, float hc_eps, float norm_eps, const BlockBufs &bb, const StepBufs &sb,
               cudaStream_t st, const long long *pos_dev = nullptr) {
    if (block_attn_half(L, S, h, hn, B, pos, hc, iters, hc_eps, norm_eps, bb, sb, st, pos_dev)) return 1;
    if (block_ffn_pre(L, *h, B, hc, iters, hc_eps, norm_eps, bb, st)) return 1;
    if (apus_cuda_moe_forward_dev(L.moe, bb.x, ids, B, bb.sub, st)) return 1;
    return block_ffn_post(L, bb.sub, h, hn, B, hc, bb, st);
}

// A chunk of s positions of B sequences through one block: the same pieces on s * B time-major rows.
int block_chunk(const LayerDev &L, StateDev &S, float **h, float **hn, const int64_t *ids, int B, int s, long long pos0,
                int hc, int iters, float hc_eps, float norm_eps, const BlockBufs &bb, const StepBufs &sb, cudaStream_t st) {
    const int dim = L.attn.cfg.dim, T = B * s;
    APUS_REQUIRE(pos0 + s <= L.rope_rows, "position %lld is beyond the rope table (%d rows)", pos0 + s - 1, L.rope_rows);
    if (mhc_pre(*h, dim, hc, L.hc_attn_fn, L.hc_attn_scale, L.hc_attn_base, norm_eps, hc_eps, iters, L.attn_norm_w,
                norm_eps, nullptr, bb.post, bb.comb, bb.y, bb.x, T, st, bb.raw))
        return 1;
    if (attn_chunk(L.attn, S, bb.x, pos0, s, L.cs, bb.sub, sb, st)) return 1;
    if (block_ffn_post(L, bb.sub, h, hn, T, hc, bb, st)) return 1;               // mHC post of the attention half
    if (block_ffn_pre(L, *h, T, hc, iters, hc_eps, norm_eps, bb, st)) return 1;
    if (apus_cuda_moe_forward_dev(L.moe, bb.x, ids, T, bb.sub, st)) return 1;
    return block_ffn_post(L, bb.sub, h, hn, T, hc, bb, st);
}

// own == NULL: weights of the global cache (host-pointer tier); otherwise they
// belong to `own` and the MoE object to the caller.
int layer_weights(const ApusCudaLayerDesc &d, int hc, int vocab, LayerDev *L, WeightOwner *own, int e_lo = 0,
                  int e_hi = -1) {
    const int dim = d.acfg.dim;
    const size_t nmix = (size_t)(2 + hc) * hc, nx = (size_t)hc * dim;
    if (attn_weights(&d.acfg, &d.aw, &L->attn, own)) return 1;
    L->moe = own ? apus_cuda_moe_create(&d.mw, e_lo, e_hi < 0 ? d.mw.E : e_hi) : apus_cuda_moe_get(&d.mw);
    if (!L->moe) return 1;
    if (d.mw.hash && vocab < (1 << 30) && apus_cuda_moe_set_hash_table(L->moe, d.mw.tid2eid, vocab)) return 1;
    L->attn_norm_w = (const float *)get_dense(own, d.attn_norm_w, (size_t)dim * 4);
    L->ffn_norm_w = (const float *)get_dense(own, d.ffn_norm_w, (size_t)dim * 4);
    L->hc_attn_fn = (const float *)get_dense(own, d.hc_attn_fn, nmix * nx * 4);
    L->hc_attn_base = (const float *)get_dense(own, d.hc_attn_base, nmix * 4);
    L->hc_attn_scale = (const float *)get_dense(own, d.hc_attn_scale, 3 * 4);
    L->hc_ffn_fn = (const float *)get_dense(own, d.hc_ffn_fn, nmix * nx * 4);
    L->hc_ffn_base = (const float *)get_dense(own, d.hc_ffn_base, nmix * 4);
    L->hc_ffn_scale = (const float *)get_dense(own, d.hc_ffn_scale, 3 * 4);
    if (!L->attn_norm_w || !L->ffn_norm_w || !L->hc_attn_fn || !L->hc_attn_base || !L->hc_attn_scale ||
        !L->hc_ffn_fn || !L->hc_ffn_base || !L->hc_ffn_scale)
        return 1;
    return 0;
}

// rope rows as [cos(half) | sin(half)] per position, cached by the host cos pointer
std::map<const void *, DevBuf *> g_rope;
const float *rope_rows_dev(const float *cos, const float *sin, int rows, int half,
                           std::map<const void *, DevBuf *> &cache = g_rope) {
    auto it = cache.find(cos);
    if (it != cache.end() && it->second->cap >= (size_t)rows * 2 * half * 4) return it->second->as<float>();
    std::vector<float> cs((size_t)rows * 2 * half);
    for (int t = 0; t < rows; t++) {
        memcpy(&cs[(size_t)t * 2 * half], cos + (size_t)t * half, half * 4);
        memcpy(&cs[(size_t)t * 2 * half + half], sin + (size_t)t * half, half * 4);
    }
    DevBuf *b = it != cache.end() ? it->second : new DevBuf();
    if (b->get(cs.size() * 4, nullptr)) return nullptr;
    if (cudaMemcpy(b->p, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
    cache[cos] = b;
    return b->as<float>();
}

StateDev g_block_state;
DevBuf g_block_ws[24], g_block_hb[10];

void model_release_all() {
    for (auto &kv : g_rope) { kv.second->release(); delete kv.second; }
    g_rope.clear();
    g_block_state.release();
    for (auto &b : g_block_ws) b.release();
    for (auto &b : g_block_hb) b.release();
}
void model_forget(const void *host) {
    auto it = g_rope.find(host);
    if (it == g_rope.end()) return;
    cudaDeviceSynchronize();
    it->second->release();
    delete it->second;
    g_rope.erase(it);
}
struct ModelReg { ModelReg() { apus::on_disable(model_release_all, model_forget); } } g_model_reg;

__global__ void next_ids_kernel(const int32_t *tok, int64_t *ids, int32_t *hist, int B, int step, int n_steps) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) {
        ids[b] = tok[b];
        if (hist) hist[(size_t)b * n_steps + step] = tok[b];
    }
}

}  // namespace

struct ApusCudaModel {
    int n_layers = 0, dim = 0, hc = 0, iters = 0, vocab = 0, B = 0, max_pos = 0, n_experts = 0;
    long long max_nb = 8;                  // most compressed entries any layer can hold
    float hc_eps = 0.f, norm_eps = 0.f, hc_head_scale = 0.f;
    std::vector<LayerDev> layers;
    std::vector<StateDev> states;
    const void *embed = nullptr, *head = nullptr;
    int embed_bf16 = 0, head_bf16 = 0;
    const float *norm_w = nullptr, *hc_head_fn = nullptr, *hc_head_base = nullptr;
    long long pos = 0;
    // the stream this model's work is enqueued on: the library stream unless the model was
    // given one of its own (models that step side by side, apus_cuda_model_set_stream)
    cudaStream_t stream = nullptr, own_stream = nullptr;
    int e_lo = 0, e_hi = 0;                // routed experts resident here (expert parallelism)
    float *h_cur = nullptr, *h_alt = nullptr;   // hidden state between the pieces of a step
    // the position also lives on the device: the kernels of a step read it there, so
    // a step is the same launch sequence at every position and is replayed from a
    // CUDA graph (one with the head, one without) after the first step ran eagerly
    DevBuf pos_dev;
    cudaGraphExec_t gexec[2] = {nullptr, nullptr};
    unsigned long long graph_epoch = 0;    // sum_order_epoch() the recorded steps were captured under
    // sampling (temp <= 0: greedy argmax): per-sequence splitmix64 states and the
    // probability scratch live on the device
    float temp = 0.f, top_p = 1.f;
    DevBuf rng, probs;
    bool use_graph = true;
    bool capturing = false;               // the caller is recording a step into its own graph
    long long steps_run = 0;
    WeightOwner own;                       // every weight copy made for this model
    std::map<const void *, DevBuf *> rope; // rope rows by host table (layers of a kind share one)
    DevBuf h0, h1, x, y, sub, post, comb, yh, yn, logits, tok, ids, hist, raw, sa, ws[24];
    StepBufs sb;
    // a chunk of positions in one pass (s > 1 calls): the same buffers for positions x sequences rows,
    // allocated by the first such call
    struct Chunk {
        int rows = 0, s = 0;
        DevBuf h0, h1, x, y, sub, post, comb, raw, sa, ext, logits, tok, hx, mhx, ws[24];
        StepBufs sb;
        void release() {
            DevBuf *b[] = {&h0, &h1, &x, &y, &sub, &post, &comb, &raw, &sa, &ext, &logits, &tok, &hx, &mhx};
            for (DevBuf *p : b) p->release();
            for (auto &w : ws) w.release();
            rows = s = 0;
        }
    } ck;
};

// What a rollback needs (reference c/mtp.h:113-138, 398-439): per layer the ring, the
// compressor carries and the entry counts -- cache entries past a restored count are
// dead capacity, so rollback is a copy plus truncation -- and the position; here also
// the device-side position, the fed-back token and the sampler streams.
struct ApusCudaSnap {
    struct Layer { DevBuf win, ckv, csc, ikv, isc; int comp_nb = 0, idx_nb = 0; };
    std::vector<Layer> layers;
    int B = 0;
    long long pos = 0;
    DevBuf pos_dev, tok, ids, rng;
    bool has_rng = false;
};

static inline cudaStream_t mstream(const ApusCudaModel *m) { return m->stream ? m->stream : ctx().stream; }
static BlockBufs model_bufs(ApusCudaModel *m) {
    return {m->x.as<float>(), m->y.as<float>(), m->sub.as<float>(), m->post.as<float>(), m->comb.as<float>(),
            m->raw.as<float>()};
}
static int model_embed(ApusCudaModel *m, cudaStream_t st) {
    m->h_cur = m->h0.as<float>(); m->h_alt = m->h1.as<float>();
    return embed_rows(m->embed, m->embed_bf16, m->ids.as<int64_t>(), m->B, m->hc, m->dim, m->h_cur, st);
}
static int head_rows(ApusCudaModel *m, const float *h, int rows, float *yh, float *yn, float *logits, int32_t *tok,
                     cudaStream_t st);
// head of one position (reference c/model.h:706-718) and the pick
static int model_head(ApusCudaModel *m, cudaStream_t st) {
    return head_rows(m, m->h_cur, m->B, m->yh.as<float>(), m->yn.as<float>(), m->logits.as<float>(), m->tok.as<int32_t>(), st);
}
__global__ void advance_pos_kernel(long long *pos) {
    APUS_PDL_WAIT();
    APUS_PDL_GO(); *pos += 1; }

// host mirror of what a step does to the sequence state: entry counts follow the position
static int model_host_advance(ApusCudaModel *m) {
    for (int i = 0; i < m->n_layers; i++) {
        const ApusAttnCfg &c = m->layers[i].attn.cfg;
        if (c.ratio && (m->pos + 1) % c.ratio == 0) {
            m->states[i].comp.nb++;
            if (c.has_indexer) m->states[i].idx.nb++;
        }
    }
    m->pos++;
    m->steps_run++;
    return 0;
}

// every launch of one position of all sequences, position read on the device
static int model_step_enqueue(ApusCudaModel *m, bool want_logits, cudaStream_t st) {
    if (model_embed(m, st)) return 1;
    BlockBufs bb = model_bufs(m);
    const long long *pd = m->pos_dev.as<long long>();
    for (int i = 0; i < m->n_layers; i++)
        if (block_step(m->layers[i], m->states[i], &m->h_cur, &m->h_alt, m->ids.as<int64_t>(), m->B, m->pos, m->hc,
                       m->iters, m->hc_eps, m->norm_eps, bb, m->sb, st, pd))
            return 1;
    if (want_logits && model_head(m, st)) return 1;
    launch_k(advance_pos_kernel, 1, 1, 0, st, m->pos_dev.as<long long>());
    APUS_LAUNCHED();
    return 0;
}

int apus_cuda_moe_timing_enabled(const ApusCudaMoe *m);      // api_moe.cu
static bool model_timing_on(ApusCudaModel *m) {
    for (auto &L : m->layers) if (L.moe && apus_cuda_moe_timing_enabled(L.moe)) return true;
    return false;
}

static int model_step(ApusCudaModel *m, bool want_logits, cudaStream_t st) {
    APUS_REQUIRE(m->e_lo == 0 && m->e_hi == m->n_experts,
                 "this model holds experts [%d,%d) of %d: drive it layer by layer (apus_cuda_model_attn_half ...)",
                 m->e_lo, m->e_hi, m->n_experts);
    APUS_REQUIRE(m->pos < m->max_pos, "model step: position %lld reaches max_pos %d", m->pos, m->max_pos);
    for (int i = 0; i < m->n_layers; i++) {
        const ApusAttnCfg &c = m->layers[i].attn.cfg;
        if (c.ratio && (m->pos + 1) % c.ratio == 0)
            APUS_REQUIRE(m->states[i].comp.nb < m->states[i].comp.cap, "layer %d: compressed cache is full", i);
    }
    const int gi = want_logits ? 1 : 0;
    if (m->graph_epoch != sum_order_epoch()) {            // the sum order picks the kernels: record again
        for (int i = 0; i < 2; i++)
            if (m->gexec[i]) { cudaGraphExecDestroy(m->gexec[i]); m->gexec[i] = nullptr; }
        m->graph_epoch = sum_order_epoch();
    }
    if (m->use_graph && m->steps_run >= 1 && !model_timing_on(m)) {
        if (!m->gexec[gi]) {
            // capture the launches of one step; nothing in here allocates or synchronises
            // because the first step already ran eagerly with the same shapes
            cudaGraph_t graph = nullptr;
            bool ok = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
            const int rc = ok ? model_step_enqueue(m, want_logits, st) : 1;
            if (ok) ok = cudaStreamEndCapture(st, &graph) == cudaSuccess && rc == 0 && graph;
            if (ok) ok = cudaGraphInstantiate(&m->gexec[gi], graph, 0) == cudaSuccess;
            if (graph) cudaGraphDestroy(graph);
            if (!ok) {                         // fall back to plain launches for good
                cudaGetLastError();
                m->gexec[gi] = nullptr;
                m->use_graph = false;
            }
        }
        if (m->gexec[gi]) {
            APUS_CUDA_OK(cudaGraphLaunch(m->gexec[gi], st));
            g_dispatches++;
            return model_host_advance(m);
        }
    }
    if (model_step_enqueue(m, want_logits, st)) return 1;
    return model_host_advance(m);
}

// ---- a chunk of positions in one pass (reference c/model.h:651-720 with s > 1) ---------------------
// Rows are time-major (row = t * B + sequence).  Every operator of a step is row-wise except the
// attention state, which attn_chunk walks in position order, so a chunk leaves the hidden states,
// the state and the logits of s consecutive steps, bit for bit; what it saves is reading every
// weight once per chunk instead of once per position.
__global__ void advance_pos_by_kernel(long long *pos, int by) {
    APUS_PDL_WAIT();
    APUS_PDL_GO(); *pos += by; }

static int model_chunk_bufs(ApusCudaModel *m, int s) {
    ApusCudaModel::Chunk &C = m->ck;
    const size_t T = (size_t)m->B * s, dim = m->dim, hc = m->hc;
    if ((int)T <= C.rows && s <= C.s) return 0;
    const int rows = (int)T > C.rows ? (int)T : C.rows, sc = s > C.s ? s : C.s;
    const size_t R = rows;
    if (C.h0.get(R * hc * dim * 4, nullptr) || C.h1.get(R * hc * dim * 4, nullptr) || C.x.get(R * dim * 4, nullptr) ||
        C.y.get(R * dim * 4, nullptr) || C.sub.get(R * dim * 4, nullptr) || C.post.get(R * hc * 4, nullptr) ||
        C.comb.get(R * hc * hc * 4, nullptr) || C.raw.get(R * ((2 + hc) * hc + 1) * 4, nullptr))
        return 1;
    ApusAttnCfg widest = m->layers[0].attn.cfg;
    size_t ext = 0;
    for (int i = 0; i < m->n_layers; i++) {
        const ApusAttnCfg &c = m->layers[i].attn.cfg;
        if (c.has_indexer) { widest.idx_heads = c.idx_heads; widest.idx_dim = c.idx_dim; widest.idx_topk = c.idx_topk; }
        const size_t e = (size_t)m->B * (c.window + sc) * c.head_dim * 4;
        if (e > ext) ext = e;
    }
    widest.has_indexer = 0;                      // size the index row for the dense (largest) case
    const long long wide_nb = m->max_nb > widest.idx_topk ? m->max_nb : widest.idx_topk;
    if (attn_step_bufs(widest, wide_nb, rows, C.ws, &C.sb)) return 1;
    C.sb.sa_cap = sparse_attn_scratch(widest.n_heads, (int)(widest.window + wide_nb + 8), rows);
    if (C.sa.get(C.sb.sa_cap, &C.sb.sa)) return 1;
    if (C.ext.get(ext, nullptr)) return 1;
    C.sb.ext = C.ext.as<float>();
    C.rows = rows; C.s = sc;
    return 0;
}

// What a chunk may leave besides the state (device pointers, time-major rows, all nullable):
//   logits_all / tok_all: the head and the pick of EVERY row (c/model.h:706-718 with logits_all)
//   h_all: the hidden state after the last block, [rows][hc * dim] (c/model.h:694-696, the MTP input)
//   mh_all: after each layer listed in `targets`, the mean over the hc streams of every row, BF16,
//           [rows][n_targets * dim] (c/model.h:676-693, the DSpark input)
struct ChunkExtra {
    float *logits_all = nullptr;
    int32_t *tok_all = nullptr;
    float *h_all = nullptr;
    float *mh_all = nullptr;
    const int *targets = nullptr;
    int n_targets = 0;
};

// mean over the hc streams in stream order, one accumulator, then BF16 (c/model.h:684-690)
__global__ void hc_mean_kernel(const float *__restrict__ h, int hc, int dim, float *__restrict__ out, int out_ld) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int r = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dim) return;
    float acc = 0.f;
    for (int j = 0; j < hc; j++) acc = __fadd_rn(acc, h[((size_t)r * hc + j) * dim + i]);
    out[(size_t)r * out_ld + i] = bf16_round(__fdiv_rn(acc, (float)hc));
}

// head: hc_head collapse -> BF16 -> RMSNorm -> LM-head GEMV -> pick, on `rows` rows of hidden states;
// a sampled pick draws one uniform per sequence and position, in position order (c/sample.h:173-178)
static int head_rows(ApusCudaModel *m, const float *h, int rows, float *yh, float *yn, float *logits, int32_t *tok,
                     cudaStream_t st) {
    const int dim = m->dim, B = m->B;
    if (mhc_head(h, dim, m->hc, m->hc_head_fn, m->hc_head_scale, m->hc_head_base, m->norm_eps, m->hc_eps, yh, rows, st,
                 rows <= B ? m->raw.as<float>() : m->ck.raw.as<float>()))
        return 1;
    if (rms_norm(yh, m->norm_w, m->norm_eps, yn, dim, rows, st)) return 1;
    if (f32_linear(m->head, yn, logits, rows, dim, m->vocab,
                   (m->head_bf16 ? APUS_CUDA_W_BF16 : 0) | APUS_LIN_CLASS(APUS_CUDA_TREE_HEAD), st))
        return 1;
    if (!tok) return 0;
    if (m->temp > 0.f) {
        for (int t = 0; t < rows / B; t++)
            if (sample_rows(logits + (size_t)t * B * m->vocab, m->vocab, B, m->temp, m->top_p, nullptr,
                            m->rng.as<unsigned long long>(), m->probs.as<float>(), tok + (size_t)t * B, st))
                return 1;
        return 0;
    }
    return argmax_rows(logits, m->vocab, rows, tok, st);
}

// ids_tm: device, [s][B].  want_head: the head and the pick run on the last position's rows.
static int model_chunk(ApusCudaModel *m, const int64_t *ids_tm, int s, bool want_head, cudaStream_t st,
                       const ChunkExtra *ex = nullptr) {
    APUS_REQUIRE(m->e_lo == 0 && m->e_hi == m->n_experts,
                 "this model holds experts [%d,%d) of %d: drive it layer by layer (apus_cuda_model_attn_half ...)",
                 m->e_lo, m->e_hi, m->n_experts);
    APUS_REQUIRE(m->pos + s <= m->max_pos, "model chunk: position %lld + %d exceeds max_pos %d", m->pos, s, m->max_pos);
    if (model_chunk_bufs(m, s)) return 1;
    ApusCudaModel::Chunk &C = m->ck;
    const int T = m->B * s, dim = m->dim, hc = m->hc;
    float *h = C.h0.as<float>(), *hn = C.h1.as<float>();
    const BlockBufs bb = {C.x.as<float>(), C.y.as<float>(), C.sub.as<float>(), C.post.as<float>(), C.comb.as<float>(),
                          C.raw.as<float>()};
    if (embed_rows(m->embed, m->embed_bf16, ids_tm, T, hc, dim, h, st)) return 1;
    for (int i = 0; i < m->n_layers; i++) {
        if (block_chunk(m->layers[i], m->states[i], &h, &hn, ids_tm, m->B, s, m->pos, hc, m->iters, m->hc_eps, m->norm_eps,
                        bb, C.sb, st))
            return 1;
        if (ex && ex->mh_all)
            for (int tg = 0; tg < ex->n_targets; tg++)
                if (ex->targets[tg] == i) {
                    launch_k(hc_mean_kernel, dim3(ceil_div(dim, 256), T), 256, 0, st, h, hc, dim, ex->mh_all + (size_t)tg * dim,
                                                                               ex->n_targets * dim);
                    APUS_LAUNCHED();
                }
    }
    if (ex && ex->h_all)
        APUS_CUDA_OK(cudaMemcpyAsync(ex->h_all, h, (size_t)T * hc * dim * 4, cudaMemcpyDeviceToDevice, st));
    if (ex && ex->logits_all) {
        // x and y of the chunk are free by now: they hold the collapsed and the normed rows
        if (head_rows(m, h, T, bb.x, bb.y, ex->logits_all, ex->tok_all, st)) return 1;
        // the last position's rows are also what a plain call leaves in the model's own buffers
        const size_t last = (size_t)(s - 1) * m->B;
        APUS_CUDA_OK(cudaMemcpyAsync(m->logits.p, ex->logits_all + last * m->vocab, (size_t)m->B * m->vocab * 4,
                                     cudaMemcpyDeviceToDevice, st));
        if (ex->tok_all)
            APUS_CUDA_OK(cudaMemcpyAsync(m->tok.p, ex->tok_all + last, (size_t)m->B * 4, cudaMemcpyDeviceToDevice, st));
    } else if (want_head) {
        m->h_cur = h + (size_t)(s - 1) * m->B * hc * dim;
        if (model_head(m, st)) return 1;
    }
    m->h_cur = m->h0.as<float>(); m->h_alt = m->h1.as<float>();
    launch_k(advance_pos_by_kernel, 1, 1, 0, st, m->pos_dev.as<long long>(), s);
    APUS_LAUNCHED();
    m->pos += s;                                  // the entry counts were advanced by attn_chunk
    return 0;
}

// s positions from device ids [s][B]: chunks of at most chunk_rows() rows, or one step per position
static int model_consume(ApusCudaModel *m, const int64_t *ids_tm, int s, bool want_head, cudaStream_t st) {
    const int per = chunks_enabled() && s > 1 && m->e_lo == 0 && m->e_hi == m->n_experts ? chunk_rows() / m->B : 0;
    if (per < 2) {
        for (int t = 0; t < s; t++) {
            APUS_CUDA_OK(cudaMemcpyAsync(m->ids.p, ids_tm + (size_t)t * m->B, (size_t)m->B * 8, cudaMemcpyDeviceToDevice, st));
            if (model_step(m, want_head && t == s - 1, st)) return 1;
        }
        return 0;
    }
    for (int t = 0; t < s; t += per) {
        const int n = s - t < per ? s - t : per;
        if (model_chunk(m, ids_tm + (size_t)t * m->B, n, want_head && t + n == s, st)) return 1;
    }
    return 0;
}

extern "C" {

void apus_cuda_model_destroy(ApusCudaModel *m) {
    if (!m) return;
    cudaDeviceSynchronize();
    for (auto &s : m->states) s.release();
    for (int i = 0; i < 2; i++) if (m->gexec[i]) cudaGraphExecDestroy(m->gexec[i]);
    if (m->own_stream) cudaStreamDestroy(m->own_stream);
    m->pos_dev.release();
    m->rng.release(); m->probs.release();
    for (auto &L : m->layers) if (L.moe) apus_cuda_moe_destroy(L.moe);
    m->own.release();
    for (auto &kv : m->rope) { kv.second->release(); delete kv.second; }
    DevBuf *bufs[] = {&m->h0, &m->h1, &m->x, &m->y, &m->sub, &m->post, &m->comb, &m->yh, &m->yn, &m->logits,
                      &m->tok, &m->ids, &m->hist, &m->raw, &m->sa};
    for (DevBuf *b : bufs) b->release();
    for (auto &b : m->ws) b.release();
    m->ck.release();
    delete m;
}

int apus_cuda_model_reset(ApusCudaModel *m) {
    if (!m) { set_error("NULL model"); return 1; }
    for (int i = 0; i < m->n_layers; i++) {
        const ApusAttnCfg &c = m->layers[i].attn.cfg;
        const int cap = c.ratio ? m->max_pos / c.ratio + 2 : 0;
        if (attn_state_init(c, m->states[i], m->B, cap)) return 1;
    }
    if (m->pos_dev.get(256, nullptr)) return 1;
    APUS_CUDA_OK(cudaMemsetAsync(m->pos_dev.p, 0, 256, mstream(m)));
    APUS_CUDA_OK(cudaStreamSynchronize(ctx().stream));   // the state was cleared on the library stream
    APUS_CUDA_OK(cudaStreamSynchronize(mstream(m)));
    m->pos = 0;
    return 0;
}

ApusCudaModel *apus_cuda_model_create(const ApusCudaModelDesc *d, int batch, int max_pos) {
    return apus_cuda_model_create_ep(d, batch, max_pos, 0, -1);
}

// A model is put together in three steps so that a loader can hand over one layer
// at a time (its host copy is no longer needed once model_add_layer returned:
// uploads are synchronous): sizes, the layers in order, the top-level tensors.
static ApusCudaModel *model_begin(const ApusCudaModelDesc &d, int E, int batch, int max_pos, int e_lo, int e_hi) {
    if (ensure_enabled()) return nullptr;
    if (batch < 1 || batch > 32 || d.n_layers < 1) { set_error("model_create: bad arguments (batch 1..32)"); return nullptr; }
    if (e_hi < 0) e_hi = E;
    if (e_lo < 0 || e_lo > e_hi || e_hi > E) { set_error("model_create: bad expert range [%d,%d) of %d", e_lo, e_hi, E); return nullptr; }
    ApusCudaModel *m = new ApusCudaModel();
    m->n_experts = E; m->e_lo = e_lo; m->e_hi = e_hi;
    m->n_layers = d.n_layers; m->dim = d.dim; m->hc = d.hc_mult; m->iters = d.hc_sinkhorn_iters;
    m->vocab = d.vocab; m->B = batch; m->max_pos = max_pos;
    m->hc_eps = d.hc_eps; m->norm_eps = d.norm_eps; m->hc_head_scale = d.hc_head_scale;
    m->layers.resize(d.n_layers);
    m->states.resize(d.n_layers);
    return m;
}

static int model_add_layer(ApusCudaModel *m, int i, const ApusCudaLayerDesc &ld) {
    if (layer_weights(ld, m->hc, m->vocab, &m->layers[i], &m->own, m->e_lo, m->e_hi)) return 1;
    const int half = ld.acfg.rope_dim / 2;
    m->layers[i].cs = rope_rows_dev(ld.cos, ld.sin, ld.rope_rows, half, m->rope);
    m->layers[i].rope_rows = ld.rope_rows;
    if (!m->layers[i].cs || ld.rope_rows < m->max_pos) {
        set_error("model_create: layer %d rope table has %d rows, %d needed", i, ld.rope_rows, m->max_pos);
        return 1;
    }
    if (ld.acfg.ratio && m->max_pos / ld.acfg.ratio + 2 > m->max_nb) m->max_nb = m->max_pos / ld.acfg.ratio + 2;
    return 0;
}

static int model_finish(ApusCudaModel *m, const ApusCudaModelDesc &d) {
    const size_t B = m->B, dim = d.dim, hc = d.hc_mult;
    const size_t esz_e = d.embed_bf16 ? 2 : 4, esz_h = d.head_bf16 ? 2 : 4;
    m->embed = get_dense(&m->own, d.embed, (size_t)d.vocab * dim * esz_e);
    m->head = d.head == d.embed && esz_e == esz_h ? m->embed : get_dense(&m->own, d.head, (size_t)d.vocab * dim * esz_h);
    m->embed_bf16 = d.embed_bf16; m->head_bf16 = d.head_bf16;
    m->norm_w = (const float *)get_dense(&m->own, d.norm_w, dim * 4);
    m->hc_head_fn = (const float *)get_dense(&m->own, d.hc_head_fn, hc * hc * dim * 4);
    m->hc_head_base = (const float *)get_dense(&m->own, d.hc_head_base, hc * 4);
    if (!(m->embed && m->head && m->norm_w && m->hc_head_fn && m->hc_head_base)) return 1;
    if (m->h0.get(B * hc * dim * 4, nullptr) || m->h1.get(B * hc * dim * 4, nullptr) ||
        m->x.get(B * dim * 4, nullptr) || m->y.get(B * dim * 4, nullptr) || m->sub.get(B * dim * 4, nullptr) ||
        m->post.get(B * hc * 4, nullptr) || m->comb.get(B * hc * hc * 4, nullptr) ||
        m->yh.get(B * dim * 4, nullptr) || m->yn.get(B * dim * 4, nullptr) ||
        m->logits.get(B * (size_t)d.vocab * 4, nullptr) || m->tok.get(B * 4, nullptr) || m->ids.get(B * 8, nullptr) ||
        m->raw.get(B * ((2 + hc) * hc + 1) * 4, nullptr))
        return 1;
    // step buffers sized for the widest layer configuration
    ApusAttnCfg widest = m->layers[0].attn.cfg;
    for (int i = 1; i < m->n_layers; i++) {
        const ApusAttnCfg &c = m->layers[i].attn.cfg;
        if (c.has_indexer) { widest.has_indexer = 1; widest.idx_heads = c.idx_heads; widest.idx_dim = c.idx_dim; widest.idx_topk = c.idx_topk; }
    }
    widest.has_indexer = 0;                      // size the index row for the dense (largest) case
    const long long wide_nb = m->max_nb > widest.idx_topk ? m->max_nb : widest.idx_topk;
    if (attn_step_bufs(widest, wide_nb, m->B, m->ws, &m->sb)) return 1;
    m->sb.sa_cap = sparse_attn_scratch(widest.n_heads, (int)(widest.window + wide_nb + 8), m->B);
    if (m->sa.get(m->sb.sa_cap, &m->sb.sa)) return 1;
    return apus_cuda_model_reset(m);
}

ApusCudaModel *apus_cuda_model_create_ep(const ApusCudaModelDesc *d, int batch, int max_pos, int e_lo, int e_hi) {
    if (!d || d->n_layers < 1 || !d->layers) { set_error("model_create: bad arguments (batch 1..32)"); return nullptr; }
    ApusCudaModel *m = model_begin(*d, d->layers[0].mw.E, batch, max_pos, e_lo, e_hi);
    if (!m) return nullptr;
    bool ok = true;
    for (int i = 0; i < d->n_layers && ok; i++) ok = model_add_layer(m, i, d->layers[i]) == 0;
    if (ok) ok = model_finish(m, *d) == 0;
    if (!ok) { apus_cuda_model_destroy(m); return nullptr; }
    return m;
}

// c/model.h:396-470 with HBM as the destination: one layer in host memory at a time.
ApusCudaModel *apus_cuda_model_load(const char *dir, int batch, int max_pos, int e_lo, int e_hi) {
    char err[512] = "";
    ApusCudaCkpt *c = apus_cuda_ckpt_open(dir, err, sizeof err);
    if (!c) return nullptr;                           // message already recorded
    const ApusCudaCkptCfg &cfg = c->cfg;
    if (max_pos <= 0 || max_pos > cfg.max_pos) max_pos = cfg.max_pos;
    ApusCudaModelDesc top;
    memset(&top, 0, sizeof top);
    top.n_layers = cfg.n_layers; top.dim = cfg.dim; top.hc_mult = cfg.hc_mult;
    top.hc_sinkhorn_iters = cfg.hc_sinkhorn_iters; top.vocab = cfg.vocab_size;
    top.hc_eps = cfg.hc_eps; top.norm_eps = cfg.norm_eps;
    ApusCudaModel *m = model_begin(top, cfg.n_routed_experts, batch, max_pos, e_lo, e_hi);
    if (!m) { apus_cuda_ckpt_close(c); return nullptr; }
    // one rope table per theta class (c/layer.h:145-166), shared by the layers of the class
    const size_t half = cfg.rope_head_dim / 2;
    std::vector<float> rope[2][2];                    // [class][cos | sin]
    bool ok = true;
    std::string why;
    for (int i = 0; i < cfg.n_layers && ok; i++) {
        CkLayerHost L;
        if (ckpt_load_layer(c, i, m->e_lo, m->e_hi, &L, &why)) { set_error("%s", why.c_str()); ok = false; break; }
        const int cls = c->ratios[i] ? 1 : 0;
        if (rope[cls][0].empty()) {
            rope[cls][0].resize((size_t)max_pos * half); rope[cls][1].resize((size_t)max_pos * half);
            ckpt_rope(cfg, c->ratios[i], max_pos, rope[cls][0].data(), rope[cls][1].data());
        }
        L.desc.cos = rope[cls][0].data(); L.desc.sin = rope[cls][1].data(); L.desc.rope_rows = max_pos;
        L.desc.acfg.max_pos = max_pos;
        ok = model_add_layer(m, i, L.desc) == 0;
    }
    if (ok) {
        // c/model.h:432-467: embed/head [vocab, dim] BF16 or F32, norm, hc_head_*
        const size_t V = cfg.vocab_size, dim = cfg.dim, hc = cfg.hc_mult;
        std::vector<uint8_t> embed, head;
        std::vector<float> norm_w(dim), hfn(hc * hc * dim), hbase(hc);
        auto mat = [&](const char *name, std::vector<uint8_t> *buf, int *bf16) -> bool {
            const CkTensor *t = c->find(name, &why);
            if (!t || (t->dtype != APUS_CUDA_ST_BF16 && t->dtype != APUS_CUDA_ST_F32) || t->ndim != 2 ||
                t->shape[0] != (int64_t)V || t->shape[1] != (int64_t)dim) {
                set_error("model: bad tensor %s", name);
                return false;
            }
            buf->resize(t->nbytes);
            *bf16 = t->dtype == APUS_CUDA_ST_BF16;
            if (c->read(*t, buf->data(), &why)) { set_error("%s", why.c_str()); return false; }
            return true;
        };
        auto vec = [&](const char *name, float *out, size_t n, bool f32_only) -> bool {
            const CkTensor *t = c->find(name, &why);
            if (!t || t->nelem() != n || (f32_only && t->dtype != APUS_CUDA_ST_F32) ||
                apus_cuda_ckpt_read_f32(c, name, out, n)) {
                set_error("model: bad tensor %s", name);
                return false;
            }
            return true;
        };
        ok = mat("embed.weight", &embed, &top.embed_bf16) && mat("head.weight", &head, &top.head_bf16) &&
             vec("norm.weight", norm_w.data(), dim, false) && vec("hc_head_fn", hfn.data(), hc * hc * dim, true) &&
             vec("hc_head_base", hbase.data(), hc, false) && vec("hc_head_scale", &top.hc_head_scale, 1, false);
        if (ok) {
            top.embed = embed.data(); top.head = head.data();
            top.norm_w = norm_w.data(); top.hc_head_fn = hfn.data(); top.hc_head_base = hbase.data();
            m->hc_head_scale = top.hc_head_scale;
            ok = model_finish(m, top) == 0;
        }
    }
    apus_cuda_ckpt_close(c);
    if (!ok) { apus_cuda_model_destroy(m); return nullptr; }
    return m;
}

int apus_cuda_block_forward(const ApusCudaLayerDesc *d, int hc, int iters, float hc_eps, float norm_eps,
                            ApusAttnS *st, float *h, const int64_t *ids, int s, int64_t start_pos) {
    return apus_cuda_block_forward_v(d, hc, iters, hc_eps, norm_eps, st, h, ids, s, start_pos, 0);
}

int apus_cuda_block_forward_v(const ApusCudaLayerDesc *d, int hc, int iters, float hc_eps, float norm_eps,
                              ApusAttnS *st, float *h, const int64_t *ids, int s, int64_t start_pos, int64_t vocab) {
    if (ensure_enabled()) return 1;
    if (s <= 0) return 0;
    cudaStream_t sm = ctx().stream;
    const ApusAttnCfg &c = d->acfg;
    const int dim = c.dim, half = c.rope_dim / 2;
    APUS_REQUIRE(start_pos + s <= d->rope_rows, "block_forward: rope table too short");
    LayerDev L;
    if (d->mw.hash && (vocab <= 0 || !ids)) {
        set_error("block_forward: a hash-routed layer needs the token ids and the vocabulary size "
                  "(apus_cuda_block_forward_v)");
        return 1;
    }
    if (layer_weights(*d, hc, d->mw.hash ? (int)vocab : 1 << 30, &L, nullptr)) return 1;
    L.cs = rope_rows_dev(d->cos, d->sin, d->rope_rows, half);
    L.rope_rows = d->rope_rows;
    if (!L.cs) return 1;
    StateDev &S = g_block_state;
    DevBuf *ws = g_block_ws, *hb = g_block_hb;
    StepBufs sb;
    const long long max_nb = c.ratio ? (start_pos + s) / c.ratio + 2 : 0;
    if (s > 1 && chunks_enabled()) {
        // the s positions in passes of at most chunk_rows() rows (one sequence: rows are positions)
        const int per = chunk_rows() < s ? chunk_rows() : s;
        if (attn_step_bufs(c, max_nb, per, ws, &sb)) return 1;
        if (attn_state_upload(c, st, S, c.ratio ? s / c.ratio + 2 : 0, sm)) return 1;
        void *q[11];
        const size_t R = per;
        size_t qs[11] = {(size_t)s * hc * dim * 4, R * hc * dim * 4, R * dim * 4, R * dim * 4, R * dim * 4, R * hc * 4,
                         R * hc * hc * 4, (size_t)s * 8, R * ((2 + hc) * hc + 1) * 4, (size_t)(c.window + per) * c.head_dim * 4,
                         sparse_attn_scratch(c.n_heads, (int)(c.window + (c.has_indexer && c.idx_topk > max_nb ? c.idx_topk : max_nb) + 8), per)};
        for (int i = 0; i < 8; i++) if (hb[i].get(qs[i], &q[i])) return 1;
        if (hb[8].get(qs[8], &q[8]) || hb[9].get(qs[9], &q[9]) || ws[22].get(qs[10], &q[10])) return 1;
        sb.ext = (float *)q[9]; sb.sa = q[10]; sb.sa_cap = qs[10];
        float *hall = (float *)q[0];
        APUS_CUDA_OK(cudaMemcpyAsync(hall, h, qs[0], cudaMemcpyHostToDevice, sm));
        if (ids) APUS_CUDA_OK(cudaMemcpyAsync(q[7], ids, (size_t)s * 8, cudaMemcpyHostToDevice, sm));
        BlockBufs bb = {(float *)q[2], (float *)q[3], (float *)q[4], (float *)q[5], (float *)q[6], (float *)q[8]};
        for (int t = 0; t < s; t += per) {
            const int n = s - t < per ? s - t : per;
            float *ht = hall + (size_t)t * hc * dim;
            float *cur = ht, *alt = (float *)q[1];
            if (block_chunk(L, S, &cur, &alt, ids ? (const int64_t *)q[7] + t : nullptr, 1, n, start_pos + t, hc, iters, hc_eps,
                            norm_eps, bb, sb, sm))
                return 1;
            if (cur != ht) APUS_CUDA_OK(cudaMemcpyAsync(ht, cur, (size_t)n * hc * dim * 4, cudaMemcpyDeviceToDevice, sm));
        }
        APUS_CUDA_OK(cudaMemcpyAsync(h, hall, qs[0], cudaMemcpyDeviceToHost, sm));
        if (attn_state_download(c, st, S, sm)) return 1;
        APUS_CUDA_OK(cudaStreamSynchronize(sm));
        attn_state_commit(c, st, S);
        int stt2 = gemm_tc_status(1);
        APUS_REQUIRE(stt2 == 0, "block_forward: a bounded wait expired inside a tcgen05 kernel (code %d)", stt2);
        return 0;
    }
    if (attn_step_bufs(c, max_nb, 1, ws, &sb)) return 1;
    if (attn_state_upload(c, st, S, c.ratio ? s / c.ratio + 2 : 0, sm)) return 1;
    void *p[8];
    size_t sz[8] = {(size_t)s * hc * dim * 4, (size_t)hc * dim * 4, (size_t)dim * 4, (size_t)dim * 4, (size_t)dim * 4,
                    (size_t)hc * 4, (size_t)hc * hc * 4, (size_t)s * 8};
    for (int i = 0; i < 8; i++) if (hb[i].get(sz[i], &p[i])) return 1;
    float *hall = (float *)p[0];
    APUS_CUDA_OK(cudaMemcpyAsync(hall, h, sz[0], cudaMemcpyHostToDevice, sm));
    if (ids) APUS_CUDA_OK(cudaMemcpyAsync(p[7], ids, (size_t)s * 8, cudaMemcpyHostToDevice, sm));
    BlockBufs bb = {(float *)p[2], (float *)p[3], (float *)p[4], (float *)p[5], (float *)p[6], nullptr};
    for (int t = 0; t < s; t++) {
        float *ht = hall + (size_t)t * hc * dim, *hn = (float *)p[1];
        float *cur = ht, *alt = hn;
        if (block_step(L, S, &cur, &alt, ids ? (const int64_t *)p[7] + t : nullptr, 1, start_pos + t, hc, iters,
                       hc_eps, norm_eps, bb, sb, sm))
            return 1;
        if (cur != ht) APUS_CUDA_OK(cudaMemcpyAsync(ht, cur, (size_t)hc * dim * 4, cudaMemcpyDeviceToDevice, sm));
    }
    APUS_CUDA_OK(cudaMemcpyAsync(h, hall, sz[0], cudaMemcpyDeviceToHost, sm));
    if (attn_state_download(c, st, S, sm)) return 1;
    APUS_CUDA_OK(cudaStreamSynchronize(sm));
    attn_state_commit(c, st, S);
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "block_forward: a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
    return 0;
}

int64_t apus_cuda_model_pos(const ApusCudaModel *m) { return m ? m->pos : -1; }

int apus_cuda_model_info(const ApusCudaModel *m, int *batch, int *max_pos, int *vocab, int *n_layers) {
    if (!m) { set_error("NULL model"); return 1; }
    if (batch) *batch = m->B;
    if (max_pos) *max_pos = m->max_pos;
    if (vocab) *vocab = m->vocab;
    if (n_layers) *n_layers = m->n_layers;
    return 0;
}

int apus_cuda_model_set_sampling(ApusCudaModel *m, float temp, float top_p, uint64_t seed) {
    if (!m) { set_error("NULL model"); return 1; }
    cudaStream_t st = mstream(m);
    APUS_CUDA_OK(cudaStreamSynchronize(st));
    for (int i = 0; i < 2; i++)                       // the head of a recorded step changes
        if (m->gexec[i]) { cudaGraphExecDestroy(m->gexec[i]); m->gexec[i] = nullptr; }
    m->temp = temp; m->top_p = top_p;
    if (temp <= 0.f) return 0;
    if (m->rng.get((size_t)m->B * 8, nullptr) || m->probs.get((size_t)m->B * m->vocab * 4, nullptr)) return 1;
    std::vector<unsigned long long> s((size_t)m->B);
    for (int b = 0; b < m->B; b++) s[b] = seed + (unsigned long long)b;
    APUS_CUDA_OK(cudaMemcpyAsync(m->rng.p, s.data(), s.size() * 8, cudaMemcpyHostToDevice, st));
    APUS_CUDA_OK(cudaStreamSynchronize(st));
    return 0;
}

int apus_cuda_model_use_graph(ApusCudaModel *m, int enable) {
    if (!m) return -1;
    if (enable >= 0) m->use_graph = enable != 0;
    return m->use_graph ? 1 : 0;
}

ApusCudaMoe *apus_cuda_model_moe(ApusCudaModel *m, int layer) {
    if (!m || layer < 0 || layer >= m->n_layers) return nullptr;
    return m->layers[layer].moe;
}

int apus_cuda_model_set_stream(ApusCudaModel *m, void *stream, int create) {
    if (!m) { set_error("NULL model"); return 1; }
    APUS_CUDA_OK(cudaStreamSynchronize(mstream(m)));
    for (int i = 0; i < 2; i++)                       // a recorded step belongs to the stream it was recorded on
        if (m->gexec[i]) { cudaGraphExecDestroy(m->gexec[i]); m->gexec[i] = nullptr; }
    if (create) {
        if (!m->own_stream) APUS_CUDA_OK(cudaStreamCreateWithFlags(&m->own_stream, cudaStreamNonBlocking));
        m->stream = m->own_stream;
    } else {
        m->stream = (cudaStream_t)stream;
    }
    m->steps_run = 0;                                 // the next step runs eagerly on the new stream first
    return 0;
}

// Every stream of the group waits for what the others have enqueued so far, then
// `ev` is recorded on the first one: a time stamp all of the group's work lies
// before (or after) without stopping the host.
static int group_mark(ApusCudaModel *const *ms, int n, cudaEvent_t *tmp, cudaEvent_t ev) {
    cudaStream_t s0 = mstream(ms[0]);
    for (int i = 1; i < n; i++) {
        APUS_CUDA_OK(cudaEventRecord(tmp[i], mstream(ms[i])));
        APUS_CUDA_OK(cudaStreamWaitEvent(s0, tmp[i], 0));
    }
    APUS_CUDA_OK(cudaEventRecord(ev, s0));
    for (int i = 1; i < n; i++) APUS_CUDA_OK(cudaStreamWaitEvent(mstream(ms[i]), ev, 0));
    return 0;
}
static int group_sync(ApusCudaModel *const *ms, int n) {
    for (int i = 0; i < n; i++) APUS_CUDA_OK(cudaStreamSynchronize(mstream(ms[i])));
    return 0;
}
static int group_check(ApusCudaModel *const *ms, int n, const char *who) {
    APUS_REQUIRE(ms && n >= 1 && n <= 16, "%s: 1..16 models", who);
    for (int i = 0; i < n; i++) {
        APUS_REQUIRE(ms[i], "%s: NULL model", who);
        for (int j = 0; j < i; j++)
            APUS_REQUIRE(mstream(ms[i]) != mstream(ms[j]) || n == 1,
                         "%s: models %d and %d share a stream (apus_cuda_model_set_stream)", who, j, i);
    }
    return 0;
}

// Token ids index the embedding table (and the hash-routing table): one outside [0, vocab) is
// refused on the host, where the reference would read past its table (c/model.h:663-671).
static int ids_in_range(const ApusCudaModel *m, const int64_t *ids, size_t n, const char *what) {
    for (size_t i = 0; i < n; i++)
        APUS_REQUIRE(ids[i] >= 0 && ids[i] < m->vocab, "%s: token id %lld at index %zu is outside [0, %d)", what,
                     (long long)ids[i], i, m->vocab);
    return 0;
}

int apus_cuda_model_forward_group(ApusCudaModel *const *ms, int n, const int64_t *const *ids, int s,
                                  float *const *logits, int32_t *const *next) {
    if (group_check(ms, n, "model_forward")) return 1;
    if (s <= 0) return 0;
    for (int i = 0; i < n; i++) {
        APUS_REQUIRE(ms[i]->pos + s <= ms[i]->max_pos, "model_forward: position %lld + %d exceeds max_pos %d",
                     ms[i]->pos, s, ms[i]->max_pos);
        if (ids_in_range(ms[i], ids[i], (size_t)ms[i]->B * s, "model_forward")) return 1;
    }
    // the ids of every position go to the device first, time-major ([s][B]); one model after the
    // other when a call holds several positions, position by position side by side otherwise
    std::vector<std::vector<int64_t>> cols((size_t)n);
    std::vector<void *> dcols((size_t)n);
    for (int i = 0; i < n; i++) {
        ApusCudaModel *m = ms[i];
        cols[i].resize((size_t)s * m->B);
        for (int t = 0; t < s; t++)
            for (int b = 0; b < m->B; b++) cols[i][(size_t)t * m->B + b] = ids[i][(size_t)b * s + t];
        if (m->ws[23].get(cols[i].size() * 8, &dcols[i])) return 1;
        APUS_CUDA_OK(cudaMemcpyAsync(dcols[i], cols[i].data(), cols[i].size() * 8, cudaMemcpyHostToDevice, mstream(m)));
    }
    if (s > 1 && chunks_enabled()) {
        for (int i = 0; i < n; i++)
            if (model_consume(ms[i], (const int64_t *)dcols[i], s, true, mstream(ms[i]))) return 1;
    } else {
        for (int t = 0; t < s; t++)
            for (int i = 0; i < n; i++) {
                ApusCudaModel *m = ms[i];
                APUS_CUDA_OK(cudaMemcpyAsync(m->ids.p, (const int64_t *)dcols[i] + (size_t)t * m->B, (size_t)m->B * 8,
                                             cudaMemcpyDeviceToDevice, mstream(m)));
                if (model_step(m, t == s - 1, mstream(m))) return 1;
            }
    }
    for (int i = 0; i < n; i++) {
        ApusCudaModel *m = ms[i];
        if (logits && logits[i])
            APUS_CUDA_OK(cudaMemcpyAsync(logits[i], m->logits.p, (size_t)m->B * m->vocab * 4, cudaMemcpyDeviceToHost, mstream(m)));
        if (next && next[i])
            APUS_CUDA_OK(cudaMemcpyAsync(next[i], m->tok.p, (size_t)m->B * 4, cudaMemcpyDeviceToHost, mstream(m)));
    }
    if (group_sync(ms, n)) return 1;
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "model_forward: a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
    return 0;
}

int apus_cuda_model_forward(ApusCudaModel *m, const int64_t *ids, int s, float *logits, int32_t *next) {
    if (!m) { set_error("NULL model"); return 1; }
    return apus_cuda_model_forward_group(&m, 1, &ids, s, &logits, &next);
}

// c/model.h:651-720 with every output the reference's variants offer (logits_all, h_out of
// apus_model_forward_h, mh_out of apus_model_forward_mh), B sequences: ids [B][s]; logits
// [B][V] (last position) or [B][s][V]; next [B] or [B][s]; h_out [B][s][hc*dim]; mh_out
// [B][s][n_targets*dim].  The positions run as chunks; a row of a chunk equals the step's.
static int forward_ex(ApusCudaModel *m, const int64_t *ids, int s, float *logits, int logits_all, int32_t *next,
                      float *h_out, float *mh_out, const int *targets, int n_targets, const char *what,
                      bool keep_h_dev = false, bool keep_mh_dev = false) {
    if (!m) { set_error("NULL model"); return 1; }
    if (s <= 0) return 0;
    APUS_REQUIRE(m->pos + s <= m->max_pos, "%s: position %lld + %d exceeds max_pos %d", what, m->pos, s, m->max_pos);
    APUS_REQUIRE(!(mh_out || keep_mh_dev) || (targets && n_targets >= 1), "%s: mh_out needs the target layers", what);
    for (int i = 0; (mh_out || keep_mh_dev) && i < n_targets; i++)
        APUS_REQUIRE(targets[i] >= 0 && targets[i] < m->n_layers, "%s: target layer %d of %d", what, targets[i], m->n_layers);
    if (ids_in_range(m, ids, (size_t)m->B * s, what)) return 1;
    cudaStream_t st = mstream(m);
    const size_t B = m->B, V = m->vocab, hd = (size_t)m->hc * m->dim, md = (size_t)n_targets * m->dim;
    std::vector<int64_t> cols((size_t)s * B);
    for (int t = 0; t < s; t++)
        for (size_t b = 0; b < B; b++) cols[(size_t)t * B + b] = ids[b * s + t];
    void *dcols;
    if (m->ws[23].get(cols.size() * 8, &dcols)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dcols, cols.data(), cols.size() * 8, cudaMemcpyHostToDevice, st));
    int per = chunks_enabled() ? chunk_rows() / (int)B : 1;
    if (per < 1) per = 1;
    if (per > s) per = s;
    ApusCudaModel::Chunk &C = m->ck;
    const bool all = logits_all != 0;
    if (all && (C.logits.get((size_t)per * B * V * 4, nullptr) || C.tok.get((size_t)per * B * 4, nullptr))) return 1;
    APUS_REQUIRE(!(keep_h_dev || keep_mh_dev) || per >= s, "%s: %d positions do not fit one chunk", what, s);
    if ((h_out || keep_h_dev) && C.hx.get((size_t)per * B * hd * 4, nullptr)) return 1;
    if ((mh_out || keep_mh_dev) && C.mhx.get((size_t)per * B * md * 4, nullptr)) return 1;
    for (int t0 = 0; t0 < s; t0 += per) {
        const int n = s - t0 < per ? s - t0 : per;
        ChunkExtra ex;
        if (all) { ex.logits_all = C.logits.as<float>(); ex.tok_all = C.tok.as<int32_t>(); }
        if (h_out || keep_h_dev) ex.h_all = C.hx.as<float>();
        if (mh_out || keep_mh_dev) { ex.mh_all = C.mhx.as<float>(); ex.targets = targets; ex.n_targets = n_targets; }
        if (model_chunk(m, (const int64_t *)dcols + (size_t)t0 * B, n, !all && t0 + n == s, st, &ex)) return 1;
        for (int t = 0; t < n; t++) {                      // row (t, b) of the chunk -> [b][t0 + t] of the caller
            if (all && logits)
                APUS_CUDA_OK(cudaMemcpy2DAsync(logits + (size_t)(t0 + t) * V, (size_t)s * V * 4, C.logits.as<float>() + (size_t)t * B * V,
                                               V * 4, V * 4, B, cudaMemcpyDeviceToHost, st));
            if (all && next)
                APUS_CUDA_OK(cudaMemcpy2DAsync(next + t0 + t, (size_t)s * 4, C.tok.as<int32_t>() + (size_t)t * B, 4, 4, B,
                                               cudaMemcpyDeviceToHost, st));
            if (h_out)
                APUS_CUDA_OK(cudaMemcpy2DAsync(h_out + (size_t)(t0 + t) * hd, (size_t)s * hd * 4, C.hx.as<float>() + (size_t)t * B * hd,
                                               hd * 4, hd * 4, B, cudaMemcpyDeviceToHost, st));
            if (mh_out)
                APUS_CUDA_OK(cudaMemcpy2DAsync(mh_out + (size_t)(t0 + t) * md, (size_t)s * md * 4, C.mhx.as<float>() + (size_t)t * B * md,
                                               md * 4, md * 4, B, cudaMemcpyDeviceToHost, st));
        }
    }
    if (!all) {
        if (logits) APUS_CUDA_OK(cudaMemcpyAsync(logits, m->logits.p, B * V * 4, cudaMemcpyDeviceToHost, st));
        if (next) APUS_CUDA_OK(cudaMemcpyAsync(next, m->tok.p, B * 4, cudaMemcpyDeviceToHost, st));
    }
    APUS_CUDA_OK(cudaStreamSynchronize(st));
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "%s: a bounded wait expired inside a tcgen05 kernel (code %d)", what, stt);
    return 0;
}

int apus_cuda_model_forward_h(ApusCudaModel *m, const int64_t *ids, int s, float *logits, int logits_all, int32_t *next,
                              float *h_out) {
    return forward_ex(m, ids, s, logits, logits_all, next, h_out, nullptr, nullptr, 0, "model_forward_h");
}
int apus_cuda_model_forward_mh(ApusCudaModel *m, const int64_t *ids, int s, float *logits, int logits_all, int32_t *next,
                               const int *targets, int n_targets, float *mh_out) {
    return forward_ex(m, ids, s, logits, logits_all, next, nullptr, mh_out, targets, n_targets, "model_forward_mh");
}

// c/model.h:651-720 with logits_all: the rows of every position (the verify batch of
// speculative decoding, c/mtp.h step 2), in one pass over the positions unless chunks are off.
int apus_cuda_model_forward_all(ApusCudaModel *m, const int64_t *ids, int s, float *logits_all, int32_t *next_all) {
    if (!m) { set_error("NULL model"); return 1; }
    if (s <= 0) return 0;
    if (chunks_enabled() && m->e_lo == 0 && m->e_hi == m->n_experts)
        return forward_ex(m, ids, s, logits_all, 1, next_all, nullptr, nullptr, nullptr, 0, "model_forward_all");
    APUS_REQUIRE(m->pos + s <= m->max_pos, "model_forward: position %lld + %d exceeds max_pos %d", m->pos, s, m->max_pos);
    if (ids_in_range(m, ids, (size_t)m->B * s, "model_forward_all")) return 1;
    cudaStream_t st = mstream(m);
    const size_t B = m->B, V = m->vocab;
    std::vector<int64_t> cols((size_t)s * B);
    for (int t = 0; t < s; t++)
        for (size_t b = 0; b < B; b++) cols[(size_t)t * B + b] = ids[b * s + t];
    void *dcols;
    if (m->ws[23].get(cols.size() * 8, &dcols)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dcols, cols.data(), cols.size() * 8, cudaMemcpyHostToDevice, st));
    for (int t = 0; t < s; t++) {
        APUS_CUDA_OK(cudaMemcpyAsync(m->ids.p, (const int64_t *)dcols + (size_t)t * B, B * 8, cudaMemcpyDeviceToDevice, st));
        if (model_step(m, true, st)) return 1;
        if (logits_all)        // row b of this position -> logits_all[b][t]
            APUS_CUDA_OK(cudaMemcpy2DAsync(logits_all + (size_t)t * V, (size_t)s * V * 4, m->logits.p, V * 4, V * 4, B,
                                           cudaMemcpyDeviceToHost, st));
        if (next_all)
            APUS_CUDA_OK(cudaMemcpy2DAsync(next_all + t, (size_t)s * 4, m->tok.p, 4, 4, B, cudaMemcpyDeviceToHost, st));
    }
    APUS_CUDA_OK(cudaStreamSynchronize(st));
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "model_forward: a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
    return 0;
}

int apus_cuda_model_generate_group(ApusCudaModel *const *ms, int n, const int64_t *const *prompts, int n_prompt,
                                   int n_gen, int32_t *const *out_tokens, float *ms_prefill, float *ms_decode) {
    if (group_check(ms, n, "model_generate")) return 1;
    APUS_REQUIRE(n_prompt >= 1 && n_gen >= 1, "model_generate: needs a prompt and at least one token to generate");
    for (int i = 0; i < n; i++) {
        APUS_REQUIRE(ms[i]->pos + n_prompt + n_gen - 1 <= ms[i]->max_pos, "model_generate: %d + %d tokens exceed max_pos %d",
                     n_prompt, n_gen, ms[i]->max_pos);
        if (ids_in_range(ms[i], prompts[i], (size_t)ms[i]->B * n_prompt, "model_generate")) return 1;
    }
    cudaEvent_t e0, e1, e2, tmp[16];
    APUS_CUDA_OK(cudaEventCreate(&e0)); APUS_CUDA_OK(cudaEventCreate(&e1)); APUS_CUDA_OK(cudaEventCreate(&e2));
    for (int i = 0; i < n; i++) APUS_CUDA_OK(cudaEventCreateWithFlags(&tmp[i], cudaEventDisableTiming));
    // the prompt columns are staged on the device first so the loop has no host copies
    std::vector<std::vector<int64_t>> cols((size_t)n);
    std::vector<void *> dcols((size_t)n);
    for (int i = 0; i < n; i++) {
        ApusCudaModel *m = ms[i];
        if (m->hist.get((size_t)m->B * n_gen * 4, nullptr)) return 1;
        cols[i].resize((size_t)n_prompt * m->B);
        for (int t = 0; t < n_prompt; t++)
            for (int b = 0; b < m->B; b++) cols[i][(size_t)t * m->B + b] = prompts[i][(size_t)b * n_prompt + t];
        if (m->ws[23].get(cols[i].size() * 8, &dcols[i])) return 1;
        APUS_CUDA_OK(cudaMemcpyAsync(dcols[i], cols[i].data(), cols[i].size() * 8, cudaMemcpyHostToDevice, mstream(m)));
    }
    if (group_mark(ms, n, tmp, e0)) return 1;
    if (n_prompt > 1 && chunks_enabled()) {
        for (int i = 0; i < n; i++)
            if (model_consume(ms[i], (const int64_t *)dcols[i], n_prompt, true, mstream(ms[i]))) return 1;
    } else {
        for (int t = 0; t < n_prompt; t++)
            for (int i = 0; i < n; i++) {
                ApusCudaModel *m = ms[i];
                APUS_CUDA_OK(cudaMemcpyAsync(m->ids.p, (const int64_t *)dcols[i] + (size_t)t * m->B, (size_t)m->B * 8,
                                             cudaMemcpyDeviceToDevice, mstream(m)));
                if (model_step(m, t == n_prompt - 1, mstream(m))) return 1;
            }
    }
    if (group_mark(ms, n, tmp, e1)) return 1;
    for (int g = 0; g < n_gen; g++)
        for (int i = 0; i < n; i++) {                     // the models' steps alternate, each on its own stream
            ApusCudaModel *m = ms[i];
            launch_k(next_ids_kernel, 1, 32, 0, mstream(m), m->tok.as<int32_t>(), m->ids.as<int64_t>(), m->hist.as<int32_t>(),
                                                     m->B, g, n_gen);
            if (g + 1 < n_gen && model_step(m, true, mstream(m))) return 1;
        }
    if (group_mark(ms, n, tmp, e2)) return 1;
    for (int i = 0; i < n; i++)
        APUS_CUDA_OK(cudaMemcpyAsync(out_tokens[i], ms[i]->hist.p, (size_t)ms[i]->B * n_gen * 4, cudaMemcpyDeviceToHost,
                                     mstream(ms[i])));
    if (group_sync(ms, n)) return 1;
    float a = 0, b = 0;
    cudaEventElapsedTime(&a, e0, e1); cudaEventElapsedTime(&b, e1, e2);
    if (ms_prefill) *ms_prefill = a;
    if (ms_decode) *ms_decode = b;
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(e2);
    for (int i = 0; i < n; i++) cudaEventDestroy(tmp[i]);
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "model_generate: a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
    return 0;
}

int apus_cuda_model_generate(ApusCudaModel *m, const int64_t *prompt, int n_prompt, int n_gen, int32_t *out_tokens,
                             float *ms_prefill, float *ms_decode) {
    if (!m) { set_error("NULL model"); return 1; }
    return apus_cuda_model_generate_group(&m, 1, &prompt, n_prompt, n_gen, &out_tokens, ms_prefill, ms_decode);
}

// ---- snapshots (c/mtp.h:113-138, 398-439) -------------------------------------------------------
static int snap_copy(DevBuf &dst, const DevBuf &src, size_t bytes, bool to_snap, cudaStream_t st) {
    if (!bytes) return 0;
    if (to_snap && dst.get(bytes, nullptr)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dst.p, src.p, bytes, cudaMemcpyDeviceToDevice, st));
    return 0;
}
static int snap_layer(const ApusAttnCfg &c, StateDev &S, ApusCudaSnap::Layer &L, size_t B, bool take, cudaStream_t st) {
    const size_t wb = B * c.window * c.head_dim * 4, cb = S.comp.carry * B * 4, ib = S.idx.carry * B * 4;
    DevBuf *pairs[5][2] = {{&L.win, &S.win}, {&L.ckv, &S.comp.kv}, {&L.csc, &S.comp.sc}, {&L.ikv, &S.idx.kv},
                           {&L.isc, &S.idx.sc}};
    const size_t bytes[5] = {wb, c.ratio ? cb : 0, c.ratio ? cb : 0, c.ratio && c.has_indexer ? ib : 0,
                             c.ratio && c.has_indexer ? ib : 0};
    for (int k = 0; k < 5; k++)
        if (take ? snap_copy(*pairs[k][0], *pairs[k][1], bytes[k], true, st)
                 : snap_copy(*pairs[k][1], *pairs[k][0], bytes[k], false, st))
            return 1;
    if (take) { L.comp_nb = S.comp.nb; L.idx_nb = S.idx.nb; }
    else { S.comp.nb = L.comp_nb; S.idx.nb = L.idx_nb; }
    return 0;
}
static int snap_move(ApusCudaModel *m, ApusCudaSnap *sn, bool take) {
    cudaStream_t st = mstream(m);
    const size_t B = m->B;
    for (int i = 0; i < m->n_layers; i++)
        if (snap_layer(m->layers[i].attn.cfg, m->states[i], sn->layers[i], B, take, st)) return 1;
    DevBuf *top[3][2] = {{&sn->pos_dev, &m->pos_dev}, {&sn->tok, &m->tok}, {&sn->ids, &m->ids}};
    const size_t tb[3] = {256, B * 4, B * 8};
    for (int k = 0; k < 3; k++)
        if (take ? snap_copy(*top[k][0], *top[k][1], tb[k], true, st) : snap_copy(*top[k][1], *top[k][0], tb[k], false, st))
            return 1;
    if (take) sn->has_rng = m->temp > 0.f && m->rng.p;
    if (sn->has_rng && m->rng.p &&
        (take ? snap_copy(sn->rng, m->rng, B * 8, true, st) : snap_copy(m->rng, sn->rng, B * 8, false, st)))
        return 1;
    if (take) sn->pos = m->pos; else m->pos = sn->pos;
    return 0;
}

ApusCudaSnap *apus_cuda_model_snapshot(ApusCudaModel *m, ApusCudaSnap *reuse) {
    if (!m) { set_error("NULL model"); return nullptr; }
    if (reuse && ((int)reuse->layers.size() != m->n_layers || reuse->B != m->B)) {
        set_error("model_snapshot: the snapshot to reuse belongs to another model shape");
        return nullptr;
    }
    ApusCudaSnap *sn = reuse ? reuse : new ApusCudaSnap();
    if (!reuse) { sn->layers.resize(m->n_layers); sn->B = m->B; }
    if (snap_move(m, sn, true)) {
        if (!reuse) apus_cuda_snap_free(sn);
        return nullptr;
    }
    return sn;
}

int apus_cuda_model_restore(ApusCudaModel *m, const ApusCudaSnap *sn) {
    if (!m || !sn) { set_error("model_restore: NULL argument"); return 1; }
    APUS_REQUIRE((int)sn->layers.size() == m->n_layers && sn->B == m->B, "model_restore: snapshot of another model shape");
    for (int i = 0; i < m->n_layers; i++) {               // same layer count and batch is not enough: sizes too
        const ApusAttnCfg &c = m->layers[i].attn.cfg;
        const ApusCudaSnap::Layer &L = sn->layers[i];
        const size_t wb = (size_t)m->B * c.window * c.head_dim * 4, cb = m->states[i].comp.carry * (size_t)m->B * 4,
                     ib = m->states[i].idx.carry * (size_t)m->B * 4;
        APUS_REQUIRE(L.win.cap >= wb && (!c.ratio || (L.ckv.cap >= cb && L.csc.cap >= cb)) &&
                         (!(c.ratio && c.has_indexer) || (L.ikv.cap >= ib && L.isc.cap >= ib)),
                     "model_restore: layer %d of the snapshot has other sizes than the model's", i);
    }
    return snap_move(m, const_cast<ApusCudaSnap *>(sn), false);
}

void apus_cuda_snap_free(ApusCudaSnap *sn) {
    if (!sn) return;
    cudaDeviceSynchronize();
    for (auto &L : sn->layers) { L.win.release(); L.ckv.release(); L.csc.release(); L.ikv.release(); L.isc.release(); }
    sn->pos_dev.release(); sn->tok.release(); sn->ids.release(); sn->rng.release();
    delete sn;
}

// ---- speculative decoding engine (c/mtp.h:142-190, 531-616 with a caller-supplied proposer) --------
// The reference's accept rule: every emitted token is the main model's own pick from its
// own logits row (greedy, or the sampler's draw: one uniform per token in position order),
// a draft is accepted iff it equals that pick -- so the emitted stream is bit for bit the
// non-speculative one.  Round: snapshot, verify batch [held, d2..dD], walk, and on a partial
// match roll back and feed the true prefix again.  The picks are drawn on the device; the
// rollback rewinds the sampler streams with the rest of the state, so a round consumes
// exactly one uniform per token that stays.
// ---- MTP draft head (c/mtp.h:66-110, 303-357) -----------------------------------------------------
// e = enorm(embed(id)) -> e_proj; x_j = hnorm(h_j) -> h_proj per hc stream; bf16(e + x_j) -> one full
// block (its own attention state) -> its own hc_head collapse and norm -> the parent's LM head.
struct ApusCudaMtp {
    ApusCudaModel *m = nullptr;
    LayerDev block;
    StateDev state;
    DevQW *e_proj = nullptr, *h_proj = nullptr;
    const float *enorm_w = nullptr, *hnorm_w = nullptr, *norm_w = nullptr, *hc_head_fn = nullptr, *hc_head_base = nullptr;
    float hc_head_scale = 0.f;
    WeightOwner own;
    int rows = 0, s_cap = 0;                     // capacity of the buffers below: rows = positions x sequences
    DevBuf e, en, ep, hn, hp, x0, x1, bx, by, bsub, post, comb, raw, sa, ext, xq, xs, ids, hin, yh, yn, logits, tok, hlast, ws[24];
    StepBufs sb;
    ApusCudaSnap::Layer snap;
    void release() {
        DevBuf *b[] = {&e, &en, &ep, &hn, &hp, &x0, &x1, &bx, &by, &bsub, &post, &comb, &raw, &sa, &ext, &xq, &xs, &ids, &hin,
                       &yh, &yn, &logits, &tok, &hlast, &snap.win, &snap.ckv, &snap.csc, &snap.ikv, &snap.isc};
        for (DevBuf *p : b) p->release();
        for (auto &w : ws) w.release();
        state.release();
        if (block.moe) apus_cuda_moe_destroy(block.moe);
        block.moe = nullptr;
        own.release();
    }
};

__global__ void mtp_mix_kernel(const float *__restrict__ ep, const float *__restrict__ hp, int hc, int dim, float *__restrict__ x) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int r = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;       // r = token * hc + stream
    if (i < dim) x[(size_t)r * dim + i] = bf16_round(__fadd_rn(ep[(size_t)(r / hc) * dim + i], hp[(size_t)r * dim + i]));
}

static int mtp_bufs(ApusCudaMtp *mt, int s) {
    ApusCudaModel *m = mt->m;
    const size_t T = (size_t)m->B * s, dim = m->dim, hc = m->hc;
    if ((int)T <= mt->rows && s <= mt->s_cap) return 0;
    const size_t R = (int)T > mt->rows ? T : (size_t)mt->rows;
    const int sc = s > mt->s_cap ? s : mt->s_cap;
    const ApusAttnCfg &c = mt->block.attn.cfg;
    const long long max_nb = c.ratio ? m->max_pos / c.ratio + 2 : 8;
    const long long wide = c.has_indexer && c.idx_topk > max_nb ? c.idx_topk : max_nb;
    if (mt->e.get(R * dim * 4, nullptr) || mt->en.get(R * dim * 4, nullptr) || mt->ep.get(R * dim * 4, nullptr) ||
        mt->hn.get(R * hc * dim * 4, nullptr) || mt->hp.get(R * hc * dim * 4, nullptr) || mt->x0.get(R * hc * dim * 4, nullptr) ||
        mt->x1.get(R * hc * dim * 4, nullptr) || mt->bx.get(R * dim * 4, nullptr) || mt->by.get(R * dim * 4, nullptr) ||
        mt->bsub.get(R * dim * 4, nullptr) || mt->post.get(R * hc * 4, nullptr) || mt->comb.get(R * hc * hc * 4, nullptr) ||
        mt->raw.get(R * ((2 + hc) * hc + 1) * 4, nullptr) || mt->xq.get(R * hc * dim, nullptr) ||
        mt->xs.get(R * hc * (dim / 128 + 1) * 4, nullptr) || mt->ids.get(R * 8, nullptr) ||
        mt->ext.get((size_t)m->B * (c.window + sc) * c.head_dim * 4, nullptr))
        return 1;
    ApusAttnCfg sized = c;
    sized.has_indexer = 0;
    if (attn_step_bufs(sized, wide, (int)R, mt->ws, &mt->sb)) return 1;
    mt->sb.sa_cap = sparse_attn_scratch(c.n_heads, (int)(c.window + wide + 8), (int)R);
    if (mt->sa.get(mt->sb.sa_cap, &mt->sb.sa)) return 1;
    mt->sb.ext = mt->ext.as<float>();
    mt->rows = (int)R; mt->s_cap = sc;
    return 0;
}

// h_in (device) [s][B][hc*dim] time-major, ids_tm (device) [s][B]; leaves the last position's logits,
// pick and post-block hidden in mt->logits / tok / hlast.  Positions start_pos .. start_pos + s - 1.
static int mtp_forward_dev(ApusCudaMtp *mt, const float *h_in, const int64_t *ids_tm, int s, long long start_pos,
                           cudaStream_t st) {
    ApusCudaModel *m = mt->m;
    const int B = m->B, dim = m->dim, hc = m->hc;
    APUS_REQUIRE(s >= 1 && start_pos >= 0 && start_pos + s <= m->max_pos, "mtp_forward: positions %lld + %d exceed max_pos %d",
                 start_pos, s, m->max_pos);
    int per = chunk_rows() / B;
    if (per < 1) per = 1;
    if (per > s) per = s;
    if (mtp_bufs(mt, per)) return 1;
    const BlockBufs bb = {mt->bx.as<float>(), mt->by.as<float>(), mt->bsub.as<float>(), mt->post.as<float>(),
                          mt->comb.as<float>(), mt->raw.as<float>()};
    float *last = nullptr;
    for (int t0 = 0; t0 < s; t0 += per) {
        const int n = s - t0 < per ? s - t0 : per, T = n * B;
        const int64_t *ids = ids_tm + (size_t)t0 * B;
        const float *hin = h_in + (size_t)t0 * B * hc * dim;
        if (embed_rows(m->embed, m->embed_bf16, ids, T, 1, dim, mt->e.as<float>(), st)) return 1;
        if (rms_norm(mt->e.as<float>(), mt->enorm_w, m->norm_eps, mt->en.as<float>(), dim, T, st)) return 1;
        if (qlinear_dev(mt->e_proj, mt->en.as<float>(), mt->ep.as<float>(), T, mt->xq.as<uint8_t>(), mt->xs.as<float>(), true, st)) return 1;
        if (rms_norm(hin, mt->hnorm_w, m->norm_eps, mt->hn.as<float>(), dim, (int64_t)T * hc, st)) return 1;
        if (qlinear_dev(mt->h_proj, mt->hn.as<float>(), mt->hp.as<float>(), T * hc, mt->xq.as<uint8_t>(), mt->xs.as<float>(), true, st)) return 1;
        float *x = mt->x0.as<float>(), *xa = mt->x1.as<float>();
        launch_k(mtp_mix_kernel, dim3(ceil_div(dim, 256), T * hc), 256, 0, st, mt->ep.as<float>(), mt->hp.as<float>(), hc, dim, x);
        APUS_LAUNCHED();
        if (block_chunk(mt->block, mt->state, &x, &xa, ids, B, n, start_pos + t0, hc, m->iters, m->hc_eps, m->norm_eps, bb,
                        mt->sb, st))
            return 1;
        last = x + (size_t)(n - 1) * B * hc * dim;
    }
    // the block's own collapse and norm, the parent's head (c/mtp.h:341-355), last position only
    if (mt->hlast.get((size_t)B * hc * dim * 4, nullptr) || mt->yh.get((size_t)B * dim * 4, nullptr) ||
        mt->yn.get((size_t)B * dim * 4, nullptr) || mt->logits.get((size_t)B * m->vocab * 4, nullptr) ||
        mt->tok.get((size_t)B * 4, nullptr))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(mt->hlast.p, last, (size_t)B * hc * dim * 4, cudaMemcpyDeviceToDevice, st));
    if (mhc_head(last, dim, hc, mt->hc_head_fn, mt->hc_head_scale, mt->hc_head_base, m->norm_eps, m->hc_eps,
                 mt->yh.as<float>(), B, st, mt->raw.as<float>()))
        return 1;
    if (rms_norm(mt->yh.as<float>(), mt->norm_w, m->norm_eps, mt->yn.as<float>(), dim, B, st)) return 1;
    if (f32_linear(m->head, mt->yn.as<float>(), mt->logits.as<float>(), B, dim, m->vocab,
                   (m->head_bf16 ? APUS_CUDA_W_BF16 : 0) | APUS_LIN_CLASS(APUS_CUDA_TREE_HEAD), st))
        return 1;
    return argmax_rows(mt->logits.as<float>(), m->vocab, B, mt->tok.as<int32_t>(), st);
}

void apus_cuda_mtp_destroy(ApusCudaMtp *mt) {
    if (!mt) return;
    cudaDeviceSynchronize();
    mt->release();
    delete mt;
}

int apus_cuda_mtp_reset(ApusCudaMtp *mt) {
    if (!mt) { set_error("NULL mtp"); return 1; }
    const ApusAttnCfg &c = mt->block.attn.cfg;
    if (attn_state_init(c, mt->state, mt->m->B, c.ratio ? mt->m->max_pos / c.ratio + 2 : 0)) return 1;
    APUS_CUDA_OK(cudaStreamSynchronize(ctx().stream));
    return 0;
}

ApusCudaMtp *apus_cuda_mtp_create(ApusCudaModel *m, const ApusCudaMtpDesc *d) {
    if (!m || !d) { set_error("mtp_create: NULL argument"); return nullptr; }
    if (m->e_lo != 0 || m->e_hi != m->n_experts) { set_error("mtp_create: the parent holds a slice of the experts"); return nullptr; }
    const int dim = m->dim, hc = m->hc;
    if (d->block.acfg.dim != dim || d->e_proj.O != dim || d->e_proj.K != dim || d->h_proj.O != dim || d->h_proj.K != dim) {
        set_error("mtp_create: block / e_proj / h_proj do not match the parent's dim %d", dim);
        return nullptr;
    }
    ApusCudaMtp *mt = new ApusCudaMtp();
    mt->m = m;
    bool ok = layer_weights(d->block, hc, m->vocab, &mt->block, &mt->own, 0, -1) == 0;
    if (ok) {
        const int half = d->block.acfg.rope_dim / 2;
        mt->block.cs = rope_rows_dev(d->block.cos, d->block.sin, d->block.rope_rows, half, m->rope);
        mt->block.rope_rows = d->block.rope_rows;
        if (!mt->block.cs || d->block.rope_rows < m->max_pos) {
            set_error("mtp_create: the block's rope table has %d rows, %d needed", d->block.rope_rows, m->max_pos);
            ok = false;
        }
    }
    if (ok) {
        mt->e_proj = get_qw(&mt->own, 8, d->e_proj.codes, d->e_proj.scales, dim, dim);
        mt->h_proj = get_qw(&mt->own, 8, d->h_proj.codes, d->h_proj.scales, dim, dim);
        mt->enorm_w = (const float *)get_dense(&mt->own, d->enorm_w, (size_t)dim * 4);
        mt->hnorm_w = (const float *)get_dense(&mt->own, d->hnorm_w, (size_t)dim * 4);
        mt->norm_w = (const float *)get_dense(&mt->own, d->norm_w, (size_t)dim * 4);
        mt->hc_head_fn = (const float *)get_dense(&mt->own, d->hc_head_fn, (size_t)hc * hc * dim * 4);
        mt->hc_head_base = (const float *)get_dense(&mt->own, d->hc_head_base, (size_t)hc * 4);
        mt->hc_head_scale = d->hc_head_scale;
        ok = mt->e_proj && mt->h_proj && mt->enorm_w && mt->hnorm_w && mt->norm_w && mt->hc_head_fn && mt->hc_head_base;
    }
    if (ok) ok = apus_cuda_mtp_reset(mt) == 0;
    if (!ok) { apus_cuda_mtp_destroy(mt); return nullptr; }
    return mt;
}

// c/mtp.h:303-357 apus_mtp_forward for every sequence: h_in [B][s][hc*dim], ids [B][s] (host);
// logits [B][V], next [B], h_last [B][hc*dim] of the last position (all nullable).
int apus_cuda_mtp_forward(ApusCudaMtp *mt, const float *h_in, const int64_t *ids, int s, int64_t start_pos, float *logits,
                          int32_t *next, float *h_last) {
    if (!mt || !h_in || !ids) { set_error("mtp_forward: NULL argument"); return 1; }
    if (s <= 0) return 0;
    ApusCudaModel *m = mt->m;
    cudaStream_t st = mstream(m);
    const size_t B = m->B, hd = (size_t)m->hc * m->dim;
    if (ids_in_range(m, ids, B * s, "mtp_forward")) return 1;
    std::vector<int64_t> cols((size_t)s * B);
    for (int t = 0; t < s; t++)
        for (size_t b = 0; b < B; b++) cols[(size_t)t * B + b] = ids[b * s + t];
    if (mt->ids.get(cols.size() * 8, nullptr) || mt->hin.get((size_t)s * B * hd * 4, nullptr)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(mt->ids.p, cols.data(), cols.size() * 8, cudaMemcpyHostToDevice, st));
    for (int t = 0; t < s; t++)                          // [b][t] of the caller -> row (t, b)
        APUS_CUDA_OK(cudaMemcpy2DAsync(mt->hin.as<float>() + (size_t)t * B * hd, hd * 4, h_in + (size_t)t * hd, (size_t)s * hd * 4,
                                       hd * 4, B, cudaMemcpyHostToDevice, st));
    if (mtp_forward_dev(mt, mt->hin.as<float>(), mt->ids.as<int64_t>(), s, start_pos, st)) return 1;
    if (logits) APUS_CUDA_OK(cudaMemcpyAsync(logits, mt->logits.p, B * m->vocab * 4, cudaMemcpyDeviceToHost, st));
    if (next) APUS_CUDA_OK(cudaMemcpyAsync(next, mt->tok.p, B * 4, cudaMemcpyDeviceToHost, st));
    if (h_last) APUS_CUDA_OK(cudaMemcpyAsync(h_last, mt->hlast.p, B * hd * 4, cudaMemcpyDeviceToHost, st));
    APUS_CUDA_OK(cudaStreamSynchronize(st));
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "mtp_forward: a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
    return 0;
}

// ---- DSpark draft module (c/dspark.h) --------------------------------------------------------------
// n_stages full sliding-window blocks whose rings hold, for every TRUE position, the KV row made from
// main_x = main_norm(main_proj(main_hidden)) (one projection shared by the stages), plus a block of B
// draft rows [anchor, noise x (B-1)] that attend over the ring and over each other (one shared,
// non-causal index row), the last stage's own hc_head + norm, the parent's LM head, a bigram bias
// w2 . w1[previous token] added row by row before each pick, and a confidence head (telemetry).
struct ApusCudaDspark {
    ApusCudaModel *m = nullptr;
    int n_stages = 0, B = 0, noise_id = 0, rank = 0, n_targets = 0, targets[8] = {0};
    std::vector<LayerDev> stages;
    std::vector<StateDev> states;
    DevQW *main_proj = nullptr;
    const float *main_norm_w = nullptr, *norm_w = nullptr, *hc_head_fn = nullptr, *hc_head_base = nullptr,
                *markov_w1 = nullptr, *markov_w2 = nullptr, *conf_proj = nullptr;
    float hc_head_scale = 0.f;
    WeightOwner own;
    int rows_cap = 0;
    DevBuf mh, mxa, mx, pq, ps, kva, kv, h0, h1, x, y, sub, post, comb, raw, sa, ids, idxs, yh, yn, logits, emb, tok, cur,
        conf, drafts, drng, probs, ws[24];
    float temp = 0.f;                       // > 0: the drafts are drawn at this temperature from the module's own stream (drng)
    StepBufs sb;
    void release() {
        DevBuf *b[] = {&mh, &mxa, &mx, &pq, &ps, &kva, &kv, &h0, &h1, &x, &y, &sub, &post, &comb, &raw, &sa, &ids, &idxs,
                       &yh, &yn, &logits, &emb, &tok, &cur, &conf, &drafts, &drng, &probs};
        for (DevBuf *p : b) p->release();
        for (auto &w : ws) w.release();
        for (auto &st : states) st.release();
        for (auto &L : stages) if (L.moe) { apus_cuda_moe_destroy(L.moe); L.moe = nullptr; }
        own.release();
    }
};

// bias[v] = sum_r e[r] * w2[v][r] in index order (c/attn.h:460-465 apus_dot_f32_scalar: one accumulator,
// product rounded before the add), e = w1[previous token]; row[v] += bias[v] (c/dspark.h:661-672)
__global__ void markov_bias_kernel(const float *__restrict__ w1, const float *__restrict__ w2, const long long *__restrict__ cur,
                                   int rank, int V, float *__restrict__ row, float *__restrict__ embed) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const float *e = w1 + (size_t)(*cur) * rank;
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (blockIdx.x == 0 && embed)
        for (int r = threadIdx.x; r < rank; r += blockDim.x) embed[r] = e[r];
    if (v >= V) return;
    float acc = 0.f;
    for (int r = 0; r < rank; r++) acc = __fadd_rn(acc, __fmul_rn(e[r], w2[(size_t)v * rank + r]));
    row[v] = __fadd_rn(row[v], acc);
}
__global__ void markov_take_kernel(const int32_t *__restrict__ tok, long long *__restrict__ cur, long long *__restrict__ drafts, int i) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    *cur = *tok;
    drafts[i] = *tok;
}
// confidence[t] = sum over [collapsed row | bigram embedding] * proj, index order (c/dspark.h:679-694)
__global__ void confidence_kernel(const float *__restrict__ xh, const float *__restrict__ emb, const float *__restrict__ proj,
                                  int dim, int rank, float *__restrict__ out) {
    APUS_PDL_WAIT();
    APUS_PDL_GO();
    const int t = blockIdx.x;
    if (threadIdx.x) return;
    float acc = 0.f;
    for (int i = 0; i < dim; i++) acc = __fadd_rn(acc, __fmul_rn(xh[(size_t)t * dim + i], proj[i]));
    for (int r = 0; r < rank; r++) acc = __fadd_rn(acc, __fmul_rn(emb[(size_t)t * rank + r], proj[dim + r]));
    out[t] = acc;
}

static int ds_bufs(ApusCudaDspark *ds, int rows) {
    ApusCudaModel *m = ds->m;
    if (rows <= ds->rows_cap) return 0;
    const size_t R = rows, dim = m->dim, hc = m->hc, mhd = (size_t)ds->n_targets * dim;
    const ApusAttnCfg &c = ds->stages[0].attn.cfg;
    if (ds->mh.get(R * mhd * 4, nullptr) || ds->mxa.get(R * dim * 4, nullptr) || ds->mx.get(R * dim * 4, nullptr) ||
        ds->pq.get(R * mhd, nullptr) || ds->ps.get(R * (mhd / 128 + 1) * 4, nullptr) ||
        ds->kva.get(R * c.head_dim * 4, nullptr) || ds->kv.get(R * c.head_dim * 4, nullptr))
        return 1;
    ds->rows_cap = rows;
    return 0;
}

// main_x rows (c/dspark.h:365-376) from main-hidden rows on the device
static int ds_project(ApusCudaDspark *ds, const float *mh, int rows, cudaStream_t st) {
    ApusCudaModel *m = ds->m;
    if (ds_bufs(ds, rows)) return 1;
    if (qlinear_dev(ds->main_proj, mh, ds->mxa.as<float>(), rows, ds->pq.as<uint8_t>(), ds->ps.as<float>(), true, st)) return 1;
    return rms_norm(ds->mxa.as<float>(), ds->main_norm_w, m->norm_eps, ds->mx.as<float>(), m->dim, rows, st);
}
// every stage's ring rows of positions pos0 .. pos0 + rows - 1 from ds->mx (c/dspark.h:378-455)
static int ds_ring_rows(ApusCudaDspark *ds, int rows, long long pos0, cudaStream_t st) {
    ApusCudaModel *m = ds->m;
    if (act_quant(ds->mx.as<float>(), nullptr, rows, m->dim, ds->pq.as<uint8_t>(), ds->ps.as<float>(), nullptr, st)) return 1;
    for (int k = 0; k < ds->n_stages; k++) {
        const LayerDev &L = ds->stages[k];
        const ApusAttnCfg &c = L.attn.cfg;
        APUS_REQUIRE(pos0 + rows <= L.rope_rows, "dspark: position %lld is beyond the rope table", pos0 + rows - 1);
        if (qgemm_dev(L.attn.wkv, nullptr, ds->pq.as<uint8_t>(), ds->ps.as<float>(), rows, ds->kva.as<float>(), true, 0.f, st)) return 1;
        if (row_ops(ds->kva.as<float>(), c.head_dim, ds->kv.as<float>(), c.head_dim, rows, c.head_dim,
                    ROW_RMS_W | ROW_ROPE | ROW_FP8QAT | ROW_BF16_OUT, L.attn.kv_norm, c.eps, c.rope_dim,
                    L.cs + (size_t)pos0 * c.rope_dim, 1, c.rope_dim, st))
            return 1;
        if (ring_update(ds->states[k].win.as<float>(), ds->kv.as<float>(), c.window, rows, c.head_dim, 1, pos0, st)) return 1;
    }
    return 0;
}

// c/dspark.h:459-575: the B draft rows through one stage's attention
static int ds_attn(ApusCudaDspark *ds, int k, const float *x, long long start_pos, float *out, cudaStream_t st) {
    const LayerDev &L = ds->stages[k];
    const AttnDev &A = L.attn;
    const ApusAttnCfg &c = A.cfg;
    const StepBufs &b = ds->sb;
    const int B = ds->B, h = c.n_heads, d = c.head_dim, rd = c.rope_dim, win = c.window, hd = h * d;
    const float *cs1 = L.cs + (size_t)(start_pos + 1) * rd;            // draft row t rotates at start_pos + 1 + t
    if (act_quant(x, nullptr, B, c.dim, b.xq, b.xs, nullptr, st)) return 1;
    if (qgemm_dev(A.wq_a, nullptr, b.xq, b.xs, B, b.qa, true, 0.f, st)) return 1;
    if (row_ops(b.qa, c.q_lora, b.qr, c.q_lora, B, c.q_lora, ROW_RMS_W, A.q_norm, c.eps, 0, nullptr, 1, 0, st, nullptr, b.xq2,
                b.xs2))
        return 1;
    if (qgemm_dev(A.wq_b, nullptr, b.xq2, b.xs2, B, b.q, true, 0.f, st)) return 1;
    if (row_ops(b.q, d, b.q, d, B * h, d, ROW_RMS_PLAIN | ROW_ROPE, nullptr, c.eps, rd, cs1, h, rd, st)) return 1;
    // the draft rows' own KV: after the ring in the candidate list, never written into it
    if (qgemm_dev(A.wkv, nullptr, b.xq, b.xs, B, b.kva, true, 0.f, st)) return 1;
    if (row_ops(b.kva, d, b.kv, d, B, d, ROW_RMS_W | ROW_ROPE | ROW_FP8QAT | ROW_BF16_OUT, A.kv_norm, c.eps, rd, cs1, 1, rd, st))
        return 1;
    const int nwin = (int)(start_pos + 1 < win ? start_pos + 1 : win), idxw = nwin + B;
    const float scale = (float)pow((double)d, -0.5);
    if (sparse_attn(b.q, A.sink, h, d, ds->idxs.as<int32_t>(), idxw, B, scale, ds->states[k].win.p, win, b.kv, B, 0, b.o, st, 0, 0,
                    b.sa, b.sa_cap))
        return 1;
    if (row_ops(b.o, d, b.o, d, B * h, d, ROW_ROPE_INV, nullptr, 0.f, rd, cs1, h, rd, st)) return 1;
    const int G = c.o_groups, ol = c.o_lora, sub = hd / G;
    if (f32_linear_batched(A.wo_a, (long long)ol * sub, b.o, sub, hd, b.y, ol, G * ol, G, B, sub, ol,
                           APUS_CUDA_W_BF16 | APUS_CUDA_R_OUT | APUS_LIN_CLASS(APUS_CUDA_TREE_WO_A), st))
        return 1;
    return qlinear_dev(A.wo_b, b.y, out, B, b.xq, b.xs, true, st);
}

// c/dspark.h:611-697 one draft round; mh_row (device) = main hidden of position start_pos.  Leaves the
// B drafts in ds->drafts (device, int64) and copies them to `drafts` (host).
static int ds_round(ApusCudaDspark *ds, long long anchor, const float *mh_row, long long start_pos, int64_t *drafts,
                    float *confidence, float *logits_final, float *stage_h, cudaStream_t st) {
    ApusCudaModel *m = ds->m;
    const int B = ds->B, dim = m->dim, hc = m->hc, V = m->vocab;
    APUS_REQUIRE(start_pos >= 0 && start_pos + 1 + B <= m->max_pos, "dspark: draft positions %lld + %d exceed max_pos %d",
                 start_pos + 1, B, m->max_pos);
    // ring slot of position start_pos in every stage (idempotent with the catch-up writes)
    if (ds_project(ds, mh_row, 1, st) || ds_ring_rows(ds, 1, start_pos, st)) return 1;
    const ApusAttnCfg &c0 = ds->stages[0].attn.cfg;
    const int win = c0.window, nwin = (int)(start_pos + 1 < win ? start_pos + 1 : win), idxw = nwin + B;
    std::vector<int64_t> ids((size_t)B, (int64_t)ds->noise_id);
    ids[0] = anchor;
    std::vector<int32_t> idx((size_t)B * idxw);
    for (int t = 0; t < B; t++) {                        // one shared, non-causal row: ring slots in slot order, then the draft rows
        for (int j = 0; j < nwin; j++) idx[(size_t)t * idxw + j] = j;
        for (int j = 0; j < B; j++) idx[(size_t)t * idxw + nwin + j] = win + j;
    }
    if (ds->ids.get((size_t)B * 8, nullptr) || ds->idxs.get((size_t)B * (win + B) * 4, nullptr) || ds->cur.get(8, nullptr) ||
        ds->drafts.get((size_t)B * 8, nullptr))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(ds->ids.p, ids.data(), (size_t)B * 8, cudaMemcpyHostToDevice, st));
    APUS_CUDA_OK(cudaMemcpyAsync(ds->idxs.p, idx.data(), idx.size() * 4, cudaMemcpyHostToDevice, st));
    APUS_CUDA_OK(cudaMemcpyAsync(ds->cur.p, &ids[0], 8, cudaMemcpyHostToDevice, st));
    float *h = ds->h0.as<float>(), *hn = ds->h1.as<float>();
    const BlockBufs bb = {ds->x.as<float>(), ds->y.as<float>(), ds->sub.as<float>(), ds->post.as<float>(), ds->comb.as<float>(),
                          ds->raw.as<float>()};
    if (embed_rows(m->embed, m->embed_bf16, ds->ids.as<int64_t>(), B, hc, dim, h, st)) return 1;
    for (int k = 0; k < ds->n_stages; k++) {
        const LayerDev &L = ds->stages[k];
        if (mhc_pre(h, dim, hc, L.hc_attn_fn, L.hc_attn_scale, L.hc_attn_base, m->norm_eps, m->hc_eps, m->iters, L.attn_norm_w,
                    m->norm_eps, nullptr, bb.post, bb.comb, bb.y, bb.x, B, st, bb.raw))
            return 1;
        if (ds_attn(ds, k, bb.x, start_pos, bb.sub, st)) return 1;
        if (block_ffn_post(L, bb.sub, &h, &hn, B, hc, bb, st)) return 1;
        if (block_ffn_pre(L, h, B, hc, m->iters, m->hc_eps, m->norm_eps, bb, st)) return 1;
        if (apus_cuda_moe_forward_dev(L.moe, bb.x, ds->ids.as<int64_t>(), B, bb.sub, st)) return 1;
        if (block_ffn_post(L, bb.sub, &h, &hn, B, hc, bb, st)) return 1;
        if (stage_h)
            APUS_CUDA_OK(cudaMemcpyAsync(stage_h + (size_t)k * B * hc * dim, h, (size_t)B * hc * dim * 4, cudaMemcpyDeviceToHost, st));
    }
    // head of the last stage, the parent's LM head, the bigram bias row by row
    if (mhc_head(h, dim, hc, ds->hc_head_fn, ds->hc_head_scale, ds->hc_head_base, m->norm_eps, m->hc_eps, ds->yh.as<float>(), B, st,
                 ds->raw.as<float>()))
        return 1;
    if (rms_norm(ds->yh.as<float>(), ds->norm_w, m->norm_eps, ds->yn.as<float>(), dim, B, st)) return 1;
    if (f32_linear(m->head, ds->yn.as<float>(), ds->logits.as<float>(), B, dim, V,
                   (m->head_bf16 ? APUS_CUDA_W_BF16 : 0) | APUS_LIN_CLASS(APUS_CUDA_TREE_HEAD), st))
        return 1;
    for (int i = 0; i < B; i++) {
        float *row = ds->logits.as<float>() + (size_t)i * V;
        launch_k(markov_bias_kernel, ceil_div(V, 256), 256, 0, st, ds->markov_w1, ds->markov_w2, ds->cur.as<long long>(), ds->rank, V,
                 row, ds->emb.as<float>() + (size_t)i * ds->rank);
        APUS_LAUNCHED();
        // the pick of the row: greedy, or one draw at the draft temperature with top_p 1 from the module's own
        // generator stream, one uniform per draft row (c/dspark.h:666-676)
        if (sample_rows(row, V, 1, ds->temp, 1.0f, nullptr, ds->drng.as<unsigned long long>(), ds->probs.as<float>(),
                        ds->tok.as<int32_t>(), st))
            return 1;
        launch_k(markov_take_kernel, 1, 1, 0, st, ds->tok.as<int32_t>(), ds->cur.as<long long>(), ds->drafts.as<long long>(), i);
        APUS_LAUNCHED();
    }
    if (confidence) {
        launch_k(confidence_kernel, B, 32, 0, st, ds->yh.as<float>(), ds->emb.as<float>(), ds->conf_proj, dim, ds->rank,
                 ds->conf.as<float>());
        APUS_LAUNCHED();
        APUS_CUDA_OK(cudaMemcpyAsync(confidence, ds->conf.p, (size_t)B * 4, cudaMemcpyDeviceToHost, st));
    }
    if (logits_final) APUS_CUDA_OK(cudaMemcpyAsync(logits_final, ds->logits.p, (size_t)B * V * 4, cudaMemcpyDeviceToHost, st));
    APUS_CUDA_OK(cudaMemcpyAsync(drafts, ds->drafts.p, (size_t)B * 8, cudaMemcpyDeviceToHost, st));
    APUS_CUDA_OK(cudaStreamSynchronize(st));
    return 0;
}

void apus_cuda_dspark_destroy(ApusCudaDspark *ds) {
    if (!ds) return;
    cudaDeviceSynchronize();
    ds->release();
    delete ds;
}

// c/dspark.h:702-711 (apus_dspec_init): the temperature of the draft picks and the seed of the stream they are
// drawn from -- a splitmix64 stream of its own (c/sample.h:159-170), advanced by one draw per draft row and
// never rolled back.  temp <= 0: greedy drafts.
int apus_cuda_dspark_set_sampling(ApusCudaDspark *ds, float temp, uint64_t draft_seed) {
    if (!ds) { set_error("NULL dspark"); return 1; }
    cudaStream_t st = mstream(ds->m);
    ds->temp = temp > 0.f ? temp : 0.f;
    if (ds->drng.get(8, nullptr) || ds->probs.get((size_t)ds->m->vocab * 4, nullptr)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(ds->drng.p, &draft_seed, 8, cudaMemcpyHostToDevice, st));
    APUS_CUDA_OK(cudaStreamSynchronize(st));
    return 0;
}

// c/dspark.h:353-356: fresh (empty) stage rings
int apus_cuda_dspark_reset(ApusCudaDspark *ds) {
    if (!ds) { set_error("NULL dspark"); return 1; }
    for (int k = 0; k < ds->n_stages; k++)
        if (attn_state_init(ds->stages[k].attn.cfg, ds->states[k], 1, 0)) return 1;
    APUS_CUDA_OK(cudaStreamSynchronize(ctx().stream));
    return 0;
}

ApusCudaDspark *apus_cuda_dspark_create(ApusCudaModel *m, const ApusCudaDsparkDesc *d) {
    if (!m || !d || !d->stages) { set_error("dspark_create: NULL argument"); return nullptr; }
    const int dim = m->dim, hc = m->hc, V = m->vocab;
    if (m->B != 1 || m->e_lo != 0 || m->e_hi != m->n_experts) { set_error("dspark_create: needs a one-sequence model that holds every expert"); return nullptr; }
    if (d->n_stages < 1 || d->n_stages > 8 || d->block_size < 1 || d->block_size > 32 || d->n_targets < 1 || d->n_targets > 8 ||
        d->noise_id < 0 || d->noise_id >= V || d->markov_rank < 1) {
        set_error("dspark: bad config (stages %d, block %d, targets %d, noise %d, rank %d)", d->n_stages, d->block_size,
                  d->n_targets, d->noise_id, d->markov_rank);
        return nullptr;
    }
    for (int i = 0; i < d->n_targets; i++)
        if (d->targets[i] < 0 || d->targets[i] >= m->n_layers) { set_error("dspark: target layer %d out of range", d->targets[i]); return nullptr; }
    if (d->main_proj.O != dim || d->main_proj.K != (int64_t)d->n_targets * dim) { set_error("dspark: bad tensor main_proj"); return nullptr; }
    ApusCudaDspark *ds = new ApusCudaDspark();
    ds->m = m;
    ds->n_stages = d->n_stages; ds->B = d->block_size; ds->noise_id = d->noise_id; ds->rank = d->markov_rank;
    ds->n_targets = d->n_targets;
    for (int i = 0; i < d->n_targets; i++) ds->targets[i] = d->targets[i];
    ds->stages.resize(d->n_stages);
    ds->states.resize(d->n_stages);
    bool ok = true;
    for (int k = 0; k < d->n_stages && ok; k++) {
        const ApusCudaLayerDesc &ld = d->stages[k];
        if (ld.acfg.ratio != 0 || ld.mw.hash || ld.acfg.dim != dim) { set_error("dspark: stage %d must be a sliding-window block with scored routing", k); ok = false; break; }
        ok = layer_weights(ld, hc, V, &ds->stages[k], &ds->own, 0, -1) == 0;
        if (!ok) break;
        ds->stages[k].cs = rope_rows_dev(ld.cos, ld.sin, ld.rope_rows, ld.acfg.rope_dim / 2, m->rope);
        ds->stages[k].rope_rows = ld.rope_rows;
        if (!ds->stages[k].cs || ld.rope_rows < m->max_pos) { set_error("dspark: stage %d rope table has %d rows, %d needed", k, ld.rope_rows, m->max_pos); ok = false; }
    }
    if (ok) {
        const size_t B = ds->B;
        ds->main_proj = get_qw(&ds->own, 8, d->main_proj.codes, d->main_proj.scales, dim, d->n_targets * dim);
        ds->main_norm_w = (const float *)get_dense(&ds->own, d->main_norm_w, (size_t)dim * 4);
        ds->norm_w = (const float *)get_dense(&ds->own, d->norm_w, (size_t)dim * 4);
        ds->hc_head_fn = (const float *)get_dense(&ds->own, d->hc_head_fn, (size_t)hc * hc * dim * 4);
        ds->hc_head_base = (const float *)get_dense(&ds->own, d->hc_head_base, (size_t)hc * 4);
        ds->hc_head_scale = d->hc_head_scale;
        ds->markov_w1 = (const float *)get_dense(&ds->own, d->markov_w1, (size_t)V * d->markov_rank * 4);
        ds->markov_w2 = (const float *)get_dense(&ds->own, d->markov_w2, (size_t)V * d->markov_rank * 4);
        ds->conf_proj = (const float *)get_dense(&ds->own, d->conf_proj, (size_t)(dim + d->markov_rank) * 4);
        ok = ds->main_proj && ds->main_norm_w && ds->norm_w && ds->hc_head_fn && ds->hc_head_base && ds->markov_w1 && ds->markov_w2 &&
             ds->conf_proj;
        const ApusAttnCfg &c = ds->stages[0].attn.cfg;
        ApusAttnCfg sized = c;
        sized.has_indexer = 0;
        const long long wide = B + 8;
        ok = ok && !(ds->h0.get(B * hc * dim * 4, nullptr) || ds->h1.get(B * hc * dim * 4, nullptr) || ds->x.get(B * dim * 4, nullptr) ||
                     ds->y.get(B * dim * 4, nullptr) || ds->sub.get(B * dim * 4, nullptr) || ds->post.get(B * hc * 4, nullptr) ||
                     ds->comb.get(B * hc * hc * 4, nullptr) || ds->raw.get(B * ((2 + hc) * hc + 1) * 4, nullptr) ||
                     ds->yh.get(B * dim * 4, nullptr) || ds->yn.get(B * dim * 4, nullptr) || ds->logits.get(B * (size_t)V * 4, nullptr) ||
                     ds->emb.get(B * d->markov_rank * 4, nullptr) || ds->tok.get(4, nullptr) || ds->conf.get(B * 4, nullptr) ||
                     attn_step_bufs(sized, wide, (int)B, ds->ws, &ds->sb));
        if (ok) {
            ds->sb.sa_cap = sparse_attn_scratch(c.n_heads, (int)(c.window + wide + 8), (int)B);
            ok = ds->sa.get(ds->sb.sa_cap, &ds->sb.sa) == 0;
        }
    }
    if (ok) ok = apus_cuda_dspark_reset(ds) == 0;
    if (!ok) { apus_cuda_dspark_destroy(ds); return nullptr; }
    return ds;
}

// c/dspark.h:397-434 (rows = the whole prompt from position 0) and 436-455 (catch-up from pos0): the
// stages' ring rows of n true positions from their main hiddens mh [n, n_targets * dim] (host).
int apus_cuda_dspark_feed(ApusCudaDspark *ds, const float *mh, int64_t pos0, int n) {
    if (!ds || !mh) { set_error("dspark_feed: NULL argument"); return 1; }
    if (n <= 0) return 0;
    ApusCudaModel *m = ds->m;
    cudaStream_t st = mstream(m);
    APUS_REQUIRE(pos0 >= 0 && pos0 + n <= m->max_pos, "dspark_feed: positions %lld + %d exceed max_pos %d", (long long)pos0, n, m->max_pos);
    const size_t mhd = (size_t)ds->n_targets * m->dim;
    if (ds_bufs(ds, n)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(ds->mh.p, mh, (size_t)n * mhd * 4, cudaMemcpyHostToDevice, st));
    if (ds_project(ds, ds->mh.as<float>(), n, st) || ds_ring_rows(ds, n, pos0, st)) return 1;
    APUS_CUDA_OK(cudaStreamSynchronize(st));
    return 0;
}

// c/dspark.h:611 apus_dspark_draft_round, greedy drafts: mh_row [n_targets * dim] (host) = main hidden of position
// start_pos; drafts [block_size]; confidence [block_size], logits_final [block_size, vocab], stage_h
// [n_stages, block_size, hc * dim] nullable.
int apus_cuda_dspark_draft_round(ApusCudaDspark *ds, int64_t anchor, const float *mh_row, int64_t start_pos, int64_t *drafts,
                                 float *confidence, float *logits_final, float *stage_h) {
    if (!ds || !mh_row || !drafts) { set_error("dspark_draft_round: NULL argument"); return 1; }
    ApusCudaModel *m = ds->m;
    cudaStream_t st = mstream(m);
    APUS_REQUIRE(anchor >= 0 && anchor < m->vocab, "dspark_draft_round: anchor %lld is outside [0, %d)", (long long)anchor, m->vocab);
    if (ds_bufs(ds, 1)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(ds->mh.p, mh_row, (size_t)ds->n_targets * m->dim * 4, cudaMemcpyHostToDevice, st));
    if (ds_round(ds, anchor, ds->mh.as<float>(), start_pos, drafts, confidence, logits_final, stage_h, st)) return 1;
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "dspark_draft_round: a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
    return 0;
}

// c/dspark.h:747-862 apus_dspec_prefill + apus_dspec_step until n_gen tokens are out (greedy or sampled main
// stream; the drafts are greedy unless apus_cuda_dspark_set_sampling gave them a temperature).  stats [7]: emitted, batches, batch_tokens, refeed_tokens, offered,
// accepted, bonus_rounds.
int apus_cuda_model_spec_generate_dspark(ApusCudaModel *m, ApusCudaDspark *ds, const int64_t *prompt, int n_prompt, int n_gen,
                                         int32_t *out_tokens, uint64_t *stats) {
    if (!m || !ds || ds->m != m) { set_error("model_spec_generate_dspark: the draft module belongs to another model"); return 1; }
    APUS_REQUIRE(n_prompt >= 1 && n_gen >= 1, "model_spec_generate_dspark: bad sizes");
    APUS_REQUIRE(chunks_enabled() && n_prompt <= chunk_rows(), "model_spec_generate_dspark: a prompt of %d tokens does not fit one chunk",
                 n_prompt);
    enum { EMITTED, BATCHES, BATCH_TOKENS, REFEED_TOKENS, OFFERED, ACCEPTED, BONUS };
    uint64_t s7[7] = {0, 0, 0, 0, 0, 0, 0};
    cudaStream_t st = mstream(m);
    const int B = ds->B;
    const size_t mhd = (size_t)ds->n_targets * m->dim;
    if (apus_cuda_dspark_reset(ds)) return 1;
    int32_t pick = 0;
    // main prefill collecting the mean hiddens, the stage rings from them
    if (forward_ex(m, prompt, n_prompt, nullptr, 0, &pick, nullptr, nullptr, ds->targets, ds->n_targets, "model_spec_generate_dspark",
                   false, true))
        return 1;
    DevBuf mh_last;
    if (mh_last.get(mhd * 4, nullptr)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(mh_last.p, m->ck.mhx.as<float>() + (size_t)(n_prompt - 1) * mhd, mhd * 4, cudaMemcpyDeviceToDevice, st));
    if (ds_project(ds, m->ck.mhx.as<float>(), n_prompt, st) || ds_ring_rows(ds, n_prompt, 0, st)) { mh_last.release(); return 1; }
    long long f = n_prompt - 1;
    int64_t held = pick;
    std::vector<int64_t> drafts((size_t)B), batch((size_t)B + 1);
    std::vector<int32_t> picks((size_t)B + 1);
    ApusCudaSnap *snap = nullptr;
    int emitted = 0, rc = 0;
    while (emitted < n_gen && !rc) {
        int Be = B;
        if (f + 2 + Be > m->max_pos) Be = (int)(m->max_pos - f - 2);
        if (Be <= 0) { set_error("model_spec_generate_dspark: position %lld reaches max_pos %d", f, m->max_pos); rc = 1; break; }
        if (ds_round(ds, held, mh_last.as<float>(), f, drafts.data(), nullptr, nullptr, nullptr, st)) { rc = 1; break; }
        ApusCudaSnap *s2 = apus_cuda_model_snapshot(m, snap);
        if (!s2) { rc = 1; break; }
        snap = s2;
        batch[0] = held;
        for (int j = 1; j <= Be; j++) batch[j] = drafts[j - 1];
        if (forward_ex(m, batch.data(), Be + 1, nullptr, 1, picks.data(), nullptr, nullptr, ds->targets, ds->n_targets,
                       "model_spec_generate_dspark", false, true)) { rc = 1; break; }
        s7[BATCHES]++; s7[BATCH_TOKENS] += (uint64_t)(Be + 1);
        int a = 0;
        int64_t newheld = -1;
        if (emitted < n_gen) out_tokens[emitted++] = (int32_t)held;
        for (int j = 1; j <= Be; j++) {
            const int32_t mj = picks[j - 1];
            s7[OFFERED]++;
            if (drafts[j - 1] == mj) {
                a = j; s7[ACCEPTED]++;
                if (emitted < n_gen) out_tokens[emitted++] = mj;
            } else { newheld = mj; break; }
        }
        if (newheld < 0) { newheld = picks[Be]; s7[BONUS]++; }
        // the verify batch's mean hiddens outlive the re-feed: the next round's main hidden, the rings' new rows
        if (cudaMemcpyAsync(mh_last.p, m->ck.mhx.as<float>() + (size_t)a * mhd, mhd * 4, cudaMemcpyDeviceToDevice, st) != cudaSuccess ||
            ds_project(ds, m->ck.mhx.as<float>(), a + 1, st) || ds_ring_rows(ds, a + 1, f + 1, st)) { rc = 1; break; }
        if (a < Be) {
            if (apus_cuda_model_restore(m, snap) || apus_cuda_model_forward_all(m, batch.data(), a + 1, nullptr, picks.data())) { rc = 1; break; }
            s7[REFEED_TOKENS] += (uint64_t)(a + 1);
        }
        held = newheld;
        f += 1 + a;
    }
    s7[EMITTED] = (uint64_t)emitted;
    if (snap) apus_cuda_snap_free(snap);
    cudaStreamSynchronize(st);
    mh_last.release();
    if (stats) memcpy(stats, s7, sizeof s7);
    return rc;
}

// The proposer of the draft/verify loop below when it is the MTP head (c/mtp.h:441-470, 500-528, 600-612).
struct MtpProposer {
    ApusCudaMtp *mt;
    DevBuf ids1;                  // one draft token on the device
    // draft chain from the logits the last mtp_forward_dev left: d1 = their argmax; d_{i+1} = MTP(own hidden, d_i)
    int chain(long long start_pos, int64_t *drafts, int depth) {
        ApusCudaModel *m = mt->m;
        cudaStream_t st = mstream(m);
        int32_t tok = 0;
        if (ids1.get(8, nullptr)) return 1;
        for (int i = 0; i < depth; i++) {
            APUS_CUDA_OK(cudaMemcpyAsync(&tok, mt->tok.p, 4, cudaMemcpyDeviceToHost, st));
            APUS_CUDA_OK(cudaStreamSynchronize(st));
            drafts[i] = tok;
            if (i + 1 == depth || start_pos + i >= m->max_pos) { for (int j = i + 1; j < depth; j++) drafts[j] = tok; break; }
            const int64_t id = tok;
            APUS_CUDA_OK(cudaMemcpyAsync(ids1.p, &id, 8, cudaMemcpyHostToDevice, st));
            // the head's own hidden (copied out of its buffers first: the next call overwrites them)
            if (mt->hin.get((size_t)m->hc * m->dim * 4, nullptr)) return 1;
            APUS_CUDA_OK(cudaMemcpyAsync(mt->hin.p, mt->hlast.p, (size_t)m->hc * m->dim * 4, cudaMemcpyDeviceToDevice, st));
            if (mtp_forward_dev(mt, mt->hin.as<float>(), ids1.as<int64_t>(), 1, start_pos + i, st)) return 1;
        }
        return 0;
    }
    int snap(bool take) {
        return snap_layer(mt->block.attn.cfg, mt->state, mt->snap, (size_t)mt->m->B, take, mstream(mt->m));
    }
};

static int spec_loop(ApusCudaModel *m, const int64_t *prompt, int n_prompt, int n_gen, int depth, ApusCudaDraftFn draft,
                     void *draft_ctx, ApusCudaMtp *mt, int32_t *out_tokens, uint64_t *stats);

int apus_cuda_model_spec_generate_mtp(ApusCudaModel *m, ApusCudaMtp *mt, const int64_t *prompt, int n_prompt, int n_gen,
                                      int depth, int32_t *out_tokens, uint64_t *stats) {
    if (!m || !mt || mt->m != m) { set_error("model_spec_generate_mtp: the draft head belongs to another model"); return 1; }
    return spec_loop(m, prompt, n_prompt, n_gen, depth, nullptr, nullptr, mt, out_tokens, stats);
}

int apus_cuda_model_spec_generate(ApusCudaModel *m, const int64_t *prompt, int n_prompt, int n_gen, int depth,
                                  ApusCudaDraftFn draft, void *draft_ctx, int32_t *out_tokens, uint64_t *stats) {
    if (!m || !draft) { set_error("model_spec_generate: NULL argument"); return 1; }
    return spec_loop(m, prompt, n_prompt, n_gen, depth, draft, draft_ctx, nullptr, out_tokens, stats);
}

// c/mtp.h:472-616: prefill, then draft / verify / accept-walk / state fix-up per step.
static int spec_loop(ApusCudaModel *m, const int64_t *prompt, int n_prompt, int n_gen, int depth, ApusCudaDraftFn draft,
                     void *draft_ctx, ApusCudaMtp *mt, int32_t *out_tokens, uint64_t *stats) {
    APUS_REQUIRE(m->B == 1, "model_spec_generate: one sequence per model (batch %d given)", m->B);
    APUS_REQUIRE(n_prompt >= 1 && n_gen >= 1 && depth >= 1 && depth <= 64, "model_spec_generate: bad sizes");
    APUS_REQUIRE(!mt || chunks_enabled(), "model_spec_generate_mtp: needs the chunked forward (apus_cuda_set_prefill_chunk)");
    enum { EMITTED, BATCHES, BATCH_TOKENS, REFEED_TOKENS, OFFERED, ACCEPTED, D1_OFFERED, D1_HITS };
    uint64_t st8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    cudaStream_t st = mstream(m);
    const size_t hd = (size_t)m->hc * m->dim;
    int32_t pick = 0;
    std::vector<int64_t> drafts((size_t)depth), batch((size_t)depth);
    std::vector<int32_t> picks((size_t)depth);
    MtpProposer mp{mt, {}};
    DevBuf h_keep, ids_keep;                              // hiddens and ids of the rows the draft head replays
    if (mt) {
        // main prefill keeping every position's hidden, then the head over the true (hidden, id) pairs
        APUS_REQUIRE(n_prompt * m->B <= chunk_rows(), "model_spec_generate_mtp: a prompt of %d tokens does not fit one chunk", n_prompt);
        if (apus_cuda_mtp_reset(mt)) return 1;
        if (forward_ex(m, prompt, n_prompt, nullptr, 0, &pick, nullptr, nullptr, nullptr, 0, "model_spec_generate_mtp", true)) return 1;
        if (ids_keep.get((size_t)(n_prompt > depth ? n_prompt : depth) * 8, nullptr)) return 1;
        APUS_CUDA_OK(cudaMemcpyAsync(ids_keep.p, prompt, (size_t)n_prompt * 8, cudaMemcpyHostToDevice, st));
        if (mtp_forward_dev(mt, m->ck.hx.as<float>(), ids_keep.as<int64_t>(), n_prompt, 0, st)) return 1;
        if (mp.snap(true) || mp.chain(m->pos, drafts.data(), depth)) return 1;
    } else {
        if (apus_cuda_model_forward(m, prompt, n_prompt, nullptr, &pick)) return 1;
        draft(draft_ctx, m->pos, drafts.data(), depth);
    }
    int64_t held = pick, q = m->pos;
    ApusCudaSnap *snap = nullptr;
    int emitted = 0, rc = 0;
    while (emitted < n_gen && !rc) {
        int D = depth;
        if (q + D > m->max_pos) D = (int)(m->max_pos - q);
        if (D <= 0) { set_error("model_spec_generate: position %lld reaches max_pos %d", (long long)q, m->max_pos); rc = 1; break; }
        st8[D1_OFFERED]++;
        if (drafts[0] == held) st8[D1_HITS]++;
        ApusCudaSnap *s2 = apus_cuda_model_snapshot(m, snap);
        if (!s2) { rc = 1; break; }
        snap = s2;
        batch[0] = held;
        for (int j = 1; j < D; j++) batch[j] = drafts[j];
        // verify batch: one pass over the D positions, every row's pick (and hidden, for the draft head)
        if (mt ? forward_ex(m, batch.data(), D, nullptr, 1, picks.data(), nullptr, nullptr, nullptr, 0, "model_spec_generate_mtp", true)
               : apus_cuda_model_forward_all(m, batch.data(), D, nullptr, picks.data())) { rc = 1; break; }
        st8[BATCHES]++; st8[BATCH_TOKENS] += (uint64_t)D;
        int matched = 0;
        int64_t last = -1;
        if (emitted < n_gen) out_tokens[emitted++] = (int32_t)held;
        for (int j = 1; j < D; j++) {
            const int32_t x = picks[j - 1];
            st8[OFFERED]++;
            if (drafts[j] == x) {
                matched++; st8[ACCEPTED]++;
                if (emitted < n_gen) out_tokens[emitted++] = x;
            } else { last = x; break; }
        }
        if (last < 0) last = picks[D - 1];               // full match: the bonus token
        if (mt) {                                         // the verify batch's hiddens outlive the re-feed below
            if (h_keep.get((size_t)depth * hd * 4, nullptr)) { rc = 1; break; }
            if (cudaMemcpyAsync(h_keep.p, m->ck.hx.p, (size_t)(matched + 1) * hd * 4, cudaMemcpyDeviceToDevice, st) != cudaSuccess) { rc = 1; break; }
        }
        if (matched < D - 1) {                           // partial: roll back, feed the true prefix again
            if (apus_cuda_model_restore(m, snap) || apus_cuda_model_forward_all(m, batch.data(), matched + 1, nullptr, picks.data())) {
                rc = 1;
                break;
            }
            st8[REFEED_TOKENS] += (uint64_t)(matched + 1);
        }
        held = last;
        q += matched + 1;
        if (mt) {
            // the head's clean state (true pairs only), the newly accepted pairs in one pass, the next chain
            if (mp.snap(false)) { rc = 1; break; }
            if (cudaMemcpyAsync(ids_keep.p, batch.data(), (size_t)(matched + 1) * 8, cudaMemcpyHostToDevice, st) != cudaSuccess) { rc = 1; break; }
            if (mtp_forward_dev(mt, h_keep.as<float>(), ids_keep.as<int64_t>(), matched + 1, q - matched - 1, st) || mp.snap(true) ||
                mp.chain(q, drafts.data(), depth)) { rc = 1; break; }
        } else {
            draft(draft_ctx, q, drafts.data(), depth);
        }
    }
    st8[EMITTED] = (uint64_t)emitted;
    if (snap) apus_cuda_snap_free(snap);
    if (mt) cudaStreamSynchronize(st);
    h_keep.release(); ids_keep.release(); mp.ids1.release();
    if (stats) memcpy(stats, st8, sizeof st8);
    return rc;
}

// ---- one step in pieces (expert parallelism: the caller runs the MoE sublayer) ----------------
int apus_cuda_model_set_ids(ApusCudaModel *m, const int64_t *ids) {
    if (!m) { set_error("NULL model"); return 1; }
    APUS_CUDA_OK(cudaMemcpyAsync(m->ids.p, ids, (size_t)m->B * 8, cudaMemcpyDefault, mstream(m)));
    return 0;
}
int apus_cuda_model_begin_step(ApusCudaModel *m) {
    if (!m) { set_error("NULL model"); return 1; }
    APUS_REQUIRE(m->pos < m->max_pos, "model step: position %lld reaches max_pos %d", m->pos, m->max_pos);
    return model_embed(m, mstream(m));
}
int apus_cuda_model_attn_half(ApusCudaModel *m, int layer) {
    if (!m || layer < 0 || layer >= m->n_layers) { set_error("model_attn_half: bad layer"); return 1; }
    return block_attn_half(m->layers[layer], m->states[layer], &m->h_cur, &m->h_alt, m->B, m->pos, m->hc, m->iters,
                           m->hc_eps, m->norm_eps, model_bufs(m), m->sb, mstream(m), m->pos_dev.as<long long>());
}
const float *apus_cuda_model_ffn_input(ApusCudaModel *m, int layer) {
    if (!m || layer < 0 || layer >= m->n_layers) { set_error("model_ffn_input: bad layer"); return nullptr; }
    if (block_ffn_pre(m->layers[layer], m->h_cur, m->B, m->hc, m->iters, m->hc_eps, m->norm_eps, model_bufs(m),
                      mstream(m)))
        return nullptr;
    return m->x.as<float>();
}
int apus_cuda_model_ffn_output(ApusCudaModel *m, int layer, const float *sub) {
    if (!m || layer < 0 || layer >= m->n_layers) { set_error("model_ffn_output: bad layer"); return 1; }
    return block_ffn_post(m->layers[layer], sub, &m->h_cur, &m->h_alt, m->B, m->hc, model_bufs(m), mstream(m));
}
int apus_cuda_model_end_step(ApusCudaModel *m, int want_logits, int feed_back) {
    if (!m) { set_error("NULL model"); return 1; }
    cudaStream_t st = mstream(m);
    if (want_logits) {
        if (model_head(m, st)) return 1;
        if (feed_back)
            launch_k(next_ids_kernel, 1, 32, 0, st, m->tok.as<int32_t>(), m->ids.as<int64_t>(), nullptr, m->B, 0, 1);
    }
    launch_k(advance_pos_kernel, 1, 1, 0, st, m->pos_dev.as<long long>());
    APUS_LAUNCHED();
    return m->capturing ? 0 : model_host_advance(m);
}
/* While the caller records a step into a CUDA graph of its own (stream capture on
 * the stream given to apus_cuda_use_stream), the host-side position must not move:
 * capturing(1) before, capturing(0) after; then, after every replay of that graph,
 * note_step() moves the host-side position and entry counts like the step did on
 * the device. */
int apus_cuda_model_capturing(ApusCudaModel *m, int on) {
    if (!m) return 1;
    m->capturing = on != 0;
    return 0;
}
int apus_cuda_model_note_step(ApusCudaModel *m) {
    if (!m) { set_error("NULL model"); return 1; }
    APUS_REQUIRE(m->pos < m->max_pos, "model step: position %lld reaches max_pos %d", m->pos, m->max_pos);
    return model_host_advance(m);
}
const int64_t *apus_cuda_model_ids(ApusCudaModel *m) { return m ? m->ids.as<int64_t>() : nullptr; }
int apus_cuda_model_read(ApusCudaModel *m, float *logits, int32_t *next) {
    if (!m) { set_error("NULL model"); return 1; }
    cudaStream_t st = mstream(m);
    if (logits) APUS_CUDA_OK(cudaMemcpyAsync(logits, m->logits.p, (size_t)m->B * m->vocab * 4, cudaMemcpyDeviceToHost, st));
    if (next) APUS_CUDA_OK(cudaMemcpyAsync(next, m->tok.p, (size_t)m->B * 4, cudaMemcpyDeviceToHost, st));
    APUS_CUDA_OK(cudaStreamSynchronize(st));
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "model: a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
    return 0;
}

}  // extern "C"
