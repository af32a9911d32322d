// Device-side attention engine shared by the host-pointer attention entry
// point and the device-resident model (api_attn.cu, api_model.cu).
#pragma once
#include "runtime.cuh"

namespace apus {

struct CompDev {
    const float *wkv = nullptr, *wgate = nullptr, *ape = nullptr, *norm = nullptr;
    int ratio = 0, overlap = 0, d = 0, rd = 0, rotate = 0;
    float eps = 0.f;
};
// Compressor state of B sequences in lockstep: carries [B][rows*cols], cache
// [B][cap][d]; nb entries valid in every sequence.
struct CompStateDev {
    DevBuf kv, sc, cache;
    int nb = 0, cap = 0;
    size_t carry = 0;         // rows*cols
};
struct AttnDev {
    ApusAttnCfg cfg;
    DevQW *wq_a, *wq_b, *wkv, *wo_b, *idx_wq_b;
    const uint16_t *wo_a;
    const float *q_norm, *kv_norm, *sink, *idx_wproj;
    CompDev comp, idx_comp;
};
struct StateDev {
    DevBuf win;               // [B][window][head_dim]
    CompStateDev comp, idx;
    int B = 1;
    void release();
};
struct StepBufs {
    float *qa, *qr, *q, *kva, *kv, *iq, *ckv, *csc, *pooled, *wt, *scores, *o, *y;
    uint8_t *xq;
    float *xs;
    int32_t *sel, *idxs;
    // second set for the chains that run beside the main one (see attn_step)
    uint8_t *xq2;
    float *xs2, *ckv2, *csc2, *pooled2;
    // sparse-attention scratch of the owner (NULL: the library's shared one)
    void *sa = nullptr;
    size_t sa_cap = 0;
    // chunks of positions only (attn_chunk): the position-ordered window rows [B][window + s][head_dim]
    float *ext = nullptr;
};

// Device copies that belong to one object (a model) instead of the global cache.
struct WeightOwner {
    std::vector<DevQW *> qws;
    std::vector<DevBuf *> bufs;
    void release();
};
DevQW *get_qw(WeightOwner *own, int fmt, const uint8_t *codes, const uint8_t *scales, int O, int K);
const void *get_dense(WeightOwner *own, const void *src, size_t bytes);
int attn_weights(const ApusAttnCfg *cfg, const ApusAttnW *w, AttnDev *A, WeightOwner *own = nullptr);
// Allocates (grows) and initialises the state of B sequences: zero ring and
// carries, score carries at -inf, caches of `cap` entries.
int attn_state_init(const ApusAttnCfg &c, StateDev &S, int B, int cap);
int attn_step_bufs(const ApusAttnCfg &c, long long max_nb, int B, DevBuf *ws, StepBufs *b);
// One token of B sequences in lockstep at position pos. x [B, dim] -> out [B, dim].
// pos_dev != NULL: the position is read on the device from *pos_dev and the rope
// rows from cs_table ([pos][cos | sin]); the launch sequence is then the same at
// every position, and the entry counts S.*.nb are left to the caller.
int attn_step(const AttnDev &A, StateDev &S, const float *x, long long pos, const float *cs_pos,
              const float *cs_rp, float *out, const StepBufs &b, int *idx_k_out, cudaStream_t st,
              const long long *pos_dev = nullptr, const float *cs_table = nullptr,
              bool x_codes = false);    // b.xq / b.xs already hold the activation codes of x

// A chunk of s consecutive positions of the B sequences in one pass (batched prefill, the
// s > 1 calls of reference c/attn.h:1514-1740): x, out [s * B, dim] with time-major rows
// (row = t * B + sequence), positions pos0 .. pos0 + s - 1, rope rows from cs_table.  `b` holds
// step buffers for s * B rows plus b.ext.  Every row goes through the operations of attn_step in
// the same order, so outputs and final state equal those of s consecutive steps bit for bit; the
// entry counts S.*.nb are advanced here.
int attn_chunk(const AttnDev &A, StateDev &S, const float *x, long long pos0, int s, const float *cs_table,
               float *out, const StepBufs &b, cudaStream_t st);

// Host-state exchange of the host-pointer tier (one sequence).
int attn_state_upload(const ApusAttnCfg &c, const ApusAttnS *st, StateDev &S, int extra, cudaStream_t sm);
int attn_state_download(const ApusAttnCfg &c, ApusAttnS *st, const StateDev &S, cudaStream_t sm);
void attn_state_commit(const ApusAttnCfg &c, ApusAttnS *st, const StateDev &S);

}  // namespace apus
