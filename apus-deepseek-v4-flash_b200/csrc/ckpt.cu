// Checkpoint directory -> host tensors: config.json (fixture and real schema),
// model.safetensors.index.json, safetensors shards read with pread (reference
// c/st.h, c/model.h:165-376, c/layer.h:145-330).  Host code only: nothing here
// touches the GPU, so it runs on machines without one.
//
// Differences from the reference's reader that do not change what is loaded:
// payloads are read straight into the caller's (or the layer's) buffer instead
// of being cached until close, a routed expert's six tensors come in with one
// read when the container keeps them adjacent, and the experts of a layer are
// read by several threads (APUS_IO_THREADS, default 8; pread is positional).
#include <errno.h>
#include <fcntl.h>
#include <math.h>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>
#include <memory>
#include <thread>
#include "ckpt.cuh"
#include "common.cuh"

namespace apus {

namespace {

// ---- a small JSON reader -----------------------------------------------------
struct JV {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<JV> arr;
    std::vector<std::pair<std::string, JV>> obj;      // insertion order kept
    const JV *get(const char *key) const {
        if (kind != OBJ) return nullptr;
        for (auto &kv : obj) if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool truthy() const {
        return kind == BOOL ? b : kind == NUM ? num != 0.0 : kind == STR ? !str.empty() : kind == ARR || kind == OBJ;
    }
};

struct JParser {
    const char *p, *end;
    std::string err;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool fail(const char *what) { if (err.empty()) err = what; return false; }
    static void utf8(std::string &s, unsigned cp) {
        if (cp < 0x80) s += (char)cp;
        else if (cp < 0x800) { s += (char)(0xC0 | (cp >> 6)); s += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { s += (char)(0xE0 | (cp >> 12)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
        else { s += (char)(0xF0 | (cp >> 18)); s += (char)(0x80 | ((cp >> 12) & 0x3F)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
    }
    bool hex4(unsigned *out) {
        if (end - p < 4) return fail("json: short \\u escape");
        unsigned v = 0;
        for (int i = 0; i < 4; i++) {
            char c = *p++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else return fail("json: bad \\u escape");
        }
        *out = v;
        return true;
    }
    bool string(std::string *s) {
        if (p >= end || *p != '"') return fail("json: string expected");
        p++;
        while (p < end && *p != '"') {
            if (*p != '\\') { *s += *p++; continue; }
            if (++p >= end) break;
            char c = *p++;
            switch (c) {
                case 'n': *s += '\n'; break; case 't': *s += '\t'; break; case 'r': *s += '\r'; break;
                case 'b': *s += '\b'; break; case 'f': *s += '\f'; break;
                case 'u': {
                    unsigned cp, lo;
                    if (!hex4(&cp)) return false;
                    if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                        p += 2;
                        if (!hex4(&lo)) return false;
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(*s, cp);
                    break;
                }
                default: *s += c;                     // \" \\ \/
            }
        }
        if (p >= end) return fail("json: unterminated string");
        p++;
        return true;
    }
    bool value(JV *v, int depth) {
        if (depth > 64) return fail("json: nesting too deep");
        ws();
        if (p >= end) return fail("json: unexpected end");
        if (*p == '{') {
            v->kind = JV::OBJ; p++; ws();
            if (p < end && *p == '}') { p++; return true; }
            for (;;) {
                ws();
                std::string key;
                if (!string(&key)) return false;
                ws();
                if (p >= end || *p != ':') return fail("json: ':' expected");
                p++;
                v->obj.emplace_back(std::move(key), JV());
                if (!value(&v->obj.back().second, depth + 1)) return false;
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == '}') { p++; return true; }
                return fail("json: ',' or '}' expected");
            }
        }
        if (*p == '[') {
            v->kind = JV::ARR; p++; ws();
            if (p < end && *p == ']') { p++; return true; }
            for (;;) {
                v->arr.emplace_back();
                if (!value(&v->arr.back(), depth + 1)) return false;
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == ']') { p++; return true; }
                return fail("json: ',' or ']' expected");
            }
        }
        if (*p == '"') { v->kind = JV::STR; return string(&v->str); }
        if (end - p >= 4 && !strncmp(p, "true", 4)) { v->kind = JV::BOOL; v->b = true; p += 4; return true; }
        if (end - p >= 5 && !strncmp(p, "false", 5)) { v->kind = JV::BOOL; v->b = false; p += 5; return true; }
        if (end - p >= 4 && !strncmp(p, "null", 4)) { v->kind = JV::NUL; p += 4; return true; }
        // number: copy the token so strtod cannot run past the buffer
        const char *q = p;
        while (q < end && (strchr("+-.eE", *q) || (*q >= '0' && *q <= '9'))) q++;
        if (q == p) return fail("json: unexpected character");
        std::string tok(p, q);
        char *stop = nullptr;
        v->num = strtod(tok.c_str(), &stop);
        if (!stop || *stop) return fail("json: bad number");
        v->kind = JV::NUM;
        p = q;
        return true;
    }
};

bool json_parse(const char *buf, size_t n, JV *out, std::string *err) {
    JParser ps{buf, buf + n, ""};
    if (!ps.value(out, 0)) { *err = ps.err; return false; }
    ps.ws();
    if (ps.p != ps.end) { *err = "json: trailing characters"; return false; }
    return true;
}

bool read_file(const std::string &path, std::string *out) {
    int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) return false;
    struct stat sb;
    if (fstat(fd, &sb)) { close(fd); return false; }
    out->resize((size_t)sb.st_size);
    size_t done = 0;
    while (done < out->size()) {
        ssize_t r = pread(fd, &(*out)[done], out->size() - done, (off_t)done);
        if (r <= 0) { close(fd); return false; }
        done += (size_t)r;
    }
    close(fd);
    return true;
}

std::string fmt(const char *f, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, f);
    vsnprintf(buf, sizeof buf, f, ap);
    va_end(ap);
    return buf;
}

int dtype_of(const std::string &s) {
    static const char *names[] = {"I8", "U8", "F8_E8M0", "F8_E4M3", "BF16", "F16", "F32", "I32", "I64"};
    for (int i = 0; i < 9; i++) if (s == names[i]) return i;
    return APUS_CUDA_ST_OTHER;
}

// ---- config (c/model.h:195-376) ----------------------------------------------
// k1: fixture key, k2: key of the real checkpoint's config.json
bool cfg_num(const JV &root, const char *k1, const char *k2, double *out) {
    const JV *v = k1 ? root.get(k1) : nullptr;
    if (!v && k2) v = root.get(k2);
    if (!v || v->kind != JV::NUM) return false;
    *out = v->num;
    return true;
}

// ds (nullable) [13]: the DSpark section -- block_size, noise_id, markov_rank, n_stages, n_targets, targets[8]
int parse_config(const std::string &path, ApusCudaCkptCfg *c, std::vector<int> *ratios, std::vector<int> *hash,
                 std::string *why, int *ds = nullptr) {
    std::string text, jerr;
    if (!read_file(path, &text)) { *why = fmt("json: cannot open %s", path.c_str()); return 1; }
    JV root;
    if (!json_parse(text.data(), text.size(), &root, &jerr) || root.kind != JV::OBJ) {
        *why = jerr.empty() ? "config: not a JSON object" : jerr;
        return 1;
    }
    memset(c, 0, sizeof *c);
    double v;
    int n_stages = 0;                                   // DSpark speculative stages
#define CK_NEED(field, type, k1, k2)                                                     \
    do {                                                                                 \
        if (!cfg_num(root, k1, k2, &v)) { *why = fmt("config: missing %s", k1); return 1; } \
        c->field = (type)v;                                                              \
    } while (0)
    const JV *dj = root.get("dspark");
    const bool dj_obj = dj && dj->kind == JV::OBJ;
    c->dspark = dj_obj || root.get("dspark_block_size") || root.get("dspark_noise_token_id") ||
                root.get("dspark_target_layer_ids") || root.get("dspark_markov_rank");
    CK_NEED(dim, int, "dim", "hidden_size");
    CK_NEED(n_heads, int, "n_heads", "num_attention_heads");
    CK_NEED(head_dim, int, "head_dim", "head_dim");
    CK_NEED(rope_head_dim, int, "rope_head_dim", "qk_rope_head_dim");
    CK_NEED(q_lora_rank, int, "q_lora_rank", "q_lora_rank");
    CK_NEED(o_groups, int, "o_groups", "o_groups");
    CK_NEED(o_lora_rank, int, "o_lora_rank", "o_lora_rank");
    CK_NEED(window_size, int, "window_size", "sliding_window");
    CK_NEED(moe_inter_dim, int, "moe_inter_dim", "moe_intermediate_size");
    CK_NEED(n_routed_experts, int, "n_routed_experts", "n_routed_experts");
    CK_NEED(n_activated_experts, int, "n_activated_experts", "num_experts_per_tok");
    CK_NEED(index_n_heads, int, "index_n_heads", "index_n_heads");
    CK_NEED(index_head_dim, int, "index_head_dim", "index_head_dim");
    CK_NEED(index_topk, int, "index_topk", "index_topk");
    CK_NEED(hc_mult, int, "hc_mult", "hc_mult");
    CK_NEED(hc_sinkhorn_iters, int, "hc_sinkhorn_iters", "hc_sinkhorn_iters");
    CK_NEED(vocab_size, int, "vocab_size", "vocab_size");
    CK_NEED(max_pos, int, "max_pos", "max_position_embeddings");
    // YaRN parameters: top level in the fixture schema, under rope_scaling in the real one
    if (cfg_num(root, "beta_fast", nullptr, &v)) c->beta_fast = (int)v;
    if (cfg_num(root, "beta_slow", nullptr, &v)) c->beta_slow = (int)v;
    if (cfg_num(root, "original_seq_len", nullptr, &v)) c->original_seq_len = (int)v;
    if (cfg_num(root, "rope_factor", nullptr, &v)) c->rope_factor = v;
    CK_NEED(hc_eps, float, "hc_eps", "hc_eps");
    CK_NEED(norm_eps, float, "norm_eps", "rms_norm_eps");
    CK_NEED(route_scale, float, "route_scale", "routed_scaling_factor");
    CK_NEED(swiglu_limit, float, "swiglu_limit", "swiglu_limit");
    CK_NEED(rope_theta, double, "rope_theta", "rope_theta");
    CK_NEED(compress_rope_theta, double, "compress_rope_theta", "compress_rope_theta");
#undef CK_NEED
    if (const JV *rs = root.get("rope_scaling")) {
        if (cfg_num(*rs, nullptr, "factor", &v)) c->rope_factor = v;
        // the reference assigns original_seq_len here when the key is ABSENT (it tests
        // its lookup for failure, c/model.h:258-259): v then still holds the factor, or 0
        if (!cfg_num(*rs, nullptr, "factor", &v)) v = 0.0;
        double o;
        if (!cfg_num(*rs, nullptr, "original_max_position_embeddings", &o)) c->original_seq_len = (int)v;
        if (cfg_num(*rs, nullptr, "beta_fast", &v)) c->beta_fast = (int)v;
        if (cfg_num(*rs, nullptr, "beta_slow", &v)) c->beta_slow = (int)v;
    }
    c->bos_id = cfg_num(root, "bos_token_id", nullptr, &v) ? (int)v : -1;
    c->eos_id = cfg_num(root, "eos_token_id", nullptr, &v) ? (int)v : -1;
    // layer schedule: the fixture's "layers" array, else compress_ratios + num_hash_layers
    const JV *layers = root.get("layers"), *cr = root.get("compress_ratios");
    if (layers && layers->kind == JV::ARR) {
        c->n_layers = (int)layers->arr.size();
        for (int i = 0; i < c->n_layers; i++) {
            const JV &L = layers->arr[i];
            const JV *r = L.get("compress_ratio"), *h = L.get("hash");
            if (!r || r->kind != JV::NUM) { *why = fmt("config: layers[%d].compress_ratio", i); return 1; }
            ratios->push_back((int)r->num);
            hash->push_back(h ? (int)h->truthy() : 0);
        }
        const JV *mj = root.get("mtp");
        if (mj && mj->kind == JV::ARR && !mj->arr.empty()) {
            const JV *r = mj->arr[0].get("compress_ratio"), *h = mj->arr[0].get("hash");
            c->n_mtp = (int)mj->arr.size();
            c->mtp_ratio = r && r->kind == JV::NUM ? (int)r->num : 0;
            c->mtp_hash = h ? (int)h->truthy() : 0;
        }
    } else if (cr && cr->kind == JV::ARR) {
        double nh = 0, nextn = 0, nhl = 0;
        const int ncr = (int)cr->arr.size();
        cfg_num(root, "num_hidden_layers", nullptr, &nh);
        cfg_num(root, "num_nextn_predict_layers", nullptr, &nextn);
        cfg_num(root, "num_hash_layers", nullptr, &nhl);
        // entries past num_hidden_layers belong to the speculative stages
        if ((int)nh > 0 && ncr < (int)nh) { *why = "config: num_hidden_layers != compress_ratios"; return 1; }
        c->n_layers = (int)nh > 0 ? (int)nh : ncr;
        if (c->dspark && (int)nh > 0) n_stages = ncr - (int)nh;      // the trailing ratios are the stages
        for (int i = 0; i < c->n_layers; i++) {
            ratios->push_back(cr->arr[i].kind == JV::NUM ? (int)cr->arr[i].num : 0);
            hash->push_back(i < (int)nhl);
        }
        if (!c->dspark && (int)nextn > 0 && ncr >= (int)nh + (int)nextn) {
            c->n_mtp = (int)nextn;
            c->mtp_ratio = cr->arr[(int)nh].kind == JV::NUM ? (int)cr->arr[(int)nh].num : 0;
            c->mtp_hash = 0;
        }
    } else {
        *why = "config: no layer schedule (layers|compress_ratios)";
        return 1;
    }
    // DSpark section (c/model.h:336-373): the fixture's nested "dspark" object or the
    // top-level dspark_* keys; an incomplete one is refused like the reference does
    if (c->dspark) {
        const JV &src = dj_obj ? *dj : root;
        int block = 0, rank = 0, targets = 0;
        if (cfg_num(src, nullptr, dj_obj ? "block_size" : "dspark_block_size", &v)) block = (int)v;
        if (cfg_num(src, nullptr, dj_obj ? "markov_rank" : "dspark_markov_rank", &v)) rank = (int)v;
        if (dj_obj && cfg_num(src, nullptr, "n_mtp_layers", &v)) n_stages = (int)v;
        const JV *tj = src.get(dj_obj ? "target_layer_ids" : "dspark_target_layer_ids");
        if (tj && tj->kind == JV::ARR) targets = (int)tj->arr.size() > 8 ? 8 : (int)tj->arr.size();
        if (ds) {
            int noise = 0;
            if (cfg_num(src, nullptr, dj_obj ? "noise_token_id" : "dspark_noise_token_id", &v)) noise = (int)v;
            ds[0] = block; ds[1] = noise; ds[2] = rank; ds[3] = n_stages; ds[4] = targets;
            for (int i = 0; i < targets; i++) ds[5 + i] = tj->arr[i].kind == JV::NUM ? (int)tj->arr[i].num : 0;
        }
        if (block <= 0 || n_stages <= 0 || targets <= 0 || rank <= 0) {
            *why = fmt("config: incomplete DSpark section (block_size %d, stages %d, targets %d, markov_rank %d)",
                       block, n_stages, targets, rank);
            return 1;
        }
    }
    return 0;
}

}  // namespace

// ---- rope tables (c/attn.h:247-281, class choice c/layer.h:145-166) -----------
int ckpt_rope(const ApusCudaCkptCfg &cfg, int ratio, int64_t rows, float *cos, float *sin) {
    const int dim = cfg.rope_head_dim, half = dim / 2;
    const double base = ratio ? cfg.compress_rope_theta : cfg.rope_theta;
    const int osl = ratio ? cfg.original_seq_len : 0;        // 0: no YaRN (sliding-window layers)
    std::vector<float> freqs(half);
    for (int j = 0; j < half; j++) freqs[j] = 1.0f / powf((float)base, (float)(2 * j) / (float)dim);
    if (osl > 0) {
        const double two_pi = 2.0 * M_PI;
        double low = floor(dim * log(osl / (cfg.beta_fast * two_pi)) / (2.0 * log(base)));
        double high = ceil(dim * log(osl / (cfg.beta_slow * two_pi)) / (2.0 * log(base)));
        if (low < 0) low = 0;
        if (high > dim - 1) high = dim - 1;
        if (low == high) high += 0.001;
        for (int j = 0; j < half; j++) {
            float ramp = (float)(((double)j - low) / (high - low));
            ramp = ramp < 0.0f ? 0.0f : ramp > 1.0f ? 1.0f : ramp;
            const float smooth = 1.0f - ramp;
            // two roundings per term, left to right, as the reference's f32 expression
            volatile float a = freqs[j] / (float)cfg.rope_factor;
            volatile float b = a * (1.0f - smooth);
            volatile float d = freqs[j] * smooth;
            freqs[j] = b + d;
        }
    }
    for (int64_t t = 0; t < rows; t++)
        for (int j = 0; j < half; j++) {
            const float ang = (float)t * freqs[j];
            cos[t * half + j] = cosf(ang);
            sin[t * half + j] = sinf(ang);
        }
    return 0;
}

namespace {

// the reference's e4m3 decode and BF16 rounding on the host (c/fp4.h:255-280)
inline float e4m3_host(uint8_t c) {
    const int e = (c >> 3) & 15, m = c & 7;
    const float v = e ? ldexpf((float)(8 + m), e - 10) : ldexpf((float)m, -9);
    return (c & 0x80) ? -v : v;
}
inline float ue8m0_host(uint8_t b) {
    const uint32_t bits = b == 0 ? 0x00400000u : (uint32_t)b << 23;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
inline uint16_t bf16_bits_host(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)(u >> 16);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

struct QView { const CkTensor *w, *s; int64_t O, K; };

// c/st.h:445-462: name.weight F8_E4M3 [O,K] + name.scale F8_E8M0 [O/128,K/128]
bool fp8_view(ApusCudaCkpt *c, const std::string &name, QView *q, std::string *why) {
    q->w = c->find(name + ".weight", why);
    q->s = q->w ? c->find(name + ".scale", why) : nullptr;
    if (!q->w || !q->s || q->w->dtype != APUS_CUDA_ST_F8_E4M3 || q->s->dtype != APUS_CUDA_ST_F8_E8M0 ||
        q->w->ndim != 2 || q->s->ndim != 2 || q->s->shape[0] * 128 != q->w->shape[0] ||
        q->s->shape[1] * 128 != q->w->shape[1])
        return false;
    q->O = q->w->shape[0]; q->K = q->w->shape[1];
    return true;
}
// c/st.h:464-481: name.weight I8 packed FP4 [O,K/2] + name.scale F8_E8M0 [O,K/32]
bool fp4_view(ApusCudaCkpt *c, const std::string &name, QView *q, std::string *why) {
    q->w = c->find(name + ".weight", why);
    q->s = q->w ? c->find(name + ".scale", why) : nullptr;
    if (!q->w || !q->s || q->w->dtype != APUS_CUDA_ST_I8 || q->s->dtype != APUS_CUDA_ST_F8_E8M0 ||
        q->w->ndim != 2 || q->s->ndim != 2 || q->w->shape[0] != q->s->shape[0] ||
        q->w->shape[1] * 2 != q->s->shape[1] * 32)
        return false;
    q->O = q->w->shape[0]; q->K = q->w->shape[1] * 2;
    return true;
}

int read_f32(ApusCudaCkpt *c, const CkTensor &t, float *out, std::string *why) {
    if (t.dtype == APUS_CUDA_ST_F32) return c->read(t, out, why);
    if (t.dtype != APUS_CUDA_ST_BF16) { *why = fmt("st: %s is neither F32 nor BF16", t.name.c_str()); return 1; }
    std::vector<uint16_t> h(t.nelem());
    if (c->read(t, h.data(), why)) return 1;
    for (size_t i = 0; i < h.size(); i++) {
        const uint32_t u = (uint32_t)h[i] << 16;
        memcpy(&out[i], &u, 4);
    }
    return 0;
}

// Experts [e_lo, e_hi) of a layer: the six tensors of each into one slab.
struct ExpertPlan { QView q[3]; uint64_t total; bool adjacent; uint64_t lo; int shard; };

bool plan_expert(ApusCudaCkpt *c, const std::string &px, int e, ExpertPlan *p, std::string *why) {
    static const char *wn[3] = {"w1", "w2", "w3"};
    uint64_t lo = ~0ull, hi = 0;
    p->total = 0; p->shard = -1; p->adjacent = true;
    for (int i = 0; i < 3; i++) {
        if (!fp4_view(c, px + fmt(".ffn.experts.%d.%s", e, wn[i]), &p->q[i], why)) {
            if (why->empty()) *why = px + fmt(" expert %d", e);
            return false;
        }
        for (const CkTensor *t : {p->q[i].w, p->q[i].s}) {
            if (p->shard < 0) p->shard = t->shard;
            if (t->shard != p->shard) p->adjacent = false;
            lo = t->off < lo ? t->off : lo;
            hi = t->off + t->nbytes > hi ? t->off + t->nbytes : hi;
            p->total += t->nbytes;
        }
    }
    p->lo = lo;
    if (hi - lo != p->total) p->adjacent = false;      // gaps or other tensors in between
    return true;
}

int read_expert(ApusCudaCkpt *c, const ExpertPlan &p, uint8_t *slab, ApusFp4W *w, std::string *why) {
    if (p.adjacent && c->read_at(p.shard, p.lo, slab, p.total, why)) return 1;
    uint64_t at = 0;
    for (int i = 0; i < 3; i++) {
        const CkTensor *ts[2] = {p.q[i].w, p.q[i].s};
        const uint8_t *ptr[2];
        for (int k = 0; k < 2; k++) {
            if (p.adjacent) ptr[k] = slab + (ts[k]->off - p.lo);
            else {
                if (c->read(*ts[k], slab + at, why)) return 1;
                ptr[k] = slab + at;
                at += ts[k]->nbytes;
            }
        }
        w[i].packed = ptr[0]; w[i].scales = ptr[1]; w[i].O = p.q[i].O; w[i].K = p.q[i].K;
    }
    return 0;
}

}  // namespace

// ---- one layer (c/layer.h:202-330) ---------------------------------------------
int ckpt_load_layer(ApusCudaCkpt *c, int layer, int e_lo, int e_hi, CkLayerHost *out, std::string *why) {
    return ckpt_load_layer_named(c, fmt("layers.%d", layer), c->ratios[layer], c->hash[layer], layer, e_lo, e_hi, out, why);
}

// c/layer.h:202 apus_layer_load_named: the block under any prefix ("layers.<i>", "mtp.<k>"), its kind given
int ckpt_load_layer_named(ApusCudaCkpt *c, const std::string &px, int ratio, int hash, int layer, int e_lo, int e_hi,
                          CkLayerHost *out, std::string *why) {
    const ApusCudaCkptCfg &cfg = c->cfg;
    const int dim = cfg.dim, h = cfg.n_heads, d = cfg.head_dim, ql = cfg.q_lora_rank, G = cfg.o_groups,
              ol = cfg.o_lora_rank, E = cfg.n_routed_experts, topk = cfg.n_activated_experts, hc = cfg.hc_mult,
              mix = (2 + hc) * hc, rd = cfg.rope_head_dim, idm = cfg.index_head_dim;
    ApusCudaLayerDesc &D = out->desc;
    memset(&D, 0, sizeof D);
    out->raw.clear(); out->f32.clear();
    out->raw.reserve(64); out->f32.reserve(64);

    auto fp8 = [&](const std::string &name, int64_t O, int64_t K, ApusFp8W *w) -> bool {
        QView q;
        if (!fp8_view(c, name, &q, why) || (O && (q.O != O || q.K != K))) return false;
        out->raw.emplace_back(q.w->nbytes);
        out->raw.emplace_back(q.s->nbytes);
        uint8_t *pw = out->raw[out->raw.size() - 2].data(), *psc = out->raw.back().data();
        if (c->read(*q.w, pw, why) || c->read(*q.s, psc, why)) return false;
        w->codes = pw; w->scales = psc; w->O = q.O; w->K = q.K;
        return true;
    };
    auto f32 = [&](const std::string &name, size_t n) -> const float * {
        const CkTensor *t = c->find(name, why);
        if (!t || (t->dtype != APUS_CUDA_ST_F32 && t->dtype != APUS_CUDA_ST_BF16) || t->nelem() != n) {
            *why = fmt("layer: bad tensor %s", name.c_str());
            return nullptr;
        }
        out->f32.emplace_back(n);
        if (read_f32(c, *t, out->f32.back().data(), why)) return nullptr;
        return out->f32.back().data();
    };
#define CK_F32(dst, name, n) do { if (!((dst) = f32(px + (name), (n)))) return 1; } while (0)

    if (!fp8(px + ".attn.wq_a", ql, dim, &D.aw.wq_a) || !fp8(px + ".attn.wq_b", (int64_t)h * d, ql, &D.aw.wq_b) ||
        !fp8(px + ".attn.wkv", d, dim, &D.aw.wkv) || !fp8(px + ".attn.wo_b", dim, (int64_t)G * ol, &D.aw.wo_b)) {
        *why = px + ": fp8 attn weights";
        return 1;
    }
    {   // wo_a: FP8 on disk, BF16 bits in use (dequantise, round)
        ApusFp8W wa;
        if (!fp8(px + ".attn.wo_a", (int64_t)G * ol, (int64_t)h * d / G, &wa)) { *why = px + ": wo_a"; return 1; }
        const size_t nbk = (size_t)(wa.K + 127) / 128;
        out->wo_a.resize((size_t)wa.O * wa.K);
        for (int64_t o = 0; o < wa.O; o++) {
            const uint8_t *codes = wa.codes + o * wa.K, *sc = wa.scales + (o / 128) * nbk;
            uint16_t *dst = out->wo_a.data() + o * wa.K;
            for (int64_t k = 0; k < wa.K; k++) dst[k] = bf16_bits_host(e4m3_host(codes[k]) * ue8m0_host(sc[k / 128]));
        }
        out->raw.pop_back(); out->raw.pop_back();         // the FP8 form is not kept
        D.aw.wo_a = out->wo_a.data();
    }
    CK_F32(D.aw.q_norm, ".attn.q_norm.weight", (size_t)ql);
    CK_F32(D.aw.kv_norm, ".attn.kv_norm.weight", (size_t)d);
    CK_F32(D.aw.sink, ".attn.attn_sink", (size_t)h);
    CK_F32(D.attn_norm_w, ".attn_norm.weight", (size_t)dim);
    CK_F32(D.ffn_norm_w, ".ffn_norm.weight", (size_t)dim);
    if (ratio) {
        const int coff = ratio == 4 ? 2 : 1;
        ApusCompW &cw = D.aw.comp;
        CK_F32(cw.wkv, ".attn.compressor.wkv.weight", (size_t)coff * d * dim);
        CK_F32(cw.wgate, ".attn.compressor.wgate.weight", (size_t)coff * d * dim);
        CK_F32(cw.ape, ".attn.compressor.ape", (size_t)ratio * coff * d);
        CK_F32(cw.norm, ".attn.compressor.norm.weight", (size_t)d);
        cw.ratio = ratio; cw.overlap = ratio == 4; cw.d = d; cw.rd = rd; cw.rotate = 0; cw.eps = cfg.norm_eps;
        if (ratio == 4) {
            if (!fp8(px + ".attn.indexer.wq_b", (int64_t)cfg.index_n_heads * idm, ql, &D.aw.idx_wq_b)) {
                *why = px + ": indexer wq_b";
                return 1;
            }
            ApusCompW &ic = D.aw.idx_comp;
            CK_F32(D.aw.idx_wproj, ".attn.indexer.weights_proj.weight", (size_t)cfg.index_n_heads * dim);
            CK_F32(ic.wkv, ".attn.indexer.compressor.wkv.weight", (size_t)2 * idm * dim);
            CK_F32(ic.wgate, ".attn.indexer.compressor.wgate.weight", (size_t)2 * idm * dim);
            CK_F32(ic.ape, ".attn.indexer.compressor.ape", (size_t)ratio * 2 * idm);
            CK_F32(ic.norm, ".attn.indexer.compressor.norm.weight", (size_t)idm);
            ic.ratio = ratio; ic.overlap = 1; ic.d = idm; ic.rd = rd; ic.rotate = 1; ic.eps = cfg.norm_eps;
        }
    }
    // MoE
    ApusMoeW &mw = D.mw;
    CK_F32(mw.gate_w, ".ffn.gate.weight", (size_t)E * dim);
    if (hash) {
        const CkTensor *t = c->find(px + ".ffn.gate.tid2eid", why);
        if (!t || t->dtype != APUS_CUDA_ST_I64 || t->nelem() != (uint64_t)cfg.vocab_size * topk) {
            *why = px + ": tid2eid";
            return 1;
        }
        out->tid2eid.resize(t->nelem());
        if (c->read(*t, out->tid2eid.data(), why)) return 1;
        mw.tid2eid = out->tid2eid.data();
    } else {
        CK_F32(mw.gate_bias, ".ffn.gate.bias", (size_t)E);
    }
    if (e_hi < 0 || e_hi > E) e_hi = E;
    if (e_lo < 0) e_lo = 0;
    out->w1.assign(E, ApusFp4W{nullptr, nullptr, 0, 0});
    out->w2 = out->w1; out->w3 = out->w1;
    {
        const int n = e_hi > e_lo ? e_hi - e_lo : 0;
        std::vector<ExpertPlan> plans(n);
        for (int i = 0; i < n; i++)                        // shard headers are parsed here, on this thread
            if (!plan_expert(c, px, e_lo + i, &plans[i], why)) return 1;
        const size_t base = out->raw.size();
        for (int i = 0; i < n; i++) out->raw.emplace_back(plans[i].total);
        const char *env = getenv("APUS_IO_THREADS");
        int nthr = env ? atoi(env) : 8;
        nthr = nthr < 1 ? 1 : nthr > n ? (n ? n : 1) : nthr;
        std::vector<std::string> errs(nthr);
        std::vector<int> rc(nthr, 0);
        auto work = [&](int tix) {
            for (int i = tix; i < n && !rc[tix]; i += nthr) {
                ApusFp4W w[3];
                rc[tix] = read_expert(c, plans[i], out->raw[base + i].data(), w, &errs[tix]);
                out->w1[e_lo + i] = w[0]; out->w2[e_lo + i] = w[1]; out->w3[e_lo + i] = w[2];
            }
        };
        std::vector<std::thread> pool;
        for (int t = 1; t < nthr; t++) pool.emplace_back(work, t);
        work(0);
        for (auto &t : pool) t.join();
        for (int t = 0; t < nthr; t++) if (rc[t]) { *why = errs[t]; return 1; }
    }
    if (!fp8(px + ".ffn.shared_experts.w1", cfg.moe_inter_dim, dim, &mw.sw1) ||
        !fp8(px + ".ffn.shared_experts.w2", dim, cfg.moe_inter_dim, &mw.sw2) ||
        !fp8(px + ".ffn.shared_experts.w3", cfg.moe_inter_dim, dim, &mw.sw3)) {
        *why = px + ": shared experts";
        return 1;
    }
    mw.E = E; mw.topk = topk; mw.inter = cfg.moe_inter_dim; mw.dim = dim; mw.hash = hash;
    mw.route_scale = cfg.route_scale; mw.limit = cfg.swiglu_limit;
    mw.w1 = out->w1.data(); mw.w2 = out->w2.data(); mw.w3 = out->w3.data();
    mw.layer_id = layer;
    // mHC (all F32)
    CK_F32(D.hc_attn_fn, ".hc_attn_fn", (size_t)mix * hc * dim);
    CK_F32(D.hc_attn_base, ".hc_attn_base", (size_t)mix);
    CK_F32(D.hc_attn_scale, ".hc_attn_scale", 3);
    CK_F32(D.hc_ffn_fn, ".hc_ffn_fn", (size_t)mix * hc * dim);
    CK_F32(D.hc_ffn_base, ".hc_ffn_base", (size_t)mix);
    CK_F32(D.hc_ffn_scale, ".hc_ffn_scale", 3);
#undef CK_F32
    ApusAttnCfg &a = D.acfg;
    a.dim = dim; a.n_heads = h; a.head_dim = d; a.rope_dim = rd; a.q_lora = ql; a.o_groups = G; a.o_lora = ol;
    a.window = cfg.window_size; a.ratio = ratio; a.has_indexer = ratio == 4;
    a.idx_heads = cfg.index_n_heads; a.idx_dim = idm; a.idx_topk = cfg.index_topk;
    a.eps = cfg.norm_eps; a.max_pos = cfg.max_pos;
    return 0;
}

}  // namespace apus

// ---- the checkpoint object ---------------------------------------------------------
using namespace apus;

ApusCudaCkpt::~ApusCudaCkpt() {
    for (auto &s : shards) if (s.fd >= 0) close(s.fd);
}

int ApusCudaCkpt::read_at(int shard, uint64_t off, void *dst, uint64_t n, std::string *why) {
    CkShard &s = shards[shard];
    uint64_t done = 0;
    while (done < n) {
        ssize_t r = pread(s.fd, (char *)dst + done, n - done, (off_t)(off + done));
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) { *why = fmt("st: short read in %s", s.file.c_str()); return 1; }
        done += (uint64_t)r;
    }
    reads++;
    read_bytes += n;
    return 0;
}

// Bytes per element of a safetensors dtype this reader knows; 0 = unknown (such tensors are
// listed but never read through a typed accessor).
static uint64_t dtype_size(int dt) {
    switch (dt) {
    case APUS_CUDA_ST_I8: case APUS_CUDA_ST_U8: case APUS_CUDA_ST_F8_E8M0: case APUS_CUDA_ST_F8_E4M3: return 1;
    case APUS_CUDA_ST_BF16: case APUS_CUDA_ST_F16: return 2;
    case APUS_CUDA_ST_F32: case APUS_CUDA_ST_I32: return 4;
    case APUS_CUDA_ST_I64: return 8;
    default: return 0;
    }
}

// Parses the header of a shard on first use (c/st.h:212-276).  Unlike the reference,
// which reads a payload into a buffer of the payload's own size, the loader here sizes
// its buffers from the shape, so a tensor whose data_offsets disagree with dtype x shape
// is rejected here (as are negative or overflowing shapes).
static int parse_shard_body(ApusCudaCkpt *c, int si, std::string *why) {
    CkShard &s = c->shards[si];
    const std::string path = c->wdir + "/" + s.file;
    s.fd = open(path.c_str(), O_RDONLY);
    if (s.fd < 0) { *why = fmt("st: cannot open %s", path.c_str()); return 1; }
    struct stat sb;
    if (fstat(s.fd, &sb)) { *why = fmt("st: stat failed %s", path.c_str()); return 1; }
    const uint64_t fsz = (uint64_t)sb.st_size;
    if (fsz < 8) { *why = fmt("st: %s too small", path.c_str()); return 1; }
    uint64_t hlen = 0;
    if (pread(s.fd, &hlen, 8, 0) != 8 || hlen > fsz - 8) { *why = fmt("st: bad header in %s", path.c_str()); return 1; }
    std::string hdr((size_t)hlen, '\0');
    uint64_t done = 0;
    while (done < hlen) {
        ssize_t r = pread(s.fd, &hdr[done], hlen - done, (off_t)(8 + done));
        if (r <= 0) { *why = fmt("st: header read failed %s", path.c_str()); return 1; }
        done += (uint64_t)r;
    }
    JV root;
    std::string jerr;
    if (!json_parse(hdr.data(), hdr.size(), &root, &jerr) || root.kind != JV::OBJ) {
        *why = fmt("st: header JSON: %s", jerr.c_str());
        return 1;
    }
    const uint64_t data_base = 8 + hlen;
    for (auto &kv : root.obj) {
        if (kv.first == "__metadata__") continue;
        CkTensor t;
        t.name = kv.first;
        const JV *dt = kv.second.get("dtype"), *sh = kv.second.get("shape"), *off = kv.second.get("data_offsets");
        t.dtype = dtype_of(dt && dt->kind == JV::STR ? dt->str : "");
        uint64_t nelem = 1;
        if (sh && sh->kind == JV::ARR) {
            if (sh->arr.size() > 8) { *why = fmt("st: %s has more than 8 dimensions in %s", t.name.c_str(), path.c_str()); return 1; }
            t.ndim = (int)sh->arr.size();
            for (int d = 0; d < t.ndim; d++) {
                const double v = sh->arr[d].num;
                if (!(v >= 0) || v > 9.0e15 || v != (double)(int64_t)v) {
                    *why = fmt("st: bad shape of %s in %s", t.name.c_str(), path.c_str());
                    return 1;
                }
                t.shape[d] = (int64_t)v;
                if (t.shape[d] && nelem > (uint64_t)1 << 62) { *why = fmt("st: bad shape of %s in %s", t.name.c_str(), path.c_str()); return 1; }
                if (t.shape[d] && nelem > ((uint64_t)1 << 62) / (uint64_t)t.shape[d]) {
                    *why = fmt("st: bad shape of %s in %s", t.name.c_str(), path.c_str());
                    return 1;
                }
                nelem *= (uint64_t)t.shape[d];
            }
        }
        if (!off || off->kind != JV::ARR || off->arr.size() != 2) { *why = fmt("st: bad header in %s", path.c_str()); return 1; }
        const uint64_t a = (uint64_t)off->arr[0].num, b = (uint64_t)off->arr[1].num;
        if (b < a || data_base + b > fsz) { *why = fmt("st: tensor past EOF in %s", path.c_str()); return 1; }
        t.shard = si; t.off = data_base + a; t.nbytes = b - a;
        const uint64_t esz = dtype_size(t.dtype);
        if (esz && t.nbytes != nelem * esz) {
            *why = fmt("st: %s holds %llu bytes but its shape and dtype need %llu in %s", t.name.c_str(),
                       (unsigned long long)t.nbytes, (unsigned long long)(nelem * esz), path.c_str());
            return 1;
        }
        s.by_name[t.name] = (int)s.tensors.size();
        s.tensors.push_back(std::move(t));
    }
    s.parsed = true;
    return 0;
}
static int parse_shard(ApusCudaCkpt *c, int si, std::string *why) {
    CkShard &s = c->shards[si];
    if (s.parsed) return 0;
    if (parse_shard_body(c, si, why) == 0) return 0;
    if (s.fd >= 0) { close(s.fd); s.fd = -1; }          // leave nothing half-filled behind
    s.tensors.clear();
    s.by_name.clear();
    return 1;
}

const CkTensor *ApusCudaCkpt::find(const std::string &name, std::string *why) {
    auto it = shard_of.find(name);
    if (it == shard_of.end()) return nullptr;
    if (parse_shard(this, it->second, why)) return nullptr;
    CkShard &s = shards[it->second];
    auto jt = s.by_name.find(name);
    return jt == s.by_name.end() ? nullptr : &s.tensors[jt->second];
}

static void put_err(char *err, size_t cap, const std::string &msg) {
    if (err && cap) snprintf(err, cap, "%s", msg.c_str());
    apus::set_error("%s", msg.c_str());
}

extern "C" {

ApusCudaCkpt *apus_cuda_ckpt_open(const char *dir, char *err, size_t errcap) {
    if (!dir) { put_err(err, errcap, "ckpt_open: no directory"); return nullptr; }
    std::unique_ptr<ApusCudaCkpt> c(new ApusCudaCkpt());
    c->dir = dir;
    std::string why;
    int ds[13] = {0};
    if (parse_config(c->dir + "/config.json", &c->cfg, &c->ratios, &c->hash, &why, ds)) { put_err(err, errcap, why); return nullptr; }
    c->ds_block = ds[0]; c->ds_noise = ds[1]; c->ds_rank = ds[2]; c->ds_stages = ds[3]; c->ds_ntargets = ds[4];
    for (int i = 0; i < 8; i++) c->ds_targets[i] = ds[5 + i];
    // <dir>/model.safetensors.index.json, else <dir>/weights/...
    c->wdir = c->dir;
    std::string text;
    if (!read_file(c->wdir + "/model.safetensors.index.json", &text)) {
        c->wdir = c->dir + "/weights";
        if (!read_file(c->wdir + "/model.safetensors.index.json", &text)) {
            put_err(err, errcap, fmt("stset: json: cannot open %s/model.safetensors.index.json", c->wdir.c_str()));
            return nullptr;
        }
    }
    JV idx;
    if (!json_parse(text.data(), text.size(), &idx, &why)) { put_err(err, errcap, "stset: " + why); return nullptr; }
    const JV *wm = idx.get("weight_map");
    if (!wm || wm->kind != JV::OBJ) {
        put_err(err, errcap, fmt("stset: no weight_map in %s/model.safetensors.index.json", c->wdir.c_str()));
        return nullptr;
    }
    std::map<std::string, int> shard_ix;
    for (auto &kv : wm->obj) {
        if (kv.second.kind != JV::STR) continue;
        auto it = shard_ix.find(kv.second.str);
        if (it == shard_ix.end()) {
            it = shard_ix.emplace(kv.second.str, (int)c->shards.size()).first;
            c->shards.emplace_back();
            c->shards.back().file = kv.second.str;
        }
        c->shard_of[kv.first] = it->second;
    }
    return c.release();
}

void apus_cuda_ckpt_close(ApusCudaCkpt *c) { delete c; }

const ApusCudaCkptCfg *apus_cuda_ckpt_cfg(const ApusCudaCkpt *c) { return c ? &c->cfg : nullptr; }

int apus_cuda_ckpt_layer_kind(const ApusCudaCkpt *c, int layer, int *ratio, int *hash) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers) { set_error("ckpt_layer_kind: bad layer %d", layer); return 1; }
    if (ratio) *ratio = c->ratios[layer];
    if (hash) *hash = c->hash[layer];
    return 0;
}

int apus_cuda_ckpt_tensor(ApusCudaCkpt *c, const char *name, int *dtype, int *ndim, int64_t *shape, uint64_t *nbytes) {
    std::string why;
    const CkTensor *t = c && name ? c->find(name, &why) : nullptr;
    if (!t) { set_error("%s", why.empty() ? fmt("st: no tensor %s", name ? name : "(null)").c_str() : why.c_str()); return 1; }
    if (dtype) *dtype = t->dtype;
    if (ndim) *ndim = t->ndim;
    if (shape) memcpy(shape, t->shape, sizeof t->shape);
    if (nbytes) *nbytes = t->nbytes;
    return 0;
}

int apus_cuda_ckpt_read(ApusCudaCkpt *c, const char *name, void *dst, uint64_t nbytes) {
    std::string why;
    const CkTensor *t = c && name ? c->find(name, &why) : nullptr;
    if (!t) { set_error("%s", why.empty() ? fmt("st: no tensor %s", name ? name : "(null)").c_str() : why.c_str()); return 1; }
    if (t->nbytes != nbytes) { set_error("st: %s has %llu bytes, %llu asked", name, (unsigned long long)t->nbytes, (unsigned long long)nbytes); return 1; }
    if (c->read(*t, dst, &why)) { set_error("%s", why.c_str()); return 1; }
    return 0;
}

int apus_cuda_ckpt_read_f32(ApusCudaCkpt *c, const char *name, float *out, uint64_t n) {
    std::string why;
    const CkTensor *t = c && name ? c->find(name, &why) : nullptr;
    if (!t) { set_error("%s", why.empty() ? fmt("st: no tensor %s", name ? name : "(null)").c_str() : why.c_str()); return 1; }
    if (t->nelem() != n) { set_error("st: %s has %llu elements, %llu asked", name, (unsigned long long)t->nelem(), (unsigned long long)n); return 1; }
    if (read_f32(c, *t, out, &why)) { set_error("%s", why.c_str()); return 1; }
    return 0;
}

int apus_cuda_ckpt_wo_a(ApusCudaCkpt *c, int layer, uint16_t *out, uint64_t n) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers) { set_error("ckpt_wo_a: bad layer %d", layer); return 1; }
    std::string why;
    QView q;
    const std::string name = fmt("layers.%d.attn.wo_a", layer);
    if (!fp8_view(c, name, &q, &why) || (uint64_t)(q.O * q.K) != n) { set_error("layers.%d: wo_a", layer); return 1; }
    std::vector<uint8_t> codes(q.w->nbytes), sc(q.s->nbytes);
    if (c->read(*q.w, codes.data(), &why) || c->read(*q.s, sc.data(), &why)) { set_error("%s", why.c_str()); return 1; }
    const size_t nbk = (size_t)(q.K + 127) / 128;
    for (int64_t o = 0; o < q.O; o++)
        for (int64_t k = 0; k < q.K; k++)
            out[o * q.K + k] = bf16_bits_host(e4m3_host(codes[o * q.K + k]) * ue8m0_host(sc[(o / 128) * nbk + k / 128]));
    return 0;
}

int apus_cuda_ckpt_rope(const ApusCudaCkpt *c, int ratio, int64_t rows, float *cos, float *sin) {
    if (!c || rows < 0 || !cos || !sin) { set_error("ckpt_rope: bad arguments"); return 1; }
    return ckpt_rope(c->cfg, ratio, rows, cos, sin);
}

int apus_cuda_ckpt_expert(ApusCudaCkpt *c, int layer, int expert, void *slab, uint64_t cap, ApusFp4W *w1, ApusFp4W *w2,
                          ApusFp4W *w3) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers || expert < 0 || expert >= c->cfg.n_routed_experts) {
        set_error("ckpt_expert: bad layer %d / expert %d", layer, expert);
        return 1;
    }
    std::string why;
    ExpertPlan p;
    if (!plan_expert(c, fmt("layers.%d", layer), expert, &p, &why)) { set_error("%s", why.c_str()); return 1; }
    if (p.total > cap) { set_error("ckpt_expert: slab of %llu bytes needed", (unsigned long long)p.total); return 1; }
    ApusFp4W w[3];
    if (read_expert(c, p, (uint8_t *)slab, w, &why)) { set_error("%s", why.c_str()); return 1; }
    if (w1) *w1 = w[0];
    if (w2) *w2 = w[1];
    if (w3) *w3 = w[2];
    return 0;
}

int apus_cuda_ckpt_layer_digest(ApusCudaCkpt *c, int layer, int e_lo, int e_hi, uint64_t *digest, uint64_t *bytes) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers) { set_error("ckpt_layer_digest: bad layer %d", layer); return 1; }
    CkLayerHost L;
    std::string why;
    if (ckpt_load_layer(c, layer, e_lo, e_hi, &L, &why)) { set_error("%s", why.c_str()); return 1; }
    // FNV-1a over every tensor as the model would receive it, in descriptor order
    uint64_t h = 1469598103934665603ull, n = 0;
    auto eat = [&](const void *p, size_t len) {
        const unsigned char *b = (const unsigned char *)p;
        for (size_t i = 0; i < len; i++) { h ^= b[i]; h *= 1099511628211ull; }
        n += len;
    };
    const ApusCudaLayerDesc &D = L.desc;
    const ApusCudaCkptCfg &cf = c->cfg;
    auto q8 = [&](const ApusFp8W &w) { eat(w.codes, (size_t)w.O * w.K); eat(w.scales, (size_t)(w.O / 128) * (w.K / 128)); };
    q8(D.aw.wq_a); q8(D.aw.wq_b); q8(D.aw.wkv); q8(D.aw.wo_b);
    eat(D.aw.wo_a, L.wo_a.size() * 2);
    for (auto &v : L.f32) eat(v.data(), v.size() * 4);          // in load order (fixed for a layer kind)
    if (D.mw.tid2eid) eat(D.mw.tid2eid, L.tid2eid.size() * 8);
    for (int e = 0; e < cf.n_routed_experts; e++)
        for (const ApusFp4W *w : {&D.mw.w1[e], &D.mw.w2[e], &D.mw.w3[e]})
            if (w->packed) { eat(w->packed, (size_t)w->O * w->K / 2); eat(w->scales, (size_t)w->O * w->K / 32); }
    q8(D.mw.sw1); q8(D.mw.sw2); q8(D.mw.sw3);
    if (D.acfg.has_indexer) q8(D.aw.idx_wq_b);
    if (digest) *digest = h;
    if (bytes) *bytes = n;
    return 0;
}

uint64_t apus_cuda_ckpt_read_count(const ApusCudaCkpt *c) { return c ? c->reads.load() : 0; }
uint64_t apus_cuda_ckpt_read_bytes(const ApusCudaCkpt *c) { return c ? c->read_bytes.load() : 0; }


// ---- NDJSON serve loop (reference c/apus.c:451-662, `apus serve`) -------------------------------
// One JSON object per line in, one per line out; every response carries the request's "id" and a
// "type".  generate: {"id", "cmd":"generate", "ids":[...], "max_tokens", "temperature", "top_p",
// "seed"} -> {"type":"prompt","prompt_tokens"}, one {"type":"token","token_id"} per emitted token,
// {"type":"done","finish_reason","prompt_tokens","completion_tokens","text"}.  The reference's
// defaults and clamps are kept (max_tokens 32, temperature 1, top_p 1, seed 0; the prompt must be
// shorter than max_pos and the completion is cut to fit; the end-of-sequence token ends the
// completion with finish_reason "stop" and is not emitted).  The tokenizer is outside this library,
// so "text" / "messages" prompts and "encode" get the reference's "no tokenizer in model dir" error
// and tokens carry no text; a front end that speaks ids (the reference's tools/server.py does when
// the engine reports no tokenizer) works unchanged.
}  // extern "C"

namespace apus {
namespace {

void json_dump(const JV &v, std::string *o) {
    char buf[64];
    switch (v.kind) {
    case JV::NUL: *o += "null"; break;
    case JV::BOOL: *o += v.b ? "true" : "false"; break;
    case JV::NUM:
        if (v.num == (double)(long long)v.num && fabs(v.num) < 9e15) snprintf(buf, sizeof buf, "%lld", (long long)v.num);
        else snprintf(buf, sizeof buf, "%.17g", v.num);
        *o += buf;
        break;
    case JV::STR:
        *o += '"';
        for (unsigned char c : v.str) {
            if (c == '"' || c == '\\') { *o += '\\'; *o += (char)c; }
            else if (c == '\n') *o += "\\n";
            else if (c == '\r') *o += "\\r";
            else if (c == '\t') *o += "\\t";
            else if (c < 0x20) { snprintf(buf, sizeof buf, "\\u%04x", c); *o += buf; }
            else *o += (char)c;
        }
        *o += '"';
        break;
    case JV::ARR:
        *o += '[';
        for (size_t i = 0; i < v.arr.size(); i++) { if (i) *o += ','; json_dump(v.arr[i], o); }
        *o += ']';
        break;
    case JV::OBJ:
        *o += '{';
        for (size_t i = 0; i < v.obj.size(); i++) {
            if (i) *o += ',';
            JV k; k.kind = JV::STR; k.str = v.obj[i].first;
            json_dump(k, o); *o += ':'; json_dump(v.obj[i].second, o);
        }
        *o += '}';
        break;
    }
}

struct Serve {
    ApusCudaModel *m;
    int out_fd, eos, max_pos;
    // {"id":<id>,"type":"<type>"<rest>}\n, written in one piece
    void send(const JV *id, const char *type, const std::string &rest) {
        std::string s = "{\"id\":";
        if (id) json_dump(*id, &s); else s += "null";
        s += ",\"type\":\""; s += type; s += "\"" + rest + "}\n";
        size_t done = 0;
        while (done < s.size()) {
            ssize_t w = write(out_fd, s.data() + done, s.size() - done);
            if (w <= 0) return;
            done += (size_t)w;
        }
    }
    void error(const JV *id, const char *msg) {
        JV t; t.kind = JV::STR; t.str = msg;
        std::string r = ",\"message\":";
        json_dump(t, &r);
        send(id, "error", r);
    }
    void generate(const JV &req, const JV *id) {
        const JV *jids = req.get("ids");
        if (!jids || jids->kind != JV::ARR) {
            if ((req.get("text") && req.get("text")->kind == JV::STR) || req.get("messages")) error(id, "no tokenizer in model dir");
            else error(id, "generate needs messages, text, or ids");
            return;
        }
        std::vector<int64_t> ids;
        for (const JV &v : jids->arr) {
            if (v.kind != JV::NUM) { error(id, "ids must be an array of numbers"); return; }
            ids.push_back((int64_t)v.num);
        }
        if (ids.empty()) { error(id, "empty prompt"); return; }
        int max_tokens = 32;
        double temperature = 1.0, top_p = 1.0;
        uint64_t seed = 0;
        const JV *v;
        if ((v = req.get("max_tokens")) && v->kind == JV::NUM) max_tokens = (int)v->num;
        if (max_tokens < 0) max_tokens = 0;
        if ((v = req.get("temperature")) && v->kind == JV::NUM) temperature = v->num;
        if ((v = req.get("top_p")) && v->kind == JV::NUM) top_p = v->num;
        if ((v = req.get("seed")) && v->kind == JV::NUM) seed = (uint64_t)v->num;
        if ((int64_t)ids.size() >= max_pos) { error(id, "prompt too long for model max_pos"); return; }
        if ((int64_t)ids.size() + max_tokens > max_pos) max_tokens = (int)(max_pos - (int64_t)ids.size());
        char buf[96];
        snprintf(buf, sizeof buf, ",\"prompt_tokens\":%zu", ids.size());
        send(id, "prompt", buf);
        int completion = 0;
        const char *finish = "length";
        bool ok = apus_cuda_model_reset(m) == 0 && apus_cuda_model_set_sampling(m, (float)temperature, (float)top_p, seed) == 0;
        int32_t t = 0;
        // the pick after the prompt, then one step per emitted token (c/apus.c:541-585)
        if (ok && max_tokens > 0) ok = apus_cuda_model_forward(m, ids.data(), (int)ids.size(), nullptr, &t) == 0;
        for (int step = 0; ok && step < max_tokens; step++) {
            if (t == eos) { finish = "stop"; break; }
            completion++;
            snprintf(buf, sizeof buf, ",\"token_id\":%d", (int)t);
            send(id, "token", buf);
            if (step + 1 < max_tokens) {
                const int64_t next = t;
                ok = apus_cuda_model_forward(m, &next, 1, nullptr, &t) == 0;
            }
        }
        if (!ok) { error(id, apus_cuda_last_error()); return; }
        snprintf(buf, sizeof buf, "\",\"prompt_tokens\":%zu,\"completion_tokens\":%d,\"text\":\"\"", ids.size(), completion);
        send(id, "done", std::string(",\"finish_reason\":\"") + finish + buf);
    }
};

}  // namespace
}  // namespace apus

// ---- draft modules from the checkpoint directory (c/mtp.h:213-281, c/dspark.h:272-341) -------------
namespace apus {
namespace {

// Host copies of what a draft module adds to its blocks, alive until the module is created.
struct GlueHost {
    std::vector<std::vector<uint8_t>> raw;
    std::vector<std::vector<float>> f32;
    std::string why;
    bool fp8(ApusCudaCkpt *c, const std::string &name, int64_t O, int64_t K, ApusFp8W *w) {
        QView q;
        if (!fp8_view(c, name, &q, &why) || q.O != O || q.K != K) { why = "bad tensor " + name; return false; }
        raw.emplace_back(q.w->nbytes);
        raw.emplace_back(q.s->nbytes);
        uint8_t *pw = raw[raw.size() - 2].data(), *ps = raw.back().data();
        if (c->read(*q.w, pw, &why) || c->read(*q.s, ps, &why)) return false;
        w->codes = pw; w->scales = ps; w->O = q.O; w->K = q.K;
        return true;
    }
    const float *vec(ApusCudaCkpt *c, const std::string &name, size_t n, bool f32_only = false) {
        const CkTensor *t = c->find(name, &why);
        if (!t || t->nelem() != n || (f32_only ? t->dtype != APUS_CUDA_ST_F32
                                               : (t->dtype != APUS_CUDA_ST_F32 && t->dtype != APUS_CUDA_ST_BF16))) {
            why = "bad tensor " + name;
            return nullptr;
        }
        f32.emplace_back(n);
        if (read_f32(c, *t, f32.back().data(), &why)) return nullptr;
        return f32.back().data();
    }
};

// a draft block "mtp.<k>" with the rope table of its kind over max_pos rows
int load_draft_block(ApusCudaCkpt *c, int k, int ratio, int hash, int max_pos, CkLayerHost *L, std::vector<float> *cs,
                     std::string *why) {
    if (ckpt_load_layer_named(c, fmt("mtp.%d", k), ratio, hash, c->cfg.n_layers + k, 0, -1, L, why)) return 1;
    const size_t half = c->cfg.rope_head_dim / 2;
    cs[0].resize((size_t)max_pos * half); cs[1].resize((size_t)max_pos * half);
    ckpt_rope(c->cfg, ratio, max_pos, cs[0].data(), cs[1].data());
    L->desc.cos = cs[0].data(); L->desc.sin = cs[1].data(); L->desc.rope_rows = max_pos;
    L->desc.acfg.max_pos = max_pos;
    return 0;
}

}  // namespace
}  // namespace apus

extern "C" {

// c/mtp.h:213-281 apus_mtp_load: MTP block `idx` ("mtp.<idx>.*") of the checkpoint the model came from.
ApusCudaMtp *apus_cuda_mtp_load(ApusCudaModel *m, const char *dir, int idx) {
    int max_pos = 0;
    if (!m || apus_cuda_model_info(m, nullptr, &max_pos, nullptr, nullptr)) { set_error("mtp_load: NULL model"); return nullptr; }
    char err[512] = "";
    ApusCudaCkpt *c = apus_cuda_ckpt_open(dir, err, sizeof err);
    if (!c) { set_error("mtp_load: %s", err); return nullptr; }
    const ApusCudaCkptCfg &cfg = c->cfg;
    ApusCudaMtp *mt = nullptr;
    std::string why;
    do {
        if (idx < 0 || cfg.n_mtp <= idx) { why = fmt("mtp: model has no MTP block %d", idx); break; }
        CkLayerHost L;
        std::vector<float> cs[2];
        GlueHost g;
        if (load_draft_block(c, idx, cfg.mtp_ratio, cfg.mtp_hash, max_pos, &L, cs, &why)) break;
        const std::string px = fmt("mtp.%d", idx);
        const size_t dim = cfg.dim, hc = cfg.hc_mult;
        ApusCudaMtpDesc d;
        memset(&d, 0, sizeof d);
        d.block = L.desc;
        const float *scale = nullptr;
        if (!g.fp8(c, px + ".e_proj", dim, dim, &d.e_proj) || !g.fp8(c, px + ".h_proj", dim, dim, &d.h_proj) ||
            !(d.enorm_w = g.vec(c, px + ".enorm.weight", dim)) || !(d.hnorm_w = g.vec(c, px + ".hnorm.weight", dim)) ||
            !(d.norm_w = g.vec(c, px + ".norm.weight", dim)) || !(d.hc_head_fn = g.vec(c, px + ".hc_head_fn", hc * hc * dim, true)) ||
            !(d.hc_head_base = g.vec(c, px + ".hc_head_base", hc)) || !(scale = g.vec(c, px + ".hc_head_scale", 1))) {
            why = "mtp: " + g.why;
            break;
        }
        d.hc_head_scale = scale[0];
        mt = apus_cuda_mtp_create(m, &d);               // copies everything to HBM
        if (!mt) why = apus_cuda_last_error();
    } while (0);
    apus_cuda_ckpt_close(c);
    if (!mt) set_error("%s", why.c_str());
    return mt;
}

// c/dspark.h:272-341 apus_dspark_load: the DSpark stages "mtp.0 .. mtp.<n_stages-1>" and their glue.
ApusCudaDspark *apus_cuda_dspark_load(ApusCudaModel *m, const char *dir) {
    int max_pos = 0;
    if (!m || apus_cuda_model_info(m, nullptr, &max_pos, nullptr, nullptr)) { set_error("dspark_load: NULL model"); return nullptr; }
    char err[512] = "";
    ApusCudaCkpt *c = apus_cuda_ckpt_open(dir, err, sizeof err);
    if (!c) { set_error("dspark_load: %s", err); return nullptr; }
    const ApusCudaCkptCfg &cfg = c->cfg;
    ApusCudaDspark *ds = nullptr;
    std::string why;
    do {
        if (!cfg.dspark || c->ds_stages <= 0 || c->ds_stages > 8) { why = "dspark: model declares no DSpark stages"; break; }
        const int n = c->ds_stages, last = n - 1;
        std::vector<CkLayerHost> Ls((size_t)n);
        std::vector<std::vector<float>> cs((size_t)2 * n);
        bool ok = true;
        for (int k = 0; k < n && ok; k++) ok = load_draft_block(c, k, 0, 0, max_pos, &Ls[k], &cs[2 * k], &why) == 0;
        if (!ok) break;
        std::vector<ApusCudaLayerDesc> descs((size_t)n);
        for (int k = 0; k < n; k++) descs[k] = Ls[k].desc;
        GlueHost g;
        const size_t dim = cfg.dim, hc = cfg.hc_mult, V = cfg.vocab_size, rank = (size_t)c->ds_rank;
        ApusCudaDsparkDesc d;
        memset(&d, 0, sizeof d);
        d.n_stages = n; d.block_size = c->ds_block; d.noise_id = c->ds_noise; d.markov_rank = c->ds_rank;
        d.n_targets = c->ds_ntargets;
        for (int i = 0; i < 8; i++) d.targets[i] = c->ds_targets[i];
        d.stages = descs.data();
        const float *scale = nullptr;
        const std::string pl = fmt("mtp.%d", last);
        if (!g.fp8(c, "mtp.0.main_proj", dim, (int64_t)d.n_targets * dim, &d.main_proj) ||
            !(d.main_norm_w = g.vec(c, "mtp.0.main_norm.weight", dim)) || !(d.norm_w = g.vec(c, pl + ".norm.weight", dim)) ||
            !(d.hc_head_fn = g.vec(c, pl + ".hc_head_fn", hc * hc * dim, true)) || !(d.hc_head_base = g.vec(c, pl + ".hc_head_base", hc)) ||
            !(scale = g.vec(c, pl + ".hc_head_scale", 1)) ||
            !(d.markov_w1 = g.vec(c, pl + ".markov_head.markov_w1.weight", V * rank)) ||
            !(d.markov_w2 = g.vec(c, pl + ".markov_head.markov_w2.weight", V * rank)) ||
            !(d.conf_proj = g.vec(c, pl + ".confidence_head.proj.weight", dim + rank))) {
            why = "dspark: " + g.why;
            break;
        }
        d.hc_head_scale = scale[0];
        ds = apus_cuda_dspark_create(m, &d);
        if (!ds) why = apus_cuda_last_error();
    } while (0);
    apus_cuda_ckpt_close(c);
    if (!ds) set_error("%s", why.c_str());
    return ds;
}

}  // extern "C"

extern "C" int apus_cuda_serve(ApusCudaModel *m, int in_fd, int out_fd, int eos_id) {
    int batch = 0, max_pos = 0;
    if (apus_cuda_model_info(m, &batch, &max_pos, nullptr, nullptr)) return 1;
    APUS_REQUIRE(batch == 1, "serve: the model must hold one sequence (batch %d given)", batch);
    Serve sv = {m, out_fd, eos_id, max_pos};
    std::string pending;
    char chunk[4096];
    for (;;) {
        size_t nl;
        while ((nl = pending.find('\n')) == std::string::npos) {
            ssize_t r = read(in_fd, chunk, sizeof chunk);
            if (r <= 0) {                               // end of input: a last line without a newline still counts
                if (pending.empty()) return 0;
                pending += '\n';
                continue;
            }
            pending.append(chunk, (size_t)r);
        }
        std::string line = pending.substr(0, nl);
        pending.erase(0, nl + 1);
        if (line.find_first_not_of(" \t\r") == std::string::npos) continue;
        JV req;
        std::string perr;
        if (!json_parse(line.data(), line.size(), &req, &perr) || req.kind != JV::OBJ) {
            sv.error(nullptr, "bad request line (not a JSON object)");
            continue;
        }
        const JV *id = req.get("id"), *cmd = req.get("cmd");
        if (cmd && cmd->kind == JV::STR && cmd->str == "generate") sv.generate(req, id);
        else if (cmd && cmd->kind == JV::STR && cmd->str == "encode") sv.error(id, "no tokenizer in model dir");
        else sv.error(id, "unknown cmd (want encode|generate)");
    }
}
