// C ABI, part 1: lifecycle, weight cache, kernel-level host-pointer entry points
// and the single-matrix device-resident entry points (include/apus_b200.h).
#include <stdarg.h>
#include <tuple>
#include <stdlib.h>

#include "runtime.cuh"

namespace apus {

// ---- errors / counters -----------------------------------------------------------
static thread_local char t_err[512] = "";
unsigned long long g_dispatches = 0;

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof t_err, fmt, ap);
    va_end(ap);
}

// ---- device buffers ------------------------------------------------------------------
// A buffer that grows moves: steps recorded into CUDA graphs hold the old address.  Every such move
// advances the epoch recorded steps are checked against (sum_order_epoch), so they are recorded again.
static unsigned long long g_buf_moves = 0;
int DevBuf::get(size_t bytes, void **out) {
    if (bytes > cap) {
        if (p) { cudaDeviceSynchronize(); cudaFree(p); p = nullptr; cap = 0; g_buf_moves++; }
        size_t want = bytes + (bytes >> 2) + 256;
        APUS_CUDA_OK(cudaMalloc(&p, want));
        cap = want;
    }
    if (out) *out = p;
    return 0;
}
void DevBuf::release() {
    if (p) cudaFree(p);
    p = nullptr; cap = 0;
}

size_t DevQW::bytes() const {
    if (fmt == 4) return (size_t)O * K / 2 + (size_t)O * K / 32;
    return (size_t)O * K + (size_t)((O + 127) / 128) * (K / 128);
}
void DevQW::release() {
    for (auto &kv : tables) cudaFree(kv.second);
    tables.clear();
    if (owned) { if (codes) cudaFree(codes); if (scales) cudaFree(scales); }
    else if (tc && scales) cudaFree(scales);        // adopted codes, own scale copy
    codes = scales = nullptr;
}

// Work-item table for M rows against this matrix (chunks of 32 rows), cached on
// the handle so that steady-state calls do no host->device copies.
int DevQW::table_for(int M, bool pair, const DevQW *other, GemmGroup **out, int *n_groups) {
    int n = ceil_div(M, 32);
    int key = M * 2 + (pair ? 1 : 0);
    auto it = tables.find(key);
    if (it == tables.end()) {
        std::vector<GemmGroup> h(n);
        for (int i = 0; i < n; i++) {
            h[i].wa = codes; h[i].sa = scales;
            h[i].wb = pair ? other->codes : nullptr;
            h[i].sb = pair ? other->scales : nullptr;
            h[i].row0 = i * 32;
            h[i].nrows = M - i * 32 < 32 ? M - i * 32 : 32;
        }
        GemmGroup *d = nullptr;
        APUS_CUDA_OK(cudaMalloc(&d, n * sizeof(GemmGroup)));
        APUS_CUDA_OK(cudaMemcpy(d, h.data(), n * sizeof(GemmGroup), cudaMemcpyHostToDevice));
        it = tables.emplace(key, d).first;
    }
    *out = it->second;
    *n_groups = n;
    return 0;
}

// ---- context ----------------------------------------------------------------------------
Ctx &ctx() {
    static Ctx c;
    return c;
}

int ensure_enabled() {
    Ctx &c = ctx();
    if (c.enabled) return 0;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        set_error("no CUDA device available (%s); this backend has no CPU fallback",
                  e == cudaSuccess ? "device count 0" : cudaGetErrorString(e));
        return 1;
    }
    APUS_CUDA_OK(cudaGetDevice(&c.device));
    cudaDeviceProp prop;
    APUS_CUDA_OK(cudaGetDeviceProperties(&prop, c.device));
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library is built for sm_100a only", c.device,
                  prop.major, prop.minor);
        return 1;
    }
    APUS_CUDA_OK(cudaStreamCreateWithFlags(&c.own_stream, cudaStreamNonBlocking));
    c.stream = c.own_stream;
    for (int i = 0; i < Ctx::N_AUX; i++) {
        APUS_CUDA_OK(cudaStreamCreateWithFlags(&c.aux[i], cudaStreamNonBlocking));
        APUS_CUDA_OK(cudaEventCreateWithFlags(&c.ev_fork[i], cudaEventDisableTiming));
        APUS_CUDA_OK(cudaEventCreateWithFlags(&c.ev_join[i], cudaEventDisableTiming));
    }
    c.enabled = true;
    return 0;
}

// which main chain each side stream is working for right now (set when a branch begins; enqueueing
// is host-sequential, so this is the chain whose launches are being issued)
static cudaStream_t g_aux_owner[Ctx::N_AUX] = {};
static bool g_aux_owned[Ctx::N_AUX] = {};    // the owner may be the default stream (a null handle)

cudaStream_t branch_begin(cudaStream_t main, int i) {
    Ctx &c = ctx();
    static const bool off = getenv("APUS_NO_BRANCH") && getenv("APUS_NO_BRANCH")[0] == '1';
    if (off || i < 0 || i >= Ctx::N_AUX) return main;
    if (cudaEventRecord(c.ev_fork[i], main) != cudaSuccess || cudaStreamWaitEvent(c.aux[i], c.ev_fork[i], 0) != cudaSuccess) {
        cudaGetLastError();
        return main;                            // no side stream: the chain simply runs in line
    }
    g_aux_owner[i] = main;
    g_aux_owned[i] = true;
    return c.aux[i];
}
int branch_end(int i, cudaStream_t main) {
    Ctx &c = ctx();
    static const bool off = getenv("APUS_NO_BRANCH") && getenv("APUS_NO_BRANCH")[0] == '1';
    if (off || i < 0 || i >= Ctx::N_AUX) return 0;
    APUS_CUDA_OK(cudaEventRecord(c.ev_join[i], c.aux[i]));
    APUS_CUDA_OK(cudaStreamWaitEvent(main, c.ev_join[i], 0));
    return 0;
}

// ---- uploads ----------------------------------------------------------------------------------
int upload_qw(int fmt, const uint8_t *codes, const uint8_t *scales, int O, int K,
              uint8_t *dst_codes, uint8_t *dst_scales, int *zero_scale) {
    Ctx &c = ctx();
    size_t cb = fmt == 4 ? (size_t)O * K / 2 : (size_t)O * K;
    size_t sb = fmt == 4 ? (size_t)O * K / 32 : (size_t)((O + 127) / 128) * ((K + 127) / 128);
    void *stg = nullptr;
    const size_t off_s = (cb + 255) & ~(size_t)255;
    if (c.stage.get(off_s + sb + 256, &stg)) return 1;
    uint8_t *sc = (uint8_t *)stg, *ss = sc + off_s;
    // the source may be host memory or (for weights generated or already resident
    // on the device) device memory; the copy kind is inferred from the pointer
    APUS_CUDA_OK(cudaMemcpyAsync(sc, codes, cb, cudaMemcpyDefault, c.stream));
    if (fmt == 4) {
        APUS_CUDA_OK(cudaMemcpyAsync(ss, scales, sb, cudaMemcpyDefault, c.stream));
        int *flag = nullptr;
        void *fp = nullptr;
        if (c.ws[15].get(256, &fp)) return 1;
        flag = (int *)fp;
        APUS_CUDA_OK(cudaMemsetAsync(flag, 0, sizeof(int), c.stream));
        if (repack_fp4(sc, ss, O, K, dst_codes, dst_scales, flag, c.stream)) return 1;
        int hz = 0;
        APUS_CUDA_OK(cudaMemcpyAsync(&hz, flag, sizeof(int), cudaMemcpyDeviceToHost, c.stream));
        APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
        if (zero_scale) *zero_scale = hz;
    } else {
        if (repack_fp8(sc, O, K, dst_codes, c.stream)) return 1;
        APUS_CUDA_OK(cudaMemcpyAsync(dst_scales, scales, sb, cudaMemcpyDefault, c.stream));
        APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
        if (zero_scale) *zero_scale = 0;
    }
    c.bytes_uploaded += cb + sb;
    return 0;
}

DevQW *new_qw(int fmt, const uint8_t *codes, const uint8_t *scales, int O, int K) {
    if (ensure_enabled()) return nullptr;
    if (O % 16 || K % 128) {
        set_error("quantised weight [%d,%d]: O must be a multiple of 16 and K of 128", O, K);
        return nullptr;
    }
    DevQW *w = new DevQW();
    w->fmt = fmt; w->O = O; w->K = K;
    size_t cb = fmt == 4 ? (size_t)O * K / 2 : (size_t)O * K;
    size_t sb = fmt == 4 ? (size_t)O * K / 32 : (size_t)((O + 127) / 128) * (K / 128);
    static const bool fp8_tc = !(getenv("APUS_FP8_TC") && getenv("APUS_FP8_TC")[0] == '0');
    if (fmt == 8 && fp8_tc && O % 128 == 0 && K <= 16384) {
        // tcgen05 kernel: no re-tiling; a device buffer of the caller is used in place
        const bool adopt = is_device_ptr(codes) && ((uintptr_t)codes & 15) == 0;
        bool ok = cudaMalloc(&w->scales, sb) == cudaSuccess &&
                  cudaMemcpy(w->scales, scales, sb, cudaMemcpyDefault) == cudaSuccess;
        if (ok && adopt) { w->codes = const_cast<uint8_t *>(codes); w->owned = false; }
        else if (ok) {
            ok = cudaMalloc(&w->codes, cb) == cudaSuccess &&
                 cudaMemcpy(w->codes, codes, cb, cudaMemcpyDefault) == cudaSuccess;
            if (ok) ctx().bytes_uploaded += cb + sb;
        }
        if (!ok) set_error("upload of %zu FP8 weight bytes failed", cb + sb);
        if (ok) ok = tc8_make_weight_map(w->map, w->codes, O, K) == 0;
        if (!ok) {
            if (!w->owned) { w->codes = nullptr; if (w->scales) cudaFree(w->scales); w->scales = nullptr; }
            w->release(); delete w;
            return nullptr;
        }
        w->tc = true;
        return w;
    }
    if (cudaMalloc(&w->codes, cb) != cudaSuccess || cudaMalloc(&w->scales, sb) != cudaSuccess) {
        set_error("cudaMalloc of %zu weight bytes failed", cb + sb);
        w->release(); delete w;
        return nullptr;
    }
    if (upload_qw(fmt, codes, scales, O, K, w->codes, w->scales, &w->zero_scale)) {
        w->release(); delete w;
        return nullptr;
    }
    return w;
}

DevQW *cached_qw(int fmt, const uint8_t *codes, const uint8_t *scales, int O, int K) {
    Ctx &c = ctx();
    auto it = c.qcache.find(codes);
    if (it != c.qcache.end() && it->second->fmt == fmt && it->second->O == O && it->second->K == K)
        return it->second;
    if (it != c.qcache.end()) { it->second->release(); delete it->second; c.qcache.erase(it); }
    DevQW *w = new_qw(fmt, codes, scales, O, K);
    if (w) c.qcache[codes] = w;
    return w;
}

bool is_device_ptr(const void *p) {
    cudaPointerAttributes a;
    if (!p || cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeDevice;
}

// Dense weights: a host buffer is uploaded once and cached by its address; a
// device buffer is used in place (the caller keeps it alive).
const void *cached_dense(const void *host, size_t bytes) {
    if (is_device_ptr(host)) return host;
    Ctx &c = ctx();
    auto it = c.dcache.find(host);
    if (it != c.dcache.end() && it->second->cap >= bytes) return it->second->p;
    DevBuf *b = it != c.dcache.end() ? it->second : new DevBuf();
    if (b->get(bytes, nullptr)) return nullptr;
    if (cudaMemcpy(b->p, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
        set_error("upload of %zu dense weight bytes failed", bytes);
        return nullptr;
    }
    c.bytes_uploaded += bytes;
    c.dcache[host] = b;
    return b->p;
}

// ---- composite device ops ----------------------------------------------------------------------
// Block-scaled GEMM of pre-quantised activation rows against one matrix, or a
// gate/up pair with SwiGLU (`other` != NULL): the tcgen05 FP8 kernel when the
// matrix is held in the reference storage, else the mma.sync kernel.
int qgemm_dev(DevQW *w, DevQW *other, const uint8_t *acodes, const float *ascales, int M, float *out,
              bool round_out, float limit, cudaStream_t st) {
    if (M <= 0) return 0;
    static const bool wide_ok = !(getenv("APUS_FP8_WIDE") && getenv("APUS_FP8_WIDE")[0] == '0');
    if (w->tc && !other && M >= 64 && w->K <= 8192 && wide_ok) {       // many rows: 128 per CTA
        alignas(64) unsigned char map_x[128];
        if (tc8_make_act_map_wide(map_x, acodes, M, w->K)) return 1;
        Tc8Args t = {};
        t.map_a = w->map; t.map_b = w->map; t.map_x = map_x;
        t.scales_a = w->scales; t.ascales = ascales;
        t.M = M; t.O = w->O; t.K = w->K; t.pair = 0; t.round_out = round_out; t.out = out;
        return gemm_tc8_wide(t, st);
    }
    if (w->tc && (!other || other->tc)) {
        alignas(64) unsigned char map_x[128];
        if (tc_make_act_map(map_x, acodes, M, w->K)) return 1;
        Tc8Args t = {};
        t.map_a = w->map; t.map_b = other ? other->map : w->map; t.map_x = map_x;
        t.scales_a = w->scales; t.scales_b = other ? other->scales : nullptr; t.ascales = ascales;
        t.M = M; t.O = w->O; t.K = w->K; t.pair = other ? 1 : 0; t.round_out = round_out; t.limit = limit;
        t.out = out;
        return gemm_tc8(t, st);
    }
    APUS_REQUIRE(!w->tc && (!other || !other->tc), "qgemm: gate and up matrices are held in different layouts");
    GemmSmallArgs a = {};
    a.fmt = w->fmt; a.pair = other ? 1 : 0; a.round_out = round_out; a.limit = limit; a.O = w->O; a.K = w->K;
    if (w->table_for(M, other != nullptr, other, const_cast<GemmGroup **>(&a.groups), &a.n_groups)) return 1;
    a.max_rows = M < 32 ? M : 32;
    a.acodes = acodes; a.ascales = ascales; a.out = out;
    a.zero_scale = w->zero_scale | (other ? other->zero_scale : 0);
    return gemm_small(a, st);
}

int qlinear_dev(DevQW *w, const float *x, float *out, int M, uint8_t *xq, float *xs,
                bool round_out, cudaStream_t st) {
    if (M <= 0) return 0;
    if (act_quant(x, nullptr, M, w->K, xq, xs, nullptr, st)) return 1;
    return qgemm_dev(w, nullptr, xq, xs, M, out, round_out, 0.f, st);
}

int expert_dev(DevQW *w1, DevQW *w2, DevQW *w3, float limit, const float *x, int rows,
               float *out, const ExpertWs &ws, cudaStream_t st) {
    if (rows <= 0) return 0;
    APUS_REQUIRE(w1->fmt == w3->fmt && w1->fmt == w2->fmt && w1->O == w3->O && w1->K == w3->K &&
                 w2->K == w1->O && w2->O == w1->K, "expert: inconsistent weight shapes");
    if (act_quant(x, nullptr, rows, w1->K, ws.xq, ws.xs, nullptr, st)) return 1;
    if (qgemm_dev(w1, w3, ws.xq, ws.xs, rows, ws.h, false, limit, st)) return 1;
    return qlinear_dev(w2, ws.h, out, rows, ws.hq, ws.hs, true, st);
}

}  // namespace apus

using namespace apus;

// =====================================================================================
namespace apus {
static std::vector<std::pair<void (*)(), void (*)(const void *)>> &release_hooks() {
    static std::vector<std::pair<void (*)(), void (*)(const void *)>> v;
    return v;
}
void on_disable(void (*release_all)(), void (*forget_one)(const void *)) {
    release_hooks().push_back({release_all, forget_one});
}
}  // namespace apus

namespace apus {
static int initial_tree_ops() {
    if (getenv("APUS_SUM_ORDER") && atoi(getenv("APUS_SUM_ORDER")) == 1) return APUS_CUDA_TREE_ALL;
    if (const char *e = getenv("APUS_TREE_OPS")) return atoi(e) & APUS_CUDA_TREE_ALL;
    return APUS_CUDA_TREE_DEFAULT;
}
static int g_tree_ops = initial_tree_ops();
static unsigned long long g_sum_epoch = 0;     // bumped whenever the order changes
int sum_order() { return g_tree_ops == APUS_CUDA_TREE_ALL ? APUS_CUDA_SUM_TREE : APUS_CUDA_SUM_REFERENCE; }
int tree_ops() { return g_tree_ops; }
unsigned long long sum_order_epoch() { return g_sum_epoch + g_buf_moves; }
// s > 1 calls run as chunks of positions (one pass) unless switched off: APUS_PREFILL=0 or
// apus_cuda_set_prefill_chunk(0) bring back one step per position
static int g_chunk_rows = -1;
int chunk_rows() {
    if (g_chunk_rows < 0) {
        const char *e = getenv("APUS_PREFILL");
        g_chunk_rows = e && e[0] ? atoi(e) : 2048;
        if (g_chunk_rows < 0) g_chunk_rows = 0;
    }
    return g_chunk_rows;
}
bool chunks_enabled() { return chunk_rows() > 0; }
bool pdl_enabled() {
    static const int on = [] { const char *e = getenv("APUS_PDL"); return !(e && e[0] == '0'); }();
    return on != 0;
}

int stream_scratch(cudaStream_t st, size_t bytes, void **ws, size_t n_counters, int **counters) {
    struct Slot { DevBuf ws, cnt; };
    static std::mutex mu;
    static std::map<std::tuple<int, cudaStream_t, int>, Slot> slots;
    int dev = 0;
    APUS_CUDA_OK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    // the stream the entry points without a stream argument run on is ONE chain whichever handle it
    // has at the moment (apus_cuda_use_stream lets a caller swap it, e.g. for a stream capture):
    // its scratch goes with the role, not with the handle
    // A side stream works for one main chain at a time, and recorded steps of different chains
    // (models stepping side by side) run concurrently whatever stream they were recorded on: a side
    // chain's scratch belongs to (the main chain it branched from, which branch).
    cudaStream_t owner = st;
    int branch = 0;
    for (int i = 0; i < Ctx::N_AUX; i++)
        if (st == ctx().aux[i] && g_aux_owned[i]) { owner = g_aux_owner[i]; branch = i + 1; }
    const cudaStream_t key = owner == ctx().stream ? reinterpret_cast<cudaStream_t>(~(uintptr_t)0) : owner;
    Slot &s = slots[std::make_tuple(dev, key, branch)];
    if (bytes > s.ws.cap) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(st, &cs);
        APUS_REQUIRE(cs == cudaStreamCaptureStatusNone, "stream scratch would have to grow to %zu bytes inside a stream capture", bytes);
        if (s.ws.get(bytes + bytes / 4, nullptr)) return 1;
    }
    const size_t cb = n_counters * sizeof(int);
    if (cb > s.cnt.cap) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(st, &cs);
        APUS_REQUIRE(cs == cudaStreamCaptureStatusNone, "stream counters would have to grow inside a stream capture");
        if (s.cnt.get(cb < 4096 ? 4096 : 2 * cb, nullptr)) return 1;
        APUS_CUDA_OK(cudaMemset(s.cnt.p, 0, s.cnt.cap));
    }
    if (ws) *ws = s.ws.p;
    if (counters) *counters = s.cnt.as<int>();
    return 0;
}

int ensure_dyn_smem(const void *func, size_t bytes) {
    if (bytes <= 48 * 1024) return 0;
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, size_t> set;      // (kernel, device) -> largest size set
    int dev = 0;
    APUS_CUDA_OK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    size_t &have = set[{func, dev}];
    if (bytes <= have) return 0;
    APUS_CUDA_OK(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    have = bytes;
    return 0;
}
}  // namespace apus

extern "C" {

int apus_cuda_enable(char *err, size_t errcap) {
    if (ensure_enabled()) {
        if (err && errcap) snprintf(err, errcap, "%s", t_err);
        return 1;
    }
    return 0;
}

void apus_cuda_moe_destroy(ApusCudaMoe *m);

int apus_cuda_use_stream(void *stream, int use_own) {
    if (ensure_enabled()) return 1;
    Ctx &c = ctx();
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    c.stream = use_own ? c.own_stream : (cudaStream_t)stream;
    return 0;
}

int apus_cuda_sample_logits_u(const float *logits, size_t n, float temp, float top_p, const double *u,
                              int32_t *tokens, int rows) {
    if (ensure_enabled()) return 1;
    if (rows <= 0) return 0;
    Ctx &c = ctx();
    void *dl, *dp, *du, *dt;
    if (c.ws[0].get((size_t)rows * n * 4, &dl) || c.ws[1].get((size_t)rows * n * 4, &dp) ||
        c.ws[2].get((size_t)rows * 8, &du) || c.ws[3].get((size_t)rows * 4, &dt))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dl, logits, (size_t)rows * n * 4, cudaMemcpyHostToDevice, c.stream));
    if (temp > 0.f) {
        APUS_REQUIRE(u != nullptr, "sample_logits_u: no uniforms given");
        APUS_CUDA_OK(cudaMemcpyAsync(du, u, (size_t)rows * 8, cudaMemcpyHostToDevice, c.stream));
    }
    if (sample_rows((float *)dl, (int)n, rows, temp, top_p, (double *)du, nullptr, (float *)dp, (int32_t *)dt, c.stream))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(tokens, dt, (size_t)rows * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

int apus_cuda_set_tree_ops(int mask) {
    if (mask == -2) return APUS_CUDA_TREE_DEFAULT;
    if (mask >= 0 && (mask & APUS_CUDA_TREE_ALL) != apus::g_tree_ops) {
        apus::g_tree_ops = mask & APUS_CUDA_TREE_ALL;
        apus::g_sum_epoch++;               // recorded steps chose their kernels by the old setting
    }
    return apus::g_tree_ops;
}

int apus_cuda_set_prefill_chunk(int rows) {
    const int before = apus::chunk_rows();
    if (rows >= 0) apus::g_chunk_rows = rows;
    return before;
}

int apus_cuda_set_sum_order(int order) {
    if (order == APUS_CUDA_SUM_REFERENCE) apus_cuda_set_tree_ops(0);
    else if (order == APUS_CUDA_SUM_TREE) apus_cuda_set_tree_ops(APUS_CUDA_TREE_ALL);
    return apus::sum_order();
}

void apus_cuda_disable(void) {
    Ctx &c = ctx();
    if (!c.enabled) return;
    cudaDeviceSynchronize();
    for (auto &h : apus::release_hooks()) if (h.first) h.first();
    for (auto &kv : c.qcache) { kv.second->release(); delete kv.second; }
    c.qcache.clear();
    for (auto &kv : c.dcache) { kv.second->release(); delete kv.second; }
    c.dcache.clear();
    for (auto &kv : c.moes) apus_cuda_moe_destroy(kv.second);
    c.moes.clear();
    for (auto &b : c.ws) b.release();
    c.stage.release();
    if (c.own_stream) cudaStreamDestroy(c.own_stream);
    c.stream = c.own_stream = nullptr;
    for (int i = 0; i < Ctx::N_AUX; i++) {
        if (c.aux[i]) cudaStreamDestroy(c.aux[i]);
        if (c.ev_fork[i]) cudaEventDestroy(c.ev_fork[i]);
        if (c.ev_join[i]) cudaEventDestroy(c.ev_join[i]);
        c.aux[i] = nullptr; c.ev_fork[i] = c.ev_join[i] = nullptr;
    }
    c.enabled = false;
}

int apus_cuda_is_enabled(void) { return ctx().enabled ? 1 : 0; }
uint64_t apus_cuda_bytes_uploaded(void) { return ctx().bytes_uploaded; }
uint64_t apus_cuda_dispatches(void) { return g_dispatches; }
const char *apus_cuda_last_error(void) { return t_err; }

void apus_cuda_forget(const void *host_ptr) {
    Ctx &c = ctx();
    auto q = c.qcache.find(host_ptr);
    if (q != c.qcache.end()) { cudaDeviceSynchronize(); q->second->release(); delete q->second; c.qcache.erase(q); }
    auto d = c.dcache.find(host_ptr);
    if (d != c.dcache.end()) { cudaDeviceSynchronize(); d->second->release(); delete d->second; c.dcache.erase(d); }
    auto m = c.moes.find(host_ptr);
    if (m != c.moes.end()) { cudaDeviceSynchronize(); apus_cuda_moe_destroy(m->second); c.moes.erase(m); }
    for (auto &h : apus::release_hooks()) if (h.second) h.second(host_ptr);
}

// ---- hook table ----------------------------------------------------------------------
static size_t g_st_dtype_off = 0, g_st_data_off = 0;

static int hook_fp8_linear(const ApusFp8W *w, const float *x, float *out, int M, int K, int O) {
    return apus_cuda_fp8_linear(w, x, out, M, K, O);
}
static int hook_f32_linear(const float *w, const float *x, float *out, int M, int K, int O,
                           int flags) {
    return apus_cuda_f32_linear(w, x, out, M, K, O, flags);
}
static int hook_head_gemv(const void *head, const float *x, float *out, int64_t O, int64_t K) {
    // reference c/st.h:42-46: dtype enum, BF16 = 4, F32 = 6
    int dtype = *(const int *)((const char *)head + g_st_dtype_off);
    const void *data = *(const void *const *)((const char *)head + g_st_data_off);
    if (dtype == 4) return apus_cuda_head_gemv_bf16(data, x, out, O, K);
    if (dtype == 6) return apus_cuda_f32_linear((const float *)data, x, out, 1, (int)K, (int)O, 0);
    set_error("head_gemv: unsupported tensor dtype %d", dtype);
    return 1;
}

int apus_cuda_fill_hooks(ApusCudaHooks *hooks, size_t struct_dtype_off, size_t struct_data_off) {
    if (!hooks) { set_error("fill_hooks: NULL table"); return 1; }
    if (ensure_enabled()) return 1;
    g_st_dtype_off = struct_dtype_off;
    g_st_data_off = struct_data_off;
    hooks->fp8_linear = hook_fp8_linear;
    hooks->f32_linear = hook_f32_linear;
    hooks->head_gemv = hook_head_gemv;
    return 0;
}

// ---- kernel-level host-pointer entry points ---------------------------------------------
static int host_qlinear(int fmt, const uint8_t *codes, const uint8_t *scales, int64_t wO,
                        int64_t wK, const float *x, float *out, int M, int K, int O) {
    if (ensure_enabled()) return 1;
    APUS_REQUIRE(wO == O && wK == K, "linear: weight is [%lld,%lld] but call says O=%d K=%d",
                 (long long)wO, (long long)wK, O, K);
    if (M <= 0) return 0;
    Ctx &c = ctx();
    DevQW *w = cached_qw(fmt, codes, scales, O, K);
    if (!w) return 1;
    void *dx, *dq, *ds, *dout;
    if (c.ws[0].get((size_t)M * K * 4, &dx) || c.ws[1].get((size_t)M * K, &dq) ||
        c.ws[2].get((size_t)M * (K / 128) * 4, &ds) || c.ws[3].get((size_t)M * O * 4, &dout))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dx, x, (size_t)M * K * 4, cudaMemcpyHostToDevice, c.stream));
    if (qlinear_dev(w, (float *)dx, (float *)dout, M, (uint8_t *)dq, (float *)ds, true, c.stream))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(out, dout, (size_t)M * O * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    if (w->tc) {
        int stt = gemm_tc_status(1);
        APUS_REQUIRE(stt == 0, "a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
    }
    return 0;
}

int apus_cuda_fp8_linear(const ApusFp8W *w, const float *x, float *out, int M, int K, int O) {
    return host_qlinear(8, w->codes, w->scales, w->O, w->K, x, out, M, K, O);
}
int apus_cuda_fp4_linear(const ApusFp4W *w, const float *x, float *out, int M, int K, int O) {
    return host_qlinear(4, w->packed, w->scales, w->O, w->K, x, out, M, K, O);
}

int apus_cuda_f32_linear(const float *w, const float *x, float *out, int M, int K, int O,
                         int flags) {
    if (ensure_enabled()) return 1;
    if (M <= 0) return 0;
    Ctx &c = ctx();
    size_t wbytes = (size_t)O * K * ((flags & APUS_CUDA_W_BF16) ? 2 : 4);
    const void *dw = cached_dense(w, wbytes);
    if (!dw) return 1;
    void *dx, *dout;
    if (c.ws[0].get((size_t)M * K * 4, &dx) || c.ws[3].get((size_t)M * O * 4, &dout)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dx, x, (size_t)M * K * 4, cudaMemcpyHostToDevice, c.stream));
    if (f32_linear(dw, (float *)dx, (float *)dout, M, K, O, flags, c.stream)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(out, dout, (size_t)M * O * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

int apus_cuda_head_gemv_bf16(const void *w_bf16, const float *x, float *out, int64_t O,
                             int64_t K) {
    return apus_cuda_f32_linear((const float *)w_bf16, x, out, 1, (int)K, (int)O,
                                APUS_CUDA_W_BF16);
}

static int host_qgemm(int fmt, const uint8_t *w, const uint8_t *ws, const uint8_t *acodes,
                      const float *as, float *out, int M, int O, int K) {
    if (ensure_enabled()) return 1;
    if (M <= 0) return 0;
    Ctx &c = ctx();
    DevQW *dw = cached_qw(fmt, w, ws, O, K);
    if (!dw) return 1;
    void *dq, *ds, *dout;
    if (c.ws[1].get((size_t)M * K, &dq) || c.ws[2].get((size_t)M * (K / 128) * 4, &ds) ||
        c.ws[3].get((size_t)M * O * 4, &dout))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dq, acodes, (size_t)M * K, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(ds, as, (size_t)M * (K / 128) * 4, cudaMemcpyHostToDevice, c.stream));
    if (qgemm_dev(dw, nullptr, (uint8_t *)dq, (float *)ds, M, (float *)dout, false, 0.f, c.stream)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(out, dout, (size_t)M * O * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "a bounded wait expired inside a tcgen05 kernel (code %d)", stt);
    return 0;
}

int apus_cuda_fp8_gemm(const uint8_t *w, const uint8_t *ws, const uint8_t *acodes,
                       const float *as, float *out, int M, int O, int K) {
    return host_qgemm(8, w, ws, acodes, as, out, M, O, K);
}
int apus_cuda_fp4_gemm(const uint8_t *w, const uint8_t *ws, const uint8_t *acodes,
                       const float *as, float *out, int M, int O, int K) {
    return host_qgemm(4, w, ws, acodes, as, out, M, O, K);
}

// c/fp4.h:166 on the tcgen05 path: weights stay in the reference storage and are
// unpacked by TMA; used by the kernel-level tests of gemm_tc.cu.
int apus_cuda_fp4_gemm_tc(const uint8_t *w, const uint8_t *ws, const uint8_t *acodes, const float *as,
                          float *out, int M, int O, int K) {
    if (ensure_enabled()) return 1;
    if (M <= 0) return 0;
    APUS_REQUIRE(O % 128 == 0 && K % 512 == 0, "fp4_gemm_tc: O=%d must be a multiple of 128 and K=%d of 512", O, K);
    Ctx &c = ctx();
    const size_t cb = (size_t)O * K / 2, sb = (size_t)O * K / 32;
    const int ng = ceil_div(M, 32);
    void *dw, *ds, *dq, *das, *dout, *dg;
    if (c.ws[8].get(cb, &dw) || c.ws[9].get(sb, &ds) || c.ws[1].get((size_t)M * K, &dq) ||
        c.ws[2].get((size_t)M * (K / 128) * 4, &das) || c.ws[3].get((size_t)M * O * 4, &dout) ||
        c.ws[4].get((size_t)ng * sizeof(TcGroup), &dg))
        return 1;
    std::vector<TcGroup> g(ng);
    for (int i = 0; i < ng; i++) { g[i].a_row = 0; g[i].row0 = i * 32; g[i].nrows = M - i * 32 < 32 ? M - i * 32 : 32; g[i].pad = 0; }
    APUS_CUDA_OK(cudaMemcpyAsync(dw, w, cb, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(ds, ws, sb, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(dq, acodes, (size_t)M * K, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(das, as, (size_t)M * (K / 128) * 4, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(dg, g.data(), ng * sizeof(TcGroup), cudaMemcpyHostToDevice, c.stream));
    alignas(64) unsigned char map_w[128], map_x[128];
    if (tc_make_weight_map(map_w, dw, O, K) || tc_make_act_map(map_x, dq, M, K)) return 1;
    TcArgs a = {};
    a.map_a = map_w; a.map_b = map_w; a.map_x = map_x;
    a.scales_a = (const uint8_t *)ds; a.ascales = (const float *)das;
    a.groups = (const TcGroup *)dg; a.n_groups = ng; a.O = O; a.K = K; a.pair = 0; a.round_out = 0;
    a.out = (float *)dout;
    gemm_tc_status(1);
    if (gemm_tc(a, c.stream)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(out, dout, (size_t)M * O * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    int stt = gemm_tc_status(1);
    APUS_REQUIRE(stt == 0, "fp4_gemm_tc: a bounded wait expired inside the kernel (code %d)", stt);
    return 0;
}

int apus_cuda_fp4_gemm_grouped(const ApusFp4GemmEnt *ents, size_t n_ent, const uint8_t *acodes,
                               const float *as, size_t rows, size_t O, size_t K) {
    if (ensure_enabled()) return 1;
    if (!n_ent) return 0;
    Ctx &c = ctx();
    // work items: each entry cut into runs of <= 32 rows; outputs land in one
    // device buffer laid out entry after entry, copied back per entry.
    std::vector<GemmGroup> items;
    std::vector<int> orow;           // output row (in the packed out buffer) of activation-space position
    std::vector<size_t> out_off(n_ent);
    size_t out_rows = 0;
    int zs = 0;
    std::vector<int> arow;           // activation row of each work-item position
    for (size_t e = 0; e < n_ent; e++) {
        DevQW *dw = cached_qw(4, ents[e].w, ents[e].ws, (int)O, (int)K);
        if (!dw) return 1;
        zs |= dw->zero_scale;
        out_off[e] = out_rows;
        APUS_REQUIRE(ents[e].m0 + ents[e].M <= rows, "grouped gemm: entry %zu exceeds the row space", e);
        for (size_t r = 0; r < ents[e].M; r += 32) {
            GemmGroup g = {};
            g.wa = dw->codes; g.sa = dw->scales;
            g.row0 = (int)arow.size();
            g.nrows = (int)(ents[e].M - r < 32 ? ents[e].M - r : 32);
            for (int i = 0; i < g.nrows; i++) {
                arow.push_back((int)(ents[e].m0 + r + i));
                orow.push_back((int)(out_rows + r + i));
            }
            items.push_back(g);
        }
        out_rows += ents[e].M;
    }
    if (!out_rows) return 0;
    void *dq, *ds, *dout, *dtab, *darow, *dorow;
    if (c.ws[1].get(rows * K, &dq) || c.ws[2].get(rows * (K / 128) * 4, &ds) ||
        c.ws[3].get(out_rows * O * 4, &dout) || c.ws[4].get(items.size() * sizeof(GemmGroup), &dtab) ||
        c.ws[5].get(arow.size() * 4, &darow) || c.ws[6].get(orow.size() * 4, &dorow))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dq, acodes, rows * K, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(ds, as, rows * (K / 128) * 4, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(dtab, items.data(), items.size() * sizeof(GemmGroup), cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(darow, arow.data(), arow.size() * 4, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(dorow, orow.data(), orow.size() * 4, cudaMemcpyHostToDevice, c.stream));
    GemmSmallArgs a = {};
    a.fmt = 4; a.O = (int)O; a.K = (int)K; a.round_out = 0;
    a.groups = (GemmGroup *)dtab; a.n_groups = (int)items.size(); a.max_rows = 32;
    a.acodes = (uint8_t *)dq; a.ascales = (float *)ds; a.arow = (int *)darow; a.orow = (int *)dorow;
    a.out = (float *)dout; a.zero_scale = zs;
    if (gemm_small(a, c.stream)) return 1;
    for (size_t e = 0; e < n_ent; e++)
        if (ents[e].M)
            APUS_CUDA_OK(cudaMemcpyAsync(ents[e].out, (float *)dout + out_off[e] * O,
                                         ents[e].M * O * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

int apus_cuda_fp8_act_quant(const float *x, int M, int K, uint8_t *codes, float *scales) {
    if (ensure_enabled()) return 1;
    if (M <= 0) return 0;
    Ctx &c = ctx();
    void *dx, *dq, *ds;
    if (c.ws[0].get((size_t)M * K * 4, &dx) || c.ws[1].get((size_t)M * K, &dq) ||
        c.ws[2].get((size_t)M * (K / 128) * 4, &ds))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dx, x, (size_t)M * K * 4, cudaMemcpyHostToDevice, c.stream));
    if (act_quant((float *)dx, nullptr, M, K, (uint8_t *)dq, (float *)ds, nullptr, c.stream)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(codes, dq, (size_t)M * K, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(scales, ds, (size_t)M * (K / 128) * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

int apus_cuda_rmsnorm(const float *x, const float *w, float eps, float *y, int64_t n,
                      int64_t rows) {
    if (ensure_enabled()) return 1;
    if (rows <= 0) return 0;
    Ctx &c = ctx();
    void *dx, *dw, *dy;
    if (c.ws[0].get(rows * n * 4, &dx) || c.ws[1].get(n * 4, &dw) || c.ws[3].get(rows * n * 4, &dy))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dx, x, rows * n * 4, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(dw, w, n * 4, cudaMemcpyHostToDevice, c.stream));
    if (rms_norm((float *)dx, (float *)dw, eps, (float *)dy, n, rows, c.stream)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(y, dy, rows * n * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

static int get_expert_ws(int rows, int dim, int inter, ExpertWs *ws, int base_slot) {
    Ctx &c = ctx();
    void *h, *xq, *hq, *xs, *hs;
    if (c.ws[base_slot].get((size_t)rows * inter * 4, &h) ||
        c.ws[base_slot + 1].get((size_t)rows * dim, &xq) ||
        c.ws[base_slot + 2].get((size_t)rows * inter, &hq) ||
        c.ws[base_slot + 3].get((size_t)rows * (dim / 128) * 4, &xs) ||
        c.ws[base_slot + 4].get((size_t)rows * (inter / 128) * 4, &hs))
        return 1;
    ws->h = (float *)h; ws->xq = (uint8_t *)xq; ws->hq = (uint8_t *)hq;
    ws->xs = (float *)xs; ws->hs = (float *)hs;
    return 0;
}

int apus_cuda_expert(const void *w1, const void *w2, const void *w3, int kind, float limit,
                     const float *x, int rows, int dim, int inter, float *out) {
    if (ensure_enabled()) return 1;
    if (rows <= 0) return 0;
    Ctx &c = ctx();
    // ApusFp4W and ApusFp8W share one layout (c/st.h:88-89)
    const ApusFp4W *a1 = (const ApusFp4W *)w1, *a2 = (const ApusFp4W *)w2, *a3 = (const ApusFp4W *)w3;
    int fmt = kind == 0 ? 4 : 8;
    APUS_REQUIRE(a1->O == inter && a1->K == dim && a3->O == inter && a3->K == dim &&
                 a2->O == dim && a2->K == inter, "expert: weight shapes do not match dim=%d inter=%d", dim, inter);
    DevQW *d1 = cached_qw(fmt, a1->packed, a1->scales, inter, dim);
    DevQW *d3 = cached_qw(fmt, a3->packed, a3->scales, inter, dim);
    DevQW *d2 = cached_qw(fmt, a2->packed, a2->scales, dim, inter);
    if (!d1 || !d2 || !d3) return 1;
    void *dx, *dout;
    ExpertWs ws;
    if (c.ws[0].get((size_t)rows * dim * 4, &dx) || c.ws[3].get((size_t)rows * dim * 4, &dout) ||
        get_expert_ws(rows, dim, inter, &ws, 7))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dx, x, (size_t)rows * dim * 4, cudaMemcpyHostToDevice, c.stream));
    if (expert_dev(d1, d2, d3, limit, (float *)dx, rows, (float *)dout, ws, c.stream)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(out, dout, (size_t)rows * dim * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

int apus_cuda_topk_stable(const float *row, int n, int k, int32_t *idx, int rows) {
    if (ensure_enabled()) return 1;
    if (rows <= 0) return 0;
    Ctx &c = ctx();
    void *dx, *di;
    if (c.ws[0].get((size_t)rows * n * 4, &dx) || c.ws[3].get((size_t)rows * k * 4, &di)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dx, row, (size_t)rows * n * 4, cudaMemcpyHostToDevice, c.stream));
    if (topk_stable((float *)dx, n, k, (int32_t *)di, rows, c.stream)) return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(idx, di, (size_t)rows * k * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

int apus_cuda_sparse_attn(const float *q, const float *sink, int h, int d, const int32_t *idxs,
                          int idxw, int s, float scale, const float *kv_a, int64_t na,
                          const float *kv_b, int64_t nb, float *o) {
    if (ensure_enabled()) return 1;
    if (s <= 0) return 0;
    Ctx &c = ctx();
    size_t qb = (size_t)s * h * d * 4;
    void *dq, *dsink, *di, *da, *db, *dout;
    if (c.ws[0].get(qb, &dq) || c.ws[1].get((size_t)h * 4, &dsink) ||
        c.ws[2].get((size_t)s * idxw * 4 + 16, &di) || c.ws[4].get((size_t)na * d * 4 + 16, &da) ||
        c.ws[5].get((size_t)nb * d * 4 + 16, &db) || c.ws[3].get(qb, &dout))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dq, q, qb, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(dsink, sink, (size_t)h * 4, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(di, idxs, (size_t)s * idxw * 4, cudaMemcpyHostToDevice, c.stream));
    if (na) APUS_CUDA_OK(cudaMemcpyAsync(da, kv_a, (size_t)na * d * 4, cudaMemcpyHostToDevice, c.stream));
    if (nb) APUS_CUDA_OK(cudaMemcpyAsync(db, kv_b, (size_t)nb * d * 4, cudaMemcpyHostToDevice, c.stream));
    if (sparse_attn((float *)dq, (float *)dsink, h, d, (int32_t *)di, idxw, s, scale, da, na, db, nb,
                    0, (float *)dout, c.stream))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(o, dout, qb, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

// ---- mHC host-pointer entry points ------------------------------------------------------------
static int mhc_host(const float *x4, size_t d, size_t n, const float *fn, const float *scale,
                    float head_scale, const float *base, float norm_eps, float hc_eps, int iters,
                    const float *norm_w, float rms_eps, float *pre, float *post, float *comb,
                    float *y, float *y_normed, int rows, int head) {
    if (ensure_enabled()) return 1;
    if (rows <= 0) return 0;
    Ctx &c = ctx();
    size_t nmix = head ? n : (2 + n) * n, nx = n * d;
    const float *dfn = (const float *)cached_dense(fn, nmix * nx * 4);
    if (!dfn) return 1;
    void *dx, *dsc, *dbase, *dnw, *dpre, *dpost, *dcomb, *dy, *dyn;
    if (c.ws[0].get((size_t)rows * nx * 4, &dx) || c.ws[1].get(64, &dsc) ||
        c.ws[2].get(nmix * 4, &dbase) || c.ws[4].get(d * 4, &dnw) ||
        c.ws[5].get((size_t)rows * n * 4, &dpre) || c.ws[6].get((size_t)rows * n * 4, &dpost) ||
        c.ws[7].get((size_t)rows * n * n * 4, &dcomb) || c.ws[3].get((size_t)rows * d * 4, &dy) ||
        c.ws[8].get((size_t)rows * d * 4, &dyn))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(dx, x4, (size_t)rows * nx * 4, cudaMemcpyHostToDevice, c.stream));
    if (!head) APUS_CUDA_OK(cudaMemcpyAsync(dsc, scale, 3 * 4, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(dbase, base, nmix * 4, cudaMemcpyHostToDevice, c.stream));
    if (norm_w) APUS_CUDA_OK(cudaMemcpyAsync(dnw, norm_w, d * 4, cudaMemcpyHostToDevice, c.stream));
    int rc;
    if (head)
        rc = mhc_head((float *)dx, (int)d, (int)n, dfn, head_scale, (float *)dbase, norm_eps, hc_eps,
                      (float *)dy, rows, c.stream);
    else
        rc = mhc_pre((float *)dx, (int)d, (int)n, dfn, (float *)dsc, (float *)dbase, norm_eps, hc_eps,
                     iters, norm_w ? (float *)dnw : nullptr, rms_eps, (float *)dpre, (float *)dpost,
                     (float *)dcomb, y ? (float *)dy : nullptr, (float *)dyn, rows, c.stream);
    if (rc) return 1;
    if (pre) APUS_CUDA_OK(cudaMemcpyAsync(pre, dpre, (size_t)rows * n * 4, cudaMemcpyDeviceToHost, c.stream));
    if (post) APUS_CUDA_OK(cudaMemcpyAsync(post, dpost, (size_t)rows * n * 4, cudaMemcpyDeviceToHost, c.stream));
    if (comb) APUS_CUDA_OK(cudaMemcpyAsync(comb, dcomb, (size_t)rows * n * n * 4, cudaMemcpyDeviceToHost, c.stream));
    if (y) APUS_CUDA_OK(cudaMemcpyAsync(y, dy, (size_t)rows * d * 4, cudaMemcpyDeviceToHost, c.stream));
    if (y_normed && norm_w)
        APUS_CUDA_OK(cudaMemcpyAsync(y_normed, dyn, (size_t)rows * d * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

int apus_cuda_mhc_prepost(const float *x4, size_t d, size_t n, const float *fn, const float *scale,
                          const float *base, float norm_eps, float hc_eps, int iters, float *pre,
                          float *post, float *comb, int rows) {
    return mhc_host(x4, d, n, fn, scale, 0.f, base, norm_eps, hc_eps, iters, nullptr, 0.f, pre, post,
                    comb, nullptr, nullptr, rows, 0);
}

int apus_cuda_hc_pre(const float *x4, size_t d, size_t n, const float *fn, const float *scale,
                     const float *base, float norm_eps, float hc_eps, int iters, const float *norm_w,
                     float rms_eps, float *y, float *y_normed, float *post, float *comb, int rows) {
    APUS_REQUIRE(y != nullptr, "hc_pre: y must not be NULL");
    return mhc_host(x4, d, n, fn, scale, 0.f, base, norm_eps, hc_eps, iters, norm_w, rms_eps, nullptr,
                    post, comb, y, y_normed, rows, 0);
}

int apus_cuda_hc_head(const float *x4, size_t d, size_t n, const float *fn, float scale,
                      const float *base, float norm_eps, float hc_eps, float *y, int rows) {
    return mhc_host(x4, d, n, fn, nullptr, scale, base, norm_eps, hc_eps, 0, nullptr, 0.f, nullptr,
                    nullptr, nullptr, y, nullptr, rows, 1);
}

int apus_cuda_hc_post(const float *f, const float *res4, const float *post, const float *comb,
                      float *y4, size_t d, size_t n, int rows) {
    if (ensure_enabled()) return 1;
    if (rows <= 0) return 0;
    Ctx &c = ctx();
    void *df, *dres, *dpost, *dcomb, *dy;
    if (c.ws[0].get((size_t)rows * d * 4, &df) || c.ws[1].get((size_t)rows * n * d * 4, &dres) ||
        c.ws[5].get((size_t)rows * n * 4, &dpost) || c.ws[6].get((size_t)rows * n * n * 4, &dcomb) ||
        c.ws[3].get((size_t)rows * n * d * 4, &dy))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(df, f, (size_t)rows * d * 4, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(dres, res4, (size_t)rows * n * d * 4, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(dpost, post, (size_t)rows * n * 4, cudaMemcpyHostToDevice, c.stream));
    APUS_CUDA_OK(cudaMemcpyAsync(dcomb, comb, (size_t)rows * n * n * 4, cudaMemcpyHostToDevice, c.stream));
    if (mhc_post((float *)df, (float *)dres, (float *)dpost, (float *)dcomb, (float *)dy, (int)d,
                 (int)n, rows, c.stream))
        return 1;
    APUS_CUDA_OK(cudaMemcpyAsync(y4, dy, (size_t)rows * n * d * 4, cudaMemcpyDeviceToHost, c.stream));
    APUS_CUDA_OK(cudaStreamSynchronize(c.stream));
    return 0;
}

// ---- single matrices, device-resident ------------------------------------------------------------
ApusCudaFp4 *apus_cuda_fp4_upload(const ApusFp4W *w) {
    return static_cast<ApusCudaFp4 *>(new_qw(4, w->packed, w->scales, (int)w->O, (int)w->K));
}
ApusCudaFp8 *apus_cuda_fp8_upload(const ApusFp8W *w) {
    return static_cast<ApusCudaFp8 *>(new_qw(8, w->codes, w->scales, (int)w->O, (int)w->K));
}
void apus_cuda_fp4_free(ApusCudaFp4 *w) { if (w) { cudaDeviceSynchronize(); w->release(); delete static_cast<DevQW *>(w); } }
void apus_cuda_fp8_free(ApusCudaFp8 *w) { if (w) { cudaDeviceSynchronize(); w->release(); delete static_cast<DevQW *>(w); } }

// per-handle activation workspaces for the *_dev calls (grown on demand)
static DevBuf g_dev_ws[8];

static int qlinear_handle(DevQW *w, const float *x, float *out, int M, void *stream) {
    if (ensure_enabled()) return 1;
    void *dq, *ds;
    if (g_dev_ws[0].get((size_t)M * w->K, &dq) || g_dev_ws[1].get((size_t)M * (w->K / 128) * 4, &ds))
        return 1;
    return qlinear_dev(w, x, out, M, (uint8_t *)dq, (float *)ds, true, (cudaStream_t)stream);
}
int apus_cuda_fp4_linear_dev(const ApusCudaFp4 *w, const float *x, float *out, int M, void *stream) {
    return qlinear_handle(const_cast<ApusCudaFp4 *>(w), x, out, M, stream);
}
int apus_cuda_fp8_linear_dev(const ApusCudaFp8 *w, const float *x, float *out, int M, void *stream) {
    return qlinear_handle(const_cast<ApusCudaFp8 *>(w), x, out, M, stream);
}

int apus_cuda_expert_fp4_dev(const ApusCudaFp4 *w1, const ApusCudaFp4 *w2, const ApusCudaFp4 *w3,
                             float limit, const float *x, int rows, float *out, void *stream) {
    if (ensure_enabled()) return 1;
    if (rows <= 0) return 0;
    int dim = w1->K, inter = w1->O;
    void *h, *xq, *hq, *xs, *hs;
    if (g_dev_ws[2].get((size_t)rows * inter * 4, &h) || g_dev_ws[3].get((size_t)rows * dim, &xq) ||
        g_dev_ws[4].get((size_t)rows * inter, &hq) || g_dev_ws[5].get((size_t)rows * (dim / 128) * 4, &xs) ||
        g_dev_ws[6].get((size_t)rows * (inter / 128) * 4, &hs))
        return 1;
    ExpertWs ws = {(float *)h, (uint8_t *)xq, (uint8_t *)hq, (float *)xs, (float *)hs};
    return expert_dev(const_cast<ApusCudaFp4 *>(w1), const_cast<ApusCudaFp4 *>(w2),
                      const_cast<ApusCudaFp4 *>(w3), limit, x, rows, out, ws, (cudaStream_t)stream);
}

int apus_cuda_topk_stable_dev(const float *scores, int n, int k, int32_t *idx, int rows,
                              void *stream) {
    if (ensure_enabled()) return 1;
    return topk_stable(scores, n, k, idx, rows, (cudaStream_t)stream);
}

int apus_cuda_sparse_attn_dev(const float *q, const float *sink, int h, int d, const int32_t *idxs,
                              int idxw, int s, float scale, const uint16_t *kv_a, int64_t na,
                              const uint16_t *kv_b, int64_t nb, float *o, void *stream) {
    if (ensure_enabled()) return 1;
    return sparse_attn(q, sink, h, d, idxs, idxw, s, scale, kv_a, na, kv_b, nb, 1, o,
                       (cudaStream_t)stream);
}

int apus_cuda_sparse_attn_batch_dev(const float *q, const float *sink, int h, int d, const int32_t *idxs,
                                    int idxw, int s, float scale, const uint16_t *kv_a, int64_t na,
                                    int64_t kv_a_stride, const uint16_t *kv_b, int64_t nb, int64_t kv_b_stride,
                                    float *o, void *stream) {
    if (ensure_enabled()) return 1;
    APUS_REQUIRE(kv_a_stride >= 0 && kv_b_stride >= 0, "sparse_attn_batch: negative stride");
    return sparse_attn(q, sink, h, d, idxs, idxw, s, scale, kv_a, na, kv_b, nb, 1, o, (cudaStream_t)stream,
                       (long long)kv_a_stride * d, (long long)kv_b_stride * d);
}

}  // extern "C"
